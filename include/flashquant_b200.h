/*
 * flashquant_b200 - C ABI of the B200 (sm_100a) TurboQuant KV-cache kernels.
 *
 * Every entry point takes raw DEVICE pointers, sizes and a CUDA stream, allocates
 * nothing, never synchronises the stream and never aborts: it returns FQ_OK (0) or a
 * negative fq_status, and fq_last_error_string() describes the last failure of the
 * calling thread.  All launches are asynchronous on `stream`.
 *
 * Each declaration names the interface of ayinedjimi/flashquant it stands in for
 * (paths relative to that repository).
 */
#ifndef FLASHQUANT_B200_H_
#define FLASHQUANT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* fq_stream_t; /* same type as cudaStream_t */

typedef enum fq_dtype {
  FQ_F32 = 0,
  FQ_F16 = 1,
  FQ_BF16 = 2
} fq_dtype;

typedef enum fq_status {
  FQ_OK = 0,
  FQ_ERR_INVALID_ARGUMENT = -1, /* null pointer, negative size, bad enum            */
  FQ_ERR_UNSUPPORTED = -2,      /* shape outside what the kernels are built for     */
  FQ_ERR_WORKSPACE = -3,        /* workspace missing, misaligned or too small       */
  FQ_ERR_CUDA = -4,             /* a CUDA runtime call failed (launch, attribute)   */
  FQ_ERR_ALIGNMENT = -5         /* a pointer or stride breaks an alignment rule     */
} fq_status;

/* Bits of the device-side status word kept at the start of a decode workspace. */
#define FQ_DEV_BAD_BLOCK_INDEX 1u /* a block_table entry was outside [0, num_blocks) */
#define FQ_DEV_WAIT_TIMEOUT 2u    /* a bounded wait on a shared-memory barrier ran out */
#define FQ_DEV_BAD_LENGTH 4u      /* fq_paged_tq4_prefill: a chunk of cu_seqlens_q lies outside
                                     the query tokens or is longer than max_q_len; its rows (or
                                     their tail) were not computed */

int fq_version(void);
const char* fq_last_error_string(void);
/* Number of kernels this library has launched in the process so far (all threads). */
uint64_t fq_launch_count(void);

/*
 * TQ4 compress, contiguous outputs.
 * Replaces tq4_compress_cuda (csrc/cuda/compress.cuh:38-48) as reached from
 * flashquant.kernels.compress.tq4_compress (src/flashquant/kernels/compress.py:83-92);
 * arithmetic of compress_reference (src/flashquant/kernels/cpu_reference.py:22-61):
 * n = |x|, y = (x/(n+1e-10)) Pi^T, code = #{b : b < y}, byte j = code[2j]<<4 | code[2j+1].
 *   x            n_vectors x head_dim values of `dtype`, row stride head_dim
 *   rot_T_even   (head_dim, head_dim/2) fp32: columns 0,2,4.. of Pi^T
 *   rot_T_odd    (head_dim, head_dim/2) fp32: columns 1,3,5.. of Pi^T
 *   boundaries   n_boundaries (<= 15) ascending fp32
 *   packed       n_vectors x head_dim/2 bytes out
 *   norms        n_vectors fp32 out
 * head_dim is 64 or 128.
 */
int fq_tq4_compress(const void* x, fq_dtype dtype, const float* rot_T_even,
                    const float* rot_T_odd, const float* boundaries, int n_boundaries,
                    uint8_t* packed, float* norms, int64_t n_vectors, int head_dim,
                    fq_stream_t stream);

/*
 * TQ4 compress straight into the pre-allocated per-head buffers of a contiguous cache.
 * Replaces CompressedDynamicCache._compress_tensor (src/flashquant/cache/hf_cache.py:170-194:
 * ValueCompressor.compress + nibble_pack) followed by CompressedBuffer.append
 * (src/flashquant/cache/buffer_pool.py:86-110: two slice copies): the codes and norms of
 * the new tokens are written at their final place, rows position .. position+n_new-1 of
 * every segment, in one launch.
 *   x         (n_segments, n_new, head_dim) values of `dtype`, contiguous; a segment is one
 *             (batch, head) pair
 *   packed    (n_segments, capacity, head_dim/2) bytes, 4-byte aligned
 *   norms     (n_segments, capacity) fp32
 * position + n_new must not exceed capacity (FQ_ERR_INVALID_ARGUMENT, nothing written).
 * Arithmetic and the other arguments as fq_tq4_compress.
 */
int fq_tq4_compress_into(const void* x, fq_dtype dtype, const float* rot_T_even,
                         const float* rot_T_odd, const float* boundaries, int n_boundaries,
                         uint8_t* packed, float* norms, int64_t n_segments, int64_t n_new,
                         int64_t capacity, int64_t position, int head_dim, fq_stream_t stream);

/*
 * Stage-1 + stage-2 (QJL) quantiser, contiguous outputs.
 * Arithmetic of TurboQuantProd.quantize (src/flashquant/core/quantizer.py:270-304):
 * codes/norm as above with the (bits-1)-bit tables, r = x - (c[code] Pi) n,
 * gamma = |r|, sign_j = sgn(sum_k r_k S[j][k]) with 0 -> +1.
 *   rotation     (head_dim, head_dim) fp32 row-major Pi
 *   centroids    n_boundaries + 1 fp32
 *   qjl          (head_dim, head_dim) fp32 row-major S (qjl_dim must equal head_dim)
 *   sign_bits    n_vectors x head_dim/8 bytes out; bit (j%8) of byte j/8 is 1 iff sign_j=+1
 *   gamma        n_vectors fp32 out
 */
int fq_tq_prod_quantize(const void* x, fq_dtype dtype, const float* rotation,
                        const float* boundaries, int n_boundaries, const float* centroids,
                        const float* qjl, uint8_t* packed, float* norms, uint8_t* sign_bits,
                        float* gamma, int64_t n_vectors, int head_dim, fq_stream_t stream);

/*
 * 2-bit code packing, four codes per byte: byte = c0<<6 | c1<<4 | c2<<2 | c3.
 * Replaces pack_2bit / unpack_2bit of the reference's C++ core (csrc/core/packing.cpp:48-79;
 * the Python-side restatement its tests use is tests/conftest.py:245-265).
 *   codes          n_codes bytes, one code (0..3) per byte, 16-byte aligned
 *   packed         n_codes/4 bytes, 4-byte aligned
 *   out_of_range   optional device word: bit 0 is OR-ed in when a code above 3 was seen (the
 *                  reference validates before packing; its low two bits are packed here)
 * n_codes must be a multiple of 16.
 */
int fq_pack_2bit(const uint8_t* codes, uint8_t* packed, int64_t n_codes, uint32_t* out_of_range,
                 fq_stream_t stream);
int fq_unpack_2bit(const uint8_t* packed, uint8_t* codes, int64_t n_codes, fq_stream_t stream);

/*
 * TQ4 decompress (rotated space): out[v][2j] = c[byte>>4]*n, out[v][2j+1] = c[byte&15]*n.
 * Replaces tq4_decompress_cuda (csrc/cuda/decompress.cuh:40-48) as reached from
 * flashquant.kernels.decompress.tq4_decompress (src/flashquant/kernels/decompress.py:75-77);
 * arithmetic of decompress_reference (src/flashquant/kernels/cpu_reference.py:64-94).
 * head_dim must be a multiple of 8; `out` holds n_vectors x head_dim values of out_dtype.
 */
int fq_tq4_decompress(const uint8_t* packed, const float* norms, const float* centroids,
                      int n_centroids, void* out, fq_dtype out_dtype, int64_t n_vectors,
                      int head_dim, fq_stream_t stream);

/*
 * One update of a contiguous compressed cache in one call.
 * Replaces the body of CompressedDynamicCache._compressed_update
 * (src/flashquant/cache/hf_cache.py:260-365): _compress_tensor and CompressedBuffer.append for
 * keys and values, then _dequantize_tensor of the NEW tokens and their concatenation behind
 * the de-quantised tokens of earlier updates (torch.cat there, rows out_position .. of a
 * caller-owned growing tensor here).  Four launches on `stream` for up to 1024 new vectors
 * (the back-rotation expands the codes itself and the workspace is not used), six above;
 * no allocation, no sync.
 *   key, value          (n_segments, n_new, head_dim) of `dtype`, contiguous
 *   rot_T_even/odd_k/v  the split transposed rotations of keys / values (fq_tq4_compress)
 *   rotation_k/v        (head_dim, head_dim) fp32 row-major Pi of keys / values
 *   k_packed, v_packed  (n_segments, capacity, head_dim/2) bytes; k_norms, v_norms
 *                       (n_segments, capacity) fp32; rows position .. position+n_new-1 written
 *   k_out, v_out        (n_segments, out_capacity, head_dim) of `dtype`, rows out_position ..
 *                       written with round_dtype((c[code] n) Pi); both null = fused mode,
 *                       nothing is de-quantised and rotation_k/v, centroids, workspace are unused
 *   workspace           16-byte aligned, fq_cache_update_workspace_bytes(...) bytes
 * head_dim is 64 or 128.
 */
size_t fq_cache_update_workspace_bytes(int64_t n_segments, int64_t n_new, int head_dim);
int fq_cache_update(const void* key, const void* value, fq_dtype dtype,
                    const float* rot_T_even_k, const float* rot_T_odd_k, const float* rotation_k,
                    const float* rot_T_even_v, const float* rot_T_odd_v, const float* rotation_v,
                    const float* boundaries, int n_boundaries, const float* centroids,
                    int n_centroids, uint8_t* k_packed, float* k_norms, uint8_t* v_packed,
                    float* v_norms, int64_t n_segments, int64_t n_new, int64_t capacity,
                    int64_t position, void* k_out, void* v_out, int64_t out_capacity,
                    int64_t out_position, int head_dim, void* workspace, size_t workspace_bytes,
                    fq_stream_t stream);

/*
 * TQ4 decompress to the ORIGINAL space: out[v] = round_dtype((c[code] * n) Pi).
 * Replaces CompressedDynamicCache._dequantize_tensor (src/flashquant/cache/hf_cache.py:196-219:
 * nibble_unpack + ValueCompressor.decompress, src/flashquant/core/compressor.py:252-262, i.e.
 *  TurboQuantMSE.dequantize, src/flashquant/core/quantizer.py:161-195, cast to the model dtype).
 *   rotation    (head_dim, head_dim) fp32 row-major Pi
 *   out         n_vectors x head_dim values of out_dtype (FQ_F32, FQ_F16 or FQ_BF16), 16-byte aligned
 *   workspace   caller-owned, 16-byte aligned, fq_tq4_decompress_original_workspace_bytes(...)
 *               bytes (the fp32 rotated-space rows)
 * head_dim is 64 or 128.
 */
size_t fq_tq4_decompress_original_workspace_bytes(int64_t n_vectors, int head_dim);
int fq_tq4_decompress_original(const uint8_t* packed, const float* norms, const float* centroids,
                               int n_centroids, const float* rotation, void* out,
                               fq_dtype out_dtype, int64_t n_vectors, int head_dim,
                               void* workspace, size_t workspace_bytes, fq_stream_t stream);

/*
 * Compress-on-append: K and V of n_tokens new tokens are compressed and their packed
 * rows written straight into the paged cache at row slot_mapping[token].
 * Replaces FlashQuantAttentionImpl._compress_and_store (src/flashquant/vllm/impl.py:220-263):
 * two tq4_compress calls, eight slice copies and one index_put become one launch.
 * Row layout (src/flashquant/vllm/impl.py:132-138): [K codes H*D/2 | K norms H*4 |
 * V codes H*D/2 | V norms H*4], heads in order inside each region.
 *   key, value          (n_tokens, num_kv_heads, head_dim) of `dtype`; the stride between
 *                       tokens is token_stride elements (>= num_kv_heads*head_dim)
 *   rotation            (head_dim, head_dim) fp32 row-major Pi, shared by K and V
 *   boundaries_k / _v   ascending fp32 tables (may be the same pointer)
 *   kv_cache            num_slots rows of num_kv_heads*(head_dim+8) bytes
 *   slot_mapping        n_tokens entries, int64 if slot_is_int64 else int32; entries < 0 or
 *                       >= num_slots are skipped (padding)
 */
int fq_tq4_compress_append(const void* key, const void* value, fq_dtype dtype,
                           int64_t n_tokens, int num_kv_heads, int head_dim,
                           int64_t token_stride, const float* rotation,
                           const float* boundaries_k, int n_boundaries_k,
                           const float* boundaries_v, int n_boundaries_v, uint8_t* kv_cache,
                           int64_t num_slots, const void* slot_mapping, int slot_is_int64,
                           fq_stream_t stream);

/*
 * Compress-on-append with K through the two-stage quantiser: as above, and the QJL sign
 * bits and residual norm of every K vector go to a side plane with one row of
 * num_kv_heads*(head_dim/8+4) bytes per slot: [sign bits H*D/8 | gamma H*4].
 * The reference has no packed QJL storage (src/flashquant/vllm/impl.py:109-111 uses the
 * one-stage quantiser for K); the arithmetic is TurboQuantProd.quantize
 * (src/flashquant/core/quantizer.py:270-304).
 */
int fq_tq4_compress_append_qjl(const void* key, const void* value, fq_dtype dtype,
                               int64_t n_tokens, int num_kv_heads, int head_dim,
                               int64_t token_stride, const float* rotation,
                               const float* boundaries_k, int n_boundaries_k,
                               const float* centroids_k, const float* boundaries_v,
                               int n_boundaries_v, const float* qjl, uint8_t* kv_cache,
                               uint8_t* kq_cache, int64_t num_slots,
                               const void* slot_mapping, int slot_is_int64,
                               fq_stream_t stream);

/*
 * Split-K paged decode over the packed cache, un-rotated q in, original-space out.
 * Replaces paged_tq4_decode_cuda + split_k_reduce_cuda (csrc/cuda/paged_decode.cu:346-421,
 * csrc/cuda/split_k_reduce.cu:145-181) as reached from
 * flashquant.kernels.paged_decode.split_k_paged_decode
 * (src/flashquant/kernels/paged_decode.py:103-110); arithmetic of the CPU branch
 * (paged_decode.py:112-128 + src/flashquant/kernels/cpu_reference.py:230-368):
 * q_rot = round(q Pi^T), softmax(sm_scale q_rot K^T) V in rotated space with
 * K = c_k[code] n_k and V = c_v[code] n_v, rounded, then out = round(o_rot Pi).
 *   q, out         (num_seqs, num_q_heads, head_dim), FQ_F16, FQ_BF16 or FQ_F32 (an fp32
 *                  query, as in the reference's CPU-sized cases, is not rounded after its
 *                  rotation and neither is its output; it always takes the three-launch form)
 *   kv_cache       (num_blocks, block_size, num_kv_heads*(head_dim+8)) bytes, 16-byte aligned
 *   block_table    (num_seqs, block_table_stride) int32; a sequence never reads more than
 *                  block_table_stride entries of its row: a seq_len beyond
 *                  block_table_stride * block_size is cut there and FQ_DEV_BAD_BLOCK_INDEX is
 *                  set (the reference's CPU path would raise an IndexError)
 *   seq_lens       (num_seqs) int32; a length of 0 gives a zero output row
 *   num_splits     partitions of each sequence (1..64); every partition boundary is a
 *                  boundary between partial rows.  The pages of the whole batch are spread
 *                  evenly over the SMs whatever this number is; 0 means 1
 *   workspace      caller-owned, 256-byte aligned, at least
 *                  fq_paged_decode_workspace_bytes(...) bytes.  Its first 32 KiB must be zero
 *                  before the first call: word 0 is a status word (FQ_DEV_* bits are OR-ed
 *                  in), the rest holds per-sequence counters that the CTAs of the single
 *                  launch signal each other through and that every successful call leaves at
 *                  zero again.  After a call that set a status bit, zero those 32 KiB before
 *                  the workspace is used again.  Calls that overlap on the GPU need separate
 *                  workspaces.
 * The call is one cooperative launch with one CTA per SM: it needs the whole GPU to itself
 * while it runs (kernels of other streams delay it, they cannot deadlock it: every wait in
 * the kernel is bounded and ends in FQ_DEV_WAIT_TIMEOUT).
 * head_dim 128 (or 64), block_size a multiple of 16, num_kv_heads in {1,2,4,8,16},
 * num_q_heads/num_kv_heads <= 8, num_seqs <= 2048.
 */
size_t fq_paged_decode_workspace_bytes(int num_seqs, int num_q_heads, int num_kv_heads,
                                       int head_dim, int num_splits);
int fq_split_k_paged_decode(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                            const int32_t* block_table, int64_t block_table_stride,
                            const int32_t* seq_lens, const float* centroids_k,
                            int n_centroids_k, const float* centroids_v, int n_centroids_v,
                            const float* rotation, int num_seqs, int num_q_heads,
                            int num_kv_heads, int head_dim, int block_size,
                            int64_t num_blocks, float sm_scale, void* out, int num_splits,
                            void* workspace, size_t workspace_bytes, fq_stream_t stream);

/*
 * Decode steps of n_q tokens per sequence (speculative or chunked decode).
 * The reference takes its fused decode only for a step of exactly one token
 * (src/flashquant/vllm/impl.py:441) and otherwise de-quantises the whole cache for a causal
 * varlen attention (impl.py:265-336, 477-509).  Here the last n_q tokens of every sequence,
 * already appended to the cache and counted in seq_lens, attend in one decode launch: query i
 * of a sequence sees keys 0 .. seq_len - n_q + i (a query without a visible key gives zeros).
 * Where the specialised kernel applies (head_dim 128, 8 KV heads, pages of 16 tokens) the
 * (token, head) pairs of a KV head share the eight columns of its products: with 4 query heads
 * per KV head two tokens are served by ONE pass over the sequence's pages, and a step of
 * n_q tokens takes n_q / 2 passes instead of n_q.
 *   q, out        (num_seqs, n_q, num_q_heads, head_dim)
 *   block_table   (num_seqs, block_table_stride) int32, max_blocks (<= stride) columns used
 *   scratch       caller-owned, 16-byte aligned, fq_split_k_paged_decode_multi_scratch_bytes(...)
 *                 bytes: the per-(sequence, token) lengths and block-table rows a small kernel
 *                 writes before the decode
 * num_seqs * n_q <= 2048; workspace as for fq_split_k_paged_decode, at least
 * fq_split_k_paged_decode_multi_workspace_bytes(...) bytes; everything else as
 * fq_split_k_paged_decode.
 */
size_t fq_split_k_paged_decode_multi_scratch_bytes(int num_seqs, int n_q, int max_blocks);
size_t fq_split_k_paged_decode_multi_workspace_bytes(int num_seqs, int n_q, int num_q_heads,
                                                     int num_kv_heads, int head_dim,
                                                     int num_splits);
int fq_split_k_paged_decode_multi(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                                  const int32_t* block_table, int64_t block_table_stride,
                                  int max_blocks, const int32_t* seq_lens,
                                  const float* centroids_k, int n_centroids_k,
                                  const float* centroids_v, int n_centroids_v,
                                  const float* rotation, int num_seqs, int n_q, int num_q_heads,
                                  int num_kv_heads, int head_dim, int block_size,
                                  int64_t num_blocks, float sm_scale, void* out, int num_splits,
                                  void* workspace, size_t workspace_bytes, void* scratch,
                                  size_t scratch_bytes, fq_stream_t stream);

/*
 * fq_split_k_paged_decode normally is one cooperative launch with one CTA per SM.  On a GPU
 * that cannot hold such a launch (shared with other contexts, partitioned) the call falls
 * back by itself to three ordinary launches (q rotation, streaming, merge) with the same
 * result; fq_paged_decode_set_single_launch(0) selects that form for the whole process,
 * (1) restores the default.  (No counterpart in the reference.)
 */
void fq_paged_decode_set_single_launch(int enabled);

/*
 * Process-wide switches of the paged decode.  (No counterpart in the reference.)
 *
 * fq_paged_decode_set_fast_path(0) routes every call through the generic streaming kernel;
 * by default a cache of head_dim 128, 8 KV heads and pages of 16 tokens takes a kernel
 * specialised for that layout (same results up to the order of the fp32 sums).
 *
 * fq_paged_decode_set_weight_split(0) makes the specialised kernel carry every softmax
 * weight into the value product as one fp16 number (2^-12 relative) instead of two (2^-22).
 * The second term rides in product columns that are otherwise idle when a KV head serves at
 * most four (token, head) columns, so it costs a dozen instructions per 16-token tile (about
 * 3 % of the streaming phase); on by default.
 */
void fq_paged_decode_set_fast_path(int enabled);
void fq_paged_decode_set_weight_split(int enabled);

/*
 * Every wait inside a kernel - on a shared-memory barrier, on a counter another CTA of the
 * launch bumps - gives up after this many nanoseconds of the GPU's global timer, ORs
 * FQ_DEV_WAIT_TIMEOUT into the status word and lets the kernel return; nothing spins for
 * ever.  Default 200 ms; the value is read when a call is launched.  (No counterpart in the
 * reference, whose kernels have no such waits.)
 */
void fq_set_device_wait_limit_ns(uint64_t nanoseconds);
uint64_t fq_get_device_wait_limit_ns(void);

/*
 * Test hook: the merge phase of the single-launch decode waits for `n` more segment arrivals
 * than its sequence will ever produce, so that a test can watch the bounded wait give up
 * (status FQ_DEV_WAIT_TIMEOUT, the call still returns).  0 restores normal operation.
 */
void fq_paged_decode_test_expect_extra_segments(int n);

/*
 * fq_split_k_paged_decode with the two-stage estimator in the logits:
 *   logit = sm_scale * ( |k| <q_rot, c[code]> + gamma * sqrt(pi/2)/m * <S q, signs> )
 * i.e. TurboQuantProd.estimate_inner_product (src/flashquant/core/quantizer.py:349-370,
 * also KeyCompressor.asymmetric_attention_scores, src/flashquant/core/compressor.py:151-192)
 * evaluated against the paged cache; the reference never runs it at decode time (its
 * decode dequantises K through the first stage only), so this is an addition that gives the
 * sign bits and gamma written by fq_tq4_compress_append_qjl a consumer.  Values as in
 * fq_split_k_paged_decode.
 *   kq_cache   (num_blocks, block_size, num_kv_heads*(head_dim/8+4)) side plane, 16-byte aligned
 *   qjl        (head_dim, head_dim) fp32 row-major S; q S^T is computed in the same launch
 * head_dim 128 only, q FQ_F16 or FQ_BF16.  Traffic per (token, KV head): 156 bytes instead of
 * 136.  This entry exists only as the single cooperative launch: where the driver refuses
 * that launch it returns FQ_ERR_UNSUPPORTED.
 */
int fq_split_k_paged_decode_qjl(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                                const uint8_t* kq_cache, const int32_t* block_table,
                                int64_t block_table_stride, const int32_t* seq_lens,
                                const float* centroids_k, int n_centroids_k,
                                const float* centroids_v, int n_centroids_v,
                                const float* rotation, const float* qjl, int num_seqs,
                                int num_q_heads, int num_kv_heads, int head_dim, int block_size,
                                int64_t num_blocks, float sm_scale, void* out, int num_splits,
                                void* workspace, size_t workspace_bytes, fq_stream_t stream);

/*
 * fq_split_k_paged_decode for callers that cannot allocate.  (No counterpart in the
 * reference.)  Same arguments and result as fq_split_k_paged_decode, minus the workspace:
 * the scratch is a 16 MiB array built into the library, so nothing is allocated by the
 * caller or by the call - meant for a serving engine that has given all device memory to
 * the KV cache, or for code inside another framework's memory pool.
 *   - shapes whose scratch exceeds fq_split_k_paged_decode_static_max_bytes() are refused
 *     with FQ_ERR_WORKSPACE (the message names the size needed);
 *   - the first call on each device looks up the array's device address; make that first
 *     call outside any stream capture;
 *   - all calls on a device share the array: calls that overlap on the GPU race on it;
 *   - like fq_split_k_paged_decode it is one cooperative launch, or three ordinary launches
 *     when fq_paged_decode_set_single_launch(0) is in force or the driver refuses the
 *     cooperative launch;
 *   - the caller has no pointer to the array, so the device status word (FQ_DEV_* bits) of
 *     the last call is read with fq_split_k_paged_decode_static_status, which synchronises
 *     the stream; the next static call clears the word.
 */
size_t fq_split_k_paged_decode_static_max_bytes(void);
int fq_split_k_paged_decode_static(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                                   const int32_t* block_table, int64_t block_table_stride,
                                   const int32_t* seq_lens, const float* centroids_k,
                                   int n_centroids_k, const float* centroids_v,
                                   int n_centroids_v, const float* rotation, int num_seqs,
                                   int num_q_heads, int num_kv_heads, int head_dim,
                                   int block_size, int64_t num_blocks, float sm_scale, void* out,
                                   int num_splits, fq_stream_t stream);
int fq_split_k_paged_decode_static_status(uint32_t* status, fq_stream_t stream);

/*
 * The two halves of fq_split_k_paged_decode, for a sequence whose tokens are spread over
 * several GPUs: each GPU produces one partial row per (sequence, query head) over the pages
 * it holds, the rows are exchanged (one all-gather) and every GPU merges all of them.
 *
 * fq_paged_decode_partials: `partials` (16-byte aligned) receives (num_seqs, num_q_heads,
 * head_dim+4) fp32 rows: head_dim un-normalised accumulator values, then m (base-2
 * reference exponent: within 6 of the running maximum of logit*log2(e) + log2|v|, never above
 * it), l (sum of 2^(logit*log2(e) - m)) and two zero pads; a sequence of length 0 gives
 * (0.., -inf, 0).  Rows merge like any online-softmax triple: only differences of m matter.
 * Workspace as for fq_split_k_paged_decode.  The partial-softmax triple follows the sketch
 * in csrc/cuda/paged_decode.cu:198-275.
 *
 * fq_paged_decode_partials_rotated: the same for a query that is already in rotated space
 * and stored as fp16 (num_seqs, num_q_heads, head_dim) - the calling convention of
 * paged_decode_reference (src/flashquant/kernels/cpu_reference.py:230-241), which also
 * takes the pre-rotated query.  No rotation kernel is launched.
 *
 * fq_split_k_merge: `partials` is (n_groups, num_seqs, num_q_heads, head_dim+4), i.e.
 * n_groups buffers of the layout above back to back (n_groups = number of GPUs after an
 * all-gather).  out = round(round(sum w_g acc_g / sum w_g l_g) Pi), w_g = 2^(m_g - max m).
 * Stands in for split_k_reduce_cuda (csrc/cuda/split_k_reduce.cu:145-181), whose weighting
 * (acc_s * l_s) is not the softmax.
 */
int fq_paged_decode_partials(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                             const int32_t* block_table, int64_t block_table_stride,
                             const int32_t* seq_lens, const float* centroids_k,
                             int n_centroids_k, const float* centroids_v, int n_centroids_v,
                             const float* rotation, int num_seqs, int num_q_heads,
                             int num_kv_heads, int head_dim, int block_size,
                             int64_t num_blocks, float sm_scale, int num_splits,
                             float* partials, void* workspace, size_t workspace_bytes,
                             fq_stream_t stream);
int fq_paged_decode_partials_rotated(const void* q_rot_f16, const uint8_t* kv_cache,
                                     const int32_t* block_table, int64_t block_table_stride,
                                     const int32_t* seq_lens, const float* centroids_k,
                                     int n_centroids_k, const float* centroids_v,
                                     int n_centroids_v, int num_seqs, int num_q_heads,
                                     int num_kv_heads, int head_dim, int block_size,
                                     int64_t num_blocks, float sm_scale, int num_splits,
                                     float* partials, void* workspace, size_t workspace_bytes,
                                     fq_stream_t stream);
/*
 * The streaming stage alone (rotated fp16 query in, per-segment partial rows left in the
 * workspace): what a profiler or a benchmark times when it wants the memory-bound kernel
 * without the two small kernels around it.  No counterpart in the reference.
 */
int fq_paged_decode_stream(const void* q_rot_f16, const uint8_t* kv_cache,
                           const int32_t* block_table, int64_t block_table_stride,
                           const int32_t* seq_lens, const float* centroids_k,
                           int n_centroids_k, const float* centroids_v, int n_centroids_v,
                           int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                           int block_size, int64_t num_blocks, float sm_scale, int num_splits,
                           void* workspace, size_t workspace_bytes, fq_stream_t stream);
int fq_split_k_merge(const float* partials, int n_groups, const float* rotation,
                     int num_seqs, int num_q_heads, int head_dim, void* out, fq_dtype dtype,
                     fq_stream_t stream);

/*
 * Fused TQ4 attention over contiguous (non-paged) compressed K and V, causal or not.
 * Replaces fused_tq_attention_cuda (csrc/cuda/fused_tq_attention.cu:468-511) as reached from
 * flashquant.kernels.attention.fused_tq_attention (src/flashquant/kernels/attention.py:91-97);
 * arithmetic of the CPU branch (attention.py:99-107 +
 * src/flashquant/kernels/cpu_reference.py:154-227): q_rot = round(q Pi^T), K = c_k[code] n_k,
 * V = c_v[code] n_v, softmax(sm_scale q_rot K^T [causal: key j > query i masked]) V in fp32,
 * out = round(o_rot Pi).
 *   q, out              (batch, num_q_heads, n_q, head_dim), FQ_F16 or FQ_BF16, 16-byte aligned
 *   k_packed, v_packed  (batch, num_kv_heads, n_kv, head_dim/2) bytes, 16-byte aligned
 *   k_norms, v_norms    (batch, num_kv_heads, n_kv) fp32
 *   workspace           caller-owned, 256-byte aligned, fq_fused_tq_attention_workspace_bytes(...)
 *                       bytes (rotated fp16 query and fp32 rotated output); first word = status
 * head_dim 128; with is_causal, n_q must equal n_kv (or be 1).
 */
size_t fq_fused_tq_attention_workspace_bytes(int batch, int num_q_heads, int n_q, int head_dim);
int fq_fused_tq_attention(const void* q, fq_dtype dtype, const uint8_t* k_packed,
                          const float* k_norms, const uint8_t* v_packed, const float* v_norms,
                          const float* centroids_k, int n_centroids_k, const float* centroids_v,
                          int n_centroids_v, const float* rotation, int batch, int num_q_heads,
                          int num_kv_heads, int n_q, int n_kv, int head_dim, float sm_scale,
                          int is_causal, void* out, void* workspace, size_t workspace_bytes,
                          fq_stream_t stream);

/*
 * The same attention over the buffers of a contiguous cache whose keys and values were
 * compressed with different rotations (CompressedDynamicCache: key seed 42, value seed 43,
 * src/flashquant/cache/hf_cache.py:137-142) and read in place: get_compressed
 * (hf_cache.py:387-414) hands out views of n_kv valid tokens inside buffers with room for
 * kv_capacity tokens per (batch, head).  q_rot = round(q Pi_k^T), out = round(o_rot Pi_v).
 *   k_packed, v_packed  (batch, num_kv_heads, kv_capacity, head_dim/2) bytes
 *   k_norms, v_norms    (batch, num_kv_heads, kv_capacity) fp32
 * Everything else as fq_fused_tq_attention (same workspace).
 */
int fq_fused_tq_attention_kv(const void* q, fq_dtype dtype, const uint8_t* k_packed,
                             const float* k_norms, const uint8_t* v_packed,
                             const float* v_norms, const float* centroids_k, int n_centroids_k,
                             const float* centroids_v, int n_centroids_v,
                             const float* rotation_k, const float* rotation_v, int batch,
                             int num_q_heads, int num_kv_heads, int n_q, int n_kv,
                             int64_t kv_capacity, int head_dim, float sm_scale, int is_causal,
                             void* out, void* workspace, size_t workspace_bytes,
                             fq_stream_t stream);

/*
 * Fused TQ4 attention over the PAGED cache for prefill chunks of any length: replaces
 * FlashQuantAttentionImpl's prefill path (src/flashquant/vllm/impl.py:265-336, 477-509), which
 * de-quantises the whole cache and calls flash_attn_varlen_func on every prefill step.  Here
 * the pages of each sequence are read through its block-table row, de-quantised tile by tile
 * in shared memory and attended to on the tensor cores; nothing de-quantised reaches memory.
 *
 *   q, out          (total_q_tokens, num_q_heads, head_dim), FQ_F16 or FQ_BF16: the query
 *                   tokens of all sequences one after the other (vLLM's layout)
 *   cu_seqlens_q    (num_seqs + 1) int32: sequence b owns tokens cu[b] .. cu[b+1]
 *   seq_lens        (num_seqs) int32: keys of sequence b INCLUDING its query tokens, whose
 *                   K/V must already be in the cache (compress-on-append runs first, as in
 *                   the reference); the mask is causal and aligned at the END of the keys:
 *                   query i of a chunk of n sees keys 0 .. seq_lens[b] - n + i.  A query
 *                   without visible keys gives zeros.
 *   block_table     (num_seqs, block_table_stride) int32 page ids; an id outside
 *                   [0, num_blocks) or a length beyond the row sets FQ_DEV_BAD_BLOCK_INDEX in
 *                   word 0 of the workspace and is not followed
 *   max_q_len       longest chunk (sizes the grid); a longer chunk, or one that does not lie
 *                   inside [0, total_q_tokens), sets FQ_DEV_BAD_LENGTH and is cut / skipped
 *   rounding        q Pi^T and the attention rows are rounded to the activation type before
 *                   the products with K and Pi, as the reference's two matmul + cast steps do
 *   workspace       256-byte aligned, fq_paged_tq4_prefill_workspace_bytes(...) bytes; word 0
 *                   is the status word (zero it before the first call)
 * head_dim 128 and a multiple of 4 KV heads (16-byte gathers from the token rows) only.
 */
size_t fq_paged_tq4_prefill_workspace_bytes(int total_q_tokens, int num_q_heads, int head_dim);
int fq_paged_tq4_prefill(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                         const int32_t* block_table, int64_t block_table_stride,
                         const int32_t* seq_lens, const int32_t* cu_seqlens_q,
                         const float* centroids_k, int n_centroids_k, const float* centroids_v,
                         int n_centroids_v, const float* rotation, int num_seqs,
                         int total_q_tokens, int max_q_len, int num_q_heads, int num_kv_heads,
                         int head_dim, int block_size, int64_t num_blocks, float sm_scale,
                         void* out, void* workspace, size_t workspace_bytes, fq_stream_t stream);

/*
 * One decode step with HOST buffers: the host-side form of
 * FlashQuantAttentionImpl._fused_decode_path (src/flashquant/vllm/impl.py:362-395), which
 * compresses the step's new K/V token of every sequence into the paged cache and then runs
 * the fused paged decode.  Here the inputs of the step are host arrays (pinned memory makes
 * the copies asynchronous): they are copied into `staging` on the device, the two kernels
 * run, the result is copied to out_host and the stream is synchronised before returning.
 *   q_host, out_host        (num_seqs, num_q_heads, head_dim) of `dtype` (FQ_F16 / FQ_BF16)
 *   key_host, value_host    (num_seqs, num_kv_heads, head_dim): one new token per sequence
 *   slot_mapping_host       num_seqs cache rows for the new tokens (int64 or int32)
 *   block_table_host        (num_seqs, block_table_stride) int32;  seq_lens_host (num_seqs)
 *                           int32, lengths that already count the new token
 *   kv_cache, kq_cache      device-resident packed cache and QJL side plane; kq_cache NULL
 *                           selects the one-stage quantiser for K (fq_tq4_compress_append),
 *                           otherwise fq_tq4_compress_append_qjl is used and qjl is required
 *   rotation ... qjl        device-resident constants, as for the calls this one is made of
 *   staging                 device scratch, 256-byte aligned, at least
 *                           fq_decode_step_host_staging_bytes(...) bytes
 *   workspace               as for fq_split_k_paged_decode
 */
size_t fq_decode_step_host_staging_bytes(int num_seqs, int num_q_heads, int num_kv_heads,
                                         int head_dim, int64_t block_table_stride,
                                         int slot_is_int64);
int fq_decode_step_host(const void* q_host, const void* key_host, const void* value_host,
                        fq_dtype dtype, const void* slot_mapping_host, int slot_is_int64,
                        const int32_t* block_table_host, int64_t block_table_stride,
                        const int32_t* seq_lens_host, uint8_t* kv_cache, uint8_t* kq_cache,
                        const float* rotation, const float* boundaries_k, int n_boundaries_k,
                        const float* centroids_k, int n_centroids_k, const float* boundaries_v,
                        int n_boundaries_v, const float* centroids_v, int n_centroids_v,
                        const float* qjl, int num_seqs, int num_q_heads, int num_kv_heads,
                        int head_dim, int block_size, int64_t num_blocks, float sm_scale,
                        int num_splits, void* out_host, void* staging, size_t staging_bytes,
                        void* workspace, size_t workspace_bytes, fq_stream_t stream);

/* The same step with the host inputs in ONE page-locked block, laid out like the staging
 * area: the step is one host-to-device copy (overlap_copies = 0), or two halves of the block
 * with the second - sequence lengths, block table, query - in flight under the
 * compress-on-append (overlap_copies = 1), the two launches, one copy of the result to
 * out_host (which may point into the same block, at offsets[6]) and a synchronise.
 *
 * fq_decode_step_offsets fills offsets[0..7] with the byte offsets of
 *   key, value, slot_mapping, seq_lens, block_table, q, out, and the total size;
 * every part starts on a 256-byte boundary, shapes and dtypes as for fq_decode_step_host.
 * The caller writes each step's inputs at those offsets of its block, then calls
 * fq_decode_step_host_packed(block, ...); the staging area has the same size as before.
 */
/* The packed step is captured once per distinct argument set and replayed as a CUDA graph
 * (one submission for the copies in, the two launches and the copy out; with overlap_copies
 * the second half of the block is a branch of the graph that joins before the decode);
 * 0 switches that off for the whole process, the step is then issued call by call. */
void fq_decode_step_set_graph(int enabled);
int fq_decode_step_offsets(int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                           int64_t block_table_stride, int slot_is_int64, uint64_t offsets[8]);
int fq_decode_step_host_packed(const void* block_host, void* out_host, int overlap_copies,
                               fq_dtype dtype, int slot_is_int64, int64_t block_table_stride,
                               uint8_t* kv_cache, uint8_t* kq_cache, const float* rotation,
                               const float* boundaries_k, int n_boundaries_k,
                               const float* centroids_k, int n_centroids_k,
                               const float* boundaries_v, int n_boundaries_v,
                               const float* centroids_v, int n_centroids_v, const float* qjl,
                               int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                               int block_size, int64_t num_blocks, float sm_scale, int num_splits,
                               void* staging, size_t staging_bytes, void* workspace,
                               size_t workspace_bytes, fq_stream_t stream);

/* Copies the device status word of a decode workspace to *status (synchronises stream). */
int fq_workspace_status(const void* workspace, uint32_t* status, fq_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASHQUANT_B200_H_ */
