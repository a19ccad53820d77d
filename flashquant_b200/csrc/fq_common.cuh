// Shared helpers for the sm_100a TurboQuant kernels: status plumbing, dtype loads,
// mbarrier / bulk-copy PTX wrappers with bounded waits, warp-level MMA wrappers.
#pragma once

#include <nvtx3/nvToolsExt.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/flashquant_b200.h"

namespace fq {

// ------------------------------------------------------------------------------------
// Host-side error plumbing (no exceptions, no abort across the C ABI)
// ------------------------------------------------------------------------------------
char* last_error_buffer();  // thread-local, 512 bytes (defined in capi.cu)

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

void count_launch(uint64_t n = 1);  // library-wide counter of kernel launches (capi.cu)
uint64_t settings_epoch();  // changes whenever a process-wide setter is called (capi.cu)
void settings_changed();

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  count_launch();
  return FQ_OK;
}

#define FQ_REQUIRE(cond, code, ...)              \
  do {                                           \
    if (!(cond)) return fq::fail(code, __VA_ARGS__); \
  } while (0)

// A named range around every launcher, for timeline tools (the reference wraps its dispatchers
// the same way: src/flashquant/profiling.py:31-82).  Without a tool attached the calls are
// no-ops of the header-only NVTX layer.
struct NvtxRange {
  explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
  ~NvtxRange() { nvtxRangePop(); }
  NvtxRange(const NvtxRange&) = delete;
  NvtxRange& operator=(const NvtxRange&) = delete;
};
#define FQ_RANGE(name) fq::NvtxRange fq_nvtx_range_(name)

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// ------------------------------------------------------------------------------------
// dtype helpers
// ------------------------------------------------------------------------------------
template <int DT>
struct Elem;
template <>
struct Elem<FQ_F32> {
  using type = float;
};
template <>
struct Elem<FQ_F16> {
  using type = __half;
};
template <>
struct Elem<FQ_BF16> {
  using type = __nv_bfloat16;
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f32(float v);
template <>
__device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Load 4 consecutive elements (pointer aligned to 4 elements) as fp32.
__device__ __forceinline__ void load4(const float* p, float (&v)[4]) {
  float4 t = *reinterpret_cast<const float4*>(p);
  v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load4(const __half* p, float (&v)[4]) {
  uint2 t = *reinterpret_cast<const uint2*>(p);
  float2 a = __half22float2(*reinterpret_cast<__half2*>(&t.x));
  float2 b = __half22float2(*reinterpret_cast<__half2*>(&t.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&v)[4]) {
  uint2 t = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(t.x << 16);
  v[1] = __uint_as_float(t.x & 0xffff0000u);
  v[2] = __uint_as_float(t.y << 16);
  v[3] = __uint_as_float(t.y & 0xffff0000u);
}
__device__ __forceinline__ void load2(const float* p, float (&v)[2]) {
  float2 t = *reinterpret_cast<const float2*>(p);
  v[0] = t.x; v[1] = t.y;
}
__device__ __forceinline__ void load2(const __half* p, float (&v)[2]) {
  float2 a = __half22float2(*reinterpret_cast<const __half2*>(p));
  v[0] = a.x; v[1] = a.y;
}
__device__ __forceinline__ void load2(const __nv_bfloat16* p, float (&v)[2]) {
  uint32_t t = *reinterpret_cast<const uint32_t*>(p);
  v[0] = __uint_as_float(t << 16);
  v[1] = __uint_as_float(t & 0xffff0000u);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------------------
// Shared-memory barriers and bulk copies (PTX).  Every wait is bounded IN TIME: when the
// limit (nanoseconds of %globaltimer) has passed since the first failed poll, the caller gets
// `false` and must record an error and leave.  The limit is a kernel argument set from
// fq_set_device_wait_limit_ns(); waits that take no argument use the default.
// ------------------------------------------------------------------------------------
constexpr uint64_t kDefaultWaitNs = 2000000000ull;  // 2 s: far beyond any legitimate wait

// Limit the launchers pass to their kernels (capi.cu; fq_set_device_wait_limit_ns).
uint64_t device_wait_limit_ns();

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// One look at the barrier that never suspends the warp (try_wait may hold it for a while when
// the phase is still open): for opportunistic polls whose answer may well be "not yet".
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Returns false when the limit ran out.  One poll that succeeds costs no timer read.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity,
                                          uint64_t limit_ns = kDefaultWaitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
#pragma unroll 1
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > limit_ns) return false;
  }
}
// The same for a whole warp (all 32 lanes call it): every lane gets the same answer, so the
// warp can leave a loop together.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
  if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
  const uint64_t t0 = global_timer_ns();
#pragma unroll 1
  while (true) {
    const bool ok = mbar_try_wait(bar, parity);
    const bool late = global_timer_ns() - t0 > limit_ns;
    if (__all_sync(0xffffffffu, ok)) return true;
    if (__any_sync(0xffffffffu, late)) return false;
  }
}
// Waits until *counter >= target (a counter other CTAs of the launch bump with
// red_release_add).  Lane 0 polls, every lane gets the same answer.
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p);
__device__ __forceinline__ bool counter_wait_warp(const uint32_t* counter, uint32_t target,
                                                  uint64_t limit_ns, int lane) {
  int state = 0;  // 1 = reached, 2 = gave up
  uint64_t t0 = 0;
#pragma unroll 1
  while (true) {
    if (lane == 0) {
      if (ld_acquire_u32(counter) >= target) {
        state = 1;
      } else {
        const uint64_t now = global_timer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > limit_ns) state = 2;
      }
    }
    state = __shfl_sync(0xffffffffu, state, 0);
    if (state) return state == 1;
    __nanosleep(64);
  }
}

// 1-D bulk copy global -> shared, completion counted in bytes on `bar`.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                         uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// The same with an L2 eviction hint: streamed data that is read once (cache pages) is marked
// evict-first so that it does not push the small, hot inputs of the next call (tables, block
// table, lengths, query) out of the L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                              uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(smem_dst)),
      "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// Orders this thread's earlier generic-proxy accesses (and those it has acquired from other
// threads) before its later bulk copies, which go through the async proxy.
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// Counters in global memory that CTAs of one launch signal each other through.  The add is a
// release: everything the warp wrote before its __syncwarp() is visible to whoever acquires
// the new count, and the warp does not wait for that (no fence, no returned value).
__device__ __forceinline__ void red_release_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ------------------------------------------------------------------------------------
// Warp-level MMA (fp16 operands, fp32 accumulate) and the 8x8 transpose.
// Fragment layout, lane = 4*g + t:
//   A (16x16): a0=(row g, k 2t..2t+1) a1=(row g+8, k 2t..) a2=(row g, k 2t+8..) a3=(row g+8, k 2t+8..)
//   B (16x8):  b0=(k 2t..2t+1, col g) b1=(k 2t+8..2t+9, col g)
//   C (16x8):  c0=(row g, col 2t) c1=(row g, col 2t+1) c2=(row g+8, col 2t) c3=(row g+8, col 2t+1)
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                        uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Lane (g,t) gives (row g, cols 2t,2t+1) of an 8x8 b16 matrix and receives the same
// position of its transpose.
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
  uint32_t r;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float fast_log2(float x) {
  float r;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Where row r of a contiguous list of rows lives in a buffer made of segments (the per-head
// buffers of a contiguous cache): runs of seg_len rows land seg_stride rows apart, starting at
// row seg_offset of each segment.  seg_len == 0: row r is row r.
struct RowMap {
  uint32_t seg_len = 0;
  int64_t seg_stride = 0;
  int64_t seg_offset = 0;
  __host__ __device__ __forceinline__ int64_t operator()(int64_t r) const {
    if (seg_len == 0) return r;
    const int64_t seg = r / seg_len;
    return seg * seg_stride + seg_offset + (r - seg * seg_len);
  }
};

// paged_decode.cu: the decode call for n_q query tokens per sequence in one pass (q and out
// (num_seqs, n_q, H_q, D); query token i sees keys 0 .. seq_len - n_q + i), and how many
// tokens a pass can take for a given geometry
int decode_tokens_per_pass(int num_q_heads, int num_kv_heads, int head_dim, int block_size);
int decode_tokens(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                  const int32_t* block_table, int64_t block_table_stride, const int32_t* seq_lens,
                  const float* centroids_k, int n_centroids_k, const float* centroids_v,
                  int n_centroids_v, const float* rotation, int num_seqs, int n_q, int num_q_heads,
                  int num_kv_heads, int head_dim, int block_size, int64_t num_blocks,
                  float sm_scale, void* out, int num_splits, void* workspace,
                  size_t workspace_bytes, cudaStream_t stream);

// rotate.cu: row rotations around the prefill kernel
int rotate_q_to_half(const void* q, int dtype, const float* rotation, __half* out,
                     int64_t n_rows, int head_dim, cudaStream_t stream);
int rotate_back(const float* o_rot, int dtype, const float* rotation, void* out, int64_t n_rows,
                int head_dim, cudaStream_t stream, RowMap out_map = RowMap());
// the same from the partial rows of n_splits key slices (merged on the way in); few rows only
int rotate_back_merged(const float* part, int n_splits, int dtype, const float* rotation,
                       void* out, int64_t n_rows, int head_dim, cudaStream_t stream);
bool rotate_is_few_rows(int64_t n_rows);
// the same from nibble codes + norms (rows through in_map), expanded on the way in; few rows only
int rotate_back_from_codes(const uint8_t* codes, const float* norms, const float* centroids,
                           int n_centroids, RowMap in_map, int dtype, const float* rotation,
                           void* out, int64_t n_rows, int head_dim, cudaStream_t stream,
                           RowMap out_map);
// decompress.cu: codes (rows through in_map) -> rotated-space values, contiguous
int decompress_rows(const uint8_t* packed, const float* norms, const float* centroids,
                    int n_centroids, void* out, int out_dtype, int64_t n_vectors, int head_dim,
                    RowMap in_map, cudaStream_t stream);

}  // namespace fq
