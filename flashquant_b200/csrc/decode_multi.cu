// Decode steps of several tokens per sequence.  The specialised decode kernel takes the
// (token, head) pairs of a KV head as the eight columns of its products, so with 4 query
// heads per KV head two tokens of a sequence share one pass over its pages.  A step of n_q
// tokens is cut into chunks of c tokens (c = tokens per pass, if it divides n_q, else 1);
// every (sequence, chunk) pair becomes a row of the decode with its own length - the last
// token of the chunk sees keys 0 .. L - n_q + (chunk end) - and a copy of the sequence's
// block-table row.  One small kernel builds those rows in caller-owned scratch memory, then
// the decode runs as usual.  (n_q <= c needs no rows at all: the decode takes the batch as it
// is.)
#include "fq_common.cuh"

namespace fq {

__global__ void __launch_bounds__(128) expand_decode_rows_kernel(
    const int32_t* __restrict__ block_table, int64_t block_table_stride,
    const int32_t* __restrict__ seq_lens, int n_q, int chunk, int max_blocks,
    int32_t* __restrict__ row_table, int32_t* __restrict__ row_lens) {
  const int per_seq = n_q / chunk;
  const int r = blockIdx.x, s = r / per_seq, j = r - s * per_seq;
  if (threadIdx.x == 0) {
    const int len = seq_lens[s] - (n_q - (j + 1) * chunk);  // keys the chunk's last token sees
    row_lens[r] = len < 0 ? 0 : len;
  }
  for (int b = threadIdx.x; b < max_blocks; b += blockDim.x)
    row_table[int64_t(r) * max_blocks + b] = block_table[int64_t(s) * block_table_stride + b];
}

static size_t lens_bytes(int64_t rows) { return (size_t(rows) * 4 + 255) / 256 * 256; }

}  // namespace fq

using namespace fq;

extern "C" size_t fq_split_k_paged_decode_multi_scratch_bytes(int num_seqs, int n_q,
                                                              int max_blocks) {
  if (num_seqs < 0 || n_q < 0 || max_blocks < 0) return 0;
  const int64_t rows = int64_t(num_seqs) * n_q;
  return lens_bytes(rows) + size_t(rows) * size_t(max_blocks) * 4;
}

extern "C" size_t fq_split_k_paged_decode_multi_workspace_bytes(int num_seqs, int n_q,
                                                                int num_q_heads,
                                                                int num_kv_heads, int head_dim,
                                                                int num_splits) {
  if (num_seqs < 0 || n_q < 1 || num_q_heads < 1 || num_kv_heads < 1) return 0;
  // either one decode row per (sequence, token), or rows of up to 8 / (heads per KV head)
  // tokens: room for both forms (the geometry decides at the call)
  size_t need = fq_paged_decode_workspace_bytes(num_seqs * n_q, num_q_heads, num_kv_heads,
                                                head_dim, num_splits);
  const int group = num_q_heads % num_kv_heads == 0 ? num_q_heads / num_kv_heads : 8;
  for (int c = 2; c * group <= 8 && c <= n_q; ++c) {
    if (n_q % c) continue;
    const size_t alt = fq_paged_decode_workspace_bytes(num_seqs * n_q / c, num_q_heads * c,
                                                       num_kv_heads, head_dim, num_splits);
    need = alt > need ? alt : need;
  }
  return need;
}

extern "C" int fq_split_k_paged_decode_multi(
    const void* q, fq_dtype dtype, const uint8_t* kv_cache, const int32_t* block_table,
    int64_t block_table_stride, int max_blocks, const int32_t* seq_lens,
    const float* centroids_k, int n_centroids_k, const float* centroids_v, int n_centroids_v,
    const float* rotation, int num_seqs, int n_q, int num_q_heads, int num_kv_heads,
    int head_dim, int block_size, int64_t num_blocks, float sm_scale, void* out, int num_splits,
    void* workspace, size_t workspace_bytes, void* scratch, size_t scratch_bytes,
    fq_stream_t stream) {
  FQ_RANGE("fq_split_k_paged_decode_multi");
  FQ_REQUIRE(num_seqs >= 0 && n_q >= 0 && max_blocks >= 0, FQ_ERR_INVALID_ARGUMENT,
             "multi-token decode: negative size");
  const int64_t rows = int64_t(num_seqs) * n_q;
  if (rows == 0) return FQ_OK;
  FQ_REQUIRE(rows <= 2048, FQ_ERR_UNSUPPORTED,
             "multi-token decode: %lld (sequence, token) rows (at most 2048)", (long long)rows);
  FQ_REQUIRE(block_table && seq_lens, FQ_ERR_INVALID_ARGUMENT,
             "multi-token decode: null pointer");
  FQ_REQUIRE(block_table_stride >= max_blocks, FQ_ERR_INVALID_ARGUMENT,
             "multi-token decode: block_table_stride smaller than max_blocks");
  const size_t need = fq_split_k_paged_decode_multi_scratch_bytes(num_seqs, n_q, max_blocks);
  FQ_REQUIRE(scratch && aligned(scratch, 16) && scratch_bytes >= need, FQ_ERR_WORKSPACE,
             "multi-token decode: scratch of %zu bytes needed (16-byte aligned)", need);
  int32_t* row_lens = static_cast<int32_t*>(scratch);
  int32_t* row_table =
      reinterpret_cast<int32_t*>(static_cast<unsigned char*>(scratch) + lens_bytes(rows));
  int chunk = decode_tokens_per_pass(num_q_heads, num_kv_heads, head_dim, block_size);
  if (chunk > n_q) chunk = n_q;
  if (n_q % chunk) chunk = 1;
  if (chunk == n_q)  // the whole step in one pass over the pages, no rows to build
    return decode_tokens(q, dtype, kv_cache, block_table, block_table_stride, seq_lens,
                         centroids_k, n_centroids_k, centroids_v, n_centroids_v, rotation,
                         num_seqs, n_q, num_q_heads, num_kv_heads, head_dim, block_size,
                         num_blocks, sm_scale, out, num_splits, workspace, workspace_bytes, stream);
  const int64_t chunks = rows / chunk;
  expand_decode_rows_kernel<<<unsigned(chunks), 128, 0, stream>>>(
      block_table, block_table_stride, seq_lens, n_q, chunk, max_blocks, row_table, row_lens);
  int rc = check_launch("multi-token row kernel launch");
  if (rc != FQ_OK) return rc;
  return decode_tokens(q, dtype, kv_cache, row_table, max_blocks, row_lens, centroids_k,
                       n_centroids_k, centroids_v, n_centroids_v, rotation, int(chunks), chunk,
                       num_q_heads, num_kv_heads, head_dim, block_size, num_blocks, sm_scale, out,
                       num_splits, workspace, workspace_bytes, stream);
}
