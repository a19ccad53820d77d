// One update of a contiguous compressed cache in one host call: the new keys and values are
// compressed into their rows of the pre-allocated buffers and, unless the caller attends over
// the codes directly, those rows are de-quantised to the original space and written behind
// the tokens the caller already holds.  Four launches on one stream for a few new rows (the
// back-rotation expands the codes on its way in), six otherwise; no allocation, no
// synchronisation.
#include "fq_common.cuh"

using namespace fq;

extern "C" size_t fq_cache_update_workspace_bytes(int64_t n_segments, int64_t n_new,
                                                  int head_dim) {
  if (n_segments < 0 || n_new < 0 || head_dim < 0) return 0;
  return size_t(n_segments) * size_t(n_new) * size_t(head_dim) * sizeof(float);
}

extern "C" int fq_cache_update(
    const void* key, const void* value, fq_dtype dtype, const float* rot_T_even_k,
    const float* rot_T_odd_k, const float* rotation_k, const float* rot_T_even_v,
    const float* rot_T_odd_v, const float* rotation_v, const float* boundaries, int n_boundaries,
    const float* centroids, int n_centroids, uint8_t* k_packed, float* k_norms,
    uint8_t* v_packed, float* v_norms, int64_t n_segments, int64_t n_new, int64_t capacity,
    int64_t position, void* k_out, void* v_out, int64_t out_capacity, int64_t out_position,
    int head_dim, void* workspace, size_t workspace_bytes, fq_stream_t stream) {
  FQ_RANGE("fq_cache_update");
  FQ_REQUIRE(n_segments >= 0 && n_new >= 0 && capacity >= 0 && position >= 0,
             FQ_ERR_INVALID_ARGUMENT, "fq_cache_update: negative size");
  FQ_REQUIRE(position + n_new <= capacity, FQ_ERR_INVALID_ARGUMENT,
             "fq_cache_update: %lld tokens at position %lld exceed the capacity %lld",
             (long long)n_new, (long long)position, (long long)capacity);
  if (n_segments == 0 || n_new == 0) return FQ_OK;  // an update without tokens
  FQ_REQUIRE(key && value && k_packed && k_norms && v_packed && v_norms, FQ_ERR_INVALID_ARGUMENT,
             "fq_cache_update: null pointer");
  const bool dequantise = k_out != nullptr || v_out != nullptr;
  if (dequantise) {
    FQ_REQUIRE(k_out && v_out && rotation_k && rotation_v && centroids, FQ_ERR_INVALID_ARGUMENT,
               "fq_cache_update: null pointer");
    FQ_REQUIRE(out_position >= 0 && out_position + n_new <= out_capacity,
               FQ_ERR_INVALID_ARGUMENT,
               "fq_cache_update: %lld tokens at position %lld exceed the output capacity %lld",
               (long long)n_new, (long long)out_position, (long long)out_capacity);
    // a few rows are expanded inside the rotation kernel and need no workspace
    const size_t need = rotate_is_few_rows(n_segments * n_new)
                            ? 0 : fq_cache_update_workspace_bytes(n_segments, n_new, head_dim);
    FQ_REQUIRE(need == 0 || (workspace && aligned(workspace, 16) && workspace_bytes >= need),
               FQ_ERR_WORKSPACE, "fq_cache_update: workspace of %zu bytes needed (16-byte aligned)",
               need);
    FQ_REQUIRE(aligned(k_out, 16) && aligned(v_out, 16) && aligned(rotation_k, 16) &&
                   aligned(rotation_v, 16),
               FQ_ERR_ALIGNMENT, "fq_cache_update: outputs and rotations must be 16-byte aligned");
    FQ_REQUIRE(n_centroids >= 1 && n_centroids <= 16, FQ_ERR_INVALID_ARGUMENT,
               "n_centroids %d outside [1, 16]", n_centroids);
  }
  int rc = fq_tq4_compress_into(key, dtype, rot_T_even_k, rot_T_odd_k, boundaries, n_boundaries,
                                k_packed, k_norms, n_segments, n_new, capacity, position,
                                head_dim, stream);
  if (rc != FQ_OK) return rc;
  rc = fq_tq4_compress_into(value, dtype, rot_T_even_v, rot_T_odd_v, boundaries, n_boundaries,
                            v_packed, v_norms, n_segments, n_new, capacity, position, head_dim,
                            stream);
  if (rc != FQ_OK || !dequantise) return rc;
  const int64_t n_vec = n_segments * n_new;
  if (n_vec == 0) return FQ_OK;
  FQ_REQUIRE(head_dim == 64 || head_dim == 128, FQ_ERR_UNSUPPORTED,
             "head_dim %d: the rotation kernels are built for 64 and 128", head_dim);
  RowMap in_map, out_map;
  in_map.seg_len = out_map.seg_len = uint32_t(n_new);
  in_map.seg_stride = capacity; in_map.seg_offset = position;
  out_map.seg_stride = out_capacity; out_map.seg_offset = out_position;
  const uint8_t* codes[2] = {k_packed, v_packed};
  const float* norms[2] = {k_norms, v_norms};
  const float* rot[2] = {rotation_k, rotation_v};
  void* outs[2] = {k_out, v_out};
  if (rotate_is_few_rows(n_vec)) {
    for (int s = 0; s < 2; ++s) {
      rc = rotate_back_from_codes(codes[s], norms[s], centroids, n_centroids, in_map, int(dtype),
                                  rot[s], outs[s], n_vec, head_dim, stream, out_map);
      if (rc != FQ_OK) return rc;
    }
    return FQ_OK;
  }
  for (int s = 0; s < 2; ++s) {
    // the workspace is reused for the values: the launches are ordered on the stream
    rc = decompress_rows(codes[s], norms[s], centroids, n_centroids, workspace, FQ_F32, n_vec,
                         head_dim, in_map, stream);
    if (rc != FQ_OK) return rc;
    rc = rotate_back(static_cast<const float*>(workspace), int(dtype), rot[s], outs[s], n_vec,
                     head_dim, stream, out_map);
    if (rc != FQ_OK) return rc;
  }
  return FQ_OK;
}
