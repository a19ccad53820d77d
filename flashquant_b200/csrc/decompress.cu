// TQ4 decompress for sm_100a: nibble codes + fp32 norm -> c[code] * norm in rotated space.
//
// Pure streaming work (68 B in, 2*D or 4*D bytes out per vector).  A thread takes 4 packed
// bytes (one 32-bit load) and produces 8 output values (one or two 16-byte stores), so a
// warp reads 128 contiguous bytes and writes 512 or 1024 contiguous bytes per step.
#include "fq_common.cuh"

namespace fq {

constexpr int kDecompressThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kDecompressThreads) decompress_kernel(
    const uint8_t* __restrict__ packed, const float* __restrict__ norms,
    const float* __restrict__ centroids, int n_centroids, T* __restrict__ out,
    int64_t n_words, int words_per_vec, RowMap in_map) {
  __shared__ float lut[16];
  if (threadIdx.x < 16) lut[threadIdx.x] = threadIdx.x < n_centroids ? centroids[threadIdx.x] : 0.f;
  __syncthreads();
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t w = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; w < n_words; w += stride) {
    const int64_t vec = w / words_per_vec;
    const int64_t row = in_map(vec);
    const uint32_t word =
        reinterpret_cast<const uint32_t*>(packed)[row * words_per_vec + (w - vec * words_per_vec)];
    const float n = norms[row];
    float v[8];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const uint32_t byte = (word >> (8 * b)) & 0xffu;
      v[2 * b] = lut[byte >> 4] * n;
      v[2 * b + 1] = lut[byte & 15u] * n;
    }
    T* o = out + w * 8;
    if constexpr (sizeof(T) == 4) {
      reinterpret_cast<float4*>(o)[0] = make_float4(v[0], v[1], v[2], v[3]);
      reinterpret_cast<float4*>(o)[1] = make_float4(v[4], v[5], v[6], v[7]);
    } else {
      T h[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) h[i] = from_f32<T>(v[i]);
      *reinterpret_cast<uint4*>(o) = *reinterpret_cast<uint4*>(h);
    }
  }
}

}  // namespace fq

using namespace fq;

namespace fq {

int decompress_rows(const uint8_t* packed, const float* norms, const float* centroids,
                    int n_centroids, void* out, int out_dtype, int64_t n_vectors, int head_dim,
                    RowMap in_map, cudaStream_t s) {
  FQ_REQUIRE(n_vectors >= 0, FQ_ERR_INVALID_ARGUMENT, "n_vectors is negative");
  if (n_vectors == 0) return FQ_OK;
  FQ_REQUIRE(packed && norms && centroids && out, FQ_ERR_INVALID_ARGUMENT,
             "fq_tq4_decompress: null pointer");
  FQ_REQUIRE(n_centroids >= 1 && n_centroids <= 16, FQ_ERR_INVALID_ARGUMENT,
             "n_centroids %d outside [1, 16]", n_centroids);
  FQ_REQUIRE(head_dim > 0 && head_dim % 8 == 0, FQ_ERR_UNSUPPORTED,
             "head_dim %d is not a multiple of 8", head_dim);
  FQ_REQUIRE(aligned(packed, 4) && aligned(out, 16) && aligned(norms, 4), FQ_ERR_ALIGNMENT,
             "fq_tq4_decompress: packed must be 4-byte and out 16-byte aligned");
  const int words_per_vec = head_dim / 8;
  const int64_t n_words = n_vectors * words_per_vec;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t want = (n_words + kDecompressThreads - 1) / kDecompressThreads;
  const int grid = int(want < int64_t(sms) * 8 ? want : int64_t(sms) * 8);
  switch (out_dtype) {
    case FQ_F32:
      decompress_kernel<float><<<grid, kDecompressThreads, 0, s>>>(
          packed, norms, centroids, n_centroids, static_cast<float*>(out), n_words, words_per_vec,
          in_map);
      break;
    case FQ_F16:
      decompress_kernel<__half><<<grid, kDecompressThreads, 0, s>>>(
          packed, norms, centroids, n_centroids, static_cast<__half*>(out), n_words, words_per_vec,
          in_map);
      break;
    case FQ_BF16:
      decompress_kernel<__nv_bfloat16><<<grid, kDecompressThreads, 0, s>>>(
          packed, norms, centroids, n_centroids, static_cast<__nv_bfloat16*>(out), n_words,
          words_per_vec, in_map);
      break;
    default:
      return fail(FQ_ERR_INVALID_ARGUMENT, "unknown dtype %d", out_dtype);
  }
  return check_launch("decompress kernel launch");
}

}  // namespace fq

extern "C" int fq_tq4_decompress(const uint8_t* packed, const float* norms,
                                 const float* centroids, int n_centroids, void* out,
                                 fq_dtype out_dtype, int64_t n_vectors, int head_dim,
                                 fq_stream_t stream) {
  FQ_RANGE("fq_tq4_decompress");
  return decompress_rows(packed, norms, centroids, n_centroids, out, int(out_dtype), n_vectors,
                         head_dim, RowMap(), stream);
}

// Decompress to the ORIGINAL space: (c[code] * norm) Pi, rounded to out_dtype.  The codes are
// expanded in fp32 into `workspace` (n_vectors x head_dim floats) and rotated back by the
// split-fp16 tensor-core product (fp32-level accuracy), so the result differs from
// centroids[idx] @ Pi * norm evaluated in fp32 only by fp32 rounding before the final cast.
extern "C" size_t fq_tq4_decompress_original_workspace_bytes(int64_t n_vectors, int head_dim) {
  if (n_vectors < 0 || head_dim < 0) return 0;
  return size_t(n_vectors) * size_t(head_dim) * sizeof(float);
}

extern "C" int fq_tq4_decompress_original(const uint8_t* packed, const float* norms,
                                          const float* centroids, int n_centroids,
                                          const float* rotation, void* out, fq_dtype out_dtype,
                                          int64_t n_vectors, int head_dim, void* workspace,
                                          size_t workspace_bytes, fq_stream_t stream) {
  FQ_RANGE("fq_tq4_decompress_original");
  FQ_REQUIRE(n_vectors >= 0, FQ_ERR_INVALID_ARGUMENT, "n_vectors is negative");
  if (n_vectors == 0) return FQ_OK;
  FQ_REQUIRE(rotation && out, FQ_ERR_INVALID_ARGUMENT, "fq_tq4_decompress_original: null pointer");
  FQ_REQUIRE(head_dim == 64 || head_dim == 128, FQ_ERR_UNSUPPORTED,
             "head_dim %d: the rotation kernels are built for 64 and 128", head_dim);
  FQ_REQUIRE(out_dtype == FQ_F32 || out_dtype == FQ_F16 || out_dtype == FQ_BF16,
             FQ_ERR_INVALID_ARGUMENT, "unknown dtype %d", int(out_dtype));
  const size_t need = fq_tq4_decompress_original_workspace_bytes(n_vectors, head_dim);
  FQ_REQUIRE(workspace && aligned(workspace, 16) && workspace_bytes >= need, FQ_ERR_WORKSPACE,
             "fq_tq4_decompress_original: workspace of %zu bytes needed (16-byte aligned)", need);
  FQ_REQUIRE(aligned(out, 16) && aligned(rotation, 16), FQ_ERR_ALIGNMENT,
             "fq_tq4_decompress_original: out and rotation must be 16-byte aligned");
  if (rotate_is_few_rows(n_vectors)) {
    FQ_REQUIRE(packed && norms && centroids, FQ_ERR_INVALID_ARGUMENT,
               "fq_tq4_decompress_original: null pointer");
    FQ_REQUIRE(n_centroids >= 1 && n_centroids <= 16, FQ_ERR_INVALID_ARGUMENT,
               "n_centroids %d outside [1, 16]", n_centroids);
    return rotate_back_from_codes(packed, norms, centroids, n_centroids, RowMap(), int(out_dtype),
                                  rotation, out, n_vectors, head_dim, stream, RowMap());
  }
  int rc = fq_tq4_decompress(packed, norms, centroids, n_centroids, workspace, FQ_F32, n_vectors,
                             head_dim, stream);
  if (rc != FQ_OK) return rc;
  return rotate_back(static_cast<const float*>(workspace), int(out_dtype), rotation, out,
                     n_vectors, head_dim, stream);
}
