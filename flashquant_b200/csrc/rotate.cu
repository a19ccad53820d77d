// Row rotation for sm_100a: out[r] = round_T(x[r] Pi^T) or round_T(x[r] Pi), fp32 FMA.
//
// Used around the prefill attention kernel, which works in rotated space: the query rows go
// through Pi^T before it, the attention rows through Pi after it.  The reference does both
// as fp32 matmuls followed by a cast to the activation type
// (src/flashquant/kernels/attention.py:99-101, src/flashquant/kernels/cpu_reference.py:225-226),
// so the contraction here is fp32 as well and only the result is rounded.
//
// Persistent CTAs keep the matrix in shared memory; a warp owns 8 rows of a 64-row tile, a
// lane 4 consecutive output coordinates (head_dim 128) or 2 (head_dim 64).
#include "fq_common.cuh"

namespace fq {

constexpr int kRotThreads = 256;
constexpr int kRotTile = 64;

template <int D, typename TIn, typename TOut, bool kTranspose, bool kRoundViaIn>
__global__ void __launch_bounds__(kRotThreads, 1) rotate_rows_kernel(
    const TIn* __restrict__ x, const float* __restrict__ rotation, TOut* __restrict__ out,
    int64_t n_rows) {
  constexpr int JT = D / 32;
  constexpr int VPW = kRotTile / 8;
  constexpr int LDA = D + 4;
  extern __shared__ __align__(16) unsigned char rot_smem[];
  float* bmat = reinterpret_cast<float*>(rot_smem);  // [k][j]
  float* a_tile = bmat + D * D;                      // [64][LDA]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < D * D; i += kRotThreads) {
    const int k = i / D, j = i % D;
    bmat[i] = kTranspose ? rotation[j * D + k] : rotation[i];
  }
  __syncthreads();
  const int64_t n_tiles = (n_rows + kRotTile - 1) / kRotTile;
  float* a_rows = a_tile + warp * VPW * LDA;
  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    const int64_t r0 = tile * kRotTile + warp * VPW;
#pragma unroll
    for (int v = 0; v < VPW; ++v) {
      float xv[JT];
      if (r0 + v < n_rows) {
        const TIn* src = x + (r0 + v) * D + lane * JT;
        if constexpr (JT == 4) load4(src, xv); else load2(src, xv);
      } else {
#pragma unroll
        for (int j = 0; j < JT; ++j) xv[j] = 0.f;
      }
      float* ar = a_rows + v * LDA + lane * JT;
#pragma unroll
      for (int j = 0; j < JT; ++j) ar[j] = xv[j];
    }
    __syncwarp();
    float acc[VPW][JT];
#pragma unroll
    for (int v = 0; v < VPW; ++v)
#pragma unroll
      for (int j = 0; j < JT; ++j) acc[v][j] = 0.f;
#pragma unroll 2
    for (int k4 = 0; k4 < D; k4 += 4) {
      float bb[4][JT];
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const float* bp = bmat + (k4 + kk) * D + lane * JT;
        if constexpr (JT == 4) {
          const float4 t4 = *reinterpret_cast<const float4*>(bp);
          bb[kk][0] = t4.x; bb[kk][1] = t4.y; bb[kk][2] = t4.z; bb[kk][3] = t4.w;
        } else {
          const float2 t2 = *reinterpret_cast<const float2*>(bp);
          bb[kk][0] = t2.x; bb[kk][1] = t2.y;
        }
      }
#pragma unroll
      for (int v = 0; v < VPW; ++v) {
        const float4 a = *reinterpret_cast<const float4*>(a_rows + v * LDA + k4);
#pragma unroll
        for (int j = 0; j < JT; ++j) {
          acc[v][j] = fmaf(a.x, bb[0][j], acc[v][j]);
          acc[v][j] = fmaf(a.y, bb[1][j], acc[v][j]);
          acc[v][j] = fmaf(a.z, bb[2][j], acc[v][j]);
          acc[v][j] = fmaf(a.w, bb[3][j], acc[v][j]);
        }
      }
    }
    __syncwarp();
#pragma unroll
    for (int v = 0; v < VPW; ++v) {
      if (r0 + v >= n_rows) continue;
      TOut* dst = out + (r0 + v) * D + lane * JT;
      TOut o[JT];
#pragma unroll
      for (int j = 0; j < JT; ++j) {
        float val = acc[v][j];
        if constexpr (kRoundViaIn) val = to_f32(from_f32<TIn>(val));  // round to x's type first
        o[j] = from_f32<TOut>(val);
      }
      if constexpr (sizeof(TOut) == 2) {
        if constexpr (JT == 4) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<uint2*>(o);
        else *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<uint32_t*>(o);
      } else {
#pragma unroll
        for (int j = 0; j < JT; ++j) dst[j] = o[j];
      }
    }
  }
}

template <int D, typename TIn, typename TOut, bool kTranspose, bool kRoundViaIn>
static int launch_rotate_t(const void* x, const float* rotation, void* out, int64_t n_rows,
                           cudaStream_t stream) {
  const size_t smem = (size_t(D) * D + size_t(kRotTile) * (D + 4)) * sizeof(float);
  auto kern = rotate_rows_kernel<D, TIn, TOut, kTranspose, kRoundViaIn>;
  static thread_local int set_dev = -1;
  static thread_local int sms = 148;
  int dev = 0;
  cudaGetDevice(&dev);
  if (set_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess)
      return fail(FQ_ERR_CUDA, "rotate: shared memory opt-in refused: %s", cudaGetErrorString(e));
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    set_dev = dev;
  }
  const int64_t tiles = (n_rows + kRotTile - 1) / kRotTile;
  if (tiles == 0) return FQ_OK;
  const int grid = int(tiles < 2 * int64_t(sms) ? tiles : 2 * int64_t(sms));
  kern<<<grid, kRotThreads, smem, stream>>>(static_cast<const TIn*>(x), rotation,
                                           static_cast<TOut*>(out), n_rows);
  return check_launch("rotate kernel launch");
}

// q (dtype) -> fp16 copy of round_dtype(q Pi^T)
int rotate_q_to_half(const void* q, int dtype, const float* rotation, __half* out,
                     int64_t n_rows, int head_dim, cudaStream_t stream) {
  if (head_dim == 128)
    return dtype == FQ_BF16
               ? launch_rotate_t<128, __nv_bfloat16, __half, true, true>(q, rotation, out, n_rows, stream)
               : launch_rotate_t<128, __half, __half, true, true>(q, rotation, out, n_rows, stream);
  return dtype == FQ_BF16
             ? launch_rotate_t<64, __nv_bfloat16, __half, true, true>(q, rotation, out, n_rows, stream)
             : launch_rotate_t<64, __half, __half, true, true>(q, rotation, out, n_rows, stream);
}

// o_rot (fp32) -> round_dtype(o_rot Pi)
int rotate_back(const float* o_rot, int dtype, const float* rotation, void* out, int64_t n_rows,
                int head_dim, cudaStream_t stream) {
  if (head_dim == 128)
    return dtype == FQ_BF16
               ? launch_rotate_t<128, float, __nv_bfloat16, false, false>(o_rot, rotation, out, n_rows, stream)
               : launch_rotate_t<128, float, __half, false, false>(o_rot, rotation, out, n_rows, stream);
  return dtype == FQ_BF16
             ? launch_rotate_t<64, float, __nv_bfloat16, false, false>(o_rot, rotation, out, n_rows, stream)
             : launch_rotate_t<64, float, __half, false, false>(o_rot, rotation, out, n_rows, stream);
}

}  // namespace fq
