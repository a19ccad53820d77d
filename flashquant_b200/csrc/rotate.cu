// Row rotation for sm_100a: out[r] = round_T(x[r] Pi^T) or round_T(x[r] Pi).
//
// Used around the prefill attention kernel, which works in rotated space: the query rows go
// through Pi^T before it, the attention rows through Pi after it.  The reference does both
// as fp32 matmuls followed by a cast to the activation type
// (src/flashquant/kernels/attention.py:99-101, src/flashquant/kernels/cpu_reference.py:225-226),
// so the contraction here has fp32-level accuracy as well and only the result is rounded:
// head_dim 128 runs on the tensor pipe with split-fp16 operands (below), head_dim 64 as an
// fp32 FMA contraction (persistent CTAs keep the matrix in shared memory; a warp owns 8 rows
// of a 64-row tile, a lane 2 consecutive output coordinates).
#include "fq_common.cuh"

namespace fq {

constexpr int kRotThreads = 256;
constexpr int kRotTile = 64;

template <int D, typename TIn, typename TOut, bool kTranspose, bool kRoundViaIn>
__global__ void __launch_bounds__(kRotThreads, 1) rotate_rows_kernel(
    const TIn* __restrict__ x, const float* __restrict__ rotation, TOut* __restrict__ out,
    int64_t n_rows, RowMap out_map) {
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
      TOut* dst = out + out_map(r0 + v) * D + lane * JT;
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

// ------------------------------------------------------------------------------------
// head_dim 128 on the tensor pipe.  Products of fp32-level accuracy from fp16 MMAs: every
// operand is split into hi = fp16(v) and lo' = fp16((v - hi) * 2^11); hi*hi goes to one fp32
// accumulator, hi*lo' + lo'*hi to a second one scaled by 2^-11 at the end (lo*lo, 2^-22 of a
// product, is dropped).  The matrix stays in shared memory as hi / lo' planes; a warp owns
// 16 rows end to end: their fragments come straight from global memory and stay in
// registers while the warp walks the 16 column tiles four at a time (ldmatrix for the matrix
// fragments), so the row loop has no barrier.
// ------------------------------------------------------------------------------------
constexpr int kRtThreads = 256;
constexpr int kRtLd = 128 + 8;  // halves per plane row: ldmatrix rows then hit 32 banks

__device__ __forceinline__ void rt_split(float v, __half& hi, __half& lo) {
  hi = __float2half_rn(v);
  lo = __float2half_rn((v - __half2float(hi)) * 2048.f);
}
__device__ __forceinline__ uint32_t rt_pack(__half a, __half b) {
  return uint32_t(__half_as_ushort(a)) | (uint32_t(__half_as_ushort(b)) << 16);
}
__device__ __forceinline__ float2 rt_load2(const float* p) {
  return *reinterpret_cast<const float2*>(p);
}
__device__ __forceinline__ float2 rt_load2(const __half* p) {
  return __half22float2(*reinterpret_cast<const __half2*>(p));
}
__device__ __forceinline__ float2 rt_load2(const __nv_bfloat16* p) {
  const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <typename TOut>
__device__ __forceinline__ void rt_store2(TOut* p, float a, float b);
template <>
__device__ __forceinline__ void rt_store2<__half>(__half* p, float a, float b) {
  *reinterpret_cast<__half2*>(p) = __floats2half2_rn(a, b);
}
template <>
__device__ __forceinline__ void rt_store2<__nv_bfloat16>(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}
template <>
__device__ __forceinline__ void rt_store2<float>(float* p, float a, float b) {
  *reinterpret_cast<float2*>(p) = make_float2(a, b);
}

template <typename TIn, typename TOut, bool kTranspose, bool kRoundViaIn>
__global__ void __launch_bounds__(kRtThreads, 2) rotate_rows_tc_kernel(
    const TIn* __restrict__ x, const float* __restrict__ rotation, TOut* __restrict__ out,
    int64_t n_rows, RowMap out_map) {
  constexpr int D = 128;
  extern __shared__ __align__(16) unsigned char rt_smem[];
  __half* b_hi = reinterpret_cast<__half*>(rt_smem);  // plane[n][k] = B[k][n]
  __half* b_lo = b_hi + D * kRtLd;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  // out = x Pi^T: B[k][n] = Pi[n][k] (the matrix as it is); out = x Pi: B[k][n] = Pi[k][n]
  for (int b0 = 0; b0 < D * D / kRtThreads; b0 += 16) {
    float v[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) v[u] = rotation[tid + (b0 + u) * kRtThreads];  // coalesced
#pragma unroll
    for (int u = 0; u < 16; ++u) {
      const int i = tid + (b0 + u) * kRtThreads;
      const int r = i / D, c = i % D;  // element Pi[r][c]
      const int n = kTranspose ? r : c, k = kTranspose ? c : r;
      __half h, l;
      rt_split(v[u], h, l);
      b_hi[n * kRtLd + k] = h;
      b_lo[n * kRtLd + k] = l;
    }
  }
  __syncthreads();

  const int j = lane >> 3, r8 = lane & 7;  // ldmatrix: lanes 8j..8j+7 give the rows of matrix j
  // matrix j = plane j>>1 (hi, lo'), k-segment j&1 of the column tile's 8 rows
  const __half* pb = ((j >> 1) ? b_lo : b_hi) + r8 * kRtLd + 8 * (j & 1);
  const int64_t n_mtiles = (n_rows + 15) / 16;
  for (int64_t mt = int64_t(blockIdx.x) * (kRtThreads / 32) + warp; mt < n_mtiles;
       mt += int64_t(gridDim.x) * (kRtThreads / 32)) {
    const int64_t r0 = mt * 16 + g, r1 = r0 + 8;
    const bool ok0 = r0 < n_rows, ok1 = r1 < n_rows;
    const int64_t o0 = out_map(r0), o1 = out_map(r1);
    const TIn* x0 = x + (ok0 ? r0 : 0) * D + 2 * t;
    const TIn* x1 = x + (ok1 ? r1 : 0) * D + 2 * t;
    uint32_t xh[D / 16][4], xl[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      float2 f[4];
      f[0] = ok0 ? rt_load2(x0 + 16 * ks) : make_float2(0.f, 0.f);
      f[1] = ok1 ? rt_load2(x1 + 16 * ks) : make_float2(0.f, 0.f);
      f[2] = ok0 ? rt_load2(x0 + 16 * ks + 8) : make_float2(0.f, 0.f);
      f[3] = ok1 ? rt_load2(x1 + 16 * ks + 8) : make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        __half h0, l0, h1, l1;
        rt_split(f[i].x, h0, l0);
        rt_split(f[i].y, h1, l1);
        xh[ks][i] = rt_pack(h0, h1);
        xl[ks][i] = rt_pack(l0, l1);
      }
    }
#pragma unroll 1
    for (int grp = 0; grp < 4; ++grp) {  // column tiles 4*grp .. 4*grp+3
      float hi[4][4], co[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) hi[i][c] = co[i][c] = 0.f;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t b[4];  // b0 hi, b1 hi, b0 lo', b1 lo'
          asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                       : "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3])
                       : "r"(smem_u32(pb + (grp * 4 + i) * 8 * kRtLd + 16 * ks)));
          mma_f16(hi[i], xh[ks][0], xh[ks][1], xh[ks][2], xh[ks][3], b[0], b[1]);
          mma_f16(co[i], xh[ks][0], xh[ks][1], xh[ks][2], xh[ks][3], b[2], b[3]);
          mma_f16(co[i], xl[ks][0], xl[ks][1], xl[ks][2], xl[ks][3], b[0], b[1]);
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float v[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          v[c] = fmaf(co[i][c], 1.f / 2048.f, hi[i][c]);
          if constexpr (kRoundViaIn) v[c] = to_f32(from_f32<TIn>(v[c]));  // round to x's type first
        }
        const int col = 8 * (grp * 4 + i) + 2 * t;
        if (ok0) rt_store2<TOut>(out + o0 * D + col, v[0], v[1]);
        if (ok1) rt_store2<TOut>(out + o1 * D + col, v[2], v[3]);
      }
    }
  }
}

template <typename TIn, typename TOut, bool kTranspose, bool kRoundViaIn>
static int launch_rotate_tc(const void* x, const float* rotation, void* out, int64_t n_rows,
                            cudaStream_t stream, RowMap out_map = RowMap()) {
  const size_t smem = size_t(2) * 128 * kRtLd * sizeof(__half);
  auto kern = rotate_rows_tc_kernel<TIn, TOut, kTranspose, kRoundViaIn>;
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
  const int64_t warp_tiles = (n_rows + 15) / 16;
  if (warp_tiles == 0) return FQ_OK;
  const int64_t ctas_needed = (warp_tiles + kRtThreads / 32 - 1) / (kRtThreads / 32);
  const int grid = int(ctas_needed < 2 * int64_t(sms) ? ctas_needed : 2 * int64_t(sms));
  kern<<<grid, kRtThreads, smem, stream>>>(static_cast<const TIn*>(x), rotation,
                                          static_cast<TOut*>(out), n_rows, out_map);
  return check_launch("rotate kernel launch");
}

template <int D, typename TIn, typename TOut, bool kTranspose, bool kRoundViaIn>
static int launch_rotate_t(const void* x, const float* rotation, void* out, int64_t n_rows,
                           cudaStream_t stream, RowMap out_map = RowMap()) {
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
                                           static_cast<TOut*>(out), n_rows, out_map);
  return check_launch("rotate kernel launch");
}

// ------------------------------------------------------------------------------------
// A few rows (the query or the output of one decode step): staging the matrix in shared
// memory would cost more than the product.  One thread per output column, kFewRows rows per
// CTA, the matrix read straight through L1/L2 in fp32 FMAs.  With `part` the input row is
// first merged from the partial rows of n_splits key slices, [o (D) | m | l | - | -] at
// part[(split * n_rows + row) * (D + 4)]: o = sum 2^(m_i - M) o_i / sum 2^(m_i - M) l_i.
// ------------------------------------------------------------------------------------
constexpr int kFewRows = 4;
constexpr int64_t kFewRowsMax = 1024;  // above this the tensor-core kernel wins

// Input rows given as nibble codes + norm (row r of the product is row map(r) of the buffers):
// value j of a row is centroids[code_j] * norm, code_2i the high nibble of byte i.
struct CodeRows {
  const uint8_t* codes = nullptr;
  const float* norms = nullptr;
  const float* centroids = nullptr;
  int n_centroids = 0;
  RowMap map;
};

// kFewRows * D threads.  Every thread reads D/16 or D/4 consecutive floats of the matrix as
// float4, adjacent threads adjacent chunks (coalesced, few loads in a row per thread):
//   x Pi^T: thread (j, slice of D/4 k) -> partial of column j, summed over 4 adjacent lanes;
//   x Pi:   thread (4 columns, slice of D/16 k) -> partials summed over 16 slices in shared memory.
template <int D, typename TIn, typename TOut, bool kTranspose, bool kRoundViaIn>
__global__ void __launch_bounds__(kFewRows * D) rotate_few_rows_kernel(
    const TIn* __restrict__ x, const float* __restrict__ rotation, TOut* __restrict__ out,
    int64_t n_rows, RowMap out_map, const float* __restrict__ part, int n_splits, CodeRows cr) {
  static_assert(kFewRows == 4, "thread maps below");
  __shared__ __align__(16) float xs[kFewRows][D];
  __shared__ __align__(16) float red[kTranspose ? 1 : 16][kFewRows][D];
  const int t = threadIdx.x;
  const int64_t r0 = int64_t(blockIdx.x) * kFewRows;
  {
    const int r = t / D, j = t % D;
    float v = 0.f;
    if (r0 + r < n_rows) {
      if (part) {
        float m_max = -INFINITY;
        for (int s = 0; s < n_splits; ++s)
          m_max = fmaxf(m_max, part[(int64_t(s) * n_rows + r0 + r) * (D + 4) + D]);
        float acc = 0.f, l = 0.f;
        for (int s = 0; s < n_splits; ++s) {
          const float* pr = part + (int64_t(s) * n_rows + r0 + r) * (D + 4);
          const float m = pr[D];
          if (m == -INFINITY) continue;
          const float w = fast_exp2(m - m_max);
          acc = fmaf(w, pr[j], acc);
          l = fmaf(w, pr[D + 1], l);
        }
        v = l > 0.f ? acc / l : 0.f;
      } else if (cr.codes) {
        const int64_t row_in = cr.map(r0 + r);
        const uint32_t byte = cr.codes[row_in * (D / 2) + (j >> 1)];
        const int code = (j & 1) ? int(byte & 15u) : int(byte >> 4);
        v = (code < cr.n_centroids ? cr.centroids[code] : 0.f) * cr.norms[row_in];
      } else {
        v = to_f32(x[(r0 + r) * D + j]);
      }
    }
    xs[r][j] = v;
  }
  __syncthreads();
  auto store = [&](int r, int j, float v) {
    if (r0 + r >= n_rows) return;
    if constexpr (kRoundViaIn) v = to_f32(from_f32<TIn>(v));  // round to x's type first
    out[out_map(r0 + r) * D + j] = from_f32<TOut>(v);
  };
  if constexpr (kTranspose) {  // out[r][j] = sum_k x[r][k] Pi[j][k]
    const int j = t >> 2, sl = t & 3;
    constexpr int kLen = D / 4;
    const float4* prow = reinterpret_cast<const float4*>(rotation + j * D + sl * kLen);
    float4 b[kLen / 4];
#pragma unroll
    for (int i = 0; i < kLen / 4; ++i) b[i] = prow[i];
    float acc[kFewRows];
#pragma unroll
    for (int r = 0; r < kFewRows; ++r) {
      acc[r] = 0.f;
#pragma unroll
      for (int i = 0; i < kLen / 4; ++i) {
        const float4 a = *reinterpret_cast<const float4*>(&xs[r][sl * kLen + 4 * i]);
        acc[r] = fmaf(a.x, b[i].x, acc[r]);
        acc[r] = fmaf(a.y, b[i].y, acc[r]);
        acc[r] = fmaf(a.z, b[i].z, acc[r]);
        acc[r] = fmaf(a.w, b[i].w, acc[r]);
      }
      acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], 1);
      acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], 2);
    }
    if (sl == 0) {
#pragma unroll
      for (int r = 0; r < kFewRows; ++r) store(r, j, acc[r]);
    }
  } else {  // out[r][j] = sum_k x[r][k] Pi[k][j]
    constexpr int kCols4 = D / 4, kLen = D / 16;
    const int c4 = t % kCols4, ks = t / kCols4;
    float4 b[kLen];
#pragma unroll
    for (int i = 0; i < kLen; ++i)
      b[i] = *reinterpret_cast<const float4*>(rotation + (ks * kLen + i) * D + 4 * c4);
#pragma unroll
    for (int r = 0; r < kFewRows; ++r) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < kLen; ++i) {
        const float a = xs[r][ks * kLen + i];
        acc.x = fmaf(a, b[i].x, acc.x); acc.y = fmaf(a, b[i].y, acc.y);
        acc.z = fmaf(a, b[i].z, acc.z); acc.w = fmaf(a, b[i].w, acc.w);
      }
      *reinterpret_cast<float4*>(&red[ks][r][4 * c4]) = acc;
    }
    __syncthreads();
    const int r = t / D, j = t % D;
    float v = 0.f;
#pragma unroll
    for (int s = 0; s < 16; ++s) v += red[s][r][j];
    store(r, j, v);
  }
}

template <int D, typename TIn, typename TOut, bool kTranspose, bool kRoundViaIn>
static int launch_rotate_few(const void* x, const float* rotation, void* out, int64_t n_rows,
                             cudaStream_t stream, RowMap out_map, const float* part = nullptr,
                             int n_splits = 0, CodeRows cr = CodeRows()) {
  if (n_rows == 0) return FQ_OK;
  rotate_few_rows_kernel<D, TIn, TOut, kTranspose, kRoundViaIn>
      <<<unsigned((n_rows + kFewRows - 1) / kFewRows), kFewRows * D, 0, stream>>>(
          static_cast<const TIn*>(x), rotation, static_cast<TOut*>(out), n_rows, out_map, part,
          n_splits, cr);
  return check_launch("rotate kernel launch");
}

template <int D, bool kTranspose, bool kRoundViaIn, typename TIn>
static int rotate_few_out(const void* x, int out_dtype, const float* rotation, void* out,
                          int64_t n_rows, cudaStream_t stream, RowMap m, const float* part,
                          int n_splits, CodeRows cr = CodeRows()) {
  switch (out_dtype) {
    case FQ_F32:
      return launch_rotate_few<D, TIn, float, kTranspose, kRoundViaIn>(
          x, rotation, out, n_rows, stream, m, part, n_splits, cr);
    case FQ_F16:
      return launch_rotate_few<D, TIn, __half, kTranspose, kRoundViaIn>(
          x, rotation, out, n_rows, stream, m, part, n_splits, cr);
    case FQ_BF16:
      return launch_rotate_few<D, TIn, __nv_bfloat16, kTranspose, kRoundViaIn>(
          x, rotation, out, n_rows, stream, m, part, n_splits, cr);
  }
  return fail(FQ_ERR_INVALID_ARGUMENT, "unknown dtype %d", out_dtype);
}

// merged partial rows of key slices -> round_dtype(o Pi) in one launch (few rows only)
int rotate_back_merged(const float* part, int n_splits, int dtype, const float* rotation,
                       void* out, int64_t n_rows, int head_dim, cudaStream_t stream) {
  if (head_dim == 128)
    return rotate_few_out<128, false, false, float>(nullptr, dtype, rotation, out, n_rows, stream,
                                                    RowMap(), part, n_splits);
  return rotate_few_out<64, false, false, float>(nullptr, dtype, rotation, out, n_rows, stream,
                                                 RowMap(), part, n_splits);
}
bool rotate_is_few_rows(int64_t n_rows) { return n_rows <= kFewRowsMax; }

// codes + norms (rows through in_map) -> round_dtype((c[code] n) Pi) in one launch (few rows only)
int rotate_back_from_codes(const uint8_t* codes, const float* norms, const float* centroids,
                           int n_centroids, RowMap in_map, int dtype, const float* rotation,
                           void* out, int64_t n_rows, int head_dim, cudaStream_t stream,
                           RowMap out_map) {
  CodeRows cr;
  cr.codes = codes; cr.norms = norms; cr.centroids = centroids; cr.n_centroids = n_centroids;
  cr.map = in_map;
  if (head_dim == 128)
    return rotate_few_out<128, false, false, float>(nullptr, dtype, rotation, out, n_rows, stream,
                                                    out_map, nullptr, 0, cr);
  return rotate_few_out<64, false, false, float>(nullptr, dtype, rotation, out, n_rows, stream,
                                                 out_map, nullptr, 0, cr);
}

// q (dtype) -> fp16 copy of round_dtype(q Pi^T)
int rotate_q_to_half(const void* q, int dtype, const float* rotation, __half* out,
                     int64_t n_rows, int head_dim, cudaStream_t stream) {
  if (n_rows <= kFewRowsMax) {
    if (head_dim == 128)
      return dtype == FQ_BF16
                 ? launch_rotate_few<128, __nv_bfloat16, __half, true, true>(q, rotation, out, n_rows, stream, RowMap())
                 : launch_rotate_few<128, __half, __half, true, true>(q, rotation, out, n_rows, stream, RowMap());
    return dtype == FQ_BF16
               ? launch_rotate_few<64, __nv_bfloat16, __half, true, true>(q, rotation, out, n_rows, stream, RowMap())
               : launch_rotate_few<64, __half, __half, true, true>(q, rotation, out, n_rows, stream, RowMap());
  }
  if (head_dim == 128)
    return dtype == FQ_BF16
               ? launch_rotate_tc<__nv_bfloat16, __half, true, true>(q, rotation, out, n_rows, stream)
               : launch_rotate_tc<__half, __half, true, true>(q, rotation, out, n_rows, stream);
  return dtype == FQ_BF16
             ? launch_rotate_t<64, __nv_bfloat16, __half, true, true>(q, rotation, out, n_rows, stream)
             : launch_rotate_t<64, __half, __half, true, true>(q, rotation, out, n_rows, stream);
}

// o_rot (fp32) -> round_dtype(o_rot Pi); row r of the result goes to row out_map(r) of `out`
int rotate_back(const float* o_rot, int dtype, const float* rotation, void* out, int64_t n_rows,
                int head_dim, cudaStream_t stream, RowMap m) {
  if (n_rows <= kFewRowsMax)
    return head_dim == 128
               ? rotate_few_out<128, false, false, float>(o_rot, dtype, rotation, out, n_rows, stream, m, nullptr, 0)
               : rotate_few_out<64, false, false, float>(o_rot, dtype, rotation, out, n_rows, stream, m, nullptr, 0);
  if (dtype == FQ_F32)
    return head_dim == 128
               ? launch_rotate_tc<float, float, false, false>(o_rot, rotation, out, n_rows, stream, m)
               : launch_rotate_t<64, float, float, false, false>(o_rot, rotation, out, n_rows, stream, m);
  if (head_dim == 128)
    return dtype == FQ_BF16
               ? launch_rotate_tc<float, __nv_bfloat16, false, false>(o_rot, rotation, out, n_rows, stream, m)
               : launch_rotate_tc<float, __half, false, false>(o_rot, rotation, out, n_rows, stream, m);
  return dtype == FQ_BF16
             ? launch_rotate_t<64, float, __nv_bfloat16, false, false>(o_rot, rotation, out, n_rows, stream, m)
             : launch_rotate_t<64, float, __half, false, false>(o_rot, rotation, out, n_rows, stream, m);
}

}  // namespace fq
