// TQ4 compress / compress-on-append / two-stage (QJL) quantiser for sm_100a.
//
// One persistent CTA per SM keeps the rotation (and, for the two-stage quantiser, Pi and
// S^T as well) resident in shared memory as fp32 and walks over tiles of vectors.  The
// rotation is an fp32 FMA contraction in the reference's operation order (normalise, then
// rotate), because the 4-bit codes must match a CPU sgemm to within the spacing of fp32:
// a coordinate closer than ~1e-7 to a Lloyd-Max boundary may land on either side.
//
// Work split inside a CTA of 8 warps: a warp owns TV/8 vectors of the tile end to end
// (load, norm, three contractions, pack, store), a lane owns D/32 consecutive output
// coordinates of each of them.  Nothing but the matrices is shared between warps, so the
// tile loop needs no block-wide barrier.
#include "fq_common.cuh"

namespace fq {

constexpr int kCompressThreads = 256;
constexpr int kCompressWarps = 8;

struct CompressArgs {
  const void* src[2];  // [0]: K (or the only source), [1]: V
  int n_src;
  int64_t n_tokens;
  int heads;
  int64_t token_stride;  // elements between consecutive tokens of a source
  const float* mat_a;    // rot_split ? even columns of Pi^T (D, D/2) : Pi (D, D) row-major
  const float* mat_b;    // rot_split ? odd columns of Pi^T : unused
  int rot_split;
  const float* bnd[2];
  int nb[2];
  const float* cent0;  // centroids of source 0 (two-stage quantiser only)
  const float* qjl;    // S (D, D) row-major (two-stage quantiser only)
  uint8_t* code[2];
  int64_t code_row_stride;
  int code_head_stride;
  uint8_t* norm[2];
  int64_t norm_row_stride;
  uint8_t* sign;
  int64_t sign_row_stride;
  uint8_t* gam;
  int64_t gam_row_stride;
  const void* slots;  // null: destination row = token index
  int slot64;
  int64_t num_slots;
};

template <int D, int TV, bool QJL>
struct CompressSmem {
  static constexpr int kLda = D + 4;
  static constexpr size_t kMatBytes = size_t(D) * D * sizeof(float);
  static constexpr size_t kBytes =
      kMatBytes * (QJL ? 3 : 1) + size_t(TV) * kLda * sizeof(float) + 2 * 16 * sizeof(float) +
      16 * sizeof(float);
};

// acc[v][j] += sum_k A[v][k] * B[k][lane*JT + j]
template <int D, int VPW, int JT>
__device__ __forceinline__ void tile_matmul(const float* __restrict__ a_rows, int lda,
                                            const float* __restrict__ b, int lane,
                                            float (&acc)[VPW][JT]) {
#pragma unroll
  for (int v = 0; v < VPW; ++v)
#pragma unroll
    for (int j = 0; j < JT; ++j) acc[v][j] = 0.f;
#pragma unroll 2
  for (int k4 = 0; k4 < D; k4 += 4) {
    float bb[4][JT];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      const float* bp = b + (k4 + kk) * D + lane * JT;
      if constexpr (JT == 4) {
        float4 t = *reinterpret_cast<const float4*>(bp);
        bb[kk][0] = t.x; bb[kk][1] = t.y; bb[kk][2] = t.z; bb[kk][3] = t.w;
      } else {
        float2 t = *reinterpret_cast<const float2*>(bp);
        bb[kk][0] = t.x; bb[kk][1] = t.y;
      }
    }
#pragma unroll
    for (int v = 0; v < VPW; ++v) {
      float4 a = *reinterpret_cast<const float4*>(a_rows + v * lda + k4);
#pragma unroll
      for (int j = 0; j < JT; ++j) {
        acc[v][j] = fmaf(a.x, bb[0][j], acc[v][j]);
        acc[v][j] = fmaf(a.y, bb[1][j], acc[v][j]);
        acc[v][j] = fmaf(a.z, bb[2][j], acc[v][j]);
        acc[v][j] = fmaf(a.w, bb[3][j], acc[v][j]);
      }
    }
  }
}

// index = #{b : b < y} over an ascending table padded with +inf to 15 entries
__device__ __forceinline__ int bucketize15(float y, const float* __restrict__ sb) {
  int idx = (y > sb[7]) ? 8 : 0;
  idx += (y > sb[idx + 3]) ? 4 : 0;
  idx += (y > sb[idx + 1]) ? 2 : 0;
  idx += (y > sb[idx]) ? 1 : 0;
  return idx;
}

template <int D, int TV, int DT, bool QJL>
__global__ void __launch_bounds__(kCompressThreads, 1) compress_kernel(CompressArgs p) {
  using T = typename Elem<DT>::type;
  using S = CompressSmem<D, TV, QJL>;
  constexpr int VPW = TV / kCompressWarps;
  constexpr int JT = D / 32;
  constexpr int LDA = S::kLda;
  static_assert(JT == 4 || JT == 2, "head_dim must be 64 or 128");

  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* b_rot = reinterpret_cast<float*>(smem_raw);           // [k][j] = Pi[j][k]
  float* b_pi = b_rot + (QJL ? D * D : 0);                     // [k][j] = Pi[k][j]
  float* b_qjl = b_pi + (QJL ? D * D : 0);                     // [k][j] = S[j][k]
  float* a_tile = b_rot + D * D * (QJL ? 3 : 1);               // [v][k], row stride LDA
  float* s_bnd = a_tile + TV * LDA;                            // [2][16]
  float* s_cent = s_bnd + 32;                                  // [16]

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;

  // ---- resident matrices -----------------------------------------------------------
  for (int i = tid; i < D * D; i += kCompressThreads) {
    const int k = i / D, j = i % D;
    float v;
    if (p.rot_split) {
      const float* m = (j & 1) ? p.mat_b : p.mat_a;
      v = m[k * (D / 2) + (j >> 1)];
    } else {
      v = p.mat_a[j * D + k];
    }
    b_rot[i] = v;
    if constexpr (QJL) {
      b_pi[i] = p.mat_a[i];
      b_qjl[i] = p.qjl[j * D + k];
    }
  }
  if (tid < 32) {
    const int s = tid >> 4, i = tid & 15;
    const int src = (s < p.n_src) ? s : 0;
    s_bnd[tid] = (i < p.nb[src]) ? p.bnd[src][i] : __int_as_float(0x7f800000);
  }
  if (tid < 16) s_cent[tid] = (QJL && tid <= p.nb[0]) ? p.cent0[tid] : 0.f;
  __syncthreads();

  const int64_t n_vec = p.n_tokens * p.heads;
  const int64_t n_tiles = (n_vec + TV - 1) / TV;
  float* a_rows = a_tile + warp * VPW * LDA;

  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    for (int s = 0; s < p.n_src; ++s) {
      const T* src = reinterpret_cast<const T*>(p.src[s]);
      const float* sb = s_bnd + 16 * s;
      const int64_t v0 = tile * TV + warp * VPW;

      // ---- load, norm, normalise ----------------------------------------------------
      float nrm[VPW];
      int64_t row[VPW];
      int head[VPW];
      const T* xptr[VPW];
#pragma unroll
      for (int v = 0; v < VPW; ++v) {
        const int64_t vec = v0 + v;
        float x[JT];
        row[v] = -1;
        head[v] = 0;
        xptr[v] = nullptr;
        if (vec < n_vec) {
          const int64_t tok = vec / p.heads;
          head[v] = int(vec - tok * p.heads);
          xptr[v] = src + tok * p.token_stride + int64_t(head[v]) * D + lane * JT;
          if constexpr (JT == 4) load4(xptr[v], x); else load2(xptr[v], x);
          int64_t r = tok;
          if (p.slots) {
            r = p.slot64 ? reinterpret_cast<const int64_t*>(p.slots)[tok]
                         : int64_t(reinterpret_cast<const int32_t*>(p.slots)[tok]);
            if (r >= p.num_slots) r = -1;
          }
          row[v] = r;
        } else {
#pragma unroll
          for (int j = 0; j < JT; ++j) x[j] = 0.f;
        }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < JT; ++j) ss = fmaf(x[j], x[j], ss);
        ss = warp_sum(ss);
        nrm[v] = sqrtf(ss);
        const float denom = nrm[v] + 1e-10f;
        float* ar = a_rows + v * LDA + lane * JT;
#pragma unroll
        for (int j = 0; j < JT; ++j) ar[j] = x[j] / denom;
      }
      __syncwarp();

      // ---- y = x_hat Pi^T, codes --------------------------------------------------
      float acc[VPW][JT];
      tile_matmul<D, VPW, JT>(a_rows, LDA, b_rot, lane, acc);
      int idx[VPW][JT];
#pragma unroll
      for (int v = 0; v < VPW; ++v) {
#pragma unroll
        for (int j = 0; j < JT; ++j) idx[v][j] = bucketize15(acc[v][j], sb);
        if (row[v] >= 0) {
          uint8_t* dst = p.code[s] + row[v] * p.code_row_stride +
                         int64_t(head[v]) * p.code_head_stride + lane * (JT / 2);
          if constexpr (JT == 4) {
            const uint32_t two = uint32_t((idx[v][0] << 4) | idx[v][1]) |
                                 (uint32_t((idx[v][2] << 4) | idx[v][3]) << 8);
            *reinterpret_cast<uint16_t*>(dst) = uint16_t(two);
          } else {
            *dst = uint8_t((idx[v][0] << 4) | idx[v][1]);
          }
          if (lane == 0)
            *reinterpret_cast<float*>(p.norm[s] + row[v] * p.norm_row_stride + head[v] * 4) =
                nrm[v];
        }
      }

      if constexpr (QJL) {
        if (s == 0) {
          // ---- x_tilde = (c[code] Pi) n ; r = x - x_tilde ; gamma = |r| ----------------
          __syncwarp();
#pragma unroll
          for (int v = 0; v < VPW; ++v) {
            float* ar = a_rows + v * LDA + lane * JT;
#pragma unroll
            for (int j = 0; j < JT; ++j) ar[j] = s_cent[idx[v][j]];
          }
          __syncwarp();
          tile_matmul<D, VPW, JT>(a_rows, LDA, b_pi, lane, acc);
          __syncwarp();
#pragma unroll
          for (int v = 0; v < VPW; ++v) {
            float x[JT];
            if (xptr[v]) {
              if constexpr (JT == 4) load4(xptr[v], x); else load2(xptr[v], x);
            } else {
#pragma unroll
              for (int j = 0; j < JT; ++j) x[j] = 0.f;
            }
            float ss = 0.f;
            float* ar = a_rows + v * LDA + lane * JT;
#pragma unroll
            for (int j = 0; j < JT; ++j) {
              const float r = x[j] - acc[v][j] * nrm[v];
              ar[j] = r;
              ss = fmaf(r, r, ss);
            }
            ss = warp_sum(ss);
            if (lane == 0 && row[v] >= 0)
              *reinterpret_cast<float*>(p.gam + row[v] * p.gam_row_stride + head[v] * 4) =
                  sqrtf(ss);
          }
          __syncwarp();
          // ---- sign(r S^T) -----------------------------------------------------------
          tile_matmul<D, VPW, JT>(a_rows, LDA, b_qjl, lane, acc);
#pragma unroll
          for (int v = 0; v < VPW; ++v) {
            uint32_t bits = 0;
#pragma unroll
            for (int j = 0; j < JT; ++j) bits |= (acc[v][j] >= 0.f ? 1u : 0u) << j;
            // 32 coordinates per word: lanes sharing lane/(32/JT) build one word
            constexpr int LPW = 32 / JT;  // lanes per 32-bit word
            uint32_t word = bits << (JT * (lane % LPW));
#pragma unroll
            for (int o = 1; o < LPW; o <<= 1) word |= __shfl_xor_sync(0xffffffffu, word, o);
            if ((lane % LPW) == 0 && row[v] >= 0)
              *reinterpret_cast<uint32_t*>(p.sign + row[v] * p.sign_row_stride +
                                           head[v] * (D / 8) + (lane / LPW) * 4) = word;
          }
        }
      }
      __syncwarp();
    }
  }
}

template <int D, int TV, int DT, bool QJL>
static int launch_compress_t(const CompressArgs& a, cudaStream_t stream) {
  using S = CompressSmem<D, TV, QJL>;
  auto kern = compress_kernel<D, TV, DT, QJL>;
  static thread_local int configured_device = -1;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(FQ_ERR_CUDA, "cudaGetDevice failed");
  static thread_local int sm_count = 0;
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         int(S::kBytes));
    if (e != cudaSuccess)
      return fail(FQ_ERR_CUDA, "compress: shared memory opt-in of %zu bytes refused: %s",
                  S::kBytes, cudaGetErrorString(e));
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    configured_device = dev;
  }
  const int64_t n_vec = a.n_tokens * a.heads;
  const int64_t tiles = (n_vec + TV - 1) / TV;
  if (tiles == 0) return FQ_OK;
  const int per_sm = (S::kBytes <= 110 * 1024) ? 2 : 1;
  const int grid = int(tiles < int64_t(sm_count) * per_sm ? tiles : int64_t(sm_count) * per_sm);
  kern<<<grid, kCompressThreads, S::kBytes, stream>>>(a);
  return check_launch("compress kernel launch");
}

template <int D, bool QJL>
static int launch_compress_d(const CompressArgs& a, int dtype, cudaStream_t stream) {
  constexpr int TV = QJL ? 32 : 64;
  switch (dtype) {
    case FQ_F32: return launch_compress_t<D, TV, FQ_F32, QJL>(a, stream);
    case FQ_F16: return launch_compress_t<D, TV, FQ_F16, QJL>(a, stream);
    case FQ_BF16: return launch_compress_t<D, TV, FQ_BF16, QJL>(a, stream);
  }
  return fail(FQ_ERR_INVALID_ARGUMENT, "unknown dtype %d", dtype);
}

static int launch_compress(const CompressArgs& a, int dtype, int head_dim, bool qjl,
                           cudaStream_t stream) {
  if (head_dim == 128)
    return qjl ? launch_compress_d<128, true>(a, dtype, stream)
               : launch_compress_d<128, false>(a, dtype, stream);
  if (head_dim == 64)
    return qjl ? launch_compress_d<64, true>(a, dtype, stream)
               : launch_compress_d<64, false>(a, dtype, stream);
  return fail(FQ_ERR_UNSUPPORTED, "head_dim %d: the compress kernels are built for 64 and 128",
              head_dim);
}

static int elem_bytes(int dtype) { return dtype == FQ_F32 ? 4 : 2; }

}  // namespace fq

using namespace fq;

extern "C" int fq_tq4_compress(const void* x, fq_dtype dtype, const float* rot_T_even,
                               const float* rot_T_odd, const float* boundaries,
                               int n_boundaries, uint8_t* packed, float* norms,
                               int64_t n_vectors, int head_dim, fq_stream_t stream) {
  FQ_REQUIRE(n_vectors >= 0, FQ_ERR_INVALID_ARGUMENT, "n_vectors is negative");
  if (n_vectors == 0) return FQ_OK;
  FQ_REQUIRE(x && rot_T_even && rot_T_odd && boundaries && packed && norms,
             FQ_ERR_INVALID_ARGUMENT, "fq_tq4_compress: null pointer");
  FQ_REQUIRE(n_boundaries >= 1 && n_boundaries <= 15, FQ_ERR_INVALID_ARGUMENT,
             "n_boundaries %d outside [1, 15]", n_boundaries);
  FQ_REQUIRE(aligned(x, 4 * elem_bytes(dtype)) && aligned(packed, 2) && aligned(norms, 4),
             FQ_ERR_ALIGNMENT, "fq_tq4_compress: x must be aligned to 4 elements");
  CompressArgs a{};
  a.src[0] = x; a.n_src = 1;
  a.n_tokens = n_vectors; a.heads = 1; a.token_stride = head_dim;
  a.mat_a = rot_T_even; a.mat_b = rot_T_odd; a.rot_split = 1;
  a.bnd[0] = a.bnd[1] = boundaries; a.nb[0] = a.nb[1] = n_boundaries;
  a.code[0] = packed; a.code_row_stride = head_dim / 2; a.code_head_stride = 0;
  a.norm[0] = reinterpret_cast<uint8_t*>(norms); a.norm_row_stride = 4;
  return launch_compress(a, dtype, head_dim, false, stream);
}

extern "C" int fq_tq_prod_quantize(const void* x, fq_dtype dtype, const float* rotation,
                                   const float* boundaries, int n_boundaries,
                                   const float* centroids, const float* qjl, uint8_t* packed,
                                   float* norms, uint8_t* sign_bits, float* gamma,
                                   int64_t n_vectors, int head_dim, fq_stream_t stream) {
  FQ_REQUIRE(n_vectors >= 0, FQ_ERR_INVALID_ARGUMENT, "n_vectors is negative");
  if (n_vectors == 0) return FQ_OK;
  FQ_REQUIRE(x && rotation && boundaries && centroids && qjl && packed && norms && sign_bits &&
                 gamma,
             FQ_ERR_INVALID_ARGUMENT, "fq_tq_prod_quantize: null pointer");
  FQ_REQUIRE(n_boundaries >= 1 && n_boundaries <= 15, FQ_ERR_INVALID_ARGUMENT,
             "n_boundaries %d outside [1, 15]", n_boundaries);
  FQ_REQUIRE(aligned(x, 4 * elem_bytes(dtype)) && aligned(packed, 2) && aligned(norms, 4) &&
                 aligned(sign_bits, 4) && aligned(gamma, 4),
             FQ_ERR_ALIGNMENT, "fq_tq_prod_quantize: misaligned buffer");
  CompressArgs a{};
  a.src[0] = x; a.n_src = 1;
  a.n_tokens = n_vectors; a.heads = 1; a.token_stride = head_dim;
  a.mat_a = rotation; a.rot_split = 0;
  a.bnd[0] = a.bnd[1] = boundaries; a.nb[0] = a.nb[1] = n_boundaries;
  a.cent0 = centroids; a.qjl = qjl;
  a.code[0] = packed; a.code_row_stride = head_dim / 2; a.code_head_stride = 0;
  a.norm[0] = reinterpret_cast<uint8_t*>(norms); a.norm_row_stride = 4;
  a.sign = sign_bits; a.sign_row_stride = head_dim / 8;
  a.gam = reinterpret_cast<uint8_t*>(gamma); a.gam_row_stride = 4;
  return launch_compress(a, dtype, head_dim, true, stream);
}

static int append_common(const void* key, const void* value, fq_dtype dtype, int64_t n_tokens,
                         int num_kv_heads, int head_dim, int64_t token_stride,
                         const float* rotation, const float* boundaries_k, int n_boundaries_k,
                         const float* centroids_k, const float* boundaries_v,
                         int n_boundaries_v, const float* qjl, uint8_t* kv_cache,
                         uint8_t* kq_cache, int64_t num_slots, const void* slot_mapping,
                         int slot_is_int64, bool with_qjl, fq_stream_t stream) {
  FQ_REQUIRE(n_tokens >= 0 && num_kv_heads >= 1 && num_slots >= 0, FQ_ERR_INVALID_ARGUMENT,
             "compress_append: negative size");
  if (n_tokens == 0) return FQ_OK;
  FQ_REQUIRE(key && value && rotation && boundaries_k && boundaries_v && kv_cache &&
                 slot_mapping,
             FQ_ERR_INVALID_ARGUMENT, "compress_append: null pointer");
  FQ_REQUIRE(!with_qjl || (centroids_k && qjl && kq_cache), FQ_ERR_INVALID_ARGUMENT,
             "compress_append_qjl: null pointer");
  FQ_REQUIRE(n_boundaries_k >= 1 && n_boundaries_k <= 15 && n_boundaries_v >= 1 &&
                 n_boundaries_v <= 15,
             FQ_ERR_INVALID_ARGUMENT, "boundary count outside [1, 15]");
  FQ_REQUIRE(token_stride >= int64_t(num_kv_heads) * head_dim, FQ_ERR_INVALID_ARGUMENT,
             "token_stride smaller than num_kv_heads*head_dim");
  const int eb = elem_bytes(dtype);
  FQ_REQUIRE(aligned(key, 4 * eb) && aligned(value, 4 * eb) && (token_stride % 4) == 0,
             FQ_ERR_ALIGNMENT, "key/value must be aligned to 4 elements");
  FQ_REQUIRE(aligned(kv_cache, 4) && (!with_qjl || aligned(kq_cache, 4)), FQ_ERR_ALIGNMENT,
             "cache base must be 4-byte aligned");
  const int64_t half = head_dim / 2;
  const int64_t row_bytes = int64_t(num_kv_heads) * (head_dim + 8);
  CompressArgs a{};
  a.src[0] = key; a.src[1] = value; a.n_src = 2;
  a.n_tokens = n_tokens; a.heads = num_kv_heads; a.token_stride = token_stride;
  a.mat_a = rotation; a.rot_split = 0;
  a.bnd[0] = boundaries_k; a.nb[0] = n_boundaries_k;
  a.bnd[1] = boundaries_v; a.nb[1] = n_boundaries_v;
  a.code[0] = kv_cache;
  a.norm[0] = kv_cache + num_kv_heads * half;
  a.code[1] = kv_cache + num_kv_heads * half + num_kv_heads * 4;
  a.norm[1] = kv_cache + 2 * num_kv_heads * half + num_kv_heads * 4;
  a.code_row_stride = row_bytes; a.code_head_stride = int(half);
  a.norm_row_stride = row_bytes;
  if (with_qjl) {
    const int64_t qrow = int64_t(num_kv_heads) * (head_dim / 8 + 4);
    a.cent0 = centroids_k; a.qjl = qjl;
    a.sign = kq_cache; a.sign_row_stride = qrow;
    a.gam = kq_cache + num_kv_heads * (head_dim / 8); a.gam_row_stride = qrow;
  }
  a.slots = slot_mapping; a.slot64 = slot_is_int64; a.num_slots = num_slots;
  return launch_compress(a, dtype, head_dim, with_qjl, stream);
}

extern "C" int fq_tq4_compress_append(const void* key, const void* value, fq_dtype dtype,
                                      int64_t n_tokens, int num_kv_heads, int head_dim,
                                      int64_t token_stride, const float* rotation,
                                      const float* boundaries_k, int n_boundaries_k,
                                      const float* boundaries_v, int n_boundaries_v,
                                      uint8_t* kv_cache, int64_t num_slots,
                                      const void* slot_mapping, int slot_is_int64,
                                      fq_stream_t stream) {
  return append_common(key, value, dtype, n_tokens, num_kv_heads, head_dim, token_stride,
                       rotation, boundaries_k, n_boundaries_k, nullptr, boundaries_v,
                       n_boundaries_v, nullptr, kv_cache, nullptr, num_slots, slot_mapping,
                       slot_is_int64, false, stream);
}

extern "C" int fq_tq4_compress_append_qjl(
    const void* key, const void* value, fq_dtype dtype, int64_t n_tokens, int num_kv_heads,
    int head_dim, int64_t token_stride, const float* rotation, const float* boundaries_k,
    int n_boundaries_k, const float* centroids_k, const float* boundaries_v, int n_boundaries_v,
    const float* qjl, uint8_t* kv_cache, uint8_t* kq_cache, int64_t num_slots,
    const void* slot_mapping, int slot_is_int64, fq_stream_t stream) {
  return append_common(key, value, dtype, n_tokens, num_kv_heads, head_dim, token_stride,
                       rotation, boundaries_k, n_boundaries_k, centroids_k, boundaries_v,
                       n_boundaries_v, qjl, kv_cache, kq_cache, num_slots, slot_mapping,
                       slot_is_int64, true, stream);
}
