// TQ4 compress / compress-on-append / two-stage (QJL) quantiser for sm_100a.
//
// The contractions (y = x_hat Pi^T, x_tilde = y_tilde Pi, r S^T) run on the tensor pipe with
// fp32-level accuracy: every operand is split into two fp16 terms, hi = fp16(v) and
// lo' = fp16((v - hi) * 2048), and a product is accumulated as hi*hi into one fp32 accumulator
// and hi*lo' + lo'*hi into a second one that is scaled by 2^-11 at the end (the lo*lo term,
// 2^-22 of the product, is dropped).  That keeps the codes within the reference's own sgemm
// rounding of a Lloyd-Max boundary (a coordinate closer than ~1e-7 to a boundary may land on
// either side with any summation order) at a third of the multiply-add issue slots of an fp32
// FMA contraction, which was the bound of this kernel before.
//
// A CTA of 8 warps keeps the matrices resident in shared memory as fp16 hi / lo' planes (the
// same bytes as fp32).  A warp owns a tile of 16 vectors end to end, K of the tile then V:
// the rows come from global memory straight into MMA fragments, the products walk the column
// tiles four at a time with the matrix fragments from ldmatrix, and the chain of the
// two-stage quantiser stays in registers - an accumulator tile pair is exactly the left
// operand fragment of the next product (codes -> centroids -> x_tilde -> residual -> signs) -
// so the tile loop has no barrier and no shared-memory exchange.  The operation order is the
// reference's (normalise, then rotate); the tie rule is bucketize(right=False).
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
  // Without a slot list and with seg_len > 0 the tokens form runs of seg_len that land in
  // segments of seg_stride rows: row = (token / seg_len) * seg_stride + seg_offset + token % seg_len
  // (the per-head buffers of a contiguous cache, each with room for seg_stride tokens).
  uint32_t seg_len;
  int64_t seg_stride;
  int64_t seg_offset;
};

__device__ __forceinline__ int64_t segment_row(const CompressArgs& p, uint32_t tok) {
  const uint32_t seg = tok / p.seg_len;
  return int64_t(seg) * p.seg_stride + p.seg_offset + int64_t(tok - seg * p.seg_len);
}

constexpr int kTileRows = 16;         // vectors per tile = rows of one MMA
constexpr float kLoScale = 2048.f;    // lo' = (v - hi) * 2^11
constexpr float kLoUnscale = 1.f / 2048.f;

// Shared-memory plan.  Matrices and left operands are fp16 planes with rows padded by 8
// halves: fragment loads (4 bytes at row g / column pair t, or row n = g) then hit 32 banks.
template <int D, bool QJL>
struct CompressSmem {
  static constexpr int kLd = D + 8;                        // halves per row
  static constexpr size_t kPlane = size_t(D) * kLd * 2;    // one matrix plane, bytes
  static constexpr int kMats = QJL ? 3 : 1;
  static constexpr size_t kOffMeta = kPlane * 2 * kMats;   // hi and lo' plane per matrix
  // meta: bnd[2][16] f32, cent[16] f32
  static constexpr size_t kBytes = kOffMeta + (32 + 16) * 4;
};

__device__ __forceinline__ void split_hi_lo(float v, __half& hi, __half& lo) {
  hi = __float2half_rn(v);
  lo = __float2half_rn((v - __half2float(hi)) * kLoScale);
}
__device__ __forceinline__ uint32_t pack_h2(__half a, __half b) {
  return uint32_t(__half_as_ushort(a)) | (uint32_t(__half_as_ushort(b)) << 16);
}

// index = #{b : b < y} over an ascending table padded with +inf to 15 entries
__device__ __forceinline__ int bucketize15(float y, const float* __restrict__ sb) {
  int idx = (y > sb[7]) ? 8 : 0;
  idx += (y > sb[idx + 3]) ? 4 : 0;
  idx += (y > sb[idx + 1]) ? 2 : 0;
  idx += (y > sb[idx]) ? 1 : 0;
  return idx;
}

// Stage one D x D matrix as hi / lo' planes: plane[n][k] = get(n, k).  Thread i walks the
// matrix in the order that makes `get` read global memory contiguously (`k_fast`: k runs
// fastest, else n).
template <int D, int kThreads = kCompressThreads, typename Get>
__device__ __forceinline__ void stage_matrix(__half* hi, __half* lo, int ld, bool k_fast, Get get,
                                             int tid) {
  constexpr int kPer = D * D / kThreads;  // elements per thread
  constexpr int kBatch = kPer < 16 ? kPer : 16;   // loads in flight per thread
  static_assert(kPer % kBatch == 0, "matrix size must be a multiple of the batch");
#pragma unroll 1
  for (int b = 0; b < kPer; b += kBatch) {
    float v[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = tid + (b + u) * kThreads;
      v[u] = get(k_fast ? i / D : i % D, k_fast ? i % D : i / D);
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = tid + (b + u) * kThreads;
      const int n = k_fast ? i / D : i % D, k = k_fast ? i % D : i / D;
      __half h, l;
      split_hi_lo(v[u], h, l);
      hi[n * ld + k] = h;
      lo[n * ld + k] = l;
    }
  }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* row_ptr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(row_ptr)));
}

// One product of a 16-row tile held in registers with a resident matrix, four column tiles at
// a time: acc[i][c] (C-fragment layout: c0,c1 = row g, columns 8*nt + 2t, +1; c2,c3 = row g+8)
// for nt = 4*grp + i.  ah / al: the left operand's hi / lo' fragments, [k-step][a0..a3].
template <int D>
__device__ __forceinline__ void reg_mma_group(const uint32_t (&ah)[D / 16][4],
                                              const uint32_t (&al)[D / 16][4],
                                              const __half* __restrict__ pb, int ld, int grp,
                                              float (&acc)[4][4]) {
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
      ldmatrix_x4(b, pb + (grp * 4 + i) * 8 * ld + 16 * ks);
      mma_f16(hi[i], ah[ks][0], ah[ks][1], ah[ks][2], ah[ks][3], b[0], b[1]);
      mma_f16(co[i], ah[ks][0], ah[ks][1], ah[ks][2], ah[ks][3], b[2], b[3]);
      mma_f16(co[i], al[ks][0], al[ks][1], al[ks][2], al[ks][3], b[0], b[1]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] = fmaf(co[i][c], kLoUnscale, hi[i][c]);
}

__device__ __forceinline__ float2 load_pair(const float* p) {
  return *reinterpret_cast<const float2*>(p);
}
__device__ __forceinline__ float2 load_pair(const __half* p) {
  return __half22float2(*reinterpret_cast<const __half2*>(p));
}
__device__ __forceinline__ float2 load_pair(const __nv_bfloat16* p) {
  const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
  return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

template <int D, int DT, bool QJL>
__global__ void __launch_bounds__(kCompressThreads, QJL ? 1 : 2) compress_kernel(CompressArgs p) {
  using T = typename Elem<DT>::type;
  using S = CompressSmem<D, QJL>;
  constexpr int LD = S::kLd;
  constexpr int KS = D / 16;  // k-steps of a product
  constexpr int NG = D / 32;  // groups of four column tiles
  static_assert(D == 64 || D == 128, "head_dim must be 64 or 128");

  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* m_hi[3];
  __half* m_lo[3];
#pragma unroll
  for (int m = 0; m < 3; ++m) {
    m_hi[m] = reinterpret_cast<__half*>(smem_raw + S::kPlane * 2 * (m < S::kMats ? m : 0));
    m_lo[m] = m_hi[m] + D * LD;
  }
  float* s_bnd = reinterpret_cast<float*>(smem_raw + S::kOffMeta);  // [2][16]
  float* s_cent = s_bnd + 32;                                       // [16]

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;

  // ---- resident matrices -----------------------------------------------------------------
  // [0]: Pi as it is  (y = x_hat Pi^T:      B[k][n] = Pi[n][k])
  // [1]: Pi transposed (x_tilde = y_tilde Pi: B[k][n] = Pi[k][n])
  // [2]: S as it is   (r S^T:               B[k][n] = S[n][k])
  if (p.rot_split) {
    stage_matrix<D>(m_hi[0], m_lo[0], LD, false, [&](int n, int k) {
      return ((n & 1) ? p.mat_b : p.mat_a)[k * (D / 2) + (n >> 1)];
    }, tid);
  } else {
    stage_matrix<D>(m_hi[0], m_lo[0], LD, true, [&](int n, int k) { return p.mat_a[n * D + k]; }, tid);
  }
  if constexpr (QJL) {
    stage_matrix<D>(m_hi[1], m_lo[1], LD, false, [&](int n, int k) { return p.mat_a[k * D + n]; }, tid);
    stage_matrix<D>(m_hi[2], m_lo[2], LD, true, [&](int n, int k) { return p.qjl[n * D + k]; }, tid);
  }
  if (tid < 32) {
    const int s = tid >> 4, i = tid & 15;
    const int src = (s < p.n_src) ? s : 0;
    s_bnd[tid] = (i < p.nb[src]) ? p.bnd[src][i] : __int_as_float(0x7f800000);
  }
  if (tid < 16) s_cent[tid] = (QJL && tid <= p.nb[0]) ? p.cent0[tid] : 0.f;
  __syncthreads();

  // ldmatrix: lanes 8j..8j+7 give the rows of matrix j = plane j>>1 (hi, lo'), k-segment j&1
  const int lj = lane >> 3, lr = lane & 7;
  const __half* pb[3];
#pragma unroll
  for (int m = 0; m < 3; ++m) pb[m] = ((lj >> 1) ? m_lo[m] : m_hi[m]) + lr * LD + 8 * (lj & 1);

  // (the host side keeps n_vec below 2^31: 32-bit index arithmetic, no 64-bit divisions)
  const uint32_t n_vec = uint32_t(p.n_tokens * p.heads);
  const uint32_t n_tiles = (n_vec + kTileRows - 1) / kTileRows;
  const uint32_t heads = uint32_t(p.heads);
  const uint32_t warps_total = gridDim.x * kCompressWarps;

  // A warp owns a tile of 16 vectors end to end, K of the tile then V: no barrier in the loop.
  for (uint32_t tile = blockIdx.x * kCompressWarps + warp; tile < n_tiles; tile += warps_total) {
    // rows g and g+8 of the tile
    const uint32_t v0 = tile * kTileRows + g, v1 = v0 + 8;
    const bool ok0 = v0 < n_vec, ok1 = v1 < n_vec;
    const uint32_t tok0 = ok0 ? v0 / heads : 0u, tok1 = ok1 ? v1 / heads : 0u;
    const int head0 = int(v0 - tok0 * heads), head1 = int(v1 - tok1 * heads);
    int64_t slot0 = ok0 ? int64_t(tok0) : -1, slot1 = ok1 ? int64_t(tok1) : -1;
    if (p.slots) {
      if (ok0)
        slot0 = p.slot64 ? reinterpret_cast<const int64_t*>(p.slots)[tok0]
                         : int64_t(reinterpret_cast<const int32_t*>(p.slots)[tok0]);
      if (ok1)
        slot1 = p.slot64 ? reinterpret_cast<const int64_t*>(p.slots)[tok1]
                         : int64_t(reinterpret_cast<const int32_t*>(p.slots)[tok1]);
      if (slot0 >= p.num_slots) slot0 = -1;
      if (slot1 >= p.num_slots) slot1 = -1;
    } else if (p.seg_len) {
      if (ok0) slot0 = segment_row(p, tok0);
      if (ok1) slot1 = segment_row(p, tok1);
    }

    for (int s = 0; s < p.n_src; ++s) {
      const T* src = reinterpret_cast<const T*>(p.src[s]);
      const float* sb = s_bnd + 16 * s;
      // the lane's share of the two rows: columns 16*ks + 2t, +1 and 16*ks + 8 + 2t, +1
      const T* x0 = src + int64_t(tok0) * p.token_stride + int64_t(head0) * D + 2 * t;
      const T* x1 = src + int64_t(tok1) * p.token_stride + int64_t(head1) * D + 2 * t;

      // ---- norms: sum of squares over the lane's share, then over the four lanes of a row ----
      float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        if (ok0) {
          const float2 a = load_pair(x0 + 16 * ks), b = load_pair(x0 + 16 * ks + 8);
          ss0 = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(b.x, b.x, fmaf(b.y, b.y, ss0))));
        }
        if (ok1) {
          const float2 a = load_pair(x1 + 16 * ks), b = load_pair(x1 + 16 * ks + 8);
          ss1 = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(b.x, b.x, fmaf(b.y, b.y, ss1))));
        }
      }
      ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1);
      ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1);
      ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
      ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
      const float nrm0 = sqrtf(ss0), nrm1 = sqrtf(ss1);
      // one reciprocal per vector instead of a division per coordinate: x_hat may differ from
      // x / (n + 1e-10) in the last bit, far inside the rounding of the contraction
      const float inv0 = 1.f / (nrm0 + 1e-10f), inv1 = 1.f / (nrm1 + 1e-10f);
      if (t == 0 && slot0 >= 0)
        *reinterpret_cast<float*>(p.norm[s] + slot0 * p.norm_row_stride + head0 * 4) = nrm0;
      if (t == 1 && slot1 >= 0)
        *reinterpret_cast<float*>(p.norm[s] + slot1 * p.norm_row_stride + head1 * 4) = nrm1;

      // ---- x_hat as hi / lo' fragments (the rows come from the L1 this time) ----------------
      uint32_t xh[KS][4], xl[KS][4];
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        float2 f[4];
        f[0] = ok0 ? load_pair(x0 + 16 * ks) : make_float2(0.f, 0.f);
        f[1] = ok1 ? load_pair(x1 + 16 * ks) : make_float2(0.f, 0.f);
        f[2] = ok0 ? load_pair(x0 + 16 * ks + 8) : make_float2(0.f, 0.f);
        f[3] = ok1 ? load_pair(x1 + 16 * ks + 8) : make_float2(0.f, 0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float sc = (i & 1) ? inv1 : inv0;
          __half h0, l0, h1, l1;
          split_hi_lo(f[i].x * sc, h0, l0);
          split_hi_lo(f[i].y * sc, h1, l1);
          xh[ks][i] = pack_h2(h0, h1);
          xl[ks][i] = pack_h2(l0, l1);
        }
      }

      // ---- y = x_hat Pi^T, codes; for the two-stage quantiser the centroid vector becomes the
      // left operand of the next product: C tiles 2ks, 2ks+1 are A k-step ks -----------------
      [[maybe_unused]] uint32_t yh[KS][4], yl[KS][4];
      // code bytes: after the shuffles all four lanes of a row hold the 16 bytes of a group;
      // lane t keeps those of group t, so that the row leaves in one 64-byte store instruction
      uint32_t keep0[4] = {0u, 0u, 0u, 0u}, keep1[4] = {0u, 0u, 0u, 0u};
#pragma unroll
      for (int grp = 0; grp < NG; ++grp) {
        float acc[4][4];
        reg_mma_group<D>(xh, xl, pb[0], LD, grp, acc);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int nt = grp * 4 + i;
          int idx[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) idx[c] = bucketize15(acc[i][c], sb);
          // code byte = (even coordinate << 4) | odd coordinate; the four lanes of a row hold
          // bytes 4*nt .. 4*nt+3 of it
          uint32_t w_lo = uint32_t((idx[0] << 4) | idx[1]) << (8 * t);
          uint32_t w_hi = uint32_t((idx[2] << 4) | idx[3]) << (8 * t);
          w_lo |= __shfl_xor_sync(0xffffffffu, w_lo, 1);
          w_hi |= __shfl_xor_sync(0xffffffffu, w_hi, 1);
          w_lo |= __shfl_xor_sync(0xffffffffu, w_lo, 2);
          w_hi |= __shfl_xor_sync(0xffffffffu, w_hi, 2);
          if (t == grp) {
            keep0[i] = w_lo;
            keep1[i] = w_hi;
          }
          if constexpr (QJL) {
            if (s == 0) {
              __half h[4], l[4];
#pragma unroll
              for (int c = 0; c < 4; ++c) split_hi_lo(s_cent[idx[c]], h[c], l[c]);
              yh[nt >> 1][(nt & 1) * 2 + 0] = pack_h2(h[0], h[1]);  // a0 / a2: row g
              yh[nt >> 1][(nt & 1) * 2 + 1] = pack_h2(h[2], h[3]);  // a1 / a3: row g+8
              yl[nt >> 1][(nt & 1) * 2 + 0] = pack_h2(l[0], l[1]);
              yl[nt >> 1][(nt & 1) * 2 + 1] = pack_h2(l[2], l[3]);
            }
          }
        }
      }

      if (t < NG) {  // 16 bytes of each row per lane: whole sectors when the row is aligned
        uint8_t* d0 = p.code[s] + slot0 * p.code_row_stride + int64_t(head0) * p.code_head_stride + 16 * t;
        uint8_t* d1 = p.code[s] + slot1 * p.code_row_stride + int64_t(head1) * p.code_head_stride + 16 * t;
        if (slot0 >= 0) {
          if ((reinterpret_cast<uintptr_t>(d0) & 15) == 0) {
            *reinterpret_cast<uint4*>(d0) = make_uint4(keep0[0], keep0[1], keep0[2], keep0[3]);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) reinterpret_cast<uint32_t*>(d0)[i] = keep0[i];
          }
        }
        if (slot1 >= 0) {
          if ((reinterpret_cast<uintptr_t>(d1) & 15) == 0) {
            *reinterpret_cast<uint4*>(d1) = make_uint4(keep1[0], keep1[1], keep1[2], keep1[3]);
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) reinterpret_cast<uint32_t*>(d1)[i] = keep1[i];
          }
        }
      }

      if constexpr (QJL) {
        if (s == 0) {
          // ---- x_tilde = (c[code] Pi) n ; r = x - x_tilde ; gamma = |r| ; r becomes the left
          // operand of the last product (the registers of x_hat are free now) ------------------
          float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
          for (int grp = 0; grp < NG; ++grp) {
            float acc[4][4];
            reg_mma_group<D>(yh, yl, pb[1], LD, grp, acc);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int nt = grp * 4 + i;
              const float2 a = ok0 ? load_pair(x0 + 8 * nt) : make_float2(0.f, 0.f);
              const float2 b = ok1 ? load_pair(x1 + 8 * nt) : make_float2(0.f, 0.f);
              const float r0 = a.x - acc[i][0] * nrm0, r1 = a.y - acc[i][1] * nrm0;
              const float r2 = b.x - acc[i][2] * nrm1, r3 = b.y - acc[i][3] * nrm1;
              rs0 = fmaf(r0, r0, fmaf(r1, r1, rs0));
              rs1 = fmaf(r2, r2, fmaf(r3, r3, rs1));
              __half h[4], l[4];
              split_hi_lo(r0, h[0], l[0]);
              split_hi_lo(r1, h[1], l[1]);
              split_hi_lo(r2, h[2], l[2]);
              split_hi_lo(r3, h[3], l[3]);
              xh[nt >> 1][(nt & 1) * 2 + 0] = pack_h2(h[0], h[1]);
              xh[nt >> 1][(nt & 1) * 2 + 1] = pack_h2(h[2], h[3]);
              xl[nt >> 1][(nt & 1) * 2 + 0] = pack_h2(l[0], l[1]);
              xl[nt >> 1][(nt & 1) * 2 + 1] = pack_h2(l[2], l[3]);
            }
          }
          rs0 += __shfl_xor_sync(0xffffffffu, rs0, 1);
          rs1 += __shfl_xor_sync(0xffffffffu, rs1, 1);
          rs0 += __shfl_xor_sync(0xffffffffu, rs0, 2);
          rs1 += __shfl_xor_sync(0xffffffffu, rs1, 2);
          if (t == 0 && slot0 >= 0)
            *reinterpret_cast<float*>(p.gam + slot0 * p.gam_row_stride + head0 * 4) = sqrtf(rs0);
          if (t == 1 && slot1 >= 0)
            *reinterpret_cast<float*>(p.gam + slot1 * p.gam_row_stride + head1 * 4) = sqrtf(rs1);
          // ---- sign(r S^T): bit j%8 of byte j/8 is 1 for a projection >= 0 -------------------
          uint32_t sb0 = 0, sb1 = 0;  // lane t keeps bytes 4t .. 4t+3 of the rows' sign bytes
#pragma unroll
          for (int grp = 0; grp < NG; ++grp) {
            float acc[4][4];
            reg_mma_group<D>(xh, xl, pb[2], LD, grp, acc);
            uint32_t b_lo = 0, b_hi = 0;  // bytes 4*grp .. 4*grp+3 of the row's sign bytes
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              b_lo |= ((acc[i][0] >= 0.f ? 1u : 0u) | (acc[i][1] >= 0.f ? 2u : 0u)) << (8 * i + 2 * t);
              b_hi |= ((acc[i][2] >= 0.f ? 1u : 0u) | (acc[i][3] >= 0.f ? 2u : 0u)) << (8 * i + 2 * t);
            }
            b_lo |= __shfl_xor_sync(0xffffffffu, b_lo, 1);
            b_hi |= __shfl_xor_sync(0xffffffffu, b_hi, 1);
            b_lo |= __shfl_xor_sync(0xffffffffu, b_lo, 2);
            b_hi |= __shfl_xor_sync(0xffffffffu, b_hi, 2);
            if (t == grp) {
              sb0 = b_lo;
              sb1 = b_hi;
            }
          }
          if (t < NG) {
            if (slot0 >= 0)
              *reinterpret_cast<uint32_t*>(p.sign + slot0 * p.sign_row_stride + head0 * (D / 8) +
                                           4 * t) = sb0;
            if (slot1 >= 0)
              *reinterpret_cast<uint32_t*>(p.sign + slot1 * p.sign_row_stride + head1 * (D / 8) +
                                           4 * t) = sb1;
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------------------------
// Small calls (a decode step appends one token per sequence: a few tiles in all): the whole
// CTA works on one tile at a time.  16 warps; warp w loads and normalises vector w of the tile,
// the first eight warps (head_dim 128) own two column tiles each of every product; the left
// operand (x_hat, then the centroid vector, then the residual) is exchanged through shared
// memory as hi / lo' planes, six block-wide barriers per K tile of the two-stage quantiser.
// Latency of one tile is what counts here: the products of a tile are spread over the warps
// instead of running one after the other in a single warp.
// ------------------------------------------------------------------------------------
constexpr int kCoopThreads = 512;
constexpr int kCoopWarps = 16;

template <int D, bool QJL>
struct CoopSmem {
  static constexpr int kLd = D + 8;                        // halves per row
  static constexpr size_t kPlane = size_t(D) * kLd * 2;    // one matrix plane, bytes
  static constexpr size_t kAPlane = size_t(kTileRows) * kLd * 2;
  static constexpr int kMats = QJL ? 3 : 1;
  static constexpr size_t kOffA = kPlane * 2 * kMats;      // hi and lo' plane per matrix
  static constexpr size_t kOffX = kOffA + 2 * kAPlane;      // the tile's vectors as fp32
  static constexpr size_t kOffMeta = kOffX + (QJL ? size_t(kTileRows) * (D + 8) * 4 : 0);
  // meta: nrm[16] f32, gpart[16][16] f32, bnd[2][16] f32, cent[16] f32, slot[16] i64, head[16] i32
  static constexpr size_t kBytes = kOffMeta + (16 + 256 + 32 + 16) * 4 + 16 * 8 + 16 * 4;
};

// acc[i][c] = sum_k A[row][k] * B[n][k] for the NTW column tiles nt0 .. nt0+NTW-1 (C-fragment
// layout: c0,c1 = row g, columns 8*nt + 2t, +1; c2,c3 = row g+8), A and B as hi / lo' planes.
// Per 16 values of k: two ldmatrix for the left operand, shared by the tiles, then one ldmatrix
// and three MMAs per tile.
template <int D, int NTW>
__device__ __forceinline__ void plane_mma(const __half* __restrict__ ah,
                                          const __half* __restrict__ al,
                                          const __half* __restrict__ bh,
                                          const __half* __restrict__ bl, int ld, int nt0, int lane,
                                          float (&acc)[NTW][4]) {
  const int j = lane >> 3, r = lane & 7;  // ldmatrix: lanes 8j..8j+7 give the rows of matrix j
  // A: matrix j = rows 8*(j&1).., k-segment j>>1;  B: matrix j = plane j>>1 (hi, lo'), k-segment j&1
  const __half* pa_h = ah + ((j & 1) * 8 + r) * ld + 8 * (j >> 1);
  const __half* pa_l = al + ((j & 1) * 8 + r) * ld + 8 * (j >> 1);
  const __half* pb = ((j >> 1) ? bl : bh) + (8 * nt0 + r) * ld + 8 * (j & 1);
  float hi[NTW][4], co[NTW][4];
#pragma unroll
  for (int i = 0; i < NTW; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) hi[i][c] = co[i][c] = 0.f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t xh[4], xl[4];
    ldmatrix_x4(xh, pa_h + 16 * ks);
    ldmatrix_x4(xl, pa_l + 16 * ks);
#pragma unroll
    for (int i = 0; i < NTW; ++i) {
      uint32_t b[4];  // b0 hi, b1 hi, b0 lo', b1 lo'
      ldmatrix_x4(b, pb + i * 8 * ld + 16 * ks);
      mma_f16(hi[i], xh[0], xh[1], xh[2], xh[3], b[0], b[1]);
      mma_f16(co[i], xh[0], xh[1], xh[2], xh[3], b[2], b[3]);
      mma_f16(co[i], xl[0], xl[1], xl[2], xl[3], b[0], b[1]);
    }
  }
#pragma unroll
  for (int i = 0; i < NTW; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[i][c] = fmaf(co[i][c], kLoUnscale, hi[i][c]);
}

template <int D, int DT, bool QJL>
__global__ void __launch_bounds__(kCoopThreads, QJL ? 1 : 2) compress_coop_kernel(CompressArgs p) {
  using T = typename Elem<DT>::type;
  using S = CoopSmem<D, QJL>;
  constexpr int LD = S::kLd;
  constexpr int JT = D / 32;   // elements per lane when a warp walks one vector
  constexpr int NT = D / 8;    // column tiles of a product
  constexpr int NTW = 2;  // ... of which a product warp takes this many
  constexpr int MW = NT / NTW;          // product warps: warps 0 .. MW-1
  static_assert(D == 64 || D == 128, "head_dim must be 64 or 128");

  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* m_hi[3];
  __half* m_lo[3];
#pragma unroll
  for (int m = 0; m < 3; ++m) {
    m_hi[m] = reinterpret_cast<__half*>(smem_raw + S::kPlane * 2 * (m < S::kMats ? m : 0));
    m_lo[m] = m_hi[m] + D * LD;
  }
  __half* a_hi = reinterpret_cast<__half*>(smem_raw + S::kOffA);
  __half* a_lo = a_hi + kTileRows * LD;
  [[maybe_unused]] float* s_x = reinterpret_cast<float*>(smem_raw + S::kOffX);  // [16][D+8]
  float* s_nrm = reinterpret_cast<float*>(smem_raw + S::kOffMeta);
  float* s_gpart = s_nrm + 16;   // [16 warps][16 rows]
  float* s_bnd = s_gpart + 256;  // [2][16]
  float* s_cent = s_bnd + 32;    // [16]
  int64_t* s_slot = reinterpret_cast<int64_t*>(s_cent + 16);
  int* s_head = reinterpret_cast<int*>(s_slot + 16);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const bool col_warp = warp < MW;  // takes part in the products

  // ---- resident matrices -----------------------------------------------------------------
  // [0]: Pi as it is  (y = x_hat Pi^T:      B[k][n] = Pi[n][k])
  // [1]: Pi transposed (x_tilde = y_tilde Pi: B[k][n] = Pi[k][n])
  // [2]: S as it is   (r S^T:               B[k][n] = S[n][k])
  if (p.rot_split) {
    stage_matrix<D, kCoopThreads>(m_hi[0], m_lo[0], LD, false, [&](int n, int k) {
      return ((n & 1) ? p.mat_b : p.mat_a)[k * (D / 2) + (n >> 1)];
    }, tid);
  } else {
    stage_matrix<D, kCoopThreads>(m_hi[0], m_lo[0], LD, true, [&](int n, int k) { return p.mat_a[n * D + k]; }, tid);
  }
  if constexpr (QJL) {
    stage_matrix<D, kCoopThreads>(m_hi[1], m_lo[1], LD, false, [&](int n, int k) { return p.mat_a[k * D + n]; }, tid);
    stage_matrix<D, kCoopThreads>(m_hi[2], m_lo[2], LD, true, [&](int n, int k) { return p.qjl[n * D + k]; }, tid);
  }
  if (tid < 32) {
    const int s = tid >> 4, i = tid & 15;
    const int src = (s < p.n_src) ? s : 0;
    s_bnd[tid] = (i < p.nb[src]) ? p.bnd[src][i] : __int_as_float(0x7f800000);
  }
  if (tid < 16) s_cent[tid] = (QJL && tid <= p.nb[0]) ? p.cent0[tid] : 0.f;
  __syncthreads();

  const int64_t n_vec = p.n_tokens * p.heads;
  const int64_t n_tiles = (n_vec + kTileRows - 1) / kTileRows;

  // The vector of the next work item (tile, source) is requested before the current one is
  // worked on, so that its latency hides behind the contractions.  Warp w holds row w.
  struct Row {
    float x[JT];
    int64_t slot;
    int head;
  };
  // (the host side keeps n_vec below 2^31: 32-bit index arithmetic, no 64-bit divisions)
  const uint32_t heads = uint32_t(p.heads);
  auto fetch = [&](uint32_t tile, int s, Row& f) {
    const T* src = reinterpret_cast<const T*>(p.src[s]);
    const uint32_t vec = tile * kTileRows + warp;
    f.slot = -1;
    f.head = 0;
#pragma unroll
    for (int j = 0; j < JT; ++j) f.x[j] = 0.f;
    if (vec < uint32_t(n_vec)) {
      const uint32_t tok32 = vec / heads;
      const int64_t tok = tok32;
      f.head = int(vec - tok32 * heads);
      const T* xp = src + tok * p.token_stride + int64_t(f.head) * D + lane * JT;
      if constexpr (JT == 4) load4(xp, f.x); else load2(xp, f.x);
      int64_t slot = tok;
      if (p.slots) {
        slot = p.slot64 ? reinterpret_cast<const int64_t*>(p.slots)[tok]
                        : int64_t(reinterpret_cast<const int32_t*>(p.slots)[tok]);
        if (slot >= p.num_slots) slot = -1;
      } else if (p.seg_len) {
        slot = segment_row(p, tok32);
      }
      f.slot = slot;
    }
  };
  Row cur, nxt;
  uint32_t tile = blockIdx.x;
  int s = 0;
  if (tile < uint32_t(n_tiles)) fetch(tile, 0, cur);

  while (tile < uint32_t(n_tiles)) {
    const float* sb = s_bnd + 16 * s;
    // the next work item: the other source of this tile, or the first source of the next tile
    int s_next = s + 1;
    uint32_t tile_next = tile;
    if (s_next == p.n_src) {
      s_next = 0;
      tile_next = tile + gridDim.x;
    }
    if (tile_next < uint32_t(n_tiles)) fetch(tile_next, s_next, nxt);

    // ---- norm, normalise, hi / lo' planes of x_hat -------------------------------------------
    {
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < JT; ++j) ss = fmaf(cur.x[j], cur.x[j], ss);
      ss = warp_sum(ss);
      const float nrm = sqrtf(ss);
      // one reciprocal per vector instead of a division per coordinate: x_hat may differ from
      // x / (n + 1e-10) in the last bit, far inside the rounding of the contraction
      const float inv = 1.f / (nrm + 1e-10f);
      __half h[JT], l[JT];
#pragma unroll
      for (int j = 0; j < JT; ++j) split_hi_lo(cur.x[j] * inv, h[j], l[j]);
      if constexpr (JT == 4) {
        *reinterpret_cast<uint2*>(a_hi + warp * LD + lane * 4) =
            make_uint2(pack_h2(h[0], h[1]), pack_h2(h[2], h[3]));
        *reinterpret_cast<uint2*>(a_lo + warp * LD + lane * 4) =
            make_uint2(pack_h2(l[0], l[1]), pack_h2(l[2], l[3]));
      } else {
        *reinterpret_cast<uint32_t*>(a_hi + warp * LD + lane * 2) = pack_h2(h[0], h[1]);
        *reinterpret_cast<uint32_t*>(a_lo + warp * LD + lane * 2) = pack_h2(l[0], l[1]);
      }
      if constexpr (QJL) {
        if (s == 0) {
          float* xr = s_x + warp * (D + 8) + lane * JT;
#pragma unroll
          for (int j = 0; j < JT; ++j) xr[j] = cur.x[j];
        }
      }
      if (lane == 0) {
        s_nrm[warp] = nrm;
        s_head[warp] = cur.head;
        s_slot[warp] = cur.slot;
        if (cur.slot >= 0)
          *reinterpret_cast<float*>(p.norm[s] + cur.slot * p.norm_row_stride + cur.head * 4) = nrm;
      }
    }
    __syncthreads();

    // ---- y = x_hat Pi^T, codes -------------------------------------------------------------
    float acc[NTW][4];
    int idx[NTW][4];
    const int64_t slot_lo = s_slot[g], slot_hi = s_slot[g + 8];
    const int head_lo = s_head[g], head_hi = s_head[g + 8];
    if (col_warp) {
      plane_mma<D, NTW>(a_hi, a_lo, m_hi[0], m_lo[0], LD, warp * NTW, lane, acc);
#pragma unroll
      for (int i = 0; i < NTW; ++i) {
#pragma unroll
        for (int c = 0; c < 4; ++c) idx[i][c] = bucketize15(acc[i][c], sb);
        // code byte = (even coordinate << 4) | odd coordinate; the four lanes of a row hold
        // bytes 4*nt .. 4*nt+3 of it
        uint32_t w_lo = uint32_t((idx[i][0] << 4) | idx[i][1]) << (8 * t);
        uint32_t w_hi = uint32_t((idx[i][2] << 4) | idx[i][3]) << (8 * t);
        w_lo |= __shfl_xor_sync(0xffffffffu, w_lo, 1);
        w_hi |= __shfl_xor_sync(0xffffffffu, w_hi, 1);
        w_lo |= __shfl_xor_sync(0xffffffffu, w_lo, 2);
        w_hi |= __shfl_xor_sync(0xffffffffu, w_hi, 2);
        const int byte0 = 4 * (warp * NTW + i);
        if (t == 0 && slot_lo >= 0)
          *reinterpret_cast<uint32_t*>(p.code[s] + slot_lo * p.code_row_stride +
                                       int64_t(head_lo) * p.code_head_stride + byte0) = w_lo;
        if (t == 1 && slot_hi >= 0)
          *reinterpret_cast<uint32_t*>(p.code[s] + slot_hi * p.code_row_stride +
                                       int64_t(head_hi) * p.code_head_stride + byte0) = w_hi;
      }
    }
    __syncthreads();  // every warp has read x_hat: the planes may be overwritten

    if constexpr (QJL) {
      if (s == 0) {
        // ---- x_tilde = (c[code] Pi) n ; r = x - x_tilde ; gamma = |r| ------------------------
        if (col_warp) {
#pragma unroll
          for (int i = 0; i < NTW; ++i) {
            const int col = 8 * (warp * NTW + i) + 2 * t;
            __half h[4], l[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) split_hi_lo(s_cent[idx[i][c]], h[c], l[c]);
            *reinterpret_cast<uint32_t*>(a_hi + g * LD + col) = pack_h2(h[0], h[1]);
            *reinterpret_cast<uint32_t*>(a_lo + g * LD + col) = pack_h2(l[0], l[1]);
            *reinterpret_cast<uint32_t*>(a_hi + (g + 8) * LD + col) = pack_h2(h[2], h[3]);
            *reinterpret_cast<uint32_t*>(a_lo + (g + 8) * LD + col) = pack_h2(l[2], l[3]);
          }
        }
        __syncthreads();
        if (col_warp) plane_mma<D, NTW>(a_hi, a_lo, m_hi[1], m_lo[1], LD, warp * NTW, lane, acc);
        __syncthreads();  // every warp has read the centroid planes
        if (col_warp) {
          const float n_lo = s_nrm[g], n_hi = s_nrm[g + 8];
          float ss_lo = 0.f, ss_hi = 0.f;
#pragma unroll
          for (int i = 0; i < NTW; ++i) {
            const int col = 8 * (warp * NTW + i) + 2 * t;
            const float2 x_lo = *reinterpret_cast<const float2*>(s_x + g * (D + 8) + col);
            const float2 x_hi = *reinterpret_cast<const float2*>(s_x + (g + 8) * (D + 8) + col);
            const float r0 = x_lo.x - acc[i][0] * n_lo, r1 = x_lo.y - acc[i][1] * n_lo;
            const float r2 = x_hi.x - acc[i][2] * n_hi, r3 = x_hi.y - acc[i][3] * n_hi;
            ss_lo = fmaf(r0, r0, fmaf(r1, r1, ss_lo));
            ss_hi = fmaf(r2, r2, fmaf(r3, r3, ss_hi));
            __half h[4], l[4];
            split_hi_lo(r0, h[0], l[0]);
            split_hi_lo(r1, h[1], l[1]);
            split_hi_lo(r2, h[2], l[2]);
            split_hi_lo(r3, h[3], l[3]);
            *reinterpret_cast<uint32_t*>(a_hi + g * LD + col) = pack_h2(h[0], h[1]);
            *reinterpret_cast<uint32_t*>(a_lo + g * LD + col) = pack_h2(l[0], l[1]);
            *reinterpret_cast<uint32_t*>(a_hi + (g + 8) * LD + col) = pack_h2(h[2], h[3]);
            *reinterpret_cast<uint32_t*>(a_lo + (g + 8) * LD + col) = pack_h2(l[2], l[3]);
          }
          ss_lo += __shfl_xor_sync(0xffffffffu, ss_lo, 1);
          ss_hi += __shfl_xor_sync(0xffffffffu, ss_hi, 1);
          ss_lo += __shfl_xor_sync(0xffffffffu, ss_lo, 2);
          ss_hi += __shfl_xor_sync(0xffffffffu, ss_hi, 2);
          if (t == 0) {
            s_gpart[warp * 16 + g] = ss_lo;
            s_gpart[warp * 16 + g + 8] = ss_hi;
          }
        }
        __syncthreads();
        if (tid < 16 && s_slot[tid] >= 0) {
          float ss = 0.f;
#pragma unroll
          for (int w = 0; w < MW; ++w) ss += s_gpart[w * 16 + tid];
          *reinterpret_cast<float*>(p.gam + s_slot[tid] * p.gam_row_stride + s_head[tid] * 4) =
              sqrtf(ss);
        }
        // ---- sign(r S^T): bit j%8 of byte j/8 is 1 for a projection >= 0 ---------------------
        if (col_warp) {
          plane_mma<D, NTW>(a_hi, a_lo, m_hi[2], m_lo[2], LD, warp * NTW, lane, acc);
          uint32_t b_lo = 0, b_hi = 0;
#pragma unroll
          for (int i = 0; i < NTW; ++i) {
            b_lo |= ((acc[i][0] >= 0.f ? 1u : 0u) | (acc[i][1] >= 0.f ? 2u : 0u)) << (8 * i + 2 * t);
            b_hi |= ((acc[i][2] >= 0.f ? 1u : 0u) | (acc[i][3] >= 0.f ? 2u : 0u)) << (8 * i + 2 * t);
          }
          b_lo |= __shfl_xor_sync(0xffffffffu, b_lo, 1);
          b_hi |= __shfl_xor_sync(0xffffffffu, b_hi, 1);
          b_lo |= __shfl_xor_sync(0xffffffffu, b_lo, 2);
          b_hi |= __shfl_xor_sync(0xffffffffu, b_hi, 2);
          // bytes NTW*warp .. of the row's D/8 sign bytes
          uint8_t* d_lo = p.sign + slot_lo * p.sign_row_stride + head_lo * (D / 8) + NTW * warp;
          uint8_t* d_hi = p.sign + slot_hi * p.sign_row_stride + head_hi * (D / 8) + NTW * warp;
#pragma unroll
          for (int i = 0; i < NTW; ++i) {
            if (t == 0 && slot_lo >= 0) d_lo[i] = uint8_t(b_lo >> (8 * i));
            if (t == 1 && slot_hi >= 0) d_hi[i] = uint8_t(b_hi >> (8 * i));
          }
        }
        __syncthreads();  // planes and row data are rewritten by the next item
      }
    }
    cur = nxt;
    tile = tile_next;
    s = s_next;
  }
}

// below this many tiles the CTA-per-tile kernel is the faster one (measured cross-over at
// about 1000 tiles: it starts in 12 us and needs 6.6 us per wave of tiles, the warp-per-tile
// kernel 30 us and 33 us per eight tiles and SM)
constexpr int64_t kCoopMaxTiles = 1024;

template <int D, int DT, bool QJL>
static int launch_compress_coop(const CompressArgs& a, int64_t tiles, cudaStream_t stream) {
  using S = CoopSmem<D, QJL>;
  auto kern = compress_coop_kernel<D, DT, QJL>;
  static thread_local int configured_device = -1;
  static thread_local int sm_count = 0;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return fail(FQ_ERR_CUDA, "cudaGetDevice failed");
  if (configured_device != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         int(S::kBytes));
    if (e != cudaSuccess)
      return fail(FQ_ERR_CUDA, "compress: shared memory opt-in of %zu bytes refused: %s",
                  S::kBytes, cudaGetErrorString(e));
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    configured_device = dev;
  }
  const int per_sm = (S::kBytes <= 110 * 1024) ? 2 : 1;
  const int grid = int(tiles < int64_t(sm_count) * per_sm ? tiles : int64_t(sm_count) * per_sm);
  kern<<<grid, kCoopThreads, S::kBytes, stream>>>(a);
  return check_launch("compress kernel launch");
}

template <int D, int DT, bool QJL>
static int launch_compress_t(const CompressArgs& a, cudaStream_t stream) {
  using S = CompressSmem<D, QJL>;
  auto kern = compress_kernel<D, DT, QJL>;
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
  const int64_t tiles = (n_vec + kTileRows - 1) / kTileRows;
  if (tiles == 0) return FQ_OK;
  if (tiles < kCoopMaxTiles) return launch_compress_coop<D, DT, QJL>(a, tiles, stream);
  FQ_REQUIRE(n_vec < (int64_t(1) << 31) - 16 * 4096, FQ_ERR_UNSUPPORTED,
             "compress: %lld vectors in one call (at most 2^31)", (long long)n_vec);
  const int per_sm = QJL ? 1 : 2;
  const int64_t ctas = (tiles + kCompressWarps - 1) / kCompressWarps;  // a warp per tile
  const int grid = int(ctas < int64_t(sm_count) * per_sm ? ctas : int64_t(sm_count) * per_sm);
  kern<<<grid, kCompressThreads, S::kBytes, stream>>>(a);
  return check_launch("compress kernel launch");
}

template <int D, bool QJL>
static int launch_compress_d(const CompressArgs& a, int dtype, cudaStream_t stream) {
  switch (dtype) {
    case FQ_F32: return launch_compress_t<D, FQ_F32, QJL>(a, stream);
    case FQ_F16: return launch_compress_t<D, FQ_F16, QJL>(a, stream);
    case FQ_BF16: return launch_compress_t<D, FQ_BF16, QJL>(a, stream);
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
  FQ_RANGE("fq_tq4_compress");
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

extern "C" int fq_tq4_compress_into(const void* x, fq_dtype dtype, const float* rot_T_even,
                                    const float* rot_T_odd, const float* boundaries,
                                    int n_boundaries, uint8_t* packed, float* norms,
                                    int64_t n_segments, int64_t n_new, int64_t capacity,
                                    int64_t position, int head_dim, fq_stream_t stream) {
  FQ_RANGE("fq_tq4_compress_into");
  FQ_REQUIRE(n_segments >= 0 && n_new >= 0 && capacity >= 0 && position >= 0,
             FQ_ERR_INVALID_ARGUMENT, "fq_tq4_compress_into: negative size");
  FQ_REQUIRE(position + n_new <= capacity, FQ_ERR_INVALID_ARGUMENT,
             "fq_tq4_compress_into: %lld tokens at position %lld exceed the capacity %lld",
             (long long)n_new, (long long)position, (long long)capacity);
  if (n_segments == 0 || n_new == 0) return FQ_OK;
  FQ_REQUIRE(x && rot_T_even && rot_T_odd && boundaries && packed && norms,
             FQ_ERR_INVALID_ARGUMENT, "fq_tq4_compress_into: null pointer");
  FQ_REQUIRE(n_boundaries >= 1 && n_boundaries <= 15, FQ_ERR_INVALID_ARGUMENT,
             "n_boundaries %d outside [1, 15]", n_boundaries);
  FQ_REQUIRE(n_new < (int64_t(1) << 31), FQ_ERR_UNSUPPORTED,
             "fq_tq4_compress_into: %lld new tokens per segment", (long long)n_new);
  FQ_REQUIRE(aligned(x, 4 * elem_bytes(dtype)) && aligned(packed, 4) && aligned(norms, 4),
             FQ_ERR_ALIGNMENT, "fq_tq4_compress_into: x must be aligned to 4 elements");
  CompressArgs a{};
  a.src[0] = x; a.n_src = 1;
  a.n_tokens = n_segments * n_new; a.heads = 1; a.token_stride = head_dim;
  a.mat_a = rot_T_even; a.mat_b = rot_T_odd; a.rot_split = 1;
  a.bnd[0] = a.bnd[1] = boundaries; a.nb[0] = a.nb[1] = n_boundaries;
  a.code[0] = packed; a.code_row_stride = head_dim / 2; a.code_head_stride = 0;
  a.norm[0] = reinterpret_cast<uint8_t*>(norms); a.norm_row_stride = 4;
  a.seg_len = uint32_t(n_new); a.seg_stride = capacity; a.seg_offset = position;
  return launch_compress(a, dtype, head_dim, false, stream);
}

extern "C" int fq_tq_prod_quantize(const void* x, fq_dtype dtype, const float* rotation,
                                   const float* boundaries, int n_boundaries,
                                   const float* centroids, const float* qjl, uint8_t* packed,
                                   float* norms, uint8_t* sign_bits, float* gamma,
                                   int64_t n_vectors, int head_dim, fq_stream_t stream) {
  FQ_RANGE("fq_tq_prod_quantize");
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
  FQ_RANGE("fq_tq4_compress_append");
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
  FQ_RANGE("fq_tq4_compress_append_qjl");
  return append_common(key, value, dtype, n_tokens, num_kv_heads, head_dim, token_stride,
                       rotation, boundaries_k, n_boundaries_k, centroids_k, boundaries_v,
                       n_boundaries_v, qjl, kv_cache, kq_cache, num_slots, slot_mapping,
                       slot_is_int64, true, stream);
}
