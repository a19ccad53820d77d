// Split-K paged decode over the packed TQ4 cache for sm_100a.
//
// Three launches per call:
//   1. rotate_q_kernel   q_rot = round_to_q_dtype(q Pi^T), stored as fp16
//   2. paged_decode_kernel  one CTA per (sequence, split): streams whole cache pages through a
//      shared-memory ring with bulk copies and produces one (acc, m, l) partial per q head
//   3. merge_rotate_kernel  merges the partials of a sequence, rounds, multiplies by Pi
//
// The streaming kernel is bound by HBM traffic (136 B per token and KV head), but only if
// the per-byte instruction count stays near 3: a nibble code is two table look-ups and,
// with 4 query heads per KV head, eight multiply-adds per byte, which the fp32 pipe cannot
// sustain at 7 TB/s.  So the multiply-adds go to the tensor pipe (mma.sync m16n8k16, the
// N dimension being the query heads of the group) and a byte is turned into two fp16
// centroids by ONE shared-memory look-up in a 256-entry table of fp16 pairs, replicated per
// lane so that the look-ups never conflict.  Operand fragments are built directly in
// registers in the order the look-ups deliver them; the k-dimension of the QK product and
// the row dimension of the PV product are permuted accordingly (the query fragment and the
// output write-back apply the same permutation).
#include "fq_common.cuh"

namespace fq {

constexpr int kDecodeWarps = 8;                             // compute warps per CTA
constexpr int kDecodeThreads = (kDecodeWarps + 1) * 32;     // + one producer warp
constexpr int kLutBytes = 256 * 32 * 4;                     // one table, one copy per lane
constexpr int kMaxStages = 32;
constexpr int kPartPad = 4;                                 // partial row = D + 4 floats
constexpr float kPScaleLog2 = 14.f;                         // P is scaled by 2^14 for fp16

struct DecodeArgs {
  const __half* q_rot;  // (num_seqs, Hq, D)
  const uint8_t* kv_cache;
  const int32_t* block_table;
  int64_t bt_stride;
  const int32_t* seq_lens;
  const float* cent_k;
  int nck;
  const float* cent_v;
  int ncv;
  int num_seqs, hq, hkv, block_size;
  int64_t num_blocks;
  float scale_log2;
  int num_splits;
  int stages;
  float* partials;  // (num_seqs, Hq, S, D+4)
  uint32_t* status;
};

// ------------------------------------------------------------------------------------
// 1. q rotation: out[r][j] = fp16(round_T(sum_k q[r][k] * Pi[j][k]))
// ------------------------------------------------------------------------------------
template <int D, typename T>
__global__ void __launch_bounds__(256) rotate_q_kernel(const T* __restrict__ q,
                                                      const float* __restrict__ rotation,
                                                      __half* __restrict__ out, int n_rows) {
  constexpr int ROWS = 8;
  extern __shared__ __align__(16) float rq_smem[];
  float* bt = rq_smem;           // [k][j] = Pi[j][k]
  float* qs = rq_smem + D * D;   // [ROWS][D]
  const int tid = threadIdx.x;
  for (int i = tid; i < D * D; i += 256) {
    const int k = i / D, j = i % D;
    bt[i] = rotation[j * D + k];
  }
  const int row0 = blockIdx.x * ROWS;
  for (int i = tid; i < ROWS * D; i += 256) {
    const int r = row0 + i / D;
    qs[i] = r < n_rows ? to_f32(q[int64_t(r) * D + i % D]) : 0.f;
  }
  __syncthreads();
  constexpr int GROUPS = 256 / D;       // thread groups, each covers all D outputs
  constexpr int RPG = ROWS / GROUPS;    // rows per group
  const int j = tid % D, grp = tid / D;
  float acc[RPG];
#pragma unroll
  for (int r = 0; r < RPG; ++r) acc[r] = 0.f;
#pragma unroll 4
  for (int k4 = 0; k4 < D; k4 += 4) {
    const float b0 = bt[(k4 + 0) * D + j], b1 = bt[(k4 + 1) * D + j];
    const float b2 = bt[(k4 + 2) * D + j], b3 = bt[(k4 + 3) * D + j];
#pragma unroll
    for (int r = 0; r < RPG; ++r) {
      const float4 a = *reinterpret_cast<const float4*>(qs + (grp * RPG + r) * D + k4);
      acc[r] = fmaf(a.x, b0, acc[r]);
      acc[r] = fmaf(a.y, b1, acc[r]);
      acc[r] = fmaf(a.z, b2, acc[r]);
      acc[r] = fmaf(a.w, b3, acc[r]);
    }
  }
#pragma unroll
  for (int r = 0; r < RPG; ++r) {
    const int row = row0 + grp * RPG + r;
    if (row < n_rows) out[int64_t(row) * D + j] = __float2half_rn(to_f32(from_f32<T>(acc[r])));
  }
}

// ------------------------------------------------------------------------------------
// 2. streaming kernel
// ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t lut_get(const unsigned char* lut_lane, uint32_t word,
                                            int byte_i) {
  // byte address of entry e for this lane: e * 128 + lane * 4 (lane part is in lut_lane)
  const uint32_t off = (byte_i == 0) ? ((word << 7) & 0x7f80u)
                                     : ((word >> (8 * byte_i - 7)) & 0x7f80u);
  return *reinterpret_cast<const uint32_t*>(lut_lane + off);
}

template <int D>
__global__ void __launch_bounds__(kDecodeThreads, 1) paged_decode_kernel(DecodeArgs p) {
  constexpr int KS = D / 16;  // k-steps of the QK product = m-tiles of the PV product
  constexpr int KW = D / 32;  // 32-bit words of K codes per lane and row
  constexpr int VB = D / 16;  // bytes of V codes per lane and row

  extern __shared__ __align__(1024) unsigned char smem[];
  unsigned char* lut_k = smem;
  unsigned char* lut_v = smem + kLutBytes;
  const int half_d = D / 2;
  const int row_bytes = p.hkv * (D + 8);
  const uint32_t page_bytes = uint32_t(p.block_size) * row_bytes;
  unsigned char* ring = smem + 2 * kLutBytes;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ring + size_t(p.stages) * page_bytes);
  uint64_t* empty_bar = full_bar + p.stages;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int seq = blockIdx.y, split = blockIdx.x;
  const int group = p.hq / p.hkv;  // q heads per KV head (<= 8)

  // ---- page range of this CTA ---------------------------------------------------------
  int seq_len = p.seq_lens[seq];
  if (seq_len < 0) seq_len = 0;
  const int n_pages = (seq_len + p.block_size - 1) / p.block_size;
  const int pps = (n_pages + p.num_splits - 1) / p.num_splits;
  const int page0 = split * pps;
  int my_pages = n_pages - page0;
  my_pages = my_pages < 0 ? 0 : (my_pages > pps ? pps : my_pages);

  // ---- set-up: barriers, look-up tables ----------------------------------------------
  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, kDecodeWarps);
    }
    mbar_fence_init();
  }
  for (int i = tid; i < 256 * 32; i += kDecodeThreads) {
    const int e = i >> 5;
    const int hi = e >> 4, lo = e & 15;
    const float kh = hi < p.nck ? p.cent_k[hi] : 0.f, kl = lo < p.nck ? p.cent_k[lo] : 0.f;
    const float vh = hi < p.ncv ? p.cent_v[hi] : 0.f, vl = lo < p.ncv ? p.cent_v[lo] : 0.f;
    reinterpret_cast<uint32_t*>(lut_k)[i] = pack_half2(kh, kl);  // low half: even coordinate
    reinterpret_cast<uint32_t*>(lut_v)[i] = pack_half2(vh, vl);
  }
  __syncthreads();

  const int units_per_page = p.block_size / 16;
  bool timed_out = false;

  // per-warp softmax state (compute warps)
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float oacc[KS][4];
#pragma unroll
  for (int j = 0; j < KS; ++j)
#pragma unroll
    for (int c = 0; c < 4; ++c) oacc[j][c] = 0.f;

  if (warp == kDecodeWarps) {
    // ================= producer =================
    if (lane == 0) {
      for (int i = 0; i < my_pages; ++i) {
        const int stage = i % p.stages;
        if (i >= p.stages) {
          if (!mbar_wait(empty_bar + stage, ((i / p.stages) & 1) ^ 1)) {
            atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
            break;
          }
        }
        int64_t phys = p.block_table[int64_t(seq) * p.bt_stride + page0 + i];
        if (phys < 0 || phys >= p.num_blocks) {
          atomicOr(p.status, FQ_DEV_BAD_BLOCK_INDEX);
          phys = 0;
        }
        mbar_expect_tx(full_bar + stage, page_bytes);
        bulk_g2s(ring + size_t(stage) * page_bytes, p.kv_cache + phys * int64_t(page_bytes),
                 page_bytes, full_bar + stage);
      }
    }
  } else {
    // ================= consumers =================
    const int wph = kDecodeWarps / p.hkv;  // warps per KV head
    const int head = warp % p.hkv;
    const int sub = warp / p.hkv;
    const unsigned char* lk = lut_k + lane * 4;
    const unsigned char* lv = lut_v + lane * 4;

    // query fragments: lane (g,t) holds, for k-step s, the coordinates of cache bytes
    // (D/8)*t + 2s and (D/8)*t + 2s + 1 of q head `head*group + g`
    uint32_t qf[KS][2];
    {
      const bool valid = g < group;
      const __half* qrow = p.q_rot + (int64_t(seq) * p.hq + head * group + (valid ? g : 0)) * D;
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        const int b0 = (D / 8) * t + 2 * s;
        const uint2 v = *reinterpret_cast<const uint2*>(qrow + 2 * b0);
        qf[s][0] = valid ? v.x : 0u;
        qf[s][1] = valid ? v.y : 0u;
      }
    }

    const int k_norm_off = p.hkv * half_d + 4 * head;
    const int v_code_off = p.hkv * half_d + 4 * p.hkv + head * half_d;
    const int v_norm_off = 2 * p.hkv * half_d + 4 * p.hkv + 4 * head;
    const int k_code_off = head * half_d;
    const bool wide = (p.hkv & 1) == 0;  // vector loads need an even number of KV heads

    int unit = 0;  // running unit index over this CTA's pages
    for (int i = 0; i < my_pages && !timed_out; ++i) {
      const int stage = i % p.stages;
      if (!mbar_wait(full_bar + stage, (i / p.stages) & 1)) {
        timed_out = true;
        break;
      }
      const unsigned char* page = ring + size_t(stage) * page_bytes;
      const int tok_page0 = (page0 + i) * p.block_size;
      for (int u = 0; u < units_per_page; ++u, ++unit) {
        if (unit % wph != sub) continue;
        const int tok0 = tok_page0 + u * 16;
        if (tok0 >= seq_len) continue;
        const unsigned char* rows = page + size_t(u) * 16 * row_bytes;
        const unsigned char* r_lo = rows + size_t(g) * row_bytes;
        const unsigned char* r_hi = rows + size_t(g + 8) * row_bytes;

        // ---------- S^T = K q^T : rows = 16 tokens, cols = q heads of the group ----------
        uint32_t ka[KW], kb[KW];
        if constexpr (KW == 4) {
          if (wide) {
            const uint4 a = *reinterpret_cast<const uint4*>(r_lo + k_code_off + 16 * t);
            const uint4 b = *reinterpret_cast<const uint4*>(r_hi + k_code_off + 16 * t);
            ka[0] = a.x; ka[1] = a.y; ka[2] = a.z; ka[3] = a.w;
            kb[0] = b.x; kb[1] = b.y; kb[2] = b.z; kb[3] = b.w;
          } else {  // odd number of KV heads: rows are only 8-byte aligned
            const uint2* pa = reinterpret_cast<const uint2*>(r_lo + k_code_off + 16 * t);
            const uint2* pb = reinterpret_cast<const uint2*>(r_hi + k_code_off + 16 * t);
            const uint2 a0 = pa[0], a1 = pa[1], b0 = pb[0], b1 = pb[1];
            ka[0] = a0.x; ka[1] = a0.y; ka[2] = a1.x; ka[3] = a1.y;
            kb[0] = b0.x; kb[1] = b0.y; kb[2] = b1.x; kb[3] = b1.y;
          }
        } else {
          const uint2 a = *reinterpret_cast<const uint2*>(r_lo + k_code_off + 8 * t);
          const uint2 b = *reinterpret_cast<const uint2*>(r_hi + k_code_off + 8 * t);
          ka[0] = a.x; ka[1] = a.y;
          kb[0] = b.x; kb[1] = b.y;
        }
        float sacc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < KS; ++s) {
          const int w = s >> 1, bi = (s & 1) * 2;
          const uint32_t a0 = lut_get(lk, ka[w], bi);
          const uint32_t a1 = lut_get(lk, kb[w], bi);
          const uint32_t a2 = lut_get(lk, ka[w], bi + 1);
          const uint32_t a3 = lut_get(lk, kb[w], bi + 1);
          mma_f16(sacc, a0, a1, a2, a3, qf[s][0], qf[s][1]);
        }

        // ---------- online softmax in the accumulator layout -----------------------------
        const float nk_lo = *reinterpret_cast<const float*>(r_lo + k_norm_off);
        const float nk_hi = *reinterpret_cast<const float*>(r_hi + k_norm_off);
        const float nv_lo = *reinterpret_cast<const float*>(r_lo + v_norm_off);
        const float nv_hi = *reinterpret_cast<const float*>(r_hi + v_norm_off);
        const bool ok_lo = tok0 + g < seq_len, ok_hi = tok0 + g + 8 < seq_len;
        // log2 of the value norm is folded into the exponent so that the fp16 weights stay
        // in range whatever the norms are; clamped below so that l cannot overflow
        const float lv_lo = fmaxf(fast_log2(nv_lo), -40.f), lv_hi = fmaxf(fast_log2(nv_hi), -40.f);
        float s_lo[2], s_hi[2], e_lo[2], e_hi[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          s_lo[c] = sacc[c] * (nk_lo * p.scale_log2);
          s_hi[c] = sacc[2 + c] * (nk_hi * p.scale_log2);
          e_lo[c] = ok_lo ? s_lo[c] + lv_lo : -INFINITY;
          e_hi[c] = ok_hi ? s_hi[c] + lv_hi : -INFINITY;
        }
        float mx[2] = {fmaxf(e_lo[0], e_hi[0]), fmaxf(e_lo[1], e_hi[1])};
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], o));
          mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], o));
        }
        const float m_new[2] = {fmaxf(m_run[0], mx[0]), fmaxf(m_run[1], mx[1])};
        const bool grew = (m_new[0] > m_run[0]) || (m_new[1] > m_run[1]);
        if (__any_sync(0xffffffffu, grew)) {
          const float a0 = (m_run[0] == -INFINITY) ? 0.f : fast_exp2(m_run[0] - m_new[0]);
          const float a1 = (m_run[1] == -INFINITY) ? 0.f : fast_exp2(m_run[1] - m_new[1]);
          l_run[0] *= a0;
          l_run[1] *= a1;
#pragma unroll
          for (int j = 0; j < KS; ++j) {
            oacc[j][0] *= a0; oacc[j][2] *= a0;
            oacc[j][1] *= a1; oacc[j][3] *= a1;
          }
          m_run[0] = m_new[0];
          m_run[1] = m_new[1];
        }
        float w_lo[2], w_hi[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const float mref = (m_run[c] == -INFINITY) ? 0.f : m_run[c];
          // a zero value norm has lg2 = -inf before the clamp: give it weight 0 exactly
          w_lo[c] = (ok_lo && nv_lo > 0.f)
                        ? fast_exp2(s_lo[c] + fast_log2(nv_lo) - mref + kPScaleLog2) : 0.f;
          w_hi[c] = (ok_hi && nv_hi > 0.f)
                        ? fast_exp2(s_hi[c] + fast_log2(nv_hi) - mref + kPScaleLog2) : 0.f;
          const float p_lo = ok_lo ? fast_exp2(s_lo[c] - mref) : 0.f;
          const float p_hi = ok_hi ? fast_exp2(s_hi[c] - mref) : 0.f;
          l_run[c] += p_lo + p_hi;
        }
        // weights as the B operand of the PV product: transpose (token, head) -> (head, token)
        const uint32_t pb0 = movmatrix_trans(pack_half2(w_lo[0], w_lo[1]));
        const uint32_t pb1 = movmatrix_trans(pack_half2(w_hi[0], w_hi[1]));

        // ---------- O^T += V^T P^T : rows = value coordinates, cols = q heads -------------
        // lane (g,t) needs tokens 2t, 2t+1, 2t+8, 2t+9 and cache bytes VB*g .. VB*g+VB-1
        const unsigned char* vr = rows + v_code_off + VB * g;
        uint32_t vw[4][VB / 4];
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const int tokr = 2 * t + (r & 1) + (r >> 1) * 8;
          const unsigned char* src = vr + size_t(tokr) * row_bytes;
          if constexpr (VB == 8) {
            if (wide) {
              const uint2 x = *reinterpret_cast<const uint2*>(src);
              vw[r][0] = x.x; vw[r][1] = x.y;
            } else {  // the V region starts at an odd multiple of 4 bytes
              vw[r][0] = reinterpret_cast<const uint32_t*>(src)[0];
              vw[r][1] = reinterpret_cast<const uint32_t*>(src)[1];
            }
          } else {
            vw[r][0] = *reinterpret_cast<const uint32_t*>(src);
          }
        }
#pragma unroll
        for (int j = 0; j < KS; ++j) {
          const int w = j >> 2, bi = j & 3;
          const uint32_t l0 = lut_get(lv, vw[0][w], bi);
          const uint32_t l1 = lut_get(lv, vw[1][w], bi);
          const uint32_t l2 = lut_get(lv, vw[2][w], bi);
          const uint32_t l3 = lut_get(lv, vw[3][w], bi);
          const uint32_t a0 = prmt(l0, l1, 0x5410);  // even coordinate, tokens 2t, 2t+1
          const uint32_t a1 = prmt(l0, l1, 0x7632);  // odd coordinate
          const uint32_t a2 = prmt(l2, l3, 0x5410);  // even coordinate, tokens 2t+8, 2t+9
          const uint32_t a3 = prmt(l2, l3, 0x7632);
          mma_f16(oacc[j], a0, a1, a2, a3, pb0, pb1);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(empty_bar + stage);
    }
    if (timed_out && lane == 0) atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
  }

  // ---- CTA-level merge of the warps that shared a KV head, then the partial row ----------
  __syncthreads();  // every page is consumed: tables and ring are free
  float* mbuf = reinterpret_cast<float*>(smem);  // [warp][8 cols][D + 2]
  constexpr int MROW = D + 2;
  if (warp < kDecodeWarps) {
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], o);
      l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], o);
    }
    float* mine = mbuf + size_t(warp) * 8 * MROW;
#pragma unroll
    for (int j = 0; j < KS; ++j) {
      const int b = VB * g + j;  // cache byte -> coordinates 2b (row g) and 2b+1 (row g+8)
      mine[(2 * t) * MROW + 2 * b] = oacc[j][0];
      mine[(2 * t + 1) * MROW + 2 * b] = oacc[j][1];
      mine[(2 * t) * MROW + 2 * b + 1] = oacc[j][2];
      mine[(2 * t + 1) * MROW + 2 * b + 1] = oacc[j][3];
    }
    if (g == 0) {
      mine[(2 * t) * MROW + D] = m_run[0];
      mine[(2 * t) * MROW + D + 1] = l_run[0];
      mine[(2 * t + 1) * MROW + D] = m_run[1];
      mine[(2 * t + 1) * MROW + D + 1] = l_run[1];
    }
  }
  __syncthreads();
  {
    const int wph = kDecodeWarps / p.hkv;
    const int items = p.hq * (D / 4);
    for (int it = tid; it < items; it += kDecodeThreads) {
      const int hq = it / (D / 4), chunk = it % (D / 4);
      const int head = hq / group, col = hq % group;
      float m_star = -INFINITY;
      for (int s = 0; s < wph; ++s)
        m_star = fmaxf(m_star, mbuf[(size_t(head + s * p.hkv) * 8 + col) * MROW + D]);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      float l = 0.f;
      for (int s = 0; s < wph; ++s) {
        const float* src = mbuf + (size_t(head + s * p.hkv) * 8 + col) * MROW;
        const float m = src[D];
        const float wgt = (m == -INFINITY) ? 0.f : fast_exp2(m - m_star);
        acc.x += wgt * src[4 * chunk + 0];
        acc.y += wgt * src[4 * chunk + 1];
        acc.z += wgt * src[4 * chunk + 2];
        acc.w += wgt * src[4 * chunk + 3];
        l += wgt * src[D + 1];
      }
      const float unscale = 1.f / 16384.f;  // 2^-kPScaleLog2
      acc.x *= unscale; acc.y *= unscale; acc.z *= unscale; acc.w *= unscale;
      float* dst = p.partials +
                   ((int64_t(seq) * p.hq + hq) * p.num_splits + split) * (D + kPartPad);
      *reinterpret_cast<float4*>(dst + 4 * chunk) = acc;
      if (chunk == 0) *reinterpret_cast<float4*>(dst + D) = make_float4(m_star, l, 0.f, 0.f);
    }
  }
}

// ------------------------------------------------------------------------------------
// 3. merge of partials + rounding + out = o_rot Pi
//    partials: (n_groups, num_seqs, Hq, n_splits, D+4); grid (ceil(Hq/HPB), num_seqs)
// ------------------------------------------------------------------------------------
template <int D, typename T>
__global__ void __launch_bounds__(D) merge_rotate_kernel(const float* __restrict__ partials,
                                                        int n_groups, int n_splits,
                                                        const float* __restrict__ rotation,
                                                        T* __restrict__ out, int num_seqs,
                                                        int hq) {
  constexpr int HPB = 8;
  __shared__ __align__(16) float o_s[HPB][D];
  const int d = threadIdx.x;
  const int seq = blockIdx.y, h0 = blockIdx.x * HPB;
  const int64_t group_stride = int64_t(num_seqs) * hq * n_splits * (D + kPartPad);
#pragma unroll 1
  for (int hh = 0; hh < HPB; ++hh) {
    const int h = h0 + hh;
    float o = 0.f;
    if (h < hq) {
      const float* base = partials + (int64_t(seq) * hq + h) * n_splits * (D + kPartPad);
      float m_star = -INFINITY;
      for (int gi = 0; gi < n_groups; ++gi)
        for (int s = 0; s < n_splits; ++s)
          m_star = fmaxf(m_star, base[gi * group_stride + int64_t(s) * (D + kPartPad) + D]);
      float num = 0.f, den = 0.f;
      for (int gi = 0; gi < n_groups; ++gi)
        for (int s = 0; s < n_splits; ++s) {
          const float* row = base + gi * group_stride + int64_t(s) * (D + kPartPad);
          const float m = row[D];
          const float w = (m == -INFINITY) ? 0.f : exp2f(m - m_star);
          num = fmaf(w, row[d], num);
          den = fmaf(w, row[D + 1], den);
        }
      o = den > 0.f ? num / den : 0.f;
      o = to_f32(from_f32<T>(o));  // the reference rounds the rotated output to q's dtype
    }
    o_s[hh][d] = o;
  }
  __syncthreads();
  float acc[HPB];
#pragma unroll
  for (int hh = 0; hh < HPB; ++hh) acc[hh] = 0.f;
#pragma unroll 2
  for (int k4 = 0; k4 < D; k4 += 4) {
    const float r0 = rotation[(k4 + 0) * D + d], r1 = rotation[(k4 + 1) * D + d];
    const float r2 = rotation[(k4 + 2) * D + d], r3 = rotation[(k4 + 3) * D + d];
#pragma unroll
    for (int hh = 0; hh < HPB; ++hh) {
      const float4 a = *reinterpret_cast<const float4*>(&o_s[hh][k4]);
      acc[hh] = fmaf(a.x, r0, acc[hh]);
      acc[hh] = fmaf(a.y, r1, acc[hh]);
      acc[hh] = fmaf(a.z, r2, acc[hh]);
      acc[hh] = fmaf(a.w, r3, acc[hh]);
    }
  }
#pragma unroll
  for (int hh = 0; hh < HPB; ++hh) {
    const int h = h0 + hh;
    if (h < hq) out[(int64_t(seq) * hq + h) * D + d] = from_f32<T>(acc[hh]);
  }
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
struct WorkspaceLayout {
  size_t q_rot_off, partials_off, total;
};

static WorkspaceLayout workspace_layout(int num_seqs, int hq, int d, int splits) {
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  WorkspaceLayout w;
  w.q_rot_off = 256;
  w.partials_off = up(w.q_rot_off + size_t(num_seqs) * hq * d * sizeof(__half));
  w.total = up(w.partials_off + size_t(num_seqs) * hq * splits * (d + kPartPad) * sizeof(float));
  return w;
}

static int auto_splits(int num_seqs, int sm_count) {
  int s = (2 * sm_count + num_seqs - 1) / num_seqs;
  if (s < 1) s = 1;
  if (s > 32) s = 32;
  return s;
}

static int device_sm_count() {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return sms;
}

template <int D>
static int launch_partials(const DecodeArgs& a, cudaStream_t stream) {
  const size_t page_bytes = size_t(a.block_size) * a.hkv * (D + 8);
  const size_t smem = 2 * size_t(kLutBytes) + size_t(a.stages) * page_bytes +
                      2 * size_t(a.stages) * sizeof(uint64_t);
  auto kern = paged_decode_kernel<D>;
  // opt in once per (thread, device, size): the attribute call is not free
  static thread_local int set_dev = -1;
  static thread_local size_t set_bytes = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (set_dev != dev || set_bytes < smem) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess)
      return fail(FQ_ERR_CUDA, "paged decode: shared memory opt-in of %zu bytes refused: %s",
                  smem, cudaGetErrorString(e));
    set_dev = dev;
    set_bytes = smem;
  }
  dim3 grid(a.num_splits, a.num_seqs);
  kern<<<grid, kDecodeThreads, smem, stream>>>(a);
  return check_launch("paged decode kernel launch");
}

template <int D>
static int rotate_q(const void* q, int dtype, const float* rotation, __half* out, int rows,
                    cudaStream_t stream) {
  const size_t smem = (size_t(D) * D + 8 * D) * sizeof(float);
  const int grid = (rows + 7) / 8;
  static thread_local int set_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (set_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(rotate_q_kernel<D, __nv_bfloat16>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(rotate_q_kernel<D, __half>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess)
      return fail(FQ_ERR_CUDA, "rotate_q: shared memory opt-in refused: %s",
                  cudaGetErrorString(e));
    set_dev = dev;
  }
  if (dtype == FQ_BF16)
    rotate_q_kernel<D, __nv_bfloat16><<<grid, 256, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(q), rotation, out, rows);
  else
    rotate_q_kernel<D, __half><<<grid, 256, smem, stream>>>(static_cast<const __half*>(q),
                                                            rotation, out, rows);
  return check_launch("rotate_q kernel launch");
}

template <int D>
static int merge_rotate(const float* partials, int n_groups, int n_splits, const float* rotation,
                        void* out, int dtype, int num_seqs, int hq, cudaStream_t stream) {
  dim3 grid((hq + 7) / 8, num_seqs);
  if (dtype == FQ_BF16)
    merge_rotate_kernel<D, __nv_bfloat16><<<grid, D, 0, stream>>>(
        partials, n_groups, n_splits, rotation, static_cast<__nv_bfloat16*>(out), num_seqs, hq);
  else
    merge_rotate_kernel<D, __half><<<grid, D, 0, stream>>>(
        partials, n_groups, n_splits, rotation, static_cast<__half*>(out), num_seqs, hq);
  return check_launch("merge kernel launch");
}

static int validate_decode(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                           const int32_t* block_table, const int32_t* seq_lens,
                           const float* centroids_k, int nck, const float* centroids_v, int ncv,
                           const float* rotation, int num_seqs, int hq, int hkv, int head_dim,
                           int block_size, int64_t num_blocks, int num_splits) {
  FQ_REQUIRE(num_seqs >= 0 && hq >= 1 && hkv >= 1 && num_blocks >= 0 && num_splits >= 0,
             FQ_ERR_INVALID_ARGUMENT, "paged decode: negative size");
  FQ_REQUIRE(q && kv_cache && block_table && seq_lens && centroids_k && centroids_v && rotation,
             FQ_ERR_INVALID_ARGUMENT, "paged decode: null pointer");
  FQ_REQUIRE(dtype == FQ_F16 || dtype == FQ_BF16, FQ_ERR_UNSUPPORTED,
             "paged decode: q must be fp16 or bf16");
  FQ_REQUIRE(nck >= 1 && nck <= 16 && ncv >= 1 && ncv <= 16, FQ_ERR_INVALID_ARGUMENT,
             "centroid count outside [1, 16]");
  FQ_REQUIRE(head_dim == 128 || head_dim == 64, FQ_ERR_UNSUPPORTED,
             "paged decode: head_dim %d (built for 64 and 128)", head_dim);
  FQ_REQUIRE(hkv == 1 || hkv == 2 || hkv == 4 || hkv == 8, FQ_ERR_UNSUPPORTED,
             "paged decode: num_kv_heads %d (built for 1, 2, 4, 8)", hkv);
  FQ_REQUIRE(hq % hkv == 0 && hq / hkv <= 8, FQ_ERR_UNSUPPORTED,
             "paged decode: %d q heads per KV head (at most 8, and a whole number)", hq / hkv);
  FQ_REQUIRE(block_size >= 16 && block_size % 16 == 0, FQ_ERR_UNSUPPORTED,
             "paged decode: block_size %d is not a multiple of 16", block_size);
  FQ_REQUIRE(aligned(kv_cache, 16) && aligned(q, 16), FQ_ERR_ALIGNMENT,
             "paged decode: kv_cache and q must be 16-byte aligned");
  return FQ_OK;
}

static int pick_stages(int block_size, int hkv, int head_dim) {
  const size_t page_bytes = size_t(block_size) * hkv * (head_dim + 8);
  const size_t budget = 227 * 1024 - 2 * size_t(kLutBytes) - 1024;
  size_t n = budget / (page_bytes + 16);
  // enough bytes in flight per SM to cover HBM latency, no more
  const size_t want = (96 * 1024 + page_bytes - 1) / page_bytes;
  if (n > want) n = want;
  if (n > size_t(kMaxStages)) n = kMaxStages;
  return int(n);
}

}  // namespace fq

using namespace fq;

extern "C" size_t fq_paged_decode_workspace_bytes(int num_seqs, int num_q_heads, int head_dim,
                                                  int num_splits) {
  if (num_seqs < 0 || num_q_heads < 0 || head_dim < 0) return 0;
  if (num_splits <= 0) num_splits = 32;  // upper bound of the automatic choice
  return workspace_layout(num_seqs, num_q_heads, head_dim, num_splits).total;
}

static int decode_front(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                        const int32_t* block_table, int64_t block_table_stride,
                        const int32_t* seq_lens, const float* centroids_k, int nck,
                        const float* centroids_v, int ncv, const float* rotation, int num_seqs,
                        int hq, int hkv, int head_dim, int block_size, int64_t num_blocks,
                        float sm_scale, int num_splits, float* partials, void* workspace,
                        size_t workspace_bytes, size_t need, cudaStream_t stream) {
  FQ_REQUIRE(workspace && aligned(workspace, 256), FQ_ERR_WORKSPACE,
             "paged decode: workspace is null or not 256-byte aligned");
  FQ_REQUIRE(workspace_bytes >= need, FQ_ERR_WORKSPACE,
             "paged decode: workspace has %zu bytes, %zu needed", workspace_bytes, need);
  const int stages = pick_stages(block_size, hkv, head_dim);
  FQ_REQUIRE(stages >= 2, FQ_ERR_UNSUPPORTED,
             "paged decode: a page of %d tokens x %d heads does not fit the shared-memory ring",
             block_size, hkv);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  const __half* q_rot = reinterpret_cast<const __half*>(ws + 256);
  if (rotation) {
    __half* dst = reinterpret_cast<__half*>(ws + 256);
    int rc = head_dim == 128 ? rotate_q<128>(q, dtype, rotation, dst, num_seqs * hq, stream)
                             : rotate_q<64>(q, dtype, rotation, dst, num_seqs * hq, stream);
    if (rc != FQ_OK) return rc;
  } else {
    q_rot = static_cast<const __half*>(q);  // caller supplied the rotated fp16 query
  }
  DecodeArgs a{};
  a.q_rot = q_rot;
  a.kv_cache = kv_cache;
  a.block_table = block_table;
  a.bt_stride = block_table_stride;
  a.seq_lens = seq_lens;
  a.cent_k = centroids_k; a.nck = nck;
  a.cent_v = centroids_v; a.ncv = ncv;
  a.num_seqs = num_seqs; a.hq = hq; a.hkv = hkv; a.block_size = block_size;
  a.num_blocks = num_blocks;
  a.scale_log2 = sm_scale * 1.4426950408889634f;
  a.num_splits = num_splits;
  a.stages = stages;
  a.partials = partials;
  a.status = reinterpret_cast<uint32_t*>(ws);
  return head_dim == 128 ? launch_partials<128>(a, stream) : launch_partials<64>(a, stream);
}

extern "C" int fq_split_k_paged_decode(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                                       const int32_t* block_table, int64_t block_table_stride,
                                       const int32_t* seq_lens, const float* centroids_k,
                                       int n_centroids_k, const float* centroids_v,
                                       int n_centroids_v, const float* rotation, int num_seqs,
                                       int num_q_heads, int num_kv_heads, int head_dim,
                                       int block_size, int64_t num_blocks, float sm_scale,
                                       void* out, int num_splits, void* workspace,
                                       size_t workspace_bytes, fq_stream_t stream) {
  int rc = validate_decode(q, dtype, kv_cache, block_table, seq_lens, centroids_k, n_centroids_k,
                           centroids_v, n_centroids_v, rotation, num_seqs, num_q_heads,
                           num_kv_heads, head_dim, block_size, num_blocks, num_splits);
  if (rc != FQ_OK) return rc;
  FQ_REQUIRE(out && aligned(out, 2), FQ_ERR_INVALID_ARGUMENT, "paged decode: out is null");
  if (num_seqs == 0) return FQ_OK;
  if (num_splits == 0) num_splits = auto_splits(num_seqs, device_sm_count());
  const WorkspaceLayout w = workspace_layout(num_seqs, num_q_heads, head_dim, num_splits);
  float* partials = workspace
                        ? reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) +
                                                   w.partials_off)
                        : nullptr;
  rc = decode_front(q, dtype, kv_cache, block_table, block_table_stride, seq_lens, centroids_k,
                    n_centroids_k, centroids_v, n_centroids_v, rotation, num_seqs, num_q_heads,
                    num_kv_heads, head_dim, block_size, num_blocks, sm_scale, num_splits,
                    partials, workspace, workspace_bytes, w.total, stream);
  if (rc != FQ_OK) return rc;
  return head_dim == 128
             ? merge_rotate<128>(partials, 1, num_splits, rotation, out, dtype, num_seqs,
                                 num_q_heads, stream)
             : merge_rotate<64>(partials, 1, num_splits, rotation, out, dtype, num_seqs,
                                num_q_heads, stream);
}

extern "C" int fq_paged_decode_partials(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                                        const int32_t* block_table, int64_t block_table_stride,
                                        const int32_t* seq_lens, const float* centroids_k,
                                        int n_centroids_k, const float* centroids_v,
                                        int n_centroids_v, const float* rotation, int num_seqs,
                                        int num_q_heads, int num_kv_heads, int head_dim,
                                        int block_size, int64_t num_blocks, float sm_scale,
                                        int num_splits, float* partials, void* workspace,
                                        size_t workspace_bytes, fq_stream_t stream) {
  int rc = validate_decode(q, dtype, kv_cache, block_table, seq_lens, centroids_k, n_centroids_k,
                           centroids_v, n_centroids_v, rotation, num_seqs, num_q_heads,
                           num_kv_heads, head_dim, block_size, num_blocks, num_splits);
  if (rc != FQ_OK) return rc;
  FQ_REQUIRE(num_splits >= 1, FQ_ERR_INVALID_ARGUMENT,
             "fq_paged_decode_partials: num_splits must be given (>= 1)");
  FQ_REQUIRE(partials && aligned(partials, 16), FQ_ERR_ALIGNMENT,
             "fq_paged_decode_partials: partials must be 16-byte aligned");
  if (num_seqs == 0) return FQ_OK;
  // only the status word and q_rot live in the workspace here
  const WorkspaceLayout w = workspace_layout(num_seqs, num_q_heads, head_dim, 0);
  return decode_front(q, dtype, kv_cache, block_table, block_table_stride, seq_lens, centroids_k,
                      n_centroids_k, centroids_v, n_centroids_v, rotation, num_seqs, num_q_heads,
                      num_kv_heads, head_dim, block_size, num_blocks, sm_scale, num_splits,
                      partials, workspace, workspace_bytes, w.partials_off, stream);
}

extern "C" int fq_paged_decode_partials_rotated(
    const void* q_rot_f16, const uint8_t* kv_cache, const int32_t* block_table,
    int64_t block_table_stride, const int32_t* seq_lens, const float* centroids_k,
    int n_centroids_k, const float* centroids_v, int n_centroids_v, int num_seqs, int num_q_heads,
    int num_kv_heads, int head_dim, int block_size, int64_t num_blocks, float sm_scale,
    int num_splits, float* partials, void* workspace, size_t workspace_bytes,
    fq_stream_t stream) {
  static const float kDummy = 0.f;  // validate_decode wants a non-null rotation
  int rc = validate_decode(q_rot_f16, FQ_F16, kv_cache, block_table, seq_lens, centroids_k,
                           n_centroids_k, centroids_v, n_centroids_v, &kDummy, num_seqs,
                           num_q_heads, num_kv_heads, head_dim, block_size, num_blocks,
                           num_splits);
  if (rc != FQ_OK) return rc;
  FQ_REQUIRE(num_splits >= 1, FQ_ERR_INVALID_ARGUMENT, "num_splits must be given (>= 1)");
  FQ_REQUIRE(partials && aligned(partials, 16), FQ_ERR_ALIGNMENT,
             "partials must be 16-byte aligned");
  if (num_seqs == 0) return FQ_OK;
  return decode_front(q_rot_f16, FQ_F16, kv_cache, block_table, block_table_stride, seq_lens,
                      centroids_k, n_centroids_k, centroids_v, n_centroids_v, nullptr, num_seqs,
                      num_q_heads, num_kv_heads, head_dim, block_size, num_blocks, sm_scale,
                      num_splits, partials, workspace, workspace_bytes, 256, stream);
}

extern "C" int fq_split_k_merge(const float* partials, int n_groups, int n_splits,
                                const float* rotation, int num_seqs, int num_q_heads,
                                int head_dim, void* out, fq_dtype dtype, fq_stream_t stream) {
  FQ_REQUIRE(partials && rotation && out, FQ_ERR_INVALID_ARGUMENT, "fq_split_k_merge: null pointer");
  FQ_REQUIRE(n_groups >= 1 && n_splits >= 1 && num_seqs >= 0 && num_q_heads >= 1,
             FQ_ERR_INVALID_ARGUMENT, "fq_split_k_merge: bad size");
  FQ_REQUIRE(dtype == FQ_F16 || dtype == FQ_BF16, FQ_ERR_UNSUPPORTED,
             "fq_split_k_merge: out must be fp16 or bf16");
  FQ_REQUIRE(head_dim == 128 || head_dim == 64, FQ_ERR_UNSUPPORTED,
             "fq_split_k_merge: head_dim %d (built for 64 and 128)", head_dim);
  if (num_seqs == 0) return FQ_OK;
  return head_dim == 128 ? merge_rotate<128>(partials, n_groups, n_splits, rotation, out, dtype,
                                             num_seqs, num_q_heads, stream)
                         : merge_rotate<64>(partials, n_groups, n_splits, rotation, out, dtype,
                                            num_seqs, num_q_heads, stream);
}

extern "C" int fq_workspace_status(const void* workspace, uint32_t* status, fq_stream_t stream) {
  FQ_REQUIRE(workspace && status, FQ_ERR_INVALID_ARGUMENT, "fq_workspace_status: null pointer");
  cudaError_t e = cudaMemcpyAsync(status, workspace, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "fq_workspace_status: %s", cudaGetErrorString(e));
  return FQ_OK;
}
