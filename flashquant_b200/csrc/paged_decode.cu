// Split-K paged decode over the packed TQ4 cache for sm_100a.
//
// Three launches per call:
//   1. rotate_q_kernel      q_rot = round_to_q_dtype(q Pi^T), stored as fp16
//   2. paged_decode_kernel  persistent, one CTA per SM: the pages of all sequences form one
//                           flat list that is cut into equal runs, one per CTA; a run is
//                           processed as segments that never cross a boundary of the
//                           caller's split partition, and every segment leaves one
//                           (acc, m, l) partial row per query head
//   3. merge_rotate_kernel  merges the partial rows of a sequence, rounds to the output type,
//                           multiplies by Pi
//
// The streaming kernel is bound by HBM traffic (136 B per token and KV head) only if the
// per-byte instruction count stays near 3: a nibble code costs two table look-ups and, with
// 4 query heads per KV head, eight multiply-adds per byte, which the fp32 pipe cannot
// sustain at 7 TB/s.  So the multiply-adds go to the tensor pipe (mma.sync m16n8k16, the N
// dimension being the query heads of the group) and a byte is turned into two fp16
// centroids by ONE shared-memory look-up in a 256-entry table of fp16 pairs, replicated per
// lane so that look-ups never conflict.  Operand fragments are built directly in registers
// in the order the look-ups deliver them; the k-dimension of the QK product and the row
// dimension of the PV product are permuted accordingly (the query fragment and the
// write-back apply the same permutation).
//
// Pages reach shared memory by 1-D bulk copies issued by a producer warp into a ring of
// stages guarded by full/empty mbarriers; every wait is bounded and reports through the
// status word instead of spinning forever.
#include "fq_common.cuh"

namespace fq {

constexpr int kCW = 16;                         // compute warps per CTA
constexpr int kDecodeThreads = (kCW + 1) * 32;  // + one producer warp
constexpr int kComputeThreads = kCW * 32;
constexpr int kLutBytes = 256 * 32 * 4;         // one table, one copy per lane
constexpr int kMaxStages = 24;
constexpr int kMaxSeqs = 2048;                  // page-count prefix lives in shared memory
constexpr int kMaxSplits = 64;
constexpr int kPartPad = 4;                     // partial row = D + 4 floats (acc, m, l, 0, 0)
constexpr float kPScaleLog2 = 14.f;             // fp16 weights are scaled by 2^14

enum : int { kSegStart = 1, kSegEnd = 2, kQNew = 4, kLast = 8 };

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
  float* slots;  // (num_seqs * S + gridDim.x, Hq, D+4)
  uint32_t* status;
  uint32_t off_ring, off_mbuf, off_q, off_prefix, off_desc, off_bar;
};

struct PageDesc {  // 32 bytes, written by the producer, read by every compute warp
  int seq, tok0, seq_len, flags, slot, qslot, pad0, pad1;
};

// ------------------------------------------------------------------------------------
// page-count prefix of the batch, built by one warp into shared memory
// ------------------------------------------------------------------------------------
__device__ __forceinline__ void build_page_prefix(const int32_t* __restrict__ seq_lens, int n,
                                                  int block_size, int* prefix, int lane) {
  int carry = 0;
  if (lane == 0) prefix[0] = 0;
  for (int base = 0; base < n; base += 32) {
    const int i = base + lane;
    int len = i < n ? seq_lens[i] : 0;
    if (len < 0) len = 0;
    int v = (len + block_size - 1) / block_size;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += up;
    }
    v += carry;
    if (i < n) prefix[i + 1] = v;
    carry = __shfl_sync(0xffffffffu, v, 31);
  }
  __syncwarp();
}

// CTA that owns flat page f when `total` pages are cut into `active` equal runs
// (run c starts at floor(total * c / active)).
__host__ __device__ __forceinline__ int cta_of_page(int64_t f, int64_t total, int64_t active) {
  return int(((f + 1) * active + total - 1) / total - 1);
}

// ------------------------------------------------------------------------------------
// 1. q rotation: out[r][j] = fp16(round_T(sum_k q[r][k] * Pi[j][k]))
// ------------------------------------------------------------------------------------
template <int D, typename T>
__global__ void __launch_bounds__(256) rotate_q_kernel(const T* __restrict__ q,
                                                      const float* __restrict__ rotation,
                                                      __half* __restrict__ out, int n_rows) {
  constexpr int ROWS = 8;
  constexpr int LD = D + 1;  // padded: thread j walks row j, rows land in different banks
  extern __shared__ __align__(16) float rq_smem[];
  float* pi = rq_smem;           // [j][k], row stride LD
  float* qs = rq_smem + D * LD;  // [ROWS][D]
  const int tid = threadIdx.x;
  // coalesced 16-byte loads, all issued before the first use
  constexpr int V4 = D * D / 4 / 256;
  float4 tmp[V4];
#pragma unroll
  for (int i = 0; i < V4; ++i) tmp[i] = reinterpret_cast<const float4*>(rotation)[tid + i * 256];
  const int row0 = blockIdx.x * ROWS;
  for (int i = tid; i < ROWS * D; i += 256) {
    const int r = row0 + i / D;
    qs[i] = r < n_rows ? to_f32(q[int64_t(r) * D + i % D]) : 0.f;
  }
#pragma unroll
  for (int i = 0; i < V4; ++i) {
    const int e = (tid + i * 256) * 4;
    const int j = e / D, k = e % D;
    float* dst = pi + j * LD + k;
    dst[0] = tmp[i].x; dst[1] = tmp[i].y; dst[2] = tmp[i].z; dst[3] = tmp[i].w;
  }
  __syncthreads();
  constexpr int GROUPS = 256 / D;     // thread groups, each covers all D outputs
  constexpr int RPG = ROWS / GROUPS;  // rows per group
  const int j = tid % D, grp = tid / D;
  float acc[RPG];
#pragma unroll
  for (int r = 0; r < RPG; ++r) acc[r] = 0.f;
  const float* prow = pi + j * LD;
#pragma unroll 8
  for (int k4 = 0; k4 < D; k4 += 4) {
    const float b0 = prow[k4], b1 = prow[k4 + 1], b2 = prow[k4 + 2], b3 = prow[k4 + 3];
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
__device__ __forceinline__ void compute_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kComputeThreads) : "memory");
}

template <int D>
__global__ void __launch_bounds__(kDecodeThreads, 1) paged_decode_kernel(DecodeArgs p) {
  constexpr int KS = D / 16;  // k-steps of the QK product = m-tiles of the PV product
  constexpr int KW = D / 32;  // 32-bit words of K codes per lane and row
  constexpr int VB = D / 16;  // bytes of V codes per lane and row
  constexpr int ROWF = D + kPartPad;

  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t half_d = D / 2;
  const uint32_t row_bytes = uint32_t(p.hkv) * (D + 8);
  const uint32_t page_bytes = uint32_t(p.block_size) * row_bytes;
  int* prefix = reinterpret_cast<int*>(smem + p.off_prefix);
  PageDesc* descs = reinterpret_cast<PageDesc*>(smem + p.off_desc);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + p.off_bar);
  uint64_t* empty_bar = full_bar + p.stages;
  uint64_t* qfull_bar = empty_bar + p.stages;
  uint64_t* qempty_bar = qfull_bar + 2;
  float* mbuf = reinterpret_cast<float*>(smem + p.off_mbuf);

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int group = p.hq / p.hkv;  // q heads per KV head (<= 8)
  const uint32_t q_bytes = uint32_t(p.hq) * D * 2;

  // ---- set-up: barriers, page prefix (producer warp), look-up tables (compute warps) ---
  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, kCW);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(qfull_bar + s, 1);
      mbar_init(qempty_bar + s, kCW);
    }
    mbar_fence_init();
  }
  if (warp == kCW) {
    build_page_prefix(p.seq_lens, p.num_seqs, p.block_size, prefix, lane);
  } else {
    for (int i = tid; i < 256 * 32; i += kComputeThreads) {
      const int e = i >> 5;
      const int hi = e >> 4, lo = e & 15;
      const float kh = hi < p.nck ? p.cent_k[hi] : 0.f, kl = lo < p.nck ? p.cent_k[lo] : 0.f;
      const float vh = hi < p.ncv ? p.cent_v[hi] : 0.f, vl = lo < p.ncv ? p.cent_v[lo] : 0.f;
      reinterpret_cast<uint32_t*>(smem)[i] = pack_half2(kh, kl);  // low half: even coordinate
      reinterpret_cast<uint32_t*>(smem + kLutBytes)[i] = pack_half2(vh, vl);
    }
  }
  __syncthreads();

  // ---- this CTA's run of the flat page list -------------------------------------------------
  const int64_t total = prefix[p.num_seqs];
  const int64_t active = total < int64_t(gridDim.x) ? total : int64_t(gridDim.x);
  const int cta = blockIdx.x;
  if (cta >= active) return;
  const int64_t f0 = total * cta / active, f1 = total * (cta + 1) / active;
  if (f0 >= f1) return;

  if (warp == kCW) {
    // ================= producer (lane 0 waits and issues, the warp fetches table entries) ==
    int lo = 0, hi = p.num_seqs - 1;  // the sequence that holds flat page f0
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (prefix[mid] <= f0) lo = mid; else hi = mid - 1;
    }
    int seq = lo;
    int stage = 0, ephase = 1, it = 0, cur_q_seq = -1, qn = 0;
    int64_t f = f0;
    bool dead = false;
    while (f < f1 && !dead) {
      const int p0 = prefix[seq];
      const int n_pages = prefix[seq + 1] - p0;
      int pg = int(f - p0);
      const int pps = (n_pages + p.num_splits - 1) / p.num_splits;
      const int s = pg / pps;
      int seg_pages_end = (s + 1) * pps;
      if (seg_pages_end > n_pages) seg_pages_end = n_pages;
      int64_t seg_end = int64_t(p0) + seg_pages_end;
      if (seg_end > f1) seg_end = f1;
      const int slot = seq * p.num_splits + s + cta;
      const int seq_len = p.seq_lens[seq];
      const bool qnew = seq != cur_q_seq;
      int qslot = (qn - 1) & 1;
      if (qnew) {
        qslot = qn & 1;
        int ok = 1;
        if (lane == 0) {
          if (qn >= 2 && !mbar_wait(qempty_bar + qslot, ((qn >> 1) & 1) ^ 1)) {
            atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
            ok = 0;
          } else {
            mbar_expect_tx(qfull_bar + qslot, q_bytes);
            bulk_g2s(smem + p.off_q + qslot * q_bytes, p.q_rot + int64_t(seq) * p.hq * D,
                     q_bytes, qfull_bar + qslot);
          }
        }
        if (!__shfl_sync(0xffffffffu, ok, 0)) break;
        cur_q_seq = seq;
        ++qn;
      }
      bool first = true;
      while (f < seg_end && !dead) {
        const int chunk = int(seg_end - f < 32 ? seg_end - f : 32);
        int my_phys = 0;
        if (lane < chunk) my_phys = p.block_table[int64_t(seq) * p.bt_stride + pg + lane];
        for (int k = 0; k < chunk; ++k, ++f, ++pg) {
          int64_t phys = __shfl_sync(0xffffffffu, my_phys, k);
          int ok = 1;
          if (lane == 0) {
            if (it >= p.stages && !mbar_wait(empty_bar + stage, ephase)) {
              atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
              ok = 0;
            } else {
              if (phys < 0 || phys >= p.num_blocks) {
                atomicOr(p.status, FQ_DEV_BAD_BLOCK_INDEX);
                phys = 0;
              }
              PageDesc d;
              d.seq = seq; d.tok0 = pg * p.block_size; d.seq_len = seq_len;
              d.flags = (first ? kSegStart : 0) | ((first && qnew) ? kQNew : 0) |
                        (f + 1 == seg_end ? kSegEnd : 0) | (f + 1 == f1 ? kLast : 0);
              d.slot = slot; d.qslot = qslot; d.pad0 = 0; d.pad1 = 0;
              descs[stage] = d;
              mbar_expect_tx(full_bar + stage, page_bytes);
              bulk_g2s(smem + p.off_ring + uint32_t(stage) * page_bytes,
                       p.kv_cache + phys * int64_t(page_bytes), page_bytes, full_bar + stage);
            }
          }
          if (!__shfl_sync(0xffffffffu, ok, 0)) {
            dead = true;
            break;
          }
          if (++stage == p.stages) { stage = 0; ephase ^= 1; }
          ++it;
          first = false;
        }
      }
      if (f == prefix[seq + 1]) {
        ++seq;
        while (seq < p.num_seqs - 1 && prefix[seq + 1] == prefix[seq]) ++seq;
      }
    }
    return;
  }

  // ================= consumers =================
  const int wph = kCW / p.hkv;  // warps per KV head (power of two)
  const int head = warp & (p.hkv - 1);
  const int sub = warp / p.hkv;
  const uint32_t lane4 = uint32_t(lane) * 4;
  const bool wide = (p.hkv & 1) == 0;  // 16-byte row alignment needs an even head count
  const uint32_t k_code_off = head * half_d;
  const uint32_t k_norm_off = p.hkv * half_d + 4 * head;
  const uint32_t v_code_off = p.hkv * half_d + 4 * p.hkv + head * half_d;
  const uint32_t v_norm_off = 2 * p.hkv * half_d + 4 * p.hkv + 4 * head;
  const int units_per_page = p.block_size >> 4;

  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  float oacc[KS][4];
  uint32_t qf[KS][2];
#pragma unroll
  for (int j = 0; j < KS; ++j) {
    qf[j][0] = qf[j][1] = 0u;
#pragma unroll
    for (int c = 0; c < 4; ++c) oacc[j][c] = 0.f;
  }

  int stage = 0, fphase = 0, qcnt = 0, unit_ctr = 0;
  bool timed_out = false;
  while (true) {
    if (!mbar_wait(full_bar + stage, fphase)) {
      timed_out = true;
      break;
    }
    const int4 d0 = *reinterpret_cast<const int4*>(descs + stage);
    const int2 d1 = *reinterpret_cast<const int2*>(reinterpret_cast<const int*>(descs + stage) + 4);
    const int tok_page0 = d0.y, seq_len = d0.z, flags = d0.w;

    if (flags & kSegStart) {
      m_run[0] = m_run[1] = -INFINITY;
      l_run[0] = l_run[1] = 0.f;
#pragma unroll
      for (int j = 0; j < KS; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) oacc[j][c] = 0.f;
      if (flags & kQNew) {
        const int qslot = d1.y;
        if (!mbar_wait(qfull_bar + qslot, (qcnt >> 1) & 1)) {
          timed_out = true;
          break;
        }
        // lane (g,t), k-step s: coordinates of cache bytes (D/8)t + 2s, +1 of q head head*G+g
        const bool valid = g < group;
        const uint32_t qoff = p.off_q + qslot * q_bytes +
                              uint32_t(head * group + (valid ? g : 0)) * D * 2 + (D / 8) * t * 4;
#pragma unroll
        for (int s = 0; s < KS; ++s) {
          const uint2 v = *reinterpret_cast<const uint2*>(smem + qoff + 8 * s);
          qf[s][0] = valid ? v.x : 0u;
          qf[s][1] = valid ? v.y : 0u;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(qempty_bar + qslot);
        ++qcnt;
      }
    }

    const uint32_t page_off = p.off_ring + uint32_t(stage) * page_bytes;
    for (int u = 0; u < units_per_page; ++u, ++unit_ctr) {
      if ((unit_ctr & (wph - 1)) != sub) continue;
      const int tok0 = tok_page0 + u * 16;
      if (tok0 >= seq_len) continue;
      const uint32_t rows = page_off + uint32_t(u) * 16 * row_bytes;
      const uint32_t r_lo = rows + uint32_t(g) * row_bytes;
      const uint32_t r_hi = r_lo + 8 * row_bytes;

      // ---------- S^T = K q^T : rows = 16 tokens, cols = q heads of the group ------------
      uint32_t ka[KW], kb[KW];
      if constexpr (KW == 4) {
        if (wide) {
          const uint4 a = *reinterpret_cast<const uint4*>(smem + r_lo + k_code_off + 16 * t);
          const uint4 b = *reinterpret_cast<const uint4*>(smem + r_hi + k_code_off + 16 * t);
          ka[0] = a.x; ka[1] = a.y; ka[2] = a.z; ka[3] = a.w;
          kb[0] = b.x; kb[1] = b.y; kb[2] = b.z; kb[3] = b.w;
        } else {  // odd number of KV heads: rows are only 8-byte aligned
          const uint2* pa = reinterpret_cast<const uint2*>(smem + r_lo + k_code_off + 16 * t);
          const uint2* pb = reinterpret_cast<const uint2*>(smem + r_hi + k_code_off + 16 * t);
          const uint2 a0 = pa[0], a1 = pa[1], b0 = pb[0], b1 = pb[1];
          ka[0] = a0.x; ka[1] = a0.y; ka[2] = a1.x; ka[3] = a1.y;
          kb[0] = b0.x; kb[1] = b0.y; kb[2] = b1.x; kb[3] = b1.y;
        }
      } else {
        const uint2 a = *reinterpret_cast<const uint2*>(smem + r_lo + k_code_off + 8 * t);
        const uint2 b = *reinterpret_cast<const uint2*>(smem + r_hi + k_code_off + 8 * t);
        ka[0] = a.x; ka[1] = a.y;
        kb[0] = b.x; kb[1] = b.y;
      }
      // value codes: lane (g,t) needs tokens 2t, 2t+1, 2t+8, 2t+9, cache bytes VB*g .. +VB-1
      uint32_t vw[4][(VB + 3) / 4];
      {
        const uint32_t vbase = rows + v_code_off + VB * g + uint32_t(2 * t) * row_bytes;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const uint32_t src = vbase + uint32_t((r & 1) + (r >> 1) * 8) * row_bytes;
          if constexpr (VB == 8) {
            if (wide) {
              const uint2 x = *reinterpret_cast<const uint2*>(smem + src);
              vw[r][0] = x.x; vw[r][1] = x.y;
            } else {  // the V region starts at an odd multiple of 4 bytes
              vw[r][0] = *reinterpret_cast<const uint32_t*>(smem + src);
              vw[r][1] = *reinterpret_cast<const uint32_t*>(smem + src + 4);
            }
          } else {
            vw[r][0] = *reinterpret_cast<const uint32_t*>(smem + src);
          }
        }
      }
      const float nk_lo = *reinterpret_cast<const float*>(smem + r_lo + k_norm_off);
      const float nk_hi = *reinterpret_cast<const float*>(smem + r_hi + k_norm_off);
      const float nv_lo = *reinterpret_cast<const float*>(smem + r_lo + v_norm_off);
      const float nv_hi = *reinterpret_cast<const float*>(smem + r_hi + v_norm_off);

      float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        const int w = s >> 1;
        const uint32_t wa = ka[w], wb = kb[w];
        uint32_t i0, i1, i2, i3;
        if ((s & 1) == 0) {
          i0 = ((wa << 7) & 0x7f80u) | lane4;
          i1 = ((wb << 7) & 0x7f80u) | lane4;
          i2 = ((wa >> 1) & 0x7f80u) | lane4;
          i3 = ((wb >> 1) & 0x7f80u) | lane4;
        } else {
          i0 = ((wa >> 9) & 0x7f80u) | lane4;
          i1 = ((wb >> 9) & 0x7f80u) | lane4;
          i2 = ((wa >> 17) & 0x7f80u) | lane4;
          i3 = ((wb >> 17) & 0x7f80u) | lane4;
        }
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(smem + i0);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(smem + i1);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(smem + i2);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(smem + i3);
        mma_f16(sacc[s & 1], a0, a1, a2, a3, qf[s][0], qf[s][1]);  // two accumulator chains
      }

      // ---------- online softmax in the accumulator layout ---------------------------------
      const bool ok_lo = tok0 + g < seq_len, ok_hi = tok0 + g + 8 < seq_len;
      // log2 of the value norm is folded into the exponent so that the fp16 weights stay in
      // range whatever the norms are; the running reference clamps it below so that l
      // cannot overflow
      const float lg_lo = fast_log2(nv_lo), lg_hi = fast_log2(nv_hi);
      const float lv_lo = fmaxf(lg_lo, -40.f), lv_hi = fmaxf(lg_hi, -40.f);
      const float ks_lo = nk_lo * p.scale_log2, ks_hi = nk_hi * p.scale_log2;
      float s_lo[2], s_hi[2], mx[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        s_lo[c] = (sacc[0][c] + sacc[1][c]) * ks_lo;
        s_hi[c] = (sacc[0][2 + c] + sacc[1][2 + c]) * ks_hi;
        mx[c] = fmaxf(ok_lo ? s_lo[c] + lv_lo : -INFINITY, ok_hi ? s_hi[c] + lv_hi : -INFINITY);
      }
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], o));
        mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], o));
      }
      const bool grew = (mx[0] > m_run[0]) || (mx[1] > m_run[1]);
      if (__any_sync(0xffffffffu, grew)) {
        const float n0 = fmaxf(m_run[0], mx[0]), n1 = fmaxf(m_run[1], mx[1]);
        const float a0 = (m_run[0] == -INFINITY) ? 0.f : fast_exp2(m_run[0] - n0);
        const float a1 = (m_run[1] == -INFINITY) ? 0.f : fast_exp2(m_run[1] - n1);
        l_run[0] *= a0;
        l_run[1] *= a1;
#pragma unroll
        for (int j = 0; j < KS; ++j) {
          oacc[j][0] *= a0; oacc[j][2] *= a0;
          oacc[j][1] *= a1; oacc[j][3] *= a1;
        }
        m_run[0] = n0;
        m_run[1] = n1;
      }
      float w_lo[2], w_hi[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const float mref = (m_run[c] == -INFINITY) ? 0.f : m_run[c];
        // lg2(0) = -inf makes the weight of a zero-norm value exactly 0
        w_lo[c] = ok_lo ? fast_exp2(s_lo[c] + lg_lo - mref + kPScaleLog2) : 0.f;
        w_hi[c] = ok_hi ? fast_exp2(s_hi[c] + lg_hi - mref + kPScaleLog2) : 0.f;
        const float p_lo = ok_lo ? fast_exp2(s_lo[c] - mref) : 0.f;
        const float p_hi = ok_hi ? fast_exp2(s_hi[c] - mref) : 0.f;
        l_run[c] += p_lo + p_hi;
      }
      // weights as the B operand of the PV product: transpose (token, head) -> (head, token)
      const uint32_t pb0 = movmatrix_trans(pack_half2(w_lo[0], w_lo[1]));
      const uint32_t pb1 = movmatrix_trans(pack_half2(w_hi[0], w_hi[1]));

      // ---------- O^T += V^T P^T : rows = value coordinates, cols = q heads ------------------
#pragma unroll
      for (int j = 0; j < KS; ++j) {
        const int w = j >> 2;
        uint32_t i0, i1, i2, i3;
        if ((j & 3) == 0) {
          i0 = ((vw[0][w] << 7) & 0x7f80u) | lane4;
          i1 = ((vw[1][w] << 7) & 0x7f80u) | lane4;
          i2 = ((vw[2][w] << 7) & 0x7f80u) | lane4;
          i3 = ((vw[3][w] << 7) & 0x7f80u) | lane4;
        } else {
          const int sh = 8 * (j & 3) - 7;
          i0 = ((vw[0][w] >> sh) & 0x7f80u) | lane4;
          i1 = ((vw[1][w] >> sh) & 0x7f80u) | lane4;
          i2 = ((vw[2][w] >> sh) & 0x7f80u) | lane4;
          i3 = ((vw[3][w] >> sh) & 0x7f80u) | lane4;
        }
        const uint32_t l0 = *reinterpret_cast<const uint32_t*>(smem + kLutBytes + i0);
        const uint32_t l1 = *reinterpret_cast<const uint32_t*>(smem + kLutBytes + i1);
        const uint32_t l2 = *reinterpret_cast<const uint32_t*>(smem + kLutBytes + i2);
        const uint32_t l3 = *reinterpret_cast<const uint32_t*>(smem + kLutBytes + i3);
        const uint32_t a0 = prmt(l0, l1, 0x5410);  // even coordinate, tokens 2t, 2t+1
        const uint32_t a1 = prmt(l0, l1, 0x7632);  // odd coordinate
        const uint32_t a2 = prmt(l2, l3, 0x5410);  // even coordinate, tokens 2t+8, 2t+9
        const uint32_t a3 = prmt(l2, l3, 0x7632);
        mma_f16(oacc[j], a0, a1, a2, a3, pb0, pb1);
      }
    }

    if (flags & kSegEnd) {
      // ---- fold the warps that shared a KV head, then write this segment's partial rows --
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], o);
        l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], o);
      }
      const bool c_ok[2] = {2 * t < group, 2 * t + 1 < group};
      float* rowp[2] = {mbuf + (head * group + (c_ok[0] ? 2 * t : 0)) * ROWF,
                        mbuf + (head * group + (c_ok[1] ? 2 * t + 1 : 0)) * ROWF};
      for (int r = 0; r < wph; ++r) {
        if (sub == r) {
          float a_old[2] = {0.f, 0.f}, a_me[2] = {1.f, 1.f}, m_n[2], l_n[2];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            m_n[c] = m_run[c];
            l_n[c] = l_run[c];
            if (r > 0) {
              const float m_o = rowp[c][D], l_o = rowp[c][D + 1];
              m_n[c] = fmaxf(m_o, m_run[c]);
              a_old[c] = (m_o == -INFINITY) ? 0.f : fast_exp2(m_o - m_n[c]);
              a_me[c] = (m_run[c] == -INFINITY) ? 0.f : fast_exp2(m_run[c] - m_n[c]);
              l_n[c] = l_o * a_old[c] + l_run[c] * a_me[c];
            }
          }
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            if (!c_ok[c]) continue;
#pragma unroll
            for (int j = 0; j < KS; ++j) {
              const int b = VB * g + j;  // cache byte -> coordinates 2b (row g), 2b+1 (row g+8)
              float e = oacc[j][c] * a_me[c], o = oacc[j][2 + c] * a_me[c];
              if (r > 0) {
                e = fmaf(rowp[c][2 * b], a_old[c], e);
                o = fmaf(rowp[c][2 * b + 1], a_old[c], o);
              }
              *reinterpret_cast<float2*>(rowp[c] + 2 * b) = make_float2(e, o);
            }
            if (g == 0) *reinterpret_cast<float2*>(rowp[c] + D) = make_float2(m_n[c], l_n[c]);
          }
        }
        compute_barrier();
      }
      {
        float4* dst = reinterpret_cast<float4*>(p.slots + int64_t(d1.x) * p.hq * ROWF);
        const float4* src = reinterpret_cast<const float4*>(mbuf);
        const int n4 = p.hq * (ROWF / 4);
        const float unscale = 1.f / 16384.f;  // 2^-kPScaleLog2
        for (int i = tid; i < n4; i += kComputeThreads) {
          float4 v = src[i];
          if (i % (ROWF / 4) < D / 4) {
            v.x *= unscale; v.y *= unscale; v.z *= unscale; v.w *= unscale;
          } else {
            v.z = 0.f; v.w = 0.f;
          }
          dst[i] = v;
        }
      }
      compute_barrier();
    }

    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar + stage);
    if (flags & kLast) break;
    if (++stage == p.stages) { stage = 0; fphase ^= 1; }
  }
  if (timed_out && lane == 0) atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
}

// ------------------------------------------------------------------------------------
// 3. merge of partial rows + rounding + out = o_rot Pi
//
//    kFromSlots: the rows of sequence `seq` are the segments of the streaming kernel,
//                found again from the page prefix and the run arithmetic;
//    else:       rows come as (n_groups, num_seqs, Hq, D+4), one per group.
//    kFinal:     normalise, round, rotate, store to `out`;
//    else:       store the merged, still un-normalised row (acc, m, l) to `row_out`.
//    grid (ceil(Hq/8), num_seqs), 8*D threads: thread (head hh, coordinate d).
// ------------------------------------------------------------------------------------
struct MergeArgs {
  const float* rows;
  int n_groups;    // !kFromSlots
  int num_splits;  // kFromSlots
  int num_ctas;    // kFromSlots: grid size of the streaming kernel
  const int32_t* seq_lens;
  int block_size;
  const float* rotation;
  void* out;
  float* row_out;
  int num_seqs, hq;
};

constexpr int kMergeHeads = 8;
constexpr int kMaxParts = 256;

template <int D, typename T, bool kFromSlots, bool kFinal>
__global__ void __launch_bounds__(kMergeHeads* D) merge_rotate_kernel(MergeArgs p) {
  constexpr int ROWF = D + kPartPad;
  constexpr int NT = kMergeHeads * D;
  extern __shared__ __align__(16) unsigned char msm[];
  float* pi_s = reinterpret_cast<float*>(msm);                  // [k][j] (kFinal only)
  float* o_s = pi_s + (kFinal ? D * D : 0);                     // [8][D]
  float* w_s = o_s + kMergeHeads * D;                           // [parts][8]: m, then weight
  float* l_s = w_s + kMaxParts * kMergeHeads;                   // [parts][8]
  float* den_s = l_s + kMaxParts * kMergeHeads;                 // [8] den, [8] m*
  int* part_row = reinterpret_cast<int*>(den_s + 2 * kMergeHeads);  // [parts]
  int* prefix = part_row + kMaxParts;                           // [num_seqs + 1]
  __shared__ uint64_t pi_bar;
  __shared__ int n_parts_s;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int seq = blockIdx.y, h0 = blockIdx.x * kMergeHeads;

  if constexpr (kFinal) {
    if (tid == 0) {
      mbar_init(&pi_bar, 1);
      mbar_fence_init();
      mbar_expect_tx(&pi_bar, D * D * 4);
      bulk_g2s(pi_s, p.rotation, D * D * 4, &pi_bar);
    }
  }

  // ---- which rows belong to this sequence ----------------------------------------------
  if constexpr (kFromSlots) {
    if (warp == 0) {
      build_page_prefix(p.seq_lens, p.num_seqs, p.block_size, prefix, lane);
      if (lane == 0) {
        const int64_t total = prefix[p.num_seqs];
        const int64_t active = total < p.num_ctas ? total : int64_t(p.num_ctas);
        const int p0 = prefix[seq], n_pages = prefix[seq + 1] - p0;
        int n = 0;
        if (n_pages > 0) {
          const int pps = (n_pages + p.num_splits - 1) / p.num_splits;
          for (int s = 0; s < p.num_splits; ++s) {
            const int a = s * pps;
            int b = a + pps;
            if (b > n_pages) b = n_pages;
            if (a >= b) break;
            const int c_first = cta_of_page(int64_t(p0) + a, total, active);
            const int c_last = cta_of_page(int64_t(p0) + b - 1, total, active);
            for (int c = c_first; c <= c_last && n < kMaxParts; ++c)
              part_row[n++] = seq * p.num_splits + s + c;
          }
        }
        n_parts_s = n;
      }
    }
  } else {
    if (tid < p.n_groups && tid < kMaxParts) part_row[tid] = tid * p.num_seqs + seq;
    if (tid == 0) n_parts_s = p.n_groups < kMaxParts ? p.n_groups : kMaxParts;
  }
  __syncthreads();
  const int n_parts = n_parts_s;
  // part i, head h: rows + (part_row[i] * Hq + h) * ROWF  (a slot index plays the role of
  // (group, sequence))
  auto row_ptr = [&](int i, int h) { return p.rows + (int64_t(part_row[i]) * p.hq + h) * ROWF; };

  // ---- m and l of every (part, head), then the weights ------------------------------------
  for (int i = tid; i < n_parts * kMergeHeads; i += NT) {
    const int part = i / kMergeHeads, hh = i % kMergeHeads;
    float m = -INFINITY, l = 0.f;
    if (h0 + hh < p.hq) {
      const float2 ml = *reinterpret_cast<const float2*>(row_ptr(part, h0 + hh) + D);
      m = ml.x;
      l = ml.y;
    }
    w_s[i] = m;
    l_s[i] = l;
  }
  __syncthreads();
  if (tid < kMergeHeads) {
    float m_star = -INFINITY;
    for (int i = 0; i < n_parts; ++i) m_star = fmaxf(m_star, w_s[i * kMergeHeads + tid]);
    float den = 0.f;
    for (int i = 0; i < n_parts; ++i) {
      const float m = w_s[i * kMergeHeads + tid];
      const float w = (m == -INFINITY) ? 0.f : exp2f(m - m_star);
      w_s[i * kMergeHeads + tid] = w;
      den = fmaf(w, l_s[i * kMergeHeads + tid], den);
    }
    den_s[tid] = den;
    den_s[kMergeHeads + tid] = m_star;
  }
  __syncthreads();

  // ---- accumulate: thread (hh, d) ---------------------------------------------------------
  const int d = tid % D, hh = tid / D;
  const bool head_ok = h0 + hh < p.hq;
  float num = 0.f;
  if (head_ok) {
    for (int i0 = 0; i0 < n_parts; i0 += 8) {
      float v[8];
#pragma unroll
      for (int x = 0; x < 8; ++x) v[x] = (i0 + x < n_parts) ? row_ptr(i0 + x, h0 + hh)[d] : 0.f;
#pragma unroll
      for (int x = 0; x < 8; ++x)
        if (i0 + x < n_parts) num = fmaf(w_s[(i0 + x) * kMergeHeads + hh], v[x], num);
    }
  }

  if constexpr (!kFinal) {
    if (head_ok) {
      float* dst = p.row_out + (int64_t(seq) * p.hq + h0 + hh) * ROWF;
      dst[d] = num;
      if (d == 0)
        *reinterpret_cast<float4*>(dst + D) =
            make_float4(den_s[kMergeHeads + hh], den_s[hh], 0.f, 0.f);
    }
  } else {
    const float den = den_s[hh];
    const float o = (head_ok && den > 0.f) ? num / den : 0.f;
    o_s[hh * D + d] = to_f32(from_f32<T>(o));  // the reference rounds the rotated output
    __syncthreads();
    if (!mbar_wait(&pi_bar, 0)) return;  // only if the copy were lost; out stays unwritten
    float acc = 0.f;
#pragma unroll 8
    for (int k4 = 0; k4 < D; k4 += 4) {
      const float4 a = *reinterpret_cast<const float4*>(o_s + hh * D + k4);
      acc = fmaf(a.x, pi_s[(k4 + 0) * D + d], acc);
      acc = fmaf(a.y, pi_s[(k4 + 1) * D + d], acc);
      acc = fmaf(a.z, pi_s[(k4 + 2) * D + d], acc);
      acc = fmaf(a.w, pi_s[(k4 + 3) * D + d], acc);
    }
    if (head_ok) static_cast<T*>(p.out)[(int64_t(seq) * p.hq + h0 + hh) * D + d] = from_f32<T>(acc);
  }
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
static int device_sm_count() {
  static thread_local int cached_dev = -1, cached = 148;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev != cached_dev) {
    cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev);
    cached_dev = dev;
  }
  return cached;
}

struct WorkspaceLayout {
  size_t q_rot_off, slots_off, total;
};

static size_t up256(size_t v) { return (v + 255) / 256 * 256; }

// `splits` <= 0 sizes for the largest split count
static WorkspaceLayout workspace_layout(int num_seqs, int hq, int d, int splits, int ctas) {
  if (splits <= 0) splits = kMaxSplits;
  WorkspaceLayout w;
  w.q_rot_off = 256;
  w.slots_off = up256(w.q_rot_off + size_t(num_seqs) * hq * d * sizeof(__half));
  w.total = up256(w.slots_off +
                  (size_t(num_seqs) * splits + ctas) * hq * (d + kPartPad) * sizeof(float));
  return w;
}

// The flat page list is balanced over the SMs whatever the split count is; more splits
// only add partial rows, so one split per sequence is the automatic choice.
static int auto_splits() { return 1; }

struct SmemPlan {
  int stages;
  uint32_t off_ring, off_mbuf, off_q, off_prefix, off_desc, off_bar, total;
};

static SmemPlan plan_smem(int num_seqs, int hq, int hkv, int d, int block_size) {
  SmemPlan s{};
  const uint32_t page_bytes = uint32_t(block_size) * hkv * (d + 8);
  auto up16 = [](uint32_t v) { return (v + 15u) & ~15u; };
  const uint32_t mbuf = up16(uint32_t(hq) * (d + kPartPad) * 4);
  const uint32_t qring = 2 * up16(uint32_t(hq) * d * 2);
  const uint32_t prefix = up16(uint32_t(num_seqs + 1) * 4);
  const uint32_t fixed = 2 * kLutBytes + mbuf + qring + prefix;
  const uint32_t budget = 227 * 1024 - 512;
  int stages = 0;
  if (budget > fixed)
    stages = int((budget - fixed) / (page_bytes + uint32_t(sizeof(PageDesc)) + 16));
  // enough bytes in flight per SM to cover HBM latency, no more
  const int want = int((112 * 1024 + page_bytes - 1) / page_bytes);
  if (stages > want) stages = want;
  if (stages > kMaxStages) stages = kMaxStages;
  s.stages = stages;
  s.off_ring = 2 * kLutBytes;
  s.off_mbuf = s.off_ring + uint32_t(stages < 0 ? 0 : stages) * page_bytes;
  s.off_q = s.off_mbuf + mbuf;
  s.off_prefix = s.off_q + qring;
  s.off_desc = s.off_prefix + prefix;
  s.off_bar = s.off_desc + uint32_t(stages) * uint32_t(sizeof(PageDesc));
  s.total = s.off_bar + (2 * uint32_t(stages) + 4) * 8;
  return s;
}

template <int D>
static int launch_stream(DecodeArgs& a, const SmemPlan& sp, int ctas, cudaStream_t stream) {
  auto kern = paged_decode_kernel<D>;
  // opt in once per (thread, device, size): the attribute call is not free
  static thread_local int set_dev = -1;
  static thread_local size_t set_bytes = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (set_dev != dev || set_bytes < sp.total) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sp.total));
    if (e != cudaSuccess)
      return fail(FQ_ERR_CUDA, "paged decode: shared memory opt-in of %u bytes refused: %s",
                  sp.total, cudaGetErrorString(e));
    set_dev = dev;
    set_bytes = sp.total;
  }
  a.stages = sp.stages;
  a.off_ring = sp.off_ring; a.off_mbuf = sp.off_mbuf; a.off_q = sp.off_q;
  a.off_prefix = sp.off_prefix; a.off_desc = sp.off_desc; a.off_bar = sp.off_bar;
  kern<<<ctas, kDecodeThreads, sp.total, stream>>>(a);
  return check_launch("paged decode kernel launch");
}

template <int D>
static int rotate_q(const void* q, int dtype, const float* rotation, __half* out, int rows,
                    cudaStream_t stream) {
  const size_t smem = (size_t(D) * (D + 1) + 8 * D) * sizeof(float);
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

template <int D, typename T, bool kFromSlots, bool kFinal>
static int launch_merge_t(const MergeArgs& m, cudaStream_t stream) {
  const size_t smem = (kFinal ? size_t(D) * D * 4 : 0) + kMergeHeads * D * 4 +
                      2 * kMaxParts * kMergeHeads * 4 + 2 * kMergeHeads * 4 + kMaxParts * 4 +
                      (kFromSlots ? size_t(m.num_seqs + 1) * 4 : 0) + 16;
  auto kern = merge_rotate_kernel<D, T, kFromSlots, kFinal>;
  static thread_local int set_dev = -1;
  static thread_local size_t set_bytes = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (set_dev != dev || set_bytes < smem) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess)
      return fail(FQ_ERR_CUDA, "merge: shared memory opt-in of %zu bytes refused: %s", smem,
                  cudaGetErrorString(e));
    set_dev = dev;
    set_bytes = smem;
  }
  dim3 grid((m.hq + kMergeHeads - 1) / kMergeHeads, m.num_seqs);
  kern<<<grid, kMergeHeads * D, smem, stream>>>(m);
  return check_launch("merge kernel launch");
}

template <bool kFromSlots, bool kFinal>
static int launch_merge(const MergeArgs& m, int head_dim, int dtype, cudaStream_t stream) {
  if (head_dim == 128)
    return dtype == FQ_BF16 ? launch_merge_t<128, __nv_bfloat16, kFromSlots, kFinal>(m, stream)
                            : launch_merge_t<128, __half, kFromSlots, kFinal>(m, stream);
  return dtype == FQ_BF16 ? launch_merge_t<64, __nv_bfloat16, kFromSlots, kFinal>(m, stream)
                          : launch_merge_t<64, __half, kFromSlots, kFinal>(m, stream);
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
  FQ_REQUIRE(hkv == 1 || hkv == 2 || hkv == 4 || hkv == 8 || hkv == 16, FQ_ERR_UNSUPPORTED,
             "paged decode: num_kv_heads %d (built for 1, 2, 4, 8, 16)", hkv);
  FQ_REQUIRE(hq % hkv == 0 && hq / hkv <= 8, FQ_ERR_UNSUPPORTED,
             "paged decode: %d q heads per KV head (at most 8, and a whole number)", hq / hkv);
  FQ_REQUIRE(block_size >= 16 && block_size % 16 == 0, FQ_ERR_UNSUPPORTED,
             "paged decode: block_size %d is not a multiple of 16", block_size);
  FQ_REQUIRE(num_seqs <= kMaxSeqs, FQ_ERR_UNSUPPORTED,
             "paged decode: %d sequences per call (at most %d)", num_seqs, kMaxSeqs);
  FQ_REQUIRE(num_splits <= kMaxSplits, FQ_ERR_UNSUPPORTED,
             "paged decode: num_splits %d (at most %d)", num_splits, kMaxSplits);
  FQ_REQUIRE(aligned(kv_cache, 16) && aligned(q, 16) && aligned(rotation, 16), FQ_ERR_ALIGNMENT,
             "paged decode: kv_cache, q and rotation must be 16-byte aligned");
  return FQ_OK;
}

// q rotation (unless the caller already rotated) and the streaming kernel
static int decode_front(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                        const int32_t* block_table, int64_t block_table_stride,
                        const int32_t* seq_lens, const float* centroids_k, int nck,
                        const float* centroids_v, int ncv, const float* rotation, int num_seqs,
                        int hq, int hkv, int head_dim, int block_size, int64_t num_blocks,
                        float sm_scale, int num_splits, void* workspace, size_t workspace_bytes,
                        int ctas, cudaStream_t stream) {
  FQ_REQUIRE(workspace && aligned(workspace, 256), FQ_ERR_WORKSPACE,
             "paged decode: workspace is null or not 256-byte aligned");
  const WorkspaceLayout w = workspace_layout(num_seqs, hq, head_dim, num_splits, ctas);
  FQ_REQUIRE(workspace_bytes >= w.total, FQ_ERR_WORKSPACE,
             "paged decode: workspace has %zu bytes, %zu needed", workspace_bytes, w.total);
  const SmemPlan sp = plan_smem(num_seqs, hq, hkv, head_dim, block_size);
  FQ_REQUIRE(sp.stages >= 2, FQ_ERR_UNSUPPORTED,
             "paged decode: a page of %d tokens x %d heads does not fit the shared-memory ring",
             block_size, hkv);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  const __half* q_rot = reinterpret_cast<const __half*>(ws + w.q_rot_off);
  if (rotation) {
    __half* dst = reinterpret_cast<__half*>(ws + w.q_rot_off);
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
  a.slots = reinterpret_cast<float*>(ws + w.slots_off);
  a.status = reinterpret_cast<uint32_t*>(ws);
  return head_dim == 128 ? launch_stream<128>(a, sp, ctas, stream)
                         : launch_stream<64>(a, sp, ctas, stream);
}

static MergeArgs slot_merge_args(void* workspace, int num_seqs, int hq, int head_dim,
                                 int num_splits, int ctas, const int32_t* seq_lens,
                                 int block_size) {
  const WorkspaceLayout w = workspace_layout(num_seqs, hq, head_dim, num_splits, ctas);
  MergeArgs m{};
  m.rows = reinterpret_cast<const float*>(static_cast<unsigned char*>(workspace) + w.slots_off);
  m.num_splits = num_splits;
  m.num_ctas = ctas;
  m.seq_lens = seq_lens;
  m.block_size = block_size;
  m.num_seqs = num_seqs;
  m.hq = hq;
  return m;
}

}  // namespace fq

using namespace fq;

extern "C" size_t fq_paged_decode_workspace_bytes(int num_seqs, int num_q_heads, int head_dim,
                                                  int num_splits) {
  if (num_seqs < 0 || num_q_heads < 0 || head_dim < 0) return 0;
  return workspace_layout(num_seqs, num_q_heads, head_dim, num_splits, 256).total;
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
  const int ctas = device_sm_count();
  if (num_splits == 0) num_splits = auto_splits();
  rc = decode_front(q, dtype, kv_cache, block_table, block_table_stride, seq_lens, centroids_k,
                    n_centroids_k, centroids_v, n_centroids_v, rotation, num_seqs, num_q_heads,
                    num_kv_heads, head_dim, block_size, num_blocks, sm_scale, num_splits,
                    workspace, workspace_bytes, ctas, stream);
  if (rc != FQ_OK) return rc;
  MergeArgs m = slot_merge_args(workspace, num_seqs, num_q_heads, head_dim, num_splits, ctas,
                                seq_lens, block_size);
  m.rotation = rotation;
  m.out = out;
  return launch_merge<true, true>(m, head_dim, dtype, stream);
}

static int partials_common(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                           const int32_t* block_table, int64_t block_table_stride,
                           const int32_t* seq_lens, const float* centroids_k, int n_centroids_k,
                           const float* centroids_v, int n_centroids_v, const float* rotation,
                           int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                           int block_size, int64_t num_blocks, float sm_scale, int num_splits,
                           float* partials, void* workspace, size_t workspace_bytes,
                           cudaStream_t stream) {
  FQ_REQUIRE(partials && aligned(partials, 16), FQ_ERR_ALIGNMENT,
             "partials must be 16-byte aligned");
  if (num_seqs == 0) return FQ_OK;
  const int ctas = device_sm_count();
  if (num_splits == 0) num_splits = auto_splits();
  int rc = decode_front(q, dtype, kv_cache, block_table, block_table_stride, seq_lens,
                        centroids_k, n_centroids_k, centroids_v, n_centroids_v, rotation,
                        num_seqs, num_q_heads, num_kv_heads, head_dim, block_size, num_blocks,
                        sm_scale, num_splits, workspace, workspace_bytes, ctas, stream);
  if (rc != FQ_OK) return rc;
  MergeArgs m = slot_merge_args(workspace, num_seqs, num_q_heads, head_dim, num_splits, ctas,
                                seq_lens, block_size);
  m.row_out = partials;
  return launch_merge<true, false>(m, head_dim, FQ_F16, stream);
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
  return partials_common(q, dtype, kv_cache, block_table, block_table_stride, seq_lens,
                         centroids_k, n_centroids_k, centroids_v, n_centroids_v, rotation,
                         num_seqs, num_q_heads, num_kv_heads, head_dim, block_size, num_blocks,
                         sm_scale, num_splits, partials, workspace, workspace_bytes, stream);
}

extern "C" int fq_paged_decode_partials_rotated(
    const void* q_rot_f16, const uint8_t* kv_cache, const int32_t* block_table,
    int64_t block_table_stride, const int32_t* seq_lens, const float* centroids_k,
    int n_centroids_k, const float* centroids_v, int n_centroids_v, int num_seqs, int num_q_heads,
    int num_kv_heads, int head_dim, int block_size, int64_t num_blocks, float sm_scale,
    int num_splits, float* partials, void* workspace, size_t workspace_bytes,
    fq_stream_t stream) {
  alignas(16) static const float kDummy[4] = {0.f, 0.f, 0.f, 0.f};  // validate wants non-null
  int rc = validate_decode(q_rot_f16, FQ_F16, kv_cache, block_table, seq_lens, centroids_k,
                           n_centroids_k, centroids_v, n_centroids_v, kDummy, num_seqs,
                           num_q_heads, num_kv_heads, head_dim, block_size, num_blocks,
                           num_splits);
  if (rc != FQ_OK) return rc;
  return partials_common(q_rot_f16, FQ_F16, kv_cache, block_table, block_table_stride, seq_lens,
                         centroids_k, n_centroids_k, centroids_v, n_centroids_v, nullptr,
                         num_seqs, num_q_heads, num_kv_heads, head_dim, block_size, num_blocks,
                         sm_scale, num_splits, partials, workspace, workspace_bytes, stream);
}

extern "C" int fq_split_k_merge(const float* partials, int n_groups, const float* rotation,
                                int num_seqs, int num_q_heads, int head_dim, void* out,
                                fq_dtype dtype, fq_stream_t stream) {
  FQ_REQUIRE(partials && rotation && out, FQ_ERR_INVALID_ARGUMENT, "fq_split_k_merge: null pointer");
  FQ_REQUIRE(n_groups >= 1 && n_groups <= kMaxParts && num_seqs >= 0 && num_q_heads >= 1,
             FQ_ERR_INVALID_ARGUMENT, "fq_split_k_merge: bad size");
  FQ_REQUIRE(dtype == FQ_F16 || dtype == FQ_BF16, FQ_ERR_UNSUPPORTED,
             "fq_split_k_merge: out must be fp16 or bf16");
  FQ_REQUIRE(head_dim == 128 || head_dim == 64, FQ_ERR_UNSUPPORTED,
             "fq_split_k_merge: head_dim %d (built for 64 and 128)", head_dim);
  FQ_REQUIRE(aligned(rotation, 16) && aligned(partials, 16), FQ_ERR_ALIGNMENT,
             "fq_split_k_merge: rotation and partials must be 16-byte aligned");
  if (num_seqs == 0) return FQ_OK;
  MergeArgs m{};
  m.rows = partials;
  m.n_groups = n_groups;
  m.rotation = rotation;
  m.out = out;
  m.num_seqs = num_seqs;
  m.hq = num_q_heads;
  return launch_merge<false, true>(m, head_dim, dtype, stream);
}

extern "C" int fq_workspace_status(const void* workspace, uint32_t* status, fq_stream_t stream) {
  FQ_REQUIRE(workspace && status, FQ_ERR_INVALID_ARGUMENT, "fq_workspace_status: null pointer");
  cudaError_t e = cudaMemcpyAsync(status, workspace, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return fail(FQ_ERR_CUDA, "fq_workspace_status: %s", cudaGetErrorString(e));
  return FQ_OK;
}
