// Streaming phase of the split-K paged decode, specialised for the layout the cache has in
// practice: head_dim 128, 8 KV heads, pages of 16 tokens (a token row is 1088 bytes, a page
// 17 408).  Included by paged_decode.cu after the generic kernel, whose set-up, query rotation
// and merge phases it shares.
//
// What differs from the generic streaming loop:
//   * A page lands in shared memory as eight copies of two token rows each, 2224 bytes apart.
//     With the cache's own pitch of 1088 bytes (272 words = 16 mod 32) the rows a warp reads
//     together - eight rows for the norms, four for the value codes - fall on the same banks
//     and every such load takes four passes.  Inside a pair the 16-word shift is what the
//     key loads want (two rows x 64 bytes cover all banks); between pairs a shift of 12 words
//     spreads the eight norm rows and the four value rows over distinct banks.  Shared-memory
//     passes, not instruction issue, bound the tile loop.  (One copy per row would do the
//     same but costs the producer twice the issue time.)
//   * Every stride is a compile-time constant, loads take 32-bit shared addresses with
//     immediate offsets, a full page takes a path without length masks, and the running
//     maximum is a large negative number instead of -inf, so no select guards the exponent.
//   * Two producer warps per team (even / odd pages; eight lanes copy two rows each) block on
//     the stage barriers instead of polling; page descriptors (valid tokens, segment flags,
//     partial row, physical page) are produced 32 at a time, one lane per page.
//   * The tile loop is software-pipelined by one page: the raw codes of the next tile travel
//     from shared memory to registers under the softmax and value product of this one.
//   * The eight columns of the 16x8 products are (token, head) pairs: with 4 query heads per
//     KV head a step of two tokens per sequence reads every page once.
#pragma once

namespace fq {

constexpr int kFD = 128;                       // head_dim
constexpr int kFH = 8;                         // KV heads
constexpr int kFBS = 16;                       // tokens per page
constexpr int kFRowG = kFH * (kFD + 8);        // 1088: token row in the cache
constexpr int kFPair = 2 * kFRowG + 48;        // 2224: pitch of a pair of rows in shared memory
constexpr int kFStage = kFBS / 2 * kFPair;     // 17 792: a page in shared memory
constexpr int kFDescRing = 128;                // page descriptors per team (16 bytes each)
// shared-memory offset of token row r of a page: pairs (2k, 2k+1) keep the cache's pitch
__host__ __device__ constexpr int fast_row(int r) { return (r >> 1) * kFPair + (r & 1) * kFRowG; }
constexpr int kFTeams = kCW / kFH;             // 2
constexpr float kNegBig = -1.0e30f;            // "no score yet": finite, so m - m is 0, not NaN

template <int IMM>
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(a), "n"(IMM));
  return v;
}
template <int IMM>
__device__ __forceinline__ float ldsf(uint32_t a) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(a), "n"(IMM));
  return v;
}
template <int IMM>
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(a), "n"(IMM));
  return v;
}
template <int IMM>
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(a), "n"(IMM));
  return v;
}
// The same barrier / copy wrappers as in fq_common.cuh on 32-bit shared addresses (no pointer
// conversion, one register per address).
__device__ __forceinline__ bool mbar_try_wait_s(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_warp_s(uint32_t bar, uint32_t parity, uint64_t limit_ns) {
  if (__all_sync(0xffffffffu, mbar_try_wait_s(bar, parity))) return true;
  const uint64_t t0 = global_timer_ns();
#pragma unroll 1
  while (true) {
    const bool ok = mbar_try_wait_s(bar, parity);
    const bool late = global_timer_ns() - t0 > limit_ns;
    if (__all_sync(0xffffffffu, ok)) return true;
    if (__any_sync(0xffffffffu, late)) return false;
  }
}
__device__ __forceinline__ void mbar_arrive_s(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_s(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_g2s_s(uint32_t dst, const void* src, uint32_t bytes,
                                           uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_g2s_hint_s(uint32_t dst, const void* src, uint32_t bytes,
                                                uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1], %2, [%3], %4;" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void sts128(uint32_t a, int x, int y, int z, int w) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(a), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}
__device__ __forceinline__ float2 unpack_half2(uint32_t h) {
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

// Per-warp state of the streaming loop that lives in registers across pages.
struct FastWarp {
  uint32_t lut;     // shared address of the look-up table (K copy at +0, V copy at +128)
  uint32_t laneK;   // row(g) + head*64 + 16t: the lane's 16 key-code bytes of row g
  uint32_t laneN;   // row(g) + 512 + 4*head: key norm of row g (value norm 544 further)
  uint32_t laneV;   // row(2t) + 544 + head*64 + 8g: value codes of token 2t, bytes 8g..8g+7
  uint32_t lane4;   // 4 * lane: the lane's copy inside a table entry
  uint32_t tab[4];  // 8-entry key table for byte permutes: low bytes (2 words), high bytes
};

// The part of a tile's raw data that is fetched one page ahead: the key codes of rows g and
// g+8, bytes 16t..16t+15 of the head.  (The value codes and the norms are loaded when the tile
// starts - the key product that comes first hides their latency - so that only eight
// registers are live across the loop edge.)
struct FastRaw {
  uint4 ka, kb;
};

__device__ __forceinline__ void fast_load(const FastWarp& w, uint32_t rows, FastRaw& r) {
  constexpr int HI = fast_row(8);  // rows g+8, tokens 2t+8: four pairs further
  const uint32_t kaddr = rows + w.laneK;
  r.ka = lds128<0>(kaddr);
  r.kb = lds128<HI>(kaddr);
}

// What the first half of a tile hands to the second.
struct FastMid {
  float sacc[2][4];                              // S^T in two partial sums
  uint32_t ev01[2], od01[2], ev23[2], od23[2];   // value codes paired into table indices
  float nk_lo, nk_hi, nv_lo, nv_hi;
};

// First half of a tile: S^T = K q^T (rows = 16 tokens, columns = (token, head) pairs of the
// group) and the pairing of the value codes.  After it every register of `r` has been used,
// so the stage can be given back and `r` refilled for the next tile.
template <bool KPRMT>
__device__ __forceinline__ void fast_front(const FastWarp& w, const FastRaw& r, uint32_t rows,
                                           const uint32_t (&qf)[8][2], FastMid& m) {
  constexpr int HI = fast_row(8);
  // value codes of tokens 2t, 2t+1, 2t+8, 2t+9, bytes 8g..8g+7 of the head, and the norms of
  // rows g and g+8: on their way while the key product runs
  const uint32_t naddr = rows + w.laneN, vaddr = rows + w.laneV;
  const uint2 x0 = lds64<0>(vaddr), x1 = lds64<kFRowG>(vaddr);
  const uint2 x2 = lds64<HI>(vaddr), x3 = lds64<HI + kFRowG>(vaddr);
  m.nk_lo = ldsf<0>(naddr);
  m.nk_hi = ldsf<HI>(naddr);
  m.nv_lo = ldsf<544>(naddr);
  m.nv_hi = ldsf<544 + HI>(naddr);
  const uint32_t ka[4] = {r.ka.x, r.ka.y, r.ka.z, r.ka.w};
  const uint32_t kb[4] = {r.kb.x, r.kb.y, r.kb.z, r.kb.w};
#pragma unroll
  for (int c = 0; c < 4; ++c) m.sacc[0][c] = m.sacc[1][c] = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // word i of the lane's chunk = cache bytes 4i..4i+3 = k-steps 2i (bytes 0,1) and 2i+1
    uint32_t a[2][4];
    if (KPRMT && !(i & 1)) {
#pragma unroll
      for (int hw = 0; hw < 2; ++hw) {
        const uint32_t sa = hw ? (ka[i] >> 16) : ka[i], sb = hw ? (kb[i] >> 16) : kb[i];
        const uint32_t la = prmt(w.tab[0], w.tab[1], sa), ha = prmt(w.tab[2], w.tab[3], sa);
        const uint32_t lb = prmt(w.tab[0], w.tab[1], sb), hb = prmt(w.tab[2], w.tab[3], sb);
        a[hw][0] = prmt(la, ha, 0x5140);  // row g, first byte: (odd, even) coordinate
        a[hw][1] = prmt(lb, hb, 0x5140);  // row g+8
        a[hw][2] = prmt(la, ha, 0x7362);  // row g, second byte
        a[hw][3] = prmt(lb, hb, 0x7362);
      }
    } else {
      a[0][0] = lds32<0>(w.lut + prmt(ka[i], w.lane4, 0x5504));
      a[0][1] = lds32<0>(w.lut + prmt(kb[i], w.lane4, 0x5504));
      a[0][2] = lds32<0>(w.lut + prmt(ka[i], w.lane4, 0x5514));
      a[0][3] = lds32<0>(w.lut + prmt(kb[i], w.lane4, 0x5514));
      a[1][0] = lds32<0>(w.lut + prmt(ka[i], w.lane4, 0x5524));
      a[1][1] = lds32<0>(w.lut + prmt(kb[i], w.lane4, 0x5524));
      a[1][2] = lds32<0>(w.lut + prmt(ka[i], w.lane4, 0x5534));
      a[1][3] = lds32<0>(w.lut + prmt(kb[i], w.lane4, 0x5534));
    }
    mma_f16(m.sacc[0], a[0][0], a[0][1], a[0][2], a[0][3], qf[2 * i][0], qf[2 * i][1]);
    mma_f16(m.sacc[1], a[1][0], a[1][1], a[1][2], a[1][3], qf[2 * i + 1][0], qf[2 * i + 1][1]);
  }
  // even coordinates sit in the high nibbles, odd ones in the low nibbles; equal nibbles of
  // two tokens are paired into one table index
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t c0 = h ? x0.y : x0.x, c1 = h ? x1.y : x1.x;
    const uint32_t c2 = h ? x2.y : x2.x, c3 = h ? x3.y : x3.x;
    m.ev01[h] = ((c0 >> 4) & 0x0f0f0f0fu) | (c1 & 0xf0f0f0f0u);
    m.od01[h] = (c0 & 0x0f0f0f0fu) | ((c1 << 4) & 0xf0f0f0f0u);
    m.ev23[h] = ((c2 >> 4) & 0x0f0f0f0fu) | (c3 & 0xf0f0f0f0u);
    m.od23[h] = (c2 & 0x0f0f0f0fu) | ((c3 << 4) & 0xf0f0f0f0u);
  }
}

// Second half of a tile: online softmax in the accumulator layout, then O^T += V^T P^T.
// `lim0/lim1`: tokens of the tile that columns 2t / 2t+1 may see (MASKED only).
template <bool MASKED, bool PSPLIT>
__device__ __forceinline__ void fast_back(const FastWarp& w, const FastMid& m, int g,
                                          bool second_term, int lim0, int lim1,
                                          float scale_log2, float (&oacc)[8][4],
                                          float (&m_run)[2], float (&l_run)[2]) {
  // log2 of the value norm is folded into the exponent so that the fp16 weights stay in range
  // whatever the norms are (clamped below so that l cannot overflow)
  const float lv_lo = fmaxf(fast_log2(m.nv_lo), -40.f), lv_hi = fmaxf(fast_log2(m.nv_hi), -40.f);
  const float ks_lo = m.nk_lo * scale_log2, ks_hi = m.nk_hi * scale_log2;
  float s_lo[2], s_hi[2], mx[2];
  [[maybe_unused]] bool ok_lo[2], ok_hi[2];
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    s_lo[c] = (m.sacc[0][c] + m.sacc[1][c]) * ks_lo;
    s_hi[c] = (m.sacc[0][2 + c] + m.sacc[1][2 + c]) * ks_hi;
    if constexpr (MASKED) {
      const int lim = c ? lim1 : lim0;
      ok_lo[c] = g < lim;
      ok_hi[c] = g + 8 < lim;
      mx[c] = fmaxf(ok_lo[c] ? s_lo[c] + lv_lo : kNegBig, ok_hi[c] ? s_hi[c] + lv_hi : kNegBig);
    } else {
      mx[c] = fmaxf(s_lo[c] + lv_lo, s_hi[c] + lv_hi);
    }
  }
  // The reference exponent m only has to stay within kMaxSlack bits of the true running
  // maximum (the weights then stay below 2^(kMaxSlack + kPScaleLog2) <= 2^14 in fp16), so the
  // reduction over the 16 tokens and the rescaling run only when some score outgrows it
  const bool grew = fmaxf(mx[0] - m_run[0], mx[1] - m_run[1]) > kMaxSlack;
  if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], o));
      mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], o));
    }
    const float n0 = fmaxf(m_run[0], mx[0]), n1 = fmaxf(m_run[1], mx[1]);
    const float a0 = fast_exp2(m_run[0] - n0), a1 = fast_exp2(m_run[1] - n1);
    l_run[0] *= a0;
    l_run[1] *= a1;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      oacc[j][0] *= a0; oacc[j][2] *= a0;
      oacc[j][1] *= a1; oacc[j][3] *= a1;
    }
    m_run[0] = n0;
    m_run[1] = n1;
  }
  // the weight that meets the value codes carries the value norm and the fp16 scale
  constexpr float kPScale = float(1 << int(kPScaleLog2));
  const float vs_lo = m.nv_lo * kPScale, vs_hi = m.nv_hi * kPScale;
  float w_lo[2], w_hi[2];
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    float p_lo = fast_exp2(s_lo[c] - m_run[c]);
    float p_hi = fast_exp2(s_hi[c] - m_run[c]);
    w_lo[c] = p_lo * vs_lo;
    w_hi[c] = p_hi * vs_hi;
    if constexpr (MASKED) {
      // rows past the end of the sequence hold whatever the page held: neither their scores
      // nor their norms may reach the sums
      if (!ok_lo[c]) p_lo = w_lo[c] = 0.f;
      if (!ok_hi[c]) p_hi = w_hi[c] = 0.f;
    }
    l_run[c] += p_lo + p_hi;
  }
  // weights as the B operand of the PV product: transpose (token, column) -> (column, token)
  uint32_t h_lo = pack_half2(w_lo[0], w_lo[1]), h_hi = pack_half2(w_hi[0], w_hi[1]);
  if constexpr (PSPLIT) {
    // Two fp16 terms per weight at no extra product: with at most four (token, head) columns
    // in use, columns 4-7 carry the same queries as columns 0-3, so lanes t >= 2 hold the
    // same scores and weights as lanes t - 2; they hand the product what the rounding to fp16
    // dropped, and their accumulators are added to the others' when the segment ends.
    const float2 f_lo = unpack_half2(h_lo), f_hi = unpack_half2(h_hi);
    const uint32_t r_lo = pack_half2(w_lo[0] - f_lo.x, w_lo[1] - f_lo.y);
    const uint32_t r_hi = pack_half2(w_hi[0] - f_hi.x, w_hi[1] - f_hi.y);
    if (second_term) {
      h_lo = r_lo;
      h_hi = r_hi;
    }
  }
  const uint32_t pb0 = movmatrix_trans(h_lo), pb1 = movmatrix_trans(h_hi);
  // ---------- O^T += V^T P^T: rows = value coordinates, columns as above -----------------------
  const uint32_t lutv = w.lut + 128;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
#define FQ_FAST_PV(I, SEL)                                                  \
  {                                                                         \
    const uint32_t a0 = lds32<0>(lutv + prmt(m.ev01[h], w.lane4, SEL));     \
    const uint32_t a1 = lds32<0>(lutv + prmt(m.od01[h], w.lane4, SEL));     \
    const uint32_t a2 = lds32<0>(lutv + prmt(m.ev23[h], w.lane4, SEL));     \
    const uint32_t a3 = lds32<0>(lutv + prmt(m.od23[h], w.lane4, SEL));     \
    mma_f16(oacc[4 * h + I], a0, a1, a2, a3, pb0, pb1);                     \
  }
    FQ_FAST_PV(0, 0x5504)
    FQ_FAST_PV(1, 0x5514)
    FQ_FAST_PV(2, 0x5524)
    FQ_FAST_PV(3, 0x5534)
#undef FQ_FAST_PV
  }
}

// Where (sequence, page) of flat page f is: the last sequence whose first page is <= f.
__device__ __forceinline__ int seq_of_page(const int* prefix, int num_seqs, int64_t f) {
  int lo = 0, hi = num_seqs - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (prefix[mid] <= f) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// FUSE: 0 = streaming phase only; 1 / 2 = single-launch form for bf16 / fp16 q and out

template <bool KPRMT, int FUSE, bool PSPLIT>
__global__ void __launch_bounds__(kDecodeThreads, 1) paged_decode_fast_kernel(DecodeArgs p) {
  using TQ = typename std::conditional<FUSE == 2, __half, __nv_bfloat16>::type;
  constexpr int D = kFD;
  constexpr int ROWF = D + kPartPad;
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x;
  // the warp index through a shuffle: the compiler then knows that it - and every address,
  // counter and flag derived from it - is the same in all lanes and keeps those in uniform
  // registers, which the tile loop needs for its accumulators
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int n_q = p.n_q;
  const int hq_real = p.hq / n_q;
  const int group = hq_real / kFH;   // query heads per KV head
  const int ncols = group * n_q;     // (token, head) columns in use (<= 8)
  const uint32_t q_bytes = uint32_t(p.hq) * D * 2;
  const int team = warp / kFH;       // compute warps: 0 / 1
  const int head = warp - team * kFH;
  const int stages = p.stages;

  int* prefix = reinterpret_cast<int*>(smem + p.off_prefix);
  int* rank = prefix + (p.num_seqs + 1);  // rank[s]: sequences before s that own pages
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_bar);
  const uint32_t sbase = smem_u32(smem);

  const int q_tiles = ((p.hq + 15) / 16) * (D / 8);  // rotated tiles per sequence
  [[maybe_unused]] RotTileOperands<D> rot_op;
  [[maybe_unused]] int rot_len = 0;
  [[maybe_unused]] const int rot_jobs = p.num_seqs * q_tiles;
  [[maybe_unused]] const int rot_job0 = blockIdx.x * kCW + warp;
  [[maybe_unused]] const int m_tiles = (p.hq + 15) / 16;

  // ---- set-up: barriers, page prefix (warp 0), centroids (warp 1) ------------------------------
  if (tid < kFTeams) {
    uint64_t* b = bars + tid * (2 * stages + 2);
    for (int s = 0; s < stages; ++s) {
      mbar_init(b + s, 1);                 // full: the producer's arrive + the bytes
      mbar_init(b + stages + s, kFH);      // empty: one arrive per compute warp
    }
    mbar_init(b + 2 * stages, 1);          // query there
    mbar_init(b + 2 * stages + 1, kFH);    // query consumed
    if (FUSE && tid == 0) mbar_init(bars + kFTeams * (2 * stages + 2), 1);
    mbar_fence_init();
  }
  const unsigned short* cs = reinterpret_cast<const unsigned short*>(smem + p.off_cent);
  float cent_val = 0.f;
  if (warp == 1) {
    const int i = lane & 15;
    if (lane < 16) { if (i < p.nck) cent_val = p.cent_k[i]; } else { if (i < p.ncv) cent_val = p.cent_v[i]; }
  }
  if constexpr (FUSE != 0) {
    if (warp < kCW && rot_job0 < rot_jobs) {
      const int seq = rot_job0 / q_tiles, r = rot_job0 - seq * q_tiles;
      rot_len = p.seq_lens[seq];
      rotate_q_tile_load<D, TQ>(rot_op, static_cast<const TQ*>(p.q_src), p.rotation, p.hq, seq,
                                r % m_tiles, r / m_tiles, lane);
    }
    if (tid == 64) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.block_table));
    if (tid == 65) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.q_count));
    if (tid == 66) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.q_rot_w));
  }
  if (warp == 1)
    stage_centroids(smem + p.off_cent, cent_val, p.nck, p.ncv,
                    p.status + kScaleCacheOffset / 4, lane);
  if (warp == 0) {
    build_page_prefix(p.seq_lens, p.num_seqs, kFBS, p.max_pages,
                      blockIdx.x == 0 ? p.status : nullptr, prefix, lane);
    int carry = 0;
    for (int base = 0; base < p.num_seqs; base += 32) {
      const int i = base + lane;
      const unsigned owns = __ballot_sync(0xffffffffu, i < p.num_seqs && prefix[i + 1] > prefix[i]);
      if (i < p.num_seqs) rank[i] = carry + __popc(owns & ((1u << lane) - 1u));
      carry += __popc(owns);
    }
  }
  __syncthreads();

  // ---- tables, by the compute warps, while the operands of their rotation tiles and the
  // first pages (producer warps, further down) are on their way ------------------------------------
  if (warp < kCW) {
    // scaled fp16 centroid tables (see scale_centroid_tables), then the look-up table: entry e (a
    // cache byte) holds, once per lane, the fp16 pair of its two codes
    scale_centroid_tables(smem + p.off_cent, p.nck, p.ncv, tid,
                          blockIdx.x == 0 ? p.status + kScaleCacheOffset / 4 : nullptr);
    for (int i = tid; i < 256 * 32; i += kComputeThreads) {
      const int e = i >> 5, l = i & 31;
      const uint32_t hi = e >> 4, lo = e & 15;
      // K entry: byte of one token -> (even coordinate, odd coordinate); the byte-permute path
      // delivers (odd, even), so with it the table does too
      // V entry: (code of token 2t+1) << 4 | (code of token 2t) -> (token 2t, token 2t+1)
      *reinterpret_cast<uint32_t*>(smem + e * kLutStride + l * 4) =
          KPRMT ? uint32_t(cs[lo]) | (uint32_t(cs[hi]) << 16)
                : uint32_t(cs[hi]) | (uint32_t(cs[lo]) << 16);
      *reinterpret_cast<uint32_t*>(smem + e * kLutStride + 128 + l * 4) =
          uint32_t(cs[16 + lo]) | (uint32_t(cs[16 + hi]) << 16);
    }
    compute_sync();  // the table is complete
  }

  // ---- phase a: one rotated query tile per warp of the grid --------------------------------------
  if constexpr (FUSE != 0) {
    if (warp < kCW)
      for (int job = rot_job0; job < rot_jobs; job += gridDim.x * kCW) {
        const int seq = job / q_tiles, r = job - seq * q_tiles;
        if (job != rot_job0) {
          rot_len = p.seq_lens[seq];
          rotate_q_tile_load<D, TQ>(rot_op, static_cast<const TQ*>(p.q_src), p.rotation, p.hq,
                                    seq, r % m_tiles, r / m_tiles, lane);
        }
        if (rot_len <= 0) continue;  // nobody reads the query of an empty sequence
        rotate_q_tile_finish<D, TQ>(rot_op, p.q_rot_w, p.hq, seq, r % m_tiles, r / m_tiles, lane);
        __syncwarp();
        if (lane == 0) red_release_add(p.q_count + seq, 1u);
      }
  }

  // ---- the flat page list and its cut into runs -----------------------------------------------------
  const int64_t total = prefix[p.num_seqs];
  const int64_t workers = int64_t(gridDim.x) * kFTeams;
  const int64_t active = total < workers ? total : workers;

  // ---------------------------------------------------------------------------------------------
  // Producer warps.  Issuing a page costs a warp about a thousand cycles of barrier and copy
  // instructions one after the other, so every team has two: warp kCW + T takes the even pages
  // of the team's run, warp kCW + 2 + T the odd ones.  The even warp also describes the pages,
  // 32 at a time with one lane per page (sequence, valid tokens, segment flags, partial-row
  // slot, physical page, which query to load), into a ring of descriptors that the compute
  // warps read, and issues every query copy, in order.  Per page: wait for the stage, arm its
  // barrier, eight lanes copy two token rows each.
  // ---------------------------------------------------------------------------------------------
  if (warp >= kCW) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
    const int T = (warp - kCW) & 1;
    const bool describer = warp < kCW + kFTeams;
    const int64_t wk = int64_t(blockIdx.x) * kFTeams + T;
    if (wk >= active) return;
    const int f0 = int(total * wk / active);
    const int n_run = int(total * (wk + 1) / active) - f0;
    // barriers and buffers as 32-bit shared addresses: the warp lives on 24 registers
    const uint32_t full = sbase + p.off_bar + uint32_t(T) * (2 * stages + 2) * 8;
    const uint32_t empty = full + stages * 8, qfull = empty + stages * 8, qempty = qfull + 8;
    const uint32_t ring = sbase + p.off_ring + uint32_t(T) * stages * kFStage;
    const uint32_t desc = sbase + p.off_desc + uint32_t(T) * kFDescRing * 16;
    const uint64_t stream_policy = l2_evict_first_policy();  // pages are read once
    int q_issued = 0;
    int stage = describer ? 0 : 1 % stages;  // stage of run page i = i % stages ...
    uint32_t parity = (describer || stages > 1) ? 1u : 0u;  // ... used for the (i / stages)-th time
    int32_t entry = 0;   // physical page of run page (chunk base + own stride * lane)
    bool bad = false;
    const int first_seq = seq_of_page(prefix, p.num_seqs, f0);
#pragma unroll 1
    for (int i = describer ? 0 : 1; i < n_run; i += 2) {
      if (describer) {
        if ((i & 31) == 0) {
          // ---- run pages i .. i+31: x = valid tokens | flags << 8 | query number << 12,
          // y = sequence, z = partial-row slot, w = physical page ---------------------------------
          const int r = i + lane;
          int4 dsc = make_int4(0, 0, 0, 0);
          if (r < n_run) {
            const int f = f0 + r;
            const int seq = seq_of_page(prefix, p.num_seqs, f);
            const int pg = f - prefix[seq], n_pages = prefix[seq + 1] - prefix[seq];
            const int pps = (n_pages + p.num_splits - 1) / p.num_splits;
            const int sp = pg / pps;
            const int split_end = min((sp + 1) * pps, n_pages);
            const bool q_new = r == 0 || pg == 0;
            const bool seg_first = r == 0 || pg == sp * pps;
            const bool seg_last = pg + 1 == split_end || r + 1 == n_run;
            // tokens from this page on, capped (not at 16: a step of several tokens masks up to
            // n_q - 1 tokens before the end, which may reach into the page before the last)
            const int left = min(p.seq_lens[seq] - pg * kFBS, 127);
            // the n-th query this run loads: sequences that own pages, counted from the first
            const int qn = rank[seq] - rank[first_seq];
            int phys = p.block_table[int64_t(seq) * p.bt_stride + pg];
            if (phys < 0 || phys >= p.num_blocks) {
              phys = 0;
              bad = true;
            }
            const int flags =
                (seg_first ? kSegStart : 0) | (seg_last ? kSegEnd : 0) | (q_new ? kQNew : 0);
            dsc = make_int4(left | (flags << 8) | (qn << 12), seq,
                            seq * p.num_splits + sp + int(wk), phys);
          }
          sts128(desc + uint32_t(r & (kFDescRing - 1)) * 16, dsc.x, dsc.y, dsc.z, dsc.w);
          __syncwarp();
        }
      } else if (((i - 1) & 63) == 0) {
        // physical pages of this warp's next 32 pages (run pages i, i+2, ...), one per lane
        const int r = i + 2 * lane;
        entry = 0;
        if (r < n_run) {
          const int f = f0 + r;
          const int seq = seq_of_page(prefix, p.num_seqs, f);
          entry = p.block_table[int64_t(seq) * p.bt_stride + (f - prefix[seq])];
          if (entry < 0 || entry >= p.num_blocks) {
            entry = 0;
            bad = true;
          }
        }
      }
      int phys;
      uint4 d0 = make_uint4(0u, 0u, 0u, 0u);
      if (describer) {
        d0 = lds128<0>(desc + uint32_t(i & (kFDescRing - 1)) * 16);
        phys = int(d0.w);
      } else {
        phys = __shfl_sync(0xffffffffu, entry, ((i - 1) >> 1) & 31);
      }
      if (i >= stages && !mbar_wait_warp_s(empty + stage * 8, parity, p.wait_ns)) {
        if (lane == 0) atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
        break;
      }
      const uint32_t st = ring + uint32_t(stage) * kFStage;
      if (lane == 0) mbar_expect_tx_s(full + stage * 8, kFBS * kFRowG);
      __syncwarp();
      if (lane < kFBS / 2)
        bulk_g2s_hint_s(st + lane * kFPair,
                        p.kv_cache + int64_t(phys) * (kFBS * kFRowG) + lane * (2 * kFRowG),
                        2 * kFRowG, full + stage * 8, stream_policy);
      if (describer) {
        // queries of this page and of the other warp's next page, in run order.  The buffer is
        // single: the team must have taken the previous query into registers, and (single
        // launch) the rotated rows of this one must be stored
        bool ok = true;
#pragma unroll 1
        for (int k = 0; k < 2 && ok; ++k) {
          const uint4 dq = k == 0 ? d0
                                  : (i + 1 < n_run ? lds128<0>(desc + uint32_t((i + 1) & (kFDescRing - 1)) * 16)
                                                   : make_uint4(0u, 0u, 0u, 0u));
          if (!((dq.x >> 8) & kQNew)) continue;
          const int seq = int(dq.y);
          ok = q_issued == 0 || mbar_wait_warp_s(qempty, (q_issued - 1) & 1, p.wait_ns);
          if constexpr (FUSE != 0) {
            if (ok) {
              ok = counter_wait_warp(p.q_count + seq, uint32_t(q_tiles), p.wait_ns, lane);
              fence_proxy_async();  // lane 0 acquired the rows and issues the copy
            }
          }
          if (!ok) break;
          if (lane == 0) {
            mbar_expect_tx_s(qfull, q_bytes);
            bulk_g2s_s(sbase + p.off_q + uint32_t(T) * q_bytes,
                       p.q_rot + int64_t(seq) * p.hq * D, q_bytes, qfull);
          }
          ++q_issued;
        }
        if (!ok) {
          if (lane == 0) atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
          break;
        }
      }
      stage += 2;
      while (stage >= stages) { stage -= stages; parity ^= 1u; }
    }
    if (__any_sync(0xffffffffu, bad) && lane == 0) atomicOr(p.status, FQ_DEV_BAD_BLOCK_INDEX);
    return;
  }
  asm volatile("setmaxnreg.inc.sync.aligned.u32 112;");

  // ---- compute warps ----------------------------------------------------------------------------
  const int64_t wk = int64_t(blockIdx.x) * kFTeams + team;
  const int n_run = wk < active ? int(total * (wk + 1) / active - total * wk / active) : 0;

  const float beta_k = reinterpret_cast<const float*>(smem + p.off_cent + 192)[0];
  const float beta_v = reinterpret_cast<const float*>(smem + p.off_cent + 192)[1];
  const float k_scale_log2 = p.scale_log2 * beta_k;  // the key table is c / beta_k

  if (n_run > 0) {  // ---- phase b ----------------------------------------------------------------
    FastWarp w;
    w.lut = sbase;
    w.laneK = uint32_t(fast_row(g)) + head * 64 + 16 * t;
    w.laneN = uint32_t(fast_row(g)) + 512 + 4 * head;
    w.laneV = uint32_t(fast_row(2 * t)) + 544 + head * 64 + 8 * g;
    w.lane4 = uint32_t(lane) * 4;
    w.tab[0] = w.tab[1] = w.tab[2] = w.tab[3] = 0u;
    if constexpr (KPRMT) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t h = cs[i];
        const uint32_t lo8 = (h & 0xffu) << (8 * (i & 3)), hi8 = (h >> 8) << (8 * (i & 3));
        if (i < 4) { w.tab[0] |= lo8; w.tab[2] |= hi8; } else { w.tab[1] |= lo8; w.tab[3] |= hi8; }
      }
    }
    const uint32_t full = sbase + p.off_bar + uint32_t(team) * (2 * stages + 2) * 8;
    const uint32_t empty = full + stages * 8, qfull = empty + stages * 8, qempty = qfull + 8;
    const uint32_t ring = sbase + p.off_ring + uint32_t(team) * stages * kFStage;
    const uint32_t desc = sbase + p.off_desc + uint32_t(team) * kFDescRing * 16;
    const uint32_t qbuf = p.off_q + uint32_t(team) * q_bytes;
    // column g of the B operand is (token g / group, head g % group); the partial row of
    // column c belongs to query row col_row(c)
    // (with two-term weights columns 4-7 repeat columns 0-3: see fast_back)
    const int my_col = PSPLIT ? (g & 3) : g;
    const int my_tok = my_col / group, my_head = my_col - my_tok * group;
    const bool col_ok = my_col < ncols;
    const uint32_t q_lane =
        qbuf + uint32_t(col_ok ? my_tok * hq_real + head * group + my_head : 0) * D * 2 + (D / 8) * t * 4;
    // tokens that this lane's two accumulator columns (2t, 2t+1) cannot see at the end of a
    // sequence: query token i of n_q sees keys up to L - n_q + i
    const int col0 = PSPLIT ? (2 * t) & 3 : 2 * t;  // real column behind accumulator column 2t
    const int back0 = col0 < ncols ? n_q - 1 - col0 / group : 0;
    const int back1 = col0 + 1 < ncols ? n_q - 1 - (col0 + 1) / group : 0;

    float m_run[2] = {kNegBig, kNegBig};
    float l_run[2] = {0.f, 0.f};
    float oacc[8][4];
    uint32_t qf[8][2];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      qf[j][0] = qf[j][1] = 0u;
#pragma unroll
      for (int c = 0; c < 4; ++c) oacc[j][c] = 0.f;
    }
    // The loop is software-pipelined by one page: while the second half of tile `it` (softmax
    // and value product) runs, the raw codes of tile `it + 1` are already on their way from
    // shared memory to registers, and the stage of tile `it` is back with the producer.
    int stage = 0, fphase = 0, qcnt = 0;
    bool timed_out = false;
    FastRaw raw;
    uint4 d = make_uint4(0u, 0u, 0u, 0u);  // descriptor of the page in `raw`
    {
      if (!mbar_wait_warp_s(full, 0, p.wait_ns)) {
        timed_out = true;
      } else {
        d = lds128<0>(desc);
        fast_load(w, ring, raw);
      }
    }
#pragma unroll 1
    for (int it = 0; it < n_run && !timed_out; ++it) {
      const int n_valid = d.x & 0xff, flags = (d.x >> 8) & 0xf;
      const int seg_seq = d.y, seg_slot = d.z;
      if (flags & kSegStart) {
        m_run[0] = m_run[1] = kNegBig;
        l_run[0] = l_run[1] = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
          for (int c = 0; c < 4; ++c) oacc[j][c] = 0.f;
        if (flags & kQNew) {
          if (!mbar_wait_warp_s(qfull, qcnt & 1, p.wait_ns)) {
            timed_out = true;
            break;
          }
          // lane (g,t), k-step s: coordinates of cache bytes 16t + 2s, +1 of the column's row
#pragma unroll
          for (int s = 0; s < 8; ++s) {
            uint2 v = *reinterpret_cast<const uint2*>(smem + q_lane + 8 * s);
            if constexpr (KPRMT) {  // the byte-permute path delivers (odd, even) pairs
              v.x = prmt(v.x, v.x, 0x1032);
              v.y = prmt(v.y, v.y, 0x1032);
            }
            qf[s][0] = col_ok ? v.x : 0u;
            qf[s][1] = col_ok ? v.y : 0u;
          }
          // The loads above must have delivered before the buffer is handed back: nothing else
          // orders a shared-memory load that is still in flight before the arrive, and the
          // producer's next copy may land on the buffer as soon as the eighth warp has arrived.
          __threadfence_block();
          __syncwarp();
          if (lane == 0) mbar_arrive_s(qempty);
          ++qcnt;
        }
      }
      FastMid mid;
      fast_front<KPRMT>(w, raw, ring + uint32_t(stage) * kFStage, qf, mid);
      // every load from the stage has been issued above; the fence makes them deliver before
      // the stage goes back to the producers (costs nothing measurable: they are long done)
      __threadfence_block();
      __syncwarp();
      if (lane == 0) mbar_arrive_s(empty + stage * 8);
      if (++stage == stages) { stage = 0; fphase ^= 1; }
      // the next page: its descriptor and raw codes travel under the second half of this tile
      if (it + 1 < n_run) {
        if (!mbar_wait_warp_s(full + stage * 8, fphase, p.wait_ns)) {
          timed_out = true;  // this tile is still finished below
        } else {
          d = lds128<0>(desc + uint32_t((it + 1) & (kFDescRing - 1)) * 16);
          fast_load(w, ring + uint32_t(stage) * kFStage, raw);
        }
      }
      // one path for the whole warp (both hold warp-wide operations): the unmasked one only if
      // even the first query token of the step sees all 16 tokens of the page
      const int lim0 = n_valid - back0, lim1 = n_valid - back1;
      if (n_valid - (n_q - 1) >= kFBS)
        fast_back<false, PSPLIT>(w, mid, g, t >= 2, 16, 16, k_scale_log2, oacc, m_run, l_run);
      else
        fast_back<true, PSPLIT>(w, mid, g, t >= 2, lim0, lim1, k_scale_log2, oacc, m_run, l_run);
      if (flags & kSegEnd) {
        // ---- this warp's partial rows of the segment --------------------------------------------
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], o);
          l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], o);
        }
        const float unscale = beta_v / float(1 << int(kPScaleLog2));  // the value table is c / beta_v
        if constexpr (PSPLIT) {  // second-term accumulators of lanes t+2 join those of lanes t
#pragma unroll
          for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) oacc[j][c] += __shfl_xor_sync(0xffffffffu, oacc[j][c], 2);
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col = 2 * t + c;
          if (col >= ncols || (PSPLIT && t >= 2)) continue;
          const int ct = col / group;
          float* row = p.slots + (int64_t(seg_slot) * p.hq + ct * hq_real + head * group + (col - ct * group)) * ROWF;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int b = 8 * g + j;  // cache byte -> coordinates 2b (row g), 2b+1 (row g+8)
            *reinterpret_cast<float2*>(row + 2 * b) =
                make_float2(oacc[j][c] * unscale, oacc[j][2 + c] * unscale);
          }
          if (g == 0)
            *reinterpret_cast<float4*>(row + D) =
                make_float4(l_run[c] > 0.f ? m_run[c] : -INFINITY, l_run[c], 0.f, 0.f);
        }
        if constexpr (FUSE != 0) {
          __syncwarp();
          if (lane == 0) red_release_add(p.seg_count + seg_seq, 1u);
        }
      }
    }

    if (timed_out && lane == 0) atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
  }  // phase b

  if constexpr (FUSE != 0) {
    fused_merge<D, TQ>(p, smem, prefix, total, active, kFTeams, stages);
  }
}

}  // namespace fq
