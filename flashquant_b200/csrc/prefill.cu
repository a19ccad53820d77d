// Fused causal TQ4 FlashAttention-2 prefill for sm_100a on the 5th-generation tensor cores.
//
// One CTA of 256 threads owns 128 query rows of one (batch, query head) - two threads per
// row, each with half of the columns - and walks the KV sequence in tiles of 64 tokens,
// skipping tiles above the causal diagonal.  Per tile:
//   * the packed K and V codes and their norms arrive by 1-D bulk copies, one tile ahead;
//   * all threads turn codes into fp16 centroids (256-entry table of fp16 pairs) and store
//     them as tcgen05 shared-memory operands; the norms are NOT applied here: |k| scales the
//     score column, |v| is folded into the softmax weight, as in the decode kernel;
//   * one thread issues S = Q K^T (tcgen05.mma, fp16 x fp16 -> fp32 in TMEM) - for the NEXT
//     tile, into the other of two score buffers, so that it runs under this tile's softmax;
//   * the two threads of row r read their halves of row r of S from TMEM (tcgen05.ld), apply
//     |k|, the scale and - on tiles that touch the diagonal or the end - the causal mask,
//     update the online softmax and write the fp16 weights as the A operand of the second
//     product;
//   * one thread issues O += P V into TMEM, where the accumulator stays across all tiles: the
//     reference exponent of the online softmax is raised lazily (only when a row's scores
//     outgrow it by more than 6 bits), and only then do the threads of that warp rescale their
//     rows of O in TMEM (tcgen05.ld / tcgen05.st); the epilogue reads O once.  The product
//     runs under the next tile's key dequantisation.
// Two such CTAs fit an SM (110 KB of shared memory, 256 of the 512 TMEM columns each).
//
// Shared-memory operands use the un-swizzled canonical layout: 8 x 16-byte core matrices,
// laid out [k-chunk of 8 elements][row][16 bytes]; each k-chunk slab is padded by 16 bytes
// so that the cooperative stores do not conflict.
//
// The query arrives already rotated and rounded (fp16 copy of round(q Pi^T)), the output
// leaves in rotated space as fp32 (the reference rounds only after the multiplication by
// Pi); rotate.cu does both rotations.
#include <type_traits>

#include "fq_common.cuh"
#include "centroid_scale.cuh"

namespace fq {

constexpr int kPfM = 128;       // query rows per CTA
constexpr int kPfN = 64;        // KV tokens per tile
constexpr int kPfThreads = 256;  // two threads per query row: each takes half of the columns
constexpr int kPfTmemCols = 256;
constexpr float kPfPScaleLog2 = 8.f;  // fp16 weights are scaled by 2^8 ...
constexpr float kPfMaxSlack = 6.f;    // ... and may exceed 1 by 2^6 before the reference exponent is raised

// ---- tcgen05 wrappers -------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* holder_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(holder_smem)),
               "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem], fp16 inputs, fp32 accumulate; issued by ONE thread
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// all previously issued MMAs of this thread arrive on `bar` when they have completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
// lane l of the warp receives 32 consecutive fp32 columns of TMEM lane (lane_base + l)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  tc_wait_ld();
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// the reverse: lane l stores 32 consecutive fp32 columns of TMEM lane (lane_base + l)
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  uint32_t r[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(v[i]);
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor, no swizzle, descriptor version 1.
// lbo / sbo in bytes (multiples of 16): for a K-major operand lbo is the distance between
// the two 8-element k-chunks of one MMA and sbo the distance between 8-row groups; for an
// MN-major operand sbo is the distance between 8-element groups along M/N and lbo the
// distance between 8-row groups along K.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  return uint64_t((addr >> 4) & 0x3fffu) | (uint64_t((lbo >> 4) & 0x3fffu) << 16) |
         (uint64_t((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}
// Instruction descriptor: fp16 A and B, fp32 D, A K-major, B K-major or MN-major.
__host__ __device__ constexpr uint32_t umma_idesc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (b_mn_major ? (1u << 16) : 0u) | (uint32_t(n >> 3) << 17) |
         (uint32_t(m >> 4) << 24);
}

struct PrefillArgs {
  const __half* q_rot;      // (B, Hq, Nq, D) fp16, rotated and rounded
  const uint8_t* k_packed;  // (B, Hkv, Nkv, D/2)
  const float* k_norms;     // (B, Hkv, Nkv)
  const uint8_t* v_packed;
  const float* v_norms;
  const float* cent_k;
  int nck;
  const float* cent_v;
  int ncv;
  float* o_rot;  // (B, Hq, Nq, D) fp32, rotated space (the reference rounds only after Pi)
  int batch, hq, hkv, nq, nkv;
  int64_t kv_stride;  // tokens between consecutive (batch, head) rows of the K/V buffers (>= nkv)
  float scale_log2;
  int causal;
  uint32_t* status;
  // Split mode (n_splits > 1, one query tile, no mask): blockIdx.x is a slice of split_tokens
  // (a multiple of the key tile) keys and values; the CTA stores an un-normalised partial row
  // [o * 2^0 (D) | m | l | - | -] per query row at part[(split * total_rows + row) * (D + 4)].
  int n_splits;
  int split_tokens;
  int64_t total_rows;
  float* part;
  // Paged, variable-length mode (PAGED kernel): q_rot / o_rot are (tokens, Hq, D); sequence b
  // owns query tokens cu_q[b] .. cu_q[b+1] - the LAST ones of its seq_lens[b] keys, so query i
  // sees keys 0 .. seq_lens[b] - q_len + i - and its keys and values sit in the pages
  // block_table[b][*] of the packed cache ([K codes | K norms | V codes | V norms] per token).
  const uint8_t* kv_cache;
  const int32_t* block_table;
  int64_t bt_stride;
  const int32_t* seq_lens;
  const int32_t* cu_q;
  int block_size;
  int64_t num_blocks;
  int total_q;    // query tokens in q_rot / o_rot (chunks must lie inside)
  int round_out;  // FQ_BF16 / FQ_F16: rows are rounded to that type before they are stored
  // beta_k, beta_v of the scaled fp16 centroid tables (centroid_scale_kernel, run just before)
  const float* scales;
};

template <int D>
struct PrefillSmem {
  static constexpr uint32_t kChunks = D / 8;                      // 16-byte chunks per row
  static constexpr uint32_t kSlabQ = (kPfM + 1) * 16;             // one k-chunk of the Q tile
  static constexpr uint32_t kSlabKV = (kPfN + 1) * 16;            // one k-chunk of a K/V tile
  static constexpr uint32_t kSlabP = (kPfM + 1) * 16;             // one k-chunk of the P tile
  static constexpr uint32_t kOpKV = kChunks * kSlabKV;            // one K or V operand tile
  static constexpr uint32_t kOffQ = 0;
  static constexpr uint32_t kOffK = kOffQ + kChunks * kSlabQ;     // two K operand tiles
  static constexpr uint32_t kOffV = kOffK + 2 * kOpKV;
  static constexpr uint32_t kOffP = kOffV + kOpKV;
  static constexpr uint32_t kOffRaw = kOffP + (kPfN / 8) * kSlabP;  // K codes, V codes
  static constexpr uint32_t kRawTile = kPfN * (D / 2);
  static constexpr uint32_t kOffNormRaw = kOffRaw + 2 * kRawTile;   // |k|, |v| as they arrive
  static constexpr uint32_t kOffNorm = kOffNormRaw + 2 * kPfN * 4;  // 2 x nk*scale, nv*2^8, lg2 nv
  static constexpr uint32_t kOffLut = kOffNorm + 4 * kPfN * 4;
  static constexpr uint32_t kOffXch = kOffLut + 2 * 256 * 4;       // row maxima / sums exchange
  static constexpr uint32_t kOffBar = kOffXch + kPfThreads * 4;
  static constexpr uint32_t kBytes = kOffBar + 64;
};

// Per tile the CUDA cores turn codes into operands and run the softmax, the tensor cores run
// two products; the loop is arranged so that the two overlap inside one CTA as well:
//   iteration t:  dequantise K(t+1)  |  wait for PV(t-1)  |  dequantise V(t)
//                 issue S(t+1) = Q K(t+1)^T into the other score buffer        (tensor)
//                 softmax of S(t) (issued one iteration earlier) -> P           (CUDA cores)
//                 issue O += P V(t)                                             (tensor)
// so a score product always has a whole softmax to complete in, and the PV product the next
// tile's key dequantisation.  Codes and norms arrive by bulk copies one tile ahead.
// 16 or 4 bytes global -> shared without a register in between; `valid` false writes zeros
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
               "r"(valid ? 16u : 0u)
               : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src, bool valid) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src),
               "r"(valid ? 4u : 0u)
               : "memory");
}
// the barrier receives one arrival from this thread once all its copies above have landed
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

template <int D, bool PAGED>
__global__ void __launch_bounds__(kPfThreads, 2) prefill_attention_kernel(PrefillArgs p) {
  using S = PrefillSmem<D>;
  constexpr uint32_t kIdescS = umma_idesc(kPfM, kPfN, false);
  constexpr uint32_t kIdescO = umma_idesc(kPfM, D, true);
  extern __shared__ __align__(1024) unsigned char smem[];
  uint64_t* bar_k = reinterpret_cast<uint64_t*>(smem + S::kOffBar);  // K codes (+ norms) landed
  uint64_t* bar_v = bar_k + 1;
  uint64_t* bar_s = bar_k + 2;  // [2]: score product of an even / odd tile completed
  uint64_t* bar_o = bar_k + 4;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bar_k + 5);
  float* nk_raw = reinterpret_cast<float*>(smem + S::kOffNormRaw);
  float* nv_raw = nk_raw + kPfN;
  float* nk_s = reinterpret_cast<float*>(smem + S::kOffNorm);  // [2][64], by tile parity
  float* vs_s = nk_s + 2 * kPfN;
  float* lv_s = vs_s + kPfN;
  uint32_t* lut_k = reinterpret_cast<uint32_t*>(smem + S::kOffLut);
  uint32_t* lut_v = lut_k + 256;
  float* xch = reinterpret_cast<float*>(smem + S::kOffXch);

  const int tid = threadIdx.x, warp = tid >> 5;
  // threads r and r + 128 share query row r: the first takes columns 0..31 of a score tile
  // (0..63 of the output), the second the rest; a warp reaches TMEM lanes 32*(warp%4)..+31
  const int row = tid & (kPfM - 1), half = tid >> 7;
  // heavy (late) query tiles first: the causal work per tile grows with its index
  const bool split_mode = p.n_splits > 1;
  const int m_tile = split_mode ? 0 : int(gridDim.x) - 1 - int(blockIdx.x);
  const int split = split_mode ? int(blockIdx.x) : 0;
  const int hq = blockIdx.y, b = blockIdx.z;
  const int group = p.hq / p.hkv;
  const int hkv = hq / group;
  const int m0 = m_tile * kPfM;
  // paged mode: this sequence's query tokens and keys; ctx keys precede the first query token
  int q_first = 0, q_len = p.nq, kv_len = p.nkv, ctx = 0;
  bool clamped = false;
  if constexpr (PAGED) {
    q_first = p.cu_q[b];
    q_len = p.cu_q[b + 1] - q_first;
    kv_len = p.seq_lens[b];
    const int64_t room = p.bt_stride * int64_t(p.block_size);  // keys a block-table row can name
    if (kv_len > room) {
      kv_len = int(room);
      clamped = true;
    }
    ctx = kv_len - q_len;
    // a chunk outside the query tokens is not touched; one longer than the grid covers is cut
    const bool outside = q_first < 0 || q_len < 0 || int64_t(q_first) + q_len > p.total_q;
    if ((outside || q_len > int(gridDim.x) * kPfM) && m_tile == 0 && tid == 0 && p.status)
      atomicOr(p.status, FQ_DEV_BAD_LENGTH);
    if (outside || m0 >= q_len) return;  // the grid is sized for the longest chunk
  }
  const int rows = q_len - m0 < kPfM ? q_len - m0 : kPfM;

  int kv_end = kv_len;
  if (p.causal && ctx + m0 + rows < kv_end) kv_end = ctx + m0 + rows;
  if (kv_end < 0) kv_end = 0;
  // a slice of the keys: move the bases, the loop below then sees tokens 0 .. kv_end of it
  const int kv_begin = split * p.split_tokens;
  if (split_mode) {
    kv_end = kv_end - kv_begin < p.split_tokens ? kv_end - kv_begin : p.split_tokens;
    if (kv_end < 0) kv_end = 0;
  }
  const int n_tiles = (kv_end + kPfN - 1) / kPfN;

  const int64_t kv_row0 = PAGED ? 0 : (int64_t(b) * p.hkv + hkv) * p.kv_stride + kv_begin;
  const uint8_t* kc_base = PAGED ? nullptr : p.k_packed + kv_row0 * (D / 2);
  const uint8_t* vc_base = PAGED ? nullptr : p.v_packed + kv_row0 * (D / 2);
  const float* kn_base = PAGED ? nullptr : p.k_norms + kv_row0;
  const float* vn_base = PAGED ? nullptr : p.v_norms + kv_row0;
  // norms ride along with the codes when a bulk copy can take them (16-byte granularity);
  // in paged mode they always arrive with the codes
  const bool norm_bulk =
      PAGED || ((reinterpret_cast<uintptr_t>(kn_base) | reinterpret_cast<uintptr_t>(vn_base)) & 15) == 0;

  // ---- set-up ---------------------------------------------------------------------------
  if (tid == 0) {
    mbar_init(bar_k, PAGED ? kPfThreads : 1);  // paged: one arrival per thread and tile
    mbar_init(bar_v, PAGED ? kPfThreads : 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 1, 1);
    mbar_init(bar_o, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_holder, kPfTmemCols);
    tmem_relinquish();
  }
  // tables of fp16(c / beta): beta_k folds into the score scale, beta_v into the weights
  const float beta_k = p.scales[0], beta_v = p.scales[1];
  const float rbk = 1.f / beta_k, rbv = 1.f / beta_v;
  for (int e = tid; e < 256; e += kPfThreads) {
    const int hi = e >> 4, lo = e & 15;
    lut_k[e] = pack_half2(hi < p.nck ? p.cent_k[hi] * rbk : 0.f, lo < p.nck ? p.cent_k[lo] * rbk : 0.f);
    lut_v[e] = pack_half2(hi < p.ncv ? p.cent_v[hi] * rbv : 0.f, lo < p.ncv ? p.cent_v[lo] * rbv : 0.f);
  }
  // Q tile -> [k-chunk][row][16 B]
  {
    const __half* qsrc = PAGED ? p.q_rot + (int64_t(q_first + m0) * p.hq + hq) * D
                               : p.q_rot + ((int64_t(b) * p.hq + hq) * p.nq + m0) * D;
    const int64_t q_pitch = PAGED ? int64_t(p.hq) * D : D;
    for (int i = tid; i < kPfM * int(S::kChunks); i += kPfThreads) {
      const int r = i / int(S::kChunks), kc = i % int(S::kChunks);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < rows) v = *reinterpret_cast<const uint4*>(qsrc + int64_t(r) * q_pitch + kc * 8);
      *reinterpret_cast<uint4*>(smem + S::kOffQ + kc * S::kSlabQ + r * 16) = v;
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_o = tmem_base + 2 * kPfN;  // behind the two score buffers; D columns
  const uint32_t lane_sel = uint32_t((warp & 3) * 32) << 16;

  // 8-entry key table in registers: low and high bytes of the fp16 centroids
  const bool k_by_permute = p.nck <= 8;
  uint32_t tl0 = 0, tl1 = 0, th0 = 0, th1 = 0;
  if (k_by_permute) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t h =
          uint32_t(__half_as_ushort(__float2half_rn(i < p.nck ? p.cent_k[i] * rbk : 0.f)));
      const uint32_t lo8 = (h & 0xffu) << (8 * (i & 3)), hi8 = (h >> 8) << (8 * (i & 3));
      if (i < 4) { tl0 |= lo8; th0 |= hi8; } else { tl1 |= lo8; th1 |= hi8; }
    }
  }
  auto tile_tokens = [&](int tile) {
    const int left = kv_end - tile * kPfN;
    return left < kPfN ? left : kPfN;
  };
  // thread 0: codes of one tile (and its norms, when a bulk copy can take them)
  auto issue_codes = [&](int tile, bool is_k) {
    const int t0 = tile * kPfN, n_tok = tile_tokens(tile);
    const uint32_t bytes = uint32_t(n_tok) * (D / 2);
    const bool with_norms = norm_bulk && n_tok == kPfN;
    uint64_t* bar = is_k ? bar_k : bar_v;
    mbar_expect_tx(bar, bytes + (with_norms ? kPfN * 4 : 0));
    bulk_g2s(smem + S::kOffRaw + (is_k ? 0 : S::kRawTile),
             (is_k ? kc_base : vc_base) + int64_t(t0) * (D / 2), bytes, bar);
    if (with_norms)
      bulk_g2s(is_k ? nk_raw : nv_raw, (is_k ? kn_base : vn_base) + t0, kPfN * 4, bar);
  };
  // Paged mode, ALL threads: the tile's codes and norms gathered through the block table, 16
  // bytes per thread (thread = (token, quarter of its 64 code bytes)) and one norm for the
  // first 64 threads; tokens past the end arrive as zeros.  The token rows of a tile (byte
  // offsets into the cache, -1 past the end) are looked up one tile before its key gather, so
  // that no gather waits for a block-table load; the value gather of the same tile, one
  // iteration later, reuses them.
  [[maybe_unused]] bool bad_page = false;
  [[maybe_unused]] auto token_row = [&](int t) -> int64_t {
    if (t >= kv_end) return -1;
    const int page = t / p.block_size;
    int64_t phys = p.block_table[int64_t(b) * p.bt_stride + page];
    if (phys < 0 || phys >= p.num_blocks) {  // reported, not followed
      phys = 0;
      bad_page = true;
    }
    return (phys * p.block_size + (t - page * p.block_size)) * int64_t(p.hkv * (D + 8));
  };
  struct TileRows {
    int64_t code, norm;  // rows of token tid/4 (codes) and of token tid (norm; threads 0..63)
  };
  [[maybe_unused]] auto tile_rows = [&](int tile) {
    TileRows r;
    r.code = token_row(tile * kPfN + (tid >> 2));
    r.norm = tid < kPfN ? token_row(tile * kPfN + tid) : -1;
    return r;
  };
  [[maybe_unused]] auto gather_codes = [&](const TileRows& r, bool is_k) {
    const int piece = tid & 3;
    const int code_off = (is_k ? 0 : p.hkv * (D / 2 + 4)) + hkv * (D / 2);
    const int norm_off = (is_k ? 0 : p.hkv * (D / 2 + 4)) + p.hkv * (D / 2) + 4 * hkv;
    cp_async16(smem_u32(smem + S::kOffRaw + (is_k ? 0 : S::kRawTile)) + tid * 16,
               p.kv_cache + (r.code < 0 ? 0 : r.code) + code_off + piece * 16, r.code >= 0);
    if (tid < kPfN)
      cp_async4(smem_u32(is_k ? nk_raw : nv_raw) + tid * 4,
                p.kv_cache + (r.norm < 0 ? 0 : r.norm) + norm_off, r.norm >= 0);
    cp_async_arrive(is_k ? bar_k : bar_v);
  };
  // rows of the tile whose values are gathered next / whose keys are gathered next
  [[maybe_unused]] TileRows rows_v{-1, -1}, rows_k{-1, -1};
  // all threads: codes of the landed tile -> fp16 operand tile at `op_off`
  auto dequantise = [&](int tile, bool is_k, uint32_t op_off) {
    const int n_tok = tile_tokens(tile);
    const uint32_t* raw =
        reinterpret_cast<const uint32_t*>(smem + S::kOffRaw + (is_k ? 0 : S::kRawTile));
    const uint32_t* lut = is_k ? lut_k : lut_v;
    constexpr int kWords = kPfN * (D / 8);  // 4 code bytes = 8 values = one 16-byte chunk
    if (is_k && k_by_permute) {
      // at most 8 key centroids: the codes select bytes of a register-resident table, no
      // shared-memory look-ups (whose random addresses conflict in the banks)
      for (int i = tid; i < kWords; i += kPfThreads) {
        const int tok = i / int(S::kChunks), kc = i % int(S::kChunks);
        const uint32_t w = tok < n_tok ? raw[i] : 0u;
        // nibbles of w, low to high: odd0, even0, odd1, even1, ...
        const uint32_t la = prmt(tl0, tl1, w), ha = prmt(th0, th1, w);
        const uint32_t lb = prmt(tl0, tl1, w >> 16), hb = prmt(th0, th1, w >> 16);
        uint4 o;
        o.x = prmt(la, ha, 0x4051);  // (even0, odd0)
        o.y = prmt(la, ha, 0x6273);
        o.z = prmt(lb, hb, 0x4051);
        o.w = prmt(lb, hb, 0x6273);
        *reinterpret_cast<uint4*>(smem + op_off + kc * S::kSlabKV + tok * 16) = o;
      }
      return;
    }
    for (int i = tid; i < kWords; i += kPfThreads) {
      const int tok = i / int(S::kChunks), kc = i % int(S::kChunks);
      const uint32_t w = tok < n_tok ? raw[i] : 0u;
      uint4 o;
      o.x = lut[w & 0xff]; o.y = lut[(w >> 8) & 0xff];
      o.z = lut[(w >> 16) & 0xff]; o.w = lut[w >> 24];
      *reinterpret_cast<uint4*>(smem + op_off + kc * S::kSlabKV + tok * 16) = o;
    }
  };
  // threads 0..63: the norm of token `tid` of the tile, from the bulk copy or from memory
  auto tile_norm = [&](int tile, bool is_k) {
    const int t0 = tile * kPfN, n_tok = tile_tokens(tile);
    if (PAGED || (norm_bulk && n_tok == kPfN)) return (is_k ? nk_raw : nv_raw)[tid];
    return tid < n_tok ? (is_k ? kn_base : vn_base)[t0 + tid] : 0.f;
  };
  auto issue_scores = [&](int tile) {  // thread 0
    const uint32_t qa = smem_u32(smem + S::kOffQ);
    const uint32_t ka = smem_u32(smem + S::kOffK + (tile & 1) * S::kOpKV);
#pragma unroll
    for (int s = 0; s < D / 16; ++s)
      umma_f16(tmem_base + (tile & 1) * kPfN, smem_desc(qa + 2 * s * S::kSlabQ, S::kSlabQ, 128),
               smem_desc(ka + 2 * s * S::kSlabKV, S::kSlabKV, 128), kIdescS, s > 0);
    umma_commit(bar_s + (tile & 1));
  };

  const float k_scale = p.scale_log2 * beta_k, v_scale = 256.f * beta_v;
  float m_run = -INFINITY, l_run = 0.f;
  const int q_pos = m0 + row;
  bool dead = false;

  // ---- prologue: K(0) -> operand, S(0) issued, K(1) and V(0) on their way ------------------
  if (n_tiles > 0) {
    if constexpr (PAGED) {
      rows_v = tile_rows(0);
      gather_codes(rows_v, true);
      gather_codes(rows_v, false);
      rows_v = tile_rows(1);  // keys of tile 1 below, its values in iteration 0
      rows_k = tile_rows(2);
    } else if (tid == 0) {
      issue_codes(0, true);
      issue_codes(0, false);
    }
    if (!mbar_wait(bar_k, 0)) dead = true;
    if (!dead) {
      if (tid < kPfN) nk_s[tid] = tile_norm(0, true) * k_scale;
      dequantise(0, true, S::kOffK);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && !dead) {
      tc_fence_after();
      issue_scores(0);
      if (!PAGED && n_tiles > 1) issue_codes(1, true);
    }
    if (PAGED && n_tiles > 1) gather_codes(rows_v, true);
  }

  for (int tile = 0; tile < n_tiles && !dead; ++tile) {
    const int t0 = tile * kPfN;
    const int n_tok = tile_tokens(tile);
    const bool more = tile + 1 < n_tiles;
    // ---- K(t+1): codes -> operand (the other K buffer), |k| * scale by tile parity -----------
    if (more) {
      if (!mbar_wait(bar_k, (tile + 1) & 1)) dead = true;
      if (!dead) {
        if (tid < kPfN) nk_s[((tile + 1) & 1) * kPfN + tid] = tile_norm(tile + 1, true) * k_scale;
        dequantise(tile + 1, true, S::kOffK + ((tile + 1) & 1) * S::kOpKV);
      }
    }
    // ---- V(t): the previous tile's P V still reads the V and P operands ----------------------
    if (tile > 0 && !mbar_wait(bar_o, (tile - 1) & 1)) dead = true;
    tc_fence_after();
    if (!mbar_wait(bar_v, tile & 1)) dead = true;
    if (!dead) {
      if (tid < kPfN) {
        const float nv = tile_norm(tile, false);
        vs_s[tid] = nv * v_scale;  // beta_v 2^kPfPScaleLog2
        lv_s[tid] = fmaxf(fast_log2(nv), -40.f);
      }
      dequantise(tile, false, S::kOffV);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && !dead) {
      tc_fence_after();
      if (more) issue_scores(tile + 1);  // runs while this tile's softmax does
      if constexpr (!PAGED) {
        if (tile + 2 < n_tiles) issue_codes(tile + 2, true);
        if (more) issue_codes(tile + 1, false);
      }
    }
    if constexpr (PAGED) {
      if (tile + 2 < n_tiles) gather_codes(rows_k, true);
      if (more) gather_codes(rows_v, false);
      rows_v = rows_k;                // tile + 2: its values go in the next iteration
      rows_k = tile_rows(tile + 3);   // looked up now, used in the next iteration
    }
    // ---- S(t), issued one iteration ago -----------------------------------------------------
    if (!mbar_wait(bar_s + (tile & 1), (tile >> 1) & 1)) dead = true;
    tc_fence_after();
    const uint32_t tmem_s = tmem_base + (tile & 1) * kPfN;
    const float* nk_t = nk_s + (tile & 1) * kPfN;

    // ---- online softmax on row `row` ---------------------------------------------------------
    // A tile that lies wholly below the diagonal of every row of the CTA and is full needs no
    // masking: the common case gets a loop body without predicates.
    const bool unmasked = n_tok == kPfN && (!p.causal || t0 + kPfN - 1 <= m0 + ctx);
    // pass 1: row maximum of logit*log2e + clamped log2|v| over this thread's half of the tile
    float mx = -INFINITY;
    auto row_max = [&](auto masked) {
      const int c0 = half * 32;
      float sv[32];
      tmem_ld32(tmem_s + lane_sel + c0, sv);
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 nk4 = *reinterpret_cast<const float4*>(nk_t + c0 + j);
        const float4 lv4 = *reinterpret_cast<const float4*>(lv_s + c0 + j);
        const float nk[4] = {nk4.x, nk4.y, nk4.z, nk4.w}, lv[4] = {lv4.x, lv4.y, lv4.z, lv4.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float e = fmaf(sv[j + u], nk[u], lv[u]);
          if constexpr (decltype(masked)::value) {
            const int col = c0 + j + u;
            const bool ok = col < n_tok && (!p.causal || t0 + col <= q_pos + ctx);
            e = ok ? e : -INFINITY;
          }
          mx = fmaxf(mx, e);
        }
      }
    };
    if (!dead) {
      if (unmasked) row_max(std::false_type{}); else row_max(std::true_type{});
    }
    xch[tid] = mx;
    __syncthreads();
    mx = fmaxf(mx, xch[tid ^ kPfM]);  // the other half of the row
    // The reference exponent m only has to stay within kPfMaxSlack bits of the running maximum
    // (weights then stay below 2^14 in fp16), so the accumulator O, which lives in TMEM across
    // all tiles, is rescaled only when some row of the warp outgrows it by more than that.
    const bool grew = mx > m_run + kPfMaxSlack;
    if (__any_sync(0xffffffffu, grew) && !dead) {
      const float m_new = grew ? mx : m_run;
      const float alpha = (m_run == -INFINITY || !grew) ? 1.f : fast_exp2(m_run - m_new);
      if (tile > 0) {
#pragma unroll
        for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
          float o[32];
          tmem_ld32(tmem_o + lane_sel + c0, o);
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] *= alpha;
          tmem_st32(tmem_o + lane_sel + c0, o);
        }
      }
      l_run *= alpha;
      m_run = m_new;
    }
    const float mref = (m_run == -INFINITY) ? 0.f : m_run;
    // pass 2: p = 2^(logit*log2e - m) feeds the denominator; the weight that meets the value
    // codes is p*|v|*2^8 (<= 2^14 because m >= logit*log2e + log2|v| - 6), stored as the fp16 A
    // operand of the second product, [token chunk][row][16 B]
    auto weights = [&](auto masked) {
      const float neg_m = -mref;
      const int c0 = half * 32;
      float sv[32];
      tmem_ld32(tmem_s + lane_sel + c0, sv);
      uint32_t packed[16];
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        const float4 nk4 = *reinterpret_cast<const float4*>(nk_t + c0 + j);
        const float4 vs4 = *reinterpret_cast<const float4*>(vs_s + c0 + j);
        const float nk[4] = {nk4.x, nk4.y, nk4.z, nk4.w}, vs[4] = {vs4.x, vs4.y, vs4.z, vs4.w};
        float w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float pe = fast_exp2(fmaf(sv[j + u], nk[u], neg_m));
          if constexpr (decltype(masked)::value) {
            const int col = c0 + j + u;
            const bool ok = col < n_tok && (!p.causal || t0 + col <= q_pos + ctx);
            pe = ok ? pe : 0.f;
          }
          l_run += pe;
          w[u] = pe * vs[u];
        }
        packed[j / 2] = pack_half2(w[0], w[1]);
        packed[j / 2 + 1] = pack_half2(w[2], w[3]);
      }
#pragma unroll
      for (int ch = 0; ch < 4; ++ch)
        *reinterpret_cast<uint4*>(smem + S::kOffP + (c0 / 8 + ch) * S::kSlabP + row * 16) =
            make_uint4(packed[4 * ch], packed[4 * ch + 1], packed[4 * ch + 2], packed[4 * ch + 3]);
    };
    if (!dead) {
      if (unmasked) weights(std::false_type{}); else weights(std::true_type{});
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- O += P V(t) ------------------------------------------------------------------------------
    if (tid == 0 && !dead) {
      tc_fence_after();
      const uint32_t pa = smem_u32(smem + S::kOffP), va = smem_u32(smem + S::kOffV);
#pragma unroll
      for (int s = 0; s < kPfN / 16; ++s)
        umma_f16(tmem_o, smem_desc(pa + 2 * s * S::kSlabP, S::kSlabP, 128),
                 smem_desc(va + s * 256, 128, S::kSlabKV), kIdescO, (tile > 0 || s > 0) ? 1u : 0u);
      umma_commit(bar_o);
    }
    tc_fence_before();
  }
  if (n_tiles > 0 && !dead && !mbar_wait(bar_o, (n_tiles - 1) & 1)) dead = true;
  tc_fence_after();

  // ---- epilogue: normalise, round, store the rotated-space row -----------------------------
  if (dead && tid == 0 && p.status) atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
  if constexpr (PAGED) {
    if ((bad_page || clamped) && p.status) atomicOr(p.status, FQ_DEV_BAD_BLOCK_INDEX);
  }
  {
    __syncthreads();  // the last tile's maxima have been read
    xch[tid] = l_run;
    __syncthreads();
    const float l_row = l_run + xch[tid ^ kPfM];  // both halves of the row
    const int64_t row_global = PAGED ? int64_t(q_first + q_pos) * p.hq + hq
                                     : (int64_t(b) * p.hq + hq) * p.nq + q_pos;
    // 2^-kPfPScaleLog2, and 1/l unless the rows of the slices are still to be merged
    const float inv = split_mode ? 1.f / 256.f : (l_row > 0.f ? 1.f / (l_row * 256.f) : 0.f);
    float* dst = split_mode ? p.part + (int64_t(split) * p.total_rows + row_global) * (D + 4)
                            : p.o_rot + row_global * D;
    if (split_mode && half == 0 && row < rows) {
      dst[D] = m_run;
      dst[D + 1] = l_row;
    }
#pragma unroll
    for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
      float o[32];
      if (n_tiles > 0 && !dead) {
        tmem_ld32(tmem_o + lane_sel + c0, o);  // whole warps: the load is warp-collective
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] = 0.f;
      }
      if (row < rows) {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          o[j] *= inv;
          // the reference's attention over de-quantised pages returns rows of the activation
          // type, which it then rotates (src/flashquant/vllm/impl.py:477-509): round here too
          if (p.round_out == FQ_BF16) o[j] = __bfloat162float(__float2bfloat16_rn(o[j]));
          if (p.round_out == FQ_F16) o[j] = __half2float(__float2half_rn(o[j]));
        }
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(dst + c0 + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
      }
    }
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_base, kPfTmemCols);
}

__global__ void __launch_bounds__(kScaleThreads) centroid_scale_kernel(
    const float* __restrict__ cent_k, int nck, const float* __restrict__ cent_v, int ncv,
    uint32_t* __restrict__ cache) {
  __shared__ __align__(16) unsigned char cent[kCentBytes];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (warp == 1) {
    const int i = lane & 15;
    float c = 0.f;
    if (lane < 16) { if (i < nck) c = cent_k[i]; } else { if (i < ncv) c = cent_v[i]; }
    stage_centroids(cent, c, nck, ncv, cache, lane);
  }
  __syncthreads();
  scale_centroid_tables(cent, nck, ncv, tid, cache);
}

// Merge of the slices' partial rows: o = sum_i 2^(m_i - M) o_i / sum_i 2^(m_i - M) l_i with
// M = max_i m_i (a slice without keys has m = -inf, l = 0).  32 threads per query row.
template <int D>
__global__ void __launch_bounds__(256) prefill_merge_kernel(const float* __restrict__ part,
                                                           int n_splits, int64_t total_rows,
                                                           float* __restrict__ o_rot) {
  static_assert(D == 128, "four columns per thread");
  const int64_t row = int64_t(blockIdx.x) * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= total_rows) return;
  float m_max = -INFINITY;
  for (int s = 0; s < n_splits; ++s)
    m_max = fmaxf(m_max, part[(int64_t(s) * total_rows + row) * (D + 4) + D]);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float l = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float* pr = part + (int64_t(s) * total_rows + row) * (D + 4);
    const float m = pr[D];
    if (m == -INFINITY) continue;
    const float w = fast_exp2(m - m_max);
    const float4 o = *reinterpret_cast<const float4*>(pr + 4 * lane);
    acc.x = fmaf(w, o.x, acc.x); acc.y = fmaf(w, o.y, acc.y);
    acc.z = fmaf(w, o.z, acc.z); acc.w = fmaf(w, o.w, acc.w);
    l = fmaf(w, pr[D + 1], l);
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  *reinterpret_cast<float4*>(o_rot + row * D + 4 * lane) =
      make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
}

// ------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------
template <int D, bool PAGED = false>
static int launch_prefill_t(const PrefillArgs& a, cudaStream_t stream) {
  using S = PrefillSmem<D>;
  auto kern = prefill_attention_kernel<D, PAGED>;
  static thread_local int set_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (set_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(S::kBytes));
    if (e != cudaSuccess)
      return fail(FQ_ERR_CUDA, "prefill: shared memory opt-in of %u bytes refused: %s", S::kBytes,
                  cudaGetErrorString(e));
    set_dev = dev;
  }
  dim3 grid(a.n_splits > 1 ? a.n_splits : (a.nq + kPfM - 1) / kPfM, a.hq, a.batch);
  kern<<<grid, kPfThreads, S::kBytes, stream>>>(a);
  int rc = check_launch("prefill attention kernel launch");
  if (rc != FQ_OK || a.n_splits <= 1 || a.o_rot == nullptr) return rc;
  prefill_merge_kernel<D><<<unsigned((a.total_rows + 7) / 8), 256, 0, stream>>>(
      a.part, a.n_splits, a.total_rows, a.o_rot);
  return check_launch("prefill merge kernel launch");
}

// beta_k, beta_v for the launch that follows: found in (or left at) bytes 64..255 of the
// workspace head, the record the decode kernels keep in theirs
static int centroid_scales(PrefillArgs& a, unsigned char* ws, cudaStream_t stream) {
  uint32_t* cache = reinterpret_cast<uint32_t*>(ws + kScaleCacheOffset);
  centroid_scale_kernel<<<1, kScaleThreads, 0, stream>>>(a.cent_k, a.nck, a.cent_v, a.ncv, cache);
  a.scales = reinterpret_cast<const float*>(cache + 32);
  return check_launch("centroid scale kernel launch");
}

constexpr int kPfMaxSplits = 64;  // slices of the keys for a single query token

struct PrefillWorkspace {
  size_t q_rot_off, o_rot_off, part_off, total;
};
// single_token: room for the partial rows of kPfMaxSplits slices behind the rotated output
static PrefillWorkspace prefill_workspace(int64_t rows, int d, bool single_token) {
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  PrefillWorkspace w;
  w.q_rot_off = 256;
  w.o_rot_off = up(w.q_rot_off + size_t(rows) * d * 2);
  w.part_off = up(w.o_rot_off + size_t(rows) * d * 4);
  w.total = single_token ? up(w.part_off + size_t(kPfMaxSplits) * rows * (d + 4) * 4) : w.part_off;
  return w;
}

}  // namespace fq

using namespace fq;

extern "C" size_t fq_fused_tq_attention_workspace_bytes(int batch, int num_q_heads, int n_q,
                                                        int head_dim) {
  if (batch < 0 || num_q_heads < 0 || n_q < 0 || head_dim < 0) return 0;
  return prefill_workspace(int64_t(batch) * num_q_heads * n_q, head_dim, n_q == 1).total;
}

static int attention_common(const void* q, fq_dtype dtype, const uint8_t* k_packed,
                            const float* k_norms, const uint8_t* v_packed, const float* v_norms,
                            const float* centroids_k, int n_centroids_k,
                            const float* centroids_v, int n_centroids_v, const float* rotation,
                            const float* rotation_v, int batch, int num_q_heads,
                            int num_kv_heads, int n_q, int n_kv, int64_t kv_stride, int head_dim,
                            float sm_scale, int is_causal, void* out, void* workspace,
                            size_t workspace_bytes, fq_stream_t stream) {
  FQ_REQUIRE(batch >= 0 && num_q_heads >= 1 && num_kv_heads >= 1 && n_q >= 0 && n_kv >= 0,
             FQ_ERR_INVALID_ARGUMENT, "fused attention: negative size");
  FQ_REQUIRE(q && k_packed && k_norms && v_packed && v_norms && centroids_k && centroids_v &&
                 rotation && rotation_v && out,
             FQ_ERR_INVALID_ARGUMENT, "fused attention: null pointer");
  FQ_REQUIRE(kv_stride >= n_kv, FQ_ERR_INVALID_ARGUMENT,
             "fused attention: %d tokens do not fit a buffer of %lld", n_kv, (long long)kv_stride);
  FQ_REQUIRE(dtype == FQ_F16 || dtype == FQ_BF16, FQ_ERR_UNSUPPORTED,
             "fused attention: q must be fp16 or bf16");
  FQ_REQUIRE(head_dim == 128, FQ_ERR_UNSUPPORTED,
             "fused attention: head_dim %d (the tensor-core kernel is built for 128)", head_dim);
  FQ_REQUIRE(num_q_heads % num_kv_heads == 0, FQ_ERR_INVALID_ARGUMENT,
             "fused attention: q heads not a multiple of KV heads");
  FQ_REQUIRE(n_centroids_k >= 1 && n_centroids_k <= 16 && n_centroids_v >= 1 &&
                 n_centroids_v <= 16,
             FQ_ERR_INVALID_ARGUMENT, "centroid count outside [1, 16]");
  FQ_REQUIRE(!is_causal || n_q == n_kv || n_q == 1, FQ_ERR_UNSUPPORTED,
             "fused attention: the causal mask is aligned at the first token (n_q == n_kv)");
  FQ_REQUIRE(aligned(q, 16) && aligned(out, 16) && aligned(k_packed, 16) && aligned(v_packed, 16) &&
                 aligned(rotation, 16) && aligned(rotation_v, 16),
             FQ_ERR_ALIGNMENT,
             "fused attention: q, out, the rotations and the packed codes must be 16-byte aligned");
  const int64_t rows = int64_t(batch) * num_q_heads * n_q;
  if (rows == 0) return FQ_OK;
  FQ_REQUIRE(n_kv >= 1, FQ_ERR_INVALID_ARGUMENT, "fused attention: no keys");
  const PrefillWorkspace w = prefill_workspace(rows, head_dim, n_q == 1);
  FQ_REQUIRE(workspace && aligned(workspace, 256) && workspace_bytes >= w.total, FQ_ERR_WORKSPACE,
             "fused attention: workspace of %zu bytes needed (256-byte aligned)", w.total);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  __half* q_rot = reinterpret_cast<__half*>(ws + w.q_rot_off);
  float* o_rot = reinterpret_cast<float*>(ws + w.o_rot_off);
  int rc = rotate_q_to_half(q, dtype, rotation, q_rot, rows, head_dim, stream);
  if (rc != FQ_OK) return rc;
  PrefillArgs a{};
  a.q_rot = q_rot;
  a.k_packed = k_packed; a.k_norms = k_norms;
  a.v_packed = v_packed; a.v_norms = v_norms;
  a.cent_k = centroids_k; a.nck = n_centroids_k;
  a.cent_v = centroids_v; a.ncv = n_centroids_v;
  a.o_rot = o_rot;
  a.batch = batch; a.hq = num_q_heads; a.hkv = num_kv_heads; a.nq = n_q; a.nkv = n_kv;
  a.kv_stride = kv_stride;
  a.scale_log2 = sm_scale * 1.4426950408889634f;
  a.causal = (is_causal && n_q > 1) ? 1 : 0;  // a single query token never needs the mask
  a.status = reinterpret_cast<uint32_t*>(ws);
  const int group = num_q_heads / num_kv_heads;
  if (n_q == 1 && group <= kPfM) {
    // One query token: the query heads of a KV group become the rows of one query tile
    // ((B, Hq, 1, D) read as (B, Hkv, group, D)), so the group's keys and values are
    // de-quantised once, and the keys are cut into slices so that the CTAs fill the GPU.
    a.hq = num_kv_heads; a.nq = group;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = (n_kv + kPfN - 1) / kPfN;
    const int64_t per_slice = int64_t(batch) * num_kv_heads;
    int want = int(2 * int64_t(sms) / per_slice);  // two CTAs per SM: one wave
    want = want < 1 ? 1 : (want > kPfMaxSplits ? kPfMaxSplits : want);
    const int tiles_per = (tiles + want - 1) / want;
    const int n_splits = (tiles + tiles_per - 1) / tiles_per;
    if (n_splits > 1) {
      a.n_splits = n_splits;
      a.split_tokens = tiles_per * kPfN;
      a.total_rows = rows;
      a.part = reinterpret_cast<float*>(ws + w.part_off);
      // few rows: the back-rotation merges the slices on its way in, no merge launch
      if (rotate_is_few_rows(rows)) a.o_rot = nullptr;
    }
  }
  rc = centroid_scales(a, ws, stream);
  if (rc != FQ_OK) return rc;
  rc = launch_prefill_t<128>(a, stream);
  if (rc != FQ_OK) return rc;
  if (a.n_splits > 1 && a.o_rot == nullptr)
    return rotate_back_merged(a.part, a.n_splits, dtype, rotation_v, out, rows, head_dim, stream);
  return rotate_back(o_rot, dtype, rotation_v, out, rows, head_dim, stream);
}

extern "C" int fq_fused_tq_attention(const void* q, fq_dtype dtype, const uint8_t* k_packed,
                                     const float* k_norms, const uint8_t* v_packed,
                                     const float* v_norms, const float* centroids_k,
                                     int n_centroids_k, const float* centroids_v,
                                     int n_centroids_v, const float* rotation, int batch,
                                     int num_q_heads, int num_kv_heads, int n_q, int n_kv,
                                     int head_dim, float sm_scale, int is_causal, void* out,
                                     void* workspace, size_t workspace_bytes,
                                     fq_stream_t stream) {
  FQ_RANGE("fq_fused_tq_attention");
  return attention_common(q, dtype, k_packed, k_norms, v_packed, v_norms, centroids_k,
                          n_centroids_k, centroids_v, n_centroids_v, rotation, rotation, batch,
                          num_q_heads, num_kv_heads, n_q, n_kv, n_kv, head_dim, sm_scale,
                          is_causal, out, workspace, workspace_bytes, stream);
}

extern "C" int fq_fused_tq_attention_kv(const void* q, fq_dtype dtype, const uint8_t* k_packed,
                                        const float* k_norms, const uint8_t* v_packed,
                                        const float* v_norms, const float* centroids_k,
                                        int n_centroids_k, const float* centroids_v,
                                        int n_centroids_v, const float* rotation_k,
                                        const float* rotation_v, int batch, int num_q_heads,
                                        int num_kv_heads, int n_q, int n_kv,
                                        int64_t kv_capacity, int head_dim, float sm_scale,
                                        int is_causal, void* out, void* workspace,
                                        size_t workspace_bytes, fq_stream_t stream) {
  FQ_RANGE("fq_fused_tq_attention_kv");
  return attention_common(q, dtype, k_packed, k_norms, v_packed, v_norms, centroids_k,
                          n_centroids_k, centroids_v, n_centroids_v, rotation_k, rotation_v,
                          batch, num_q_heads, num_kv_heads, n_q, n_kv, kv_capacity, head_dim,
                          sm_scale, is_causal, out, workspace, workspace_bytes, stream);
}

extern "C" size_t fq_paged_tq4_prefill_workspace_bytes(int total_q_tokens, int num_q_heads,
                                                       int head_dim) {
  if (total_q_tokens < 0 || num_q_heads < 0 || head_dim < 0) return 0;
  return prefill_workspace(int64_t(total_q_tokens) * num_q_heads, head_dim, false).total;
}

extern "C" int fq_paged_tq4_prefill(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                                    const int32_t* block_table, int64_t block_table_stride,
                                    const int32_t* seq_lens, const int32_t* cu_seqlens_q,
                                    const float* centroids_k, int n_centroids_k,
                                    const float* centroids_v, int n_centroids_v,
                                    const float* rotation, int num_seqs, int total_q_tokens,
                                    int max_q_len, int num_q_heads, int num_kv_heads,
                                    int head_dim, int block_size, int64_t num_blocks,
                                    float sm_scale, void* out, void* workspace,
                                    size_t workspace_bytes, fq_stream_t stream) {
  FQ_RANGE("fq_paged_tq4_prefill");
  FQ_REQUIRE(num_seqs >= 0 && total_q_tokens >= 0 && max_q_len >= 0 && num_q_heads >= 1 &&
                 num_kv_heads >= 1 && block_size >= 1 && num_blocks >= 0 && block_table_stride >= 0,
             FQ_ERR_INVALID_ARGUMENT, "paged prefill: negative size");
  if (num_seqs == 0 || total_q_tokens == 0 || max_q_len == 0) return FQ_OK;
  FQ_REQUIRE(q && kv_cache && block_table && seq_lens && cu_seqlens_q && centroids_k &&
                 centroids_v && rotation && out,
             FQ_ERR_INVALID_ARGUMENT, "paged prefill: null pointer");
  FQ_REQUIRE(dtype == FQ_F16 || dtype == FQ_BF16, FQ_ERR_UNSUPPORTED,
             "paged prefill: q must be fp16 or bf16");
  FQ_REQUIRE(head_dim == 128, FQ_ERR_UNSUPPORTED,
             "paged prefill: head_dim %d (the tensor-core kernel is built for 128)", head_dim);
  FQ_REQUIRE(num_q_heads % num_kv_heads == 0, FQ_ERR_INVALID_ARGUMENT,
             "paged prefill: q heads not a multiple of KV heads");
  FQ_REQUIRE(n_centroids_k >= 1 && n_centroids_k <= 16 && n_centroids_v >= 1 &&
                 n_centroids_v <= 16,
             FQ_ERR_INVALID_ARGUMENT, "centroid count outside [1, 16]");
  FQ_REQUIRE(num_kv_heads % 4 == 0, FQ_ERR_UNSUPPORTED,
             "paged prefill: %d KV heads (the 16-byte gathers need a multiple of 4)", num_kv_heads);
  FQ_REQUIRE(num_seqs <= 65535 && num_q_heads <= 65535, FQ_ERR_UNSUPPORTED,
             "paged prefill: more than 65535 sequences or query heads");
  FQ_REQUIRE(aligned(q, 16) && aligned(out, 16) && aligned(kv_cache, 16) && aligned(rotation, 16),
             FQ_ERR_ALIGNMENT, "paged prefill: q, out, the cache and the rotation must be 16-byte aligned");
  const int64_t rows = int64_t(total_q_tokens) * num_q_heads;
  const PrefillWorkspace w = prefill_workspace(rows, head_dim, false);
  FQ_REQUIRE(workspace && aligned(workspace, 256) && workspace_bytes >= w.total, FQ_ERR_WORKSPACE,
             "paged prefill: workspace of %zu bytes needed (256-byte aligned)", w.total);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  __half* q_rot = reinterpret_cast<__half*>(ws + w.q_rot_off);
  float* o_rot = reinterpret_cast<float*>(ws + w.o_rot_off);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int rc = rotate_q_to_half(q, dtype, rotation, q_rot, rows, head_dim, s);
  if (rc != FQ_OK) return rc;
  PrefillArgs a{};
  a.q_rot = q_rot;
  a.cent_k = centroids_k; a.nck = n_centroids_k;
  a.cent_v = centroids_v; a.ncv = n_centroids_v;
  a.o_rot = o_rot;
  a.batch = num_seqs; a.hq = num_q_heads; a.hkv = num_kv_heads; a.nq = max_q_len; a.nkv = 0;
  a.scale_log2 = sm_scale * 1.4426950408889634f;
  a.causal = 1;
  a.status = reinterpret_cast<uint32_t*>(ws);
  a.kv_cache = kv_cache;
  a.block_table = block_table;
  a.bt_stride = block_table_stride;
  a.seq_lens = seq_lens;
  a.cu_q = cu_seqlens_q;
  a.block_size = block_size;
  a.num_blocks = num_blocks;
  a.round_out = int(dtype);
  a.total_q = total_q_tokens;
  rc = centroid_scales(a, ws, s);
  if (rc != FQ_OK) return rc;
  rc = launch_prefill_t<128, true>(a, s);
  if (rc != FQ_OK) return rc;
  return rotate_back(o_rot, dtype, rotation, out, rows, head_dim, s);
}
