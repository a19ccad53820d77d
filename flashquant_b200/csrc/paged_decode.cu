// Split-K paged decode over the packed TQ4 cache for sm_100a.
//
// fq_split_k_paged_decode is ONE cooperative launch of paged_decode_kernel, one CTA per SM:
//   a. q rotation     every warp of the grid takes one 16x8 tile of q_rot = round(q Pi^T)
//                     (bf16 tensor-core products of a three-way split of Pi, fp32 exact to
//                     ~2^-24), stores it as fp16 and counts it in on the sequence's counter;
//   b. streaming      the pages of all sequences form one flat list that is cut into equal
//                     runs, one per team of warps; a run is processed as segments that never
//                     cross a boundary of the caller's split partition, and every segment
//                     leaves one (acc, m, l) partial row per query head and counts itself in
//                     on the sequence's second counter;
//   c. merge          when its teams are done a CTA takes (sequence, 8 heads) jobs: waits
//                     until the sequence's segments are all in, merges their rows, rounds to
//                     the output type and multiplies by Pi.
// Waits across CTAs (b on a, c on b) are bounded and never circular; the cooperative launch
// guarantees that all CTAs are resident.  The partial-row entry points run phase b alone
// (rotate_q_kernel before it, merge_rotate_kernel after it, as separate launches).
//
// The streaming phase is bound by HBM traffic (136 B per token and KV head) only if the
// per-byte instruction count stays near 3: a nibble code costs two table look-ups and, with
// 4 query heads per KV head, eight multiply-adds per byte, which the fp32 pipe cannot
// sustain at 7 TB/s.  So the multiply-adds go to the tensor pipe (mma.sync m16n8k16, the N
// dimension being the query heads of the group) and a byte is turned into two fp16
// centroids by ONE shared-memory look-up in a 256-entry table of fp16 pairs, replicated per
// lane so that look-ups never conflict (with at most 8 key centroids the key side needs no
// table at all: two byte permutes on a register-resident table do four look-ups).  Operand
// fragments are built directly in registers in the order the look-ups deliver them; the
// k-dimension of the QK product and the row dimension of the PV product are permuted
// accordingly (the query fragment and the write-back apply the same permutation).
//
// Pages reach shared memory by 1-D bulk copies into per-team rings of stages guarded by
// full/empty mbarriers; every wait is bounded and reports through the status word instead
// of spinning forever.
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "fq_common.cuh"
#include "centroid_scale.cuh"

namespace fq {

constexpr int kCW = 16;                  // compute warps per CTA
constexpr int kComputeThreads = kCW * 32;
static_assert(kComputeThreads == kScaleThreads, "the scale search runs on the compute threads");
// One more group of four warps holds the producer warp.  The CTA starts with 96 registers per
// thread (20 warps); the producer group then drops to 24, and the 128 x 72 registers it gives back
// let the 512 compute threads rise by 16 to 112 (a CTA cannot take more than it released).
constexpr int kDecodeThreads = kComputeThreads + 128;
constexpr int kLutBytes = 256 * 256;     // 256 entries x (32 lanes x 4 B for K + the same for V)
constexpr int kMaxStages = 16;           // per team; the descriptor ring relies on <= 16
constexpr int kMaxSeqs = 2048;                  // page-count prefix lives in shared memory
constexpr int kMaxSplits = 64;
constexpr int kPartPad = 4;                     // partial row = D + 4 floats (acc, m, l, 0, 0)
constexpr float kPScaleLog2 = 8.f;              // fp16 weights are scaled by 2^8 ...
constexpr float kMaxSlack = 6.f;                // ... and may exceed 1 by 2^6 before m is raised

constexpr int kMergeHeads = 8;                  // query heads per merge job
constexpr int kMaxParts = 4096;   // partial rows one sequence can have (teams + splits)
constexpr int kPartChunk = 128;  // rows merged per pass
// Single-launch merge of a sequence with very many partial rows (few KV heads per GPU: sixteen
// one-warp teams per CTA): the rows are cut into up to kMaxMergeChunks chunks, one merge job
// each; the job that finishes last merges the chunks' rows.  kMaxChunkJobs bounds
// (sequences x head groups) of such a call (its counters sit behind the per-sequence ones).
constexpr int kMaxMergeChunks = 16;
constexpr int kRowsPerMergeChunk = 20;  // one batch of row loads per merge job
constexpr int kMaxChunkJobs = 1024;
// shared memory of a merge job of the single-launch form besides Pi: rounded rows, row list
constexpr uint32_t kMergeScratchBytes =
    (kMergeHeads * 128 + kMergeHeads * kComputeThreads / 2 + 64 + kMaxParts + 4) * 4;

enum : int { kSegStart = 1, kSegEnd = 2, kQNew = 4 };

struct DecodeArgs {
  const __half* q_rot;  // (num_seqs, Hq, D)
  const uint8_t* kv_cache;
  const int32_t* block_table;
  int64_t bt_stride;
  int max_pages;  // columns of a block-table row that may be read
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
  int n_q;             // query tokens per sequence (fast path; hq counts all of their heads)
  uint64_t wait_ns;    // limit of every wait on another CTA or on a copy
  uint32_t seg_extra;  // test hook: the merge expects this many segment arrivals too many
  float* slots;  // (num_seqs * S + workers, Hq, D+4), workers = gridDim.x * teams
  uint32_t* status;
  uint32_t off_ring, off_q, off_prefix, off_desc, off_bar, off_cent;
  // single-launch form only
  const void* q_src;      // (num_seqs, Hq, D) in the caller's type
  const float* rotation;  // (D, D)
  void* out;              // (num_seqs, Hq, D) in the caller's type
  __half* q_rot_w;        // where phase a writes what `q_rot` reads
  uint32_t* q_count;      // [kMaxSeqs] rotated tiles of a sequence that are stored
  uint32_t* seg_count;    // [kMaxSeqs] (segment, warp) pairs of a sequence that are stored
  uint32_t* merge_count;  // [kMaxSeqs] merge jobs of a sequence that are finished
  uint32_t* chunk_count;  // [kMaxChunkJobs] finished chunks of a (sequence, head group) merge
  float* chunk_rows;      // [(job * merge_chunks + chunk) * kMergeHeads + head][D + 4]
  int merge_chunks;       // 1: one job merges all rows of a (sequence, head group)
  // two-stage (QJL) scoring only: logit += gamma * sqrt(pi/2)/m * <S q, signs>
  const uint8_t* kq_cache;  // (num_blocks, block_size, Hkv * (D/8 + 4)): sign bits | gamma
  const float* qjl;         // S (D, D)
  __half* qs_w;             // where phase a writes fp16(q S^T), (num_seqs, Hq, D)
  float corr_scale_log2;    // sqrt(pi/2) / m * sm_scale * log2(e)
};

// ------------------------------------------------------------------------------------
// page-count prefix of the batch, built by one warp into shared memory
// ------------------------------------------------------------------------------------
// A sequence never owns more pages than its block-table row has columns: a length beyond
// max_pages * block_size is cut there (the reference's CPU path would raise an IndexError on the
// table) and, where `status` is given, reported as FQ_DEV_BAD_BLOCK_INDEX.
__device__ __forceinline__ void build_page_prefix(const int32_t* __restrict__ seq_lens, int n,
                                                  int block_size, int max_pages, uint32_t* status,
                                                  int* prefix, int lane) {
  int carry = 0;
  if (lane == 0) prefix[0] = 0;
  for (int base = 0; base < n; base += 32) {
    const int i = base + lane;
    int len = i < n ? seq_lens[i] : 0;
    if (len < 0) len = 0;
    int v = (len + block_size - 1) / block_size;
    if (v > max_pages) {
      v = max_pages;
      if (status) atomicOr(status, FQ_DEV_BAD_BLOCK_INDEX);
    }
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

// Barrier of the 16 compute warps (the producer warp group does not take part).
__device__ __forceinline__ void compute_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kComputeThreads) : "memory");
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

// The same rotation for one 16-row x 8-column tile, by one warp on the tensor pipe:
// rows = q heads 16*mt .. 16*mt+15 of sequence `seq`, columns 8*nt .. 8*nt+7.  Pi is split
// into three bf16 terms (8 + 8 + 8 significant bits), a bf16 q is used as it is and an fp16
// q is split into two bf16 terms, so every product is exact and the sum is accumulated in
// fp32, like the fp32 multiply-adds of rotate_q_kernel.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void split3_bf16(float2 v, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(v.x, v.y);
  const float rx = v.x - __low2float(h), ry = v.y - __high2float(h);
  const __nv_bfloat162 m = __floats2bfloat162_rn(rx, ry);
  hi = *reinterpret_cast<const uint32_t*>(&h);
  mid = *reinterpret_cast<const uint32_t*>(&m);
  lo = pack_bf16x2(rx - __low2float(m), ry - __high2float(m));
}

// Operands of one tile: loaded early (one round trip to L2, all loads in flight together),
// used late, so that other set-up work runs in the shadow of the loads.  The k index of the
// products may be permuted freely as long as both operands agree: lane (g,t) takes k = 32c +
// 8t .. 8t+7 of chunk c with 16-byte loads and spends them on the two k-steps of the chunk.
template <int D>
struct RotTileOperands {
  uint4 a0[D / 32], a1[D / 32];   // q rows r0 and r0+8, 8 values each per chunk
  float4 b0[D / 32], b1[D / 32];  // Pi row n: first and second four k of the lane's eight
};

template <int D, typename T>
__device__ __forceinline__ void rotate_q_tile_load(RotTileOperands<D>& op, const T* __restrict__ q,
                                                   const float* __restrict__ rotation, int hq,
                                                   int seq, int mt, int nt, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const int r0 = mt * 16 + g, r1 = r0 + 8;
  const bool ok0 = r0 < hq, ok1 = r1 < hq;
  const T* q0 = q + (int64_t(seq) * hq + (ok0 ? r0 : 0)) * D + 8 * t;
  const T* q1 = q + (int64_t(seq) * hq + (ok1 ? r1 : 0)) * D + 8 * t;
  const float* pr = rotation + (8 * nt + g) * D + 8 * t;  // B[k][n] = Pi[n][k]
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
  for (int c = 0; c < D / 32; ++c) {
    op.a0[c] = ok0 ? *reinterpret_cast<const uint4*>(q0 + 32 * c) : zero;
    op.a1[c] = ok1 ? *reinterpret_cast<const uint4*>(q1 + 32 * c) : zero;
    op.b0[c] = *reinterpret_cast<const float4*>(pr + 32 * c);
    op.b1[c] = *reinterpret_cast<const float4*>(pr + 32 * c + 4);
  }
}

template <int D, typename T, bool kRound = true>
__device__ __forceinline__ void rotate_q_tile_finish(const RotTileOperands<D>& op,
                                                     __half* __restrict__ out, int hq, int seq,
                                                     int mt, int nt, int lane) {
  const int g = lane >> 2, t = lane & 3;
  const int r0 = mt * 16 + g, r1 = r0 + 8;
  const bool ok0 = r0 < hq, ok1 = r1 < hq;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    const int c = ks >> 1;
    const bool second = ks & 1;
    const float4 bv = second ? op.b1[c] : op.b0[c];
    const uint32_t a[4] = {second ? op.a0[c].z : op.a0[c].x, second ? op.a1[c].z : op.a1[c].x,
                           second ? op.a0[c].w : op.a0[c].y, second ? op.a1[c].w : op.a1[c].y};
    uint32_t bh[2], bm[2], bl[2];
    split3_bf16(make_float2(bv.x, bv.y), bh[0], bm[0], bl[0]);
    split3_bf16(make_float2(bv.z, bv.w), bh[1], bm[1], bl[1]);
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      mma_bf16(acc, a[0], a[1], a[2], a[3], bl[0], bl[1]);
      mma_bf16(acc, a[0], a[1], a[2], a[3], bm[0], bm[1]);
      mma_bf16(acc, a[0], a[1], a[2], a[3], bh[0], bh[1]);
    } else {
      uint32_t ah[4], al[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&a[i]));
        const __nv_bfloat162 h = __floats2bfloat162_rn(f.x, f.y);
        ah[i] = *reinterpret_cast<const uint32_t*>(&h);
        al[i] = pack_bf16x2(f.x - __low2float(h), f.y - __high2float(h));  // 3 bits: exact
      }
      mma_bf16(acc, al[0], al[1], al[2], al[3], bl[0], bl[1]);
      mma_bf16(acc, ah[0], ah[1], ah[2], ah[3], bl[0], bl[1]);
      mma_bf16(acc, al[0], al[1], al[2], al[3], bm[0], bm[1]);
      mma_bf16(acc, ah[0], ah[1], ah[2], ah[3], bm[0], bm[1]);
      mma_bf16(acc, al[0], al[1], al[2], al[3], bh[0], bh[1]);
      mma_bf16(acc, ah[0], ah[1], ah[2], ah[3], bh[0], bh[1]);
    }
  }
  const int col = 8 * nt + 2 * t;
  if constexpr (kRound) {  // round to the query's type first, as the reference does
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[c] = to_f32(from_f32<T>(acc[c]));
  }
  if (ok0)
    *reinterpret_cast<__half2*>(out + (int64_t(seq) * hq + r0) * D + col) =
        __floats2half2_rn(acc[0], acc[1]);
  if (ok1)
    *reinterpret_cast<__half2*>(out + (int64_t(seq) * hq + r1) * D + col) =
        __floats2half2_rn(acc[2], acc[3]);
}

// ------------------------------------------------------------------------------------
// phase c of the single-launch form: (sequence, 8 heads) merge jobs, CTA c takes jobs c,
// c + grid, ...  The look-up table and the rings are dead by now: Pi goes where the table
// was, the job's scratch where the first ring stages were.
// ------------------------------------------------------------------------------------
template <int D, typename T>
__device__ __forceinline__ void fused_merge(const DecodeArgs& p, unsigned char* smem,
                                            const int* prefix, int64_t total, int64_t active,
                                            int teams, int stages) {
  constexpr int ROWF = D + kPartPad;
  constexpr int HP = kComputeThreads / D;  // heads handled at a time
  constexpr int PASSES = kMergeHeads / HP;
  constexpr int RP = kComputeThreads / 2 / D;  // heads covered at a time by the final rotation
  constexpr int RH = kMergeHeads / RP;         // heads per thread there
  constexpr int TPG = kMergeHeads * D / 4;  // threads that cover 8 rows, four values each
  constexpr int G = kComputeThreads / TPG;   // groups of such threads
  constexpr int kBatch = 10;                // rows a thread keeps in flight
  const int tid = threadIdx.x;
  const int hgroups = (p.hq + kMergeHeads - 1) / kMergeHeads;
  const int jobs = p.num_seqs * hgroups;
  // C > 1: the rows of a (sequence, head group) are cut into C chunks, one merge job each;
  // the job that finishes last merges the C rows the chunks leave behind
  const int C = p.merge_chunks;
  compute_sync();  // every warp of the CTA has left the table and the rings
  if (int(blockIdx.x) >= jobs * C) return;

  float* pi_s = reinterpret_cast<float*>(smem);  // [k][j]
  float* o_s = reinterpret_cast<float*>(smem + p.off_ring);  // [8][D]
  float* num_s = o_s + kMergeHeads * D;                      // [G][8][D]
  float2* ml_s = reinterpret_cast<float2*>(num_s + G * kMergeHeads * D);  // [G][8]: m, den
  int* part_row = reinterpret_cast<int*>(ml_s + G * kMergeHeads);
  int* n_parts_s = part_row + kMaxParts;
  uint64_t* pi_bar = reinterpret_cast<uint64_t*>(smem + p.off_bar) + teams * (2 * stages + 2);
  if (tid == 0) {
    fence_proxy_async();  // the table was written by ordinary stores
    mbar_expect_tx(pi_bar, D * D * 4);
    bulk_g2s(pi_s, p.rotation, D * D * 4, pi_bar);
  }
  bool pi_ready = false;
  const int d = tid % D, hh0 = tid / D;
  const int grp = tid / TPG, mh = (tid % TPG) / (D / 4), dq = tid % (D / 4);

  int* last_s = n_parts_s + 1;  // C > 1: whether this job was the last chunk of its rows
  for (int sub = blockIdx.x; sub < jobs * C; sub += gridDim.x) {
    const int job = sub / C, chunk = sub - job * C;
    const int seq = job / hgroups, h0 = (job - seq * hgroups) * kMergeHeads;
    // ---- the sequence's partial rows (one lane per split), and the wait until all of them
    // are stored ---------------------------------------------------------------------------
    if (tid < 32) {
      const int p0 = prefix[seq], n_pages = prefix[seq + 1] - p0;
      const int pps = n_pages > 0 ? (n_pages + p.num_splits - 1) / p.num_splits : 1;
      int n = 0;
      for (int sb = 0; sb < p.num_splits; sb += 32) {
        const int sp = sb + tid;
        const int a = sp * pps;
        int b = a + pps;
        if (b > n_pages) b = n_pages;
        int c_first = 0, cnt = 0;
        if (sp < p.num_splits && a < b) {
          c_first = cta_of_page(int64_t(p0) + a, total, active);
          cnt = cta_of_page(int64_t(p0) + b - 1, total, active) - c_first + 1;
        }
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, incl, o);
          if (tid >= o) incl += up;
        }
        const int at = n + incl - cnt;
        for (int c = 0; c < cnt && at + c < kMaxParts; ++c)
          part_row[at + c] = seq * p.num_splits + sp + c_first + c;
        n += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (n > kMaxParts) n = kMaxParts;
      if (tid == 0) {
        *n_parts_s = n;
        const uint32_t expected = uint32_t(n) * uint32_t(p.hkv) + p.seg_extra;
        uint64_t t0 = 0;
        while (ld_acquire_u32(p.seg_count + seq) < expected) {
          __nanosleep(32);
          const uint64_t now = global_timer_ns();
          if (t0 == 0) t0 = now;
          if (now - t0 > p.wait_ns) {
            atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
            break;
          }
        }
        // the acquire above orders the rows' stores (released with the count) before the
        // loads below, which go to the L2 (ld.global.cg) after the barrier
      }
    }
    compute_sync();
    const int n_parts = *n_parts_s;
    // rows were written by other SMs during this launch: read them past the L1
    // (`chunks`: the rows that the C chunk jobs of this (sequence, head group) left behind)
    auto row_ptr = [&](int i, int h, bool chunks) {
      return chunks ? p.chunk_rows + ((int64_t(job) * C + i) * kMergeHeads + (h - h0)) * ROWF
                    : p.slots + (int64_t(part_row[i]) * p.hq + h) * ROWF;
    };

    // ---- G groups of threads take every G-th partial row; thread (head mh, four coordinates
    // from 4*dq) keeps up to kBatch rows in registers so that all loads of a job are in
    // flight together, and recomputes the weights of its head itself -------------------------
    auto accumulate = [&](int lo, int hi, bool chunks) {
      const int h = h0 + mh;
      float m_run = -INFINITY, den = 0.f;
      float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int c0 = lo + grp; c0 < hi; c0 += G * kBatch) {
        float2 ml[kBatch];
        float4 v[kBatch];
#pragma unroll
        for (int x = 0; x < kBatch; ++x) {
          ml[x] = make_float2(-INFINITY, 0.f);
          v[x] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (c0 + x * G < hi && h < p.hq) {
            const float* row = row_ptr(c0 + x * G, h, chunks);
            ml[x] = __ldcg(reinterpret_cast<const float2*>(row + D));
            v[x] = __ldcg(reinterpret_cast<const float4*>(row) + dq);
          }
        }
        float m_new = m_run;
#pragma unroll
        for (int x = 0; x < kBatch; ++x) m_new = fmaxf(m_new, ml[x].x);
        const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_new);
        den *= alpha;
        num.x *= alpha; num.y *= alpha; num.z *= alpha; num.w *= alpha;
#pragma unroll
        for (int x = 0; x < kBatch; ++x) {
          const float w = (ml[x].x == -INFINITY) ? 0.f : exp2f(ml[x].x - m_new);
          den = fmaf(w, ml[x].y, den);
          num.x = fmaf(w, v[x].x, num.x);
          num.y = fmaf(w, v[x].y, num.y);
          num.z = fmaf(w, v[x].z, num.z);
          num.w = fmaf(w, v[x].w, num.w);
        }
        m_run = m_new;
      }
      reinterpret_cast<float4*>(num_s + (grp * kMergeHeads + mh) * D)[dq] = num;
      if (dq == 0) ml_s[grp * kMergeHeads + mh] = make_float2(m_run, den);
    };
    // ---- combine the groups; thread (head hh, coordinate d).  `finish`: normalise and round
    // into o_s; otherwise leave the un-normalised row of this chunk in the workspace -----------
    auto combine = [&](bool finish) {
#pragma unroll
      for (int ps = 0; ps < PASSES; ++ps) {
        const int hh = hh0 + ps * HP;
        float m_all = -INFINITY;
#pragma unroll
        for (int gi = 0; gi < G; ++gi) m_all = fmaxf(m_all, ml_s[gi * kMergeHeads + hh].x);
        float den = 0.f, num = 0.f;
#pragma unroll
        for (int gi = 0; gi < G; ++gi) {
          const float2 ml = ml_s[gi * kMergeHeads + hh];
          const float w = (ml.x == -INFINITY) ? 0.f : exp2f(ml.x - m_all);
          den = fmaf(w, ml.y, den);
          num = fmaf(w, num_s[(gi * kMergeHeads + hh) * D + d], num);
        }
        if (finish) {
          const float o = (h0 + hh < p.hq && den > 0.f) ? num / den : 0.f;
          o_s[hh * D + d] = to_f32(from_f32<T>(o));  // the reference rounds the rotated output
        } else {
          float* row = p.chunk_rows + ((int64_t(job) * C + chunk) * kMergeHeads + hh) * ROWF;
          row[d] = num;
          if (d == 0) *reinterpret_cast<float2*>(row + D) = make_float2(m_all, den);
        }
      }
    };
    if (C == 1) {
      accumulate(0, n_parts, false);
      compute_sync();
      combine(true);
    } else {
      accumulate(int(int64_t(n_parts) * chunk / C), int(int64_t(n_parts) * (chunk + 1) / C), false);
      compute_sync();
      combine(false);
      __threadfence();  // this thread's part of the chunk row, before the count below
      compute_sync();
      if (tid == 0) {
        const bool last = atomicAdd(p.chunk_count + job, 1u) == uint32_t(C - 1);
        if (last) p.chunk_count[job] = 0u;  // for the next call
        __threadfence();                    // the other chunks' rows, after the count
        *last_s = last ? 1 : 0;
      }
      compute_sync();
      if (*last_s == 0) {
        compute_sync();  // (last_s and the scratch are reused by the next job)
        continue;
      }
      accumulate(0, C, true);
      compute_sync();
      combine(true);
    }
    compute_sync();
    if (!pi_ready) {
      if (!mbar_wait(pi_bar, 0, p.wait_ns)) {  // only if the copy were lost
        if (tid == 0) atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
        return;
      }
      pi_ready = true;
    }
    // out = o Pi: half of the threads, each with RH heads per value of Pi it reads (reading
    // Pi from shared memory is what bounds this step)
    if (tid < kComputeThreads / 2) {
      float acc[RH];
#pragma unroll
      for (int r = 0; r < RH; ++r) acc[r] = 0.f;
#pragma unroll 2
      for (int k4 = 0; k4 < D; k4 += 4) {
        const float b0 = pi_s[(k4 + 0) * D + d], b1 = pi_s[(k4 + 1) * D + d];
        const float b2 = pi_s[(k4 + 2) * D + d], b3 = pi_s[(k4 + 3) * D + d];
#pragma unroll
        for (int r = 0; r < RH; ++r) {
          const float4 a = *reinterpret_cast<const float4*>(o_s + (hh0 + r * RP) * D + k4);
          acc[r] = fmaf(a.x, b0, acc[r]);
          acc[r] = fmaf(a.y, b1, acc[r]);
          acc[r] = fmaf(a.z, b2, acc[r]);
          acc[r] = fmaf(a.w, b3, acc[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < RH; ++r) {
        const int hh = hh0 + r * RP;
        if (h0 + hh < p.hq)
          static_cast<T*>(p.out)[(int64_t(seq) * p.hq + h0 + hh) * D + d] = from_f32<T>(acc[r]);
      }
    }
    compute_sync();  // scratch is reused by the next job
    // the last job of a sequence puts its counters back to zero for the next call
    if (tid == 0 && atomicAdd(p.merge_count + seq, 1u) == uint32_t(hgroups - 1)) {
      p.q_count[seq] = 0u;
      p.seg_count[seq] = 0u;
      p.merge_count[seq] = 0u;
    }
  }
}

// ------------------------------------------------------------------------------------
// 2. streaming kernel
//
// A CTA of 16 warps hosts T = 16 / H_kv independent teams of H_kv warps (one warp per KV
// head).  The flat page list of the batch is cut into C*T equal runs, one per team; a team
// walks its run page by page through its own ring of shared-memory stages.  The first warp
// of a team is also its producer: its lane 0 issues the bulk copies, without ever blocking,
// whenever the warp is about to wait for a page ("pump"), and the whole warp prepares the
// page descriptors (physical page, valid tokens, segment flags, partial-row slot) 32 at a
// time, one chunk ahead.  Warps of a team never synchronise with each other except through
// the stage barriers, and every warp writes its own partial rows.
// ------------------------------------------------------------------------------------
// With at most 8 key centroids every second word of key codes goes through the shared-memory
// table and the others through byte permutes on a register table: the permutes issue at half
// rate on the ALU pipe, the look-ups load the shared-memory pipe; the mix balances the two.
constexpr bool kMixKeyLookups = true;
constexpr uint32_t kLutStride = 256;  // bytes per table entry: K copy per lane, then V copy
constexpr int kDescRing = 64;

__device__ __forceinline__ uint32_t lds_u32(const unsigned char* smem, uint32_t off) {
  return *reinterpret_cast<const uint32_t*>(smem + off);
}

// fp16 pair (+-1, +-1) from two sign bits: value j is -1 when bit p+j of x is SET (x is the
// complement of the stored word, where a set bit means +1)
__device__ __forceinline__ uint32_t sign_pair(uint32_t x, int p) {
  return 0x3C003C00u | (((x >> p) << 15) & 0x8000u) | ((x >> (p + 1)) << 31);
}

// (byte i of w) * 256 + lane4 in one instruction (lane4 < 128 sits in byte 0)
template <int I>
__device__ __forceinline__ uint32_t lut_addr(uint32_t w, uint32_t lane4) {
  return prmt(w, lane4, 0x5504u | (uint32_t(I) << 4));
}

// FUSE: 0 = streaming phase only; 1 / 2 = single-launch form for bf16 / fp16 q and out;
// 3 / 4 = the same with the two-stage (QJL) estimator in the logits
template <int D, bool KPRMT, int FUSE>
__global__ void __launch_bounds__(kDecodeThreads, 1) paged_decode_kernel(DecodeArgs p) {
  using TQ = typename std::conditional<FUSE == 2 || FUSE == 4, __half, __nv_bfloat16>::type;
  constexpr bool QS = FUSE >= 3;
  static_assert(!QS || D == 128, "the two-stage estimator is built for head_dim 128");
  constexpr int KS = D / 16;  // k-steps of the QK product = m-tiles of the PV product
  constexpr int KW = D / 32;  // 32-bit words of K codes per lane and row
  constexpr int VB = D / 16;  // bytes of V codes per lane and row
  constexpr int VW = (VB + 3) / 4;
  constexpr int ROWF = D + kPartPad;

  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t half_d = D / 2;
  const uint32_t row_bytes = uint32_t(p.hkv) * (D + 8);
  const uint32_t page_bytes = uint32_t(p.block_size) * row_bytes;
  // side-plane page of the stage (QS): behind the cache page
  const uint32_t qrow_bytes = QS ? uint32_t(p.hkv) * (D / 8 + 4) : 0u;
  const uint32_t qpage_bytes = uint32_t(p.block_size) * qrow_bytes;
  const uint32_t stage_bytes = page_bytes + qpage_bytes;
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int group = p.hq / p.hkv;  // q heads per KV head (<= 8)
  const uint32_t q_bytes = uint32_t(p.hq) * D * 2;
  const uint32_t qbuf_bytes = q_bytes * (QS ? 2u : 1u);  // q_rot, then q S^T
  const int teams = kCW / p.hkv;
  const int team = warp / p.hkv;
  const int head = warp - team * p.hkv;
  const bool leader = head == 0;
  const int stages = p.stages;

  int* prefix = reinterpret_cast<int*>(smem + p.off_prefix);
  int4* desc_ring = reinterpret_cast<int4*>(smem + p.off_desc) + team * kDescRing;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + p.off_bar) + team * (2 * stages + 2);
  uint64_t* empty_bar = full_bar + stages;
  uint64_t* qfull_bar = empty_bar + stages;
  uint64_t* qempty_bar = qfull_bar + 1;
  const uint32_t ring_off = p.off_ring + uint32_t(team) * stages * stage_bytes;
  const uint32_t q_off = p.off_q + uint32_t(team) * qbuf_bytes;

  const int q_tiles = ((p.hq + 15) / 16) * (D / 8);  // rotated tiles per sequence
  [[maybe_unused]] RotTileOperands<D> rot_op;
  [[maybe_unused]] int rot_len = 0;
  // with QS every tile exists twice: job < half rotates by Pi, the rest projects by S
  [[maybe_unused]] const int rot_half = p.num_seqs * q_tiles;
  [[maybe_unused]] const int rot_jobs = rot_half * (QS ? 2 : 1);
  [[maybe_unused]] const uint32_t q_target = uint32_t(q_tiles) * (QS ? 2u : 1u);
  [[maybe_unused]] const int rot_job0 = blockIdx.x * kCW + warp;
  [[maybe_unused]] const int m_tiles = (p.hq + 15) / 16;
  // ---- set-up: barriers, page prefix (warp 0), look-up table (all warps) ---------------
  if (leader && lane == 0 && warp < kCW) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(full_bar + s, 1);
      mbar_init(empty_bar + s, p.hkv);
    }
    mbar_init(qfull_bar, 1);
    mbar_init(qempty_bar, p.hkv);
    if (FUSE && tid == 0)
      mbar_init(reinterpret_cast<uint64_t*>(smem + p.off_bar) + teams * (2 * stages + 2), 1);
    mbar_fence_init();
  }
  // The first loads of a CTA miss every cache, so the two that do not depend on each other
  // go out together: the sequence lengths (warp 0, for the page prefix) and the centroids
  // (warp 1, as fp16).  The block table can only be read once the prefix is there, and the
  // first page only after that: the leaders start both right after the barrier below, and
  // the look-up table is filled while those loads are in flight.
  const unsigned short* cs = reinterpret_cast<const unsigned short*>(smem + p.off_cent);
  float cent_val = 0.f;
  if (warp == 1) {
    const int i = lane & 15;
    if (lane < 16) { if (i < p.nck) cent_val = p.cent_k[i]; } else { if (i < p.ncv) cent_val = p.cent_v[i]; }
  }
  // ---- phase a, first half: the operands of this warp's query tile are requested now, so
  // that the rest of the set-up runs in the shadow of these (cold) loads -------------------
  if constexpr (FUSE != 0) {
    if (warp < kCW && rot_job0 < rot_jobs) {
      const int j0 = rot_job0 < rot_half ? rot_job0 : rot_job0 - rot_half;
      const int seq = j0 / q_tiles, r = j0 - seq * q_tiles;
      rot_len = p.seq_lens[seq];
      rotate_q_tile_load<D, TQ>(rot_op, static_cast<const TQ*>(p.q_src),
                                rot_job0 < rot_half ? p.rotation : p.qjl, p.hq, seq,
                                r % m_tiles, r / m_tiles, lane);
    }
    // first touch of the other buffers: address translation is warm when they are needed
    if (tid == 64) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.block_table));
    if (tid == 65) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.q_count));
    if (tid == 66) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.q_rot_w));
  }
  if (warp == 1)
    stage_centroids(smem + p.off_cent, cent_val, p.nck, p.ncv,
                    p.status + kScaleCacheOffset / 4, lane);
  if (warp == 0)
    build_page_prefix(p.seq_lens, p.num_seqs, p.block_size, p.max_pages,
                      blockIdx.x == 0 ? p.status : nullptr, prefix, lane);
  __syncthreads();

  // ---- phase a: one rotated query tile per warp of the grid (before the warps change their
  // register budgets: the tile needs few registers and the counters should go out early) ----
  if constexpr (FUSE != 0) {
    if (warp < kCW)
    for (int job = rot_job0; job < rot_jobs; job += gridDim.x * kCW) {
      const bool by_pi = job < rot_half;
      const int j0 = by_pi ? job : job - rot_half;
      const int seq = j0 / q_tiles, r = j0 - seq * q_tiles;
      if (job != rot_job0) {
        rot_len = p.seq_lens[seq];
        rotate_q_tile_load<D, TQ>(rot_op, static_cast<const TQ*>(p.q_src),
                                  by_pi ? p.rotation : p.qjl, p.hq, seq, r % m_tiles, r / m_tiles,
                                  lane);
      }
      if (rot_len <= 0) continue;  // nobody reads the query of an empty sequence
      // q Pi^T is rounded to the query's type as the reference does; q S^T is not
      if (by_pi)
        rotate_q_tile_finish<D, TQ>(rot_op, p.q_rot_w, p.hq, seq, r % m_tiles, r / m_tiles, lane);
      else
        rotate_q_tile_finish<D, TQ, false>(rot_op, p.qs_w, p.hq, seq, r % m_tiles, r / m_tiles,
                                           lane);
      __syncwarp();
      if (lane == 0) red_release_add(p.q_count + seq, 1u);
    }
  }

  // ---- the flat page list and its cut into runs ---------------------------------------------
  const int64_t total = prefix[p.num_seqs];
  const int64_t workers = int64_t(gridDim.x) * teams;
  const int64_t active = total < workers ? total : workers;

  // ------------------------------------------------------------------------------------------
  // Producer warp: lane l feeds team l.  It owns everything that is not arithmetic on codes:
  // the page descriptors (32 at a time per team, all lanes together), the bulk copies of the
  // pages into the team's ring as stages come free, and the copy of the rotated query when a
  // new sequence starts.  It keeps 24 registers and hands the rest of its share to the
  // compute warps.
  // ------------------------------------------------------------------------------------------
  if (warp >= kCW) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 24;");
    if (warp > kCW) return;
    const bool has_team = lane < teams;
    const int64_t my_wk = int64_t(blockIdx.x) * teams + lane;
    int64_t my_f0 = 0;
    int my_run = 0;
    if (has_team && my_wk < active) {
      my_f0 = total * my_wk / active;
      my_run = int(total * (my_wk + 1) / active - my_f0);
    }
    uint64_t* my_full = reinterpret_cast<uint64_t*>(smem + p.off_bar) + lane * (2 * stages + 2);
    uint64_t* my_empty = my_full + stages;
    uint64_t* my_qfull = my_empty + stages;
    uint64_t* my_qempty = my_qfull + 1;
    const int4* my_desc = reinterpret_cast<const int4*>(smem + p.off_desc) + lane * kDescRing;
    const uint32_t my_ring = p.off_ring + uint32_t(lane) * stages * stage_bytes;
    const uint32_t my_q = p.off_q + uint32_t(lane) * qbuf_bytes;
    int produced = 0, issue_idx = 0, issue_stage = 0, issue_phase = 1, q_issued = 0, q_owed = -1;
    const uint64_t stream_policy = l2_evict_first_policy();  // pages are read once
    // descriptor of run page i of team T
    auto describe = [&](int T, int i, int n_run, int64_t f0) {
      const int64_t wk = int64_t(blockIdx.x) * teams + T;
      int4* ring = reinterpret_cast<int4*>(smem + p.off_desc) + T * kDescRing;
      const int64_t f = f0 + i;
      int lo = 0, hi = p.num_seqs - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (prefix[mid] <= f) lo = mid; else hi = mid - 1;
      }
      const int seq = lo;
      const int p0 = prefix[seq], n_pages = prefix[seq + 1] - p0;
      const int pg = int(f - p0);
      const int pps = (n_pages + p.num_splits - 1) / p.num_splits;
      const int s = pg / pps;
      int split_end = (s + 1) * pps;
      if (split_end > n_pages) split_end = n_pages;
      const bool seg_first = (pg == s * pps) || (i == 0);
      const bool seg_last = (pg + 1 == split_end) || (i + 1 == n_run);
      const bool q_new = (i == 0) || (pg == 0);
      int64_t phys = p.block_table[int64_t(seq) * p.bt_stride + pg];
      if (phys < 0 || phys >= p.num_blocks) {
        atomicOr(p.status, FQ_DEV_BAD_BLOCK_INDEX);
        phys = 0;
      }
      int n_valid = p.seq_lens[seq] - pg * p.block_size;  // pg < max_pages: see the prefix
      if (n_valid > p.block_size) n_valid = p.block_size;
      const int flags =
          (seg_first ? kSegStart : 0) | (seg_last ? kSegEnd : 0) | (q_new ? kQNew : 0);
      ring[i & (kDescRing - 1)] =
          make_int4(int(phys), n_valid | (flags << 8), seq, seq * p.num_splits + s + int(wk));
    };
    bool first_round = true;
    uint64_t idle_since = 0;
#pragma unroll 1
    while (true) {
      // ---- descriptors of run pages [base, base + 32) of team T: x = physical page, y = valid
      // tokens | flags << 8, z = sequence, w = partial-row slot.  A chunk is written when fewer
      // than 16 described pages are left to issue; the ring slots it overwrites held pages
      // more than 16 behind the issue front, which every warp of the team has left (a warp is
      // never more than `stages` <= 16 pages behind it).
      if (first_round || teams > 4) {
        // All teams at once, 32 / teams pages each: every team's block-table reads are in flight
        // at the same time.  The very first descriptors always come this way; with many small
        // teams (few KV heads) every later chunk does too - one team after the other, each
        // waiting for its own reads, left the last of sixteen teams without pages for a dozen
        // microseconds.
        const int per = 32 / teams, T = lane / per, i = lane - T * per;
        const int base = first_round ? 0 : __shfl_sync(0xffffffffu, produced, T);
        const int iss = first_round ? 0 : __shfl_sync(0xffffffffu, issue_idx, T);
        const int n_run = __shfl_sync(0xffffffffu, my_run, T);
        const int64_t f0 = __shfl_sync(0xffffffffu, my_f0, T);
        const bool need = base < n_run && base - iss < 16;
        // two pages per lane and round once the first descriptors are out (they go first so
        // that the first copies start as early as possible)
        const int each = first_round ? 1 : 2;
        for (int k = 0; k < each; ++k)
          if (need && base + k * per + i < n_run) describe(T, base + k * per + i, n_run, f0);
        __syncwarp();
        const bool mine = __shfl_sync(0xffffffffu, int(need), (lane * per) & 31) != 0;
        if (has_team && mine) produced += each * per;
        first_round = false;
      } else {
#pragma unroll 1
        for (int T = 0; T < teams; ++T) {
          const int base = __shfl_sync(0xffffffffu, produced, T);
          const int iss = __shfl_sync(0xffffffffu, issue_idx, T);
          const int n_run = __shfl_sync(0xffffffffu, my_run, T);
          if (base >= n_run || base - iss >= 16) continue;
          const int64_t f0 = __shfl_sync(0xffffffffu, my_f0, T);
          if (base + lane < n_run) describe(T, base + lane, n_run, f0);
          __syncwarp();
          if (lane == T) produced += 32;
        }
      }

      // ---- this lane's team: issue every described page whose stage is free ---------------------
      bool progress = false;
      if (my_run > 0) {
        const int limit = produced < my_run ? produced : my_run;
        while (issue_idx < limit) {
          if (issue_idx >= stages && !mbar_test_wait(my_empty + issue_stage, issue_phase)) break;
          const int4 d = my_desc[issue_idx & (kDescRing - 1)];
          if ((d.y >> 8) & kQNew) {
            if (q_owed >= 0) break;  // the previous query copy has not gone out yet
            q_owed = d.z;
          }
          mbar_expect_tx(my_full + issue_stage, stage_bytes);
          bulk_g2s_hint(smem + my_ring + uint32_t(issue_stage) * stage_bytes,
                        p.kv_cache + int64_t(d.x) * int64_t(page_bytes), page_bytes,
                        my_full + issue_stage, stream_policy);
          if constexpr (QS)
            bulk_g2s_hint(smem + my_ring + uint32_t(issue_stage) * stage_bytes + page_bytes,
                          p.kq_cache + int64_t(d.x) * int64_t(qpage_bytes), qpage_bytes,
                          my_full + issue_stage, stream_policy);
          ++issue_idx;
          if (++issue_stage == stages) { issue_stage = 0; issue_phase ^= 1; }
          progress = true;
        }
        // the query copy waits for its buffer and, in the single-launch form, for the rotated
        // rows (written by other CTAs' stores, read here by a bulk copy)
        if (q_owed >= 0 && (q_issued == 0 || mbar_test_wait(my_qempty, (q_issued - 1) & 1))) {
          bool rows_there = true;
          if constexpr (FUSE != 0) {
            rows_there = ld_acquire_u32(p.q_count + q_owed) >= q_target;
            if (rows_there) fence_proxy_async();
          }
          if (rows_there) {
            mbar_expect_tx(my_qfull, qbuf_bytes);
            bulk_g2s(smem + my_q, p.q_rot + int64_t(q_owed) * p.hq * D, q_bytes, my_qfull);
            if constexpr (QS)
              bulk_g2s(smem + my_q + q_bytes, p.qs_w + int64_t(q_owed) * p.hq * D, q_bytes,
                       my_qfull);
            ++q_issued;
            q_owed = -1;
            progress = true;
          }
        }
      }
      const bool done = issue_idx >= my_run && q_owed < 0;
      if (__all_sync(0xffffffffu, done)) break;
      if (__any_sync(0xffffffffu, progress)) {
        idle_since = 0;
      } else {
        __nanosleep(32);
        // lane 0 keeps the time, every lane leaves with it
        bool late = false;
        if (lane == 0) {
          const uint64_t now = global_timer_ns();
          if (idle_since == 0) idle_since = now;
          late = now - idle_since > p.wait_ns;
        }
        if (__shfl_sync(0xffffffffu, int(late), 0)) {
          if (lane == 0) atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
          break;
        }
      }
    }
    return;
  }
  asm volatile("setmaxnreg.inc.sync.aligned.u32 112;");

  // ---- compute warps: this team's run ---------------------------------------------------------
  const int64_t wk = int64_t(blockIdx.x) * teams + team;
  const int n_run = wk < active ? int(total * (wk + 1) / active - total * wk / active) : 0;

  // ---- scaled fp16 centroid tables, then the look-up table -------------------------------------
  scale_centroid_tables(smem + p.off_cent, p.nck, p.ncv, tid,
                        blockIdx.x == 0 ? p.status + kScaleCacheOffset / 4 : nullptr);
  const float beta_k = reinterpret_cast<const float*>(smem + p.off_cent + 192)[0];
  const float beta_v = reinterpret_cast<const float*>(smem + p.off_cent + 192)[1];
  const float k_scale_log2 = p.scale_log2 * beta_k;  // the key table is c / beta_k
  for (int i = tid; i < 256 * 32; i += kComputeThreads) {
    const int e = i >> 5, l = i & 31;
    const uint32_t hi = e >> 4, lo = e & 15;
    // K entry: byte of one token -> (even coordinate, odd coordinate)
    // V entry: (code of token 2t+1) << 4 | (code of token 2t) -> (token 2t, token 2t+1)
    *reinterpret_cast<uint32_t*>(smem + e * kLutStride + l * 4) =
        KPRMT ? uint32_t(cs[lo]) | (uint32_t(cs[hi]) << 16)
              : uint32_t(cs[hi]) | (uint32_t(cs[lo]) << 16);
    *reinterpret_cast<uint32_t*>(smem + e * kLutStride + 128 + l * 4) =
        uint32_t(cs[16 + lo]) | (uint32_t(cs[16 + hi]) << 16);
  }

  compute_sync();  // the table is complete
  if (n_run > 0) {  // ---- phase b ----------------------------------------------------------

  // ---- per-warp constants -------------------------------------------------------------------
  const uint32_t lane4 = uint32_t(lane) * 4;
  const bool wide = (p.hkv & 1) == 0;  // 16-byte row alignment needs an even head count
  const uint32_t k_code_off = head * half_d;
  const uint32_t k_norm_off = p.hkv * half_d + 4 * head;
  const uint32_t v_code_off = p.hkv * half_d + 4 * p.hkv + head * half_d;
  const uint32_t v_norm_off = 2 * p.hkv * half_d + 4 * p.hkv + 4 * head;
  const int units_per_page = p.block_size >> 4;

  // 8-entry K table in registers (K by byte permute): low and high bytes of the fp16 values
  uint32_t tl0 = 0, tl1 = 0, th0 = 0, th1 = 0;
  if constexpr (KPRMT) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t h = cs[i];
      const uint32_t lo8 = (h & 0xffu) << (8 * (i & 3)), hi8 = (h >> 8) << (8 * (i & 3));
      if (i < 4) { tl0 |= lo8; th0 |= hi8; } else { tl1 |= lo8; th1 |= hi8; }
    }
  }

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

  int stage = 0, fphase = 0, qcnt = 0;
  bool timed_out = false, page_ready = false;
#pragma unroll 1
  for (int it = 0; it < n_run; ++it) {
    // ---- wait for the page ----------------------------------------------------------------
    if (!page_ready && !mbar_wait(full_bar + stage, fphase, p.wait_ns)) {
      timed_out = true;
      break;
    }
    // a look at the next page's barrier goes out now and is read at the top of the next
    // iteration (it never suspends the warp: the page may well still be on its way)
    {
      int ns = stage + 1, nph = fphase;
      if (ns == stages) { ns = 0; nph ^= 1; }
      page_ready = (it + 1 < n_run) && mbar_test_wait(full_bar + ns, nph);
    }
    const int4 d = desc_ring[it & (kDescRing - 1)];
    const int n_valid = d.y & 0xff, flags = d.y >> 8;

    if (flags & kSegStart) {
      m_run[0] = m_run[1] = -INFINITY;
      l_run[0] = l_run[1] = 0.f;
#pragma unroll
      for (int j = 0; j < KS; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) oacc[j][c] = 0.f;
      if (flags & kQNew) {
        if (!mbar_wait(qfull_bar, qcnt & 1, p.wait_ns)) {
          timed_out = true;
          break;
        }
        // lane (g,t), k-step s: coordinates of cache bytes (D/8)t + 2s, +1 of q head head*G+g
        const bool valid = g < group;
        const uint32_t qoff =
            q_off + uint32_t(head * group + (valid ? g : 0)) * D * 2 + (D / 8) * t * 4;
#pragma unroll
        for (int s = 0; s < KS; ++s) {
          uint2 v = *reinterpret_cast<const uint2*>(smem + qoff + 8 * s);
          if constexpr (KPRMT) {  // the byte-permute path delivers (odd, even) pairs
            v.x = prmt(v.x, v.x, 0x1032);
            v.y = prmt(v.y, v.y, 0x1032);
          }
          qf[s][0] = valid ? v.x : 0u;
          qf[s][1] = valid ? v.y : 0u;
        }
        // the loads must have delivered before the buffer goes back to the producer: a load in
        // flight is not ordered before the arrive by anything else
        __threadfence_block();
        __syncwarp();
        if (lane == 0) mbar_arrive(qempty_bar);
        ++qcnt;
      }
    }

    const uint32_t page_off = ring_off + uint32_t(stage) * stage_bytes;
    for (int u = 0; u < units_per_page; ++u) {
      const int tok0 = u * 16;
      if (tok0 >= n_valid) break;
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
      const float nk_lo = *reinterpret_cast<const float*>(smem + r_lo + k_norm_off);
      const float nk_hi = *reinterpret_cast<const float*>(smem + r_hi + k_norm_off);
      const float nv_lo = *reinterpret_cast<const float*>(smem + r_lo + v_norm_off);
      const float nv_hi = *reinterpret_cast<const float*>(smem + r_hi + v_norm_off);

      float sacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int w = 0; w < KW; ++w) {
        // word w of the lane's chunk = cache bytes 4w..4w+3 = k-steps 2w (bytes 0,1), 2w+1
        uint32_t a[2][4];
        if (KPRMT && !(kMixKeyLookups && (w & 1))) {
#pragma unroll
          for (int hw = 0; hw < 2; ++hw) {
            const uint32_t sa = hw ? (ka[w] >> 16) : ka[w], sb = hw ? (kb[w] >> 16) : kb[w];
            const uint32_t la = prmt(tl0, tl1, sa), ha = prmt(th0, th1, sa);
            const uint32_t lb = prmt(tl0, tl1, sb), hb = prmt(th0, th1, sb);
            a[hw][0] = prmt(la, ha, 0x5140);  // row g, first byte: (odd, even) coordinate
            a[hw][1] = prmt(lb, hb, 0x5140);  // row g+8
            a[hw][2] = prmt(la, ha, 0x7362);  // row g, second byte
            a[hw][3] = prmt(lb, hb, 0x7362);
          }
        } else {
          a[0][0] = lds_u32(smem, lut_addr<0>(ka[w], lane4));
          a[0][1] = lds_u32(smem, lut_addr<0>(kb[w], lane4));
          a[0][2] = lds_u32(smem, lut_addr<1>(ka[w], lane4));
          a[0][3] = lds_u32(smem, lut_addr<1>(kb[w], lane4));
          a[1][0] = lds_u32(smem, lut_addr<2>(ka[w], lane4));
          a[1][1] = lds_u32(smem, lut_addr<2>(kb[w], lane4));
          a[1][2] = lds_u32(smem, lut_addr<3>(ka[w], lane4));
          a[1][3] = lds_u32(smem, lut_addr<3>(kb[w], lane4));
        }
        mma_f16(sacc[0], a[0][0], a[0][1], a[0][2], a[0][3], qf[2 * w][0], qf[2 * w][1]);
        mma_f16(sacc[1], a[1][0], a[1][1], a[1][2], a[1][3], qf[2 * w + 1][0], qf[2 * w + 1][1]);
      }

      // ---------- two-stage estimator: C^T = signs (q S^T)^T, one more 16 x 8 product ---------
      // lane (g,t) takes sign word t of the head (coordinates 32t .. 32t+31) of tokens g and
      // g+8 and spends bits 4s .. 4s+3 on k-step s; the fragment of q S^T follows the same
      // order (8 consecutive bytes of the row per k-step)
      [[maybe_unused]] float cacc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      [[maybe_unused]] float gs_lo = 0.f, gs_hi = 0.f;
      if constexpr (QS) {
        const uint32_t prow = page_off + page_bytes + uint32_t(tok0 + g) * qrow_bytes;
        const uint32_t xa = ~lds_u32(smem, prow + uint32_t(head) * (D / 8) + 4 * t);
        const uint32_t xb = ~lds_u32(smem, prow + 8 * qrow_bytes + uint32_t(head) * (D / 8) + 4 * t);
        gs_lo = *reinterpret_cast<const float*>(smem + prow + p.hkv * (D / 8) + 4 * head) *
                p.corr_scale_log2;
        gs_hi = *reinterpret_cast<const float*>(smem + prow + 8 * qrow_bytes + p.hkv * (D / 8) +
                                                4 * head) * p.corr_scale_log2;
        const bool valid = g < group;
        const uint32_t qs_off =
            q_off + q_bytes + uint32_t(head * group + (valid ? g : 0)) * D * 2 + 64 * t;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          uint2 b = *reinterpret_cast<const uint2*>(smem + qs_off + 8 * ks);
          if (!valid) b = make_uint2(0u, 0u);
          mma_f16(cacc[ks & 1], sign_pair(xa, 4 * ks), sign_pair(xb, 4 * ks),
                  sign_pair(xa, 4 * ks + 2), sign_pair(xb, 4 * ks + 2), b.x, b.y);
        }
      }

      // ---------- online softmax in the accumulator layout ---------------------------------
      const bool ok_lo = tok0 + g < n_valid, ok_hi = tok0 + g + 8 < n_valid;
      // log2 of the value norm is folded into the exponent so that the fp16 weights stay in
      // range whatever the norms are; the running reference clamps it below so that l
      // cannot overflow
      const float lg_lo = fast_log2(nv_lo), lg_hi = fast_log2(nv_hi);
      const float lv_lo = fmaxf(lg_lo, -40.f), lv_hi = fmaxf(lg_hi, -40.f);
      const float ks_lo = nk_lo * k_scale_log2, ks_hi = nk_hi * k_scale_log2;
      float s_lo[2], s_hi[2], mx[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        s_lo[c] = (sacc[0][c] + sacc[1][c]) * ks_lo;
        s_hi[c] = (sacc[0][2 + c] + sacc[1][2 + c]) * ks_hi;
        if constexpr (QS) {
          s_lo[c] = fmaf(cacc[0][c] + cacc[1][c], gs_lo, s_lo[c]);
          s_hi[c] = fmaf(cacc[0][2 + c] + cacc[1][2 + c], gs_hi, s_hi[c]);
        }
        mx[c] = fmaxf(ok_lo ? s_lo[c] + lv_lo : -INFINITY, ok_hi ? s_hi[c] + lv_hi : -INFINITY);
      }
      // The reference exponent m only has to stay within kMaxSlack bits of the true running
      // maximum (the weights then stay below 2^(kMaxSlack + kPScaleLog2) <= 2^14 in fp16), so
      // the reduction over the 16 tokens and the rescaling run only when some lane's scores
      // outgrow it by more than that - rarely, once the first tokens of a segment are in
      const bool grew = (mx[0] > m_run[0] + kMaxSlack) || (mx[1] > m_run[1] + kMaxSlack);
      if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          mx[0] = fmaxf(mx[0], __shfl_xor_sync(0xffffffffu, mx[0], o));
          mx[1] = fmaxf(mx[1], __shfl_xor_sync(0xffffffffu, mx[1], o));
        }
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
      // the weight that meets the value codes carries the value norm and the fp16 scale;
      // m >= s + max(lg2 n_v, -40) - kMaxSlack, so p * n_v <= 2^kMaxSlack and p <= 2^46
      constexpr float kPScale = float(1 << int(kPScaleLog2));
      const float vs_lo = nv_lo * kPScale, vs_hi = nv_hi * kPScale;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const float mref = (m_run[c] == -INFINITY) ? 0.f : m_run[c];
        const float p_lo = ok_lo ? fast_exp2(s_lo[c] - mref) : 0.f;
        const float p_hi = ok_hi ? fast_exp2(s_hi[c] - mref) : 0.f;
        w_lo[c] = p_lo * vs_lo;
        w_hi[c] = p_hi * vs_hi;
        l_run[c] += p_lo + p_hi;
      }
      // weights as the B operand of the PV product: transpose (token, head) -> (head, token)
      const uint32_t pb0 = movmatrix_trans(pack_half2(w_lo[0], w_lo[1]));
      const uint32_t pb1 = movmatrix_trans(pack_half2(w_hi[0], w_hi[1]));

      // ---------- O^T += V^T P^T : rows = value coordinates, cols = q heads ------------------
      // lane (g,t) takes the codes of tokens 2t, 2t+1 (and 2t+8, 2t+9), cache bytes
      // VB*g .. VB*g+VB-1, and pairs equal nibbles of the two tokens into one table index
      const uint32_t vbase = rows + v_code_off + VB * g + uint32_t(2 * t) * row_bytes;
#pragma unroll
      for (int w = 0; w < VW; ++w) {
        uint32_t c0, c1, c2, c3;  // tokens 2t, 2t+1, 2t+8, 2t+9
        if constexpr (VB == 8) {
          if (wide) {
            // both words of a row come with one 8-byte load
            const uint2 x0 = *reinterpret_cast<const uint2*>(smem + vbase);
            const uint2 x1 = *reinterpret_cast<const uint2*>(smem + vbase + row_bytes);
            const uint2 x2 = *reinterpret_cast<const uint2*>(smem + vbase + 8 * row_bytes);
            const uint2 x3 = *reinterpret_cast<const uint2*>(smem + vbase + 9 * row_bytes);
            c0 = w ? x0.y : x0.x; c1 = w ? x1.y : x1.x;
            c2 = w ? x2.y : x2.x; c3 = w ? x3.y : x3.x;
          } else {
            c0 = lds_u32(smem, vbase + 4 * w);
            c1 = lds_u32(smem, vbase + row_bytes + 4 * w);
            c2 = lds_u32(smem, vbase + 8 * row_bytes + 4 * w);
            c3 = lds_u32(smem, vbase + 9 * row_bytes + 4 * w);
          }
        } else {
          c0 = lds_u32(smem, vbase);
          c1 = lds_u32(smem, vbase + row_bytes);
          c2 = lds_u32(smem, vbase + 8 * row_bytes);
          c3 = lds_u32(smem, vbase + 9 * row_bytes);
        }
        // even coordinates sit in the high nibbles, odd ones in the low nibbles
        const uint32_t ev01 = ((c0 >> 4) & 0x0f0f0f0fu) | (c1 & 0xf0f0f0f0u);
        const uint32_t od01 = (c0 & 0x0f0f0f0fu) | ((c1 << 4) & 0xf0f0f0f0u);
        const uint32_t ev23 = ((c2 >> 4) & 0x0f0f0f0fu) | (c3 & 0xf0f0f0f0u);
        const uint32_t od23 = (c2 & 0x0f0f0f0fu) | ((c3 << 4) & 0xf0f0f0f0u);
#define FQ_PV_STEP(I)                                                                   \
  if (4 * w + I < VB) {                                                                 \
    const uint32_t a0 = lds_u32(smem, lut_addr<I>(ev01, lane4) + 128);                  \
    const uint32_t a1 = lds_u32(smem, lut_addr<I>(od01, lane4) + 128);                  \
    const uint32_t a2 = lds_u32(smem, lut_addr<I>(ev23, lane4) + 128);                  \
    const uint32_t a3 = lds_u32(smem, lut_addr<I>(od23, lane4) + 128);                  \
    mma_f16(oacc[4 * w + I], a0, a1, a2, a3, pb0, pb1);                                 \
  }
        FQ_PV_STEP(0)
        FQ_PV_STEP(1)
        FQ_PV_STEP(2)
        FQ_PV_STEP(3)
#undef FQ_PV_STEP
      }
    }

    if (flags & kSegEnd) {
      // ---- this warp's partial rows of the segment --------------------------------------------
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], o);
        l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], o);
      }
      const float unscale = beta_v / float(1 << int(kPScaleLog2));  // the value table is c / beta_v
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int col = 2 * t + c;
        if (col >= group) continue;
        float* row = p.slots + (int64_t(d.w) * p.hq + head * group + col) * ROWF;
#pragma unroll
        for (int j = 0; j < KS; ++j) {
          const int b = VB * g + j;  // cache byte -> coordinates 2b (row g), 2b+1 (row g+8)
          *reinterpret_cast<float2*>(row + 2 * b) =
              make_float2(oacc[j][c] * unscale, oacc[j][2 + c] * unscale);
        }
        if (g == 0) *reinterpret_cast<float4*>(row + D) = make_float4(m_run[c], l_run[c], 0.f, 0.f);
      }
      if constexpr (FUSE != 0) {
        __syncwarp();
        if (lane == 0) red_release_add(p.seg_count + d.z, 1u);
      }
    }

    __threadfence_block();  // as for the query buffer: loads from the stage delivered, then release
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar + stage);
    if (++stage == stages) { stage = 0; fphase ^= 1; }
  }
  if (timed_out && lane == 0) atomicOr(p.status, FQ_DEV_WAIT_TIMEOUT);
  }  // phase b

  if constexpr (FUSE != 0) {
    fused_merge<D, TQ>(p, smem, prefix, total, active, teams, stages);
  }
}

}  // namespace fq
#include "paged_decode_fast.cuh"
namespace fq {

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
  int num_workers; // kFromSlots: teams of the streaming kernel (grid size x teams per CTA)
  const int32_t* seq_lens;
  int block_size;
  int max_pages;   // kFromSlots: the same cut of over-long sequences as the streaming kernel
  const float* rotation;
  void* out;
  float* row_out;
  int num_seqs, hq;
};

template <int D, typename T, bool kFromSlots, bool kFinal>
__global__ void __launch_bounds__(kMergeHeads* D) merge_rotate_kernel(MergeArgs p) {
  constexpr int ROWF = D + kPartPad;
  constexpr int NT = kMergeHeads * D;
  extern __shared__ __align__(16) unsigned char msm[];
  float* pi_s = reinterpret_cast<float*>(msm);                  // [k][j] (kFinal only)
  float* o_s = pi_s + (kFinal ? D * D : 0);                     // [8][D]
  float* w_s = o_s + kMergeHeads * D;                           // [chunk][8]: m, then weight
  float* l_s = w_s + kPartChunk * kMergeHeads;                  // [chunk][8]
  float* den_s = l_s + kPartChunk * kMergeHeads;                // [8] den, [8] m*, [8] alpha
  int* part_row = reinterpret_cast<int*>(den_s + 3 * kMergeHeads);  // [parts]
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
      build_page_prefix(p.seq_lens, p.num_seqs, p.block_size, p.max_pages, nullptr, prefix, lane);
      if (lane == 0) {
        const int64_t total = prefix[p.num_seqs];
        const int64_t active = total < p.num_workers ? total : int64_t(p.num_workers);
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

  // ---- online merge over chunks of partial rows; thread (hh, d) owns one output value ------
  const int d = tid % D, hh = tid / D;
  const bool head_ok = h0 + hh < p.hq;
  float num = 0.f;
  if (tid < kMergeHeads) {
    den_s[tid] = 0.f;
    den_s[kMergeHeads + tid] = -INFINITY;
  }
  for (int c0 = 0; c0 < n_parts; c0 += kPartChunk) {
    const int nc = n_parts - c0 < kPartChunk ? n_parts - c0 : kPartChunk;
    __syncthreads();  // previous chunk's weights are no longer read
    for (int i = tid; i < nc * kMergeHeads; i += NT) {
      const int part = c0 + i / kMergeHeads, h = i % kMergeHeads;
      float m = -INFINITY, l = 0.f;
      if (h0 + h < p.hq) {
        const float2 ml = *reinterpret_cast<const float2*>(row_ptr(part, h0 + h) + D);
        m = ml.x;
        l = ml.y;
      }
      w_s[i] = m;
      l_s[i] = l;
    }
    __syncthreads();
    if (tid < kMergeHeads) {
      const float m_old = den_s[kMergeHeads + tid];
      float m_new = m_old;
      for (int i = 0; i < nc; ++i) m_new = fmaxf(m_new, w_s[i * kMergeHeads + tid]);
      const float alpha = (m_old == -INFINITY) ? 0.f : exp2f(m_old - m_new);
      float den = den_s[tid] * alpha;
      for (int i = 0; i < nc; ++i) {
        const float m = w_s[i * kMergeHeads + tid];
        const float w = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
        w_s[i * kMergeHeads + tid] = w;
        den = fmaf(w, l_s[i * kMergeHeads + tid], den);
      }
      den_s[tid] = den;
      den_s[kMergeHeads + tid] = m_new;
      den_s[2 * kMergeHeads + tid] = alpha;
    }
    __syncthreads();
    if (head_ok) {
      num *= den_s[2 * kMergeHeads + hh];
      for (int i0 = 0; i0 < nc; i0 += 8) {
        float v[8];
#pragma unroll
        for (int x = 0; x < 8; ++x)
          v[x] = (i0 + x < nc) ? row_ptr(c0 + i0 + x, h0 + hh)[d] : 0.f;
#pragma unroll
        for (int x = 0; x < 8; ++x)
          if (i0 + x < nc) num = fmaf(w_s[(i0 + x) * kMergeHeads + hh], v[x], num);
      }
    }
  }
  __syncthreads();

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

// status word at 0; three counter arrays of kMaxSeqs words (single-launch form) at 256;
// the rotated query; the partial rows
struct WorkspaceLayout {
  size_t count_off, q_rot_off, slots_off, chunk_off, total;
  int merge_chunks;
};

static size_t up256(size_t v) { return (v + 255) / 256 * 256; }

// `splits` <= 0 sizes for the largest split count
// Chunks that the single-launch merge cuts the rows of a (sequence, head group) into: a
// sequence has about its share of the teams plus a row per split boundary.
// Never more chunk jobs than CTAs (`ctas`; a job is a CTA's work): a second round of jobs would
// cost more than the shorter chunks save.
static int merge_chunks_for(int num_seqs, int hq, int splits, int workers, int ctas) {
  const int hgroups = (hq + kMergeHeads - 1) / kMergeHeads;
  if (num_seqs <= 0 || int64_t(num_seqs) * hgroups > kMaxChunkJobs) return 1;
  const int64_t rows = (int64_t(workers) + int64_t(num_seqs) * splits) / num_seqs + 1;
  int64_t c = (rows + kRowsPerMergeChunk - 1) / kRowsPerMergeChunk;
  const int64_t fit = int64_t(ctas) / (int64_t(num_seqs) * hgroups);
  c = c > fit ? fit : c;
  return c < 1 ? 1 : (c > kMaxMergeChunks ? kMaxMergeChunks : int(c));
}

static WorkspaceLayout workspace_layout(int num_seqs, int hq, int d, int splits, int workers,
                                        int grid = 192) {
  if (splits <= 0) splits = kMaxSplits;
  const int ctas = workers;
  WorkspaceLayout w;
  w.count_off = 256;
  // three counters per sequence, then one per (sequence, head group) of a chunked merge
  w.q_rot_off = up256(w.count_off + (3 * size_t(kMaxSeqs) + kMaxChunkJobs) * sizeof(uint32_t));
  // room for fp16(q Pi^T) and, behind it, fp16(q S^T) of the two-stage estimator
  w.slots_off = up256(w.q_rot_off + 2 * size_t(num_seqs) * hq * d * sizeof(__half));
  w.chunk_off = up256(w.slots_off +
                      (size_t(num_seqs) * splits + ctas) * hq * (d + kPartPad) * sizeof(float));
  w.merge_chunks = merge_chunks_for(num_seqs, hq, splits, workers, grid);
  const size_t hgroups = size_t(hq + kMergeHeads - 1) / kMergeHeads;
  w.total = w.merge_chunks > 1
                ? up256(w.chunk_off + size_t(num_seqs) * hgroups * w.merge_chunks * kMergeHeads *
                                          (d + kPartPad) * sizeof(float))
                : w.chunk_off;
  return w;
}

// The flat page list is balanced over the SMs whatever the split count is; more splits
// only add partial rows, so one split per sequence is the automatic choice.
static int auto_splits() { return 1; }

constexpr int kCoopRefused = 1001;  // internal: the single-launch form could not be launched

// 1: fq_split_k_paged_decode uses the single cooperative launch (default); 0: three launches
static std::atomic<int> g_single_launch{1};

struct SmemPlan {
  int stages;  // per team
  uint32_t off_ring, off_q, off_prefix, off_desc, off_bar, off_cent, total;
};

// `qs`: stages also hold the page of the QJL side plane, query buffers also hold q S^T
static SmemPlan plan_smem(int num_seqs, int hq, int hkv, int d, int block_size, bool qs = false) {
  SmemPlan s{};
  const uint32_t teams = uint32_t(kCW / hkv);
  const uint32_t page_bytes =
      uint32_t(block_size) * hkv * (d + 8) + (qs ? uint32_t(block_size) * hkv * (d / 8 + 4) : 0u);
  auto up16 = [](uint32_t v) { return (v + 15u) & ~15u; };
  const uint32_t q_all = teams * up16(uint32_t(hq) * d * 2) * (qs ? 2u : 1u);
  const uint32_t prefix = up16(uint32_t(num_seqs + 1) * 4);
  const uint32_t desc = teams * kDescRing * 16;
  const uint32_t fixed = kLutBytes + q_all + prefix + desc + teams * 16 + 96 + kCentBytes;
  const uint32_t budget = 227 * 1024 - 512;
  int stages = 0;
  if (budget > fixed) stages = int((budget - fixed) / (teams * (page_bytes + 16)));
  if (stages > kMaxStages) stages = kMaxStages;
  s.stages = stages;
  s.off_ring = kLutBytes;
  s.off_q = s.off_ring + teams * uint32_t(stages < 0 ? 0 : stages) * page_bytes;
  s.off_prefix = s.off_q + q_all;
  s.off_desc = s.off_prefix + prefix;
  s.off_bar = s.off_desc + desc;
  s.off_cent = up16(s.off_bar + teams * (2 * uint32_t(stages) + 2) * 8 + 8);  // + merge barrier
  s.total = s.off_cent + kCentBytes;
  return s;
}

template <int D, bool KPRMT, int FUSE>
static int launch_stream_t(DecodeArgs& a, const SmemPlan& sp, int ctas, cudaStream_t stream) {
  auto kern = paged_decode_kernel<D, KPRMT, FUSE>;
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
  a.off_ring = sp.off_ring; a.off_q = sp.off_q;
  a.off_prefix = sp.off_prefix; a.off_desc = sp.off_desc; a.off_bar = sp.off_bar;
  a.off_cent = sp.off_cent;
  if constexpr (FUSE == 0) {
    kern<<<ctas, kDecodeThreads, sp.total, stream>>>(a);
  } else {
    // CTAs wait for one another: all of them must be resident
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kDecodeThreads);
    cfg.dynamicSmemBytes = sp.total;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeCooperative;
    attr.val.cooperative = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
    if (e == cudaErrorCooperativeLaunchTooLarge || e == cudaErrorLaunchOutOfResources) {
      // the GPU cannot hold one CTA per SM of this launch right now (shared with other work,
      // partitioned): the caller falls back to the three-launch form
      cudaGetLastError();
      fail(FQ_ERR_CUDA, "paged decode: cooperative launch of %d CTAs refused: %s", ctas,
           cudaGetErrorString(e));
      return kCoopRefused;
    }
    if (e != cudaSuccess)
      return fail(FQ_ERR_CUDA, "paged decode: cooperative launch of %d CTAs failed: %s", ctas,
                  cudaGetErrorString(e));
  }
  return check_launch("paged decode kernel launch");
}

// ---- fast path (head_dim 128, 8 KV heads, pages of 16 tokens): padded rows, one producer warp
// per team ---------------------------------------------------------------------------------
static std::atomic<int> g_fast_path{1};      // 0: always the generic kernel
// test hook: the merge phase of the single launch expects this many segment arrivals more than
// will ever come, so that its bounded wait can be seen to give up
static std::atomic<int> g_test_extra_segments{0};
static std::atomic<int> g_weight_split{1};   // 1: two fp16 terms per softmax weight (default)

static bool fast_path_fits(int hq_rows, int n_q, int hkv, int head_dim, int block_size,
                           bool two_stage) {
  if (!g_fast_path.load(std::memory_order_relaxed) || two_stage) return false;
  if (head_dim != kFD || hkv != kFH || block_size != kFBS || n_q < 1 || hq_rows % n_q) return false;
  const int hq = hq_rows / n_q;
  return hq % hkv == 0 && (hq / hkv) * n_q <= 8;
}

static SmemPlan plan_smem_fast(int num_seqs, int hq_rows) {
  SmemPlan s{};
  auto up16 = [](uint32_t v) { return (v + 15u) & ~15u; };
  const uint32_t q_all = kFTeams * up16(uint32_t(hq_rows) * kFD * 2);
  const uint32_t prefix = up16(uint32_t(2 * num_seqs + 1) * 4);  // page prefix, then ranks
  const uint32_t desc = kFTeams * kFDescRing * 16;
  const uint32_t fixed = kLutBytes + q_all + prefix + desc + kFTeams * 16 + 96 + kCentBytes;
  const uint32_t budget = 227 * 1024 - 512;
  int stages = 0;
  if (budget > fixed) stages = int((budget - fixed) / (kFTeams * (kFStage + 16)));
  if (stages > kMaxStages) stages = kMaxStages;
  s.stages = stages;
  s.off_ring = kLutBytes;
  s.off_q = s.off_ring + kFTeams * uint32_t(stages < 0 ? 0 : stages) * kFStage;
  s.off_prefix = s.off_q + q_all;
  s.off_desc = s.off_prefix + prefix;
  s.off_bar = s.off_desc + desc;
  s.off_cent = up16(s.off_bar + kFTeams * (2 * uint32_t(stages) + 2) * 8 + 8);  // + merge barrier
  s.total = s.off_cent + kCentBytes;
  return s;
}

template <bool KPRMT, int FUSE, bool PSPLIT>
static int launch_fast_t(DecodeArgs& a, const SmemPlan& sp, int ctas, cudaStream_t stream) {
  auto kern = paged_decode_fast_kernel<KPRMT, FUSE, PSPLIT>;
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
  a.off_ring = sp.off_ring; a.off_q = sp.off_q;
  a.off_prefix = sp.off_prefix; a.off_desc = sp.off_desc; a.off_bar = sp.off_bar;
  a.off_cent = sp.off_cent;
  if constexpr (FUSE == 0) {
    kern<<<ctas, kDecodeThreads, sp.total, stream>>>(a);
  } else {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(ctas);
    cfg.blockDim = dim3(kDecodeThreads);
    cfg.dynamicSmemBytes = sp.total;
    cfg.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeCooperative;
    attr.val.cooperative = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
    if (e == cudaErrorCooperativeLaunchTooLarge || e == cudaErrorLaunchOutOfResources) {
      cudaGetLastError();
      fail(FQ_ERR_CUDA, "paged decode: cooperative launch of %d CTAs refused: %s", ctas,
           cudaGetErrorString(e));
      return kCoopRefused;
    }
    if (e != cudaSuccess)
      return fail(FQ_ERR_CUDA, "paged decode: cooperative launch of %d CTAs failed: %s", ctas,
                  cudaGetErrorString(e));
  }
  return check_launch("paged decode kernel launch");
}

template <int FUSE>
static int launch_fast(DecodeArgs& a, const SmemPlan& sp, int ctas, cudaStream_t stream) {
  const bool kprmt = a.nck <= 8;
  // two-term weights ride in the spare columns of the products: at most 4 columns in use
  const bool split = g_weight_split.load(std::memory_order_relaxed) != 0 &&
                     (a.hq / a.hkv) <= 4;
  if (kprmt)
    return split ? launch_fast_t<true, FUSE, true>(a, sp, ctas, stream)
                 : launch_fast_t<true, FUSE, false>(a, sp, ctas, stream);
  return split ? launch_fast_t<false, FUSE, true>(a, sp, ctas, stream)
               : launch_fast_t<false, FUSE, false>(a, sp, ctas, stream);
}

template <int FUSE>
static int launch_stream(DecodeArgs& a, const SmemPlan& sp, int ctas, int head_dim,
                         cudaStream_t stream) {
  const bool kprmt = a.nck <= 8;  // key codes fit a register-resident 8-entry table
  if (head_dim == 128)
    return kprmt ? launch_stream_t<128, true, FUSE>(a, sp, ctas, stream)
                 : launch_stream_t<128, false, FUSE>(a, sp, ctas, stream);
  if constexpr (FUSE >= 3) {
    return fail(FQ_ERR_UNSUPPORTED, "two-stage scoring is built for head_dim 128");
  } else {
    return kprmt ? launch_stream_t<64, true, FUSE>(a, sp, ctas, stream)
                 : launch_stream_t<64, false, FUSE>(a, sp, ctas, stream);
  }
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
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(rotate_q_kernel<D, float>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess)
      return fail(FQ_ERR_CUDA, "rotate_q: shared memory opt-in refused: %s",
                  cudaGetErrorString(e));
    set_dev = dev;
  }
  if (dtype == FQ_F32)
    rotate_q_kernel<D, float><<<grid, 256, smem, stream>>>(static_cast<const float*>(q), rotation,
                                                           out, rows);
  else if (dtype == FQ_BF16)
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
                      2 * kPartChunk * kMergeHeads * 4 + 3 * kMergeHeads * 4 + kMaxParts * 4 +
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
  if (dtype == FQ_F32)
    return head_dim == 128 ? launch_merge_t<128, float, kFromSlots, kFinal>(m, stream)
                           : launch_merge_t<64, float, kFromSlots, kFinal>(m, stream);
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
  FQ_REQUIRE(dtype == FQ_F16 || dtype == FQ_BF16 || dtype == FQ_F32, FQ_ERR_INVALID_ARGUMENT,
             "paged decode: unknown dtype");
  FQ_REQUIRE(nck >= 1 && nck <= 16 && ncv >= 1 && ncv <= 16, FQ_ERR_INVALID_ARGUMENT,
             "centroid count outside [1, 16]");
  FQ_REQUIRE(head_dim == 128 || head_dim == 64, FQ_ERR_UNSUPPORTED,
             "paged decode: head_dim %d (built for 64 and 128)", head_dim);
  FQ_REQUIRE(hkv == 1 || hkv == 2 || hkv == 4 || hkv == 8 || hkv == 16, FQ_ERR_UNSUPPORTED,
             "paged decode: num_kv_heads %d (built for 1, 2, 4, 8, 16)", hkv);
  FQ_REQUIRE(hq % hkv == 0 && hq / hkv <= 8, FQ_ERR_UNSUPPORTED,
             "paged decode: %d q heads per KV head (at most 8, and a whole number)", hq / hkv);
  FQ_REQUIRE(block_size >= 16 && block_size % 16 == 0 && block_size <= 128, FQ_ERR_UNSUPPORTED,
             "paged decode: block_size %d (a multiple of 16, at most 128)", block_size);
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
                        int ctas, cudaStream_t stream, void* fused_out = nullptr,
                        const uint8_t* kq_cache = nullptr, const float* qjl = nullptr,
                        int n_q = 1) {
  // `hq` counts the query rows of a sequence: n_q tokens x heads (n_q > 1: fast path only)
  FQ_REQUIRE(workspace && aligned(workspace, 256), FQ_ERR_WORKSPACE,
             "paged decode: workspace is null or not 256-byte aligned");
  const WorkspaceLayout w =
      workspace_layout(num_seqs, hq, head_dim, num_splits, ctas * (kCW / hkv), ctas);
  FQ_REQUIRE(workspace_bytes >= w.total, FQ_ERR_WORKSPACE,
             "paged decode: workspace has %zu bytes, %zu needed", workspace_bytes, w.total);
  const bool fast = fast_path_fits(hq, n_q, hkv, head_dim, block_size, kq_cache != nullptr);
  FQ_REQUIRE(fast || n_q == 1, FQ_ERR_UNSUPPORTED,
             "paged decode: %d tokens per sequence in one pass need head_dim 128, 8 KV heads, "
             "pages of 16 tokens and at most 8 (token, head) pairs per KV head", n_q);
  const SmemPlan sp = fast ? plan_smem_fast(num_seqs, hq)
                           : plan_smem(num_seqs, hq, hkv, head_dim, block_size, kq_cache != nullptr);
  FQ_REQUIRE(sp.stages >= 2, FQ_ERR_UNSUPPORTED,
             "paged decode: a page of %d tokens x %d heads does not fit the shared-memory ring",
             block_size, hkv);
  FQ_REQUIRE(sp.off_q - sp.off_ring >= kMergeScratchBytes, FQ_ERR_UNSUPPORTED,
             "paged decode: shared-memory ring too small for the merge phase");
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  const __half* q_rot = reinterpret_cast<const __half*>(ws + w.q_rot_off);
  if (fused_out) {
    // rotation, streaming and merge in one launch
  } else if (rotation) {
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
  a.max_pages = int(block_table_stride < 0 ? 0 : (block_table_stride > (1 << 30) ? (1 << 30) : block_table_stride));
  a.seq_lens = seq_lens;
  a.cent_k = centroids_k; a.nck = nck;
  a.cent_v = centroids_v; a.ncv = ncv;
  a.num_seqs = num_seqs; a.hq = hq; a.hkv = hkv; a.block_size = block_size;
  a.num_blocks = num_blocks;
  a.scale_log2 = sm_scale * 1.4426950408889634f;
  a.num_splits = num_splits;
  a.slots = reinterpret_cast<float*>(ws + w.slots_off);
  a.status = reinterpret_cast<uint32_t*>(ws);
  a.n_q = n_q;
  a.wait_ns = device_wait_limit_ns();
  a.seg_extra = uint32_t(g_test_extra_segments.load(std::memory_order_relaxed));
  if (!fused_out)
    return fast ? launch_fast<0>(a, sp, ctas, stream) : launch_stream<0>(a, sp, ctas, head_dim, stream);
  a.q_src = q;
  a.rotation = rotation;
  a.out = fused_out;
  a.q_rot_w = reinterpret_cast<__half*>(ws + w.q_rot_off);
  a.q_count = reinterpret_cast<uint32_t*>(ws + w.count_off);
  a.seg_count = a.q_count + kMaxSeqs;
  a.merge_count = a.seg_count + kMaxSeqs;
  a.chunk_count = a.merge_count + kMaxSeqs;
  a.chunk_rows = reinterpret_cast<float*>(ws + w.chunk_off);
  a.merge_chunks = fused_out ? w.merge_chunks : 1;
  if (kq_cache) {
    a.kq_cache = kq_cache;
    a.qjl = qjl;
    a.qs_w = a.q_rot_w + size_t(num_seqs) * hq * head_dim;
    // logit += gamma * sqrt(pi/2) / m * <S q, signs>, m = head_dim rows of S
    a.corr_scale_log2 = 1.2533141373155003f / float(head_dim) * a.scale_log2;
    return dtype == FQ_BF16 ? launch_stream<3>(a, sp, ctas, head_dim, stream)
                            : launch_stream<4>(a, sp, ctas, head_dim, stream);
  }
  if (fast)
    return dtype == FQ_BF16 ? launch_fast<1>(a, sp, ctas, stream) : launch_fast<2>(a, sp, ctas, stream);
  return dtype == FQ_BF16 ? launch_stream<1>(a, sp, ctas, head_dim, stream)
                          : launch_stream<2>(a, sp, ctas, head_dim, stream);
}

static MergeArgs slot_merge_args(void* workspace, int num_seqs, int hq, int hkv, int head_dim,
                                 int num_splits, int ctas, const int32_t* seq_lens,
                                 int block_size, int64_t block_table_stride) {
  const int workers = ctas * (kCW / hkv);
  const WorkspaceLayout w = workspace_layout(num_seqs, hq, head_dim, num_splits, workers);
  MergeArgs m{};
  m.rows = reinterpret_cast<const float*>(static_cast<unsigned char*>(workspace) + w.slots_off);
  m.num_splits = num_splits;
  m.num_workers = workers;
  m.seq_lens = seq_lens;
  m.block_size = block_size;
  m.max_pages = int(block_table_stride < 0 ? 0 : (block_table_stride > (1 << 30) ? (1 << 30) : block_table_stride));
  m.num_seqs = num_seqs;
  m.hq = hq;
  return m;
}

}  // namespace fq

using namespace fq;

extern "C" size_t fq_paged_decode_workspace_bytes(int num_seqs, int num_q_heads,
                                                  int num_kv_heads, int head_dim,
                                                  int num_splits) {
  if (num_seqs < 0 || num_q_heads < 0 || head_dim < 0 || num_kv_heads < 1 || num_kv_heads > kCW)
    return 0;
  // sized for any current device: up to 192 SMs
  return workspace_layout(num_seqs, num_q_heads, head_dim, num_splits, 192 * (kCW / num_kv_heads))
      .total;
}

static int decode_call(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                       const int32_t* block_table, int64_t block_table_stride,
                       const int32_t* seq_lens, const float* centroids_k, int n_centroids_k,
                       const float* centroids_v, int n_centroids_v, const float* rotation,
                       int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                       int block_size, int64_t num_blocks, float sm_scale, void* out,
                       int num_splits, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream, int n_q = 1);

extern "C" int fq_split_k_paged_decode(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                                       const int32_t* block_table, int64_t block_table_stride,
                                       const int32_t* seq_lens, const float* centroids_k,
                                       int n_centroids_k, const float* centroids_v,
                                       int n_centroids_v, const float* rotation, int num_seqs,
                                       int num_q_heads, int num_kv_heads, int head_dim,
                                       int block_size, int64_t num_blocks, float sm_scale,
                                       void* out, int num_splits, void* workspace,
                                       size_t workspace_bytes, fq_stream_t stream) {
  FQ_RANGE("fq_split_k_paged_decode");
  return decode_call(q, dtype, kv_cache, block_table, block_table_stride, seq_lens, centroids_k,
                     n_centroids_k, centroids_v, n_centroids_v, rotation, num_seqs, num_q_heads,
                     num_kv_heads, head_dim, block_size, num_blocks, sm_scale, out, num_splits,
                     workspace, workspace_bytes, stream);
}

// The whole call: one cooperative launch, or three ordinary ones when that is switched off,
// refused by the driver, or the query is fp32.  Shared by the entry points that differ only
// in where the workspace comes from.
static int decode_call(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                       const int32_t* block_table, int64_t block_table_stride,
                       const int32_t* seq_lens, const float* centroids_k, int n_centroids_k,
                       const float* centroids_v, int n_centroids_v, const float* rotation,
                       int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
                       int block_size, int64_t num_blocks, float sm_scale, void* out,
                       int num_splits, void* workspace, size_t workspace_bytes,
                       cudaStream_t stream, int n_q) {
  // n_q > 1: every sequence brings n_q query tokens, q and out are (num_seqs, n_q, H_q, D) and
  // num_q_heads counts the heads of ONE token (fast path only, see decode_tokens_per_pass)
  const int q_rows = num_q_heads * n_q;
  int rc = validate_decode(q, dtype, kv_cache, block_table, seq_lens, centroids_k, n_centroids_k,
                           centroids_v, n_centroids_v, rotation, num_seqs, num_q_heads,
                           num_kv_heads, head_dim, block_size, num_blocks, num_splits);
  if (rc != FQ_OK) return rc;
  FQ_REQUIRE(out && aligned(out, 2), FQ_ERR_INVALID_ARGUMENT, "paged decode: out is null");
  if (num_seqs == 0) return FQ_OK;
  const int ctas = device_sm_count();
  if (num_splits == 0) num_splits = auto_splits();
  // an fp32 query (the reference's CPU-sized cases) takes the three-launch form: its rotated
  // query is not rounded (it meets the keys as fp16), its output is not rounded either
  if (g_single_launch.load(std::memory_order_relaxed) && dtype != FQ_F32) {
    rc = decode_front(q, dtype, kv_cache, block_table, block_table_stride, seq_lens, centroids_k,
                      n_centroids_k, centroids_v, n_centroids_v, rotation, num_seqs, q_rows,
                      num_kv_heads, head_dim, block_size, num_blocks, sm_scale, num_splits,
                      workspace, workspace_bytes, ctas, stream, out, nullptr, nullptr, n_q);
    if (rc != kCoopRefused) return rc;
  }
  // three launches: q rotation, streaming, merge (no CTA waits for another one)
  rc = decode_front(q, dtype, kv_cache, block_table, block_table_stride, seq_lens, centroids_k,
                    n_centroids_k, centroids_v, n_centroids_v, rotation, num_seqs, q_rows,
                    num_kv_heads, head_dim, block_size, num_blocks, sm_scale, num_splits,
                    workspace, workspace_bytes, ctas, stream, nullptr, nullptr, nullptr, n_q);
  if (rc != FQ_OK) return rc;
  MergeArgs m = slot_merge_args(workspace, num_seqs, q_rows, num_kv_heads, head_dim,
                                num_splits, ctas, seq_lens, block_size, block_table_stride);
  m.rotation = rotation;
  m.out = out;
  return launch_merge<true, true>(m, head_dim, dtype, stream);
}

namespace fq {
// How many query tokens of a sequence one pass of the decode can take together: the (token,
// head) pairs of a KV head are the eight columns of its products, so 8 / (heads per KV head)
// where the specialised kernel applies, else 1.
int decode_tokens_per_pass(int num_q_heads, int num_kv_heads, int head_dim, int block_size) {
  if (num_kv_heads < 1 || num_q_heads % num_kv_heads) return 1;
  const int group = num_q_heads / num_kv_heads;
  if (group > 8 || !fast_path_fits(num_q_heads, 1, num_kv_heads, head_dim, block_size, false))
    return 1;
  return 8 / group;
}

int decode_tokens(const void* q, fq_dtype dtype, const uint8_t* kv_cache,
                  const int32_t* block_table, int64_t block_table_stride, const int32_t* seq_lens,
                  const float* centroids_k, int n_centroids_k, const float* centroids_v,
                  int n_centroids_v, const float* rotation, int num_seqs, int n_q, int num_q_heads,
                  int num_kv_heads, int head_dim, int block_size, int64_t num_blocks,
                  float sm_scale, void* out, int num_splits, void* workspace,
                  size_t workspace_bytes, cudaStream_t stream) {
  return decode_call(q, dtype, kv_cache, block_table, block_table_stride, seq_lens, centroids_k,
                     n_centroids_k, centroids_v, n_centroids_v, rotation, num_seqs, num_q_heads,
                     num_kv_heads, head_dim, block_size, num_blocks, sm_scale, out, num_splits,
                     workspace, workspace_bytes, stream, n_q);
}
}  // namespace fq

extern "C" void fq_paged_decode_set_single_launch(int enabled) {
  g_single_launch.store(enabled ? 1 : 0, std::memory_order_relaxed);
  settings_changed();
}

extern "C" void fq_paged_decode_set_fast_path(int enabled) {
  g_fast_path.store(enabled ? 1 : 0, std::memory_order_relaxed);
  settings_changed();
}

extern "C" void fq_paged_decode_set_weight_split(int enabled) {
  g_weight_split.store(enabled ? 1 : 0, std::memory_order_relaxed);
  settings_changed();
}

extern "C" void fq_paged_decode_test_expect_extra_segments(int n) {
  g_test_extra_segments.store(n < 0 ? 0 : n, std::memory_order_relaxed);
  settings_changed();
}

extern "C" int fq_split_k_paged_decode_qjl(
    const void* q, fq_dtype dtype, const uint8_t* kv_cache, const uint8_t* kq_cache,
    const int32_t* block_table, int64_t block_table_stride, const int32_t* seq_lens,
    const float* centroids_k, int n_centroids_k, const float* centroids_v, int n_centroids_v,
    const float* rotation, const float* qjl, int num_seqs, int num_q_heads, int num_kv_heads,
    int head_dim, int block_size, int64_t num_blocks, float sm_scale, void* out, int num_splits,
    void* workspace, size_t workspace_bytes, fq_stream_t stream) {
  FQ_RANGE("fq_split_k_paged_decode_qjl");
  int rc = validate_decode(q, dtype, kv_cache, block_table, seq_lens, centroids_k, n_centroids_k,
                           centroids_v, n_centroids_v, rotation, num_seqs, num_q_heads,
                           num_kv_heads, head_dim, block_size, num_blocks, num_splits);
  if (rc != FQ_OK) return rc;
  FQ_REQUIRE(out && kq_cache && qjl, FQ_ERR_INVALID_ARGUMENT,
             "paged decode (two-stage): null pointer");
  FQ_REQUIRE(dtype != FQ_F32, FQ_ERR_UNSUPPORTED,
             "paged decode (two-stage): q must be fp16 or bf16");
  FQ_REQUIRE(head_dim == 128, FQ_ERR_UNSUPPORTED,
             "paged decode (two-stage): head_dim %d (built for 128)", head_dim);
  FQ_REQUIRE(aligned(kq_cache, 16) && aligned(qjl, 16), FQ_ERR_ALIGNMENT,
             "paged decode (two-stage): kq_cache and qjl must be 16-byte aligned");
  if (num_seqs == 0) return FQ_OK;
  const int ctas = device_sm_count();
  if (num_splits == 0) num_splits = auto_splits();
  rc = decode_front(q, dtype, kv_cache, block_table, block_table_stride, seq_lens, centroids_k,
                    n_centroids_k, centroids_v, n_centroids_v, rotation, num_seqs, num_q_heads,
                    num_kv_heads, head_dim, block_size, num_blocks, sm_scale, num_splits,
                    workspace, workspace_bytes, ctas, stream, out, kq_cache, qjl);
  // this entry has no three-launch form: a GPU that cannot hold the cooperative launch
  // (shared with other contexts, partitioned) cannot run it
  if (rc == kCoopRefused)
    return fail(FQ_ERR_UNSUPPORTED,
                "paged decode (two-stage): the single cooperative launch was refused by the "
                "driver and this entry point has no other form");
  return rc;
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
  MergeArgs m = slot_merge_args(workspace, num_seqs, num_q_heads, num_kv_heads, head_dim,
                                num_splits, ctas, seq_lens, block_size, block_table_stride);
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
  FQ_RANGE("fq_paged_decode_partials");
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
  FQ_RANGE("fq_paged_decode_partials_rotated");
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

extern "C" int fq_paged_decode_stream(const void* q_rot_f16, const uint8_t* kv_cache,
                                      const int32_t* block_table, int64_t block_table_stride,
                                      const int32_t* seq_lens, const float* centroids_k,
                                      int n_centroids_k, const float* centroids_v,
                                      int n_centroids_v, int num_seqs, int num_q_heads,
                                      int num_kv_heads, int head_dim, int block_size,
                                      int64_t num_blocks, float sm_scale, int num_splits,
                                      void* workspace, size_t workspace_bytes,
                                      fq_stream_t stream) {
  FQ_RANGE("fq_paged_decode_stream");
  alignas(16) static const float kDummy[4] = {0.f, 0.f, 0.f, 0.f};  // validate wants non-null
  int rc = validate_decode(q_rot_f16, FQ_F16, kv_cache, block_table, seq_lens, centroids_k,
                           n_centroids_k, centroids_v, n_centroids_v, kDummy, num_seqs,
                           num_q_heads, num_kv_heads, head_dim, block_size, num_blocks,
                           num_splits);
  if (rc != FQ_OK) return rc;
  if (num_seqs == 0) return FQ_OK;
  if (num_splits == 0) num_splits = auto_splits();
  return decode_front(q_rot_f16, FQ_F16, kv_cache, block_table, block_table_stride, seq_lens,
                      centroids_k, n_centroids_k, centroids_v, n_centroids_v, nullptr, num_seqs,
                      num_q_heads, num_kv_heads, head_dim, block_size, num_blocks, sm_scale,
                      num_splits, workspace, workspace_bytes, device_sm_count(), stream);
}

extern "C" int fq_split_k_merge(const float* partials, int n_groups, const float* rotation,
                                int num_seqs, int num_q_heads, int head_dim, void* out,
                                fq_dtype dtype, fq_stream_t stream) {
  FQ_RANGE("fq_split_k_merge");
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

// ------------------------------------------------------------------------------------
// Decode without any allocation by the caller or by this library
// ------------------------------------------------------------------------------------
// Some callers cannot obtain device memory at the moment they need to decode: a serving
// engine that has handed its whole memory budget to the KV cache and refuses further
// cudaMalloc calls, a plugin that runs inside another framework's memory pool, or code on a
// path where an allocation would synchronise the device.  For them the scratch that
// fq_split_k_paged_decode takes as `workspace` lives in the array below, which is part of
// the library image: every GPU that loads the library holds these 16 MiB until the process
// exits.  All calls on a device share the array, so two calls that overlap on the GPU (two
// streams, or two host threads) race on it; the status word at its start is cleared by
// every call.
constexpr size_t kStaticScratchBytes = size_t(16) << 20;
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticScratchBytes];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;
void* g_scratch_addr[kMaxDevices] = {};

// Device address of g_decode_scratch on the current device.  The array's name is only a
// host-side handle; the address a kernel can use has to be asked for, once per device, with
// that device current.
int static_scratch(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fq::fail(FQ_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices)
    return fq::fail(FQ_ERR_UNSUPPORTED, "device ordinal %d beyond %d", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_decode_scratch);
    if (e != cudaSuccess || !p)
      return fq::fail(FQ_ERR_CUDA, "cudaGetSymbolAddress(decode scratch): %s",
                      cudaGetErrorString(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return FQ_OK;
}
}  // namespace

extern "C" size_t fq_split_k_paged_decode_static_max_bytes(void) { return kStaticScratchBytes; }

extern "C" int fq_split_k_paged_decode_static(
    const void* q, fq_dtype dtype, const uint8_t* kv_cache, const int32_t* block_table,
    int64_t block_table_stride, const int32_t* seq_lens, const float* centroids_k,
    int n_centroids_k, const float* centroids_v, int n_centroids_v, const float* rotation,
    int num_seqs, int num_q_heads, int num_kv_heads, int head_dim, int block_size,
    int64_t num_blocks, float sm_scale, void* out, int num_splits, fq_stream_t stream) {
  FQ_RANGE("fq_split_k_paged_decode_static");
  int rc = validate_decode(q, dtype, kv_cache, block_table, seq_lens, centroids_k, n_centroids_k,
                           centroids_v, n_centroids_v, rotation, num_seqs, num_q_heads,
                           num_kv_heads, head_dim, block_size, num_blocks, num_splits);
  if (rc != FQ_OK) return rc;
  FQ_REQUIRE(out, FQ_ERR_INVALID_ARGUMENT, "paged decode: out is null");
  if (num_seqs == 0) return FQ_OK;
  const int ctas = device_sm_count();
  const size_t need =
      workspace_layout(num_seqs, num_q_heads, head_dim, num_splits == 0 ? auto_splits() : num_splits,
                       ctas * (kCW / num_kv_heads))
          .total;
  FQ_REQUIRE(need <= kStaticScratchBytes, FQ_ERR_WORKSPACE,
             "fq_split_k_paged_decode_static: this shape needs %zu bytes of scratch, the built-in "
             "array holds %zu; use fq_split_k_paged_decode with a caller-owned workspace",
             need, kStaticScratchBytes);
  void* scratch = nullptr;
  rc = static_scratch(&scratch);
  if (rc != FQ_OK) return rc;
  // the array keeps what the previous call left: the status word and the counters the CTAs
  // signal each other through must start at zero (bytes 64..255 keep the scaled-table record
  // of earlier calls)
  const size_t head_bytes = workspace_layout(num_seqs, num_q_heads, head_dim, num_splits, 0).q_rot_off;
  cudaError_t e = cudaMemsetAsync(scratch, 0, kScaleCacheOffset, stream);
  if (e == cudaSuccess)
    e = cudaMemsetAsync(static_cast<unsigned char*>(scratch) + 256, 0, head_bytes - 256, stream);
  if (e != cudaSuccess)
    return fail(FQ_ERR_CUDA, "clearing the scratch status word: %s", cudaGetErrorString(e));
  // same call as fq_split_k_paged_decode from here on: single launch, or three launches when
  // that is switched off or refused
  return decode_call(q, dtype, kv_cache, block_table, block_table_stride, seq_lens, centroids_k,
                     n_centroids_k, centroids_v, n_centroids_v, rotation, num_seqs, num_q_heads,
                     num_kv_heads, head_dim, block_size, num_blocks, sm_scale, out, num_splits,
                     scratch, kStaticScratchBytes, stream);
}

// Device status word of the built-in scratch array (FQ_DEV_* bits of the last static call on
// the current device); synchronises the stream.
extern "C" int fq_split_k_paged_decode_static_status(uint32_t* status, fq_stream_t stream) {
  FQ_REQUIRE(status, FQ_ERR_INVALID_ARGUMENT, "static status: null pointer");
  void* scratch = nullptr;
  int rc = static_scratch(&scratch);
  if (rc != FQ_OK) return rc;
  cudaError_t e = cudaMemcpyAsync(status, scratch, sizeof(uint32_t), cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess)
    return fail(FQ_ERR_CUDA, "fq_split_k_paged_decode_static_status: %s", cudaGetErrorString(e));
  return FQ_OK;
}

