// Centroid tables in fp16 with a common scale: the search, its cache in the workspace and the
// table build, shared by the decode kernels (which run it inside the launch) and the
// tensor-core attention kernels (which run it as a small kernel of its own before the launch).
#pragma once

#include "fq_common.cuh"

namespace fq {

constexpr int kScaleThreads = 512;  // threads that run the search together (barrier 1)
__device__ __forceinline__ void scale_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kScaleThreads) : "memory");
}

// ------------------------------------------------------------------------------------
// Centroid tables in fp16 with a common scale.
//
// The products run on fp16 operands, and fp16(c) is off by up to 2^-12 of c.  The error is
// the same for every token that carries the code, so it does not average out: with a few
// dominant key channels it moves the logits by 2^-9 of their size.  But any table beta *
// fp16(c / beta) is as cheap as fp16(c) - beta folds into the logit scale (keys) and into
// the output scale (values) - and for a table of 8 or 16 levels some beta in [1, 2) makes
// every level land several times closer to an fp16 number (the key table of 8 levels:
// typically 2^-15 instead of 2^-12).  All compute threads of the CTA try kScaleCandidates
// values of beta for each table, keep the one with the smallest worst relative error (ties:
// the smaller beta, so every CTA picks the same), and write the scaled fp16 tables.
//
// Shared-memory block at `cent` (kCentBytes): [0,64) fp16 tables (K 16, V 16) as read by the
// table builders; [64,192) the fp32 centroids (written before the call, K then V);
// [192,200) beta_k, beta_v; [256,512) scratch of the reduction; [512,640) 1/|c| (0 for a level
// of exactly zero), written with the centroids.
// ------------------------------------------------------------------------------------
constexpr int kCentBytes = 640;
constexpr int kScaleCandidates = 4096;
// The search costs a few microseconds, so its result is kept in the workspace (bytes 64..255
// of the status block: the 32 centroids it was made for, beta_k, beta_v, a magic word and the
// table sizes) and reused by later calls as long as the centroids are bit-identical.
constexpr uint32_t kScaleMagic = 0x5ca1ab1eu;
constexpr int kScaleCacheOffset = 64;  // bytes into the workspace

__device__ __forceinline__ unsigned long long shfl_xor_u64(unsigned long long v, int o) {
  const uint32_t lo = __shfl_xor_sync(0xffffffffu, uint32_t(v), o);
  const uint32_t hi = __shfl_xor_sync(0xffffffffu, uint32_t(v >> 32), o);
  return (static_cast<unsigned long long>(hi) << 32) | lo;
}

// Set-up half, by ONE warp before the CTA-wide barrier: lane i brings centroid i (K 0-15,
// V 16-31; 0 beyond the table) and learns whether the workspace holds the scales of exactly
// these tables.  Writes the fp32 centroids, their reciprocals, and the hit flag / scales.
__device__ __forceinline__ void stage_centroids(unsigned char* cent, float cent_val, int nck,
                                                int ncv, const uint32_t* cache, int lane) {
  reinterpret_cast<float*>(cent + 64)[lane] = cent_val;
  reinterpret_cast<float*>(cent + 512)[lane] = cent_val != 0.f ? 1.f / fabsf(cent_val) : 0.f;
  const uint32_t kept = __ldcg(cache + lane);
  const uint32_t extra = lane < 5 ? __ldcg(cache + 32 + lane) : 0u;  // beta_k, beta_v, magic, nck, ncv
  const bool same = kept == __float_as_uint(cent_val);
  const float as_beta = __uint_as_float(extra);
  const bool head_ok = lane < 2 ? (as_beta >= 1.f && as_beta < 2.f)
                     : lane == 2 ? extra == kScaleMagic
                     : lane == 3 ? extra == uint32_t(nck)
                     : lane == 4 ? extra == uint32_t(ncv) : true;
  const bool hit = __all_sync(0xffffffffu, same && head_ok);
  if (lane < 2) reinterpret_cast<float*>(cent + 192)[lane] = hit ? __uint_as_float(extra) : 0.f;
  if (lane == 0) reinterpret_cast<uint32_t*>(cent + 200)[0] = hit ? 1u : 0u;
}

// Called by the kScaleThreads compute threads (tid 0 .. kScaleThreads-1) after the barrier
// that follows stage_centroids; ends with a barrier of those threads.  `cache` non-null: this
// CTA records a fresh result in the workspace.
__device__ __forceinline__ void scale_centroid_tables(unsigned char* cent, int nck, int ncv,
                                                      int tid, uint32_t* cache) {
  const float* c32 = reinterpret_cast<const float*>(cent + 64);
  const float* inv = reinterpret_cast<const float*>(cent + 512);
  const bool hit = reinterpret_cast<const uint32_t*>(cent + 200)[0] != 0u;
  unsigned long long* red = reinterpret_cast<unsigned long long*>(cent + 256);  // [2][16]
  if (!hit) {
    unsigned long long best[2] = {~0ull, ~0ull};
    for (int cand = tid; cand < kScaleCandidates; cand += kScaleThreads) {
      const float beta = 1.f + float(cand) * (1.f / kScaleCandidates);
      const float rb = 1.f / beta;
#pragma unroll
      for (int tbl = 0; tbl < 2; ++tbl) {
        const int n = tbl ? ncv : nck;
        float worst = 0.f;
        for (int i = 0; i < n; ++i) {
          const float c = c32[16 * tbl + i];
          const float h = __half2float(__float2half_rn(c * rb));
          // relative error; a level of exactly zero is exact whatever beta is (its 1/|c| is 0)
          worst = fmaxf(worst, fabsf(fmaf(h, beta, -c)) * inv[16 * tbl + i]);
        }
        const unsigned long long key =
            (static_cast<unsigned long long>(__float_as_uint(worst)) << 32) | uint32_t(cand);
        best[tbl] = key < best[tbl] ? key : best[tbl];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int tbl = 0; tbl < 2; ++tbl) {
        const unsigned long long other = shfl_xor_u64(best[tbl], o);
        best[tbl] = other < best[tbl] ? other : best[tbl];
      }
    }
    if ((tid & 31) == 0) {
      red[tid >> 5] = best[0];
      red[16 + (tid >> 5)] = best[1];
    }
  }
  scale_sync();
  if (tid < 32) {
    // lanes 0-15 finish the key table, 16-31 the value table
    const int tbl = tid >> 4, i = tid & 15;
    float beta;
    if (hit) {
      beta = reinterpret_cast<const float*>(cent + 192)[tbl];
    } else {
      unsigned long long b = red[16 * tbl + i];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) {
        const unsigned long long other = shfl_xor_u64(b, o);
        b = other < b ? other : b;
      }
      beta = 1.f + float(uint32_t(b)) * (1.f / kScaleCandidates);
    }
    __syncwarp();
    const int n = tbl ? ncv : nck;
    const float c = i < n ? c32[16 * tbl + i] : 0.f;
    reinterpret_cast<__half*>(cent)[16 * tbl + i] = __float2half_rn(c * (1.f / beta));
    if (i == 0) reinterpret_cast<float*>(cent + 192)[tbl] = beta;
    if (!hit && cache) {
      // the magic word goes last: whoever sees it sees a whole record (a CTA of this launch
      // that starts late must not take half of one)
      cache[tid] = __float_as_uint(c32[tid]);
      if (i == 0) cache[32 + tbl] = __float_as_uint(beta);
      if (tid == 3) cache[35] = uint32_t(nck);
      if (tid == 4) cache[36] = uint32_t(ncv);
      __threadfence();
      __syncwarp();
      if (tid == 2) cache[34] = kScaleMagic;
    }
  }
  scale_sync();
}


// The search as a kernel of its own: one CTA of kScaleThreads threads; leaves (or finds) the
// record at `cache` (32 centroids, beta_k, beta_v, magic, table sizes).
__global__ void __launch_bounds__(kScaleThreads) centroid_scale_kernel(
    const float* __restrict__ cent_k, int nck, const float* __restrict__ cent_v, int ncv,
    uint32_t* __restrict__ cache);

}  // namespace fq
