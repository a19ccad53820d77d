// One decode step with HOST buffers in and out: what an attention backend does per layer and
// step when its inputs live on the host side of the boundary.
//
// Mirrors FlashQuantAttentionImpl._fused_decode_path (src/flashquant/vllm/impl.py:362-395):
// compress the step's new K/V token of every sequence into the paged cache, then run the
// fused paged decode.  Around those two launches the entry points here do the copies
// themselves and wait for the stream, so that one C call is the whole step and no interpreter
// time sits between the pieces.  Two forms:
//   fq_decode_step_host         six host arrays, six host-to-device copies into a caller-owned
//                               device staging area (those that only the decode needs go
//                               through a side stream and overlap the compress-on-append);
//   fq_decode_step_host_packed  the caller keeps the step's inputs in ONE page-locked block
//                               laid out like the staging area (fq_decode_step_offsets), and
//                               the step is one copy in - or two halves of the block, the
//                               second under the compress-on-append - and one copy out.
// (Letting the kernels read page-locked host arrays in place was measured and is slower: the
// sequence lengths and the block table sit at the head of the decode kernel's dependency
// chain, and every CTA would fetch them over the bus.)
#include <atomic>
#include <cstring>
#include <vector>

#include "fq_common.cuh"

namespace fq {

// Side streams per host thread and device, so that the copies the decode needs (query, block
// table, lengths) overlap the copies and the launch of the compress-on-append, and for
// recording the packed step as a graph; created on first use.
struct StepAux {
  cudaStream_t stream = nullptr;
  cudaStream_t branch = nullptr;  // second branch while `stream` records a graph
  cudaEvent_t fork = nullptr, join = nullptr;
};

static int step_aux(StepAux** out) {
  // per host thread: two threads that step on one GPU must not record into each other's
  // events, and a thread that records a graph must have the recording streams to itself
  constexpr int kMaxDevices = 64;
  static thread_local StepAux aux[kMaxDevices];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(FQ_ERR_CUDA, "decode step: cudaGetDevice: %s", cudaGetErrorString(e));
  StepAux& a = aux[dev];
  if (!a.stream) {
    e = cudaStreamCreateWithFlags(&a.stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&a.branch, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&a.fork, cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&a.join, cudaEventDisableTiming);
    if (e != cudaSuccess) {
      a = StepAux{};
      return fail(FQ_ERR_CUDA, "decode step: side stream: %s", cudaGetErrorString(e));
    }
  }
  *out = &a;
  return FQ_OK;
}

// Inputs of the compress-on-append first, then what only the decode reads, then the result:
// the packed form copies [k, sl) and [sl, out) as two contiguous halves.
struct StepLayout {
  size_t k, v, slots, sl, bt, q, out, total;
};

static size_t up256_(size_t v) { return (v + 255) / 256 * 256; }

static StepLayout step_layout(int num_seqs, int hq, int hkv, int d, int64_t bt_stride,
                              int slot_is_int64) {
  StepLayout L{};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off = up256_(off + bytes);
    return at;
  };
  L.k = take(size_t(num_seqs) * hkv * d * 2);
  L.v = take(size_t(num_seqs) * hkv * d * 2);
  L.slots = take(size_t(num_seqs) * (slot_is_int64 ? 8 : 4));
  L.sl = take(size_t(num_seqs) * 4);
  L.bt = take(size_t(num_seqs) * size_t(bt_stride) * 4);
  L.q = take(size_t(num_seqs) * hq * d * 2);
  L.out = take(size_t(num_seqs) * hq * d * 2);
  L.total = off;
  return L;
}

}  // namespace fq

namespace fq {

// The two launches and the copy of the result back to the host, on inputs that the copies
// issued before have put (or are putting: `join_side`) into the staging area.
static int step_kernels_and_result(
    const StepLayout& L, unsigned char* st, StepAux* aux, fq_dtype dtype, int slot_is_int64,
    int64_t block_table_stride, uint8_t* kv_cache, uint8_t* kq_cache, const float* rotation,
    const float* boundaries_k, int n_boundaries_k, const float* centroids_k, int n_centroids_k,
    const float* boundaries_v, int n_boundaries_v, const float* centroids_v, int n_centroids_v,
    const float* qjl, int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
    int block_size, int64_t num_blocks, float sm_scale, int num_splits, void* out_host,
    void* workspace, size_t workspace_bytes, fq_stream_t stream_, bool join_side,
    bool synchronise = true) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const size_t n = size_t(num_seqs);
  int rc = FQ_OK;
  const void *q_d = st + L.q, *k_d = st + L.k, *v_d = st + L.v, *slots_d = st + L.slots;
  const void *bt_d = st + L.bt, *sl_d = st + L.sl;
  void* out_d = st + L.out;
  const int64_t num_slots = num_blocks * block_size;
  if (kq_cache) {
    rc = fq_tq4_compress_append_qjl(k_d, v_d, dtype, num_seqs, num_kv_heads, head_dim,
                                    int64_t(num_kv_heads) * head_dim, rotation, boundaries_k,
                                    n_boundaries_k, centroids_k, boundaries_v, n_boundaries_v, qjl,
                                    kv_cache, kq_cache, num_slots, slots_d, slot_is_int64,
                                    stream_);
  } else {
    rc = fq_tq4_compress_append(k_d, v_d, dtype, num_seqs, num_kv_heads, head_dim,
                                int64_t(num_kv_heads) * head_dim, rotation, boundaries_k,
                                n_boundaries_k, boundaries_v, n_boundaries_v, kv_cache, num_slots,
                                slots_d, slot_is_int64, stream_);
  }
  if (rc != FQ_OK) return rc;
  if (join_side) {
    cudaError_t ce = cudaStreamWaitEvent(stream, aux->join, 0);
    if (ce != cudaSuccess)
      return fail(FQ_ERR_CUDA, "decode step: joining the side stream: %s", cudaGetErrorString(ce));
  }
  rc = fq_split_k_paged_decode(q_d, dtype, kv_cache, static_cast<const int32_t*>(bt_d),
                               block_table_stride, static_cast<const int32_t*>(sl_d), centroids_k,
                               n_centroids_k, centroids_v, n_centroids_v, rotation, num_seqs,
                               num_q_heads, num_kv_heads, head_dim, block_size, num_blocks,
                               sm_scale, out_d, num_splits, workspace, workspace_bytes,
                               stream_);
  if (rc != FQ_OK) return rc;
  cudaError_t e = cudaMemcpyAsync(out_host, out_d, n * num_q_heads * head_dim * 2,
                                  cudaMemcpyDeviceToHost, stream);
  if (e == cudaSuccess && synchronise) e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess)
    return fail(FQ_ERR_CUDA, "decode step: result copy or synchronise: %s", cudaGetErrorString(e));
  return FQ_OK;
}

// The packed step as a CUDA graph: one copy in, two launches, one copy out are the same nodes
// with the same arguments step after step (the block, the staging area and the cache do not
// move), so the sequence is captured once per distinct argument set and replayed - one
// submission instead of four.  Per host thread, a handful of entries (a server cycles through
// a few caches / layers; beyond that the oldest entry is dropped).
struct StepGraphKey {
  const void* block; void* out; int dtype, slot64; int64_t bt_stride;
  const void *kv, *kq, *rot, *bk, *ck, *bv, *cv, *qjl;
  int nbk, nck, nbv, ncv, num_seqs, hq, hkv, d, bs; int64_t num_blocks; float scale; int splits;
  void* staging; void* workspace; size_t workspace_bytes; cudaStream_t stream; int device;
  int overlap;  // the recorded sequence has the second half of the copy on a branch of its own
  uint64_t settings;  // process-wide switches and limits are baked into the recorded launches
};
struct StepGraph {
  StepGraphKey key;
  cudaGraphExec_t exec;
  uint64_t kernels;  // kernel nodes: what a replay adds to the library's launch counter
};
constexpr int kStepGraphs = 16;
static std::atomic<int> g_step_graph{1};

}  // namespace fq

using namespace fq;

extern "C" size_t fq_decode_step_host_staging_bytes(int num_seqs, int num_q_heads,
                                                    int num_kv_heads, int head_dim,
                                                    int64_t block_table_stride,
                                                    int slot_is_int64) {
  if (num_seqs < 0 || num_q_heads < 0 || num_kv_heads < 0 || head_dim < 0 || block_table_stride < 0)
    return 0;
  return step_layout(num_seqs, num_q_heads, num_kv_heads, head_dim, block_table_stride,
                     slot_is_int64)
      .total;
}

extern "C" int fq_decode_step_host(
    const void* q_host, const void* key_host, const void* value_host, fq_dtype dtype,
    const void* slot_mapping_host, int slot_is_int64, const int32_t* block_table_host,
    int64_t block_table_stride, const int32_t* seq_lens_host, uint8_t* kv_cache,
    uint8_t* kq_cache, const float* rotation, const float* boundaries_k, int n_boundaries_k,
    const float* centroids_k, int n_centroids_k, const float* boundaries_v, int n_boundaries_v,
    const float* centroids_v, int n_centroids_v, const float* qjl, int num_seqs,
    int num_q_heads, int num_kv_heads, int head_dim, int block_size, int64_t num_blocks,
    float sm_scale, int num_splits, void* out_host, void* staging, size_t staging_bytes,
    void* workspace, size_t workspace_bytes, fq_stream_t stream_) {
  FQ_RANGE("fq_decode_step_host");
  FQ_REQUIRE(q_host && key_host && value_host && slot_mapping_host && block_table_host &&
                 seq_lens_host && out_host,
             FQ_ERR_INVALID_ARGUMENT, "decode step: null host pointer");
  FQ_REQUIRE(dtype == FQ_F16 || dtype == FQ_BF16, FQ_ERR_UNSUPPORTED,
             "decode step: q, key and value must be fp16 or bf16");
  FQ_REQUIRE(num_seqs >= 0 && num_q_heads >= 1 && num_kv_heads >= 1 && head_dim >= 1 &&
                 block_table_stride >= 0,
             FQ_ERR_INVALID_ARGUMENT, "decode step: negative size");
  FQ_REQUIRE(staging && aligned(staging, 256), FQ_ERR_WORKSPACE,
             "decode step: staging is null or not 256-byte aligned");
  const StepLayout L = step_layout(num_seqs, num_q_heads, num_kv_heads, head_dim,
                                   block_table_stride, slot_is_int64);
  FQ_REQUIRE(staging_bytes >= L.total, FQ_ERR_WORKSPACE,
             "decode step: staging has %zu bytes, %zu needed", staging_bytes, L.total);
  if (num_seqs == 0) return FQ_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  unsigned char* st = static_cast<unsigned char*>(staging);
  const size_t n = size_t(num_seqs);
  StepAux* aux = nullptr;
  int rc = step_aux(&aux);
  if (rc != FQ_OK) return rc;
  struct Copy {
    size_t off;
    const void* src;
    size_t bytes;
    bool side;  // on the side stream: only the decode needs it
  };
  const Copy copies[6] = {
      {L.k, key_host, n * num_kv_heads * head_dim * 2, false},
      {L.v, value_host, n * num_kv_heads * head_dim * 2, false},
      {L.slots, slot_mapping_host, n * (slot_is_int64 ? 8 : 4), false},
      {L.sl, seq_lens_host, n * 4, true},
      {L.bt, block_table_host, n * size_t(block_table_stride) * 4, true},
      {L.q, q_host, n * num_q_heads * head_dim * 2, true},
  };
  // the side stream starts after whatever the caller's stream still has to do with the staging
  cudaError_t ce = cudaEventRecord(aux->fork, stream);
  if (ce == cudaSuccess) ce = cudaStreamWaitEvent(aux->stream, aux->fork, 0);
  for (const Copy& c : copies) {
    if (ce != cudaSuccess) break;
    ce = cudaMemcpyAsync(st + c.off, c.src, c.bytes, cudaMemcpyHostToDevice,
                         c.side ? aux->stream : stream);
  }
  if (ce == cudaSuccess) ce = cudaEventRecord(aux->join, aux->stream);
  if (ce != cudaSuccess)
    return fail(FQ_ERR_CUDA, "decode step: host-to-device copies: %s", cudaGetErrorString(ce));
  return step_kernels_and_result(L, st, aux, dtype, slot_is_int64, block_table_stride, kv_cache,
                                 kq_cache, rotation, boundaries_k, n_boundaries_k, centroids_k,
                                 n_centroids_k, boundaries_v, n_boundaries_v, centroids_v,
                                 n_centroids_v, qjl, num_seqs, num_q_heads, num_kv_heads, head_dim,
                                 block_size, num_blocks, sm_scale, num_splits, out_host, workspace,
                                 workspace_bytes, stream_, true);
}

extern "C" int fq_decode_step_offsets(int num_seqs, int num_q_heads, int num_kv_heads,
                                      int head_dim, int64_t block_table_stride,
                                      int slot_is_int64, uint64_t offsets[8]) {
  FQ_REQUIRE(offsets, FQ_ERR_INVALID_ARGUMENT, "decode step: null offsets array");
  FQ_REQUIRE(num_seqs >= 0 && num_q_heads >= 1 && num_kv_heads >= 1 && head_dim >= 1 &&
                 block_table_stride >= 0,
             FQ_ERR_INVALID_ARGUMENT, "decode step: negative size");
  const StepLayout L = step_layout(num_seqs, num_q_heads, num_kv_heads, head_dim,
                                   block_table_stride, slot_is_int64);
  offsets[0] = L.k;
  offsets[1] = L.v;
  offsets[2] = L.slots;
  offsets[3] = L.sl;
  offsets[4] = L.bt;
  offsets[5] = L.q;
  offsets[6] = L.out;
  offsets[7] = L.total;
  return FQ_OK;
}

extern "C" int fq_decode_step_host_packed(
    const void* block_host, void* out_host, int overlap_copies, fq_dtype dtype, int slot_is_int64,
    int64_t block_table_stride, uint8_t* kv_cache, uint8_t* kq_cache, const float* rotation,
    const float* boundaries_k, int n_boundaries_k, const float* centroids_k, int n_centroids_k,
    const float* boundaries_v, int n_boundaries_v, const float* centroids_v, int n_centroids_v,
    const float* qjl, int num_seqs, int num_q_heads, int num_kv_heads, int head_dim,
    int block_size, int64_t num_blocks, float sm_scale, int num_splits, void* staging,
    size_t staging_bytes, void* workspace, size_t workspace_bytes, fq_stream_t stream_) {
  FQ_RANGE("fq_decode_step_host_packed");
  FQ_REQUIRE(block_host && out_host, FQ_ERR_INVALID_ARGUMENT, "decode step: null host pointer");
  FQ_REQUIRE(dtype == FQ_F16 || dtype == FQ_BF16, FQ_ERR_UNSUPPORTED,
             "decode step: q, key and value must be fp16 or bf16");
  FQ_REQUIRE(num_seqs >= 0 && num_q_heads >= 1 && num_kv_heads >= 1 && head_dim >= 1 &&
                 block_table_stride >= 0,
             FQ_ERR_INVALID_ARGUMENT, "decode step: negative size");
  FQ_REQUIRE(staging && aligned(staging, 256), FQ_ERR_WORKSPACE,
             "decode step: staging is null or not 256-byte aligned");
  const StepLayout L = step_layout(num_seqs, num_q_heads, num_kv_heads, head_dim,
                                   block_table_stride, slot_is_int64);
  FQ_REQUIRE(staging_bytes >= L.total, FQ_ERR_WORKSPACE,
             "decode step: staging has %zu bytes, %zu needed", staging_bytes, L.total);
  if (num_seqs == 0) return FQ_OK;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  unsigned char* st = static_cast<unsigned char*>(staging);
  const unsigned char* src = static_cast<const unsigned char*>(block_host);
  StepAux* aux = nullptr;
  cudaError_t ce = cudaSuccess;
  if (g_step_graph.load(std::memory_order_relaxed)) {
    static thread_local std::vector<StepGraph> graphs;
    StepGraphKey key;
    std::memset(&key, 0, sizeof(key));  // padding too: the key is compared byte by byte
    key.block = block_host; key.out = out_host; key.dtype = int(dtype); key.slot64 = slot_is_int64;
    key.bt_stride = block_table_stride; key.kv = kv_cache; key.kq = kq_cache; key.rot = rotation;
    key.bk = boundaries_k; key.ck = centroids_k; key.bv = boundaries_v; key.cv = centroids_v;
    key.qjl = qjl; key.nbk = n_boundaries_k; key.nck = n_centroids_k; key.nbv = n_boundaries_v;
    key.ncv = n_centroids_v; key.num_seqs = num_seqs; key.hq = num_q_heads; key.hkv = num_kv_heads;
    key.d = head_dim; key.bs = block_size; key.num_blocks = num_blocks; key.scale = sm_scale;
    key.splits = num_splits; key.staging = staging; key.workspace = workspace;
    key.workspace_bytes = workspace_bytes; key.stream = stream; key.overlap = overlap_copies ? 1 : 0;
    cudaGetDevice(&key.device);
    key.settings = settings_epoch();
    cudaGraphExec_t exec = nullptr;
    uint64_t kernels = 0;
    for (const StepGraph& g : graphs)
      if (std::memcmp(&g.key, &key, sizeof(key)) == 0) {
        exec = g.exec;
        kernels = g.kernels;
      }
    // captured on the library's own side stream (the caller's may be the legacy default
    // stream, which cannot capture); the graph is then launched into the caller's stream
    cudaStream_t cap = nullptr;
    if (!exec && step_aux(&aux) == FQ_OK) cap = aux->stream;
    if (cap && cudaStreamBeginCapture(cap, cudaStreamCaptureModeThreadLocal) != cudaSuccess) {
      cudaGetLastError();
      cap = nullptr;
    }
    if (cap) {
      fq_stream_t cap_ = cap;
      const uint64_t launches_at_capture = fq_launch_count();
      if (overlap_copies) {
        // what the compress-on-append reads first; the rest on a branch that joins before the
        // decode, so that it travels under the compress-on-append
        ce = cudaMemcpyAsync(st + L.k, src + L.k, L.sl - L.k, cudaMemcpyHostToDevice, cap);
        if (ce == cudaSuccess) ce = cudaEventRecord(aux->fork, cap);
        if (ce == cudaSuccess) ce = cudaStreamWaitEvent(aux->branch, aux->fork, 0);
        if (ce == cudaSuccess)
          ce = cudaMemcpyAsync(st + L.sl, src + L.sl, L.out - L.sl, cudaMemcpyHostToDevice,
                               aux->branch);
        if (ce == cudaSuccess) ce = cudaEventRecord(aux->join, aux->branch);
      } else {
        ce = cudaMemcpyAsync(st, src, L.out, cudaMemcpyHostToDevice, cap);
      }
      int rc = ce == cudaSuccess
                   ? step_kernels_and_result(L, st, aux, dtype, slot_is_int64,
                                             block_table_stride, kv_cache, kq_cache, rotation,
                                             boundaries_k, n_boundaries_k, centroids_k,
                                             n_centroids_k, boundaries_v, n_boundaries_v,
                                             centroids_v, n_centroids_v, qjl, num_seqs,
                                             num_q_heads, num_kv_heads, head_dim, block_size,
                                             num_blocks, sm_scale, num_splits, out_host, workspace,
                                             workspace_bytes, cap_, overlap_copies != 0, false)
                   : FQ_ERR_CUDA;
      const uint64_t after_issue = fq_launch_count();
      cudaGraph_t graph = nullptr;
      const cudaError_t end = cudaStreamEndCapture(cap, &graph);
      kernels = 0;  // the capture counted its launches once; they only run at the replay
      const uint64_t captured = after_issue - launches_at_capture;
      if (rc == FQ_OK && end == cudaSuccess && graph &&
          cudaGraphInstantiate(&exec, graph, 0) == cudaSuccess) {
        if (int(graphs.size()) >= kStepGraphs) {
          cudaGraphExecDestroy(graphs.front().exec);
          graphs.erase(graphs.begin());
        }
        kernels = captured;
        graphs.push_back(StepGraph{key, exec, kernels});
      } else {
        exec = nullptr;
        cudaGetLastError();  // a capture that could not be completed: issue the step directly
      }
      if (graph) cudaGraphDestroy(graph);
    }
    if (exec) {
      ce = cudaGraphLaunch(exec, stream);
      if (ce == cudaSuccess) {
        // (the launches counted during the capture itself stand for this first replay)
        if (!cap) count_launch(kernels);
        ce = cudaStreamSynchronize(stream);
      }
      if (ce != cudaSuccess)
        return fail(FQ_ERR_CUDA, "decode step: graph launch or synchronise: %s",
                    cudaGetErrorString(ce));
      return FQ_OK;
    }
    ce = cudaSuccess;
  }
  if (overlap_copies) {
    // what the compress-on-append reads on the caller's stream, the rest on the side stream
    int rc = step_aux(&aux);
    if (rc != FQ_OK) return rc;
    ce = cudaEventRecord(aux->fork, stream);
    if (ce == cudaSuccess) ce = cudaStreamWaitEvent(aux->stream, aux->fork, 0);
    if (ce == cudaSuccess)
      ce = cudaMemcpyAsync(st + L.sl, src + L.sl, L.out - L.sl, cudaMemcpyHostToDevice, aux->stream);
    if (ce == cudaSuccess) ce = cudaEventRecord(aux->join, aux->stream);
    if (ce == cudaSuccess)
      ce = cudaMemcpyAsync(st + L.k, src + L.k, L.sl - L.k, cudaMemcpyHostToDevice, stream);
  } else {
    ce = cudaMemcpyAsync(st, src, L.out, cudaMemcpyHostToDevice, stream);
  }
  if (ce != cudaSuccess)
    return fail(FQ_ERR_CUDA, "decode step: host-to-device copy: %s", cudaGetErrorString(ce));
  return step_kernels_and_result(L, st, aux, dtype, slot_is_int64, block_table_stride, kv_cache,
                                 kq_cache, rotation, boundaries_k, n_boundaries_k, centroids_k,
                                 n_centroids_k, boundaries_v, n_boundaries_v, centroids_v,
                                 n_centroids_v, qjl, num_seqs, num_q_heads, num_kv_heads, head_dim,
                                 block_size, num_blocks, sm_scale, num_splits, out_host, workspace,
                                 workspace_bytes, stream_, overlap_copies != 0);
}

extern "C" void fq_decode_step_set_graph(int enabled) {
  fq::g_step_graph.store(enabled ? 1 : 0, std::memory_order_relaxed);
}
