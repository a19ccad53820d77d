// pybind11 module `_C`: the names the reference's Python layer probes for on `flashquant._C`
// (src/flashquant/kernels/compress.py:34, decompress.py:30, attention.py:34,
// paged_decode.py:37, src/flashquant/vllm/impl.py:57), implemented on the C ABI of
// libflashquant_b200.so.  torch is plumbing only: tensors give device pointers, the current
// CUDA stream, and the cached workspaces.  No `codebook` attribute is exported on purpose:
// the reference would then route its Lloyd-Max solver to it
// (src/flashquant/core/codebook.py:40-41).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <mutex>
#include <optional>
#include <tuple>

#include "flashquant_b200.h"

namespace {

namespace py = pybind11;
using torch::Tensor;

void check(int rc) {
  if (rc != FQ_OK)
    throw std::runtime_error(std::string("flashquant_b200: ") + fq_last_error_string());
}

fq_dtype dtype_of(const Tensor& t) {
  switch (t.scalar_type()) {
    case torch::kFloat32: return FQ_F32;
    case torch::kFloat16: return FQ_F16;
    case torch::kBFloat16: return FQ_BF16;
    default: throw std::runtime_error("flashquant_b200: expected float32, float16 or bfloat16");
  }
}

void need_cuda(const Tensor& t, const char* name) {
  if (!t.is_cuda())
    throw std::runtime_error(std::string("flashquant_b200: ") + name +
                             " must be a CUDA tensor (this build has no CPU path)");
}

Tensor f32_on(const Tensor& t, const torch::Device& dev) {
  return t.to(torch::TensorOptions().device(dev).dtype(torch::kFloat32)).contiguous();
}

// Constants (rotations, tables): the reference keeps several of them as CPU tensors and hands
// them to every call, which would mean a blocking host-to-device copy per call.  A constant
// that is not already a contiguous fp32 tensor on the device is copied once and found again by
// (storage address, version, device); the entry keeps the source alive, so its address cannot
// be taken by another tensor meanwhile.
Tensor const_on(const Tensor& t, const torch::Device& dev) {
  if (t.device() == dev && t.scalar_type() == torch::kFloat32 && t.is_contiguous()) return t;
  struct Entry { Tensor src, copy; };
  using Key = std::tuple<const void*, int64_t, int, int64_t, int64_t>;
  static std::mutex mu;
  static std::map<Key, Entry> cache;
  const Key key{t.data_ptr(), int64_t(t._version()), int(dev.index()), t.numel(),
                t.dim() ? t.stride(0) : 0};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it == cache.end()) {
    if (cache.size() >= 256) cache.clear();
    it = cache.emplace(key, Entry{t, f32_on(t, dev)}).first;
  }
  return it->second.copy;
}

fq_stream_t stream_of(const torch::Device& dev) {
  return reinterpret_cast<fq_stream_t>(at::cuda::getCurrentCUDAStream(dev.index()).stream());
}

// zero-initialised byte workspace per (device, stream, kind), grown on demand: calls on
// different streams may overlap on the GPU and must not share counters or partial rows
Tensor workspace(const torch::Device& dev, int kind, size_t bytes) {
  static std::mutex mu;
  static std::map<std::tuple<int, const void*, int>, Tensor> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto key = std::make_tuple(int(dev.index()), static_cast<const void*>(stream_of(dev)), kind);
  auto it = cache.find(key);
  if (it == cache.end() || size_t(it->second.numel()) < bytes) {
    size_t n = bytes < (size_t(1) << 20) ? (size_t(1) << 20) : bytes;
    cache[key] = torch::zeros({int64_t(n)}, torch::TensorOptions().device(dev).dtype(torch::kUInt8));
    it = cache.find(key);
  }
  return it->second;
}

std::tuple<Tensor, Tensor> tq4_compress(const Tensor& x, const Tensor& rot_t_even,
                                        const Tensor& rot_t_odd, const Tensor& boundaries,
                                        std::optional<std::tuple<Tensor, Tensor>> out) {
  need_cuda(x, "x");
  TORCH_CHECK(x.dim() == 3, "x must be (N, H, D)");
  c10::cuda::CUDAGuard guard(x.device());
  const auto dev = x.device();
  const int64_t n = x.size(0), h = x.size(1), d = x.size(2);
  Tensor xc = x.contiguous();
  Tensor even = const_on(rot_t_even, dev), odd = const_on(rot_t_odd, dev), bnd = const_on(boundaries, dev);
  Tensor packed, norms;
  if (out.has_value()) {
    packed = std::get<0>(*out);
    norms = std::get<1>(*out);
    TORCH_CHECK(packed.numel() == n * h * d / 2 && norms.numel() == n * h, "out buffers: wrong size");
  } else {
    packed = torch::empty({n, h, d / 2}, torch::TensorOptions().device(dev).dtype(torch::kUInt8));
    norms = torch::empty({n, h, 1}, torch::TensorOptions().device(dev).dtype(torch::kFloat32));
  }
  check(fq_tq4_compress(xc.data_ptr(), dtype_of(xc), even.data_ptr<float>(), odd.data_ptr<float>(),
                        bnd.data_ptr<float>(), int(bnd.numel()), packed.data_ptr<uint8_t>(),
                        norms.data_ptr<float>(), n * h, int(d), stream_of(dev)));
  return {packed, norms};
}

Tensor tq4_decompress(const Tensor& packed, const Tensor& norms, const Tensor& centroids,
                      py::object dtype, std::optional<Tensor> out) {
  need_cuda(packed, "packed");
  TORCH_CHECK(packed.dim() == 3, "packed must be (N, H, D/2)");
  c10::cuda::CUDAGuard guard(packed.device());
  const auto dev = packed.device();
  const int64_t n = packed.size(0), h = packed.size(1), d = 2 * packed.size(2);
  const auto st = torch::python::detail::py_object_to_dtype(dtype);
  Tensor p = packed.contiguous(), nn = f32_on(norms, dev), c = const_on(centroids, dev);
  Tensor o = out.has_value() ? *out
                             : torch::empty({n, h, d}, torch::TensorOptions().device(dev).dtype(st));
  TORCH_CHECK(o.is_contiguous() && o.numel() == n * h * d && o.scalar_type() == st,
              "out must be a contiguous (N, H, D) tensor of the requested dtype");
  check(fq_tq4_decompress(p.data_ptr<uint8_t>(), nn.data_ptr<float>(), c.data_ptr<float>(),
                          int(c.numel()), o.data_ptr(), dtype_of(o), n * h, int(d), stream_of(dev)));
  return o;
}

Tensor fused_tq_attention(const Tensor& q, const Tensor& k_packed, const Tensor& k_norms,
                          const Tensor& v_packed, const Tensor& v_norms, const Tensor& centroids_k,
                          const Tensor& centroids_v, const Tensor& rotation, double sm_scale,
                          bool is_causal) {
  need_cuda(q, "q");
  TORCH_CHECK(q.dim() == 4 && k_packed.dim() == 4, "q (B,Hq,Nq,D), k_packed (B,Hkv,Nkv,D/2)");
  c10::cuda::CUDAGuard guard(q.device());
  const auto dev = q.device();
  const int b = int(q.size(0)), hq = int(q.size(1)), nq = int(q.size(2)), d = int(q.size(3));
  const int hkv = int(k_packed.size(1)), nkv = int(k_packed.size(2));
  Tensor qc = q.contiguous(), kp = k_packed.contiguous(), vp = v_packed.contiguous();
  Tensor kn = f32_on(k_norms.reshape({b, hkv, nkv}), dev), vn = f32_on(v_norms.reshape({b, hkv, nkv}), dev);
  Tensor ck = const_on(centroids_k, dev), cv = const_on(centroids_v, dev), rot = const_on(rotation, dev);
  Tensor out = torch::empty_like(qc);
  const size_t need = fq_fused_tq_attention_workspace_bytes(b, hq, nq, d);
  Tensor ws = workspace(dev, 1, need);
  check(fq_fused_tq_attention(qc.data_ptr(), dtype_of(qc), kp.data_ptr<uint8_t>(),
                              kn.data_ptr<float>(), vp.data_ptr<uint8_t>(), vn.data_ptr<float>(),
                              ck.data_ptr<float>(), int(ck.numel()), cv.data_ptr<float>(),
                              int(cv.numel()), rot.data_ptr<float>(), b, hq, hkv, nq, nkv, d,
                              float(sm_scale), is_causal ? 1 : 0, out.data_ptr(), ws.data_ptr(),
                              size_t(ws.numel()), stream_of(dev)));
  return out;
}

Tensor split_k_paged_decode(const Tensor& q, const Tensor& kv_cache, const Tensor& block_table,
                            const Tensor& seq_lens, const Tensor& centroids_k,
                            const Tensor& centroids_v, const Tensor& rotation, int num_kv_heads,
                            int head_dim, int block_size, std::optional<double> sm_scale,
                            std::optional<Tensor> out, int num_splits) {
  need_cuda(q, "q");
  need_cuda(kv_cache, "kv_cache");
  TORCH_CHECK(q.dim() == 3, "q must be (num_seqs, H_q, D)");
  TORCH_CHECK(block_table.scalar_type() == torch::kInt32 && seq_lens.scalar_type() == torch::kInt32,
              "block_table and seq_lens must be int32");
  c10::cuda::CUDAGuard guard(q.device());
  const auto dev = q.device();
  const int num_seqs = int(q.size(0)), hq = int(q.size(1));
  Tensor qc = q.contiguous(), bt = block_table.contiguous(), sl = seq_lens.contiguous();
  TORCH_CHECK(kv_cache.is_contiguous(), "kv_cache must be contiguous");
  Tensor ck = const_on(centroids_k, dev), cv = const_on(centroids_v, dev), rot = const_on(rotation, dev);
  // `out` may be a view with another shape over the same elements (vLLM hands in
  // output[:num_actual], (tokens, H_q * D)): only contiguity, size and dtype matter
  Tensor o = out.has_value() ? *out : torch::empty_like(qc);
  TORCH_CHECK(o.is_contiguous() && o.numel() == qc.numel() && o.scalar_type() == qc.scalar_type(),
              "out must be a contiguous tensor with q's number of elements and dtype");
  const double scale = sm_scale.has_value() ? *sm_scale : 1.0 / std::sqrt(double(head_dim));
  const size_t need = fq_paged_decode_workspace_bytes(num_seqs, hq, num_kv_heads, head_dim, num_splits);
  Tensor ws = workspace(dev, 0, need);
  check(fq_split_k_paged_decode(qc.data_ptr(), dtype_of(qc), kv_cache.data_ptr<uint8_t>(),
                                bt.data_ptr<int32_t>(), bt.stride(0), sl.data_ptr<int32_t>(),
                                ck.data_ptr<float>(), int(ck.numel()), cv.data_ptr<float>(),
                                int(cv.numel()), rot.data_ptr<float>(), num_seqs, hq, num_kv_heads,
                                head_dim, block_size, kv_cache.size(0), float(scale), o.data_ptr(),
                                num_splits, ws.data_ptr(), size_t(ws.numel()), stream_of(dev)));
  return o;
}

// Prefill chunks over the paged cache: the call that stands in for the reference's
// decompress-everything + flash_attn_varlen_func prefill path
// (src/flashquant/vllm/impl.py:265-336, 477-509), with its metadata names.
Tensor paged_tq4_prefill(const Tensor& q, const Tensor& kv_cache, const Tensor& block_table,
                         const Tensor& seq_lens, const Tensor& query_start_loc, int max_query_len,
                         const Tensor& centroids_k, const Tensor& centroids_v,
                         const Tensor& rotation, int num_kv_heads, int head_dim, int block_size,
                         std::optional<double> sm_scale, std::optional<Tensor> out) {
  need_cuda(q, "q");
  need_cuda(kv_cache, "kv_cache");
  TORCH_CHECK(q.dim() == 3, "q must be (num_tokens, H_q, D)");
  TORCH_CHECK(block_table.scalar_type() == torch::kInt32 && seq_lens.scalar_type() == torch::kInt32 &&
                  query_start_loc.scalar_type() == torch::kInt32,
              "block_table, seq_lens and query_start_loc must be int32");
  TORCH_CHECK(query_start_loc.numel() == seq_lens.numel() + 1,
              "query_start_loc must have one entry more than seq_lens");
  c10::cuda::CUDAGuard guard(q.device());
  const auto dev = q.device();
  const int total = int(q.size(0)), hq = int(q.size(1));
  Tensor qc = q.contiguous(), bt = block_table.contiguous(), sl = seq_lens.contiguous();
  Tensor cu = query_start_loc.contiguous();
  TORCH_CHECK(kv_cache.is_contiguous(), "kv_cache must be contiguous");
  Tensor ck = const_on(centroids_k, dev), cv = const_on(centroids_v, dev), rot = const_on(rotation, dev);
  Tensor o = out.has_value() ? *out : torch::empty_like(qc);
  TORCH_CHECK(o.is_contiguous() && o.numel() == qc.numel() && o.scalar_type() == qc.scalar_type(),
              "out must be a contiguous tensor with q's number of elements and dtype");
  const double scale = sm_scale.has_value() ? *sm_scale : 1.0 / std::sqrt(double(head_dim));
  Tensor ws = workspace(dev, 2, fq_paged_tq4_prefill_workspace_bytes(total, hq, head_dim));
  check(fq_paged_tq4_prefill(qc.data_ptr(), dtype_of(qc), kv_cache.data_ptr<uint8_t>(),
                             bt.data_ptr<int32_t>(), bt.stride(0), sl.data_ptr<int32_t>(),
                             cu.data_ptr<int32_t>(), ck.data_ptr<float>(), int(ck.numel()),
                             cv.data_ptr<float>(), int(cv.numel()), rot.data_ptr<float>(),
                             int(sl.numel()), total, max_query_len, hq, num_kv_heads, head_dim,
                             block_size, kv_cache.size(0), float(scale), o.data_ptr(),
                             ws.data_ptr(), size_t(ws.numel()), stream_of(dev)));
  return o;
}

// Device status word (FQ_DEV_* bits) of the decode workspace of the current stream; a non-zero
// word also re-zeroes the head of the workspace, as the C ABI asks before the next call.
int64_t decode_status(const Tensor& like) {
  need_cuda(like, "tensor");
  c10::cuda::CUDAGuard guard(like.device());
  const auto dev = like.device();
  Tensor ws = workspace(dev, 0, 1);
  uint32_t st = 0;
  check(fq_workspace_status(ws.data_ptr(), &st, stream_of(dev)));
  if (st) ws.narrow(0, 0, 32768).zero_();
  return int64_t(st);
}

void tq4_compress_append_qjl(const Tensor& key, const Tensor& value, Tensor kv_cache,
                             Tensor kq_cache, const Tensor& slot_mapping, const Tensor& rotation,
                             const Tensor& boundaries_k, const Tensor& centroids_k,
                             const Tensor& boundaries_v, const Tensor& qjl_matrix) {
  need_cuda(key, "key");
  need_cuda(kv_cache, "kv_cache");
  need_cuda(kq_cache, "kq_cache");
  TORCH_CHECK(key.dim() == 3 && value.sizes() == key.sizes(), "key/value must be (N, H, D)");
  c10::cuda::CUDAGuard guard(key.device());
  const auto dev = key.device();
  const int64_t n = key.size(0);
  const int h = int(key.size(1)), d = int(key.size(2));
  Tensor k = key.contiguous(), v = value.contiguous(), slots = slot_mapping.contiguous();
  TORCH_CHECK(slots.scalar_type() == torch::kInt64 || slots.scalar_type() == torch::kInt32,
              "slot_mapping must be int32 or int64");
  Tensor rot = const_on(rotation, dev), bk = const_on(boundaries_k, dev);
  Tensor ck = const_on(centroids_k, dev), bv = const_on(boundaries_v, dev);
  Tensor S = const_on(qjl_matrix, dev);
  TORCH_CHECK(kv_cache.is_contiguous() && kv_cache.size(-1) == int64_t(h) * (d + 8),
              "kv_cache must be contiguous (num_blocks, block_size, H*(D+8))");
  TORCH_CHECK(kq_cache.is_contiguous() && kq_cache.size(-1) == int64_t(h) * (d / 8 + 4),
              "kq_cache must be contiguous (num_blocks, block_size, H*(D/8+4))");
  const int64_t num_slots = kv_cache.numel() / (int64_t(h) * (d + 8));
  TORCH_CHECK(kq_cache.numel() / (int64_t(h) * (d / 8 + 4)) == num_slots,
              "kq_cache must have as many slots as kv_cache");
  check(fq_tq4_compress_append_qjl(
      k.data_ptr(), v.data_ptr(), dtype_of(k), n, h, d, int64_t(h) * d, rot.data_ptr<float>(),
      bk.data_ptr<float>(), int(bk.numel()), ck.data_ptr<float>(), bv.data_ptr<float>(),
      int(bv.numel()), S.data_ptr<float>(), kv_cache.data_ptr<uint8_t>(),
      kq_cache.data_ptr<uint8_t>(), num_slots, slots.data_ptr(),
      slots.scalar_type() == torch::kInt64 ? 1 : 0, stream_of(dev)));
}

void tq4_compress_append(const Tensor& key, const Tensor& value, Tensor kv_cache,
                         const Tensor& slot_mapping, const Tensor& rotation,
                         const Tensor& boundaries_k, std::optional<Tensor> boundaries_v) {
  need_cuda(key, "key");
  need_cuda(kv_cache, "kv_cache");
  TORCH_CHECK(key.dim() == 3 && value.sizes() == key.sizes(), "key/value must be (N, H, D)");
  c10::cuda::CUDAGuard guard(key.device());
  const auto dev = key.device();
  const int64_t n = key.size(0);
  const int h = int(key.size(1)), d = int(key.size(2));
  Tensor k = key.contiguous(), v = value.contiguous(), slots = slot_mapping.contiguous();
  TORCH_CHECK(slots.scalar_type() == torch::kInt64 || slots.scalar_type() == torch::kInt32,
              "slot_mapping must be int32 or int64");
  Tensor rot = const_on(rotation, dev), bk = const_on(boundaries_k, dev);
  Tensor bv = boundaries_v.has_value() ? const_on(*boundaries_v, dev) : bk;
  TORCH_CHECK(kv_cache.is_contiguous() && kv_cache.size(-1) == int64_t(h) * (d + 8),
              "kv_cache must be contiguous (num_blocks, block_size, H*(D+8))");
  const int64_t num_slots = kv_cache.numel() / (int64_t(h) * (d + 8));
  check(fq_tq4_compress_append(k.data_ptr(), v.data_ptr(), dtype_of(k), n, h, d, int64_t(h) * d,
                               rot.data_ptr<float>(), bk.data_ptr<float>(), int(bk.numel()),
                               bv.data_ptr<float>(), int(bv.numel()), kv_cache.data_ptr<uint8_t>(),
                               num_slots, slots.data_ptr(),
                               slots.scalar_type() == torch::kInt64 ? 1 : 0, stream_of(dev)));
}

}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "flashquant_b200: sm_100a TurboQuant KV-cache kernels behind the reference's _C names";
  m.def("tq4_compress", &tq4_compress, py::arg("x"), py::arg("rotation_T_even"),
        py::arg("rotation_T_odd"), py::arg("boundaries"), py::arg("out") = py::none());
  m.def("tq4_decompress", &tq4_decompress, py::arg("packed"), py::arg("norms"),
        py::arg("centroids"), py::arg("dtype"), py::arg("out") = py::none());
  m.def("fused_tq_attention", &fused_tq_attention, py::arg("q"), py::arg("k_packed"),
        py::arg("k_norms"), py::arg("v_packed"), py::arg("v_norms"), py::arg("centroids_k"),
        py::arg("centroids_v"), py::arg("rotation"), py::arg("sm_scale"), py::arg("is_causal"));
  m.def("split_k_paged_decode", &split_k_paged_decode, py::arg("q"), py::arg("kv_cache"),
        py::arg("block_table"), py::arg("seq_lens"), py::arg("centroids_k"),
        py::arg("centroids_v"), py::arg("rotation"), py::arg("num_kv_heads"), py::arg("head_dim"),
        py::arg("block_size"), py::arg("sm_scale") = py::none(), py::arg("out") = py::none(),
        py::arg("num_splits") = 0);
  // same callable under the name the vLLM implementation looks for
  // (src/flashquant/vllm/impl.py:57-58, called with sm_scale= and out= keywords)
  m.def("fused_paged_tq4_decode", &split_k_paged_decode, py::arg("q"), py::arg("kv_cache"),
        py::arg("block_table"), py::arg("seq_lens"), py::arg("centroids_k"),
        py::arg("centroids_v"), py::arg("rotation"), py::arg("num_kv_heads"), py::arg("head_dim"),
        py::arg("block_size"), py::arg("sm_scale") = py::none(), py::arg("out") = py::none(),
        py::arg("num_splits") = 0);
  m.def("tq4_compress_append", &tq4_compress_append, py::arg("key"), py::arg("value"),
        py::arg("kv_cache"), py::arg("slot_mapping"), py::arg("rotation"),
        py::arg("boundaries_k"), py::arg("boundaries_v") = py::none());
  m.def("tq4_compress_append_qjl", &tq4_compress_append_qjl, py::arg("key"), py::arg("value"),
        py::arg("kv_cache"), py::arg("kq_cache"), py::arg("slot_mapping"), py::arg("rotation"),
        py::arg("boundaries_k"), py::arg("centroids_k"), py::arg("boundaries_v"),
        py::arg("qjl_matrix"));
  m.def("paged_tq4_prefill", &paged_tq4_prefill, py::arg("q"), py::arg("kv_cache"),
        py::arg("block_table"), py::arg("seq_lens"), py::arg("query_start_loc"),
        py::arg("max_query_len"), py::arg("centroids_k"), py::arg("centroids_v"),
        py::arg("rotation"), py::arg("num_kv_heads"), py::arg("head_dim"), py::arg("block_size"),
        py::arg("sm_scale") = py::none(), py::arg("out") = py::none());
  m.def("decode_status", &decode_status, py::arg("like"));
  m.def("launch_count", []() { return fq_launch_count(); });
}
