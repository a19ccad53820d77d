"""The reference-side binding on the GPU: ``flashquant_b200._C`` is the pybind11 module that
takes the place of ``flashquant._C``, and the calls below have exactly the positional and
keyword forms of the reference's own call sites (src/flashquant/kernels/compress.py:90-92,
decompress.py:77, attention.py:93-97, paged_decode.py:105-110, src/flashquant/vllm/impl.py:380-393),
with the constants as CPU tensors where the reference keeps them on the CPU and ``out=`` a slice
of a larger tensor where vLLM passes one.  Results are checked against the reference-made
fixtures and the oracle.
"""

import numpy as np
import pytest
import torch

from conftest import bf16_from_bits, load_golden
from flashquant_b200 import workloads as W
from oracle import tq_oracle as O
from parity import attention_close, check_codes, check_gamma, check_norms, check_signs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def _C():
    from flashquant_b200 import build
    build.build_pybind()
    from flashquant_b200 import _C as mod
    return mod


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def test_compress_and_decompress_as_the_dispatchers_call_them(_C, consts):
    rot, b4, c4 = consts["rotation_128_0"], consts["boundaries_128_4"], consts["centroids_128_4"]
    even, odd = O.split_rotation_T(rot)                       # CPU tensors, as in compress.py:86-89
    x = torch.randn(300, 8, 128, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16)
    packed, norms = _C.tq4_compress(x.to(DEV), even, odd, b4, None)
    ref_p, ref_n = O.compress(x.float(), rot, b4)
    assert packed.shape == (300, 8, 64) and packed.dtype == torch.uint8
    assert norms.shape == (300, 8, 1) and norms.dtype == torch.float32
    check_codes(packed, x.float(), rot, b4, ref_p)
    check_norms(norms, ref_n)
    # out=(packed, norms): written in place and returned (CUDA-graph capture in the vLLM path)
    bufs = (torch.empty_like(packed), torch.empty_like(norms))
    p2, n2 = _C.tq4_compress(x.to(DEV), even, odd, b4, bufs)
    assert p2.data_ptr() == bufs[0].data_ptr() and torch.equal(p2, packed) and torch.equal(n2, norms)
    for dt in (torch.float16, torch.bfloat16, torch.float32):
        out = _C.tq4_decompress(packed, norms, c4, dt, None)   # decompress.py:77
        assert out.dtype == dt and out.shape == (300, 8, 128)
        assert torch.equal(out.cpu(), O.decompress(packed.cpu(), norms.cpu(), c4).to(dt))
    buf = torch.empty(300, 8, 128, dtype=torch.float16, device=DEV)
    assert _C.tq4_decompress(packed, norms, c4, torch.float16, buf).data_ptr() == buf.data_ptr()


def test_fused_attention_on_the_reference_fixture(_C, consts):
    z = load_golden("prefill.npz")
    q = bf16_from_bits(z["q_bf16"])
    case = (T(z["k_packed"]), T(z["k_norms"]), T(z["v_packed"]), T(z["v_norms"]))
    c3, c4, rot = consts["centroids_128_3"], consts["centroids_128_4"], consts["rotation_128_0"]
    for causal, key in ((True, "out_causal_bf16"), (False, "out_full_bf16")):
        out = _C.fused_tq_attention(q.to(DEV), *(t.to(DEV) for t in case), c3, c4, rot,
                                    1.0 / np.sqrt(128), causal)           # attention.py:93-97
        ref32, ref = O.fused_tq_attention_stages(q, *case, c3, c4, rot, is_causal=causal)
        assert torch.equal(ref.view(torch.int16), bf16_from_bits(z[key]).view(torch.int16))
        attention_close(out, ref, ref32, rot, rounds_rotated=False, rtol=2.0 ** -10)


def test_paged_decode_positional_and_vllm_keyword_forms(_C, consts):
    z = load_golden("paged_decode.npz")
    cache, bt, sl = T(z["kv_cache"]), T(z["block_table"]), T(z["seq_lens"])
    c3, c4, rot = consts["centroids_128_3"], consts["centroids_128_4"], consts["rotation_128_0"]
    hkv, d, bs = int(z["h_kv"]), int(z["d"]), int(z["block_size"])
    q = bf16_from_bits(z["q_bf16"])
    ref32, ref = O.split_k_paged_decode_stages(q, cache, bt, sl, c3, c4, rot, hkv, d, bs)
    assert torch.equal(ref.view(torch.int16), bf16_from_bits(z["out_bf16"]).view(torch.int16))
    dev_args = (q.to(DEV), cache.to(DEV), bt.to(DEV), sl.to(DEV))
    # paged_decode.py:105-110: thirteen positional arguments, constants on the CPU
    out = _C.split_k_paged_decode(*dev_args, c3, c4, rot, hkv, d, bs, 1.0 / np.sqrt(d), None, 0)
    attention_close(out, ref, ref32, rot)
    # vllm/impl.py:380-393: ten positional arguments, sm_scale= and out=, the output a slice of
    # a larger (tokens, H_q * D) tensor
    n, hq = q.shape[0], q.shape[1]
    big = torch.full((n + 5, hq * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    ret = _C.fused_paged_tq4_decode(*dev_args, c3, c3.new_tensor(c4), rot, hkv, d, bs,
                                    sm_scale=1.0 / np.sqrt(d), out=big[:n])
    assert ret.data_ptr() == big.data_ptr()
    attention_close(big[:n].view(n, hq, d), ref, ref32, rot)
    assert torch.isnan(big[n:].float()).all()                # nothing written past the slice
    assert _C.decode_status(dev_args[0]) == 0
    # a second call with the same CPU constants finds their device copies again
    before = _C.launch_count()
    _C.split_k_paged_decode(*dev_args, c3, c4, rot, hkv, d, bs, None, None, 2)
    assert _C.launch_count() == before + 1                   # one launch: the decode itself


def test_compress_append_entries(_C, consts):
    rot, S = consts["rotation_128_0"], consts["qjl_128_0"]
    b3, c3 = consts["boundaries_128_3"], consts["centroids_128_3"]
    b4 = consts["boundaries_128_4"]
    h, d = 8, 128
    w = W.append_workload(n_tokens=700, num_slots=2048)
    cache = torch.zeros(128, 16, h * (d + 8), dtype=torch.uint8, device=DEV)
    plane = torch.zeros(128, 16, h * (d // 8 + 4), dtype=torch.uint8, device=DEV)
    _C.tq4_compress_append_qjl(w.key.to(DEV), w.value.to(DEV), cache, plane, w.slot_mapping.to(DEV),
                               rot, b3, c3, b4, S)
    ref = torch.zeros(128, 16, h * (d + 8), dtype=torch.uint8)
    O.compress_and_store(w.key, w.value, ref, w.slot_mapping, rot, b3, b4)
    rows, want = cache.cpu().view(-1, h * (d + 8))[w.slot_mapping], ref.view(-1, h * (d + 8))[w.slot_mapping]
    a = h * d // 2
    check_codes(rows[:, :a].reshape(-1, h, d // 2), w.key.float(), rot, b3, want[:, :a].reshape(-1, h, d // 2))
    knorm = rows[:, a:a + 4 * h].contiguous().view(torch.float32)
    check_norms(knorm, want[:, a:a + 4 * h].contiguous().view(torch.float32))
    idx, norms, signs, gamma = O.prod_quantize(w.key, rot, c3, b3, S)
    got = plane.cpu().view(-1, h * (d // 8 + 4))[w.slot_mapping]
    sb = h * d // 8
    codes = O.nibble_unpack(rows[:, :a].reshape(-1, h, d // 2))
    check_gamma(got[:, sb:].contiguous().view(torch.float32), gamma, w.key.float(), codes, idx, knorm, rot, c3)
    check_signs(got[:, :sb].reshape(-1, h, d // 8), signs, w.key.float(), codes, idx, knorm, rot, c3, S)
    # the one-stage entry writes the same main rows
    cache2 = torch.zeros_like(cache)
    _C.tq4_compress_append(w.key.to(DEV), w.value.to(DEV), cache2, w.slot_mapping.to(DEV), rot, b3, b4)
    assert torch.equal(cache2, cache)


def test_paged_prefill_with_vllm_metadata_names(_C, consts):
    """``_C.paged_tq4_prefill`` with the metadata the reference's prefill path hands to
    flash_attn_varlen_func (query_start_loc, max_query_len, seq_lens, block_table;
    src/flashquant/vllm/impl.py:477-509), constants on the CPU, ``out=`` a slice."""
    rot, c3, c4 = consts["rotation_128_0"], consts["centroids_128_3"], consts["centroids_128_4"]
    hq, hkv, d, bs = 32, 8, 128, 16
    seq_lens, chunks = [200, 77, 1030], [40, 77, 129]
    w = W.decode_workload(seq_lens=seq_lens, num_q_heads=hq, num_kv_heads=hkv, cfg=41)
    k, v = W.make_kv(w.total_tokens, hkv, d, 41)
    cache = torch.zeros(w.num_blocks, bs, hkv * (d + 8), dtype=torch.uint8, device=DEV)
    _C.tq4_compress_append(k.to(DEV), v.to(DEV), cache, w.slot_mapping.to(DEV), rot,
                           consts["boundaries_128_3"], consts["boundaries_128_4"])
    cu = torch.zeros(4, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(chunks), 0)
    n = int(cu[-1])
    q = torch.randn(n, hq, d, generator=torch.Generator().manual_seed(41)).to(torch.bfloat16)
    output = torch.zeros(n + 16, hq * d, dtype=torch.bfloat16, device=DEV)   # padded, 2-D
    ret = _C.paged_tq4_prefill(q.to(DEV), cache, w.block_table.to(DEV), w.seq_lens.to(DEV),
                               cu.to(DEV), max(chunks), c3, c4, rot, hkv, d, bs,
                               sm_scale=1.0 / d ** 0.5, out=output[:n])
    assert ret.data_ptr() == output.data_ptr() and (output[n:] == 0).all()
    ref32, ref = O.paged_prefill_varlen_stages(q, cache.cpu(), w.block_table, w.seq_lens, cu, c3, c4,
                                               rot, hkv, d, bs)
    attention_close(output[:n].view(n, hq, d), ref, ref32, rot, rtol=2.0 ** -10)
