"""The compressed cache behind the DynamicCache interface: oracle pinned to the reference's own
outputs (tests/golden/hf_cache.npz), host logic on the CPU, kernels against the oracle on the GPU.

Bars: codes bit-exact except next to a quantiser boundary (parity.check_codes), norms to
fp32 rounding, de-quantised keys/values within one unit in the last place of the model dtype
of the reference's values, attention within parity.attention_close.
"""

import numpy as np
import pytest
import torch

import flashquant_b200 as fq
from conftest import bf16_from_bits, load_golden
from flashquant_b200 import _native
from flashquant_b200.cache import CompressedBuffer, FlashQuantCacheError
from oracle import tq_oracle as O
from parity import attention_close, check_codes, check_norms

DEV = "cuda:0"


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a))


class MockDynamicLayer:
    def __init__(self):
        self.keys = None
        self.values = None
        self.is_initialized = False

    def lazy_initialization(self, _):
        self.is_initialized = True


class MockDynamicCache:
    """Stand-in for transformers.DynamicCache, as in the reference's tests/test_hf_cache.py."""

    def __init__(self):
        self.layers = []
        self.layer_class_to_replicate = MockDynamicLayer
        self.passed_through = 0

    def update(self, key_states, value_states, layer_idx, cache_kwargs=None):
        self.passed_through += 1
        return key_states, value_states

    def get_seq_length(self, layer_idx=0):
        return -1


def golden_inputs(z, layer):
    return [(bf16_from_bits(z[f"k_in_{layer}_{i}_bf16"]), bf16_from_bits(z[f"v_in_{layer}_{i}_bf16"]))
            for i in range(len(z["steps"]))]


def ulp_close(got, ref, dtype):
    """|got - ref| <= one unit in the last place of `dtype` at the magnitude of the entry, plus
    2^-21 of the row's length (fp32 rounding of a 128-term product before the cast; the
    reference scales by the norm after the rotation, the kernel before it)."""
    eps = {torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10, torch.float32: 0.0}[dtype]
    err = (got.float() - ref.float()).abs()
    tol = ref.float().abs() * eps + ref.float().norm(dim=-1, keepdim=True) * 2.0 ** -21 + 1e-30
    assert bool((err <= tol).all()), f"max error {err.max().item():.3e}"


# ---------------------------------------------------------------------------------------
# CPU: the oracle against the reference's outputs, and the host logic
# ---------------------------------------------------------------------------------------

def test_oracle_cache_matches_reference(consts):
    z = load_golden("hf_cache.npz")
    c4, b4 = consts["centroids_128_4"], consts["boundaries_128_4"]
    orc = O.CompressedCacheOracle(T(z["rotation_k"]), T(z["rotation_v"]), c4, b4)
    for layer in (0, 1):
        for k, v in golden_inputs(z, layer):
            ko, vo = orc.update(k, v, layer)
        kp, kn, vp, vn = orc.get_compressed(layer)
        assert orc.get_seq_length(layer) == int(z[f"seq_len_{layer}"]) == int(z["steps"].sum())
        assert (kp == T(z[f"k_packed_{layer}"])).float().mean().item() > 0.9999
        assert (vp == T(z[f"v_packed_{layer}"])).float().mean().item() > 0.9999
        torch.testing.assert_close(kn, T(z[f"k_norms_{layer}"]), rtol=1e-6, atol=0)
        torch.testing.assert_close(vn, T(z[f"v_norms_{layer}"]), rtol=1e-6, atol=0)
        assert ko.dtype == torch.bfloat16
        same_k = (ko == bf16_from_bits(z[f"k_out_{layer}_bf16"])).float().mean().item()
        same_v = (vo == bf16_from_bits(z[f"v_out_{layer}_bf16"])).float().mean().item()
        assert same_k > 0.999 and same_v > 0.999
        ulp_close(ko, bf16_from_bits(z[f"k_out_{layer}_bf16"]), torch.bfloat16)
        ulp_close(vo, bf16_from_bits(z[f"v_out_{layer}_bf16"]), torch.bfloat16)


def test_oracle_two_rotation_attention_equals_attention_over_dequantised(consts):
    # <q Pi_k^T, c[idx] n> = <q, (c[idx] n) Pi_k>: attending in the rotated spaces and rotating
    # the output back by Pi_v equals plain attention over the de-quantised keys and values
    z = load_golden("hf_cache.npz")
    c4 = consts["centroids_128_4"]
    rk, rv = T(z["rotation_k"]), T(z["rotation_v"])
    kp, kn = T(z["k_packed_0"]), T(z["k_norms_0"])
    vp, vn = T(z["v_packed_0"]), T(z["v_norms_0"])
    q = torch.randn(2, 4, 25, 128, generator=torch.Generator().manual_seed(5))
    got = O.fused_tq_attention(q, kp, kn, vp, vn, c4, c4, rk, is_causal=True, rotation_v=rv)
    kd = O.mse_dequantize(O.nibble_unpack(kp).long(), kn, rk, c4)
    vd = O.mse_dequantize(O.nibble_unpack(vp).long(), vn, rv, c4)
    ref = O.attention(q, kd, vd, None, True)
    torch.testing.assert_close(got, ref, rtol=1e-4, atol=1e-5)


def test_buffer_append_get_reset_overflow():
    # the cases of the reference's tests/test_buffer_pool.py
    buf = CompressedBuffer(max_seq=8, batch=1, heads=2, half_dim=4, dtype=torch.uint8,
                           device=torch.device("cpu"))
    idx = torch.arange(1 * 2 * 3 * 4, dtype=torch.uint8).reshape(1, 2, 3, 4)
    nrm = torch.arange(6, dtype=torch.float32).reshape(1, 2, 3, 1)
    buf.append(idx, nrm)
    assert buf.length == 3
    gi, gn = buf.get()
    assert torch.equal(gi, idx) and torch.equal(gn, nrm)
    ptr = buf._indices.data_ptr()
    buf.append(idx[:, :, :1], nrm[:, :, :1])
    assert buf.length == 4 and buf._indices.data_ptr() == ptr  # no reallocation, no copy
    gi, _ = buf.get()
    assert gi.data_ptr() == ptr and torch.equal(gi[:, :, 3], idx[:, :, 0])
    with pytest.raises(RuntimeError, match="overflow"):
        buf.append(torch.zeros(1, 2, 5, 4, dtype=torch.uint8), torch.zeros(1, 2, 5, 1))
    assert buf.length == 4  # a refused append claims nothing
    buf.reset()
    assert buf.length == 0 and buf.get()[0].shape == (1, 2, 0, 4)
    assert buf.reserve(8) == 0 and buf.length == 8


def test_wrapper_lifecycle_on_the_host():
    cache = MockDynamicCache()
    own_update = cache.update
    with pytest.raises(ValueError, match="even head_dim"):
        fq.CompressedDynamicCache(MockDynamicCache(), head_dim=127, bits=4)
    w = fq.CompressedDynamicCache(cache, head_dim=128, bits=4, max_seq_len=32)
    with pytest.raises(FlashQuantCacheError, match="already wrapped"):
        fq.CompressedDynamicCache(cache, head_dim=128, bits=4)
    assert cache.get_seq_length(0) == 0
    with pytest.raises(FlashQuantCacheError, match="has not been initialized"):
        w.get_compressed(0)
    assert w.compression_stats() == {} and w.vram_bytes() == 0
    # disabled: straight through to the cache's own methods
    w.disable()
    k = torch.zeros(1, 1, 2, 128)
    assert cache.update(k, k, 0)[0] is k and cache.passed_through == 1
    assert cache.get_seq_length(0) == -1
    w.enable()
    # enabled: CPU tensors are refused loudly, there is no CPU path
    with pytest.raises(_native.FlashQuantNativeError):
        cache.update(k, k, 0)
    w.restore()
    assert cache.update == own_update and cache._flashquant_wrapped is False
    with fq.CompressedDynamicCache(cache, head_dim=128, bits=4) as again:
        assert cache.update == again._compressed_update
    assert cache.update == own_update
    assert w.rotation_k.shape == (128, 128) and not torch.equal(w.rotation_k, w.rotation_v)
    assert w.centroids_k.numel() == 16


# ---------------------------------------------------------------------------------------
# GPU: the kernels behind the wrapper against the oracle and the reference's outputs
# ---------------------------------------------------------------------------------------

def wrap_with_rotations(cache, rotation_k, rotation_v, **kw):
    """Wrapper whose rotations are the stored ones (LAPACK's QR differs between machines in
    the last bits, and codes next to a boundary follow the matrix)."""
    w = fq.CompressedDynamicCache(cache, head_dim=rotation_k.shape[0], **kw)
    w.key_compressor.quantizer.rotation = rotation_k
    w.value_compressor.quantizer.rotation = rotation_v
    return w


@pytest.mark.gpu
def test_update_matches_reference_outputs(consts):
    z = load_golden("hf_cache.npz")
    b4 = consts["boundaries_128_4"]
    rk, rv = T(z["rotation_k"]), T(z["rotation_v"])
    cache = MockDynamicCache()
    launches0 = _native.load().fq_launch_count()
    with wrap_with_rotations(cache, rk, rv, bits=4, max_seq_len=64) as w:
        for layer in (0, 1):
            ins = golden_inputs(z, layer)
            for k, v in ins:
                ko, vo = cache.update(k.to(DEV), v.to(DEV), layer)
            assert cache.get_seq_length(layer) == int(z[f"seq_len_{layer}"])
            kp, kn, vp, vn = w.get_compressed(layer)
            assert kp.shape == (2, 2, 25, 64) and kn.shape == (2, 2, 25, 1)
            assert kp.data_ptr() == w._compressed_keys[layer].buffer._indices.data_ptr()  # views
            k_all = torch.cat([k for k, _ in ins], dim=2)
            v_all = torch.cat([v for _, v in ins], dim=2)
            check_codes(kp, k_all.float(), rk, b4, T(z[f"k_packed_{layer}"]))
            check_codes(vp, v_all.float(), rv, b4, T(z[f"v_packed_{layer}"]))
            check_norms(kn, T(z[f"k_norms_{layer}"]))
            check_norms(vn, T(z[f"v_norms_{layer}"]))
            assert ko.dtype == torch.bfloat16 and ko.shape == (2, 2, 25, 128)
            # where the codes agree the de-quantised values agree to an ulp of bf16
            same_k = (kp.cpu() == T(z[f"k_packed_{layer}"])).all(dim=-1, keepdim=True)
            ref_k = bf16_from_bits(z[f"k_out_{layer}_bf16"])
            ulp_close(torch.where(same_k, ko.cpu(), ref_k), ref_k, torch.bfloat16)
            same_v = (vp.cpu() == T(z[f"v_packed_{layer}"])).all(dim=-1, keepdim=True)
            ref_v = bf16_from_bits(z[f"v_out_{layer}_bf16"])
            ulp_close(torch.where(same_v, vo.cpu(), ref_v), ref_v, torch.bfloat16)
            assert cache.layers[layer].keys.shape == (2, 2, 25, 128)
        assert w.compressed_vram_bytes() == int(z["compressed_vram_bytes"])
        assert w.baseline_vram_bytes() == int(z["baseline_vram_bytes"])
        assert w.vram_bytes() == int(z["vram_bytes"])
        assert w.compression_stats()["compression_ratio"] == 3.76
    # per update of a few rows: two compress launches, two back-rotations that expand the codes
    assert _native.load().fq_launch_count() - launches0 == 2 * 4 * 4


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,dim,bits", [(torch.float16, 128, 4), (torch.float32, 128, 3),
                                            (torch.bfloat16, 64, 4)])
def test_update_against_oracle(consts, dtype, dim, bits):
    cent, bnd = O.lloyd_max_codebook(dim, bits)
    rk, rv = O.haar_rotation(dim, 42), O.haar_rotation(dim, 43)
    orc = O.CompressedCacheOracle(rk, rv, cent, bnd)
    cache = MockDynamicCache()
    g = torch.Generator().manual_seed(77)
    with wrap_with_rotations(cache, rk, rv, bits=bits, max_seq_len=1300) as w:
        for s_new in (1200, 1, 1, 37):  # 18 000 vectors: the bulk kernel; then small appends
            k = (torch.randn(3, 5, s_new, dim, generator=g) * 3.0).to(dtype)
            v = torch.randn(3, 5, s_new, dim, generator=g).to(dtype)
            ko, vo = cache.update(k.to(DEV), v.to(DEV), 0)
            rko, rvo = orc.update(k, v, 0)
        kp, kn, vp, vn = w.get_compressed(0)
        rkp, rkn, rvp, rvn = orc.get_compressed(0)
        assert cache.get_seq_length(0) == orc.get_seq_length(0) == 1239
        check_norms(kn, rkn)
        check_norms(vn, rvn)
        match_k = (kp.cpu() == rkp).float().mean().item()
        match_v = (vp.cpu() == rvp).float().mean().item()
        assert match_k > 0.9995 and match_v > 0.9995, (match_k, match_v)
        diff = (O.nibble_unpack(kp.cpu()).int() - O.nibble_unpack(rkp).int()).abs().max().item()
        assert diff <= 1
        same_k = (kp.cpu() == rkp).all(dim=-1, keepdim=True)
        ulp_close(torch.where(same_k, ko.cpu(), rko), rko, dtype)
        same_v = (vp.cpu() == rvp).all(dim=-1, keepdim=True)
        ulp_close(torch.where(same_v, vo.cpu(), rvo), rvo, dtype)
        with pytest.raises(RuntimeError, match="overflow"):
            cache.update(torch.zeros(3, 5, 62, dim, dtype=dtype, device=DEV),
                         torch.zeros(3, 5, 62, dim, dtype=dtype, device=DEV), 0)
        assert cache.get_seq_length(0) == 1239


@pytest.mark.gpu
@pytest.mark.parametrize("n_prompt,causal", [(200, True), (129, False)])
def test_fused_attention_over_the_cache(consts, n_prompt, causal):
    c4, b4 = consts["centroids_128_4"], consts["boundaries_128_4"]
    rk, rv = O.haar_rotation(128, 42), O.haar_rotation(128, 43)
    orc = O.CompressedCacheOracle(rk, rv, c4, b4)
    cache = MockDynamicCache()
    g = torch.Generator().manual_seed(n_prompt)
    b, hq, hkv = 2, 8, 2
    with wrap_with_rotations(cache, rk, rv, bits=4, max_seq_len=333) as w:
        w.fused_mode = True
        k = torch.randn(b, hkv, n_prompt, 128, generator=g).to(torch.bfloat16)
        v = torch.randn(b, hkv, n_prompt, 128, generator=g).to(torch.bfloat16)
        ko, vo = cache.update(k.to(DEV), v.to(DEV), 0)
        assert ko.shape == k.shape and w._decompressed_k[0] is None  # nothing de-quantised
        orc.update(k, v, 0)
        q = torch.randn(b, hq, n_prompt, 128, generator=g).to(torch.bfloat16)
        out = w.fused_attention(q.to(DEV), 0, is_causal=causal)
        # the oracle attends over ITS codes; use the GPU's codes so that a code next to a
        # boundary does not count as an attention error
        kp, kn, vp, vn = (t.cpu().contiguous() for t in w.get_compressed(0))
        ref32, ref = O.fused_tq_attention_stages(q, kp, kn, vp, vn, c4, c4, rk, is_causal=causal,
                                                 rotation_v=rv)
        attention_close(out.cpu(), ref, ref32, rv, rounds_rotated=False, rtol=2.0 ** -10)
        # decode steps: one token in, one query row over everything so far
        for _ in range(3):
            k1 = torch.randn(b, hkv, 1, 128, generator=g).to(torch.bfloat16)
            v1 = torch.randn(b, hkv, 1, 128, generator=g).to(torch.bfloat16)
            cache.update(k1.to(DEV), v1.to(DEV), 0)
            q1 = torch.randn(b, hq, 1, 128, generator=g).to(torch.bfloat16)
            out1 = w.fused_attention(q1.to(DEV), 0, is_causal=True)
            kp, kn, vp, vn = (t.cpu().contiguous() for t in w.get_compressed(0))
            ref32, ref1 = O.fused_tq_attention_stages(q1, kp, kn, vp, vn, c4, c4, rk,
                                                      is_causal=True, rotation_v=rv)
            attention_close(out1.cpu(), ref1, ref32, rv, rounds_rotated=False, rtol=2.0 ** -10)
        assert fq.kernels.attention_workspace_status(torch.device(DEV)) == 0


@pytest.mark.gpu
def test_compress_into_equals_compress_then_copy(consts):
    b4 = consts["boundaries_128_4"]
    rot = consts["rotation_128_42"]
    g = torch.Generator().manual_seed(3)
    x = torch.randn(2, 3, 50, 128, generator=g).to(torch.bfloat16).to(DEV)
    packed = torch.full((2, 3, 90, 64), 0xEE, dtype=torch.uint8, device=DEV)
    norms = torch.full((2, 3, 90, 1), -1.0, device=DEV)
    fq.tq4_compress_into(x, rot, b4, packed, norms, 17)
    p2, n2 = fq.tq4_compress(x.reshape(-1, 1, 128), rot, b4)
    assert torch.equal(packed[:, :, 17:67], p2.reshape(2, 3, 50, 64))
    assert torch.equal(norms[:, :, 17:67], n2.reshape(2, 3, 50, 1))
    # rows outside the window are untouched
    assert bool((packed[:, :, :17] == 0xEE).all()) and bool((packed[:, :, 67:] == 0xEE).all())
    assert bool((norms[:, :, :17] == -1).all()) and bool((norms[:, :, 67:] == -1).all())
    with pytest.raises(_native.FlashQuantNativeError):
        fq.tq4_compress_into(x, rot, b4, packed, norms, 41)  # 41 + 50 > 90
    # nothing to do
    fq.tq4_compress_into(x[:, :, :0], rot, b4, packed, norms, 90)


@pytest.mark.gpu
@pytest.mark.parametrize("dim,n_vec,dtype", [(128, 5000, torch.bfloat16), (128, 33, torch.float32),
                                             (64, 3000, torch.float16), (64, 7, torch.bfloat16)])
def test_decompress_to_the_original_space(consts, dim, n_vec, dtype):
    # both rotation kernels (few rows / many rows) at both head sizes
    cent, bnd = O.lloyd_max_codebook(dim, 4)
    rot = O.haar_rotation(dim, 42)
    x = torch.randn(n_vec, 1, dim, generator=torch.Generator().manual_seed(n_vec)) * 2.0
    packed, norms = O.compress(x, rot, bnd)
    ref = O.mse_dequantize(O.nibble_unpack(packed).long(), norms, rot, cent).to(dtype)
    got = fq.tq4_decompress_original(packed.to(DEV), norms.to(DEV), cent, rot, dtype=dtype)
    assert got.shape == (n_vec, 1, dim) and got.dtype == dtype
    ulp_close(got.cpu(), ref, dtype)
    empty = fq.tq4_decompress_original(packed[:0].to(DEV), norms[:0].to(DEV), cent, rot, dtype=dtype)
    assert empty.shape == (0, 1, dim)


@pytest.mark.gpu
def test_update_edge_cases(consts):
    rk, rv = O.haar_rotation(128, 42), O.haar_rotation(128, 43)
    cache = MockDynamicCache()
    with wrap_with_rotations(cache, rk, rv, bits=4, max_seq_len=40) as w:
        k = torch.randn(1, 2, 5, 128, generator=torch.Generator().manual_seed(1)).half().to(DEV)
        ko, _ = cache.update(k, k, 3)  # layers 0..2 stay empty
        assert cache.get_seq_length(3) == 5 and cache.get_seq_length(0) == 0
        assert len(cache.layers) == 4
        with pytest.raises(FlashQuantCacheError):
            w.get_compressed(1)
        # an update without tokens changes nothing
        ko2, _ = cache.update(k[:, :, :0], k[:, :, :0], 3)
        assert cache.get_seq_length(3) == 5 and torch.equal(ko2, ko)
        # the running tensor outgrows its first allocation (16 rows) and keeps its contents
        for _ in range(3):
            ko3, _ = cache.update(k, k, 3)
        assert ko3.shape == (1, 2, 20, 128) and torch.equal(ko3[:, :, :5], ko)
        assert torch.equal(ko3[:, :, 15:20], ko)  # same tokens in, same values out
        # a zero vector: norm 0, every coordinate on the middle code, de-quantised to zero
        z = torch.zeros(1, 2, 1, 128, dtype=torch.float16, device=DEV)
        kz, _ = cache.update(z, z, 3)
        kp, kn, _, _ = w.get_compressed(3)
        assert bool((kn[:, :, -1] == 0).all()) and bool((kp[:, :, -1] == 0x88).all())
        assert bool((kz[:, :, -1] == 0).all())
        # mixed dtypes are refused before anything is written
        with pytest.raises(ValueError):
            cache.update(k, k.float(), 3)
        with pytest.raises(ValueError):
            cache.update(k.float(), k.float(), 3)
        assert cache.get_seq_length(3) == 21
    # native argument checks
    lib = _native.load()
    assert lib.fq_cache_update_workspace_bytes(6, 5, 128) == 6 * 5 * 128 * 4
    tk, tv = w.key_compressor.tables(torch.device(DEV)), w.value_compressor.tables(torch.device(DEV))
    kb, vb = w._compressed_keys[3].buffer, w._compressed_values[3].buffer
    out = torch.empty(1, 2, 64, 128, dtype=torch.float16, device=DEV)
    small = torch.empty(16, dtype=torch.uint8, device=DEV)
    with pytest.raises((_native.FlashQuantNativeError, ValueError)):
        fq.kernels.cache_update(k, k, tk, tv, kb._indices, kb._norms, vb._indices, vb._norms, 0,
                                out, out.clone(), 0, small)
    with pytest.raises(_native.FlashQuantNativeError):  # 38 + 5 > 40
        fq.kernels.cache_update(k, k, tk, tv, kb._indices, kb._norms, vb._indices, vb._norms, 38)
    with pytest.raises(ValueError, match="capacity"):
        fq.fused_tq_attention_kv(k, kb._indices[:, :, :5], kb._norms[:, :, :5],
                                 vb._indices[:, :, :5].contiguous(), vb._norms[:, :, :5].contiguous(),
                                 tk[3], tv[3], tk[4], tv[4])
