"""GPU parity of compress / decompress / two-stage quantiser / compress-on-append.

Bars: codes and sign bits bit-exact except for coordinates within 1e-6 of a boundary
(mismatch fraction <= 1e-4); norms and gamma to 1e-6 relative.
"""

import numpy as np
import pytest
import torch

import flashquant_b200 as fq
from conftest import bf16_from_bits, load_golden
from flashquant_b200 import workloads as W
from oracle import tq_oracle as O
from parity import check_codes, check_gamma, check_norms, check_signs, unpack

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a))


@pytest.fixture(scope="module")
def C(consts):
    return consts


def test_compress_golden_fp32_and_bf16(C):
    z = load_golden("quantize.npz")
    rot, b4 = C["rotation_128_0"], C["boundaries_128_4"]
    v = T(z["v"])
    packed, norms = fq.tq4_compress(v.to(DEV), rot, b4)
    assert packed.shape == (24, 2, 64) and norms.shape == (24, 2, 1)
    check_codes(packed, v, rot, b4, T(z["v_packed"]))
    check_norms(norms, T(z["v_norms_c"]))
    vb = bf16_from_bits(z["vb_bf16"])
    packed, norms = fq.tq4_compress(vb.to(DEV), rot, b4)
    check_codes(packed, vb.float(), rot, b4, T(z["vb_packed"]))
    check_norms(norms, T(z["vb_norms"]))
    # zero vector: 4-bit middle boundary is negative -> code 8 everywhere, norm 0
    assert (unpack(packed)[0, 0] == 8).all() and norms[0, 0].item() == 0.0


def test_compress_out_buffers_and_presplit_rotation(C):
    rot, b4 = C["rotation_128_0"], C["boundaries_128_4"]
    x = torch.randn(40, 3, 128, generator=torch.Generator().manual_seed(11))
    even, odd = O.split_rotation_T(rot)
    out = (torch.empty(40, 3, 64, dtype=torch.uint8, device=DEV),
           torch.empty(40, 3, 1, dtype=torch.float32, device=DEV))
    p, n = fq.tq4_compress(x.to(DEV), rot, b4, rotation_T_even=even.to(DEV),
                           rotation_T_odd=odd.to(DEV), out=out)
    assert p.data_ptr() == out[0].data_ptr() and n.data_ptr() == out[1].data_ptr()
    pr, nr = O.compress(x, rot, b4)
    check_codes(p, x, rot, b4, pr)
    check_norms(n, nr)


@pytest.mark.parametrize("dim,bits,dtype", [(128, 4, torch.bfloat16), (128, 3, torch.float16),
                                            (128, 2, torch.float32), (64, 4, torch.bfloat16),
                                            (64, 3, torch.float32)])
def test_compress_vs_oracle(C, dim, bits, dtype):
    rot = C.get(f"rotation_{dim}_0")
    bnd = C[f"boundaries_{dim}_{bits}"] if f"boundaries_{dim}_{bits}" in C else \
        O.lloyd_max_codebook(dim, bits)[1]
    g = torch.Generator().manual_seed(100 + dim + bits)
    x = torch.randn(3000, 4, dim, generator=g)
    x[..., W.outlier_channels(dim)] *= 10
    x = x.to(dtype)
    p, n = fq.tq4_compress(x.to(DEV), rot, bnd)
    pr, nr = O.compress(x, rot, bnd)
    check_codes(p, x.float(), rot, bnd, pr)
    check_norms(n, nr)


def test_compress_ragged_counts(C):
    rot, b4 = C["rotation_128_0"], C["boundaries_128_4"]
    for n in (1, 7, 63, 64, 65, 129):
        x = torch.randn(n, 1, 128, generator=torch.Generator().manual_seed(n))
        p, nn = fq.tq4_compress(x.to(DEV), rot, b4)
        pr, nr = O.compress(x, rot, b4)
        check_codes(p, x, rot, b4, pr)
        check_norms(nn, nr)
    p, nn = fq.tq4_compress(torch.empty(0, 2, 128, device=DEV), rot, b4)
    assert p.shape == (0, 2, 64)


def test_decompress_golden_and_dtypes(C):
    z = load_golden("quantize.npz")
    c4 = C["centroids_128_4"]
    packed, norms = T(z["v_packed"]).to(DEV), T(z["v_norms_c"]).to(DEV)
    ref = T(z["v_decomp"])
    out = fq.tq4_decompress(packed, norms, c4, dtype=torch.float32)
    assert torch.equal(out.cpu(), ref)  # LUT * norm in fp32: bit-exact
    for dt in (torch.float16, torch.bfloat16):
        out = fq.tq4_decompress(packed, norms, c4, dtype=dt)
        assert torch.equal(out.cpu(), ref.to(dt))
    buf = torch.empty(24, 2, 128, dtype=torch.float16, device=DEV)
    assert fq.tq4_decompress(packed, norms, c4, dtype=torch.float16, out=buf).data_ptr() == buf.data_ptr()
    # 8-entry table (3-bit codes) and head_dim 64
    c3 = C["centroids_64_3"]
    idx = torch.randint(0, 8, (50, 2, 64), generator=torch.Generator().manual_seed(3))
    pk = O.nibble_pack(idx)
    nn = torch.rand(50, 2, 1) + 0.5
    out = fq.tq4_decompress(pk.to(DEV), nn.to(DEV), c3, dtype=torch.float32)
    assert torch.equal(out.cpu(), O.decompress(pk, nn, c3))


def test_prod_quantize_golden(C):
    z = load_golden("quantize.npz")
    rot, b3, c3, S = C["rotation_128_0"], C["boundaries_128_3"], C["centroids_128_3"], C["qjl_128_0"]
    k = T(z["k"])
    packed, norms, bits, gamma = fq.tq_prod_quantize(k.to(DEV), rot, b3, c3, S)
    check_codes(packed, k, rot, b3, O.nibble_pack(T(z["k_idx"])))
    check_norms(norms, T(z["k_norms"]))
    codes = O.nibble_unpack(packed.cpu())
    check_gamma(gamma, T(z["k_gamma"]), k.float(), codes, T(z["k_idx"]), norms.cpu(), rot, c3)
    check_signs(bits, T(z["k_signs"]), k.float(), codes, T(z["k_idx"]), norms.cpu(), rot, c3, S)
    signs = O.sign_bits_unpack(bits.cpu())
    # zero vector: all signs +1, gamma 0
    assert (signs[0, 1] == 1).all() and gamma[0, 1].item() == 0.0


def test_prod_quantize_vs_oracle_and_host_class(C):
    rot, b3, c3, S = C["rotation_128_0"], C["boundaries_128_3"], C["centroids_128_3"], C["qjl_128_0"]
    k, _ = W.make_kv(2048, 8, 128, cfg=2)
    idx, norms, signs, gamma = O.prod_quantize(k, rot, c3, b3, S)
    packed, n2, bits, g2 = fq.tq_prod_quantize(k.to(DEV), rot, b3, c3, S)
    check_codes(packed, k.float(), rot, b3, O.nibble_pack(idx))
    check_norms(n2, norms)
    codes = O.nibble_unpack(packed.cpu())
    check_gamma(g2, gamma, k.float(), codes, idx, n2.cpu(), rot, c3)
    check_signs(bits, signs, k.float(), codes, idx, n2.cpu(), rot, c3, S)
    # host class mirror
    q = fq.TurboQuantProd(128, 4, seed=0)
    q.mse_quantizer.rotation = rot  # identical matrices (QR is not reproducible across hosts)
    i2, n3, s2, g3 = q.quantize(k[:64].to(DEV))
    assert i2.dtype == torch.int64 and s2.shape == (64, 8, 128)
    assert (i2.cpu() != idx[:64]).float().mean().item() <= 1e-4
    assert ((s2.cpu() != signs[:64]).float().mean().item()) <= 1e-4


def test_mse_host_class_roundtrip(C):
    q = fq.TurboQuantMSE(128, 4, seed=0)
    q.rotation = C["rotation_128_0"]
    x = torch.randn(33, 5, 128, generator=torch.Generator().manual_seed(9))
    idx, norms = q.quantize(x.to(DEV))
    ri, rn, _ = O.mse_quantize(x, q.rotation, q.boundaries)
    assert (idx.cpu() != ri).float().mean().item() <= 1e-4
    check_norms(norms, rn)
    deq = q.dequantize(idx, norms).cpu()
    ref = O.mse_dequantize(ri, rn, q.rotation, q.centroids)
    assert (deq - ref).abs().max().item() < 2e-4 * ref.abs().max().item() + 1e-5
    cos = torch.nn.functional.cosine_similarity(deq.flatten(), x.flatten(), dim=0).item()
    assert cos > 0.93  # the reference's own bar for d=128, 4 bits


def _check_rows(cache_gpu, cache_ref, slots, key, value, rot, bk, bv, h, d):
    got = cache_gpu.cpu().view(-1, h * (d + 8))
    ref = cache_ref.view(-1, h * (d + 8))
    keep = slots >= 0
    s = slots[keep].long()
    a = h * d // 2
    check_codes(got[s, :a].reshape(-1, h, d // 2), key[keep].float(), rot, bk,
                ref[s, :a].reshape(-1, h, d // 2))
    check_codes(got[s, a + 4 * h:2 * a + 4 * h].reshape(-1, h, d // 2), value[keep].float(), rot,
                bv, ref[s, a + 4 * h:2 * a + 4 * h].reshape(-1, h, d // 2))
    check_norms(got[s, a:a + 4 * h].contiguous().view(torch.float32),
                ref[s, a:a + 4 * h].contiguous().view(torch.float32))
    check_norms(got[s, 2 * a + 4 * h:].contiguous().view(torch.float32),
                ref[s, 2 * a + 4 * h:].contiguous().view(torch.float32))
    mask = torch.ones(got.shape[0], dtype=torch.bool)
    mask[s] = False
    assert torch.equal(got[mask], ref[mask]), "a slot outside slot_mapping was written"


def test_append_small_with_padding_and_int32_slots(C):
    rot, b4 = C["rotation_128_0"], C["boundaries_128_4"]
    h, d = 2, 128
    g = torch.Generator().manual_seed(5)
    key = torch.randn(70, h, d, generator=g).to(torch.bfloat16)
    val = torch.randn(70, h, d, generator=g).to(torch.bfloat16)
    slots = torch.randperm(96, generator=g)[:70]
    slots[5] = -1
    slots[44] = -1
    for dt in (torch.int64, torch.int32):
        ref = torch.full((6, 16, h * (d + 8)), 0xAB, dtype=torch.uint8)
        O.compress_and_store(key, val, ref, slots, rot, b4)
        cache = torch.full((6, 16, h * (d + 8)), 0xAB, dtype=torch.uint8, device=DEV)
        fq.tq4_compress_append(key.to(DEV), val.to(DEV), cache, slots.to(dt).to(DEV), rot, b4)
        _check_rows(cache, ref, slots, key, val, rot, b4, b4, h, d)


def test_append_strided_views(C):
    # key/value as slices of one fused projection output, as an attention layer hands them over
    rot, b4 = C["rotation_128_0"], C["boundaries_128_4"]
    h, d, n = 2, 128, 37
    fused = torch.randn(n, 3 * h * d, generator=torch.Generator().manual_seed(8)).to(torch.bfloat16)
    fg = fused.to(DEV)
    key_g = fg[:, h * d:2 * h * d].view(n, h, d)
    val_g = fg[:, 2 * h * d:].view(n, h, d)
    key = fused[:, h * d:2 * h * d].reshape(n, h, d)
    val = fused[:, 2 * h * d:].reshape(n, h, d)
    slots = torch.arange(n) * 2
    ref = torch.zeros(5, 16, h * (d + 8), dtype=torch.uint8)
    O.compress_and_store(key, val, ref, slots, rot, b4)
    cache = torch.zeros(5, 16, h * (d + 8), dtype=torch.uint8, device=DEV)
    fq.tq4_compress_append(key_g, val_g, cache, slots.to(DEV), rot, b4)
    _check_rows(cache, ref, slots, key, val, rot, b4, b4, h, d)


def test_append_full_size_config(C):
    """8192 tokens x 8 heads into a 65536-slot cache (seed-3 injective map), K 3-bit + QJL,
    V 4-bit, checked row by row against the oracle."""
    rot, S = C["rotation_128_0"], C["qjl_128_0"]
    b3, c3, b4 = C["boundaries_128_3"], C["centroids_128_3"], C["boundaries_128_4"]
    w = W.append_workload()
    h, d = 8, 128
    nb = w.num_slots // w.block_size
    cache = torch.zeros(nb, 16, h * (d + 8), dtype=torch.uint8, device=DEV)
    plane = torch.zeros(nb, 16, h * (d // 8 + 4), dtype=torch.uint8, device=DEV)
    fq.tq4_compress_append_qjl(w.key.to(DEV), w.value.to(DEV), cache, plane,
                               w.slot_mapping.to(DEV), rot, b3, c3, b4, S)
    ref = torch.zeros(nb, 16, h * (d + 8), dtype=torch.uint8)
    O.compress_and_store(w.key, w.value, ref, w.slot_mapping, rot, b3, b4)
    _check_rows(cache, ref, w.slot_mapping, w.key, w.value, rot, b3, b4, h, d)
    # injective map: exactly 8192 rows written
    assert int((cache.view(-1, h * (d + 8)) != 0).any(dim=1).sum()) == 8192
    idx, norms, signs, gamma = O.prod_quantize(w.key, rot, c3, b3, S)
    ref_plane = O.qjl_plane_rows(signs, gamma)
    got = plane.cpu().view(-1, h * (d // 8 + 4))[w.slot_mapping]
    sb = h * d // 8
    rows = cache.cpu().view(-1, h * (d + 8))[w.slot_mapping]
    codes = O.nibble_unpack(rows[:, :h * d // 2].reshape(-1, h, d // 2))
    knorm = rows[:, h * d // 2:h * d // 2 + 4 * h].contiguous().view(torch.float32)
    check_gamma(got[:, sb:].contiguous().view(torch.float32), gamma, w.key.float(), codes, idx,
                knorm, rot, c3)
    check_signs(got[:, :sb].reshape(-1, h, d // 8), signs, w.key.float(), codes, idx, knorm, rot,
                c3, S)
    # the same call without the QJL plane gives the same main rows
    cache2 = torch.zeros_like(cache)
    fq.tq4_compress_append(w.key.to(DEV), w.value.to(DEV), cache2, w.slot_mapping.to(DEV), rot,
                           b3, b4)
    assert torch.equal(cache2, cache)


def test_compress_then_decompress_roundtrip_property(C):
    # size-independent property: recompressing a decompressed-and-unrotated vector
    # reproduces its own codes (idempotence of the quantiser on its reconstruction points)
    rot, b4, c4 = C["rotation_128_0"], C["boundaries_128_4"], C["centroids_128_4"]
    x = torch.randn(512, 8, 128, generator=torch.Generator().manual_seed(21))
    p, n = fq.tq4_compress(x.to(DEV), rot, b4)
    y = fq.tq4_decompress(p, n, c4, dtype=torch.float32)          # rotated space
    back = (y.reshape(-1, 128) @ rot.to(DEV)).reshape(512, 8, 128)  # original space
    p2, n2 = fq.tq4_compress(back, rot, b4)
    assert (unpack(p2) != unpack(p)).float().mean().item() < 2e-3  # renormalisation moves few
    cos = torch.nn.functional.cosine_similarity(back.flatten().cpu(), x.flatten(), dim=0).item()
    assert cos > 0.93


def test_native_errors(C):
    from flashquant_b200._native import FlashQuantNativeError
    rot, b4 = C["rotation_128_0"], C["boundaries_128_4"]
    with pytest.raises(FlashQuantNativeError) as e:
        fq.tq4_compress(torch.randn(4, 1, 96, device=DEV), torch.eye(96), b4)
    assert e.value.code == -2
    with pytest.raises(ValueError):
        fq.tq4_compress_append(torch.randn(4, 2, 128, device=DEV), torch.randn(4, 2, 128, device=DEV),
                               torch.zeros(1, 16, 100, dtype=torch.uint8, device=DEV),
                               torch.zeros(4, dtype=torch.int64, device=DEV), rot, b4)


@pytest.mark.parametrize("dim,bits,dtype", [(64, 4, torch.float32), (64, 3, torch.bfloat16),
                                            (128, 4, torch.float16), (128, 3, torch.float32)])
def test_compress_bulk_sizes_use_the_warp_per_tile_kernel(C, dim, bits, dtype):
    """More than 1024 tiles of 16 vectors: the bulk kernel, for both head sizes and all input
    types (the smaller cases above stay on the CTA-per-tile kernel)."""
    rot = C.get(f"rotation_{dim}_0")
    bnd = C[f"boundaries_{dim}_{bits}"] if f"boundaries_{dim}_{bits}" in C else \
        O.lloyd_max_codebook(dim, bits)[1]
    g = torch.Generator().manual_seed(200 + dim + bits)
    x = torch.randn(5001, 4, dim, generator=g)  # 20004 vectors: 1251 tiles, the last one ragged
    x[..., W.outlier_channels(dim)] *= 10
    x = x.to(dtype)
    p, n = fq.tq4_compress(x.to(DEV), rot, bnd)
    pr, nr = O.compress(x, rot, bnd)
    check_codes(p, x.float(), rot, bnd, pr)
    check_norms(n, nr)


def test_prod_quantize_bulk_head_dim_64(C):
    """Two-stage quantiser, head_dim 64, bulk kernel: codes, norms, gamma and signs."""
    d = 64
    q = fq.TurboQuantProd(d, 4, seed=0)
    rot, S = q.mse_quantizer.rotation, q.qjl_matrix
    b3, c3 = q.mse_quantizer.boundaries, q.mse_quantizer.centroids
    k = torch.randn(4200, 4, d, generator=torch.Generator().manual_seed(5)).bfloat16()
    idx, norms, signs, gamma = O.prod_quantize(k, rot, c3, b3, S)
    packed, n2, bits, g2 = fq.tq_prod_quantize(k.to(DEV), rot, b3, c3, S)
    check_codes(packed, k.float(), rot, b3, O.nibble_pack(idx))
    check_norms(n2, norms)
    codes = O.nibble_unpack(packed.cpu())
    check_gamma(g2, gamma, k.float(), codes, idx, n2.cpu(), rot, c3)
    check_signs(bits, signs, k.float(), codes, idx, n2.cpu(), rot, c3, S)


@pytest.mark.parametrize("shape", [(32, 128), (8, 256), (3, 20), (1, 4), (5, 7, 64)])
def test_two_bit_packing_equals_oracle(shape):
    idx = torch.randint(0, 4, shape, generator=torch.Generator().manual_seed(sum(shape)))
    packed = fq.pack_2bit(idx.to(DEV))
    assert packed.dtype == torch.uint8 and packed.shape == (*shape[:-1], shape[-1] // 4)
    assert torch.equal(packed.cpu(), O.pack_2bit(idx))
    back = fq.unpack_2bit(packed, shape[-1])
    assert back.dtype == torch.int64 and torch.equal(back.cpu(), idx)
    assert torch.equal(fq.unpack_2bit(O.pack_2bit(idx).to(DEV), shape[-1]).cpu(), idx)


def test_two_bit_packing_errors():
    with pytest.raises(ValueError, match="divisible by 4"):
        fq.pack_2bit(torch.zeros(2, 6, dtype=torch.long, device=DEV))
    with pytest.raises(ValueError, match="out of range"):
        fq.pack_2bit(torch.tensor([[4, 0, 0, 0]], device=DEV))
    with pytest.raises(ValueError, match="out of range"):
        fq.pack_2bit(torch.tensor([[0, 0, 7, 0]], dtype=torch.uint8, device=DEV))
    with pytest.raises(ValueError, match="out of range"):
        fq.pack_2bit(torch.tensor([[-1, 0, 0, 0]], device=DEV))
    assert fq.pack_2bit(torch.zeros(0, 8, dtype=torch.long, device=DEV)).shape == (0, 2)
