"""Pins the CPU oracle to outputs of the reference package (fixtures in tests/golden)."""

import math

import numpy as np
import torch

from conftest import bf16_from_bits, load_golden
from oracle import tq_oracle as O


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def test_constants_bit_identical(consts):
    for dim, bits in [(128, 2), (128, 3), (128, 4), (64, 3), (64, 4)]:
        c, b = O.lloyd_max_codebook(dim, bits)
        assert torch.equal(c, consts[f"centroids_{dim}_{bits}"])
        assert torch.equal(b, consts[f"boundaries_{dim}_{bits}"])
    # LAPACK's QR is not bit-reproducible across thread counts (differences of ~1e-6 were
    # seen between 1 and 8 threads), so Pi is always passed in as data; regenerating it
    # must only land close to the stored one.
    for dim, seed in [(128, 0), (128, 42), (64, 0)]:
        r = O.haar_rotation(dim, seed)
        assert (r - consts[f"rotation_{dim}_{seed}"]).abs().max().item() < 1e-5
        assert (r @ r.T - torch.eye(dim)).abs().max().item() < 5e-6
    assert torch.equal(O.qjl_matrix(128, 0), consts["qjl_128_0"])
    assert torch.equal(O.qjl_matrix(64, 0), consts["qjl_64_0"])


def test_middle_boundary_is_not_zero(consts):
    # the 4-bit middle boundary is a tiny negative number, the 3-bit one a tiny positive:
    # a zero vector therefore maps to index 8 (4-bit) and 3 (3-bit)
    assert consts["boundaries_128_4"][7].item() < 0
    assert consts["boundaries_128_3"][3].item() > 0


def test_packing_known_answers():
    # bytes of the reference's tests: [0,15]->0x0F, [15,0]->0xF0, [5,10]->0x5A
    assert O.nibble_pack(torch.tensor([[0, 15]], dtype=torch.uint8)).item() == 0x0F
    assert O.nibble_pack(torch.tensor([[15, 0]], dtype=torch.uint8)).item() == 0xF0
    assert O.nibble_pack(torch.tensor([[5, 10]], dtype=torch.uint8)).item() == 0x5A
    # C++ test of the reference: {5,3,15,0,7,9} -> 83, 240, 121
    assert O.nibble_pack(torch.tensor([5, 3, 15, 0, 7, 9], dtype=torch.uint8)).tolist() == [83, 240, 121]
    z = load_golden("packing.npz")
    assert torch.equal(O.nibble_pack(T(z["idx"])), T(z["packed"]))
    assert torch.equal(O.nibble_unpack(T(z["packed"])), T(z["unpacked"]))


def test_sign_bits_roundtrip():
    s = torch.sign(torch.randn(3, 2, 128))
    s[s == 0] = 1
    p = O.sign_bits_pack(s)
    assert p.shape == (3, 2, 16)
    assert torch.equal(O.sign_bits_unpack(p), s)
    one = -torch.ones(8)
    one[2] = 1
    assert O.sign_bits_pack(one).item() == 4


def test_mse_quantiser_matches_reference(consts):
    z = load_golden("quantize.npz")
    rot, b4, c4 = consts["rotation_128_0"], consts["boundaries_128_4"], consts["centroids_128_4"]
    v = T(z["v"])
    idx, norms, _ = O.mse_quantize(v, rot, b4)
    assert torch.equal(idx.to(torch.uint8), T(z["v_idx"]))
    assert torch.equal(norms, T(z["v_norms"]))
    torch.testing.assert_close(O.mse_dequantize(idx, norms, rot, c4), T(z["v_deq"]), rtol=1e-6, atol=1e-6)
    packed, n2 = O.compress(v, rot, b4)
    assert torch.equal(packed, T(z["v_packed"]))
    assert torch.equal(n2, T(z["v_norms_c"]))
    assert torch.equal(O.decompress(packed, n2, c4), T(z["v_decomp"]))
    pb, nb = O.compress(bf16_from_bits(z["vb_bf16"]), rot, b4)
    assert torch.equal(pb, T(z["vb_packed"]))
    assert torch.equal(nb, T(z["vb_norms"]))


def test_prod_quantiser_matches_reference(consts):
    z = load_golden("quantize.npz")
    rot, b3, c3 = consts["rotation_128_0"], consts["boundaries_128_3"], consts["centroids_128_3"]
    S = consts["qjl_128_0"]
    k = T(z["k"])
    idx, norms, signs, gamma = O.prod_quantize(k, rot, c3, b3, S)
    assert torch.equal(idx.to(torch.uint8), T(z["k_idx"]))
    assert torch.equal(norms, T(z["k_norms"]))
    assert torch.equal(signs.to(torch.int8), T(z["k_signs"]))
    torch.testing.assert_close(gamma, T(z["k_gamma"]), rtol=1e-6, atol=0)
    # the zero vector: all signs +1, gamma 0, index 3 everywhere
    assert (signs[0, 1] == 1).all() and gamma[0, 1].item() == 0 and (idx[0, 1] == 3).all()
    q = T(z["ip_query"])
    est = O.estimate_inner_product(q.unsqueeze(1), idx.unsqueeze(0), norms.unsqueeze(0),
                                   signs.unsqueeze(0), gamma.unsqueeze(0), rot, c3, S)
    torch.testing.assert_close(est, T(z["ip_est"]), rtol=1e-5, atol=1e-5)


def test_key_scores_match_reference(consts):
    z = load_golden("key_scores.npz")
    rot = consts["rotation_128_0"]
    c3, b3, S = consts["centroids_128_3"], consts["boundaries_128_3"], consts["qjl_128_0"]
    keys, query = T(z["keys"]), T(z["query"])
    idx, norms, signs, gamma = O.prod_quantize(keys, rot, c3, b3, S)
    est = O.estimate_inner_product(query.unsqueeze(3), idx.unsqueeze(2), norms.unsqueeze(2),
                                   signs.unsqueeze(2), gamma.unsqueeze(2), rot, c3, S)
    torch.testing.assert_close(est.squeeze(-1), T(z["scores"]), rtol=1e-5, atol=1e-5)


def _decode_case(consts):
    z = load_golden("paged_decode.npz")
    args = dict(
        kv_cache=T(z["kv_cache"]), block_table=T(z["block_table"]), seq_lens=T(z["seq_lens"]),
        centroids_k=consts["centroids_128_3"], centroids_v=consts["centroids_128_4"],
        rotation=consts["rotation_128_0"], num_kv_heads=int(z["h_kv"]), head_dim=int(z["d"]),
        block_size=int(z["block_size"]),
    )
    return z, args


def test_paged_decode_matches_reference(consts):
    z, a = _decode_case(consts)
    q = bf16_from_bits(z["q_bf16"])
    out = O.split_k_paged_decode(q, **a)
    ref = bf16_from_bits(z["out_bf16"])
    # same arithmetic, different summation order: at most one bf16 ulp on a few entries
    assert (out.float() - ref.float()).abs().max().item() <= 2e-3
    assert (out == ref).float().mean().item() > 0.98
    assert (out[0] == 0).all()  # empty sequence -> zeros
    q16 = T(z["q_f16"])
    out16 = O.split_k_paged_decode(q16, sm_scale=float(z["sm_scale_f16"]), **a)
    assert (out16.float() - T(z["out_f16"]).float()).abs().max().item() <= 5e-4


def test_loop_and_vectorised_decode_agree(consts):
    z, a = _decode_case(consts)
    q = bf16_from_bits(z["q_bf16"])
    rot = a.pop("rotation")
    q_rot = torch.matmul(q.float(), rot.T).to(q.dtype)
    v = O.paged_decode_rotated(q_rot, **a)
    l = O.paged_decode_rotated_loop(q_rot, **a)
    assert (v.float() - l.float()).abs().max().item() <= 1e-3


def test_split_k_merge_equals_unsplit(consts):
    z, a = _decode_case(consts)
    i = 5
    n = int(a["seq_lens"][i])
    k, v = O.gather_paged(a["kv_cache"], a["block_table"][i], n, a["num_kv_heads"], a["head_dim"],
                          a["block_size"], a["centroids_k"], a["centroids_v"])
    q = torch.randn(128)
    scale = 1 / math.sqrt(128)
    full = torch.softmax((k[0] @ q) * scale, dim=-1) @ v[0]
    for bounds in ([(0, n)], [(0, 16), (16, 32), (32, 48), (48, n)], [(0, 7), (7, 7), (7, n), (n, n)]):
        parts = O.split_k_partials(q, k[0], v[0], scale, bounds)
        torch.testing.assert_close(O.split_k_merge(parts), full, rtol=1e-5, atol=1e-6)
    empty = O.split_k_partials(q, k[0], v[0], scale, [(0, 0), (3, 3)])
    assert (O.split_k_merge(empty) == 0).all()


def test_prefill_matches_reference(consts):
    z = load_golden("prefill.npz")
    q = bf16_from_bits(z["q_bf16"])
    args = (T(z["k_packed"]), T(z["k_norms"]), T(z["v_packed"]), T(z["v_norms"]),
            consts["centroids_128_3"], consts["centroids_128_4"], consts["rotation_128_0"])
    for causal, key in [(True, "out_causal_bf16"), (False, "out_full_bf16")]:
        ref = bf16_from_bits(z[key])
        out = O.fused_tq_attention(q, *args, is_causal=causal)
        assert (out.float() - ref.float()).abs().max().item() <= 2e-3
        assert (out == ref).float().mean().item() > 0.98
        chunked = O.fused_tq_attention(q, *args, is_causal=causal, q_chunk=32)
        assert (chunked.float() - ref.float()).abs().max().item() <= 2e-3


def test_compress_and_store_rows(consts):
    rot, b4 = consts["rotation_128_0"], consts["boundaries_128_4"]
    g = torch.Generator().manual_seed(5)
    key = torch.randn(6, 2, 128, generator=g).to(torch.bfloat16)
    val = torch.randn(6, 2, 128, generator=g).to(torch.bfloat16)
    cache = torch.zeros(2, 16, 2 * 136, dtype=torch.uint8)
    slots = torch.tensor([3, 31, -1, 0, 17, 16])
    rows = O.compress_and_store(key, val, cache, slots, rot, b4)
    flat = cache.view(-1, 272)
    kp, kn = O.compress(key, rot, b4)
    for i, s in enumerate(slots.tolist()):
        if s < 0:
            continue
        assert torch.equal(flat[s], rows[i])
        assert torch.equal(flat[s, :128], kp[i].reshape(-1))
        assert torch.equal(flat[s, 128:136].view(torch.float32), kn[i].reshape(-1))
    untouched = [s for s in range(32) if s not in (3, 31, 0, 17, 16)]
    assert (flat[untouched] == 0).all()


def test_multi_token_decode_equals_single_token_calls(consts):
    # the last n_q tokens of a sequence, masked at the end of the keys, are n_q single-token
    # decodes at lengths L - n_q + 1 .. L (pins the mask alignment of the multi-token oracle to
    # the single-token one, which is pinned to the reference's outputs above)
    z, a = _decode_case(consts)
    n_q = 3
    q = torch.randn(a["seq_lens"].numel(), n_q, int(z["h_q"]), int(z["d"]),
                    generator=torch.Generator().manual_seed(12)).to(torch.bfloat16)
    from parity import attention_close
    multi32, multi = O.paged_decode_multi_stages(q, **a)
    for t in range(n_q):
        lens = (a["seq_lens"] - (n_q - 1) + t).clamp(min=0)
        one32, one = O.split_k_paged_decode_stages(q[:, t].contiguous(), **{**a, "seq_lens": lens})
        # the same sums in another batching: equal up to fp32 rounding before the cast, and
        # after it up to the flips such a difference can cause
        assert (one32 - multi32[:, t]).abs().max().item() <= 1e-5
        attention_close(multi[:, t], one, one32, a["rotation"], got_rot32=multi32[:, t],
                        rtol=2.0 ** -16)
        assert bool((multi[:, t][lens == 0] == 0).all())


def test_two_bit_packing_known_answers():
    # byte = c0<<6 | c1<<4 | c2<<2 | c3 (the reference's C++ core and the restatement in its tests)
    assert O.pack_2bit(torch.tensor([[0, 1, 2, 3]])).item() == 0x1B
    assert O.pack_2bit(torch.tensor([[3, 3, 3, 3]])).item() == 0xFF
    assert O.pack_2bit(torch.tensor([[1, 0, 0, 0, 0, 0, 0, 2]])).tolist() == [[0x40, 0x02]]
    idx = torch.randint(0, 4, (32, 128), generator=torch.Generator().manual_seed(4))
    packed = O.pack_2bit(idx)
    assert packed.shape == (32, 32) and packed.dtype == torch.uint8
    assert torch.equal(O.unpack_2bit(packed, 128), idx)
    assert O.pack_2bit(torch.zeros(8, 256, dtype=torch.long)).shape[-1] == 64
    import pytest
    with pytest.raises(ValueError):
        O.pack_2bit(torch.zeros(2, 6, dtype=torch.long))
