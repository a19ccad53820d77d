"""GPU parity of the fused TQ4 prefill attention (tcgen05 kernel) against the oracle.

Bar: outputs within 2e-3 max-abs of the reference's decompress-then-attend path (see
parity.attention_close for rows whose entries are of order 1).
"""

import numpy as np
import pytest
import torch

import flashquant_b200 as fq
from conftest import bf16_from_bits, load_golden
from flashquant_b200 import kernels as K
from flashquant_b200 import workloads as W
from oracle import tq_oracle as O
from parity import attention_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def make_case(consts, b, hq, hkv, n, seed, dtype=torch.bfloat16, k_bits=3, v_bits=4):
    d = 128
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(b, hq, n, d, generator=g).to(dtype)
    k = torch.randn(b * hkv, n, d, generator=g)
    k[..., W.outlier_channels(d)] *= 10.0
    v = torch.randn(b * hkv, n, d, generator=g)
    rot = consts["rotation_128_0"]
    kp, kn = O.compress(k.to(dtype), rot, consts[f"boundaries_128_{k_bits}"])
    vp, vn = O.compress(v.to(dtype), rot, consts[f"boundaries_128_{v_bits}"])
    shape4 = lambda t, last: t.reshape(b, hkv, n, last)
    return (q, shape4(kp, d // 2), shape4(kn, 1), shape4(vp, d // 2), shape4(vn, 1),
            consts[f"centroids_128_{k_bits}"], consts[f"centroids_128_{v_bits}"], rot)


# The prefill kernel uses the same scaled fp16 centroid tables as the decode kernels; its
# rows agree with the reference's un-rounded rows to 2^-10 of the entry, the decode's bound.
PREFILL_RTOL = 2.0 ** -10


def check(out, case, rotation_v=None, **kw):
    """Against the oracle's contiguous attention, whose rotated rows stay fp32 until the product
    with Pi is rounded (src/flashquant/kernels/cpu_reference.py:195, 225-226)."""
    ref32, ref = O.fused_tq_attention_stages(*case, **kw)
    return attention_close(out, ref, ref32, case[7] if rotation_v is None else rotation_v,
                           rounds_rotated=False, rtol=PREFILL_RTOL)


def run_gpu(case, **kw):
    q, kp, kn, vp, vn, ck, cv, rot = case
    out = K.fused_tq_attention(q.to(DEV), kp.to(DEV), kn.to(DEV), vp.to(DEV), vn.to(DEV), ck, cv,
                               rot, **kw)
    assert K.attention_workspace_status(torch.device(DEV)) == 0
    return out


def test_golden_fixture(consts):
    z = load_golden("prefill.npz")
    case = (bf16_from_bits(z["q_bf16"]), T(z["k_packed"]), T(z["k_norms"]), T(z["v_packed"]),
            T(z["v_norms"]), consts["centroids_128_3"], consts["centroids_128_4"],
            consts["rotation_128_0"])
    for causal, key in ((True, "out_causal_bf16"), (False, "out_full_bf16")):
        ref32, ref = O.fused_tq_attention_stages(*case, is_causal=causal)
        assert torch.equal(ref.view(torch.int16), bf16_from_bits(z[key]).view(torch.int16))
        attention_close(run_gpu(case, is_causal=causal), bf16_from_bits(z[key]), ref32, case[7],
                        rounds_rotated=False, rtol=PREFILL_RTOL)


@pytest.mark.parametrize("b,hq,hkv,n", [(1, 4, 1, 64), (2, 8, 2, 128), (1, 4, 4, 129),
                                        (1, 2, 1, 1), (1, 8, 2, 333), (1, 4, 2, 640)])
@pytest.mark.parametrize("causal", [True, False])
def test_vs_oracle(consts, b, hq, hkv, n, causal):
    case = make_case(consts, b, hq, hkv, n, seed=100 + n)
    check(run_gpu(case, is_causal=causal), case, is_causal=causal)


def test_fp16_scale_and_4bit_keys(consts):
    case = make_case(consts, 1, 4, 2, 200, seed=7, dtype=torch.float16, k_bits=4)
    check(run_gpu(case, sm_scale=0.07, is_causal=True), case, sm_scale=0.07, is_causal=True)


def test_causal_first_row_sees_only_first_key(consts):
    # size-independent property: row 0 of a causal call equals V[0] (rotated back)
    case = make_case(consts, 1, 4, 2, 300, seed=9)
    out = run_gpu(case, is_causal=True).float().cpu()
    q, kp, kn, vp, vn, ck, cv, rot = case
    v0 = O.decompress(vp[0, :, :1].reshape(2, 1, 64), vn[0, :, :1].reshape(2, 1, 1), cv)  # (2,1,128)
    v0r = v0.reshape(2, 128).repeat_interleave(2, dim=0)
    want = (v0r @ rot).to(torch.bfloat16)
    attention_close(out[0, :, 0].to(torch.bfloat16), want, v0r, rot, rounds_rotated=False,
                    rtol=PREFILL_RTOL)


def test_longer_sequence_chunked_oracle(consts):
    case = make_case(consts, 1, 8, 2, 2048, seed=11)
    check(run_gpu(case, is_causal=True), case, is_causal=True, q_chunk=256)


@pytest.mark.parametrize("b,hq,hkv,nkv", [(2, 32, 8, 4133), (1, 4, 4, 1000), (3, 8, 2, 64),
                                         (1, 16, 1, 70)])
def test_single_query_token_over_many_keys(consts, b, hq, hkv, nkv):
    # one query token per sequence (a decode step over a contiguous cache): the heads of a KV
    # group share a query tile and the keys are cut into slices that a second kernel merges
    case = list(make_case(consts, b, hq, hkv, nkv, seed=500 + nkv))
    case[0] = case[0][:, :, -1:].contiguous()
    check(run_gpu(tuple(case), is_causal=True), tuple(case), is_causal=True)
    assert K.attention_workspace_status(torch.device(DEV)) == 0


def test_argument_errors(consts):
    from flashquant_b200._native import FlashQuantNativeError
    case = make_case(consts, 1, 4, 2, 64, seed=3)
    q, kp, kn, vp, vn, ck, cv, rot = case
    with pytest.raises(FlashQuantNativeError) as e:  # causal mask needs n_q == n_kv
        K.fused_tq_attention(q[:, :, :32].to(DEV), kp.to(DEV), kn.to(DEV), vp.to(DEV), vn.to(DEV),
                             ck, cv, rot, is_causal=True)
    assert e.value.code == -2


def test_config3_shape_sliced_oracle(consts):
    """configs[3]: batch 4 x 8192 tokens, 32 q / 8 kv heads, causal.  One launch at the full
    shape; the oracle (which would need 34 GB of scores at once) attends over three
    (batch, KV group) slices, the query rows in chunks."""
    b, hq, hkv, n, d = 4, 32, 8, 8192, 128
    rot = consts["rotation_128_0"]
    b3, c3 = consts["boundaries_128_3"], consts["centroids_128_3"]
    b4, c4 = consts["boundaries_128_4"], consts["centroids_128_4"]
    k, v = W.make_kv(b * n, hkv, d, cfg=3)
    kp, kn = K.tq4_compress(k.to(DEV).reshape(b, n, hkv, d).transpose(1, 2).reshape(-1, 1, d), rot, b3)
    vp, vn = K.tq4_compress(v.to(DEV).reshape(b, n, hkv, d).transpose(1, 2).reshape(-1, 1, d), rot, b4)
    kp, vp = kp.reshape(b, hkv, n, d // 2), vp.reshape(b, hkv, n, d // 2)
    kn, vn = kn.reshape(b, hkv, n, 1), vn.reshape(b, hkv, n, 1)
    q = torch.randn(b, hq, n, d, generator=torch.Generator().manual_seed(3003)).to(torch.bfloat16)
    out = K.fused_tq_attention(q.to(DEV), kp, kn, vp, vn, c3, c4, rot, is_causal=True)
    assert K.attention_workspace_status(torch.device(DEV)) == 0
    g = hq // hkv
    for bi, h in ((0, 0), (1, 5), (3, 7)):
        case = (q[bi:bi + 1, h * g:(h + 1) * g], kp[bi:bi + 1, h:h + 1].cpu(), kn[bi:bi + 1, h:h + 1].cpu(),
                vp[bi:bi + 1, h:h + 1].cpu(), vn[bi:bi + 1, h:h + 1].cpu(), c3, c4, rot)
        check(out[bi:bi + 1, h * g:(h + 1) * g], case, is_causal=True, q_chunk=1024)
