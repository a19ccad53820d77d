"""GPU parity of the split-K paged decode against the CPU oracle and the golden fixture.

Bar (parity.attention_close): before the reference's first rounding the rotated-space rows
agree within 2e-3 max-abs and 2^-10 of the entry; after both roundings an entry may differ by
one unit in its last place plus the rounding flips the reference's own values allow.
"""

import numpy as np
import pytest
import torch

import flashquant_b200 as fq
from conftest import bf16_from_bits, load_golden
from flashquant_b200 import kernels as K
from flashquant_b200 import workloads as W
from oracle import tq_oracle as O
from parity import attention_close, rows_from_partials

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def T(a):
    return torch.from_numpy(np.ascontiguousarray(a))


def fill_cache_cpu(w, consts, k_bits=3, v_bits=4, dtype=torch.bfloat16):
    """Packed cache built by the oracle from seeded K/V (K: k_bits table, V: v_bits table)."""
    d, h = w.head_dim, w.num_kv_heads
    rot = consts[f"rotation_{d}_0"]
    bk, bv = consts[f"boundaries_{d}_{k_bits}"], consts[f"boundaries_{d}_{v_bits}"]
    k, v = W.make_kv(w.total_tokens, h, d, w.cfg, dtype)
    cache = torch.zeros(w.num_blocks, w.block_size, h * (d + 8), dtype=torch.uint8)
    O.compress_and_store(k, v, cache, w.slot_mapping, rot, bk, bv)
    return cache


def run_gpu(w, cache, consts, k_bits=3, v_bits=4, num_splits=0, q=None, sm_scale=None):
    d = w.head_dim
    q = w.q if q is None else q
    return K.split_k_paged_decode(
        q.to(DEV), cache.to(DEV), w.block_table.to(DEV), w.seq_lens.to(DEV),
        consts[f"centroids_{d}_{k_bits}"], consts[f"centroids_{d}_{v_bits}"],
        consts[f"rotation_{d}_0"], w.num_kv_heads, d, w.block_size, sm_scale=sm_scale,
        num_splits=num_splits)


def run_oracle(w, cache, consts, k_bits=3, v_bits=4, q=None, sm_scale=None):
    """(fp32 rotated-space rows before the first rounding, final output) of the reference."""
    d = w.head_dim
    q = w.q if q is None else q
    return O.split_k_paged_decode_stages(
        q, cache, w.block_table, w.seq_lens, consts[f"centroids_{d}_{k_bits}"],
        consts[f"centroids_{d}_{v_bits}"], consts[f"rotation_{d}_0"], w.num_kv_heads, d,
        w.block_size, sm_scale)


def close(out, stages, consts, d=128, **kw):
    ref32, ref = stages
    return attention_close(out, ref, ref32, consts[f"rotation_{d}_0"], **kw)


def gpu_rows(w, cache, consts, k_bits=3, v_bits=4, num_splits=0, sm_scale=None):
    """The GPU's rotated-space rows before any rounding (merged partial rows, normalised)."""
    d = w.head_dim
    parts = K.paged_decode_partials(
        w.q.to(DEV), cache.to(DEV), w.block_table.to(DEV), w.seq_lens.to(DEV),
        consts[f"centroids_{d}_{k_bits}"], consts[f"centroids_{d}_{v_bits}"],
        consts[f"rotation_{d}_0"], w.num_kv_heads, d, w.block_size, num_splits=num_splits,
        sm_scale=sm_scale)
    return rows_from_partials(parts)


def test_golden_fixture(consts):
    z = load_golden("paged_decode.npz")
    cache, bt, sl = T(z["kv_cache"]), T(z["block_table"]), T(z["seq_lens"])
    ck, cv, rot = consts["centroids_128_3"], consts["centroids_128_4"], consts["rotation_128_0"]
    geo = (int(z["h_kv"]), int(z["d"]), int(z["block_size"]))
    args = (cache.to(DEV), bt.to(DEV), sl.to(DEV), ck, cv, rot) + geo
    q = bf16_from_bits(z["q_bf16"])
    ref32, ref = O.split_k_paged_decode_stages(q, cache, bt, sl, ck, cv, rot, *geo)
    assert torch.equal(ref.view(torch.int16), bf16_from_bits(z["out_bf16"]).view(torch.int16))
    for splits in (0, 1, 3, 8):
        out = K.split_k_paged_decode(q.to(DEV), *args, num_splits=splits)
        attention_close(out, ref, ref32, rot)
        assert (out[0] == 0).all()  # empty sequence
    q16, scale = T(z["q_f16"]), float(z["sm_scale_f16"])
    ref32, ref = O.split_k_paged_decode_stages(q16, cache, bt, sl, ck, cv, rot, *geo, sm_scale=scale)
    assert torch.equal(ref.view(torch.int16), T(z["out_f16"]).view(torch.int16))
    out = K.split_k_paged_decode(q16.to(DEV), *args, sm_scale=scale, num_splits=2)
    attention_close(out, ref, ref32, rot)
    ws = K.decode_workspace(torch.device(DEV), 6, 8, 2, 128, 0)
    assert K.workspace_status(ws) == 0


@pytest.mark.parametrize("hkv,hq", [(8, 32), (1, 8), (2, 2), (4, 8), (8, 64), (16, 32)])
def test_ragged_lengths_vs_oracle(consts, hkv, hq):
    lens = [0, 1, 15, 16, 17, 31, 33, 100, 257, 700]
    w = W.decode_workload(seq_lens=lens, num_q_heads=hq, num_kv_heads=hkv, cfg=11, spare_blocks=5)
    cache = fill_cache_cpu(w, consts)
    ref = run_oracle(w, cache, consts)
    for splits in (1, 4, 8):
        out = run_gpu(w, cache, consts, num_splits=splits)
        close(out, ref, consts, got_rot32=gpu_rows(w, cache, consts, num_splits=splits))


def test_head_dim_64_and_shared_4bit_tables(consts):
    w = W.decode_workload(seq_lens=[5, 64, 333], num_q_heads=8, num_kv_heads=2, head_dim=64, cfg=12)
    cache = fill_cache_cpu(w, consts, k_bits=4, v_bits=4)
    ref = run_oracle(w, cache, consts, k_bits=4, v_bits=4)
    # head_dim 64 takes the generic kernel (one fp16 term per weight) and a 16-level key table
    # gains less from the common scale than an 8-level one: 2^-9 before the rounding
    close(run_gpu(w, cache, consts, k_bits=4, v_bits=4, num_splits=2), ref, consts, d=64,
          got_rot32=gpu_rows(w, cache, consts, k_bits=4, v_bits=4, num_splits=2), rtol=2.0 ** -9)


def test_block_size_32_and_fp16_queries(consts):
    w = W.decode_workload(seq_lens=[40, 129, 512], num_q_heads=16, num_kv_heads=4, block_size=32,
                          cfg=13, dtype=torch.float16)
    cache = fill_cache_cpu(w, consts, dtype=torch.float16)
    ref = run_oracle(w, cache, consts, sm_scale=0.11)
    close(run_gpu(w, cache, consts, num_splits=3, sm_scale=0.11), ref, consts,
          got_rot32=gpu_rows(w, cache, consts, num_splits=3, sm_scale=0.11))


def test_split_count_and_page_permutation_invariance(consts):
    """Size-independent properties: the result does not depend on the number of splits beyond
    rounding, nor on where the pages physically live."""
    w = W.decode_workload(num_seqs=4, context=2048, cfg=14)
    cache = fill_cache_cpu(w, consts)
    ref = run_oracle(w, cache, consts)
    base = gpu_rows(w, cache, consts, num_splits=1)
    for splits in (1, 2, 8, 32):
        close(run_gpu(w, cache, consts, num_splits=splits), ref, consts)
        # another partition of the keys only changes the order of the fp32 sums
        rows = gpu_rows(w, cache, consts, num_splits=splits)
        assert (rows - base).abs().max().item() <= 1e-4 * base.abs().max().item()
    # move every page: new table, same logical content
    perm = torch.randperm(w.num_blocks, generator=torch.Generator().manual_seed(77))
    cache2 = torch.empty_like(cache)
    cache2[perm] = cache
    w2 = W.decode_workload(num_seqs=4, context=2048, cfg=14)
    w2.block_table = perm[w.block_table.long()].int()
    out = run_gpu(w2, cache2, consts, num_splits=8).float().cpu()
    assert torch.equal(out, run_gpu(w, cache, consts, num_splits=8).float().cpu())


def test_partials_then_merge_equals_fused_call(consts):
    w = W.decode_workload(seq_lens=[90, 1000, 17, 0], cfg=15)
    cache = fill_cache_cpu(w, consts)
    rot = consts["rotation_128_0"]
    args = (w.q.to(DEV), cache.to(DEV), w.block_table.to(DEV), w.seq_lens.to(DEV),
            consts["centroids_128_3"], consts["centroids_128_4"], rot, 8, 128, 16)
    fused = K.split_k_paged_decode(*args, num_splits=4)
    parts = K.paged_decode_partials(*args, num_splits=4)
    assert parts.shape == (4, 32, 132)
    merged = K.split_k_merge(parts, rot, torch.bfloat16)
    ref = run_oracle(w, cache, consts)
    close(merged, ref, consts, got_rot32=rows_from_partials(parts))
    close(fused, ref, consts)
    # empty sequence: (0.., -inf, 0)
    tail = parts[3].cpu()
    assert torch.isinf(tail[:, 128]).all() and (tail[:, 129] == 0).all() and (tail[:, :128] == 0).all()
    assert (merged[3] == 0).all()


def test_short_runs_that_cross_sequences_repeat_bit_for_bit(consts):
    """637 pages over 296 page runs: runs of two or three pages, several of them with the end
    of one sequence and the start of the next, so a team switches its query while the first
    one's tile is still being computed.  The partial rows must not depend on timing."""
    w = W.decode_workload(seq_lens=[10000, 173, 16], cfg=23)
    cache = fill_cache_cpu(w, consts)
    rot = consts["rotation_128_0"]
    args = (w.q.to(DEV), cache.to(DEV), w.block_table.to(DEV), w.seq_lens.to(DEV),
            consts["centroids_128_3"], consts["centroids_128_4"], rot, 8, 128, 16)
    first = K.paged_decode_partials(*args, num_splits=1).clone()
    for _ in range(40):
        again = K.paged_decode_partials(*args, num_splits=1)
        assert torch.equal(first, again)
    merged = K.split_k_merge(first, rot, torch.bfloat16)
    close(merged, run_oracle(w, cache, consts), consts, got_rot32=rows_from_partials(first))


@pytest.mark.parametrize("hq,hkv,seq_lens", [
    (8, 1, [9000, 5000, 40]),        # 16 one-warp teams per CTA: several hundred rows per sequence
    (16, 2, [7000, 0, 3000, 555]),   # two head groups, an empty sequence
    (64, 8, [30000]),                # the specialised kernel, one sequence over all teams
])
def test_sequences_with_hundreds_of_partial_rows(consts, hq, hkv, seq_lens):
    """Few sequences over all teams of the GPU: the single launch cuts the rows of a sequence
    into chunks, merges each in its own job and the chunks' rows in the job that finishes last."""
    w = W.decode_workload(seq_lens=seq_lens, num_q_heads=hq, num_kv_heads=hkv, cfg=27)
    cache = fill_cache_cpu(w, consts)
    ref = run_oracle(w, cache, consts)
    for splits in (1, 8):
        out = run_gpu(w, cache, consts, num_splits=splits)
        close(out, ref, consts, rtol=2.0 ** -9)
        again = run_gpu(w, cache, consts, num_splits=splits)
        assert torch.equal(out, again)


@pytest.mark.parametrize("seed", [101, 102, 103, 104, 105, 106])
def test_random_ragged_batches_vs_oracle(consts, seed):
    """Seeded random batches - empty, tiny and long sequences mixed, random split counts - through
    both streaming kernels (the specialised one and, with it switched off, the generic one):
    every run of pages that crosses sequences, every short segment is a case of its own."""
    g = torch.Generator().manual_seed(seed)
    n = int(torch.randint(3, 13, (1,), generator=g))
    kind = torch.randint(0, 4, (n,), generator=g)
    lens = []
    for k in kind.tolist():
        if k == 0:
            lens.append(0 if int(torch.randint(0, 2, (1,), generator=g)) else 1)
        elif k == 1:
            lens.append(int(torch.randint(1, 41, (1,), generator=g)))
        elif k == 2:
            lens.append(int(torch.randint(100, 700, (1,), generator=g)))
        else:
            lens.append(int(torch.randint(700, 3001, (1,), generator=g)))
    splits = int(torch.randint(1, 9, (1,), generator=g))
    w = W.decode_workload(seq_lens=lens, cfg=seed)
    cache = fill_cache_cpu(w, consts)
    ref = run_oracle(w, cache, consts)
    lib = K.N.load()
    try:
        for fast in (1, 0):
            lib.fq_paged_decode_set_fast_path(fast)
            out = run_gpu(w, cache, consts, num_splits=splits)
            close(out, ref, consts, rtol=2.0 ** -9)
            rows = gpu_rows(w, cache, consts, num_splits=splits)
            close(out, ref, consts, got_rot32=rows, rtol=2.0 ** -9)
    finally:
        lib.fq_paged_decode_set_fast_path(1)


def test_token_ranges_on_two_groups_merge_like_one(consts):
    """What a cross-GPU split does: group 0 attends over the first pages of every sequence,
    group 1 over the rest; merging the two partial rows equals attending over everything."""
    w = W.decode_workload(seq_lens=[256, 1024, 48], cfg=19)
    cache = fill_cache_cpu(w, consts).to(DEV)
    rot = consts["rotation_128_0"]
    ck, cv = consts["centroids_128_3"], consts["centroids_128_4"]
    q = w.q.to(DEV)
    full = K.split_k_paged_decode(q, cache, w.block_table.to(DEV), w.seq_lens.to(DEV), ck, cv,
                                  rot, 8, 128, 16, num_splits=2)
    cut = torch.tensor([128, 512, 16], dtype=torch.int32)       # tokens held by group 0
    first = K.paged_decode_partials(q, cache, w.block_table.to(DEV), cut.to(DEV), ck, cv, rot, 8,
                                    128, 16, num_splits=2).clone()
    rest_table = torch.zeros_like(w.block_table)
    for i in range(3):
        n0 = int(cut[i]) // 16
        rest_table[i, : w.block_table.shape[1] - n0] = w.block_table[i, n0:]
    second = K.paged_decode_partials(q, cache, rest_table.to(DEV), (w.seq_lens - cut).to(DEV), ck,
                                     cv, rot, 8, 128, 16, num_splits=2)
    merged = K.split_k_merge(torch.stack([first, second]), rot, torch.bfloat16)
    ref = run_oracle(w, cache.cpu(), consts)
    close(merged, ref, consts)
    close(full, ref, consts)


def test_partials_match_oracle_formulas(consts):
    w = W.decode_workload(seq_lens=[100], num_q_heads=4, num_kv_heads=1, cfg=16)
    cache = fill_cache_cpu(w, consts)
    rot, ck, cv = consts["rotation_128_0"], consts["centroids_128_3"], consts["centroids_128_4"]
    parts = K.paged_decode_partials(w.q.to(DEV), cache.to(DEV), w.block_table.to(DEV),
                                    w.seq_lens.to(DEV), ck, cv, rot, 1, 128, 16, num_splits=2).cpu()
    k, v = O.gather_paged(cache, w.block_table[0], 100, 1, 128, 16, ck, cv)
    q_rot = (w.q.float() @ rot.T).to(torch.bfloat16).float()
    for h in range(4):
        logits = (k[0] @ q_rot[0, h]) / np.sqrt(128)
        ref = torch.softmax(logits, 0) @ v[0]
        got = parts[0, h, :128] / parts[0, h, 129]
        assert (got - ref).abs().max().item() < 3e-3 * ref.abs().max().item() + 1e-4
        # l = sum 2^(logit*log2e - m)
        lse2 = torch.logsumexp(logits, 0).item() / np.log(2)
        assert abs(parts[0, h, 128].item() + np.log2(parts[0, h, 129].item()) - lse2) < 2e-3


def test_many_short_sequences_and_more_sequences_than_sms(consts):
    lens = [(7 * i) % 50 for i in range(300)]  # many zero-length and one-page sequences
    w = W.decode_workload(seq_lens=lens, num_q_heads=8, num_kv_heads=2, cfg=20)
    cache = fill_cache_cpu(w, consts)
    ref = run_oracle(w, cache, consts)
    for splits in (0, 3):
        close(run_gpu(w, cache, consts, num_splits=splits), ref, consts)


def test_full_size_config1_vs_oracle(consts):
    """32 sequences x 4096 tokens, 8 KV heads, GQA 4:1, 8 splits, seed-2 block table."""
    w = W.decode_workload()
    assert w.num_blocks == 8192 and w.algorithmic_bytes() == 143_163_392
    cache = fill_cache_cpu(w, consts)
    out = run_gpu(w, cache, consts, num_splits=8)
    ref = run_oracle(w, cache, consts)
    stats = close(out, ref, consts, got_rot32=gpu_rows(w, cache, consts, num_splits=8))
    # with the outlier channels some heads put nearly all weight on one token, so outputs reach
    # |3.5| where one bf16 step is 0.0156: entries beyond a flat 2e-3 exist (every one of them
    # within the per-entry bound checked above) and must stay rare
    print("configs[1] decode parity:", stats)
    assert stats["pre_max_abs"] < 5e-4
    assert stats["beyond_atol"] < 1e-3
    assert stats["identical"] > 0.8
    ws = K.decode_workspace(torch.device(DEV), 32, 32, 8, 128, 8)
    assert K.workspace_status(ws) == 0


def test_bad_block_index_is_reported_not_followed(consts):
    w = W.decode_workload(seq_lens=[40, 40], num_q_heads=8, num_kv_heads=8, cfg=17)
    cache = fill_cache_cpu(w, consts)
    bt = w.block_table.clone()
    bt[1, 1] = 10_000_000  # far outside the cache
    ws = torch.zeros(4 << 20, dtype=torch.uint8, device=DEV)
    K.split_k_paged_decode(w.q.to(DEV), cache.to(DEV), bt.to(DEV), w.seq_lens.to(DEV),
                           consts["centroids_128_3"], consts["centroids_128_4"],
                           consts["rotation_128_0"], 8, 128, 16, num_splits=2, workspace=ws)
    assert K.workspace_status(ws) & 1  # FQ_DEV_BAD_BLOCK_INDEX
    torch.cuda.synchronize()


def test_argument_errors(consts):
    from flashquant_b200._native import FlashQuantNativeError
    w = W.decode_workload(seq_lens=[20], num_q_heads=6, num_kv_heads=3, cfg=18)
    cache = torch.zeros(w.num_blocks, 16, 3 * 136, dtype=torch.uint8, device=DEV)
    with pytest.raises(FlashQuantNativeError) as e:
        run_gpu(w, cache, consts)
    assert e.value.code == -2  # 3 KV heads: unsupported, reported, no fallback
    w = W.decode_workload(seq_lens=[20], cfg=18)
    cache = torch.zeros(w.num_blocks, 16, 8 * 136, dtype=torch.uint8, device=DEV)
    with pytest.raises(FlashQuantNativeError) as e:
        K.split_k_paged_decode(w.q.to(DEV), cache, w.block_table.to(DEV), w.seq_lens.to(DEV),
                               consts["centroids_128_3"], consts["centroids_128_4"],
                               consts["rotation_128_0"], 8, 128, 16, num_splits=4,
                               workspace=torch.zeros(1024, dtype=torch.uint8, device=DEV))
    assert e.value.code == -3


def test_long_sequence_spread_over_every_team(consts):
    """One sequence of 20 000 tokens is cut into ~300 partial rows (one per team of warps)."""
    w = W.decode_workload(seq_lens=[20000, 40], num_q_heads=8, num_kv_heads=2, cfg=21)
    cache = fill_cache_cpu(w, consts)
    ref = run_oracle(w, cache, consts)
    for splits in (0, 5):
        close(run_gpu(w, cache, consts, num_splits=splits), ref, consts,
              got_rot32=gpu_rows(w, cache, consts, num_splits=splits))


@pytest.mark.parametrize("with_qjl,pinned", [(False, True), (True, True), (True, False)])
def test_host_step_equals_append_then_decode(consts, with_qjl, pinned):
    """fq_decode_step_host = copies + compress-on-append + decode: same bytes as the pieces,
    with page-locked and with pageable host arrays."""
    d, hkv, hq, bs = 128, 8, 32, 16
    w = W.decode_workload(num_q_heads=hq, num_kv_heads=hkv, head_dim=d, block_size=bs, cfg=1,
                          seq_lens=[33, 1, 700, 16, 257])
    grown = fill_cache_cpu(w, consts).to(DEV)
    rot, S = consts["rotation_128_0"], consts["qjl_128_0"]
    bk, ck = consts["boundaries_128_3"], consts["centroids_128_3"]
    bv, cv = consts["boundaries_128_4"], consts["centroids_128_4"]
    # the step appends one more token to every sequence, in the row after its last one (every
    # sequence owns as many pages as the longest, so the row exists)
    new_k, new_v = W.make_kv(w.num_seqs, hkv, d, 9, torch.bfloat16)
    bt = w.block_table
    pos = w.seq_lens.long()
    new_slots = bt[torch.arange(w.num_seqs), pos // bs].long() * bs + pos % bs
    lens = w.seq_lens + 1
    plane = torch.zeros(grown.shape[0], bs, hkv * (d // 8 + 4), dtype=torch.uint8, device=DEV)

    # the pieces, on device tensors
    ref_cache, ref_plane = grown.clone(), plane.clone()
    if with_qjl:
        K.tq4_compress_append_qjl(new_k.to(DEV), new_v.to(DEV), ref_cache, ref_plane,
                                  new_slots.to(DEV), rot, bk, ck, bv, S)
    else:
        K.tq4_compress_append(new_k.to(DEV), new_v.to(DEV), ref_cache, new_slots.to(DEV), rot, bk, bv)
    ref = K.split_k_paged_decode(w.q.to(DEV), ref_cache, bt.to(DEV), lens.to(DEV), ck, cv, rot,
                                 hkv, d, bs, num_splits=2)

    # the one call, on host tensors
    step = K.HostDecodeStep(grown, plane if with_qjl else None, rot, bk, ck, bv, cv,
                            S if with_qjl else None, w.num_seqs, hq, hkv, d, bs, bt.shape[1],
                            num_splits=2)
    host = (lambda t: t.contiguous().pin_memory()) if pinned else (lambda t: t.contiguous().clone())
    hout = host(torch.zeros_like(w.q))
    step(host(w.q), host(new_k), host(new_v), host(new_slots), host(bt), host(lens), hout)
    assert torch.equal(grown, ref_cache)
    if with_qjl:
        assert torch.equal(plane, ref_plane)
    assert torch.equal(hout.view(torch.int16), ref.cpu().view(torch.int16))
    assert K.workspace_status(step.workspace) == 0
    # A serving loop reuses its arrays: new contents in the same arrays must be seen.
    hq_buf = host(w.q)
    hk, hv, hs, hb, hl = host(new_k), host(new_v), host(new_slots), host(bt), host(lens)
    for it in range(4):
        q_it = (w.q.float() * (1.0 + 0.25 * it)).to(w.q.dtype)
        hq_buf.copy_(q_it)
        step(hq_buf, hk, hv, hs, hb, hl, hout)
        ref_it = K.split_k_paged_decode(q_it.to(DEV), ref_cache, bt.to(DEV), lens.to(DEV), ck, cv,
                                        rot, hkv, d, bs, num_splits=2)
        assert torch.equal(hout.view(torch.int16), ref_it.cpu().view(torch.int16)), f"call {it}"
    assert K.workspace_status(step.workspace) == 0
    # the packed form: all inputs in one page-locked block, one or two copies in
    if pinned:
        _, views = step.host_block()
        for name, t in (("key", new_k), ("value", new_v), ("slot_mapping", new_slots),
                        ("seq_lens", lens), ("block_table", bt), ("q", w.q)):
            views[name].copy_(t)
        # (False, False: the second call replays the graph that the first one captured)
        for overlap in (False, False, True, True):
            views["out"].zero_()
            got = step.packed(overlap_copies=overlap)
            assert torch.equal(got.view(torch.int16), ref.cpu().view(torch.int16)), overlap
            assert torch.equal(grown, ref_cache)
        # new contents in the same block are seen by the replayed graph
        q_it = (w.q.float() * 1.5).to(w.q.dtype)
        views["q"].copy_(q_it)
        got = step.packed(overlap_copies=False)
        ref_it = K.split_k_paged_decode(q_it.to(DEV), ref_cache, bt.to(DEV), lens.to(DEV), ck, cv,
                                        rot, hkv, d, bs, num_splits=2)
        assert torch.equal(got.view(torch.int16), ref_it.cpu().view(torch.int16))
        # and the same step issued call by call
        K.N.load().fq_decode_step_set_graph(0)
        try:
            views["q"].copy_(w.q)
            got = step.packed(overlap_copies=False)
            assert torch.equal(got.view(torch.int16), ref.cpu().view(torch.int16))
        finally:
            K.N.load().fq_decode_step_set_graph(1)
        assert K.workspace_status(step.workspace) == 0
    hout.copy_(ref.cpu())
    # and against the oracle end to end
    ref32, ref_out = O.split_k_paged_decode_stages(w.q, ref_cache.cpu(), bt, lens, ck, cv, rot,
                                                   hkv, d, bs, None)
    attention_close(hout, ref_out, ref32, rot)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_two_stage_scoring_vs_oracle(consts, dtype):
    """Logits with the QJL correction read from the side plane: cache and plane written by the
    GPU append, decode against the oracle's estimator on the same bytes."""
    d, hkv, hq, bs = 128, 8, 32, 16
    w = W.decode_workload(num_q_heads=hq, num_kv_heads=hkv, head_dim=d, block_size=bs, cfg=1,
                          seq_lens=[70, 0, 513, 16, 1], dtype=dtype)
    rot, S = consts["rotation_128_0"], consts["qjl_128_0"]
    bk, ck = consts["boundaries_128_3"], consts["centroids_128_3"]
    bv, cv = consts["boundaries_128_4"], consts["centroids_128_4"]
    k, v = W.make_kv(w.total_tokens, hkv, d, 1, dtype)
    cache = torch.zeros(w.num_blocks, bs, hkv * (d + 8), dtype=torch.uint8, device=DEV)
    plane = torch.zeros(w.num_blocks, bs, hkv * (d // 8 + 4), dtype=torch.uint8, device=DEV)
    K.tq4_compress_append_qjl(k.to(DEV), v.to(DEV), cache, plane, w.slot_mapping.to(DEV), rot, bk,
                              ck, bv, S)
    ref32, ref = O.qjl_paged_decode_stages(w.q, cache.cpu(), plane.cpu(), w.block_table,
                                           w.seq_lens, ck, cv, rot, S, hkv, d, bs)
    for splits in (0, 4):
        out = K.split_k_paged_decode_qjl(w.q.to(DEV), cache, plane, w.block_table.to(DEV),
                                         w.seq_lens.to(DEV), ck, cv, rot, S, hkv, d, bs,
                                         num_splits=splits)
        # the generic kernel's sign-bit product runs on fp16(q S^T): 2^-9 before the rounding
        attention_close(out, ref, ref32, rot, rtol=2.0 ** -9)
        assert (out[1] == 0).all()  # empty sequence
    # the correction matters: the one-stage logits give another answer on the same cache
    plain = K.split_k_paged_decode(w.q.to(DEV), cache, w.block_table.to(DEV), w.seq_lens.to(DEV),
                                   ck, cv, rot, hkv, d, bs)
    assert (plain.float() - out.float()).abs().max().item() > 1e-2
    ws = K.decode_workspace(torch.device(DEV), w.num_seqs, hq, hkv, d, 0)
    assert K.workspace_status(ws) == 0


def test_three_launch_form_gives_the_same_answer(consts):
    """The fallback for GPUs that cannot hold the cooperative launch: rotation, streaming and
    merge as separate launches, same contract."""
    w = W.decode_workload(num_q_heads=32, num_kv_heads=8, head_dim=128, block_size=16, cfg=1,
                          seq_lens=[300, 0, 17, 2048, 64])
    cache = fill_cache_cpu(w, consts)
    ref = run_oracle(w, cache, consts)
    one = run_gpu(w, cache, consts, num_splits=3)
    K.set_single_launch(False)
    try:
        n0 = K.N.load().fq_launch_count()
        three = run_gpu(w, cache, consts, num_splits=3)
        assert K.N.load().fq_launch_count() - n0 == 3
    finally:
        K.set_single_launch(True)
    close(three, ref, consts)
    close(one, ref, consts)
    assert (three[1] == 0).all()
    # both forms round the same rotated query and merge the same partial rows
    assert (one.float() - three.float()).abs().max().item() <= 2.0 ** -6


@pytest.mark.parametrize("n_q,lens", [(4, [0, 1, 3, 4, 5, 64, 301, 1000]), (2, [17, 2048]),
                                      (1, [9, 300]), (3, [2, 40, 33, 700]),
                                      (2, [0, 1, 2, 15, 16, 17, 18, 31, 32, 33])])
def test_multi_token_steps_vs_oracle(consts, n_q, lens):
    # the last n_q tokens of every sequence in one call: query i sees keys 0 .. L - n_q + i;
    # sequences shorter than n_q have queries without any key (zeros)
    w = W.decode_workload(seq_lens=lens, num_q_heads=32, num_kv_heads=8, cfg=70 + n_q)
    cache = fill_cache_cpu(w, consts)
    args = (consts["centroids_128_3"], consts["centroids_128_4"], consts["rotation_128_0"])
    g = torch.Generator().manual_seed(900 + n_q)
    q = torch.randn(w.num_seqs, n_q, 32, 128, generator=g).to(torch.bfloat16)
    out = fq.split_k_paged_decode_multi(q.to(DEV), cache.to(DEV), w.block_table.to(DEV),
                                        w.seq_lens.to(DEV), *args, 8, 128, 16)
    ref32, ref = O.paged_decode_multi_stages(q, cache, w.block_table, w.seq_lens, *args, 8, 128, 16)
    assert out.shape == q.shape
    attention_close(out.cpu(), ref, ref32, args[2])
    # a query without visible keys: exact zeros
    for i, n in enumerate(lens):
        for t in range(n_q):
            if n - n_q + t < 0:
                assert bool((out[i, t] == 0).all())
    # the last query of each sequence is the single-token call (another partition of the keys
    # over the teams, so equal up to the order of the sums)
    one = fq.split_k_paged_decode(q[:, -1].contiguous().to(DEV), cache.to(DEV),
                                  w.block_table.to(DEV), w.seq_lens.to(DEV), *args, 8, 128, 16)
    attention_close(out[:, -1].cpu(), one.cpu(), ref32[:, -1], args[2], slack=2.0)


def test_sequence_longer_than_its_block_table_row_is_cut_and_reported(consts):
    """A seq_len beyond the row's columns would make the page walk read the next row (or past
    the table): the walk stops at the row's width and the status word says so.  The table is a
    narrow view inside a wider allocation, so nothing leaves the allocation either way."""
    w = W.decode_workload(seq_lens=[64, 64], num_q_heads=32, num_kv_heads=8, cfg=23)
    cache = fill_cache_cpu(w, consts).to(DEV)
    wide = torch.zeros(2, 16, dtype=torch.int32, device=DEV)
    wide[:, :4] = w.block_table.to(DEV)
    narrow = wide[:, :4]                       # stride 16, 4 valid columns
    lens = torch.tensor([64, 64 + 3 * 16], dtype=torch.int32, device=DEV)   # 7 pages claimed
    args = (consts["centroids_128_3"], consts["centroids_128_4"], consts["rotation_128_0"], 8, 128, 16)
    ws = torch.zeros(8 << 20, dtype=torch.uint8, device=DEV)
    lib = K.N.load()
    out = torch.empty_like(w.q, device=DEV)
    # the C ABI takes the stride as the row width: hand it the narrow width
    rot = consts["rotation_128_0"].contiguous().to(DEV)
    ck, cv = consts["centroids_128_3"].to(DEV), consts["centroids_128_4"].to(DEV)
    tight = narrow.contiguous()
    K.N.check(lib.fq_split_k_paged_decode(
        K.N.ptr(w.q.to(DEV)), K.N.dtype_code(w.q.dtype), K.N.ptr(cache), K.N.ptr(tight), 4,
        K.N.ptr(lens), K.N.ptr(ck), 8, K.N.ptr(cv), 16, K.N.ptr(rot), 2, 32, 8, 128, 16,
        cache.shape[0], 1.0 / np.sqrt(128), K.N.ptr(out), 2, K.N.ptr(ws), ws.numel(),
        K.N.stream_ptr(torch.device(DEV))))
    assert K.workspace_status(ws) & 1          # FQ_DEV_BAD_BLOCK_INDEX
    # sequence 0 is untouched by its neighbour's claim; sequence 1 attended over its 4 pages
    ws.zero_()
    ok = K.split_k_paged_decode(w.q.to(DEV), cache, tight, w.seq_lens.to(DEV), *args, num_splits=2,
                                workspace=ws)
    assert K.workspace_status(ws) == 0
    assert torch.equal(out.view(torch.int16), ok.view(torch.int16))


def test_bounded_wait_gives_up_and_the_call_returns(consts):
    """Every device-side wait is bounded in time.  The merge phase of the single launch is told
    to expect one segment more than its sequences will ever produce; with the limit at 2 ms the
    waits give up, the status word carries FQ_DEV_WAIT_TIMEOUT and the call returns promptly.
    Nothing faults and the GPU is not left spinning."""
    import time
    lib = K.N.load()
    w = W.decode_workload(seq_lens=[300, 40], num_q_heads=32, num_kv_heads=8, cfg=24)
    cache = fill_cache_cpu(w, consts).to(DEV)
    args = (w.q.to(DEV), cache, w.block_table.to(DEV), w.seq_lens.to(DEV), consts["centroids_128_3"],
            consts["centroids_128_4"], consts["rotation_128_0"], 8, 128, 16)
    ws = torch.zeros(8 << 20, dtype=torch.uint8, device=DEV)
    good = K.split_k_paged_decode(*args, num_splits=2, workspace=ws)
    old = lib.fq_get_device_wait_limit_ns()
    try:
        lib.fq_set_device_wait_limit_ns(2_000_000)
        lib.fq_paged_decode_test_expect_extra_segments(1)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        K.split_k_paged_decode(*args, num_splits=2, workspace=ws)
        torch.cuda.synchronize()
        took = time.perf_counter() - t0
    finally:
        lib.fq_paged_decode_test_expect_extra_segments(0)
        lib.fq_set_device_wait_limit_ns(old)
    assert K.workspace_status(ws) & 2          # FQ_DEV_WAIT_TIMEOUT
    assert took < 1.0, f"the call took {took:.2f} s"
    # the contract after a status bit: zero the head of the workspace, then it works again
    ws[:32768].zero_()
    again = K.split_k_paged_decode(*args, num_splits=2, workspace=ws)
    assert K.workspace_status(ws) == 0
    assert torch.equal(again.view(torch.int16), good.view(torch.int16))


def test_fp32_query_and_config0_shapes(consts):
    """configs[0]: fp32 K/V [1, 8, 1024, 128] (K two-stage, V one-stage), one fp32 query token
    of 32 heads: codes, norms, reconstruction error and the attention output."""
    from parity import check_codes, check_gamma, check_norms, check_signs
    rot, S = consts["rotation_128_0"], consts["qjl_128_0"]
    b3, c3 = consts["boundaries_128_3"], consts["centroids_128_3"]
    b4, c4 = consts["boundaries_128_4"], consts["centroids_128_4"]
    g = torch.Generator().manual_seed(1000)
    k = torch.randn(1, 8, 1024, 128, generator=g)
    k[..., W.outlier_channels(128)] *= 10.0
    v = torch.randn(1, 8, 1024, 128, generator=torch.Generator().manual_seed(2000))
    q = torch.randn(1, 32, 128, generator=torch.Generator().manual_seed(3000))
    # quantisers on the fp32 tensors
    idx, kn, signs, gamma = O.prod_quantize(k, rot, c3, b3, S)
    pk, kn2, bits, g2 = fq.tq_prod_quantize(k[0].to(DEV), rot, b3, c3, S)   # (8, 1024, 128)
    check_codes(pk, k, rot, b3, O.nibble_pack(idx))
    check_norms(kn2, kn)
    codes = O.nibble_unpack(pk.cpu())
    check_gamma(g2, gamma, k, codes, idx, kn2.cpu(), rot, c3)
    check_signs(bits, signs, k, codes, idx, kn2.cpu(), rot, c3, S)
    pv_ref, vn_ref = O.compress(v[0], rot, b4)                               # (8, 1024, ...)
    pv, vn = fq.tq4_compress(v.to(DEV).reshape(-1, 1, 128), rot, b4)
    check_codes(pv.reshape(pv_ref.shape), v, rot, b4, pv_ref)
    check_norms(vn, vn_ref)
    # reconstruction error of both, against the oracle's
    rec_v = fq.tq4_decompress_original(pv, vn, c4, rot, dtype=torch.float32).cpu().reshape(v.shape)
    ref_v = O.mse_dequantize(O.nibble_unpack(pv_ref).long(), vn_ref, rot, c4)
    mse, mse_ref = (rec_v - v).pow(2).mean().item(), (ref_v - v).pow(2).mean().item()
    assert abs(mse - mse_ref) <= 1e-4 * mse_ref, (mse, mse_ref)
    assert 0.005 < mse_ref < 0.02      # 4 bits at d = 128: about 1 % of the variance
    # the single-query attention over a paged cache built from them (token-major rows)
    kt, vt = k[0].transpose(0, 1).contiguous(), v[0].transpose(0, 1).contiguous()
    w = W.decode_workload(seq_lens=[1024], num_q_heads=32, num_kv_heads=8, cfg=0)
    cache = torch.zeros(w.num_blocks, 16, 8 * 136, dtype=torch.uint8, device=DEV)
    K.tq4_compress_append(kt.to(DEV), vt.to(DEV), cache, w.slot_mapping.to(DEV), rot, b3, b4)
    ref_cache = torch.zeros(w.num_blocks, 16, 8 * 136, dtype=torch.uint8)
    O.compress_and_store(kt, vt, ref_cache, w.slot_mapping, rot, b3, b4)
    out = K.split_k_paged_decode(q.to(DEV), cache, w.block_table.to(DEV), w.seq_lens.to(DEV), c3, c4,
                                 rot, 8, 128, 16, num_splits=4)
    assert out.dtype == torch.float32
    # with fp32 tensors the reference rounds nothing: out = (softmax(...) V) Pi in fp32
    ref32, ref = O.split_k_paged_decode_stages(q, cache.cpu(), w.block_table, w.seq_lens, c3, c4,
                                               rot, 8, 128, 16)
    err = (out.cpu() - ref).abs()
    assert err.max().item() <= 2e-3, err.max().item()
    # the rotated query meets the keys as fp16 (2^-12 of each coordinate)
    assert err.max().item() <= 2.0 ** -9 * ref.abs().max().item()


def test_config4_shapes_ragged_long_sequences(consts):
    """configs[4]: 64 query heads / 8 KV heads, batch 8, lengths uniform in [32768, 131072]
    from seed 4.  The cache is written by the (parity-tested) GPU append; the oracle attends
    over two whole sequences: the longest and the shortest."""
    lens = W.ragged_lengths()                       # the seed-4 lengths
    assert lens.min().item() >= 32768 and lens.max().item() <= 131072
    hq, hkv, d, bs = 64, 8, 128, 16
    rot = consts["rotation_128_0"]
    b3, c3 = consts["boundaries_128_3"], consts["centroids_128_3"]
    b4, c4 = consts["boundaries_128_4"], consts["centroids_128_4"]
    w = W.decode_workload(seq_lens=lens.tolist(), num_q_heads=hq, num_kv_heads=hkv, cfg=4)
    cache = torch.zeros(w.num_blocks, bs, hkv * (d + 8), dtype=torch.uint8, device=DEV)
    at = 0
    for i, n in enumerate(lens.tolist()):           # K/V of one sequence at a time
        k, v = W.make_kv(n, hkv, d, cfg=400 + i)
        K.tq4_compress_append(k.to(DEV), v.to(DEV), cache, w.slot_mapping[at:at + n].to(DEV), rot,
                              b3, b4)
        at += n
    args = (w.q.to(DEV), cache, w.block_table.to(DEV), w.seq_lens.to(DEV), c3, c4, rot, hkv, d, bs)
    out = K.split_k_paged_decode(*args, num_splits=8)
    rows = rows_from_partials(K.paged_decode_partials(*args, num_splits=8))
    ws = K.decode_workspace(torch.device(DEV), 8, hq, hkv, d, 8)
    assert K.workspace_status(ws) == 0
    cache_cpu = cache.cpu()
    for i in (int(lens.argmax()), int(lens.argmin())):
        sel = slice(i, i + 1)
        ref32, ref = O.split_k_paged_decode_stages(
            w.q[sel], cache_cpu, w.block_table[sel], w.seq_lens[sel], c3, c4, rot, hkv, d, bs,
            per_kv_head=True)
        # eight query heads per KV head fill all product columns: one fp16 term per weight,
        # 2^-9 of the entry before the rounding
        attention_close(out[sel], ref, ref32, rot, got_rot32=rows[sel], rtol=2.0 ** -9)
