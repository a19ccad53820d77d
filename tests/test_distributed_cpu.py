"""Host-side multi-GPU logic on CPU ranks (gloo, world size 2): token-range views, the single
all-gather of partial rows and the merge reproduce the unsplit decode."""

import math
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import load_golden
from flashquant_b200 import distributed as D
from flashquant_b200 import workloads as W
from oracle import tq_oracle as O


def test_partition_helpers():
    assert [D.shard_sequences(10, r, 4) for r in range(4)] == [slice(0, 2), slice(2, 5), slice(5, 7), slice(7, 10)]
    kv, qh = D.shard_kv_heads(8, 64, 3, 8)
    assert (kv, qh) == (slice(3, 4), slice(24, 32))
    with pytest.raises(ValueError):
        D.shard_kv_heads(8, 32, 0, 3)
    # ranges tile the sequence, page aligned
    for n in (0, 1, 16, 17, 131072, 40000):
        edges = [D.token_range(n, 16, r, 8) for r in range(8)]
        assert edges[0][0] == 0 and edges[-1][1] == n
        for (a, b), (c, d) in zip(edges, edges[1:]):
            assert b == c or (b == n and c >= n) and a % 16 == 0


def _partial_rows_cpu(q_rot, cache, bt, lens, ck, cv, hkv, d, bs):
    """(acc, m, l) per (sequence, q head) with the kernel's row layout, base-2 exponents."""
    n_seq, hq, _ = q_rot.shape
    g = hq // hkv
    rows = torch.zeros(n_seq, hq, d + 4)
    rows[..., d] = -math.inf
    for i in range(n_seq):
        n = int(lens[i])
        if n == 0:
            continue
        k, v = O.gather_paged(cache, bt[i], n, hkv, d, bs, ck, cv)
        for h in range(hq):
            s = (k[h // g] @ q_rot[i, h].float()) / math.sqrt(d) * math.log2(math.e)
            m = s.max()
            e = torch.exp2(s - m)
            rows[i, h, :d] = e @ v[h // g]
            rows[i, h, d] = m
            rows[i, h, d + 1] = e.sum()
    return rows


def _merge_rows_cpu(gathered, rot, dtype):
    m = gathered[..., -4]
    m_star = m.max(dim=0).values
    w = torch.where(torch.isinf(m), torch.zeros_like(m), torch.exp2(m - m_star))
    num = (w.unsqueeze(-1) * gathered[..., :-4]).sum(0)
    den = (w * gathered[..., -3]).sum(0)
    o = torch.where(den.unsqueeze(-1) > 0, num / den.unsqueeze(-1).clamp_min(1e-38), torch.zeros_like(num))
    return (o.to(dtype).float() @ rot).to(dtype)


def _worker(rank, world, port, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    z = load_golden("constants.npz")
    C = {k: torch.from_numpy(v).contiguous() for k, v in z.items()}
    rot, ck, cv = C["rotation_128_0"], C["centroids_128_3"], C["centroids_128_4"]
    w = W.decode_workload(seq_lens=[300, 16, 0, 75], num_q_heads=8, num_kv_heads=2, cfg=31)
    k, v = W.make_kv(w.total_tokens, 2, 128, 31)
    cache = torch.zeros(w.num_blocks, 16, 2 * 136, dtype=torch.uint8)
    O.compress_and_store(k, v, cache, w.slot_mapping, rot, C["boundaries_128_3"], C["boundaries_128_4"])
    q_rot = (w.q.float() @ rot.T).to(torch.bfloat16)
    bt, lens = D.local_view(w.block_table, w.seq_lens, 16, rank, world)
    out = D.cross_gpu_decode(
        lambda: _partial_rows_cpu(q_rot, cache, bt, lens, ck, cv, 2, 128, 16),
        lambda g: _merge_rows_cpu(g, rot, torch.bfloat16))
    ref = O.split_k_paged_decode(w.q, cache, w.block_table, w.seq_lens, ck, cv, rot, 2, 128, 16)
    err = (out.float() - ref.float()).abs().max().item()
    total = torch.tensor([float(lens.sum())])
    dist.all_reduce(total)
    result[rank] = (err, float(total), float(w.seq_lens.sum()))
    dist.destroy_process_group()


def test_two_rank_token_split_matches_unsplit_decode():
    world = 2
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(_worker, args=(world, 29517, result), nprocs=world, join=True)
        for r in range(world):
            err, total, want = result[r]
            assert total == want        # the local views cover every token exactly once
            assert err <= 4e-3          # one bf16 step at these magnitudes
