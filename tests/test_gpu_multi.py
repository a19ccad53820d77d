"""Two-GPU checks (skipped on a single-GPU box): the token-range split of long sequences with
one NCCL all-gather of partial rows equals the single-GPU decode, and KV-head sharding needs
no communication at all."""

import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _need_two():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")


def _setup(rank, world, port):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    return dist


def _case(cfg, hq, hkv, lens):
    from conftest import load_golden
    from flashquant_b200 import workloads as W
    from oracle import tq_oracle as O
    C = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in load_golden("constants.npz").items()}
    w = W.decode_workload(seq_lens=lens, num_q_heads=hq, num_kv_heads=hkv, cfg=cfg)
    k, v = W.make_kv(w.total_tokens, hkv, 128, cfg)
    cache = torch.zeros(w.num_blocks, 16, hkv * 136, dtype=torch.uint8)
    O.compress_and_store(k, v, cache, w.slot_mapping, C["rotation_128_0"], C["boundaries_128_3"],
                         C["boundaries_128_4"])
    return C, w, cache, k, v


def _token_split_worker(rank, world, port, result):
    import flashquant_b200 as fq
    from flashquant_b200 import distributed as D
    dist = _setup(rank, world, port)
    dev = torch.device("cuda", rank)
    C, w, cache, _, _ = _case(51, 32, 8, [20000, 333, 16])
    rot, ck, cv = C["rotation_128_0"], C["centroids_128_3"], C["centroids_128_4"]
    bt, lens = D.local_view(w.block_table, w.seq_lens, 16, rank, world)
    q, cache_d = w.q.to(dev), cache.to(dev)
    out = D.cross_gpu_decode(
        lambda: fq.paged_decode_partials(q, cache_d, bt.to(dev), lens.to(dev), ck, cv, rot, 8, 128, 16),
        lambda g: fq.split_k_merge(g, rot, q.dtype))
    full = fq.split_k_paged_decode(q, cache_d, w.block_table.to(dev), w.seq_lens.to(dev), ck, cv,
                                   rot, 8, 128, 16)
    # both against the oracle's two-stage values (checked in the parent process)
    result[rank] = {"out": out.cpu(), "full": full.cpu()}
    dist.barrier()
    dist.destroy_process_group()


def _head_shard_worker(rank, world, port, result):
    import flashquant_b200 as fq
    from flashquant_b200 import distributed as D
    from oracle import tq_oracle as O
    dist = _setup(rank, world, port)
    dev = torch.device("cuda", rank)
    C, w, cache, k, v = _case(52, 16, 2, [1000, 77])
    rot, ck, cv = C["rotation_128_0"], C["centroids_128_3"], C["centroids_128_4"]
    kv, qh = D.shard_kv_heads(2, 16, rank, world)
    # this rank's cache rows hold only its KV head
    local = torch.zeros(w.num_blocks, 16, 136, dtype=torch.uint8, device=dev)
    fq.tq4_compress_append(k[:, kv].contiguous().to(dev), v[:, kv].contiguous().to(dev), local,
                           w.slot_mapping.to(dev), rot, C["boundaries_128_3"], C["boundaries_128_4"])
    out = fq.split_k_paged_decode(w.q[:, qh].contiguous().to(dev), local, w.block_table.to(dev),
                                  w.seq_lens.to(dev), ck, cv, rot, 1, 128, 16)
    result[rank] = {"out": out.cpu(), "heads": (qh.start, qh.stop)}
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("worker,port", [(_token_split_worker, 29531), (_head_shard_worker, 29532)])
def test_two_gpus(worker, port):
    _need_two()
    import torch.multiprocessing as mp
    with mp.Manager() as mgr:
        result = mgr.dict()
        mp.spawn(worker, args=(2, port, result), nprocs=2, join=True)
        got = {r: dict(result[r]) for r in range(2)}
    from oracle import tq_oracle as O
    from parity import attention_close
    if worker is _token_split_worker:
        C, w, cache, _, _ = _case(51, 32, 8, [20000, 333, 16])
        hkv = 8
    else:
        C, w, cache, _, _ = _case(52, 16, 2, [1000, 77])
        hkv = 2
    rot = C["rotation_128_0"]
    ref32, ref = O.split_k_paged_decode_stages(w.q, cache, w.block_table, w.seq_lens,
                                               C["centroids_128_3"], C["centroids_128_4"], rot,
                                               hkv, 128, 16)
    for r in range(2):
        if worker is _token_split_worker:
            attention_close(got[r]["out"], ref, ref32, rot)
            attention_close(got[r]["full"], ref, ref32, rot)
        else:
            a, b = got[r]["heads"]
            attention_close(got[r]["out"], ref[:, a:b], ref32[:, a:b], rot)
