"""Benchmark of the TQ4 split-K paged decode (Llama-3-8B shape) on 1..8 B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A step is one attention-layer decode call over the whole batch: 32 sequences x 4096 cached
tokens, 32 query heads / 8 KV heads, head_dim 128, pages of 16 tokens, 8 splits; the call
includes the query rotation, the streaming kernel, the split-K merge and the output
rotation.  With N > 1 (launched by torchrun, one rank per GPU) every rank decodes its own
batch of the same shape - sequences are independent, so there is no collective on the data
path (weak scaling) - and the time is the maximum over ranks.

One JSON line is printed by rank 0; `python bench.py --help` lists the secondary workloads.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "tq4_paged_decode_tokens_per_s"
UNIT = "tokens/s"
NUM_SEQS, CONTEXT, HQ, HKV, D, BS, SPLITS = 32, 4096, 32, 8, 128, 16, 8
D_ = D  # (the secondary blocks import flashquant_b200.distributed as D)
CACHE_COPIES = 3  # 3 x 142.6 MB of packed cache are cycled so that no step finds its pages in L2


def workload_config(n_gpus):
    return {
        "workload": "configs[1]: Llama-3-8B-shaped paged decode, batch 32 x context 4096, "
                    "32 q / 8 kv heads, head_dim 128, block 16, K=TurboQuantProd(3-bit codes), "
                    "V=TurboQuantMSE 4-bit, 8 splits, seed-2 block table",
        "num_seqs_per_gpu": NUM_SEQS, "context": CONTEXT, "num_splits": SPLITS,
        "sharding": f"sequences, {n_gpus} independent rank(s), no collective",
        "l2": f"{CACHE_COPIES} cache copies of 142.6 MB cycled (> 126 MB L2), no flush needed",
        "seeds": {"rotation": 0, "qjl": 1, "K": 1001, "V": 2001, "Q": 3001, "block_table": 2},
    }


# --------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------
class ClockSampler:
    """Polls SM clock and throttle reasons of one GPU through NVML while a region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: report nulls
            self._nv = None

    def _run(self):
        nv = self._nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.002)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# --------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------
def run_ours(args):
    import flashquant_b200 as fq
    from flashquant_b200 import _native, kernels as K, workloads as W

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path to time)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    lib = _native.load()

    # ---- constants and inputs ------------------------------------------------------------
    q3, q4 = fq.TurboQuantProd(D, 4, seed=0), fq.TurboQuantMSE(D, 4, seed=0)
    rot = q4.rotation.to(dev)
    S = q3.qjl_matrix.to(dev)
    bk, ck = q3.mse_quantizer.boundaries.to(dev), q3.mse_quantizer.centroids.to(dev)
    bv, cv = q4.boundaries.to(dev), q4.centroids.to(dev)
    w = W.decode_workload(NUM_SEQS, CONTEXT, HQ, HKV, D, BS, cfg=1)
    k_cpu, v_cpu = W.make_kv(w.total_tokens, HKV, D, cfg=1)
    caches, planes = [], []
    slots = w.slot_mapping.to(dev)
    kd, vd = k_cpu.to(dev), v_cpu.to(dev)
    for _ in range(CACHE_COPIES):
        c = torch.zeros(w.num_blocks, BS, HKV * (D + 8), dtype=torch.uint8, device=dev)
        p = torch.zeros(w.num_blocks, BS, HKV * (D // 8 + 4), dtype=torch.uint8, device=dev)
        K.tq4_compress_append_qjl(kd, vd, c, p, slots, rot, bk, ck, bv, S)
        caches.append(c)
        planes.append(p)
    del kd, vd
    q = w.q.to(dev)
    bt, sl = w.block_table.to(dev), w.seq_lens.to(dev)
    out = torch.empty_like(q)
    ws = K.decode_workspace(dev, NUM_SEQS, HQ, HKV, D, SPLITS)
    torch.cuda.synchronize()

    def decode(i):
        return K.split_k_paged_decode(q, caches[i % CACHE_COPIES], bt, sl, ck, cv, rot, HKV, D, BS,
                                      out=out, num_splits=SPLITS, workspace=ws)

    # ---- graphs: one captured decode call per cache copy ------------------------------
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for i in range(CACHE_COPIES):
            decode(i)
    side.synchronize()
    launches_per_step = None
    graphs = []
    for i in range(CACHE_COPIES):
        g = torch.cuda.CUDAGraph()
        n0 = lib.fq_launch_count()
        with torch.cuda.graph(g):
            decode(i)
        launches_per_step = lib.fq_launch_count() - n0
        graphs.append(g)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    with sampler:
        for i in range(args.warmup):
            graphs[i % CACHE_COPIES].replay()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for i in range(args.steps):
            graphs[i % CACHE_COPIES].replay()
        t1.record()
        barrier()
        ms = t0.elapsed_time(t1)

        # ---- the same step with the two-stage (QJL) estimator in the logits --------------
        qgraphs = []
        with torch.cuda.stream(side):
            for i in range(CACHE_COPIES):
                K.split_k_paged_decode_qjl(q, caches[i], planes[i], bt, sl, ck, cv, rot, S, HKV, D,
                                           BS, out=out, num_splits=SPLITS, workspace=ws)
        side.synchronize()
        for i in range(CACHE_COPIES):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                K.split_k_paged_decode_qjl(q, caches[i], planes[i], bt, sl, ck, cv, rot, S, HKV, D,
                                           BS, out=out, num_splits=SPLITS, workspace=ws)
            qgraphs.append(g)
        qsteps = max(30, args.steps // 4)
        for i in range(3):
            qgraphs[i % CACHE_COPIES].replay()
        torch.cuda.synchronize()
        q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        q0.record()
        for i in range(qsteps):
            qgraphs[i % CACHE_COPIES].replay()
        q1.record()
        torch.cuda.synchronize()
        qjl_ms = q0.elapsed_time(q1) / qsteps

        # ---- dominant kernel alone (the streaming kernel), same inputs ------------------
        q_rot16 = (q.float() @ rot.T).to(q.dtype).to(torch.float16).contiguous()

        def stream_only(i):
            _native.check(lib.fq_paged_decode_stream(
                _native.ptr(q_rot16), _native.ptr(caches[i % CACHE_COPIES]), _native.ptr(bt),
                bt.stride(0), _native.ptr(sl), _native.ptr(ck), ck.numel(), _native.ptr(cv),
                cv.numel(), NUM_SEQS, HQ, HKV, D, BS, w.num_blocks, 1.0 / D ** 0.5, SPLITS,
                _native.ptr(ws), ws.numel(), _native.stream_ptr(dev)))

        with torch.cuda.stream(side):
            stream_only(0)
        side.synchronize()
        kg = torch.cuda.CUDAGraph()
        with torch.cuda.graph(kg):
            for i in range(CACHE_COPIES):
                stream_only(i)
        reps = max(8, args.steps // CACHE_COPIES)
        for _ in range(3):
            kg.replay()
        torch.cuda.synchronize()
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record()
        for _ in range(reps):
            kg.replay()
        k1.record()
        torch.cuda.synchronize()
        kernel_ms = k0.elapsed_time(k1) / (reps * CACHE_COPIES)

    # ---- end to end: host buffers in, host buffer out, every step -----------------------
    e2e_steps = max(args.steps, 200) if args.steps < 2000 else 2000  # 20 steps would be noise
    if args.e2e_steps:
        e2e_steps = args.e2e_steps  # short profiling runs
    hq_ = w.q.pin_memory()
    new_k = k_cpu.reshape(NUM_SEQS, CONTEXT, HKV, D)[:, -1].contiguous().pin_memory()
    new_v = v_cpu.reshape(NUM_SEQS, CONTEXT, HKV, D)[:, -1].contiguous().pin_memory()
    new_slots = w.slot_mapping.reshape(NUM_SEQS, CONTEXT)[:, -1].contiguous().pin_memory()
    hbt, hsl = w.block_table.pin_memory(), w.seq_lens.pin_memory()
    hout = torch.empty_like(hq_).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in (hq_, new_k, new_v, new_slots, hbt, hsl))
    d2h = hout.numel() * hout.element_size()
    # the reference-facing call with host buffers: one C-ABI call per step does the copies,
    # the compress-on-append, the decode and the copy back, and waits for the stream
    # (the reference's step writes the main cache row only - its _compress_and_store has no QJL
    # plane - so the step appends with the one-stage quantiser)
    step = K.HostDecodeStep(caches[0], None, rot, bk, ck, bv, cv, None, NUM_SEQS, HQ, HKV, D,
                            BS, hbt.shape[1], dtype=hq_.dtype, num_splits=SPLITS,
                            slot_dtype=new_slots.dtype)

    # three forms of the same step: six host arrays (six copies in), and the packed block with
    # one copy in or with two halves of it, the second under the compress-on-append
    _, views = step.host_block()
    for name, t in (("key", new_k), ("value", new_v), ("slot_mapping", new_slots),
                    ("seq_lens", hsl), ("block_table", hbt), ("q", hq_)):
        views[name].copy_(t)

    def six_arrays(i):
        step(hq_, new_k, new_v, new_slots, hbt, hsl, hout,
             kv_cache=caches[i % CACHE_COPIES])

    def packed(overlap):
        return lambda i: step.packed(overlap_copies=overlap, kv_cache=caches[i % CACHE_COPIES])

    e2e_forms = {}
    for form, fn in (("six_host_arrays", six_arrays), ("packed_block_one_copy", packed(False)),
                     ("packed_block_two_halves", packed(True))):
        for i in range(3):
            fn(i)
        barrier()
        n0 = lib.fq_launch_count()
        tw = time.perf_counter()
        for i in range(e2e_steps):
            fn(i)
        e2e_forms[form] = (time.perf_counter() - tw, lib.fq_launch_count() - n0)
        barrier()
    assert torch.equal(views["out"].view(torch.int16), hout.view(torch.int16))
    e2e_form = min(("packed_block_one_copy", "packed_block_two_halves"),
                   key=lambda f: e2e_forms[f][0])
    e2e_s, e2e_launches = e2e_forms[e2e_form]

    # ---- further rows of the hot path, short runs in the same process ------------------------
    extras = {}
    if not args.no_extras:
        ctx = dict(dev=dev, rank=rank, world=world, dist=dist, rot=rot, S=S, bk=bk, ck=ck, bv=bv, cv=cv,
                   peaks=_peaks(), caches=caches, w=w, ws=ws)
        for name, fn in (("strong_scaling", extra_strong_scaling), ("long_context", extra_long_context),
                         ("multi_token", extra_multi_token), ("append", extra_append),
                         ("decompress", extra_decompress), ("prefill", extra_prefill),
                         ("paged_prefill", extra_paged_prefill)):
            if world > 1 and name in ("multi_token", "append", "decompress", "prefill",
                                      "paged_prefill"):
                continue  # one-GPU rows: measured at N = 1 only
            try:
                extras[name] = fn(ctx)
            except Exception as e:  # a secondary block must not take the headline down
                extras[name] = {"error": f"{type(e).__name__}: {e}"}
            torch.cuda.synchronize()
            if dist is not None:
                dist.barrier()

    # ---- reductions over ranks ----------------------------------------------------------
    vals = torch.tensor([ms, kernel_ms, e2e_s], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
    ms, kernel_ms, e2e_s = (float(x) for x in vals.cpu())
    status = K.workspace_status(ws) | K.workspace_status(step.workspace)
    if status:
        raise SystemExit(f"device status word is {status}: results invalid")

    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except Exception:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        alg = w.algorithmic_bytes()
        # the call is ONE launch of paged_decode_kernel (rotation, streaming and merge): its
        # average duration over the timed region is the step time; the streaming phase alone
        # (the same kernel launched without the two other phases) is reported next to it
        call_ms = ms / args.steps
        achieved = alg / (call_ms * 1e-3) / 1e9
        stream_gbs = alg / (kernel_ms * 1e-3) / 1e9
        tokens = NUM_SEQS * world
        line = {
            "metric": METRIC, "value": tokens * args.steps / (ms * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp16 mma operands, fp32 accumulate, bf16 in/out",
            "data": "synthetic", "config": workload_config(world),
            "hbm_tb_s_per_gpu_whole_call": alg / (ms / args.steps * 1e-3) / 1e12,
            "two_stage_scoring": {
                "ms_per_step": qjl_ms, "tokens_per_s_per_gpu": NUM_SEQS / (qjl_ms * 1e-3),
                "what": "fq_split_k_paged_decode_qjl on the same inputs (156 B per token and KV "
                        "head instead of 136)"},
            "clocks": sampler.summary(),
            "gpu_launches": launches_per_step * args.steps,
            "launches_per_step": launches_per_step,
            "e2e": {"value": tokens * e2e_steps / e2e_s, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "gpu_launches": e2e_launches, "form": e2e_form,
                    "us_per_step_by_form": {f: t / e2e_steps * 1e6
                                            for f, (t, _) in e2e_forms.items()},
                    "what": "fq_decode_step_host_packed, one C-ABI call per step: the step's "
                            "q / new K,V token / slot / block table / lengths in one pinned "
                            "host block -> device, compress-on-append (one-stage, as the "
                            "reference's _compress_and_store), decode, output -> "
                            "pinned host, synchronise (the packed one-copy form replays the "
                            "four operations as one CUDA graph); the packed cache itself "
                            "stays in HBM"},
            "roofline": {"bound": "hbm",
                         "kernel": "paged_decode_fast_kernel<KPRMT, FUSE=1, two-term weights> "
                                   "(single cooperative launch per call)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback",
                         "algorithmic_bytes": alg, "kernel_ms": call_ms,
                         "frac_of_nominal_8TBs": achieved / 8000.0,
                         "traffic": args.traffic if args.traffic is not None else _recorded_traffic(),
                         "streaming_phase_alone": {
                             "kernel": "paged_decode_fast_kernel<KPRMT, FUSE=0, two-term weights>",
                             "kernel_ms": kernel_ms, "achieved": stream_gbs,
                             "frac": stream_gbs / peak}},
        }
        line.update(extras)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(w, caches[0].cpu(), ck.cpu(), cv.cpu(), rot.cpu(),
                                                budget_s=20.0)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# --------------------------------------------------------------------------------------
# secondary blocks of the line
# --------------------------------------------------------------------------------------
def _event_loop(fn, steps, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / steps


def _max_over_ranks(ctx, value):
    if ctx["dist"] is None:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=ctx["dev"])
    ctx["dist"].all_reduce(t, op=ctx["dist"].ReduceOp.MAX)
    return float(t.item())


def _graph_of(fn, side):
    with torch.cuda.stream(side):
        fn()
    side.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        fn()
    return g


def extra_strong_scaling(ctx):
    """configs[1] with its 32 sequences split over the ranks (32 / N each): the same total
    work at every N, next to the weak-scaling headline."""
    from flashquant_b200 import distributed as D, kernels as K
    w, world, rank, dev = ctx["w"], ctx["world"], ctx["rank"], ctx["dev"]
    mine = D.shard_sequences(NUM_SEQS, rank, world)
    n = mine.stop - mine.start
    q = w.q[mine].contiguous().to(dev)
    bt, sl = w.block_table[mine].contiguous().to(dev), w.seq_lens[mine].contiguous().to(dev)
    out = torch.empty_like(q)
    side = torch.cuda.Stream()
    graphs = [_graph_of(lambda c=c: K.split_k_paged_decode(
        q, c, bt, sl, ctx["ck"], ctx["cv"], ctx["rot"], HKV, D_, BS, out=out, num_splits=SPLITS,
        workspace=ctx["ws"]), side) for c in ctx["caches"]]
    i = [0]

    def step():
        graphs[i[0] % CACHE_COPIES].replay()
        i[0] += 1
    ms = _max_over_ranks(ctx, _event_loop(step, 300, 10))
    return {"ms_per_step": ms, "tokens_per_s": NUM_SEQS / (ms * 1e-3),
            "what": f"configs[1], {NUM_SEQS} sequences in total, {n} per rank, no collective; "
                    "time = max over ranks", "scaling": "strong"}


def extra_long_context(ctx):
    """configs[4]: 64 q / 8 kv heads, batch 8, seed-4 lengths in [32768, 131072].
    (a) KV heads sharded over the ranks (8 / N each), no communication;
    (b) one sequence of 131072 tokens split over the ranks by token range: partial rows, ONE
        all-gather of (H_q, D+4) fp32 per rank, merge on every rank."""
    from flashquant_b200 import distributed as D, kernels as K, workloads as W
    world, rank, dev, dist = ctx["world"], ctx["rank"], ctx["dev"], ctx["dist"]
    rot, bk, ck, bv, cv = ctx["rot"], ctx["bk"], ctx["ck"], ctx["bv"], ctx["cv"]
    hq, hkv, d, bs = 64, 8, 128, 16
    peak = float(ctx["peaks"].get("hbm_gbs", 6650.0))
    res = {}
    # ---- (a) head-sharded ---------------------------------------------------------------------
    if hkv % world == 0:
        lens = W.ragged_lengths()
        kv, qh = D.shard_kv_heads(hkv, hq, rank, world)
        h_loc = kv.stop - kv.start
        w = W.decode_workload(seq_lens=lens.tolist(), num_q_heads=hq, num_kv_heads=h_loc, cfg=4)
        cache = torch.zeros(w.num_blocks, bs, h_loc * (d + 8), dtype=torch.uint8, device=dev)
        at = 0
        for i, n in enumerate(lens.tolist()):
            k, v = W.make_kv(n, hkv, d, cfg=400 + i)
            K.tq4_compress_append(k[:, kv].contiguous().to(dev), v[:, kv].contiguous().to(dev), cache,
                                  w.slot_mapping[at:at + n].to(dev), rot, bk, bv)
            at += n
        q = w.q[:, qh].contiguous().to(dev)
        bt, sl = w.block_table.to(dev), w.seq_lens.to(dev)
        out = torch.empty_like(q)
        ws = K.decode_workspace(dev, 8, qh.stop - qh.start, h_loc, d, 8)
        g = _graph_of(lambda: K.split_k_paged_decode(q, cache, bt, sl, ck, cv, rot, h_loc, d, bs,
                                                     out=out, num_splits=8, workspace=ws),
                      torch.cuda.Stream())
        ms = _max_over_ranks(ctx, _event_loop(g.replay, 100, 5))
        alg = int(lens.sum()) * 136 * h_loc + 2 * q.numel() * 2
        res["head_sharded"] = {
            "ms_per_step": ms, "tokens_per_s": 8 / (ms * 1e-3), "kv_heads_per_gpu": h_loc,
            "algorithmic_bytes_per_gpu": alg, "hbm_gb_s_per_gpu": alg / (ms * 1e-3) / 1e9,
            "frac_of_peak_per_gpu": alg / (ms * 1e-3) / 1e9 / peak,
            "l2": f"{cache.numel() / 1e6:.0f} MB of cache per GPU (> 126 MB L2 only above 1 head "
                  "per GPU)" if h_loc == 1 else f"{cache.numel() / 1e6:.0f} MB of cache per GPU",
            "status": K.workspace_status(ws)}
        del cache
    # ---- (a') the same batch with whole sequences per rank (8 / N each, all 8 KV heads): the
    # other no-communication split the decode offers; the ranks' loads differ with the lengths
    if world > 1 and 8 % world == 0:
        lens = W.ragged_lengths()
        mine = D.shard_sequences(8, rank, world)
        my_lens = lens[mine]
        w = W.decode_workload(seq_lens=my_lens.tolist(), num_q_heads=hq, num_kv_heads=hkv, cfg=4)
        cache = torch.zeros(w.num_blocks, bs, hkv * (d + 8), dtype=torch.uint8, device=dev)
        at = 0
        for i, n in enumerate(my_lens.tolist()):
            k, v = W.make_kv(n, hkv, d, cfg=400 + mine.start + i)
            K.tq4_compress_append(k.to(dev), v.to(dev), cache, w.slot_mapping[at:at + n].to(dev),
                                  rot, bk, bv)
            at += n
        q = w.q.to(dev)
        bt, sl = w.block_table.to(dev), w.seq_lens.to(dev)
        out = torch.empty_like(q)
        ws = K.decode_workspace(dev, len(my_lens), hq, hkv, d, 8)
        g = _graph_of(lambda: K.split_k_paged_decode(q, cache, bt, sl, ck, cv, rot, hkv, d, bs,
                                                     out=out, num_splits=8, workspace=ws),
                      torch.cuda.Stream())
        mine_ms = _event_loop(g.replay, 100, 5)
        ms = _max_over_ranks(ctx, mine_ms)
        alg = int(my_lens.sum()) * 136 * hkv + 2 * q.numel() * 2
        res["sequence_sharded"] = {
            "ms_per_step": ms, "tokens_per_s": 8 / (ms * 1e-3), "sequences_per_gpu": len(my_lens),
            "rank0_ms": mine_ms, "rank0_algorithmic_bytes": alg,
            "rank0_frac_of_peak": alg / (mine_ms * 1e-3) / 1e9 / peak,
            "what": "configs[4]'s batch with whole sequences per rank instead of KV heads (no "
                    "collective either); step time = slowest rank, which holds the longest "
                    "sequences",
            "status": K.workspace_status(ws)}
        del cache
    # ---- (b) one long sequence, token ranges per rank ---------------------------------------------
    L = 131072
    w1 = W.decode_workload(seq_lens=[L], num_q_heads=hq, num_kv_heads=hkv, cfg=41)
    lo, hi = D.token_range(L, bs, rank, world)
    k, v = W.make_kv(L, hkv, d, cfg=441)
    # every rank writes only the pages it owns (the block table is global)
    cache = torch.zeros(w1.num_blocks, bs, hkv * (d + 8), dtype=torch.uint8, device=dev)
    K.tq4_compress_append(k[lo:hi].to(dev), v[lo:hi].to(dev), cache, w1.slot_mapping[lo:hi].to(dev),
                          rot, bk, bv)
    bt_l, len_l = D.local_view(w1.block_table, w1.seq_lens, bs, rank, world)
    q = w1.q.to(dev)
    bt_l, len_l = bt_l.to(dev), len_l.to(dev)
    ws = K.decode_workspace(dev, 1, hq, hkv, d, 8)
    part = torch.empty(1, hq, d + 4, dtype=torch.float32, device=dev)
    gathered = torch.empty(world, 1, hq, d + 4, dtype=torch.float32, device=dev)
    out = torch.empty_like(q)

    def partial():
        K.paged_decode_partials(q, cache, bt_l, len_l, ck, cv, rot, hkv, d, bs, num_splits=8,
                                partials=part, workspace=ws)

    def gather():
        if dist is not None:
            dist.all_gather_into_tensor(gathered, part)
        else:
            gathered.copy_(part.unsqueeze(0))

    def merge():
        K.split_k_merge(gathered, rot, q.dtype, out=out)

    def whole():
        partial(); gather(); merge()
    ms_whole = _max_over_ranks(ctx, _event_loop(whole, 100, 5))
    ms_part = _max_over_ranks(ctx, _event_loop(partial, 100, 5))
    ms_gather = _max_over_ranks(ctx, _event_loop(gather, 200, 10))
    ms_merge = _max_over_ranks(ctx, _event_loop(merge, 100, 5))
    whole()
    # correctness evidence that travels with the timing: against a second merge of the same
    # gathered rows on the CPU in fp64 (rounded the way the kernel rounds), on every rank
    g64 = gathered.double().cpu()
    m = g64[..., d].amax(dim=0, keepdim=True)
    wgt = torch.where(torch.isinf(g64[..., d]), torch.zeros_like(m), torch.exp2(g64[..., d] - m))
    num = (wgt.unsqueeze(-1) * g64[..., :d]).sum(0)
    den = (wgt * g64[..., d + 1]).sum(0).unsqueeze(-1)
    ref = ((num / den).float().to(q.dtype).float() @ rot.float().cpu()).to(q.dtype)
    err = _max_over_ranks(ctx, (out.float().cpu() - ref.float()).abs().max().item())
    alg = (hi - lo) * hkv * 136
    res["cross_gpu_split_k"] = {
        "tokens": L, "tokens_per_gpu": hi - lo, "ms_whole": ms_whole, "ms_partials": ms_part,
        "ms_all_gather": ms_gather, "ms_merge": ms_merge,
        "all_gather_bytes_per_rank": part.numel() * 4, "ranks_in_all_gather": world,
        "hbm_gb_s_per_gpu_partials": alg / (ms_part * 1e-3) / 1e9,
        "max_abs_err_vs_fp64_merge": err,
        "what": "fq_paged_decode_partials over the rank's token range -> one "
                "all_gather_into_tensor of (H_q, D+4) fp32 -> fq_split_k_merge on every rank; "
                "three launches + one collective per call, timed without graphs"}
    return res


def extra_multi_token(ctx):
    """Decode steps of n_q tokens per sequence at configs[1] (fq_split_k_paged_decode_multi)."""
    import flashquant_b200 as fq
    w, dev = ctx["w"], ctx["dev"]
    bt, sl = w.block_table.to(dev), w.seq_lens.to(dev)
    res = {}
    for n_q in (1, 2, 4):
        q = torch.randn(NUM_SEQS, n_q, HQ, D_, generator=torch.Generator().manual_seed(n_q)).to(
            torch.bfloat16).to(dev)
        i = [0]

        def step():
            fq.split_k_paged_decode_multi(q, ctx["caches"][i[0] % CACHE_COPIES], bt, sl, ctx["ck"],
                                          ctx["cv"], ctx["rot"], HKV, D_, BS, num_splits=SPLITS)
            i[0] += 1
        ms = _event_loop(step, 150, 5)
        res[f"n_q_{n_q}"] = {"us_per_step": ms * 1e3, "tokens_per_s": NUM_SEQS * n_q / (ms * 1e-3)}
    res["what"] = ("the last n_q tokens of every sequence in one call; with 4 query heads per KV "
                   "head two tokens share a pass over the pages; Python call, no graph")
    return res


def extra_append(ctx):
    """configs[2]: compress-on-append of 8192 tokens x 8 heads into a 65536-slot cache."""
    from flashquant_b200 import kernels as K, workloads as W
    dev = ctx["dev"]
    w = W.append_workload()
    key, val, slots = w.key.to(dev), w.value.to(dev), w.slot_mapping.to(dev)
    nb = w.num_slots // w.block_size
    cache = torch.zeros(nb, BS, HKV * (D_ + 8), dtype=torch.uint8, device=dev)
    plane = torch.zeros(nb, BS, HKV * (D_ // 8 + 4), dtype=torch.uint8, device=dev)
    ms_qjl = _event_loop(lambda: K.tq4_compress_append_qjl(key, val, cache, plane, slots, ctx["rot"],
                                                           ctx["bk"], ctx["ck"], ctx["bv"], ctx["S"]), 100)
    ms_mse = _event_loop(lambda: K.tq4_compress_append(key, val, cache, slots, ctx["rot"], ctx["bk"],
                                                       ctx["bv"]), 100)
    peak = float(ctx["peaks"].get("hbm_gbs", 6650.0))
    alg = w.algorithmic_bytes(with_qjl=True)
    return {"us_per_call_two_stage": ms_qjl * 1e3, "us_per_call_one_stage": ms_mse * 1e3,
            "tokens_per_s": 8192 / (ms_qjl * 1e-3), "algorithmic_bytes": alg,
            "hbm_gb_s": alg / (ms_qjl * 1e-3) / 1e9, "frac_of_hbm_peak": alg / (ms_qjl * 1e-3) / 1e9 / peak,
            "note": "bound by the split-fp16 rotations on mma.sync, not by HBM"}


def extra_decompress(ctx):
    """Decompress: 65536 x 8 vectors of head_dim 128, rotated space (bf16 out) and original
    space (fq_tq4_decompress_original)."""
    import flashquant_b200 as fq
    dev = ctx["dev"]
    n, h = 65536, 8
    g = torch.Generator().manual_seed(77)
    packed = torch.randint(0, 256, (n, h, D_ // 2), dtype=torch.uint8, generator=g).to(dev)
    norms = (torch.rand(n, h, 1, generator=g) + 0.5).to(dev)
    out = torch.empty(n, h, D_, dtype=torch.bfloat16, device=dev)
    ms = _event_loop(lambda: fq.tq4_decompress(packed, norms, ctx["cv"], dtype=torch.bfloat16, out=out), 100)
    ms_orig = _event_loop(lambda: fq.tq4_decompress_original(packed, norms, ctx["cv"], ctx["rot"],
                                                            dtype=torch.bfloat16), 30)
    peak = float(ctx["peaks"].get("hbm_gbs", 6650.0))
    alg = n * h * (D_ // 2 + 4 + 2 * D_)
    return {"vectors": n * h, "us_rotated_space": ms * 1e3, "us_original_space": ms_orig * 1e3,
            "algorithmic_bytes": alg, "hbm_gb_s": alg / (ms * 1e-3) / 1e9,
            "frac_of_hbm_peak": alg / (ms * 1e-3) / 1e9 / peak,
            "l2": "168 MB of codes, norms and output per call (> 126 MB L2)"}


def extra_prefill(ctx):
    """configs[3]: fused causal TQ4 prefill, batch 4 x 8192, 32 q / 8 kv heads."""
    from flashquant_b200 import kernels as K, workloads as W
    dev = ctx["dev"]
    b, n = 4, 8192
    k, v = W.make_kv(b * n, HKV, D_, cfg=3)
    kp, kn = K.tq4_compress(k.to(dev).reshape(b, n, HKV, D_).transpose(1, 2).reshape(-1, 1, D_), ctx["rot"], ctx["bk"])
    vp, vn = K.tq4_compress(v.to(dev).reshape(b, n, HKV, D_).transpose(1, 2).reshape(-1, 1, D_), ctx["rot"], ctx["bv"])
    kp, vp = kp.reshape(b, HKV, n, D_ // 2), vp.reshape(b, HKV, n, D_ // 2)
    kn, vn = kn.reshape(b, HKV, n, 1), vn.reshape(b, HKV, n, 1)
    q = torch.randn(b, HQ, n, D_, generator=torch.Generator().manual_seed(3003)).to(torch.bfloat16).to(dev)
    ms = _event_loop(lambda: K.fused_tq_attention(q, kp, kn, vp, vn, ctx["ck"], ctx["cv"], ctx["rot"],
                                                  is_causal=True), 5, 2)
    flops = 4.0 * b * HQ * n * n * D_ / 2
    peak = float(ctx["peaks"].get("bf16_tflops_sustained", 1400.0))
    return {"ms_per_call": ms, "tflops_causal_half": flops / (ms * 1e-3) / 1e12,
            "frac_of_sustained_tensor_peak": flops / (ms * 1e-3) / 1e12 / peak}


def extra_paged_prefill(ctx):
    """Prefill over the PAGED cache (fq_paged_tq4_prefill): the configs[3] shape read through a
    block table (4 whole prompts of 8192 tokens), and a chunked step (8 sequences, chunk 512
    after 4096 keys of context); the cache is filled by the compress-on-append."""
    from flashquant_b200 import kernels as K, workloads as W
    dev = ctx["dev"]
    peak = float(ctx["peaks"].get("bf16_tflops_sustained", 1400.0))
    out = {}
    for name, lens, chunks in (("whole_prompts_4x8192", [8192] * 4, [8192] * 4),
                               ("chunk_512_after_4096_x8", [4608] * 8, [512] * 8)):
        w = W.decode_workload(seq_lens=lens, num_q_heads=HQ, num_kv_heads=HKV, cfg=7)
        k, v = W.make_kv(w.total_tokens, HKV, D_, cfg=7)
        cache = torch.zeros(w.num_blocks, BS, HKV * (D_ + 8), dtype=torch.uint8, device=dev)
        K.tq4_compress_append(k.to(dev), v.to(dev), cache, w.slot_mapping.to(dev), ctx["rot"],
                              ctx["bk"], ctx["bv"])
        cu = torch.zeros(len(chunks) + 1, dtype=torch.int32)
        cu[1:] = torch.cumsum(torch.tensor(chunks), 0)
        q = torch.randn(int(cu[-1]), HQ, D_, generator=torch.Generator().manual_seed(3007)).to(
            torch.bfloat16).to(dev)
        bt, sl, cu_d = w.block_table.to(dev), w.seq_lens.to(dev), cu.to(dev)
        ws = torch.zeros(K.N.load().fq_paged_tq4_prefill_workspace_bytes(q.shape[0], HQ, D_),
                         dtype=torch.uint8, device=dev)
        o = torch.empty_like(q)
        ms = _event_loop(lambda: K.paged_tq4_prefill(q, cache, bt, sl, cu_d, max(chunks), ctx["ck"],
                                                     ctx["cv"], ctx["rot"], HKV, D_, BS, out=o,
                                                     workspace=ws), 5, 2)
        # visible (query, key) pairs: chunk rows see the context and the causal half of the chunk
        pairs = sum(c * (l - c) + c * (c + 1) / 2 for l, c in zip(lens, chunks))
        flops = 4.0 * HQ * pairs * D_
        out[name] = {"ms_per_call": ms, "tflops": flops / (ms * 1e-3) / 1e12,
                     "frac_of_sustained_tensor_peak": flops / (ms * 1e-3) / 1e12 / peak,
                     "status": K.workspace_status(ws)}
    return out


# --------------------------------------------------------------------------------------
# CPU legs: the oracle port of the reference's pure-PyTorch path
# --------------------------------------------------------------------------------------
def cpu_decode_sample(w, cache, ck, cv, rot, n_seq):
    from oracle import tq_oracle as O
    return O.split_k_paged_decode(w.q[:n_seq], cache, w.block_table[:n_seq], w.seq_lens[:n_seq],
                                  ck, cv, rot, HKV, D, BS)


def cpu_baseline(w, cache, ck, cv, rot, budget_s):
    torch.set_num_threads(os.cpu_count() or 1)
    ref_pd = _reference_package()
    if ref_pd is not None:
        # the reference's own token loop: a few seconds per sequence, so a sample of them
        t = time.perf_counter()
        n = 0
        while n < NUM_SEQS and time.perf_counter() - t < budget_s:
            ref_pd.split_k_paged_decode(w.q[n:n + 1], cache, w.block_table[n:n + 1],
                                        w.seq_lens[n:n + 1], ck, cv, rot, HKV, D, BS)
            n += 1
        dt = time.perf_counter() - t
        return {"value": n / dt, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "reference",
                "sample": f"{n} of the {NUM_SEQS} sequences (context {CONTEXT}) through the "
                          f"reference's own split_k_paged_decode CPU branch, {dt:.1f} s"}
    t = time.perf_counter()
    cpu_decode_sample(w, cache, ck, cv, rot, 1)
    one = time.perf_counter() - t
    n_seq = int(max(1, min(NUM_SEQS, budget_s / max(one, 1e-3))))
    t = time.perf_counter()
    cpu_decode_sample(w, cache, ck, cv, rot, n_seq)
    dt = time.perf_counter() - t
    return {"value": n_seq / dt, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n_seq} of the {NUM_SEQS} sequences (context {CONTEXT}), one pass of the "
                      f"vectorised oracle restatement of the reference's CPU decode, {dt:.2f} s"}


def _reference_package():
    """The reference's own package, if oracle/make_ref.py has placed it under oracle/_ref/."""
    ref_root = os.path.join(ROOT, "oracle", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "flashquant")):
        return None
    if ref_root not in sys.path:
        sys.path.insert(0, ref_root)
    try:
        from flashquant.kernels import paged_decode as ref_pd  # noqa: WPS433
        return ref_pd
    except Exception:
        return None


def run_reference(args):
    """The reference's CPU implementation of the path on this host's cores, on a bounded sample
    of the same workload: its own ``split_k_paged_decode`` (a Python loop over tokens and heads,
    src/flashquant/kernels/paged_decode.py:112-128 + cpu_reference.py:230-368) when
    oracle/_ref holds the package, else the vectorised oracle restatement."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from flashquant_b200 import workloads as W
    from flashquant_b200.quantizer import TurboQuantMSE, TurboQuantProd
    from oracle import tq_oracle as O

    torch.set_num_threads(os.cpu_count() or 1)
    q3, q4 = TurboQuantProd(D, 4, seed=0), TurboQuantMSE(D, 4, seed=0)
    rot = q4.rotation
    bk, ck = q3.mse_quantizer.boundaries, q3.mse_quantizer.centroids
    bv, cv = q4.boundaries, q4.centroids
    ref_pd = _reference_package()
    # one sequence of the 32 per step for the reference's token loop (about 4 s), two for the
    # vectorised port
    n_seq = 1 if ref_pd is not None else 2
    w = W.decode_workload(n_seq, CONTEXT, HQ, HKV, D, BS, cfg=1)
    k, v = W.make_kv(w.total_tokens, HKV, D, cfg=1)
    cache = torch.zeros(w.num_blocks, BS, HKV * (D + 8), dtype=torch.uint8)
    O.compress_and_store(k, v, cache, w.slot_mapping, rot, bk, bv)

    def step():
        if ref_pd is not None:
            return ref_pd.split_k_paged_decode(w.q, cache, w.block_table, w.seq_lens, ck, cv, rot,
                                               HKV, D, BS)
        return cpu_decode_sample(w, cache, ck, cv, rot, n_seq)

    for _ in range(1 if ref_pd is not None else max(1, min(args.warmup, 3))):
        step()
    t = time.perf_counter()
    done = 0
    for _ in range(args.steps):
        step()
        done += 1
        if time.perf_counter() - t > 100.0:  # keep the whole run within a few minutes
            break
    dt = time.perf_counter() - t
    value = n_seq * done / dt
    kind = "reference" if ref_pd is not None else "port"
    sample = (f"{n_seq} sequence(s) x context {CONTEXT} per step (of the 32 in the workload), "
              f"{done} steps timed, " +
              ("the reference's own split_k_paged_decode CPU branch (Python loop per token and "
               "KV head)" if ref_pd is not None else "vectorised oracle restatement"))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": done, "warmup": args.warmup, "ms_per_step": dt / done * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(args.gpus),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(),
                         "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# secondary workloads (one GPU): the other rows of the hot path, for their own profiles
# --------------------------------------------------------------------------------------
def _time_loop(fn, steps, warmup):
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        fn()
    t1.record()
    torch.cuda.synchronize()
    return t0.elapsed_time(t1) / steps


def run_prefill(args):
    """configs[3]: fused causal TQ4 prefill, batch 4 x 8192 tokens, 32 q / 8 kv heads."""
    import flashquant_b200 as fq
    from flashquant_b200 import kernels as K, workloads as W

    dev = torch.device("cuda", 0)
    b, n = args.prefill_batch, args.prefill_seq
    q3, q4 = fq.TurboQuantProd(D, 4, seed=0), fq.TurboQuantMSE(D, 4, seed=0)
    rot = q4.rotation.to(dev)
    bk, ck = q3.mse_quantizer.boundaries.to(dev), q3.mse_quantizer.centroids.to(dev)
    bv, cv = q4.boundaries.to(dev), q4.centroids.to(dev)
    k, v = W.make_kv(b * n, HKV, D, cfg=3)
    # (tokens, H, D) -> (B, H, N, D), compressed with the CUDA kernel
    kp, kn = K.tq4_compress(k.to(dev).reshape(b, n, HKV, D).transpose(1, 2).reshape(-1, 1, D), rot, bk)
    vp, vn = K.tq4_compress(v.to(dev).reshape(b, n, HKV, D).transpose(1, 2).reshape(-1, 1, D), rot, bv)
    kp, vp = kp.reshape(b, HKV, n, D // 2), vp.reshape(b, HKV, n, D // 2)
    kn, vn = kn.reshape(b, HKV, n, 1), vn.reshape(b, HKV, n, 1)
    q = torch.randn(b, HQ, n, D, generator=torch.Generator().manual_seed(3003)).to(torch.bfloat16).to(dev)
    ms = _time_loop(lambda: K.fused_tq_attention(q, kp, kn, vp, vn, ck, cv, rot, is_causal=True),
                    args.steps, args.warmup)
    flops = 4.0 * b * HQ * n * n * D / 2
    peaks = _peaks()
    tf = flops / (ms * 1e-3) / 1e12
    peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
    print(json.dumps({
        "metric": "tq4_fused_prefill_tflops", "value": tf, "unit": "TFLOP/s (causal half counted)",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
        "higher_is_better": True, "dtype": "fp16 tcgen05 operands, fp32 accumulate, bf16 in/out",
        "data": "synthetic",
        "config": {"workload": f"configs[3]: fused causal TQ4 prefill, batch {b}, seq {n}, "
                               "32 q / 8 kv heads, head_dim 128; the call includes both rotations"},
        "roofline": {"bound": "tensor", "achieved": tf, "peak": peak, "unit": "TFLOP/s",
                     "frac": tf / peak, "traffic": None,
                     "peak_source": "measured sustained (MEASURED_PEAKS.json)" if peaks else "fallback"},
    }), flush=True)


def run_append(args):
    """configs[2]: compress-on-append, 8192 bf16 tokens x 8 heads into a 65536-slot cache."""
    import flashquant_b200 as fq
    from flashquant_b200 import kernels as K, workloads as W

    dev = torch.device("cuda", 0)
    q3, q4 = fq.TurboQuantProd(D, 4, seed=0), fq.TurboQuantMSE(D, 4, seed=0)
    rot, S = q4.rotation.to(dev), q3.qjl_matrix.to(dev)
    bk, ck = q3.mse_quantizer.boundaries.to(dev), q3.mse_quantizer.centroids.to(dev)
    bv = q4.boundaries.to(dev)
    w = W.append_workload()
    key, val, slots = w.key.to(dev), w.value.to(dev), w.slot_mapping.to(dev)
    nb = w.num_slots // w.block_size
    cache = torch.zeros(nb, BS, HKV * (D + 8), dtype=torch.uint8, device=dev)
    plane = torch.zeros(nb, BS, HKV * (D // 8 + 4), dtype=torch.uint8, device=dev)
    ms_qjl = _time_loop(lambda: K.tq4_compress_append_qjl(key, val, cache, plane, slots, rot, bk, ck,
                                                          bv, S), args.steps, args.warmup)
    ms_mse = _time_loop(lambda: K.tq4_compress_append(key, val, cache, slots, rot, bk, bv),
                        args.steps, args.warmup)
    peaks = _peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    alg = w.algorithmic_bytes(with_qjl=True)
    gbs = alg / (ms_qjl * 1e-3) / 1e9
    print(json.dumps({
        "metric": "tq4_compress_append_tokens_per_s", "value": 8192 / (ms_qjl * 1e-3),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_qjl, "ms_per_step_without_qjl": ms_mse, "higher_is_better": True,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "configs[2]: 8192 bf16 tokens x 8 kv heads, K two-stage (3-bit + "
                               "QJL signs + gamma), V 4-bit, seed-3 slot mapping into 65536 slots"},
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s",
                     "frac": gbs / peak, "algorithmic_bytes": alg, "traffic": None,
                     "note": "the rotations (4 x 65536 x 128^2 multiply-adds as split-fp16 tensor-"
                             "core products) and the element-wise work around them are the "
                             "binding resource, not HBM",
                     "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback"},
    }), flush=True)


def run_cache(args):
    """The compressed cache behind the DynamicCache interface, one Llama-3-8B-shaped layer:
    a prompt update (batch 4 x 4096 tokens x 8 kv heads, bf16) in fused mode, then single-token
    decode updates with the de-quantised read-back, and the fused attention of one decode query
    over the buffers in place."""
    import time

    import flashquant_b200 as fq
    from oracle import tq_oracle as O

    class Layer:
        def __init__(self):
            self.keys = self.values = None
            self.is_initialized = True

    class Cache:
        def __init__(self):
            self.layers = []
            self.layer_class_to_replicate = Layer

        def update(self, k, v, layer_idx, cache_kwargs=None):
            return k, v

        def get_seq_length(self, layer_idx=0):
            return 0

    dev = torch.device("cuda", 0)
    b, n = 4, 4096
    g = torch.Generator().manual_seed(5005)
    k = torch.randn(b, HKV, n, D, generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn(b, HKV, n, D, generator=g).to(torch.bfloat16).to(dev)
    k1 = torch.randn(b, HKV, 1, D, generator=g).to(torch.bfloat16).to(dev)
    v1 = torch.randn(b, HKV, 1, D, generator=g).to(torch.bfloat16).to(dev)
    q1 = torch.randn(b, HQ, 1, D, generator=g).to(torch.bfloat16).to(dev)
    cache = Cache()
    w = fq.CompressedDynamicCache(cache, head_dim=D, bits=4, max_seq_len=n + 4096)

    def reset():
        for layer in w._compressed_keys + w._compressed_values:
            if layer is not None:
                layer.buffer.reset()

    w.fused_mode = True

    def prompt_update():
        reset()
        cache.update(k, v, 0)

    ms_prompt = _time_loop(prompt_update, args.steps, args.warmup)
    steps = min(args.steps, 2000)
    ms_attend = _time_loop(lambda: w.fused_attention(q1, 0, is_causal=True), steps, args.warmup)
    w.fused_mode = False
    prompt_update()  # the de-quantised running tensors start from the prompt
    ms_step = _time_loop(lambda: cache.update(k1, v1, 0), steps, args.warmup)
    w.restore()

    # CPU: the restatement of the reference's cache on a bounded sample of the prompt update
    cpu = None
    if not args.no_cpu_baseline:
        c4, b4 = O.lloyd_max_codebook(D, 4)
        orc = O.CompressedCacheOracle(O.haar_rotation(D, 42), O.haar_rotation(D, 43), c4, b4)
        ns = 1024
        ks, vs = k[:1, :, :ns].cpu(), v[:1, :, :ns].cpu()
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0:
            orc.layers.clear()
            orc.update(ks, vs, 0)
            reps += 1
        cpu = {"value": reps * ns / (time.perf_counter() - t0), "unit": "tokens/s",
               "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"prompt update of 1 x {ns} tokens x {HKV} heads (compress + de-quantise "
                         "of K and V, the reference's non-fused update), repeated for 10 s"}
    peaks = _peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    alg = 2 * b * HKV * n * (D * 2 + D // 2 + 4)
    gbs = alg / (ms_prompt * 1e-3) / 1e9
    print(json.dumps({
        "metric": "compressed_cache_update_tokens_per_s", "value": b * n / (ms_prompt * 1e-3),
        "unit": "tokens/s (one layer)", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_prompt, "higher_is_better": True, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"DynamicCache-style update, one layer: prompt of {b} x {n} bf16 "
                               f"tokens x {HKV} kv heads x {D} compressed into pre-allocated "
                               "buffers (fused mode); inputs 33.5 MB per tensor (K, V), larger than L2 together "
                               "with the outputs"},
        "decode_update_us": ms_step * 1e3, "decode_fused_attention_us": ms_attend * 1e3,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s",
                     "frac": gbs / peak, "algorithmic_bytes": alg, "traffic": None,
                     "note": "two launches of the compress kernel (K, V); the split-fp16 rotation "
                             "on mma.sync is the binding resource, as for compress-on-append",
                     "peak_source": "measured (MEASURED_PEAKS.json)" if peaks else "fallback"},
        "cpu_baseline": cpu,
    }), flush=True)


def _recorded_traffic():
    """DRAM bytes per decode launch from the last ncu capture, recorded next to its summary."""
    try:
        rec = json.load(open(os.path.join(ROOT, "profiles", "decode_traffic.json")))
        return float(rec["dram_bytes_per_launch"])
    except Exception:
        return None


def _peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        return {}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", choices=["decode", "prefill", "append", "cache"], default="decode",
                    help="decode is the headline; the others time further rows on one GPU")
    ap.add_argument("--prefill-batch", type=int, default=4)
    ap.add_argument("--prefill-seq", type=int, default=8192)
    ap.add_argument("--traffic", type=float, default=None,
                    help="DRAM bytes per launch of the decode kernel (dram read + write of one "
                         "ncu capture); default: the figure recorded in "
                         "profiles/decode_traffic.json, null if that file is missing")
    ap.add_argument("--e2e-steps", type=int, default=0,
                    help="host-buffer steps of the end-to-end figure (default: max(steps, 200))")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the secondary blocks of the line (append, prefill, decompress, "
                         "multi-token, long-context)")
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "prefill":
        run_prefill(args)
    elif args.workload == "append":
        run_append(args)
    elif args.workload == "cache":
        run_cache(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
