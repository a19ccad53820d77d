"""The decode entry point that allocates nothing, checked against the ordinary one.

Some users of this library cannot ask CUDA for memory when they decode: an inference server
that has already handed every free byte to its KV cache, or a plugin that must live inside
its host framework's memory pool.  ``fq_split_k_paged_decode_static`` serves them from a
16 MiB scratch array that is part of the library itself.  The test drives it through the
C ABI twice in a row (the array keeps the first call's contents) and expects the same
output as ``fq_split_k_paged_decode`` with a caller-owned workspace.  This file sorts last so
that a failure here cannot hide the result of any other test.
"""

import ctypes as C

import numpy as np
import pytest
import torch

from flashquant_b200 import _native as N
from flashquant_b200 import kernels as K
from flashquant_b200 import workloads as W
from oracle import tq_oracle as O
from parity import attention_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(consts, lens, cfg):
    w = W.decode_workload(seq_lens=lens, num_q_heads=32, num_kv_heads=8, cfg=cfg)
    k, v = W.make_kv(w.total_tokens, 8, 128, cfg)
    cache = torch.zeros(w.num_blocks, 16, 8 * 136, dtype=torch.uint8)
    O.compress_and_store(k, v, cache, w.slot_mapping, consts["rotation_128_0"],
                         consts["boundaries_128_3"], consts["boundaries_128_4"])
    return w, cache.to(DEV)


def _static_call(lib, w, cache, consts, num_splits):
    dev = torch.device(DEV)
    q, bt, sl = w.q.to(dev), w.block_table.to(dev), w.seq_lens.to(dev)
    ck = consts["centroids_128_3"].to(dev)
    cv = consts["centroids_128_4"].to(dev)
    rot = consts["rotation_128_0"].contiguous().to(dev)
    out = torch.full_like(q, float("nan"))
    rc = lib.fq_split_k_paged_decode_static(
        N.ptr(q), N.dtype_code(q.dtype), N.ptr(cache), N.ptr(bt), bt.stride(0), N.ptr(sl),
        N.ptr(ck), ck.numel(), N.ptr(cv), cv.numel(), N.ptr(rot), w.num_seqs, 32, 8, 128, 16,
        cache.shape[0], 1.0 / np.sqrt(128), N.ptr(out), num_splits, N.stream_ptr(dev))
    return rc, out


def test_static_scratch_decode_matches_workspace_decode_twice(consts):
    lib = N.load()
    assert lib.fq_split_k_paged_decode_static_max_bytes() == 16 << 20
    # two different batches back to back: the second call starts from the first one's leftovers
    for lens, cfg in (([700, 33, 0, 4096], 41), ([16, 1500, 257], 42)):
        w, cache = _inputs(consts, lens, cfg)
        rc, got = _static_call(lib, w, cache, consts, num_splits=4)
        assert rc == 0, lib.fq_last_error_string().decode()
        want = K.split_k_paged_decode(
            w.q.to(DEV), cache, w.block_table.to(DEV), w.seq_lens.to(DEV),
            consts["centroids_128_3"], consts["centroids_128_4"], consts["rotation_128_0"],
            8, 128, 16, num_splits=4)
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        # the same kernel on the same inputs: identical bits, and both within the decode's
        # tolerance of the reference
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
        ref32, ref = O.split_k_paged_decode_stages(
            w.q, cache.cpu(), w.block_table, w.seq_lens, consts["centroids_128_3"],
            consts["centroids_128_4"], consts["rotation_128_0"], 8, 128, 16)
        attention_close(got, ref, ref32, consts["rotation_128_0"])


def test_static_scratch_refuses_what_does_not_fit(consts):
    lib = N.load()
    # 2048 sequences x 64 splits of partial rows is far beyond 16 MiB; nothing may launch
    w = W.decode_workload(seq_lens=[16] * 2048, num_q_heads=32, num_kv_heads=8, cfg=43)
    cache = torch.zeros(w.num_blocks, 16, 8 * 136, dtype=torch.uint8, device=DEV)
    before = lib.fq_launch_count()
    rc, _ = _static_call(lib, w, cache, consts, num_splits=64)
    assert rc == -3 and b"16777216" in lib.fq_last_error_string()
    assert lib.fq_launch_count() == before


def test_static_scratch_three_launch_form_and_status_word(consts):
    """The static entry behaves like the ordinary one in its two other respects: it honours
    fq_paged_decode_set_single_launch(0) (three ordinary launches, same answer), and its device
    status word - the caller has no pointer to the array - is read through
    fq_split_k_paged_decode_static_status: a block index outside the cache is reported there,
    not followed."""
    lib = N.load()
    w, cache = _inputs(consts, [300, 17, 1000], 44)
    rc, one = _static_call(lib, w, cache, consts, num_splits=3)
    assert rc == 0
    K.set_single_launch(False)
    try:
        n0 = lib.fq_launch_count()
        rc, three = _static_call(lib, w, cache, consts, num_splits=3)
        assert rc == 0 and lib.fq_launch_count() - n0 == 3
    finally:
        K.set_single_launch(True)
    torch.cuda.synchronize()
    ref32, ref = O.split_k_paged_decode_stages(
        w.q, cache.cpu(), w.block_table, w.seq_lens, consts["centroids_128_3"],
        consts["centroids_128_4"], consts["rotation_128_0"], 8, 128, 16)
    attention_close(one, ref, ref32, consts["rotation_128_0"])
    attention_close(three, ref, ref32, consts["rotation_128_0"])
    st = C.c_uint32(99)
    assert lib.fq_split_k_paged_decode_static_status(C.byref(st), N.stream_ptr(torch.device(DEV))) == 0
    assert st.value == 0
    w.block_table[1, 0] = 10_000_000
    rc, _ = _static_call(lib, w, cache, consts, num_splits=3)
    assert rc == 0
    assert lib.fq_split_k_paged_decode_static_status(C.byref(st), N.stream_ptr(torch.device(DEV))) == 0
    assert st.value & 1            # FQ_DEV_BAD_BLOCK_INDEX
