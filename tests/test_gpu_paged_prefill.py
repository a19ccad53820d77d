"""GPU parity of the fused TQ4 attention over the PAGED cache for prefill chunks
(fq_paged_tq4_prefill) against the oracle's decompress-then-attend path.

Cases follow the reference's chunked-prefill situations: chunks of 1, 17 and 512 tokens,
contexts from 0 to 4096 keys before the chunk, ragged batches, GQA.
"""

import pytest
import torch

from flashquant_b200 import kernels as K
from flashquant_b200 import workloads as W
from oracle import tq_oracle as O
from parity import attention_close

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# Scaled fp16 centroid tables as in the decode kernels: the rows agree with the reference's
# un-rounded rows to 2^-10 of the entry.
PAGED_PREFILL_RTOL = 2.0 ** -10


def build(consts, seq_lens, chunks, hq=32, hkv=8, cfg=31, dtype=torch.bfloat16, block_size=16):
    """Paged cache holding seq_lens[b] keys of every sequence (oracle-compressed), and the last
    chunks[b] tokens of each as the query chunk."""
    d = 128
    w = W.decode_workload(seq_lens=seq_lens, num_q_heads=hq, num_kv_heads=hkv, head_dim=d,
                          block_size=block_size, cfg=cfg, dtype=dtype)
    rot = consts["rotation_128_0"]
    k, v = W.make_kv(w.total_tokens, hkv, d, cfg, dtype)
    cache = torch.zeros(w.num_blocks, block_size, hkv * (d + 8), dtype=torch.uint8)
    O.compress_and_store(k, v, cache, w.slot_mapping, rot, consts["boundaries_128_3"],
                         consts["boundaries_128_4"])
    cu = torch.zeros(len(chunks) + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(torch.tensor(chunks), 0)
    g = torch.Generator().manual_seed(1000 + cfg)
    q = torch.randn(int(cu[-1]), hq, d, generator=g).to(dtype)
    return w, cache, q, cu


def run_and_check(consts, w, cache, q, cu, chunks):
    rot, ck, cv = consts["rotation_128_0"], consts["centroids_128_3"], consts["centroids_128_4"]
    ws = torch.zeros(K.N.load().fq_paged_tq4_prefill_workspace_bytes(q.shape[0], q.shape[1], 128),
                     dtype=torch.uint8, device=DEV)
    out = K.paged_tq4_prefill(q.to(DEV), cache.to(DEV), w.block_table.to(DEV), w.seq_lens.to(DEV),
                              cu.to(DEV), max(chunks), ck, cv, rot, w.num_kv_heads, 128,
                              w.block_size, workspace=ws)
    assert K.workspace_status(ws) == 0
    ref32, ref = O.paged_prefill_varlen_stages(q, cache, w.block_table, w.seq_lens, cu, ck, cv, rot,
                                               w.num_kv_heads, 128, w.block_size)
    attention_close(out, ref, ref32, rot, rtol=PAGED_PREFILL_RTOL)
    return out


@pytest.mark.parametrize("seq_lens,chunks", [
    ([17], [17]),                          # whole prompt, no context, ragged tile
    ([512], [512]),                        # whole prompt, several query tiles
    ([1, 64, 65], [1, 64, 65]),            # ragged batch of whole prompts
    ([300, 1000, 4096 + 17], [1, 17, 17]),  # short chunks after long contexts
    ([4096 + 512, 777, 130], [512, 130, 1]),  # chunk 512 after 4096 keys; mixed
])
def test_chunks_vs_oracle(consts, seq_lens, chunks):
    w, cache, q, cu = build(consts, seq_lens, chunks)
    run_and_check(consts, w, cache, q, cu, chunks)


@pytest.mark.parametrize("seed", [201, 202, 203])
def test_random_ragged_chunks_vs_oracle(consts, seed):
    g = torch.Generator().manual_seed(seed)
    n = int(torch.randint(2, 7, (1,), generator=g))
    seq_lens = [int(torch.randint(1, 3001, (1,), generator=g)) for _ in range(n)]
    chunks = []
    for length in seq_lens:
        c = int(torch.randint(0, min(length, 600) + 1, (1,), generator=g))
        chunks.append(c)
    if sum(chunks) == 0:
        chunks[0] = 1
    w, cache, q, cu = build(consts, seq_lens, chunks, cfg=seed)
    run_and_check(consts, w, cache, q, cu, chunks)


def test_sequence_without_chunk_and_gqa_layouts(consts):
    """A sequence that contributes no query tokens, 64 q heads over 8 KV heads, fp16."""
    seq_lens, chunks = [200, 96, 1030], [40, 0, 129]
    w, cache, q, cu = build(consts, seq_lens, chunks, hq=64, hkv=8, cfg=33, dtype=torch.float16)
    run_and_check(consts, w, cache, q, cu, chunks)
    w, cache, q, cu = build(consts, [50, 260], [50, 4], hq=8, hkv=8, cfg=34, block_size=32)
    run_and_check(consts, w, cache, q, cu, [50, 4])


def test_chunk_equals_decode_for_single_tokens(consts):
    """One query token per sequence is the decode step: same rows as fq_split_k_paged_decode up
    to the two kernels' different operand precisions (both within the stated bounds)."""
    seq_lens = [33, 700, 16, 257]
    w, cache, q, cu = build(consts, seq_lens, [1, 1, 1, 1], cfg=35)
    out = run_and_check(consts, w, cache, q, cu, [1, 1, 1, 1])
    rot, ck, cv = consts["rotation_128_0"], consts["centroids_128_3"], consts["centroids_128_4"]
    dec = K.split_k_paged_decode(q.to(DEV), cache.to(DEV), w.block_table.to(DEV),
                                 w.seq_lens.to(DEV), ck, cv, rot, 8, 128, 16)
    assert (out.float() - dec.float()).abs().max() < 2e-2


def test_bad_page_index_is_reported_not_followed(consts):
    w, cache, q, cu = build(consts, [100], [100], cfg=36)
    rot, ck, cv = consts["rotation_128_0"], consts["centroids_128_3"], consts["centroids_128_4"]
    bt = w.block_table.clone()
    bt[0, 2] = w.num_blocks + 5
    ws = torch.zeros(K.N.load().fq_paged_tq4_prefill_workspace_bytes(100, 32, 128),
                     dtype=torch.uint8, device=DEV)
    K.paged_tq4_prefill(q.to(DEV), cache.to(DEV), bt.to(DEV), w.seq_lens.to(DEV), cu.to(DEV), 100,
                        ck, cv, rot, 8, 128, 16, workspace=ws)
    assert K.workspace_status(ws) & 1  # FQ_DEV_BAD_BLOCK_INDEX


def test_chunk_bounds_are_reported_not_followed(consts):
    """cu_seqlens_q that points past the query tokens, and a chunk longer than max_q_len: a
    status bit, no access outside the tensors, the other sequences unaffected."""
    seq_lens, chunks = [300, 200], [150, 100]
    w, cache, q, cu = build(consts, seq_lens, chunks, cfg=37)
    rot, ck, cv = consts["rotation_128_0"], consts["centroids_128_3"], consts["centroids_128_4"]
    ref32, ref = O.paged_prefill_varlen_stages(q, cache, w.block_table, w.seq_lens, cu, ck, cv, rot,
                                               8, 128, 16)
    need = K.N.load().fq_paged_tq4_prefill_workspace_bytes(q.shape[0], 32, 128)
    # (1) the second chunk claims 50 tokens more than there are
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    bad = cu.clone()
    bad[2] += 50
    out = torch.zeros_like(q, device=DEV)
    K.paged_tq4_prefill(q.to(DEV), cache.to(DEV), w.block_table.to(DEV), w.seq_lens.to(DEV),
                        bad.to(DEV), 150, ck, cv, rot, 8, 128, 16, out=out, workspace=ws)
    assert K.workspace_status(ws) & 4  # FQ_DEV_BAD_LENGTH
    attention_close(out[:150], ref[:150], ref32[:150], rot, rtol=PAGED_PREFILL_RTOL)
    assert (out[150:] == 0).all()
    # (2) max_q_len smaller than the longest chunk: its tail is not computed
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    out = torch.zeros_like(q, device=DEV)
    K.paged_tq4_prefill(q.to(DEV), cache.to(DEV), w.block_table.to(DEV), w.seq_lens.to(DEV),
                        cu.to(DEV), 128, ck, cv, rot, 8, 128, 16, out=out, workspace=ws)
    assert K.workspace_status(ws) & 4
    attention_close(out[:128], ref[:128], ref32[:128], rot, rtol=PAGED_PREFILL_RTOL)
    attention_close(out[150:], ref[150:], ref32[150:], rot, rtol=PAGED_PREFILL_RTOL)
    assert (out[128:150] == 0).all()
