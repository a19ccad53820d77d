"""Work partitioning of the decode path across GPUs (one process per GPU).

Sequences and KV heads are independent, so the usual split needs no communication: each rank
owns whole sequences (``shard_sequences``) or whole KV heads (``shard_kv_heads``; its cache
rows then hold only its heads).  The one exchange step is the split of a single long sequence
over ranks by token range (``cross_gpu_decode``): every rank attends over the pages it holds,
one all-gather moves one ``(H_q, D+4)`` fp32 partial row per sequence and rank, and every rank
merges all rows.  The reference has no multi-GPU code; the partial/merge arithmetic is the
split-K one of the single-GPU kernel.
"""

from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_sequences(num_seqs: int, rank: int, world: int) -> slice:
    """Contiguous, balanced slice of sequence indices owned by ``rank``."""
    lo = num_seqs * rank // world
    hi = num_seqs * (rank + 1) // world
    return slice(lo, hi)


def shard_kv_heads(num_kv_heads: int, num_q_heads: int, rank: int, world: int) -> Tuple[slice, slice]:
    """(KV-head slice, query-head slice) owned by ``rank``; query heads follow their KV head."""
    if num_kv_heads % world:
        raise ValueError("num_kv_heads must be a multiple of the world size")
    per = num_kv_heads // world
    group = num_q_heads // num_kv_heads
    kv = slice(rank * per, (rank + 1) * per)
    return kv, slice(kv.start * group, kv.stop * group)


def token_range(seq_len: int, block_size: int, rank: int, world: int) -> Tuple[int, int]:
    """Token range [lo, hi) of a sequence held by ``rank``: whole pages, contiguous, balanced."""
    pages = (seq_len + block_size - 1) // block_size
    lo = pages * rank // world * block_size
    hi = min(seq_len, pages * (rank + 1) // world * block_size)
    return lo, max(lo, hi)


def local_view(block_table: torch.Tensor, seq_lens: torch.Tensor, block_size: int, rank: int,
               world: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Block table and lengths restricted to the token range of ``rank`` (tables stay 2-D:
    the local pages are moved to the front of each row)."""
    bt = torch.zeros_like(block_table)
    lens = torch.zeros_like(seq_lens)
    for i in range(block_table.shape[0]):
        lo, hi = token_range(int(seq_lens[i]), block_size, rank, world)
        n_pages = (hi - lo + block_size - 1) // block_size
        p0 = lo // block_size
        bt[i, :n_pages] = block_table[i, p0:p0 + n_pages]
        lens[i] = hi - lo
    return bt, lens


def cross_gpu_decode(partial_fn: Callable[[], torch.Tensor],
                     merge_fn: Callable[[torch.Tensor], torch.Tensor],
                     group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """partial rows of this rank -> all-gather -> merged output (identical on every rank).

    ``partial_fn`` returns this rank's ``(num_seqs, H_q, D+4)`` fp32 rows
    (``flashquant_b200.paged_decode_partials`` on its local view), ``merge_fn`` takes the
    gathered ``(world, num_seqs, H_q, D+4)`` tensor (``flashquant_b200.split_k_merge``).
    """
    part = partial_fn().contiguous()
    world = dist.get_world_size(group)
    gathered = torch.empty((world,) + tuple(part.shape), dtype=part.dtype, device=part.device)
    # one collective into one buffer: the result is already in merge layout
    # (gloo wants the output as the inputs stacked along dim 0: same storage, flat view)
    dist.all_gather_into_tensor(gathered.view(world * part.shape[0], *part.shape[1:]), part,
                                group=group)
    return merge_fn(gathered)
