"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

K and V are N(0,1); K has four fixed channels (a seed-1 permutation of the 128 channels)
scaled by 10 before the dtype cast.  Block tables and slot mappings are seeded
permutations.  Everything is produced on the CPU so that the same tensors can be handed to
the CUDA kernels and to a CPU checker.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

K_SEED, V_SEED, Q_SEED = 1000, 2000, 3000


def outlier_channels(head_dim: int = 128) -> torch.Tensor:
    return torch.randperm(head_dim, generator=torch.Generator().manual_seed(1))[:4]


def make_kv(n_tokens: int, num_kv_heads: int, head_dim: int, cfg: int, dtype=torch.bfloat16):
    """K (with outlier channels) and V, each (n_tokens, num_kv_heads, head_dim)."""
    gk = torch.Generator().manual_seed(K_SEED + cfg)
    gv = torch.Generator().manual_seed(V_SEED + cfg)
    k = torch.randn(n_tokens, num_kv_heads, head_dim, generator=gk)
    v = torch.randn(n_tokens, num_kv_heads, head_dim, generator=gv)
    k[..., outlier_channels(head_dim)] *= 10.0
    return k.to(dtype), v.to(dtype)


def make_q(num_seqs: int, num_q_heads: int, head_dim: int, cfg: int, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(Q_SEED + cfg)
    return torch.randn(num_seqs, num_q_heads, head_dim, generator=g).to(dtype)


@dataclass
class DecodeWorkload:
    num_seqs: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    block_size: int
    num_blocks: int
    seq_lens: torch.Tensor      # (num_seqs,) int32
    block_table: torch.Tensor   # (num_seqs, max_blocks) int32
    slot_mapping: torch.Tensor  # (total_tokens,) int64: cache slot of token j of the flat K/V
    q: torch.Tensor             # (num_seqs, num_q_heads, head_dim)
    cfg: int

    @property
    def total_tokens(self) -> int:
        return int(self.seq_lens.sum())

    @property
    def row_bytes(self) -> int:
        return self.num_kv_heads * (self.head_dim + 8)

    def algorithmic_bytes(self) -> int:
        """Bytes one decode call has to move: 136 B per (token, KV head) at D=128, q in and
        out, and the block-table entries that are read."""
        d = self.head_dim
        kv = self.total_tokens * self.num_kv_heads * (d + 8)
        qo = 2 * self.num_seqs * self.num_q_heads * d * 2
        pages = int(((self.seq_lens + self.block_size - 1) // self.block_size).sum())
        return kv + qo + 4 * pages


def decode_workload(num_seqs=32, context=4096, num_q_heads=32, num_kv_heads=8, head_dim=128,
                    block_size=16, cfg=1, seq_lens=None, table_seed=2, dtype=torch.bfloat16,
                    spare_blocks=0) -> DecodeWorkload:
    """Paged-decode inputs: config 1 by default (32 sequences x 4096 tokens, 8192 pages whose
    block table is a seed-2 permutation)."""
    if seq_lens is None:
        seq_lens = torch.full((num_seqs,), context, dtype=torch.int32)
    else:
        seq_lens = torch.as_tensor(seq_lens, dtype=torch.int32)
        num_seqs = seq_lens.numel()
    max_blocks = max(1, int((int(seq_lens.max()) + block_size - 1) // block_size))
    num_blocks = num_seqs * max_blocks + spare_blocks
    perm = torch.randperm(num_blocks, generator=torch.Generator().manual_seed(table_seed))
    block_table = perm[: num_seqs * max_blocks].reshape(num_seqs, max_blocks).int()
    slots = []
    for i in range(num_seqs):
        t = torch.arange(int(seq_lens[i]))
        slots.append(block_table[i][t // block_size].long() * block_size + t % block_size)
    slot_mapping = torch.cat(slots) if slots else torch.empty(0, dtype=torch.int64)
    q = make_q(num_seqs, num_q_heads, head_dim, cfg, dtype)
    return DecodeWorkload(num_seqs, num_q_heads, num_kv_heads, head_dim, block_size, num_blocks,
                          seq_lens, block_table, slot_mapping, q, cfg)


def ragged_lengths(num_seqs=8, lo=32768, hi=131072, seed=4) -> torch.Tensor:
    """Config 4 lengths: uniform integers in [lo, hi] from the given seed."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(lo, hi + 1, (num_seqs,), generator=g).int()


@dataclass
class AppendWorkload:
    key: torch.Tensor           # (n_tokens, H, D)
    value: torch.Tensor
    slot_mapping: torch.Tensor  # (n_tokens,) int64, injective
    num_slots: int
    block_size: int

    def algorithmic_bytes(self, with_qjl: bool) -> int:
        n, h, d = self.key.shape
        read = 2 * n * h * d * self.key.element_size() + n * 8
        write = n * h * (d + 8) + (n * h * (d // 8 + 4) if with_qjl else 0)
        return read + write


def append_workload(n_tokens=8192, num_kv_heads=8, head_dim=128, num_slots=65536, block_size=16,
                    cfg=2, dtype=torch.bfloat16, seed=3) -> AppendWorkload:
    """Compress-on-append inputs: config 2 by default."""
    k, v = make_kv(n_tokens, num_kv_heads, head_dim, cfg, dtype)
    slots = torch.randperm(num_slots, generator=torch.Generator().manual_seed(seed))[:n_tokens]
    return AppendWorkload(k, v, slots.long(), num_slots, block_size)
