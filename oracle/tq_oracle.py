"""CPU oracle for the TurboQuant KV-cache hot path.  TEST INFRASTRUCTURE ONLY.

This file restates, with plain PyTorch CPU ops, the arithmetic of the reference's
pure-PyTorch path (ayinedjimi/flashquant).  It exists so that the CUDA kernels can be
checked against the reference's results on a machine where the reference itself is not
installed.  Nothing in the product package imports it: only the test-suite, the smoke
entry and the CPU-baseline leg of the benchmark do, and only as the checker.

Parity status: PINNED.  Every function below is compared, in ``tests/test_oracle_golden.py``,
with fixtures under ``tests/golden/`` that were produced by importing and running the
reference package itself (generator: ``tests/golden/make_golden.py``), and with the
known-answer bytes of the reference's own packing tests.

The reference does all of its arithmetic through torch CPU kernels (``torch.linalg.qr``,
``torch.randn(generator=...)``, ``matmul``, ``bucketize``, ``softmax``); the same calls are
used here so that the rotation, the QJL matrix and the codebooks are bit-identical.

Each function cites the reference file and lines it follows (paths are relative to the
reference's repository root).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

NORM_EPS = 1e-10  # src/flashquant/core/quantizer.py:150


# --------------------------------------------------------------------------------------
# Host-side constants: codebook, rotation, QJL matrix
# --------------------------------------------------------------------------------------

def lloyd_max_codebook(dim: int, bits: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Lloyd-Max centroids/boundaries for N(0, 1/dim) on +-3.5 sigma.

    Follows src/flashquant/core/codebook.py:58-140: fp64 iteration, uniform start,
    at most 200 sweeps, stop when the largest centroid shift is below 1e-10, boundaries
    are midpoints, both returned as fp32.
    """
    levels = 1 << bits
    sigma = 1.0 / math.sqrt(dim)
    lo, hi = -3.5 * sigma, 3.5 * sigma
    cent = torch.tensor(
        [lo + (hi - lo) * (i + 0.5) / levels for i in range(levels)], dtype=torch.float64
    )
    inv_sigma = 1.0 / sigma
    inv_sigma_sq2 = inv_sigma / math.sqrt(2.0)
    norm_const = 1.0 / (sigma * math.sqrt(2.0 * math.pi))

    def pdf(t):
        return norm_const * torch.exp(-0.5 * (t * inv_sigma) ** 2)

    def cdf(t):
        return 0.5 * (1.0 + torch.erf(t * inv_sigma_sq2))

    edge_lo = torch.tensor([lo], dtype=torch.float64)
    edge_hi = torch.tensor([hi], dtype=torch.float64)
    for _ in range(200):
        mids = (cent[:-1] + cent[1:]) / 2.0
        edges = torch.cat([edge_lo, mids, edge_hi])
        a, b = edges[:-1], edges[1:]
        mass = cdf(b) - cdf(a)
        safe = torch.where(mass > 1e-15, mass, torch.ones_like(mass))
        upd = (sigma ** 2) * (pdf(a) - pdf(b)) / safe
        upd = torch.where(mass > 1e-15, upd, (a + b) / 2.0)
        shift = (upd - cent).abs().max().item()
        cent = upd
        if shift < 1e-10:
            break
    mids = (cent[:-1] + cent[1:]) / 2.0
    return cent.float(), mids.float()


def haar_rotation(dim: int, seed: int) -> torch.Tensor:
    """Haar-random orthogonal matrix Pi (dim, dim) fp32.

    src/flashquant/core/quantizer.py:60-85: QR of a seeded CPU Gaussian, columns of Q
    multiplied by sign(diag(R)) (zero counted as +1).
    """
    gen = torch.Generator(device="cpu").manual_seed(seed)
    g = torch.randn(dim, dim, generator=gen, device="cpu", dtype=torch.float32)
    q, r = torch.linalg.qr(g)
    s = torch.sign(torch.diag(r))
    s[s == 0] = 1.0
    return q * s.unsqueeze(0)


def qjl_matrix(dim: int, seed: int, qjl_dim: Optional[int] = None) -> torch.Tensor:
    """QJL projection S (m, dim) fp32 = randn(seed + 1) / sqrt(m).

    src/flashquant/core/quantizer.py:264-268 (``seed`` is the quantiser's seed; the
    generator is seeded with ``seed + 1``).
    """
    m = qjl_dim or dim
    gen = torch.Generator(device="cpu").manual_seed(seed + 1)
    return torch.randn(m, dim, generator=gen, device="cpu", dtype=torch.float32) / math.sqrt(m)


def split_rotation_T(rotation: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Even / odd columns of Pi^T, each (D, D/2) contiguous.

    src/flashquant/kernels/compress.py:86-89.
    """
    rt = rotation.T.contiguous()
    return rt[:, 0::2].contiguous(), rt[:, 1::2].contiguous()


# --------------------------------------------------------------------------------------
# Packing
# --------------------------------------------------------------------------------------

def nibble_pack(idx: torch.Tensor) -> torch.Tensor:
    """byte j = (idx[2j] << 4) | idx[2j+1].  src/flashquant/core/packing.py:77-79."""
    if idx.shape[-1] % 2:
        raise ValueError("last dimension must be even")
    e = idx[..., 0::2].to(torch.uint8)
    o = idx[..., 1::2].to(torch.uint8)
    return ((e << 4) | o).to(torch.uint8)


def nibble_unpack(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of nibble_pack; int64 out.  src/flashquant/core/packing.py:96-98."""
    hi = (packed >> 4).long()
    lo = (packed & 0x0F).long()
    return torch.stack([hi, lo], dim=-1).flatten(-2)


def pack_2bit(idx: torch.Tensor) -> torch.Tensor:
    """Four 2-bit codes per byte, first code in the top two bits.

    csrc/core/packing.cpp:48-66 (v0<<6 | v1<<4 | v2<<2 | v3), as restated by the reference's
    tests (tests/conftest.py:245-257)."""
    d = idx.shape[-1]
    if d % 4 != 0:
        raise ValueError(f"Last dim must be divisible by 4, got {d}")
    f = idx.reshape(-1, d).to(torch.uint8)
    packed = (f[:, 0::4] << 6) | (f[:, 1::4] << 4) | (f[:, 2::4] << 2) | f[:, 3::4]
    return packed.reshape(*idx.shape[:-1], d // 4)


def unpack_2bit(packed: torch.Tensor, dim: int) -> torch.Tensor:
    """csrc/core/packing.cpp:68-79; tests/conftest.py:259-265."""
    parts = [((packed >> s) & 0x03).long() for s in (6, 4, 2, 0)]
    return torch.stack(parts, dim=-1).flatten(-2)


def sign_bits_pack(signs: torch.Tensor) -> torch.Tensor:
    """QJL signs (+-1 floats, (..., m)) -> (..., m/8) uint8.

    Bit (j % 8) of byte (j // 8) is 1 exactly when sign j is +1.  This packed form is
    this project's own storage format for the signs the reference returns as floats
    (src/flashquant/core/quantizer.py:296-302); the reference never stores them.
    """
    m = signs.shape[-1]
    if m % 8:
        raise ValueError("qjl_dim must be a multiple of 8")
    bits = (signs > 0).to(torch.uint8).reshape(*signs.shape[:-1], m // 8, 8)
    weights = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.uint8)
    return (bits * weights).sum(dim=-1).to(torch.uint8)


def sign_bits_unpack(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of sign_bits_pack: (..., m/8) uint8 -> (..., m) float32 of +-1."""
    shifts = torch.arange(8, dtype=torch.uint8)
    bits = (packed.unsqueeze(-1) >> shifts) & 1
    return (bits.flatten(-2).float() * 2.0 - 1.0)


# --------------------------------------------------------------------------------------
# Stage 1 (MSE) quantiser, compress / decompress
# --------------------------------------------------------------------------------------

def mse_quantize(x: torch.Tensor, rotation: torch.Tensor, boundaries: torch.Tensor):
    """Returns (indices int64 (..., D), norms fp32 (..., 1), rotated fp32 (N, D)).

    src/flashquant/core/quantizer.py:145-159: norm, divide by (norm + 1e-10), multiply by
    Pi^T, ``torch.bucketize`` (right=False: index = number of boundaries strictly below).
    ``rotated`` is returned as well so that tests can tell which coordinates sit next to
    a boundary.
    """
    d = x.shape[-1]
    flat = x.reshape(-1, d).float()
    norms = torch.norm(flat, dim=-1, keepdim=True)
    unit = flat / (norms + NORM_EPS)
    rotated = unit @ rotation.T
    idx = torch.bucketize(rotated, boundaries)
    return idx.reshape(x.shape), norms.reshape(*x.shape[:-1], 1), rotated


def mse_dequantize(idx, norms, rotation, centroids) -> torch.Tensor:
    """(c[idx] @ Pi) * norm, original space.  src/flashquant/core/quantizer.py:181-195."""
    d = idx.shape[-1]
    rec = centroids[idx.reshape(-1, d)] @ rotation
    return (rec * norms.reshape(-1, 1)).reshape(idx.shape)


def compress(x: torch.Tensor, rotation: torch.Tensor, boundaries: torch.Tensor):
    """(N, H, D) float -> packed (N, H, D/2) u8, norms (N, H, 1) fp32.

    src/flashquant/kernels/cpu_reference.py:22-61 (indices clamped to 0..15, then
    nibble-packed).
    """
    n, h, d = x.shape
    idx, norms, _ = mse_quantize(x.reshape(n * h, d), rotation, boundaries)
    idx = idx.clamp(0, 15).to(torch.uint8)
    packed = (idx[:, 0::2] << 4) | idx[:, 1::2]
    return packed.reshape(n, h, d // 2), norms.reshape(n, h, 1)


def decompress(packed: torch.Tensor, norms: torch.Tensor, centroids: torch.Tensor):
    """(N, H, D/2) u8 + (N, H, 1) fp32 -> (N, H, D) fp32, rotated space.

    src/flashquant/kernels/cpu_reference.py:64-94.
    """
    n, h, half = packed.shape
    idx = nibble_unpack(packed).reshape(n * h, 2 * half)
    return (centroids[idx] * norms.reshape(n * h, 1)).reshape(n, h, 2 * half)


# --------------------------------------------------------------------------------------
# Stage 2 (Prod): QJL residual signs and residual norm
# --------------------------------------------------------------------------------------

def prod_quantize(x, rotation, centroids, boundaries, qjl):
    """Returns (indices, norms, signs (+-1 fp32), gamma fp32 (..., 1)).

    src/flashquant/core/quantizer.py:285-304.  ``centroids``/``boundaries`` are the
    (bits-1)-bit tables (quantizer.py:262).
    """
    d = x.shape[-1]
    idx, norms, _ = mse_quantize(x, rotation, boundaries)
    recon = mse_dequantize(idx, norms, rotation, centroids)
    resid = x.float() - recon
    gamma = torch.norm(resid, dim=-1, keepdim=True)
    proj = resid.reshape(-1, d) @ qjl.T
    signs = torch.sign(proj).reshape(*x.shape[:-1], qjl.shape[0])
    signs[signs == 0] = 1.0
    return idx, norms, signs, gamma


def estimate_inner_product(query, idx, norms, signs, gamma, rotation, centroids, qjl):
    """<q,k> ~ <q,k_mse> + gamma*sqrt(pi/2)/m * <S q, signs>.

    src/flashquant/core/quantizer.py:349-370.
    """
    d = query.shape[-1]
    m = qjl.shape[0]
    k_mse = mse_dequantize(idx, norms, rotation, centroids)
    mse_term = (query.float() * k_mse).sum(dim=-1, keepdim=True)
    qp = (query.float().reshape(-1, d) @ qjl.T).reshape(*query.shape[:-1], m)
    corr = (qp * signs).sum(dim=-1, keepdim=True)
    return mse_term + gamma * math.sqrt(math.pi / 2.0) / m * corr


# --------------------------------------------------------------------------------------
# Paged cache rows (compress-on-append)
# --------------------------------------------------------------------------------------

def row_layout(num_kv_heads: int, head_dim: int):
    """Byte offsets of one token row: [K idx | K norms | V idx | V norms].

    src/flashquant/vllm/impl.py:132-138, src/flashquant/kernels/cpu_reference.py:276-280.
    Returns (k_idx_end, k_norm_end, v_idx_end, total_bytes).
    """
    half = head_dim // 2
    k_idx_end = num_kv_heads * half
    k_norm_end = k_idx_end + num_kv_heads * 4
    v_idx_end = k_norm_end + num_kv_heads * half
    total = v_idx_end + num_kv_heads * 4
    return k_idx_end, k_norm_end, v_idx_end, total


def assemble_rows(k_packed, k_norms, v_packed, v_norms):
    """(N,H,D/2) u8 / (N,H,1) fp32 pairs -> (N, total_bytes) u8 rows.

    src/flashquant/vllm/impl.py:243-258 (norms are raw little-endian fp32 bytes).
    """
    n, h, half = k_packed.shape
    k_idx_end, k_norm_end, v_idx_end, total = row_layout(h, 2 * half)
    row = torch.empty(n, total, dtype=torch.uint8)
    row[:, :k_idx_end] = k_packed.reshape(n, -1)
    row[:, k_idx_end:k_norm_end] = k_norms.reshape(n, h).contiguous().view(torch.uint8)
    row[:, k_norm_end:v_idx_end] = v_packed.reshape(n, -1)
    row[:, v_idx_end:] = v_norms.reshape(n, h).contiguous().view(torch.uint8)
    return row


def compress_and_store(key, value, kv_cache, slot_mapping, rotation, boundaries_k,
                       boundaries_v=None):
    """Compress K and V, build rows, scatter them to ``kv_cache`` (in place).

    src/flashquant/vllm/impl.py:220-263.  The reference uses one boundary table for both
    (impl.py:237-258); a second table may be given for V.  Negative slots (padding) are
    skipped - the reference does not guard them, the CUDA kernel does.
    """
    if boundaries_v is None:
        boundaries_v = boundaries_k
    kp, kn = compress(key, rotation, boundaries_k)
    vp, vn = compress(value, rotation, boundaries_v)
    rows = assemble_rows(kp, kn, vp, vn)
    flat = kv_cache.view(-1, rows.shape[1])
    slots = slot_mapping.long()
    keep = slots >= 0
    flat[slots[keep]] = rows[keep]
    return rows


def qjl_plane_rows(signs: torch.Tensor, gamma: torch.Tensor) -> torch.Tensor:
    """(N,H,m) +-1 and (N,H,1) fp32 -> (N, H*(m/8+4)) u8: [sign bits | gamma], head-major.

    Side plane of this project (the reference has no packed QJL storage): region 1 holds
    m/8 sign bytes per head, region 2 one fp32 gamma per head.
    """
    n, h, m = signs.shape
    bits = sign_bits_pack(signs).reshape(n, h * (m // 8))
    g = gamma.reshape(n, h).contiguous().view(torch.uint8)
    return torch.cat([bits, g], dim=1)


# --------------------------------------------------------------------------------------
# Attention
# --------------------------------------------------------------------------------------

def attention(q, k, v, sm_scale=None, is_causal=False):
    """Scaled dot-product attention with GQA, fp32 math, output in q.dtype.

    src/flashquant/kernels/cpu_reference.py:97-151.  q (B,Hq,Nq,D), k/v (B,Hkv,Nkv,D).
    """
    b, hq, nq, d = q.shape
    hkv, nkv = k.shape[1], k.shape[2]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    if is_causal and nq == 1:
        is_causal = False
    if hq != hkv:
        k = k.repeat_interleave(hq // hkv, dim=1)
        v = v.repeat_interleave(hq // hkv, dim=1)
    s = torch.matmul(q.float(), k.float().transpose(-2, -1)) * sm_scale
    if is_causal:
        mask = torch.triu(torch.ones(nq, nkv, dtype=torch.bool), diagonal=1)
        s = s.masked_fill(mask, float("-inf"))
    p = torch.softmax(s, dim=-1)
    return torch.matmul(p, v.float()).to(q.dtype)


def fused_tq_attention(q, k_packed, k_norms, v_packed, v_norms, centroids_k, centroids_v,
                       rotation, sm_scale=None, is_causal=False, q_chunk: int = 0,
                       rotation_v=None):
    """Un-rotated q in, original-space output out.

    ``rotation_v`` (default: ``rotation``) is the rotation the values were compressed with,
    for the cache whose keys and values use different seeds
    (src/flashquant/cache/hf_cache.py:137-142): the output is rotated back by it.

    src/flashquant/kernels/attention.py:99-107 (q_rot = (q.float() @ Pi^T).to(dtype)) then
    src/flashquant/kernels/cpu_reference.py:154-227 (decompress K and V in rotated space,
    attention, out = (out_rot.float() @ Pi).to(dtype)).

    ``q_chunk`` > 0 evaluates the same expression over slices of query heads of one KV
    group at a time so that the full score tensor never has to exist; results are
    identical because rows of the softmax are independent.
    """
    return fused_tq_attention_stages(q, k_packed, k_norms, v_packed, v_norms, centroids_k,
                                     centroids_v, rotation, sm_scale, is_causal, q_chunk,
                                     rotation_v)[1]


def fused_tq_attention_stages(q, k_packed, k_norms, v_packed, v_norms, centroids_k, centroids_v,
                              rotation, sm_scale=None, is_causal=False, q_chunk: int = 0,
                              rotation_v=None):
    """``fused_tq_attention`` with the fp32 rotated-space rows behind it: ``(o_rot_fp32, out)``
    (the reference never rounds those rows: its attention runs on ``q_rot.float()``)."""
    b, hq, nq, d = q.shape
    hkv, nkv = k_packed.shape[1], k_packed.shape[2]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    q_rot = torch.matmul(q.float(), rotation.T).to(q.dtype)
    kd = decompress(k_packed.reshape(b * hkv, nkv, d // 2), k_norms.reshape(b * hkv, nkv, 1),
                    centroids_k).reshape(b, hkv, nkv, d)
    vd = decompress(v_packed.reshape(b * hkv, nkv, d // 2), v_norms.reshape(b * hkv, nkv, 1),
                    centroids_v).reshape(b, hkv, nkv, d)
    if q_chunk <= 0:
        out_rot = attention(q_rot.float(), kd, vd, sm_scale, is_causal)
    else:
        if is_causal and nq != nkv:
            raise ValueError("chunked causal evaluation needs N_q == N_kv")
        g = hq // hkv
        out_rot = torch.empty(b, hq, nq, d, dtype=torch.float32)
        for bi in range(b):
            for h in range(hkv):
                qs = q_rot[bi, h * g:(h + 1) * g].float()
                for q0 in range(0, nq, q_chunk):
                    q1 = min(nq, q0 + q_chunk)
                    kv_hi = q1 if is_causal else nkv
                    s = torch.matmul(qs[:, q0:q1], kd[bi, h, :kv_hi].T) * sm_scale
                    if is_causal:
                        qi = torch.arange(q0, q1).unsqueeze(1)
                        ki = torch.arange(kv_hi).unsqueeze(0)
                        s = s.masked_fill(ki > qi, float("-inf"))
                    out_rot[bi, h * g:(h + 1) * g, q0:q1] = torch.matmul(
                        torch.softmax(s, dim=-1), vd[bi, h, :kv_hi])
    # flash_attention_reference casts to its q dtype, which is fp32 here
    # (cpu_reference.py:195 passes q_rot.float()), so no rounding before the rotation.
    out_rot = out_rot.float()
    return out_rot, torch.matmul(out_rot, rotation if rotation_v is None else rotation_v).to(q.dtype)


class CompressedCacheOracle:
    """What CompressedDynamicCache keeps and returns, layer by layer, on the CPU.

    src/flashquant/cache/hf_cache.py:260-365 with src/flashquant/core/compressor.py:235-262:
    an update quantises ``x.float()`` (keys with the key tables, values with the value
    tables), appends the nibble-packed codes and fp32 norms to the layer, de-quantises the
    NEW tokens only, casts them to the dtype of the update and returns them appended to what
    earlier updates returned.
    """

    def __init__(self, rotation_k, rotation_v, centroids, boundaries):
        self.rotation_k, self.rotation_v = rotation_k, rotation_v
        self.centroids, self.boundaries = centroids, boundaries
        self.layers = {}

    def _roundtrip(self, x, rotation):
        idx, norms, _ = mse_quantize(x.float(), rotation, self.boundaries)
        packed = nibble_pack(idx.to(torch.uint8))
        back = mse_dequantize(nibble_unpack(packed).long(), norms, rotation, self.centroids)
        return packed, norms.float(), back.to(x.dtype)

    def update(self, key_states, value_states, layer_idx):
        kp, kn, kd = self._roundtrip(key_states, self.rotation_k)
        vp, vn, vd = self._roundtrip(value_states, self.rotation_v)
        new = [kp, kn, vp, vn, kd, vd]
        old = self.layers.get(layer_idx)
        self.layers[layer_idx] = new if old is None else [
            torch.cat([o, n], dim=2) for o, n in zip(old, new)]
        return self.layers[layer_idx][4], self.layers[layer_idx][5]

    def get_compressed(self, layer_idx):
        return tuple(self.layers[layer_idx][:4])

    def get_seq_length(self, layer_idx=0):
        return 0 if layer_idx not in self.layers else self.layers[layer_idx][0].shape[2]


def gather_paged(kv_cache, block_row, seq_len, num_kv_heads, head_dim, block_size,
                 centroids_k, centroids_v):
    """Dequantised K and V (H_kv, L, D) fp32, rotated space, of one sequence.

    Same per-token arithmetic as src/flashquant/kernels/cpu_reference.py:293-329, done
    for all tokens at once.
    """
    half = head_dim // 2
    k_idx_end, k_norm_end, v_idx_end, total = row_layout(num_kv_heads, head_dim)
    t = torch.arange(seq_len)
    phys = block_row[t // block_size].long()
    rows = kv_cache[phys, t % block_size]  # (L, total)
    kp = rows[:, :k_idx_end].reshape(seq_len, num_kv_heads, half)
    kn = rows[:, k_idx_end:k_norm_end].contiguous().view(torch.float32).reshape(
        seq_len, num_kv_heads, 1)
    vp = rows[:, k_norm_end:v_idx_end].reshape(seq_len, num_kv_heads, half)
    vn = rows[:, v_idx_end:].contiguous().view(torch.float32).reshape(seq_len, num_kv_heads, 1)
    k = decompress(kp, kn, centroids_k).permute(1, 0, 2)
    v = decompress(vp, vn, centroids_v).permute(1, 0, 2)
    return k, v


def paged_decode_rotated(q_rot, kv_cache, block_table, seq_lens, centroids_k, centroids_v,
                         num_kv_heads, head_dim, block_size, sm_scale=None, keep_fp32=False,
                         per_kv_head=False):
    """Rotated-space paged decode (vectorised per sequence).

    src/flashquant/kernels/cpu_reference.py:230-368.  A sequence of length 0 yields zeros.
    ``keep_fp32`` returns the fp32 rows the reference holds just before it casts them to the
    query's dtype (cpu_reference.py:365-366), for checks of what precedes that rounding.
    """
    num_seqs, hq, d = q_rot.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    out = torch.zeros(q_rot.shape, dtype=torch.float32) if keep_fp32 else torch.zeros_like(q_rot)
    g = hq // num_kv_heads
    for i in range(num_seqs):
        n = int(seq_lens[i])
        if n == 0:
            continue
        k, v = gather_paged(kv_cache, block_table[i], n, num_kv_heads, head_dim, block_size,
                            centroids_k, centroids_v)
        if per_kv_head:
            # the same expression one KV head at a time (very long sequences: the repeated
            # K and V of all query heads would not fit)
            for h in range(num_kv_heads):
                s = torch.matmul(q_rot[i, h * g:(h + 1) * g].float(), k[h].T) * sm_scale
                out[i, h * g:(h + 1) * g] = torch.matmul(torch.softmax(s, dim=-1), v[h]).to(out.dtype)
            continue
        if g > 1:
            k = k.repeat_interleave(g, dim=0)
            v = v.repeat_interleave(g, dim=0)
        s = torch.bmm(q_rot[i].float().unsqueeze(1), k.transpose(-2, -1)) * sm_scale
        p = torch.softmax(s, dim=-1)
        out[i] = torch.bmm(p, v).squeeze(1).to(out.dtype)
    return out


def paged_decode_rotated_loop(q_rot, kv_cache, block_table, seq_lens, centroids_k,
                              centroids_v, num_kv_heads, head_dim, block_size,
                              sm_scale=None):
    """Token-by-token form of ``paged_decode_rotated`` for small cases.

    Walks the block table the way src/flashquant/kernels/cpu_reference.py:284-335 does
    (one row, one KV head at a time) and is used to check the vectorised form.
    """
    num_seqs, hq, d = q_rot.shape
    half = head_dim // 2
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    k_idx_end, k_norm_end, v_idx_end, _ = row_layout(num_kv_heads, head_dim)
    out = torch.zeros_like(q_rot)
    g = hq // num_kv_heads
    for i in range(num_seqs):
        n = int(seq_lens[i])
        if n == 0:
            continue
        ks = torch.empty(num_kv_heads, n, head_dim)
        vs = torch.empty(num_kv_heads, n, head_dim)
        for t in range(n):
            row = kv_cache[int(block_table[i, t // block_size]), t % block_size]
            for h in range(num_kv_heads):
                kb = row[h * half:(h + 1) * half]
                kn = row[k_idx_end + 4 * h:k_idx_end + 4 * h + 4].view(torch.float32)
                vb = row[k_norm_end + h * half:k_norm_end + (h + 1) * half]
                vn = row[v_idx_end + 4 * h:v_idx_end + 4 * h + 4].view(torch.float32)
                ks[h, t] = centroids_k[nibble_unpack(kb)] * kn
                vs[h, t] = centroids_v[nibble_unpack(vb)] * vn
        k = ks.repeat_interleave(g, dim=0)
        v = vs.repeat_interleave(g, dim=0)
        s = torch.bmm(q_rot[i].float().unsqueeze(1), k.transpose(-2, -1)) * sm_scale
        out[i] = torch.bmm(torch.softmax(s, dim=-1), v).squeeze(1).to(q_rot.dtype)
    return out


def split_k_paged_decode(q, kv_cache, block_table, seq_lens, centroids_k, centroids_v,
                         rotation, num_kv_heads, head_dim, block_size, sm_scale=None):
    """Un-rotated q in, original-space out, with the reference's three roundings.

    src/flashquant/kernels/paged_decode.py:112-128: q_rot rounded to q.dtype, rotated
    output rounded to q.dtype by the attention, final product rounded to q.dtype.
    """
    return split_k_paged_decode_stages(q, kv_cache, block_table, seq_lens, centroids_k,
                                       centroids_v, rotation, num_kv_heads, head_dim,
                                       block_size, sm_scale)[1]


def split_k_paged_decode_stages(q, kv_cache, block_table, seq_lens, centroids_k, centroids_v,
                                rotation, num_kv_heads, head_dim, block_size, sm_scale=None,
                                per_kv_head=False):
    """``split_k_paged_decode`` together with the value it rounds: returns
    ``(o_rot_fp32, out)`` where ``o_rot_fp32`` is the rotated-space attention output before
    its cast to the query's dtype and ``out = ((o_rot_fp32.to(dtype)).float() @ Pi).to(dtype)``."""
    q_rot = torch.matmul(q.float(), rotation.T).to(q.dtype)
    o32 = paged_decode_rotated(q_rot, kv_cache, block_table, seq_lens, centroids_k, centroids_v,
                               num_kv_heads, head_dim, block_size, sm_scale, keep_fp32=True,
                               per_kv_head=per_kv_head)
    return o32, torch.matmul(o32.to(q.dtype).float(), rotation).to(q.dtype)


def paged_decode_multi(q, kv_cache, block_table, seq_lens, centroids_k, centroids_v, rotation,
                       num_kv_heads, head_dim, block_size, sm_scale=None):
    """The last n_q tokens of every sequence attend causally over the paged cache.

    q (num_seqs, n_q, Hq, D); seq_lens counts the n_q new tokens.  What the reference's
    decompress-all path computes for a step of more than one token
    (src/flashquant/vllm/impl.py:477-509 feeding flash_attn_varlen_func(causal=True), whose
    mask is aligned at the END of the keys): de-quantise the sequence in rotated space, query
    i sees keys 0 .. L - n_q + i, softmax in fp32, with the roundings of the single-token path
    (src/flashquant/kernels/paged_decode.py:112-128).  A query without visible keys gives zeros.
    """
    return paged_decode_multi_stages(q, kv_cache, block_table, seq_lens, centroids_k, centroids_v,
                                     rotation, num_kv_heads, head_dim, block_size, sm_scale)[1]


def paged_decode_multi_stages(q, kv_cache, block_table, seq_lens, centroids_k, centroids_v,
                              rotation, num_kv_heads, head_dim, block_size, sm_scale=None):
    """``paged_decode_multi`` with the fp32 rotated-space rows it rounds: ``(o_rot_fp32, out)``."""
    num_seqs, n_q, hq, d = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    g = hq // num_kv_heads
    q_rot = torch.matmul(q.float(), rotation.T).to(q.dtype)
    o_rot = torch.zeros(q_rot.shape, dtype=torch.float32)
    for i in range(num_seqs):
        n = int(seq_lens[i])
        if n == 0:
            continue
        k, v = gather_paged(kv_cache, block_table[i], n, num_kv_heads, head_dim, block_size,
                            centroids_k, centroids_v)          # (Hkv, L, D)
        k = k.repeat_interleave(g, dim=0)
        v = v.repeat_interleave(g, dim=0)
        qs = q_rot[i].float().permute(1, 0, 2)                   # (Hq, n_q, D)
        s = torch.bmm(qs, k.transpose(-2, -1)) * sm_scale       # (Hq, n_q, L)
        visible = torch.arange(n).unsqueeze(0) <= (n - n_q + torch.arange(n_q)).unsqueeze(1)
        s = s.masked_fill(~visible.unsqueeze(0), float("-inf"))
        p = torch.softmax(s, dim=-1)
        p = torch.where(visible.any(dim=1).reshape(1, n_q, 1), p, torch.zeros_like(p))
        o_rot[i] = torch.bmm(p, v).permute(1, 0, 2)
    return o_rot, torch.matmul(o_rot.to(q.dtype).float(), rotation).to(q.dtype)


def paged_prefill_varlen_stages(q, kv_cache, block_table, seq_lens, cu_seqlens_q, centroids_k,
                                centroids_v, rotation, num_kv_heads, head_dim, block_size,
                                sm_scale=None):
    """Prefill chunks of different lengths over the paged cache: ``(o_rot_fp32, out)``.

    q ``(total_q_tokens, Hq, D)``, sequence b owns tokens cu[b] .. cu[b+1], the last ones of its
    seq_lens[b] keys.  The reference's prefill path (src/flashquant/vllm/impl.py:265-336,
    477-509: rotate q, de-quantise, flash_attn_varlen_func(cu_seqlens_q, seqused_k, causal=True),
    rotate back) sequence by sequence, through ``paged_decode_multi_stages``.
    """
    o32 = torch.zeros(q.shape, dtype=torch.float32)
    out = torch.zeros_like(q)
    for b in range(len(seq_lens)):
        lo, hi = int(cu_seqlens_q[b]), int(cu_seqlens_q[b + 1])
        if hi == lo:
            continue
        r32, r = paged_decode_multi_stages(q[lo:hi].unsqueeze(0), kv_cache, block_table[b:b + 1],
                                           seq_lens[b:b + 1], centroids_k, centroids_v, rotation,
                                           num_kv_heads, head_dim, block_size, sm_scale)
        o32[lo:hi], out[lo:hi] = r32[0], r[0]
    return o32, out


def split_k_partials(q_rot, k, v, sm_scale, bounds):
    """Per-split (m, l, acc) of one head: the quantities a split-K decode exchanges.

    For tokens [a, b): m = max logit, l = sum exp(logit - m), acc = sum exp(logit - m) v.
    An empty split has m = -inf, l = 0, acc = 0.  The reference only sketches this step
    (csrc/cuda/paged_decode.cu:198-275) and its merge kernel weights acc by l
    (csrc/cuda/split_k_reduce.cu:84,99), which is not the softmax; the merge below is the
    algebraically exact one and its result equals the unsplit softmax.
    """
    parts = []
    for a, b in bounds:
        if b <= a:
            parts.append((torch.tensor(-math.inf), torch.tensor(0.0), torch.zeros(v.shape[-1])))
            continue
        s = (k[a:b] @ q_rot.float()) * sm_scale
        m = s.max()
        e = torch.exp(s - m)
        parts.append((m, e.sum(), e @ v[a:b]))
    return parts


def split_k_merge(parts):
    """out = sum_s w_s acc_s / sum_s w_s l_s with w_s = exp(m_s - max m)."""
    m_star = max(float(p[0]) for p in parts)
    if m_star == -math.inf:
        return torch.zeros_like(parts[0][2])
    num = torch.zeros_like(parts[0][2])
    den = 0.0
    for m, l, acc in parts:
        w = math.exp(float(m) - m_star) if float(m) > -math.inf else 0.0
        num = num + w * acc
        den = den + w * float(l)
    return num / den


def qjl_paged_decode(q, kv_cache, kq_cache, block_table, seq_lens, centroids_k, centroids_v,
                     rotation, qjl, num_kv_heads, head_dim, block_size, sm_scale=None):
    """Decode whose logits use the two-stage inner-product estimator.

    Logit = sm_scale * (<q, k_mse> + gamma*sqrt(pi/2)/m * <S q, signs>)
    (src/flashquant/core/quantizer.py:349-370), with <q, k_mse> evaluated in rotated space
    as <q_rot, c[idx]> * norm, values as in ``paged_decode_rotated``.  ``kq_cache`` is the
    sign/gamma side plane (num_blocks, block_size, H*(m/8+4)).
    """
    return qjl_paged_decode_stages(q, kv_cache, kq_cache, block_table, seq_lens, centroids_k,
                                   centroids_v, rotation, qjl, num_kv_heads, head_dim, block_size,
                                   sm_scale)[1]


def qjl_paged_decode_stages(q, kv_cache, kq_cache, block_table, seq_lens, centroids_k,
                            centroids_v, rotation, qjl, num_kv_heads, head_dim, block_size,
                            sm_scale=None):
    """``qjl_paged_decode`` with the fp32 rotated-space rows it rounds: ``(o_rot_fp32, out)``."""
    num_seqs, hq, d = q.shape
    m = qjl.shape[0]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    g = hq // num_kv_heads
    q_rot = torch.matmul(q.float(), rotation.T).to(q.dtype)
    sq = torch.matmul(q.float(), qjl.T)  # (num_seqs, hq, m)
    out_rot = torch.zeros(q_rot.shape, dtype=torch.float32)
    for i in range(num_seqs):
        n = int(seq_lens[i])
        if n == 0:
            continue
        k, v = gather_paged(kv_cache, block_table[i], n, num_kv_heads, head_dim, block_size,
                            centroids_k, centroids_v)
        t = torch.arange(n)
        rows = kq_cache[block_table[i][t // block_size].long(), t % block_size]
        bits = rows[:, :num_kv_heads * (m // 8)].reshape(n, num_kv_heads, m // 8)
        gam = rows[:, num_kv_heads * (m // 8):].contiguous().view(torch.float32).reshape(
            n, num_kv_heads)
        signs = sign_bits_unpack(bits).permute(1, 0, 2)  # (H, n, m)
        gam = gam.permute(1, 0)  # (H, n)
        k = k.repeat_interleave(g, dim=0)
        v = v.repeat_interleave(g, dim=0)
        signs = signs.repeat_interleave(g, dim=0)
        gam = gam.repeat_interleave(g, dim=0)
        mse = torch.bmm(q_rot[i].float().unsqueeze(1), k.transpose(-2, -1)).squeeze(1)
        corr = torch.bmm(sq[i].unsqueeze(1), signs.transpose(-2, -1)).squeeze(1)
        s = (mse + gam * math.sqrt(math.pi / 2.0) / m * corr) * sm_scale
        p = torch.softmax(s, dim=-1)
        out_rot[i] = torch.bmm(p.unsqueeze(1), v).squeeze(1)
    return out_rot, torch.matmul(out_rot.to(q.dtype).float(), rotation).to(q.dtype)
