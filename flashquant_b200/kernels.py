"""Host-side mirror of the reference's kernel dispatch layer for the TurboQuant hot path.

The four functions ``tq4_compress``, ``tq4_decompress``, ``fused_tq_attention`` and
``split_k_paged_decode`` keep the names, argument order and return shapes of
``flashquant.kernels`` (reference: src/flashquant/kernels/{compress,decompress,attention,
paged_decode}.py); the remaining ones are the fused entry points this project adds.  Every
call goes through the C ABI of ``libflashquant_b200.so`` with raw device pointers.  There is
no CPU branch: tensors must be CUDA tensors.
"""

from __future__ import annotations

import ctypes as C
import math
from typing import Optional, Tuple

import torch

from . import _native as N

_PART_PAD = 4  # a partial row holds head_dim + 4 floats (acc, m, l, 2 pads)


def _contig(t: torch.Tensor) -> torch.Tensor:
    return t if t.is_contiguous() else t.contiguous()


def _f32(t: torch.Tensor, device) -> torch.Tensor:
    return _contig(t.to(device=device, dtype=torch.float32))


# --------------------------------------------------------------------------------------
# compress / decompress (contiguous)
# --------------------------------------------------------------------------------------

def tq4_compress(
    x: torch.Tensor,
    rotation: torch.Tensor,
    boundaries: torch.Tensor,
    *,
    rotation_T_even: Optional[torch.Tensor] = None,
    rotation_T_odd: Optional[torch.Tensor] = None,
    out: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(N, H, D)`` float -> packed ``(N, H, D/2)`` uint8, norms ``(N, H, 1)`` fp32.

    Same contract as the reference's ``tq4_compress`` (src/flashquant/kernels/compress.py:51-95).
    """
    N.require_cuda(x)
    n, h, d = x.shape
    dev = x.device
    if rotation_T_even is None or rotation_T_odd is None:
        rt = rotation.to(dev).T.contiguous()
        rotation_T_even = rt[:, 0::2].contiguous()
        rotation_T_odd = rt[:, 1::2].contiguous()
    even, odd = _f32(rotation_T_even, dev), _f32(rotation_T_odd, dev)
    bnd = _f32(boundaries, dev)
    x = _contig(x)
    if out is not None:
        packed, norms = out
        if packed.shape != (n, h, d // 2) or norms.numel() != n * h:
            raise ValueError("out buffers have the wrong shape")
    else:
        packed = torch.empty(n, h, d // 2, dtype=torch.uint8, device=dev)
        norms = torch.empty(n, h, 1, dtype=torch.float32, device=dev)
    lib = N.load()
    N.check(lib.fq_tq4_compress(N.ptr(x), N.dtype_code(x.dtype), N.ptr(even), N.ptr(odd),
                                N.ptr(bnd), bnd.numel(), N.ptr(packed), N.ptr(norms), n * h, d,
                                N.stream_ptr(dev)))
    return packed, norms


def tq4_decompress(
    packed: torch.Tensor,
    norms: torch.Tensor,
    centroids: torch.Tensor,
    dtype: torch.dtype = torch.float16,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """packed ``(N, H, D/2)`` + norms ``(N, H, 1)`` -> ``(N, H, D)`` in ``dtype``, rotated space.

    Same contract as the reference's ``tq4_decompress``
    (src/flashquant/kernels/decompress.py:49-86).
    """
    N.require_cuda(packed, norms)
    n, h, half = packed.shape
    dev = packed.device
    cent = _f32(centroids, dev)
    packed, norms = _contig(packed), _contig(norms)
    if out is None:
        out = torch.empty(n, h, 2 * half, dtype=dtype, device=dev)
    elif out.shape != (n, h, 2 * half) or out.dtype != dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous (N, H, D) tensor of the requested dtype")
    lib = N.load()
    N.check(lib.fq_tq4_decompress(N.ptr(packed), N.ptr(norms), N.ptr(cent), cent.numel(),
                                  N.ptr(out), N.dtype_code(dtype), n * h, 2 * half,
                                  N.stream_ptr(dev)))
    return out


def _split_rotation(rotation: torch.Tensor, dev):
    rt = rotation.to(dev).T.contiguous()
    return rt[:, 0::2].contiguous(), rt[:, 1::2].contiguous()


def tq4_compress_into(
    x: torch.Tensor,
    rotation: torch.Tensor,
    boundaries: torch.Tensor,
    packed: torch.Tensor,
    norms: torch.Tensor,
    position: int,
    *,
    rotation_T_even: Optional[torch.Tensor] = None,
    rotation_T_odd: Optional[torch.Tensor] = None,
) -> None:
    """Compress ``x (B, H, S, D)`` into rows ``position .. position+S-1`` of the pre-allocated
    ``packed (B, H, capacity, D/2)`` uint8 and ``norms (B, H, capacity, 1)`` fp32 buffers.

    One launch for what the reference does as compress + nibble_pack + two slice copies
    (src/flashquant/cache/hf_cache.py:170-194, src/flashquant/cache/buffer_pool.py:86-110).
    """
    N.require_cuda(x, packed, norms)
    b, h, s, d = x.shape
    cap = packed.shape[2]
    if packed.shape != (b, h, cap, d // 2) or norms.shape[:3] != (b, h, cap):
        raise ValueError("buffers must be (B, H, capacity, D/2) and (B, H, capacity, 1)")
    if not (packed.is_contiguous() and norms.is_contiguous()):
        raise ValueError("the cache buffers must be contiguous")
    if packed.dtype != torch.uint8 or norms.dtype != torch.float32:
        raise ValueError("buffers must be uint8 codes and fp32 norms")
    dev = x.device
    if rotation_T_even is None or rotation_T_odd is None:
        rotation_T_even, rotation_T_odd = _split_rotation(rotation, dev)
    even, odd = _f32(rotation_T_even, dev), _f32(rotation_T_odd, dev)
    bnd = _f32(boundaries, dev)
    x = _contig(x)
    lib = N.load()
    N.check(lib.fq_tq4_compress_into(N.ptr(x), N.dtype_code(x.dtype), N.ptr(even), N.ptr(odd),
                                     N.ptr(bnd), bnd.numel(), N.ptr(packed), N.ptr(norms), b * h,
                                     s, cap, int(position), d, N.stream_ptr(dev)))


def tq4_decompress_original(
    packed: torch.Tensor,
    norms: torch.Tensor,
    centroids: torch.Tensor,
    rotation: torch.Tensor,
    dtype: torch.dtype = torch.float16,
) -> torch.Tensor:
    """packed ``(..., D/2)`` + norms ``(..., 1)`` -> ``(..., D)`` in ``dtype``, ORIGINAL space.

    ``round_dtype((c[code] * n) Pi)``: what the reference's cache returns from a read
    (src/flashquant/cache/hf_cache.py:196-219).
    """
    N.require_cuda(packed, norms)
    lead, half = packed.shape[:-1], packed.shape[-1]
    dev = packed.device
    n_vec = packed.numel() // half if half else 0
    cent, rot = _f32(centroids, dev), _f32(rotation, dev)
    packed, norms = _contig(packed), _contig(norms.float())
    out = torch.empty(*lead, 2 * half, dtype=dtype, device=dev)
    lib = N.load()
    need = lib.fq_tq4_decompress_original_workspace_bytes(n_vec, 2 * half)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    N.check(lib.fq_tq4_decompress_original(N.ptr(packed), N.ptr(norms), N.ptr(cent), cent.numel(),
                                           N.ptr(rot), N.ptr(out), N.dtype_code(dtype), n_vec,
                                           2 * half, N.ptr(ws), ws.numel(), N.stream_ptr(dev)))
    return out


def cache_update(key, value, tables_k, tables_v, k_packed, k_norms, v_packed, v_norms,
                 position: int, k_out=None, v_out=None, out_position: int = 0,
                 workspace: Optional[torch.Tensor] = None) -> None:
    """One cache update in one native call: compress ``key`` / ``value`` ``(B, H, S, D)`` into
    rows ``position ..`` of the code and norm buffers and, when ``k_out`` / ``v_out``
    ``(B, H, out_capacity, D)`` are given, write the de-quantised new tokens to their rows
    ``out_position ..`` (src/flashquant/cache/hf_cache.py:260-365).

    ``tables_*``: (Pi^T even columns, Pi^T odd columns, boundaries, centroids, Pi) on the device.
    """
    N.require_cuda(key, value, k_packed, k_norms, v_packed, v_norms, k_out, v_out)
    b, h, s, d = key.shape
    if value.shape != key.shape or value.dtype != key.dtype:
        raise ValueError("key and value must have the same shape and dtype")
    cap = k_packed.shape[2]
    for codes, norms in ((k_packed, k_norms), (v_packed, v_norms)):
        if codes.shape != (b, h, cap, d // 2) or norms.shape[:3] != (b, h, cap):
            raise ValueError("buffers must be (B, H, capacity, D/2) and (B, H, capacity, 1)")
        if not (codes.is_contiguous() and norms.is_contiguous()):
            raise ValueError("the cache buffers must be contiguous")
    out_cap = 0
    if k_out is not None:
        out_cap = k_out.shape[2]
        for o in (k_out, v_out):
            if o.shape != (b, h, out_cap, d) or o.dtype != key.dtype or not o.is_contiguous():
                raise ValueError("outputs must be contiguous (B, H, out_capacity, D) of key's dtype")
    dev = key.device
    key, value = _contig(key), _contig(value)
    ek, ok_, bnd, cent, rk = tables_k
    ev, ov, _, _, rv = tables_v
    lib = N.load()
    need = lib.fq_cache_update_workspace_bytes(b * h, s, d) if k_out is not None else 0
    if need and (workspace is None or workspace.numel() < need):
        raise ValueError(f"workspace of {need} bytes needed")
    N.check(lib.fq_cache_update(
        N.ptr(key), N.ptr(value), N.dtype_code(key.dtype), N.ptr(ek), N.ptr(ok_), N.ptr(rk),
        N.ptr(ev), N.ptr(ov), N.ptr(rv), N.ptr(bnd), bnd.numel(), N.ptr(cent), cent.numel(),
        N.ptr(k_packed), N.ptr(k_norms), N.ptr(v_packed), N.ptr(v_norms), b * h, s, cap,
        int(position), N.ptr(k_out), N.ptr(v_out), out_cap, int(out_position), d,
        N.ptr(workspace) if need else None, need, N.stream_ptr(dev)))


def pack_2bit(indices: torch.Tensor) -> torch.Tensor:
    """``(..., D)`` codes 0..3 -> ``(..., D/4)`` uint8, four per byte, first code in the top bits
    (csrc/core/packing.cpp:48-66 of the reference).  Raises on a code above 3, as it does."""
    N.require_cuda(indices)
    d = indices.shape[-1]
    if d % 4 != 0:
        raise ValueError(f"Last dimension must be divisible by 4 for 2-bit packing, got {d}")
    if indices.dtype != torch.uint8 and bool(((indices < 0) | (indices > 3)).any()):
        raise ValueError("indices out of range for 2-bit packing (0..3)")
    codes = _contig(indices.to(torch.uint8))
    n = codes.numel()
    pad = (-n) % 16
    flat = codes.reshape(-1)
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    packed = torch.empty((n + pad) // 4, dtype=torch.uint8, device=codes.device)
    bad = torch.zeros(1, dtype=torch.int32, device=codes.device)
    N.check(N.load().fq_pack_2bit(N.ptr(flat), N.ptr(packed), n + pad, N.ptr(bad),
                                  N.stream_ptr(codes.device)))
    if int(bad.item()):
        raise ValueError("indices out of range for 2-bit packing (0..3)")
    return packed[: n // 4].reshape(*indices.shape[:-1], d // 4)


def unpack_2bit(packed: torch.Tensor, dim: int) -> torch.Tensor:
    """``(..., dim/4)`` uint8 -> ``(..., dim)`` int64 codes (csrc/core/packing.cpp:68-79)."""
    N.require_cuda(packed)
    if packed.shape[-1] * 4 != dim:
        raise ValueError("dim must be four times the packed last dimension")
    p = _contig(packed).reshape(-1)
    n = p.numel() * 4
    pad = (-n) % 16
    if pad:
        p = torch.cat([p, p.new_zeros(pad // 4)])
    codes = torch.empty(n + pad, dtype=torch.uint8, device=p.device)
    N.check(N.load().fq_unpack_2bit(N.ptr(p), N.ptr(codes), n + pad, N.stream_ptr(p.device)))
    return codes[:n].reshape(*packed.shape[:-1], dim).long()


def tq_prod_quantize(x, rotation, boundaries, centroids, qjl_matrix):
    """Two-stage quantiser on ``(..., D)``: packed codes, norms, packed sign bits, gamma.

    Arithmetic of ``TurboQuantProd.quantize`` (src/flashquant/core/quantizer.py:270-304);
    the signs come back as bits (bit j%8 of byte j//8 set <=> sign_j = +1).
    """
    N.require_cuda(x)
    d = x.shape[-1]
    dev = x.device
    if qjl_matrix.shape != (d, d):
        raise ValueError("qjl_dim must equal head_dim")
    flat = _contig(x.reshape(-1, d))
    nv = flat.shape[0]
    rot, bnd = _f32(rotation, dev), _f32(boundaries, dev)
    cent, s = _f32(centroids, dev), _f32(qjl_matrix, dev)
    packed = torch.empty(nv, d // 2, dtype=torch.uint8, device=dev)
    norms = torch.empty(nv, dtype=torch.float32, device=dev)
    bits = torch.empty(nv, d // 8, dtype=torch.uint8, device=dev)
    gamma = torch.empty(nv, dtype=torch.float32, device=dev)
    lib = N.load()
    N.check(lib.fq_tq_prod_quantize(N.ptr(flat), N.dtype_code(flat.dtype), N.ptr(rot),
                                    N.ptr(bnd), bnd.numel(), N.ptr(cent), N.ptr(s),
                                    N.ptr(packed), N.ptr(norms), N.ptr(bits), N.ptr(gamma), nv, d,
                                    N.stream_ptr(dev)))
    lead = x.shape[:-1]
    return (packed.reshape(*lead, d // 2), norms.reshape(*lead, 1),
            bits.reshape(*lead, d // 8), gamma.reshape(*lead, 1))


# --------------------------------------------------------------------------------------
# compress-on-append into the paged cache
# --------------------------------------------------------------------------------------

def _append_common(key, value, kv_cache, slot_mapping):
    N.require_cuda(key, value, kv_cache, slot_mapping)
    n, h, d = key.shape
    if value.shape != key.shape or value.dtype != key.dtype:
        raise ValueError("key and value must have the same shape and dtype")
    if kv_cache.dtype != torch.uint8 or kv_cache.shape[-1] != h * (d + 8) or \
            not kv_cache.is_contiguous():
        raise ValueError("kv_cache must be contiguous uint8 (num_blocks, block_size, H*(D+8))")
    if slot_mapping.dtype not in (torch.int32, torch.int64):
        raise ValueError("slot_mapping must be int32 or int64")

    def strided(t):
        # a view whose token stride differs (e.g. a slice of a fused qkv tensor) is fine
        if t.stride(2) == 1 and t.stride(1) == d and t.stride(0) % 4 == 0:
            return t, t.stride(0)
        t = t.contiguous()
        return t, h * d

    key, ks = strided(key)
    value, vs = strided(value)
    if ks != vs:
        key, value, ks = key.contiguous(), value.contiguous(), h * d
    num_slots = kv_cache.shape[0] * kv_cache.shape[1]
    return key, value, ks, n, h, d, num_slots, _contig(slot_mapping)


def tq4_compress_append(key, value, kv_cache, slot_mapping, rotation, boundaries_k,
                        boundaries_v=None) -> None:
    """Compress K and V of new tokens and write their packed rows at ``slot_mapping``.

    One launch for what ``FlashQuantAttentionImpl._compress_and_store`` does with two
    compress calls, eight slice copies and an index_put (src/flashquant/vllm/impl.py:220-263).
    Negative slots are skipped.
    """
    key, value, stride, n, h, d, num_slots, slots = _append_common(key, value, kv_cache,
                                                                   slot_mapping)
    dev = key.device
    rot = _f32(rotation, dev)
    bk = _f32(boundaries_k, dev)
    bv = bk if boundaries_v is None else _f32(boundaries_v, dev)
    lib = N.load()
    N.check(lib.fq_tq4_compress_append(
        N.ptr(key), N.ptr(value), N.dtype_code(key.dtype), n, h, d, stride, N.ptr(rot),
        N.ptr(bk), bk.numel(), N.ptr(bv), bv.numel(), N.ptr(kv_cache), num_slots, N.ptr(slots),
        int(slots.dtype == torch.int64), N.stream_ptr(dev)))


def tq4_compress_append_qjl(key, value, kv_cache, kq_cache, slot_mapping, rotation,
                            boundaries_k, centroids_k, boundaries_v, qjl_matrix) -> None:
    """As ``tq4_compress_append`` with K through the two-stage quantiser.

    Sign bits and residual norm of every K vector go to the side plane ``kq_cache``
    ``(num_blocks, block_size, H*(D/8+4))`` = [sign bits | gamma], heads in order.
    """
    key, value, stride, n, h, d, num_slots, slots = _append_common(key, value, kv_cache,
                                                                   slot_mapping)
    dev = key.device
    if kq_cache.dtype != torch.uint8 or kq_cache.shape[-1] != h * (d // 8 + 4) or \
            not kq_cache.is_contiguous() or \
            kq_cache.shape[0] * kq_cache.shape[1] != num_slots:
        raise ValueError("kq_cache must be contiguous uint8 (num_blocks, block_size, H*(D/8+4))")
    if qjl_matrix.shape != (d, d):
        raise ValueError("qjl_dim must equal head_dim")
    rot, s = _f32(rotation, dev), _f32(qjl_matrix, dev)
    bk, ck, bv = _f32(boundaries_k, dev), _f32(centroids_k, dev), _f32(boundaries_v, dev)
    if ck.numel() != bk.numel() + 1:
        raise ValueError("centroids_k must have one entry more than boundaries_k")
    lib = N.load()
    N.check(lib.fq_tq4_compress_append_qjl(
        N.ptr(key), N.ptr(value), N.dtype_code(key.dtype), n, h, d, stride, N.ptr(rot),
        N.ptr(bk), bk.numel(), N.ptr(ck), N.ptr(bv), bv.numel(), N.ptr(s), N.ptr(kv_cache),
        N.ptr(kq_cache), num_slots, N.ptr(slots), int(slots.dtype == torch.int64),
        N.stream_ptr(dev)))


# --------------------------------------------------------------------------------------
# split-K paged decode
# --------------------------------------------------------------------------------------

_workspaces = {}


def decode_workspace(device, num_seqs: int, num_q_heads: int, num_kv_heads: int, head_dim: int,
                     num_splits: int, min_bytes: int = 0) -> torch.Tensor:
    """A zero-initialised, cached workspace tensor large enough for the given decode shape."""
    lib = N.load()
    need = max(min_bytes, lib.fq_paged_decode_workspace_bytes(num_seqs, num_q_heads, num_kv_heads,
                                                              head_dim, num_splits))
    # one workspace per (device, stream): calls on different streams may overlap on the GPU
    # and must not share counters or partial rows
    key = (device.type, device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def set_single_launch(enabled: bool) -> None:
    """``split_k_paged_decode`` as one cooperative launch (default) or as three ordinary launches
    (for a GPU shared with other work; the call also falls back by itself when the cooperative
    launch is refused)."""
    N.load().fq_paged_decode_set_single_launch(1 if enabled else 0)


def workspace_status(ws: torch.Tensor, reset: bool = False) -> int:
    """Device status word of a decode workspace (0 = no error); synchronises the stream.
    ``reset`` re-zeroes the head of the workspace when the word is non-zero, which the C ABI
    asks for before the workspace is used again (the counters the CTAs signal each other
    through are only left at zero by a call that completes)."""
    st = C.c_uint32(0)
    N.check(N.load().fq_workspace_status(N.ptr(ws), C.byref(st), N.stream_ptr(ws.device)))
    if st.value and reset:
        ws[:32768].zero_()
    return st.value


def _decode_args(q, kv_cache, block_table, seq_lens, centroids_k, centroids_v, rotation,
                 num_kv_heads, head_dim, block_size):
    N.require_cuda(q, kv_cache, block_table, seq_lens)
    dev = q.device
    num_seqs, hq, d = q.shape
    if d != head_dim:
        raise ValueError("q's last dimension must equal head_dim")
    if kv_cache.dtype != torch.uint8 or not kv_cache.is_contiguous() or \
            kv_cache.shape[1] != block_size or kv_cache.shape[2] != num_kv_heads * (d + 8):
        raise ValueError("kv_cache must be contiguous uint8 (num_blocks, block_size, H*(D+8))")
    if block_table.dtype != torch.int32 or seq_lens.dtype != torch.int32:
        raise ValueError("block_table and seq_lens must be int32")
    if block_table.stride(-1) != 1:
        block_table = block_table.contiguous()
    return (dev, num_seqs, hq, d, _contig(q), block_table, _contig(seq_lens),
            _f32(centroids_k, dev), _f32(centroids_v, dev), _f32(rotation, dev))


def split_k_paged_decode(
    q: torch.Tensor,
    kv_cache: torch.Tensor,
    block_table: torch.Tensor,
    seq_lens: torch.Tensor,
    centroids_k: torch.Tensor,
    centroids_v: torch.Tensor,
    rotation: torch.Tensor,
    num_kv_heads: int,
    head_dim: int,
    block_size: int,
    sm_scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
    num_splits: int = 0,
    workspace: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """Decode attention of one query token per sequence over the packed paged cache.

    Same contract as the reference's ``split_k_paged_decode``
    (src/flashquant/kernels/paged_decode.py:56-128): un-rotated ``q`` in, output in the
    original space, ``num_splits = 0`` picks the partition count.
    """
    dev, num_seqs, hq, d, q, block_table, seq_lens, ck, cv, rot = _decode_args(
        q, kv_cache, block_table, seq_lens, centroids_k, centroids_v, rotation, num_kv_heads,
        head_dim, block_size)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous tensor of q's shape and dtype")
    if workspace is None:
        workspace = decode_workspace(dev, num_seqs, hq, num_kv_heads, d, num_splits)
    lib = N.load()
    N.check(lib.fq_split_k_paged_decode(
        N.ptr(q), N.dtype_code(q.dtype), N.ptr(kv_cache), N.ptr(block_table),
        block_table.stride(0), N.ptr(seq_lens), N.ptr(ck), ck.numel(), N.ptr(cv), cv.numel(),
        N.ptr(rot), num_seqs, hq, num_kv_heads, d, block_size, kv_cache.shape[0],
        float(sm_scale), N.ptr(out), int(num_splits), N.ptr(workspace), workspace.numel(),
        N.stream_ptr(dev)))
    return out


def split_k_paged_decode_multi(q, kv_cache, block_table, seq_lens, centroids_k, centroids_v,
                               rotation, num_kv_heads, head_dim, block_size, sm_scale=None,
                               num_splits=0):
    """Decode attention of the LAST ``n_q`` tokens of every sequence (speculative / multi-token
    steps): ``q (num_seqs, n_q, H_q, D)``; ``seq_lens`` counts the new tokens, which are already
    in the cache; query ``i`` of a sequence sees keys ``0 .. seq_len - n_q + i``.

    The reference takes its fused decode only for a step of exactly one token
    (src/flashquant/vllm/impl.py:441) and otherwise de-quantises the whole cache for a causal
    varlen attention (impl.py:265-336, 477-509).  Here every (sequence, token) pair is a row of
    the paged decode kernel with its own length and the sequence's block-table row
    (``fq_split_k_paged_decode_multi``: a small kernel writes those rows, then the decode
    launch), so nothing is de-quantised to memory.
    """
    N.require_cuda(q, kv_cache, block_table, seq_lens)
    if q.dim() != 4:
        raise ValueError("q must be (num_seqs, n_q, H_q, D)")
    num_seqs, n_q, hq, d = q.shape
    out = torch.empty_like(q)
    if n_q == 0 or num_seqs == 0:
        return out
    dev, _, _, _, q3, block_table, seq_lens, ck, cv, rot = _decode_args(
        q.reshape(num_seqs * n_q, hq, d), kv_cache, block_table, seq_lens, centroids_k,
        centroids_v, rotation, num_kv_heads, head_dim, block_size)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    lib = N.load()
    need_ws = lib.fq_split_k_paged_decode_multi_workspace_bytes(num_seqs, n_q, hq, num_kv_heads, d,
                                                                int(num_splits))
    workspace = decode_workspace(dev, num_seqs * n_q, hq, num_kv_heads, d, num_splits,
                                 min_bytes=need_ws)
    max_blocks = block_table.shape[1]
    need = lib.fq_split_k_paged_decode_multi_scratch_bytes(num_seqs, n_q, max_blocks)
    scratch = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    N.check(lib.fq_split_k_paged_decode_multi(
        N.ptr(q3), N.dtype_code(q.dtype), N.ptr(kv_cache), N.ptr(block_table),
        block_table.stride(0), max_blocks, N.ptr(seq_lens), N.ptr(ck), ck.numel(), N.ptr(cv),
        cv.numel(), N.ptr(rot), num_seqs, n_q, hq, num_kv_heads, d, block_size, kv_cache.shape[0],
        float(sm_scale), N.ptr(out), int(num_splits), N.ptr(workspace), workspace.numel(),
        N.ptr(scratch), scratch.numel(), N.stream_ptr(dev)))
    return out


def split_k_paged_decode_qjl(q, kv_cache, kq_cache, block_table, seq_lens, centroids_k,
                             centroids_v, rotation, qjl_matrix, num_kv_heads, head_dim, block_size,
                             sm_scale=None, out=None, num_splits=0, workspace=None):
    """``split_k_paged_decode`` whose logits use the two-stage inner-product estimator
    (``TurboQuantProd.estimate_inner_product``, src/flashquant/core/quantizer.py:349-370):
    ``<q,k> ~ <q,k_mse> + gamma*sqrt(pi/2)/m*<S q, signs>`` with signs and gamma read from the
    side plane ``kq_cache`` that ``tq4_compress_append_qjl`` fills."""
    dev, num_seqs, hq, d, q, block_table, seq_lens, ck, cv, rot = _decode_args(
        q, kv_cache, block_table, seq_lens, centroids_k, centroids_v, rotation, num_kv_heads,
        head_dim, block_size)
    N.require_cuda(kq_cache)
    if kq_cache.dtype != torch.uint8 or not kq_cache.is_contiguous() or \
            tuple(kq_cache.shape) != (kv_cache.shape[0], block_size, num_kv_heads * (d // 8 + 4)):
        raise ValueError("kq_cache must be contiguous uint8 (num_blocks, block_size, H*(D/8+4))")
    if tuple(qjl_matrix.shape) != (d, d):
        raise ValueError("qjl_dim must equal head_dim")
    s_mat = _f32(qjl_matrix, dev)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    if out is None:
        out = torch.empty_like(q)
    elif out.shape != q.shape or out.dtype != q.dtype or not out.is_contiguous():
        raise ValueError("out must be a contiguous tensor of q's shape and dtype")
    if workspace is None:
        workspace = decode_workspace(dev, num_seqs, hq, num_kv_heads, d, num_splits)
    N.check(N.load().fq_split_k_paged_decode_qjl(
        N.ptr(q), N.dtype_code(q.dtype), N.ptr(kv_cache), N.ptr(kq_cache), N.ptr(block_table),
        block_table.stride(0), N.ptr(seq_lens), N.ptr(ck), ck.numel(), N.ptr(cv), cv.numel(),
        N.ptr(rot), N.ptr(s_mat), num_seqs, hq, num_kv_heads, d, block_size, kv_cache.shape[0],
        float(sm_scale), N.ptr(out), int(num_splits), N.ptr(workspace), workspace.numel(),
        N.stream_ptr(dev)))
    return out


def paged_tq4_prefill(q, kv_cache, block_table, seq_lens, cu_seqlens_q, max_q_len, centroids_k,
                      centroids_v, rotation, num_kv_heads, head_dim, block_size, sm_scale=None,
                      out=None, workspace=None) -> torch.Tensor:
    """Causal attention of prefill chunks over the paged TQ4 cache (``fq_paged_tq4_prefill``).

    ``q`` ``(total_q_tokens, H_q, D)``: the chunks of all sequences one after the other,
    ``cu_seqlens_q`` ``(num_seqs + 1)`` their bounds, ``seq_lens`` the keys of each sequence
    including its chunk (already appended to the cache).  What the reference's prefill path
    computes after de-quantising the whole cache (src/flashquant/vllm/impl.py:265-336,
    477-509); ``workspace`` word 0 is the device status word.
    """
    N.require_cuda(q, kv_cache, block_table, seq_lens, cu_seqlens_q)
    dev = q.device
    total, hq, d = q.shape
    if d != head_dim:
        raise ValueError(f"q has head_dim {d}, expected {head_dim}")
    num_seqs = seq_lens.numel()
    if cu_seqlens_q.numel() != num_seqs + 1:
        raise ValueError("cu_seqlens_q must have num_seqs + 1 entries")
    q = _contig(q)
    block_table = block_table if block_table.stride(-1) == 1 else block_table.contiguous()
    seq_lens, cu = _contig(seq_lens.to(torch.int32)), _contig(cu_seqlens_q.to(torch.int32))
    ck, cv, rot = _f32(centroids_k, dev), _f32(centroids_v, dev), _f32(rotation, dev)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    if out is None:
        out = torch.empty_like(q)
    lib = N.load()
    need = lib.fq_paged_tq4_prefill_workspace_bytes(total, hq, d)
    if workspace is None:
        workspace = torch.zeros(max(need, 256), dtype=torch.uint8, device=dev)
    N.check(lib.fq_paged_tq4_prefill(
        N.ptr(q), N.dtype_code(q.dtype), N.ptr(kv_cache), N.ptr(block_table),
        block_table.stride(0), N.ptr(seq_lens), N.ptr(cu), N.ptr(ck), ck.numel(), N.ptr(cv),
        cv.numel(), N.ptr(rot), num_seqs, total, int(max_q_len), hq, num_kv_heads, d, block_size,
        kv_cache.shape[0], float(sm_scale), N.ptr(out), N.ptr(workspace), workspace.numel(),
        N.stream_ptr(dev)))
    return out


class HostDecodeStep:
    """One decode step with host tensors in and out (``fq_decode_step_host``).

    The host-side form of ``FlashQuantAttentionImpl._fused_decode_path``
    (src/flashquant/vllm/impl.py:362-395): the step's new K/V token of every sequence is
    compressed into the paged cache, then the fused paged decode runs.  The object binds what
    does not change between steps (cache, constants, shapes, device scratch); ``__call__``
    takes the step's host tensors - pinned memory keeps the copies asynchronous - and returns
    after the result has landed in ``out_host``.
    """

    def __init__(self, kv_cache, kq_cache, rotation, boundaries_k, centroids_k, boundaries_v,
                 centroids_v, qjl_matrix, num_seqs, num_q_heads, num_kv_heads, head_dim,
                 block_size, block_table_stride, dtype=torch.bfloat16, sm_scale=None,
                 num_splits=0, slot_dtype=torch.int64):
        N.require_cuda(kv_cache)
        dev = kv_cache.device
        self.lib = N.load()
        self.dev = dev
        self.kv_cache, self.kq_cache = kv_cache, kq_cache
        if kq_cache is not None and qjl_matrix is None:
            raise ValueError("a QJL side plane needs the QJL matrix")
        self.consts = [_f32(t, dev) if t is not None else None for t in
                       (rotation, boundaries_k, centroids_k, boundaries_v, centroids_v, qjl_matrix)]
        self.shape = (num_seqs, num_q_heads, num_kv_heads, head_dim, block_size)
        self.bt_stride = int(block_table_stride)
        self.dtype = dtype
        self.slot_is_int64 = 1 if slot_dtype == torch.int64 else 0
        self.slot_dtype = slot_dtype
        self.sm_scale = float(sm_scale if sm_scale is not None else 1.0 / math.sqrt(head_dim))
        self.num_splits = int(num_splits)
        need = self.lib.fq_decode_step_host_staging_bytes(
            num_seqs, num_q_heads, num_kv_heads, head_dim, self.bt_stride, self.slot_is_int64)
        self.staging = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
        self.workspace = decode_workspace(dev, num_seqs, num_q_heads, num_kv_heads, head_dim,
                                          num_splits)
        self._block = None

    def host_block(self):
        """The page-locked block of the packed form and named views into it.

        Returns ``(block, views)``: ``views`` maps ``key, value, slot_mapping, seq_lens,
        block_table, q, out`` to tensors that alias the block at the offsets of
        ``fq_decode_step_offsets``.  Write a step's inputs into the views, call ``packed()``,
        read ``views["out"]``.
        """
        if self._block is None:
            num_seqs, hq, hkv, d, _ = self.shape
            off = (C.c_uint64 * 8)()
            N.check(self.lib.fq_decode_step_offsets(num_seqs, hq, hkv, d, self.bt_stride,
                                                    self.slot_is_int64, off))
            block = torch.zeros(max(int(off[7]), 256), dtype=torch.uint8).pin_memory()

            def view(at, shape, dt):
                n = int(torch.tensor(shape).prod()) * torch.empty(0, dtype=dt).element_size()
                return block[at:at + n].view(dt).view(shape)

            views = {
                "key": view(off[0], (num_seqs, hkv, d), self.dtype),
                "value": view(off[1], (num_seqs, hkv, d), self.dtype),
                "slot_mapping": view(off[2], (num_seqs,), self.slot_dtype),
                "seq_lens": view(off[3], (num_seqs,), torch.int32),
                "block_table": view(off[4], (num_seqs, self.bt_stride), torch.int32),
                "q": view(off[5], (num_seqs, hq, d), self.dtype),
                "out": view(off[6], (num_seqs, hq, d), self.dtype),
            }
            self._block = (block, views)
        return self._block

    def packed(self, overlap_copies=True, kv_cache=None, kq_cache=None):
        """One step from the block of ``host_block()`` (``fq_decode_step_host_packed``)."""
        block, views = self.host_block()
        num_seqs, hq, hkv, d, bs = self.shape
        kv_cache = self.kv_cache if kv_cache is None else kv_cache
        kq_cache = self.kq_cache if kq_cache is None else kq_cache
        rot, bk, ck, bv, cv, qjl = self.consts
        N.check(self.lib.fq_decode_step_host_packed(
            block.data_ptr(), views["out"].data_ptr(), 1 if overlap_copies else 0,
            N.dtype_code(self.dtype), self.slot_is_int64, self.bt_stride, N.ptr(kv_cache),
            N.ptr(kq_cache) if kq_cache is not None else None, N.ptr(rot), N.ptr(bk), bk.numel(),
            N.ptr(ck), ck.numel(), N.ptr(bv), bv.numel(), N.ptr(cv), cv.numel(),
            N.ptr(qjl) if qjl is not None else None, num_seqs, hq, hkv, d, bs, kv_cache.shape[0],
            self.sm_scale, self.num_splits, N.ptr(self.staging), self.staging.numel(),
            N.ptr(self.workspace), self.workspace.numel(), N.stream_ptr(self.dev)))
        return views["out"]

    def __call__(self, q_host, key_host, value_host, slot_mapping_host, block_table_host,
                 seq_lens_host, out_host, kv_cache=None, kq_cache=None):
        """``kv_cache`` / ``kq_cache`` override the bound cache for this step (same shapes)."""
        num_seqs, hq, hkv, d, bs = self.shape
        kv_cache = self.kv_cache if kv_cache is None else kv_cache
        kq_cache = self.kq_cache if kq_cache is None else kq_cache
        for t, shape, dt in ((q_host, (num_seqs, hq, d), self.dtype),
                             (out_host, (num_seqs, hq, d), self.dtype),
                             (key_host, (num_seqs, hkv, d), self.dtype),
                             (value_host, (num_seqs, hkv, d), self.dtype),
                             (slot_mapping_host, (num_seqs,), self.slot_dtype),
                             (block_table_host, (num_seqs, self.bt_stride), torch.int32),
                             (seq_lens_host, (num_seqs,), torch.int32)):
            if t.device.type != "cpu" or tuple(t.shape) != shape or t.dtype != dt or \
                    not t.is_contiguous():
                raise ValueError(f"host tensor of shape {tuple(t.shape)} / {t.dtype}: expected "
                                 f"contiguous CPU {shape} / {dt}")
        rot, bk, ck, bv, cv, qjl = self.consts
        N.check(self.lib.fq_decode_step_host(
            q_host.data_ptr(), key_host.data_ptr(), value_host.data_ptr(),
            N.dtype_code(self.dtype), slot_mapping_host.data_ptr(), self.slot_is_int64,
            block_table_host.data_ptr(), self.bt_stride, seq_lens_host.data_ptr(),
            N.ptr(kv_cache), N.ptr(kq_cache) if kq_cache is not None else None,
            N.ptr(rot), N.ptr(bk), bk.numel(), N.ptr(ck), ck.numel(), N.ptr(bv), bv.numel(),
            N.ptr(cv), cv.numel(), N.ptr(qjl) if qjl is not None else None, num_seqs, hq, hkv, d,
            bs, kv_cache.shape[0], self.sm_scale, self.num_splits, out_host.data_ptr(),
            N.ptr(self.staging),
            self.staging.numel(), N.ptr(self.workspace), self.workspace.numel(),
            N.stream_ptr(self.dev)))
        return out_host


def paged_decode_partials(q, kv_cache, block_table, seq_lens, centroids_k, centroids_v, rotation,
                          num_kv_heads, head_dim, block_size, num_splits=0, sm_scale=None,
                          partials=None, workspace=None) -> torch.Tensor:
    """One un-normalised (acc, m, l) row per sequence and query head: ``(num_seqs, H_q, D+4)``
    fp32.  This is what a GPU contributes when the tokens of a sequence are spread over
    several GPUs; ``split_k_merge`` combines the rows of all GPUs."""
    dev, num_seqs, hq, d, q, block_table, seq_lens, ck, cv, rot = _decode_args(
        q, kv_cache, block_table, seq_lens, centroids_k, centroids_v, rotation, num_kv_heads,
        head_dim, block_size)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(head_dim)
    if partials is None:
        partials = torch.empty(num_seqs, hq, d + _PART_PAD, dtype=torch.float32, device=dev)
    if workspace is None:
        workspace = decode_workspace(dev, num_seqs, hq, num_kv_heads, d, num_splits)
    lib = N.load()
    N.check(lib.fq_paged_decode_partials(
        N.ptr(q), N.dtype_code(q.dtype), N.ptr(kv_cache), N.ptr(block_table),
        block_table.stride(0), N.ptr(seq_lens), N.ptr(ck), ck.numel(), N.ptr(cv), cv.numel(),
        N.ptr(rot), num_seqs, hq, num_kv_heads, d, block_size, kv_cache.shape[0],
        float(sm_scale), int(num_splits), N.ptr(partials), N.ptr(workspace), workspace.numel(),
        N.stream_ptr(dev)))
    return partials


def split_k_merge(partials: torch.Tensor, rotation: torch.Tensor, dtype: torch.dtype,
                  out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Merge ``(n_groups, num_seqs, H_q, D+4)`` partial rows, round, rotate back."""
    N.require_cuda(partials)
    if partials.dim() == 3:
        partials = partials.unsqueeze(0)
    ng, num_seqs, hq, dp = partials.shape
    d = dp - _PART_PAD
    dev = partials.device
    partials = _contig(partials)
    rot = _f32(rotation, dev)
    if out is None:
        out = torch.empty(num_seqs, hq, d, dtype=dtype, device=dev)
    lib = N.load()
    N.check(lib.fq_split_k_merge(N.ptr(partials), ng, N.ptr(rot), num_seqs, hq, d, N.ptr(out),
                                 N.dtype_code(dtype), N.stream_ptr(dev)))
    return out


# --------------------------------------------------------------------------------------
# fused TQ4 attention (prefill)
# --------------------------------------------------------------------------------------

_attn_workspaces = {}


def fused_tq_attention(
    q: torch.Tensor,
    k_packed: torch.Tensor,
    k_norms: torch.Tensor,
    v_packed: torch.Tensor,
    v_norms: torch.Tensor,
    centroids_k: torch.Tensor,
    centroids_v: torch.Tensor,
    rotation: torch.Tensor,
    sm_scale: Optional[float] = None,
    is_causal: bool = False,
) -> torch.Tensor:
    """Attention over contiguous compressed K and V; un-rotated ``q`` in, original space out.

    Same contract as the reference's ``fused_tq_attention``
    (src/flashquant/kernels/attention.py:53-107): ``q (B, H_Q, N_Q, D)``, packed codes
    ``(B, H_KV, N_KV, D/2)``, norms ``(B, H_KV, N_KV, 1)``.
    """
    N.require_cuda(q, k_packed, k_norms, v_packed, v_norms)
    b, hq, nq, d = q.shape
    _, hkv, nkv, half = k_packed.shape
    if half * 2 != d or v_packed.shape != k_packed.shape:
        raise ValueError("packed K/V must be (B, H_KV, N_KV, D/2)")
    dev = q.device
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    q = _contig(q)
    kp, vp = _contig(k_packed), _contig(v_packed)
    kn = _contig(k_norms.reshape(b, hkv, nkv).float())
    vn = _contig(v_norms.reshape(b, hkv, nkv).float())
    ck, cv, rot = _f32(centroids_k, dev), _f32(centroids_v, dev), _f32(rotation, dev)
    out = torch.empty_like(q)
    lib = N.load()
    need = lib.fq_fused_tq_attention_workspace_bytes(b, hq, nq, d)
    key = (dev.type, dev.index)
    ws = _attn_workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=dev)
        _attn_workspaces[key] = ws
    N.check(lib.fq_fused_tq_attention(
        N.ptr(q), N.dtype_code(q.dtype), N.ptr(kp), N.ptr(kn), N.ptr(vp), N.ptr(vn), N.ptr(ck),
        ck.numel(), N.ptr(cv), cv.numel(), N.ptr(rot), b, hq, hkv, nq, nkv, d, float(sm_scale),
        int(bool(is_causal)), N.ptr(out), N.ptr(ws), ws.numel(), N.stream_ptr(dev)))
    return out


def _buffer_view_capacity(codes: torch.Tensor, norms: torch.Tensor) -> int:
    """Tokens per (batch, head) row of the buffers that ``codes`` / ``norms`` are views of."""
    b, h, n, half = codes.shape
    if n == 0:
        return 0
    if codes.stride(3) != 1 or codes.stride(2) != half or codes.stride(1) % half:
        raise ValueError("packed codes must be a [:, :, :n] view of a contiguous buffer")
    cap = codes.stride(1) // half
    if b > 1 and codes.stride(0) != h * codes.stride(1):
        raise ValueError("packed codes must be a [:, :, :n] view of a contiguous buffer")
    nn = norms.reshape(b, h, n) if norms.dim() == 4 else norms
    if nn.stride(2) != 1 or nn.stride(1) != cap or (b > 1 and nn.stride(0) != h * cap):
        raise ValueError("norms must be a view of a buffer with the capacity of the codes")
    return cap


def fused_tq_attention_kv(
    q: torch.Tensor,
    k_packed: torch.Tensor,
    k_norms: torch.Tensor,
    v_packed: torch.Tensor,
    v_norms: torch.Tensor,
    centroids_k: torch.Tensor,
    centroids_v: torch.Tensor,
    rotation_k: torch.Tensor,
    rotation_v: torch.Tensor,
    sm_scale: Optional[float] = None,
    is_causal: bool = False,
) -> torch.Tensor:
    """``fused_tq_attention`` over the views a compressed cache hands out, read in place.

    ``k_packed`` .. ``v_norms`` are what ``CompressedDynamicCache.get_compressed`` returns
    (src/flashquant/cache/hf_cache.py:387-414): ``[:, :, :n_kv]`` views of buffers with room
    for more tokens; keys and values carry their own rotation (seeds 42 / 43).
    """
    N.require_cuda(q, k_packed, k_norms, v_packed, v_norms)
    b, hq, nq, d = q.shape
    _, hkv, nkv, half = k_packed.shape
    if half * 2 != d or v_packed.shape != k_packed.shape:
        raise ValueError("packed K/V must be (B, H_KV, N_KV, D/2)")
    if k_norms.dtype != torch.float32 or v_norms.dtype != torch.float32:
        raise ValueError("norms must be fp32")
    cap = _buffer_view_capacity(k_packed, k_norms)
    if _buffer_view_capacity(v_packed, v_norms) != cap:
        raise ValueError("K and V buffers must have the same capacity")
    dev = q.device
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(d)
    q = _contig(q)
    ck, cv = _f32(centroids_k, dev), _f32(centroids_v, dev)
    rk, rv = _f32(rotation_k, dev), _f32(rotation_v, dev)
    out = torch.empty_like(q)
    lib = N.load()
    need = lib.fq_fused_tq_attention_workspace_bytes(b, hq, nq, d)
    key = (dev.type, dev.index)
    ws = _attn_workspaces.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=dev)
        _attn_workspaces[key] = ws
    N.check(lib.fq_fused_tq_attention_kv(
        N.ptr(q), N.dtype_code(q.dtype), N.ptr(k_packed), N.ptr(k_norms), N.ptr(v_packed),
        N.ptr(v_norms), N.ptr(ck), ck.numel(), N.ptr(cv), cv.numel(), N.ptr(rk), N.ptr(rv), b, hq,
        hkv, nq, nkv, cap, d, float(sm_scale), int(bool(is_causal)), N.ptr(out), N.ptr(ws),
        ws.numel(), N.stream_ptr(dev)))
    return out


def attention_workspace_status(device) -> int:
    """Device status word of the cached attention workspace (0 = no error)."""
    ws = _attn_workspaces.get((device.type, device.index))
    return 0 if ws is None else workspace_status(ws)
