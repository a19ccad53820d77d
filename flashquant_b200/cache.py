"""Compressed KV cache behind the interface of HuggingFace's ``DynamicCache``.

Mirror of the reference's ``CompressedBuffer`` (src/flashquant/cache/buffer_pool.py:21-134)
and ``CompressedDynamicCache`` (src/flashquant/cache/hf_cache.py:69-582): same class and
method names, arguments and errors, with the arithmetic on the CUDA kernels of this package:

* an update compresses the new keys and values straight into their final rows of the
  pre-allocated buffers (one launch per tensor instead of compress + pack + two slice copies);
* a read of the new tokens (``_dequantize_tensor``) is one decompress plus one tensor-core
  back-rotation, and the running decompressed tensors grow by doubling instead of ``torch.cat``;
* ``fused_attention`` runs the fused TQ4 attention over the buffers in place, with the key and
  the value rotation.

Every tensor must live on a CUDA device; there is no CPU path here.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

import torch

from . import _native as N
from . import kernels as K
from .quantizer import TurboQuantMSE


class FlashQuantError(Exception):
    """Base of the package's errors (src/flashquant/errors.py:25-26)."""


class FlashQuantCacheError(FlashQuantError):
    """Cache lifecycle errors: double wrap, unknown layer (src/flashquant/errors.py:56-66)."""


class CompressedBuffer:
    """Pre-allocated codes ``(batch, heads, max_seq, half_dim)`` and fp32 norms
    ``(batch, heads, max_seq, 1)`` with O(1) append and zero-copy ``get()``.

    Interface of the reference class (src/flashquant/cache/buffer_pool.py:21-134).
    ``reserve`` is the addition the compress kernel uses: it claims the rows and hands back the
    position, and the kernel writes them in place.
    """

    def __init__(self, max_seq: int, batch: int, heads: int, half_dim: int, dtype: torch.dtype,
                 device: torch.device) -> None:
        self.max_seq = max_seq
        self.batch = batch
        self.heads = heads
        self.half_dim = half_dim
        self._indices = torch.empty(batch, heads, max_seq, half_dim, dtype=dtype, device=device)
        self._norms = torch.empty(batch, heads, max_seq, 1, dtype=torch.float32, device=device)
        self._len = 0

    def reserve(self, new_tokens: int) -> int:
        """Claim ``new_tokens`` rows; return the position of the first one."""
        end = self._len + new_tokens
        if end > self.max_seq:
            raise RuntimeError(
                f"CompressedBuffer overflow: appending {new_tokens} tokens "
                f"at position {self._len} would exceed max_seq={self.max_seq}. "
                f"Increase FlashQuantConfig.max_seq_len."
            )
        pos = self._len
        self._len = end
        return pos

    def append(self, indices: torch.Tensor, norms: torch.Tensor) -> None:
        """Write already compressed tokens at the current position (buffer_pool.py:86-110)."""
        new_tokens = indices.shape[2]
        pos = self.reserve(new_tokens)
        self._indices[:, :, pos:pos + new_tokens, :] = indices
        self._norms[:, :, pos:pos + new_tokens, :] = norms

    def get(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Zero-copy views of the valid part: ``(B, H, length, half_dim)``, ``(B, H, length, 1)``."""
        return self._indices[:, :, :self._len, :], self._norms[:, :, :self._len, :]

    @property
    def length(self) -> int:
        return self._len

    def reset(self) -> None:
        self._len = 0


class _GrowingTensor:
    """``(B, H, length, D)`` tensor that grows along the token axis by doubling its storage."""

    def __init__(self, batch: int, heads: int, dim: int, dtype: torch.dtype,
                 device: torch.device, first: int) -> None:
        self._cap = max(16, 2 * first)
        self._buf = torch.empty(batch, heads, self._cap, dim, dtype=dtype, device=device)
        self._len = 0

    def reserve(self, new_tokens: int) -> int:
        """Make room for ``new_tokens`` more rows; return the position of the first one."""
        if self._len + new_tokens > self._cap:
            cap = max(2 * self._cap, self._len + new_tokens)
            buf = torch.empty(*self._buf.shape[:2], cap, self._buf.shape[3], dtype=self._buf.dtype,
                              device=self._buf.device)
            buf[:, :, :self._len] = self._buf[:, :, :self._len]
            self._buf, self._cap = buf, cap
        pos = self._len
        self._len += new_tokens
        return pos

    def storage(self) -> torch.Tensor:
        return self._buf

    def view(self) -> torch.Tensor:
        return self._buf[:, :, :self._len]


class ValueCompressor:
    """Stage-1 quantiser of one tensor kind with its tables resident on the device
    (src/flashquant/core/compressor.py:200-262)."""

    def __init__(self, head_dim: int, bits: int = 4, *, seed: int = 43) -> None:
        self.head_dim = head_dim
        self.bits = bits
        self.quantizer = TurboQuantMSE(head_dim, bits, seed=seed)
        self._tables: Dict[Tuple[str, Optional[int]], Tuple[torch.Tensor, ...]] = {}

    def tables(self, device: torch.device):
        """(Pi^T even columns, Pi^T odd columns, boundaries, centroids, Pi) on ``device``."""
        key = (device.type, device.index)
        t = self._tables.get(key)
        if t is None:
            q = self.quantizer
            rt = q.rotation.to(device).T.contiguous()
            t = (rt[:, 0::2].contiguous(), rt[:, 1::2].contiguous(), q.boundaries.to(device),
                 q.centroids.to(device), q.rotation.to(device).contiguous())
            self._tables[key] = t
        return t


@dataclass
class _CompressedLayer:
    buffer: CompressedBuffer
    packed: bool = True


class CompressedDynamicCache:
    """Wraps a ``DynamicCache``-like object: ``cache.update`` compresses the new tokens into
    pre-allocated buffers and returns the de-quantised keys and values seen so far.

    Interface of the reference class (src/flashquant/cache/hf_cache.py:69-582); keys use the
    rotation of ``key_seed``, values that of ``value_seed``.  Codes are always stored
    nibble-packed (two per byte), also below 4 bits, because that is what the kernels read.
    """

    def __init__(self, cache: Any, head_dim: int, bits: int = 4, *, key_seed: int = 42,
                 value_seed: int = 43, max_seq_len: int = 32768) -> None:
        if bits == 4 and head_dim % 2 != 0:
            raise ValueError(
                f"bits=4 requires even head_dim for nibble packing, got {head_dim}")
        if not 1 <= bits <= 4:
            raise ValueError(f"bits={bits}: the kernels store codes of at most 4 bits")
        if head_dim not in (64, 128):
            raise ValueError(f"head_dim={head_dim}: the kernels are built for 64 and 128")
        self.cache = cache
        self.head_dim = head_dim
        self.bits = bits
        self._nibble_packed = True
        self.enabled = True
        self.fused_mode = False
        self._max_seq_len = max_seq_len
        self.key_compressor = ValueCompressor(head_dim, bits, seed=key_seed)
        self.value_compressor = ValueCompressor(head_dim, bits, seed=value_seed)
        self._compressed_keys: List[Optional[_CompressedLayer]] = []
        self._compressed_values: List[Optional[_CompressedLayer]] = []
        self._decompressed_k: List[Optional[_GrowingTensor]] = []
        self._decompressed_v: List[Optional[_GrowingTensor]] = []
        self._original_dtype: torch.dtype = torch.bfloat16
        self._workspace: Optional[torch.Tensor] = None
        if getattr(cache, "_flashquant_wrapped", False):
            raise FlashQuantCacheError(
                "Cache is already wrapped by FlashQuant. "
                "Call restore() on the existing wrapper first.")
        cache._flashquant_wrapped = True
        self._original_update = cache.update
        self._original_get_seq_length = cache.get_seq_length
        cache.update = self._compressed_update
        cache.get_seq_length = self._compressed_get_seq_length

    # ----- compression helpers -----

    def _compress_tensor(self, compressor: ValueCompressor,
                         tensor: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """``(B, H, S, D)`` -> (packed uint8 ``(B, H, S, D/2)``, fp32 norms ``(B, H, S, 1)``)
        (hf_cache.py:170-194)."""
        b, h, s, d = tensor.shape
        even, odd, bnd, _, rot = compressor.tables(tensor.device)
        packed, norms = K.tq4_compress(tensor.reshape(b * h * s, 1, d), rot, bnd,
                                       rotation_T_even=even, rotation_T_odd=odd)
        return packed.reshape(b, h, s, d // 2), norms.reshape(b, h, s, 1)

    def _dequantize_tensor(self, compressor: ValueCompressor, indices: torch.Tensor,
                           norms: torch.Tensor) -> torch.Tensor:
        """Packed codes + norms -> the original space, in the model dtype (hf_cache.py:196-219)."""
        _, _, _, cent, rot = compressor.tables(indices.device)
        return K.tq4_decompress_original(indices, norms, cent, rot, dtype=self._original_dtype)

    def _ensure_layer(self, layer_idx: int) -> None:
        while len(self._compressed_keys) <= layer_idx:
            self._compressed_keys.append(None)
            self._compressed_values.append(None)
            self._decompressed_k.append(None)
            self._decompressed_v.append(None)

    def _get_or_create_buffer(self, layer_idx: int, is_key: bool, batch: int, heads: int,
                              half_dim: int, dtype: torch.dtype,
                              device: torch.device) -> _CompressedLayer:
        storage = self._compressed_keys if is_key else self._compressed_values
        layer = storage[layer_idx]
        if layer is None:
            layer = _CompressedLayer(
                buffer=CompressedBuffer(max_seq=self._max_seq_len, batch=batch, heads=heads,
                                        half_dim=half_dim, dtype=dtype, device=device),
                packed=True)
            storage[layer_idx] = layer
        return layer

    # ----- patched methods -----

    def _compressed_update(self, key_states: torch.Tensor, value_states: torch.Tensor,
                           layer_idx: int, cache_kwargs: Optional[Dict[str, Any]] = None
                           ) -> Tuple[torch.Tensor, torch.Tensor]:
        """Compress the new tokens; return all keys and values of the layer, de-quantised
        (hf_cache.py:260-365).  In ``fused_mode`` nothing is de-quantised and the new tokens
        are handed back as they came."""
        if not self.enabled:
            return self._original_update(key_states, value_states, layer_idx, cache_kwargs)
        N.require_cuda(key_states, value_states)
        if value_states.shape != key_states.shape or value_states.dtype != key_states.dtype:
            raise ValueError("key_states and value_states must have the same shape and dtype")
        grown = self._decompressed_k[layer_idx] if layer_idx < len(self._decompressed_k) else None
        if grown is not None and not self.fused_mode and grown.storage().dtype != key_states.dtype:
            raise ValueError(f"layer {layer_idx} was filled with {grown.storage().dtype} tensors")
        self._original_dtype = key_states.dtype
        self._ensure_layer(layer_idx)
        batch, heads, new_seq, dim = key_states.shape
        half_dim = dim // 2
        k_layer = self._get_or_create_buffer(layer_idx, True, batch, heads, half_dim, torch.uint8,
                                             key_states.device)
        v_layer = self._get_or_create_buffer(layer_idx, False, batch, heads, half_dim,
                                             torch.uint8, value_states.device)
        kb, vb = k_layer.buffer, v_layer.buffer
        if kb.length + new_seq > kb.max_seq or vb.length + new_seq > vb.max_seq:
            kb.reserve(new_seq)  # raises the overflow error; nothing has been claimed yet
            vb.reserve(new_seq)
        tables_k = self.key_compressor.tables(key_states.device)
        tables_v = self.value_compressor.tables(key_states.device)

        if getattr(self.cache, "layer_class_to_replicate", None) is not None:
            while len(self.cache.layers) <= layer_idx:
                self.cache.layers.append(self.cache.layer_class_to_replicate())

        if self.fused_mode:
            pos = kb.reserve(new_seq)
            vb.reserve(new_seq)
            K.cache_update(key_states, value_states, tables_k, tables_v, kb._indices, kb._norms,
                           vb._indices, vb._norms, pos)
            layer = self.cache.layers[layer_idx]
            if hasattr(layer, "is_initialized") and not layer.is_initialized:
                layer.lazy_initialization(key_states)
            layer.keys = key_states
            layer.values = value_states
            return key_states, value_states

        # only the NEW tokens are de-quantised, straight into the rows behind the earlier ones
        if self._decompressed_k[layer_idx] is None:
            self._decompressed_k[layer_idx] = _GrowingTensor(
                batch, heads, dim, key_states.dtype, key_states.device, new_seq)
            self._decompressed_v[layer_idx] = _GrowingTensor(
                batch, heads, dim, key_states.dtype, key_states.device, new_seq)
        grown_k, grown_v = self._decompressed_k[layer_idx], self._decompressed_v[layer_idx]
        pos = kb.reserve(new_seq)
        vb.reserve(new_seq)
        out_pos = grown_k.reserve(new_seq)
        grown_v.reserve(new_seq)
        need = batch * heads * new_seq * dim * 4
        if self._workspace is None or self._workspace.numel() < need or \
                self._workspace.device != key_states.device:
            self._workspace = torch.empty(max(need, 1 << 16), dtype=torch.uint8,
                                          device=key_states.device)
        K.cache_update(key_states, value_states, tables_k, tables_v, kb._indices, kb._norms,
                       vb._indices, vb._norms, pos, grown_k.storage(), grown_v.storage(), out_pos,
                       self._workspace)
        decompressed_k = grown_k.view()
        decompressed_v = grown_v.view()

        if hasattr(self.cache, "layers") and layer_idx < len(self.cache.layers):
            layer = self.cache.layers[layer_idx]
            if hasattr(layer, "is_initialized") and not layer.is_initialized:
                layer.lazy_initialization(key_states)
            if hasattr(layer, "keys"):
                layer.keys = decompressed_k
                layer.values = decompressed_v
        return decompressed_k, decompressed_v

    def _compressed_get_seq_length(self, layer_idx: int = 0) -> int:
        if not self.enabled:
            return self._original_get_seq_length(layer_idx)
        if layer_idx >= len(self._compressed_keys):
            return 0
        k_layer = self._compressed_keys[layer_idx]
        return 0 if k_layer is None else k_layer.buffer.length

    # ----- fused kernel API -----

    def get_compressed(self, layer_idx: int
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        """``(k_packed, k_norms, v_packed, v_norms)`` views of the layer (hf_cache.py:387-414)."""
        if layer_idx >= len(self._compressed_keys):
            raise FlashQuantCacheError(f"Layer {layer_idx} has not been initialized")
        k_layer = self._compressed_keys[layer_idx]
        v_layer = self._compressed_values[layer_idx]
        if k_layer is None or v_layer is None:
            raise FlashQuantCacheError(f"Layer {layer_idx} has not been initialized")
        k_indices, k_norms = k_layer.buffer.get()
        v_indices, v_norms = v_layer.buffer.get()
        return k_indices, k_norms, v_indices, v_norms

    def fused_attention(self, query: torch.Tensor, layer_idx: int,
                        sm_scale: Optional[float] = None, is_causal: bool = False) -> torch.Tensor:
        """Attention of ``query (B, H_Q, N_Q, D)`` over the compressed layer, read in place."""
        kp, kn, vp, vn = self.get_compressed(layer_idx)
        tk = self.key_compressor.tables(query.device)
        tv = self.value_compressor.tables(query.device)
        return K.fused_tq_attention_kv(query, kp, kn, vp, vn, tk[3], tv[3], tk[4], tv[4],
                                       sm_scale=sm_scale, is_causal=is_causal)

    # ----- properties -----

    @property
    def rotation_k(self) -> torch.Tensor:
        return self.key_compressor.quantizer.rotation

    @property
    def rotation_v(self) -> torch.Tensor:
        return self.value_compressor.quantizer.rotation

    @property
    def centroids_k(self) -> torch.Tensor:
        return self.key_compressor.quantizer.centroids

    @property
    def centroids_v(self) -> torch.Tensor:
        return self.value_compressor.quantizer.centroids

    # ----- VRAM accounting -----

    def compressed_vram_bytes(self) -> int:
        """Bytes of the valid codes and norms over all layers (hf_cache.py:472-491)."""
        total = 0
        for k_layer, v_layer in zip(self._compressed_keys, self._compressed_values):
            for layer in (k_layer, v_layer):
                if layer is None:
                    continue
                idx, norms = layer.buffer.get()
                total += idx.nelement() * idx.element_size()
                total += norms.nelement() * norms.element_size()
        return total

    def vram_bytes(self) -> int:
        """Compressed storage plus the de-quantised running tensors (hf_cache.py:439-470)."""
        total = self.compressed_vram_bytes()
        for grown in list(self._decompressed_k) + list(self._decompressed_v):
            if grown is not None:
                t = grown.view()
                total += t.nelement() * t.element_size()
        return total

    def baseline_vram_bytes(self) -> int:
        """Bytes the same tokens would take as fp16 tensors (hf_cache.py:493-512)."""
        total = 0
        for k_layer, v_layer in zip(self._compressed_keys, self._compressed_values):
            for layer in (k_layer, v_layer):
                if layer is None:
                    continue
                idx, _ = layer.buffer.get()
                b, h, s, d = idx.shape
                total += b * h * s * (2 * d) * 2
        return total

    def compression_stats(self) -> Dict[str, Any]:
        """Sizes and ratio for reporting (hf_cache.py:514-551)."""
        num_layers = sum(1 for k in self._compressed_keys if k is not None)
        if num_layers == 0:
            return {}
        compressed_bytes = self.compressed_vram_bytes()
        baseline_bytes = self.baseline_vram_bytes()
        ratio = baseline_bytes / compressed_bytes if compressed_bytes > 0 else 0.0
        first_k = next(k for k in self._compressed_keys if k is not None)
        idx, _ = first_k.buffer.get()
        b, h, s, _ = idx.shape
        mib = 1024 * 1024
        return {
            "num_layers": num_layers,
            "seq_len": s,
            "batch_size": b,
            "num_heads": h,
            "head_dim": self.head_dim,
            "bits": self.bits,
            "nibble_packed": self._nibble_packed,
            "compressed_mib": compressed_bytes / mib,
            "baseline_mib": baseline_bytes / mib,
            "total_vram_mib": self.vram_bytes() / mib,
            "compression_ratio": round(ratio, 2),
            "savings_mib": (baseline_bytes - compressed_bytes) / mib,
        }

    # ----- lifecycle -----

    def disable(self) -> None:
        self.enabled = False

    def enable(self) -> None:
        self.enabled = True

    def restore(self) -> None:
        """Put the wrapped cache's own methods back (hf_cache.py:565-574)."""
        self.cache.update = self._original_update
        self.cache.get_seq_length = self._original_get_seq_length
        if hasattr(self.cache, "_flashquant_wrapped"):
            self.cache._flashquant_wrapped = False

    def __enter__(self) -> "CompressedDynamicCache":
        return self

    def __exit__(self, *exc: object) -> bool:
        self.restore()
        return False
