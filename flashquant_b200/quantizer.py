"""Host-side quantiser objects: constants on the host, arithmetic on the GPU.

``TurboQuantMSE`` and ``TurboQuantProd`` keep the constructor and method names of the
reference classes (src/flashquant/core/quantizer.py:93-370).  The constants (Lloyd-Max
tables, Haar rotation, QJL matrix) are computed once on the host with the same torch CPU
calls the reference uses, because they depend on torch's CPU generator and on LAPACK's QR;
``quantize`` / ``dequantize`` run the CUDA kernels and accept CUDA tensors only.
"""

from __future__ import annotations

import math
from functools import lru_cache
from typing import Tuple

import torch

from . import kernels as K


@lru_cache(maxsize=32)
def lloyd_max_codebook(dim: int, bits: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(centroids, boundaries) fp32 for N(0, 1/dim), support +-3.5 sigma.

    Iteration of the reference (src/flashquant/core/codebook.py:58-140): fp64, uniform start,
    centroid = conditional mean of its cell, boundaries = midpoints, at most 200 sweeps,
    stop below a shift of 1e-10.
    """
    levels = 1 << bits
    sigma = 1.0 / math.sqrt(dim)
    lo, hi = -3.5 * sigma, 3.5 * sigma
    cent = torch.tensor([lo + (hi - lo) * (i + 0.5) / levels for i in range(levels)],
                        dtype=torch.float64)
    k_pdf = 1.0 / (sigma * math.sqrt(2.0 * math.pi))
    inv_s = 1.0 / sigma
    inv_s2 = inv_s / math.sqrt(2.0)
    ends = (torch.tensor([lo], dtype=torch.float64), torch.tensor([hi], dtype=torch.float64))
    for _ in range(200):
        edges = torch.cat([ends[0], (cent[:-1] + cent[1:]) / 2.0, ends[1]])
        pdf = k_pdf * torch.exp(-0.5 * (edges * inv_s) ** 2)
        cdf = 0.5 * (1.0 + torch.erf(edges * inv_s2))
        mass = cdf[1:] - cdf[:-1]
        ok = mass > 1e-15
        mean = (sigma ** 2) * (pdf[:-1] - pdf[1:]) / torch.where(ok, mass, torch.ones_like(mass))
        new = torch.where(ok, mean, (edges[:-1] + edges[1:]) / 2.0)
        moved = (new - cent).abs().max().item()
        cent = new
        if moved < 1e-10:
            break
    return cent.float(), ((cent[:-1] + cent[1:]) / 2.0).float()


def haar_orthogonal(dim: int, seed: int = 42) -> torch.Tensor:
    """Seeded Haar-random orthogonal matrix, fp32 on the CPU
    (src/flashquant/core/quantizer.py:60-85).  LAPACK's QR is not bit-reproducible across
    thread counts, so a matrix generated once must be reused, not regenerated, wherever
    codes have to match."""
    gen = torch.Generator(device="cpu").manual_seed(seed)
    q, r = torch.linalg.qr(torch.randn(dim, dim, generator=gen, device="cpu", dtype=torch.float32))
    sgn = torch.sign(torch.diag(r))
    sgn[sgn == 0] = 1.0
    return q * sgn.unsqueeze(0)


class TurboQuantMSE:
    """Rotation + Lloyd-Max scalar quantiser (stage 1)."""

    def __init__(self, dim: int, bits: int, *, seed: int = 42) -> None:
        self.dim = dim
        self.bits = bits
        self.centroids, self.boundaries = lloyd_max_codebook(dim, bits)
        self.rotation = haar_orthogonal(dim, seed=seed)

    def quantize(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """CUDA ``(..., dim)`` -> (indices int64 ``(..., dim)``, norms fp32 ``(..., 1)``)."""
        lead = x.shape[:-1]
        packed, norms = K.tq4_compress(x.reshape(-1, 1, self.dim), self.rotation, self.boundaries)
        idx = torch.stack([packed >> 4, packed & 0x0F], dim=-1).flatten(-2).long()
        return idx.reshape(*lead, self.dim), norms.reshape(*lead, 1)

    def dequantize(self, indices: torch.Tensor, norms: torch.Tensor) -> torch.Tensor:
        """(c[idx] Pi) * norm in the original space, fp32."""
        lead = indices.shape[:-1]
        idx = indices.reshape(-1, self.dim).to(torch.uint8)
        packed = ((idx[:, 0::2] << 4) | idx[:, 1::2]).reshape(-1, 1, self.dim // 2)
        # centroid look-up, norm and back-rotation in the library (fq_tq4_decompress_original)
        y = K.tq4_decompress_original(packed, norms.reshape(-1, 1, 1).float(), self.centroids,
                                      self.rotation, dtype=torch.float32)
        return y.reshape(*lead, self.dim)


class TurboQuantProd:
    """Stage 1 with bits-1 bits plus one QJL sign bit per coordinate of the residual."""

    def __init__(self, dim: int, bits: int, *, qjl_dim: int | None = None, seed: int = 42) -> None:
        if bits < 2:
            raise ValueError(f"TurboQuantProd requires bits >= 2, got {bits}")
        self.dim = dim
        self.bits = bits
        self.mse_quantizer = TurboQuantMSE(dim, bits - 1, seed=seed)
        self.qjl_dim = qjl_dim or dim
        gen = torch.Generator(device="cpu").manual_seed(seed + 1)
        self.qjl_matrix = torch.randn(self.qjl_dim, dim, generator=gen, device="cpu",
                                      dtype=torch.float32) / math.sqrt(self.qjl_dim)

    def quantize(self, x: torch.Tensor):
        """CUDA ``(..., dim)`` -> (indices int64, norms, signs fp32 of +-1, residual norms)."""
        m = self.mse_quantizer
        packed, norms, bits, gamma = K.tq_prod_quantize(x, m.rotation, m.boundaries, m.centroids,
                                                        self.qjl_matrix)
        idx = torch.stack([packed >> 4, packed & 0x0F], dim=-1).flatten(-2).long()
        shifts = torch.arange(8, device=bits.device, dtype=torch.uint8)
        signs = (((bits.unsqueeze(-1) >> shifts) & 1).flatten(-2).float() * 2.0 - 1.0)
        return idx, norms, signs, gamma

    def dequantize(self, indices, norms, qjl_signs, residual_norms) -> torch.Tensor:
        return self.mse_quantizer.dequantize(indices, norms)
