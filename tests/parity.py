"""Helpers shared by the GPU parity tests (tolerances are the ones the tests state)."""

import torch

from oracle import tq_oracle as O

CODE_MISMATCH_BUDGET = 1e-4   # fraction of coordinates allowed to differ
BOUNDARY_WINDOW = 1e-6        # ... and only if the rotated value is this close to a boundary
NORM_RTOL = 1e-6


def unpack(packed):
    return O.nibble_unpack(packed.cpu())


def check_codes(packed_gpu, x_cpu, rotation, boundaries, packed_ref):
    """Codes must equal the oracle's except next to a quantiser boundary."""
    got = unpack(packed_gpu).reshape(-1, x_cpu.shape[-1])
    ref = unpack(packed_ref).reshape(-1, x_cpu.shape[-1])
    diff = got != ref
    n_bad = int(diff.sum())
    if n_bad == 0:
        return 0.0
    flat = x_cpu.reshape(-1, x_cpu.shape[-1]).double()
    unit = flat / (flat.norm(dim=-1, keepdim=True) + O.NORM_EPS)
    y = unit @ rotation.double().T
    dist = (y.unsqueeze(-1) - boundaries.double()).abs().min(dim=-1).values
    assert bool((dist[diff] < BOUNDARY_WINDOW).all()), \
        f"code differs away from a boundary (max distance {dist[diff].max().item():.3e})"
    assert bool(((got - ref).abs()[diff] == 1).all()), "a code differs by more than one level"
    frac = n_bad / diff.numel()
    assert frac <= CODE_MISMATCH_BUDGET, f"code mismatch fraction {frac:.2e}"
    return frac


def check_norms(got, ref, rtol=NORM_RTOL):
    got, ref = got.cpu().reshape(-1).double(), ref.reshape(-1).double()
    err = (got - ref).abs()
    assert bool((err <= rtol * ref.abs()).all()), \
        f"norm relative error {(err / ref.abs().clamp_min(1e-300)).max().item():.3e}"


def attention_close(got, ref, atol=2e-3):
    """Attention outputs: max-abs 2e-3, or one bf16 unit in the last place of the largest
    entry of the same output row (|row|max * 2^-7) where that is larger.

    The reference rounds twice to bf16 (rotated output, then the product with Pi), so an
    entry of the final row inherits rounding steps of the row's largest entries.  At the
    benchmark shapes (thousands of tokens per sequence) every |output| is below 0.25 and
    the plain 2e-3 bound is the one that applies; short test sequences have outputs of
    order 1, where the bf16 grid itself is coarser than 2e-3.
    """
    got, ref = got.float().cpu(), ref.float().cpu()
    rowmax = ref.abs().amax(dim=-1, keepdim=True)
    tol = torch.maximum(torch.full_like(ref, atol), rowmax * 2.0 ** -7)
    err = (got - ref).abs()
    bad = err > tol
    if bool(bad.any()):
        i = int(torch.argmax((err - tol).flatten()))
        idx = [int(v) for v in torch.unravel_index(torch.tensor(i), err.shape)]
        raise AssertionError(
            f"attention mismatch: {int(bad.sum())} of {bad.numel()} entries beyond tolerance; "
            f"worst at {idx}: got {got.flatten()[i].item():.6f} ref {ref.flatten()[i].item():.6f} "
            f"tol {tol.flatten()[i].item():.2e}; max-abs err {err.max().item():.3e}")
    return err.max().item()
