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


def _residual(x_cpu, codes, norms, rotation, centroids):
    """r = x - (c[code] Pi) n in fp64 (src/flashquant/core/quantizer.py:186-193, 290-291), with
    the fp32 norm the quantiser stored."""
    d = x_cpu.shape[-1]
    x = x_cpu.reshape(-1, d).double()
    xt = (centroids.double()[codes.reshape(-1, d).long()] @ rotation.double()) * \
        norms.reshape(-1, 1).double()
    return x - xt


def check_gamma(got, ref, x_cpu, codes_got, codes_ref, norms, rotation, centroids):
    """Residual norms gamma = |x - x~|.  The residual is a difference of nearly equal fp32
    numbers, so ANY fp32 evaluation - the reference's included - sits up to 1e-6 (relative)
    from the exact value, and two such evaluations up to 2e-6 from each other.  The check:
    the CUDA value is as close to the exact (fp64) residual norm as the reference's own value
    is (both about 1e-6 at worst), 99.8 % of the values agree with the reference to 1e-6 and
    all of them to 2.2e-6.  Vectors whose codes differ from the reference's (allowed next to
    a quantiser boundary) have another residual and are left out."""
    d = x_cpu.shape[-1]
    same = (codes_got.reshape(-1, d) == codes_ref.reshape(-1, d)).all(dim=-1)
    truth = _residual(x_cpu, codes_got, norms, rotation, centroids).norm(dim=-1)[same]
    g = got.cpu().reshape(-1).double()[same]
    r = ref.reshape(-1).double()[same]
    scale = truth.clamp_min(1e-30)
    e_got, e_ref, e_pair = (g - truth).abs() / scale, (r - truth).abs() / scale, (g - r).abs() / scale
    keep = truth > 0
    assert bool((g[~keep] == 0).all()), "gamma of a zero residual must be 0"
    e_got, e_ref, e_pair = e_got[keep], e_ref[keep], e_pair[keep]
    assert e_got.max().item() <= max(1e-6, 1.25 * e_ref.max().item()), \
        f"gamma: {e_got.max().item():.3e} from the exact value (the reference: {e_ref.max().item():.3e})"
    assert (e_pair > NORM_RTOL).double().mean().item() <= 2e-3, \
        f"gamma: {(e_pair > NORM_RTOL).double().mean().item():.2e} of the values beyond 1e-6 of the reference"
    assert e_pair.max().item() <= 2.2e-6, f"gamma relative error {e_pair.max().item():.3e}"


def check_signs(bits_got, signs_ref, x_cpu, codes_got, codes_ref, norms, rotation, centroids, qjl):
    """QJL sign bits: equal to the reference's except where the projection is within 1e-6 of
    zero relative to |r| (the same rule as for the codes), at most 1e-4 of them."""
    from oracle import tq_oracle as O
    d = x_cpu.shape[-1]
    got = O.sign_bits_unpack(bits_got.cpu()).reshape(-1, qjl.shape[0])
    ref = signs_ref.reshape(-1, qjl.shape[0]).float()
    same = (codes_got.reshape(-1, d) == codes_ref.reshape(-1, d)).all(dim=-1)
    diff = (got != ref) & same.unsqueeze(1)
    frac = diff.float().mean().item()
    assert frac <= CODE_MISMATCH_BUDGET, f"sign mismatch fraction {frac:.2e}"
    if bool(diff.any()):
        r = _residual(x_cpu, codes_got, norms, rotation, centroids)
        proj = (r @ qjl.double().T).abs() / r.norm(dim=-1, keepdim=True).clamp_min(1e-300)
        worst = proj[diff].max().item()
        assert worst < BOUNDARY_WINDOW, \
            f"a sign differs where |S r|/|r| = {worst:.3e} (not next to zero)"
    return frac


ATTN_ATOL = 2e-3           # north-star bound on attention outputs (max-abs)
PRE_RTOL = 2.0 ** -10      # agreement of the un-rounded rows, relative to the entry
PRE_OUTLIERS = 1e-4        # share of entries that may miss it (by at most a factor of two)


def ulp(x, dtype):
    """Spacing of ``dtype`` (bf16 / fp16) numbers at |x|, element-wise, as fp32."""
    mant = {torch.bfloat16: 7, torch.float16: 10}[dtype]
    tiny = {torch.bfloat16: -126, torch.float16: -14}[dtype]
    e = torch.floor(torch.log2(x.abs().float().clamp_min(2.0 ** tiny)))
    return torch.pow(2.0, e.clamp_min(tiny) - mant)


def pre_rounding_bound(ref32, atol=ATTN_ATOL, rtol=PRE_RTOL):
    """How far an un-rounded rotated-space row may be from the reference's: max-abs ``atol``
    and ``rtol`` of the entry's own magnitude.  An entry far below the typical size of its
    row is a sum that cancels, so its magnitude is floored at the row's rms."""
    rms = ref32.pow(2).mean(dim=-1, keepdim=True).sqrt()
    return torch.minimum(torch.full_like(ref32, atol), rtol * torch.maximum(ref32.abs(), rms))


def attention_close(got, ref, ref_rot32, rotation, got_rot32=None, atol=ATTN_ATOL,
                    rtol=PRE_RTOL, rounds_rotated=True, slack=1.0):
    """Attention outputs against the reference, following its two roundings.

    The reference computes the rotated-space row in fp32 (``ref_rot32``), rounds it to the
    model dtype, multiplies by Pi and rounds again.  An implementation that is not
    bit-identical before the first rounding cannot meet a flat 2e-3 after the second one: a
    coordinate that sits next to a rounding boundary lands on the other neighbour (one unit
    in the last place, 0.0156 at |x| = 2 in bf16) and the product with Pi spreads that step
    over the whole row.  So the check has two parts.

    1. Before the first rounding (``got_rot32``, when the caller has it): entries within
       ``pre_rounding_bound`` of the reference's fp32 value - max-abs 2e-3 and 2^-10 of the
       entry - except for at most one entry in 10^4, and those within twice the bound.  This is
       the accuracy statement proper; no rounding is involved.
    2. After both roundings, entry k may differ by one unit in the last place OF THAT ENTRY
       (the last rounding may fall either way) plus sum_j ulp(o_rot_j) |Pi_jk| over exactly
       those coordinates j whose fp32 value lies within the part-1 bound of a rounding
       boundary - the only ones a conforming implementation can round the other way.

    ``rounds_rotated=False`` is the prefill form of the reference, which keeps the rotated
    row in fp32 and rounds only the product with Pi (cpu_reference.py:195, 225-226): part 2
    then allows one unit in the last place of the entry plus sum_j bound_j |Pi_jk| with the
    part-1 bound of every coordinate.  ``slack`` multiplies the part-2 tolerance (2 when two
    implementations that each meet it are compared with each other).

    Returns a dict of measured figures (max errors, share of entries beyond 2e-3, share of
    identical entries, share of coordinates that could flip).
    """
    dtype = ref.dtype
    got, ref = got.float().cpu(), ref.float().cpu()
    ref_rot32, rot = ref_rot32.float().cpu(), rotation.float().cpu()
    margin = pre_rounding_bound(ref_rot32, atol, rtol)
    stats = {}
    if got_rot32 is not None:
        # the errors behave like noise of about a quarter of the bound, so among 10^5 entries a
        # handful reach it: at most PRE_OUTLIERS of the entries may exceed the bound, none by
        # more than a factor of two (which is what the flip candidates below are sized for)
        e1 = (got_rot32.float().cpu() - ref_rot32).abs()
        bad, worse = e1 > margin, e1 > 2 * margin
        stats["pre_max_abs"] = e1.max().item()
        stats["pre_beyond_bound"] = bad.float().mean().item()
        if bool(worse.any()) or int(bad.sum()) > PRE_OUTLIERS * bad.numel():
            i = int(torch.argmax((e1 - margin).flatten()))
            raise AssertionError(
                f"un-rounded rows: {int(bad.sum())} of {bad.numel()} entries beyond "
                f"min({atol}, {rtol:.2e} |entry|), {int(worse.sum())} beyond twice that; worst "
                f"error {e1.flatten()[i].item():.3e} at value {ref_rot32.flatten()[i].item():.4f} "
                f"(bound {margin.flatten()[i].item():.3e})")
        margin = 2 * margin
    if rounds_rotated:
        # coordinates of the rotated row that may round to the other neighbour
        u = ulp(ref_rot32, dtype)
        lo = ref_rot32.to(dtype).float()
        dist_to_midpoint = (u / 2 - (ref_rot32 - lo).abs()).abs()
        may_flip = (dist_to_midpoint <= margin).float()
        spread = torch.matmul(may_flip * u, rot.abs())
    else:
        may_flip = torch.zeros_like(margin)
        spread = torch.matmul(margin, rot.abs())
    tol = slack * (ulp(ref, dtype) + spread + 1e-6 * ref.abs())
    err = (got - ref).abs()
    bad = err > tol
    stats.update(max_abs=err.max().item(), beyond_atol=(err > atol).float().mean().item(),
                 identical=(err == 0).float().mean().item(), may_flip=may_flip.mean().item())
    if bool(bad.any()):
        i = int(torch.argmax((err - tol).flatten()))
        idx = [int(v) for v in torch.unravel_index(torch.tensor(i), err.shape)]
        raise AssertionError(
            f"attention mismatch: {int(bad.sum())} of {bad.numel()} entries beyond one unit in "
            f"the last place plus the rounding flips the reference's own values allow; worst at "
            f"{idx}: got {got.flatten()[i].item():.6f} ref {ref.flatten()[i].item():.6f} "
            f"tol {tol.flatten()[i].item():.2e}; max-abs err {err.max().item():.3e}")
    return stats


def rows_from_partials(parts):
    """Normalised fp32 rows (acc / l) from (…, D+4) partial rows; empty rows give zeros."""
    parts = parts.float().cpu()
    d = parts.shape[-1] - 4
    l = parts[..., d + 1:d + 2]
    return torch.where(l > 0, parts[..., :d] / l.clamp_min(1e-30), torch.zeros_like(parts[..., :d]))
