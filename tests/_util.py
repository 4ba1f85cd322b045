"""Shared helpers for the parity tests."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    return {k: torch.from_numpy(z[k]) for k in z.files}


def rel_fro(a, b):
    """Relative Frobenius error of a against b."""
    a = a.double().reshape(-1)
    b = b.double().reshape(-1)
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


def valid_row_mask(L, n, c):
    """(L, n) bool: row q sees at least one key of chunk i  <=>  q >= i*c."""
    q = torch.arange(L).view(L, 1)
    i = torch.arange(n).view(1, n)
    return q >= i * c


def fwd_errors(out, denom, ref_out, ref_denom, c):
    """max-abs errors on the causally valid region and on the fully masked one.
    out (b,h,r,L,d,n), denom (b,h,r,L,n)."""
    L, n = denom.shape[-2], denom.shape[-1]
    valid = valid_row_mask(L, n, c).to(out.device)
    dv = (out.double() - ref_out.double()).abs()
    e_out_valid = (dv * valid.view(L, 1, n)).max().item()
    e_out_masked = (dv * (~valid).view(L, 1, n)).max().item()
    dd = (denom.double() - ref_denom.double()).abs()
    e_den_valid = (dd * valid).max().item()
    masked_ok = bool((denom[..., ~valid] <= -1e11).all().item()) if (~valid).any() else True
    return dict(out_valid=e_out_valid, out_masked=e_out_masked, denom_valid=e_den_valid, masked_denom_ok=masked_ok)


def robust_rel_fro(a, b, fraction=1e-3):
    """Relative Frobenius error of a against b without the few largest elements of b.

    The gradient of log1p(-affinity) carries 1 / (1 - affinity), which reaches 1e6 for the pairs just below the clamp
    at 1 - 1e-6; there one ulp of the fp32 affinity (the summation order of k.k already moves it) changes the result by
    several per cent in the reference itself, and a single such element can hold the whole norm of a tensor.  The
    ``ceil(fraction * numel)`` elements of b of largest magnitude are left out."""
    a = a.double().reshape(-1)
    b = b.double().reshape(-1)
    k = max(1, int(-(-fraction * b.numel() // 1)))
    keep = torch.ones_like(b, dtype=torch.bool)
    keep[b.abs().topk(k).indices] = False
    return ((a - b)[keep].norm() / b[keep].norm().clamp_min(1e-30)).item()
