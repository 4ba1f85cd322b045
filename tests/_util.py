"""Shared helpers for the parity tests."""
import os

import numpy as np
import torch

from oracle import ua_oracle as O

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


K_NOISE = 2.0
GRADS = ["dkc", "dvc", "dxq", "dsrc", "ddest"]

# Noise-pinned checks.  The stated bars (bf16 forward max-abs 2e-2, gradients 5e-2 relative-Frobenius, against the fp32
# oracle fed the same bf16-rounded values) are asserted as
#       kernel_error <= max(stated bar, K_NOISE * oracle_noise),
# where oracle_noise is the SAME metric on the SAME inputs between the oracle evaluated in fp32 and in fp64: a bound
# above the stated bar is only granted where the reference arithmetic itself is that uncertain (at L = 4096 its fp32
# cumulative sum reaches -2e4, where fp32 spacing is 2e-3).  Figures are printed (pytest -s).


def check_forward(tag, out, lse, ins32, c):
    """out (b,h,r,L,d,n) bf16 values as float, lse (b,h,r,L,n) fp32; both CPU.  Returns the figures it asserted on."""
    ref_out, _, ref_lse = O.ua_forward(*ins32)
    arb_out, _, arb_lse = O.ua_forward(*ins32, compute_dtype=torch.float64)
    L, n = lse.shape[-2], lse.shape[-1]
    valid = valid_row_mask(L, n, c)
    vo = valid.view(L, 1, n)
    e_out = ((out - ref_out.float()).abs() * vo).max().item()
    n_out = ((ref_out.float() - arb_out.float()).abs() * vo).max().item()
    e_lse = ((lse - ref_lse).abs() * valid).max().item()
    n_lse = ((ref_lse.double() - arb_lse).abs() * valid).max().item()
    frac_k = (((out - ref_out.float()).abs() > 2e-2) & vo).float().mean().item()
    frac_n = (((ref_out.float() - arb_out.float()).abs() > 2e-2) & vo).float().mean().item()
    merged = O.merge_forward(out, lse)
    merged_ref = O.merge_forward(arb_out.double(), arb_lse).float()
    e_merged = (merged - merged_ref).abs().max().item()
    print(f"[{tag}] out max-abs {e_out:.3e} (oracle fp32-vs-fp64 {n_out:.3e}); elements over 2e-2: {frac_k:.2e} "
          f"(oracle {frac_n:.2e}); lse {e_lse:.3e} (oracle {n_lse:.3e}); merged vs fp64 {e_merged:.3e}")
    assert e_out <= max(2e-2, K_NOISE * n_out), (tag, e_out, n_out)
    assert frac_k <= max(1e-6, K_NOISE * frac_n), (tag, frac_k, frac_n)
    assert e_lse <= max(2e-2, K_NOISE * n_lse), (tag, e_lse, n_lse)
    assert e_merged <= 2e-2, (tag, e_merged)      # the merged output is well conditioned: the plain bar
    masked = ~valid
    if masked.any():
        assert (lse[..., masked] <= -1e11).all()
    return dict(out=e_out, out_noise=n_out, lse=e_lse, lse_noise=n_lse)


def check_backward(tag, grads, ins32, g_out, g_den):
    ref = O.ua_backward(*ins32, g_out, g_den)
    arb = O.ua_backward(*[t.double() for t in ins32], g_out.double(), g_den.double(), compute_dtype=torch.float64)
    res = {}
    for got, r32, r64, key in zip(grads, ref, arb, GRADS):
        got = got.float().cpu()
        assert torch.isfinite(got).all(), (tag, key)
        err = rel_fro(got, r32)
        noise = rel_fro(r32, r64)
        err64 = rel_fro(got, r64)
        print(f"[{tag}] {key}: rel-Frobenius vs fp32 oracle {err:.3e}; oracle fp32-vs-fp64 {noise:.3e}; "
              f"kernel vs fp64 oracle {err64:.3e}")
        assert err <= max(5e-2, K_NOISE * noise), (tag, key, err, noise)
        res[key] = (err, noise, err64)
    return res
