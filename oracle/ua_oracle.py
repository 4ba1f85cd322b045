"""CPU oracle for the Universal Attention operator.  TEST INFRASTRUCTURE ONLY.

This file is a checker: only the test-suite, the smoke test and the
``cpu_baseline`` / ``--impl reference`` legs of the benchmark may import it.
The product path (the CUDA library) never routes through it.

It restates, in whole-sequence vectorised form, the algorithm of the
reference's pure-PyTorch operator:

* forward  : ``universal_attention_autograd.py:9-38`` (1-D form) and ``:104-163``
             (2-D row-chunked form, same mathematics)
* backward : ``universal_attention_autograd.py:47-99`` / ``:172-276``
* merge    : ``universal_attention_autograd.py:278-297`` (``SMVecMatMul``)

Parity pinning: ``tests/golden/*.npz`` were produced by running the unmodified
reference (imported from its checkout) with ``tests/golden/make_golden.py``;
``tests/test_oracle_golden.py`` checks every function here against them.

Unlike the reference (which loops over key chunks and, in the 2-D form, over
row chunks carrying a running sum) everything here is evaluated on the full
``L x L`` key/row plane at once, so the fp32 summation order differs from the
reference's; agreement is to rounding noise, not bitwise.  ``compute_dtype=
torch.float64`` gives the arbiter used to decide which side of a disagreement is
closer to the exact value (the reference forces fp32 internally, so an fp64
answer cannot be had from it by casting inputs).

Layouts (same as the reference):
    kc, vc       (b, h, n, c, d)        keys / values in n chunks of c
    xq           (b, h, r, L, d)  or  (b, h, r, _n, _c, d)
    static_src   (b, h, n, c)           per-key gate in (0, 1)
    static_dest  (b, h, L)  or  (b, h, _n, _c)   per-row gate in (0, 1)
    out          (b, h, r, L, d, n)     key-chunk index innermost
    denom        (b, h, r, L, n)        per-chunk log-sum-exp
"""
from __future__ import annotations

import torch

MASK_VALUE = -1e12          # universal_attention_autograd.py:28
CLAMP_MAX = 1 - 1e-6        # universal_attention_autograd.py:26
CLAMP_MIN_BWD = 1e-6        # universal_attention_autograd.py:85


def _canon(kc, vc, xq, static_src, static_dest):
    """Bring the 1-D and 2-D argument layouts to one form; returns shapes too."""
    b, h, n, c, d = kc.shape
    L = n * c
    r = xq.shape[2]
    q = xq.reshape(b, h, r, L, d)
    t = static_dest.reshape(b, h, L)
    s = static_src.reshape(b, h, L)
    k = kc.reshape(b, h, L, d)
    v = vc.reshape(b, h, L, d)
    return k, v, q, s, t, (b, h, r, n, c, d, L)


def _decay_terms(k, s, t, cd, pow_rel_noise=0.0):
    """Steps 1-3 of the forward: Gram matrix, gated affinity, log-retention.

    Returns (gram, pw, aff, ell) on the (key, row) plane, all in ``cd``;
    ``ell`` already carries the strict-causal mask (zero where row <= key).
    Follows universal_attention_autograd.py:24-27.
    """
    L = k.shape[-2]
    kf = k.to(cd)
    gram = kf @ kf.transpose(-1, -2)                       # (b,h,Lk,Lq)
    pw = gram.clamp_min(0).pow(2.0 / 3.0)
    if pow_rel_noise:
        # conditioning probe: the power perturbed by a seeded random relative error of the given size (what a
        # hardware exp2 / log2 pair of that accuracy would do); the change of the results measures how far the
        # reference arithmetic itself pins them
        gen = torch.Generator().manual_seed(12345)
        sign = torch.randint(0, 2, pw.shape, generator=gen).to(cd) * 2 - 1
        pw = pw * (1 + pow_rel_noise * sign)
    s3 = s.to(cd).pow(1.0 / 3.0)
    t3 = t.to(cd).pow(1.0 / 3.0)
    aff = pw * s3.unsqueeze(-1) * t3.unsqueeze(-2)
    cmax = torch.tensor(CLAMP_MAX, dtype=torch.float32).to(cd)   # the reference clamps an fp32 tensor
    ell = torch.log1p(-aff.clamp(0, cmax.item()))
    idx = torch.arange(L)
    strict = idx.view(1, L) > idx.view(L, 1)               # row > key
    ell = torch.where(strict, ell, torch.zeros((), dtype=cd))
    return gram, pw, aff, ell, s3, t3, strict


def _absorb(score, before, cd):
    """In the reference's fp32 arithmetic ``k.q + (-1e12)`` IS -1e12 (fp32 spacing there is 65536), which makes the
    softmax of a fully masked block exactly uniform (universal_attention_autograd.py:28-35).  The fp64 arbiter keeps
    that semantics instead of resolving ``k.q`` next to -1e12."""
    if cd == torch.float32:
        return score
    return torch.where(before, torch.full((), MASK_VALUE, dtype=cd), score)


def ua_forward(kc, vc, xq, static_src, static_dest, compute_dtype=torch.float32, pow_rel_noise=0.0):
    """Forward of the operator; returns ``(out, denom)`` in ``xq.dtype`` plus the
    fp32/fp64 log-sum-exp before the cast, as a third value.

    universal_attention_autograd.py:9-38.
    """
    cd = compute_dtype
    k, v, q, s, t, (b, h, r, n, c, d, L) = _canon(kc, vc, xq, static_src, static_dest)
    _, _, _, ell, _, _, _ = _decay_terms(k, s, t, cd, pow_rel_noise)
    idx = torch.arange(L)
    before = idx.view(1, L) < idx.view(L, 1)               # row < key
    decay = ell.cumsum(-1)
    decay = torch.where(before, torch.full((), MASK_VALUE, dtype=cd), decay)
    score = k.to(cd).unsqueeze(2) @ q.to(cd).transpose(-1, -2)      # (b,h,r,Lk,Lq)
    score = _absorb(score + decay.unsqueeze(2), before, cd)
    score = score.view(b, h, r, n, c, L)
    lse = score.logsumexp(dim=-2)                          # (b,h,r,n,Lq)
    prob = score.softmax(dim=-2)                           # over the chunk's keys (uniform where all are -1e12)
    if cd == torch.float32:
        prob = prob.to(xq.dtype).to(cd)                    # the reference rounds P to the input dtype
    vv = v.to(cd).view(b, h, 1, n, c, d)
    out = prob.transpose(-1, -2) @ vv                      # (b,h,r,n,Lq,d)
    out = out.permute(0, 1, 2, 4, 5, 3).contiguous()       # (b,h,r,L,d,n)
    lse = lse.permute(0, 1, 2, 4, 3).contiguous()          # (b,h,r,L,n)
    return out.to(xq.dtype), lse.to(xq.dtype), lse


def ua_backward(kc, vc, xq, static_src, static_dest, g_out, g_denom, compute_dtype=torch.float32, pow_rel_noise=0.0):
    """Gradients ``(dkc, dvc, dxq, dstatic_src, dstatic_dest)`` for upstream
    ``g_out (b,h,r,L,d,n)`` and ``g_denom (b,h,r,L,n)``.

    universal_attention_autograd.py:47-99 / :172-276.  Gradients keep the
    shape and dtype of the matching input.
    """
    cd = compute_dtype
    k, v, q, s, t, (b, h, r, n, c, d, L) = _canon(kc, vc, xq, static_src, static_dest)
    round_in = (lambda x: x.to(xq.dtype).to(cd)) if cd == torch.float32 else (lambda x: x)
    gram, pw, aff, ell, s3, t3, strict = _decay_terms(k, s, t, cd, pow_rel_noise)
    idx = torch.arange(L)
    before = idx.view(1, L) < idx.view(L, 1)
    decay = torch.where(before, torch.full((), MASK_VALUE, dtype=cd), ell.cumsum(-1))
    kf, vf, qf = k.to(cd), v.to(cd), q.to(cd)
    score = _absorb(kf.unsqueeze(2) @ qf.transpose(-1, -2) + decay.unsqueeze(2), before, cd).view(b, h, r, n, c, L)
    prob = score.softmax(dim=-2)                           # (b,h,r,n,c,Lq) fp32, per key chunk
    go = g_out.to(cd).permute(0, 1, 2, 5, 3, 4)            # (b,h,r,n,Lq,d)
    gd = g_denom.to(cd).permute(0, 1, 2, 4, 3)             # (b,h,r,n,Lq)

    # value path                                            (:69, :245)
    dv = (round_in(prob) @ go).sum(2).reshape(b, h, L, d)
    # softmax + log-sum-exp                                 (:71-73, :246-248)
    dp = vf.view(b, h, 1, n, c, d) @ go.transpose(-1, -2)  # (b,h,r,n,c,Lq)
    ds = (dp - (dp * prob).sum(-2, keepdim=True)) * prob + prob * gd.unsqueeze(-2)
    ds = ds.reshape(b, h, r, L, L)                         # (key, row)
    dsr = round_in(ds)
    dq = dsr.transpose(-1, -2) @ kf.unsqueeze(2)           # (b,h,r,Lq,d)   (:75, :251)
    dk = (dsr @ qf).sum(2)                                 # (b,h,Lk,d)     (:76, :252)

    # decay path                                            (:78-93, :255-273)
    dc = ds.sum(2)                                         # (b,h,Lk,Lq)
    dell = dc.flip(-1).cumsum(-1).flip(-1)
    dell = torch.where(strict, dell, torch.zeros((), dtype=cd))
    cmax = torch.tensor(CLAMP_MAX, dtype=torch.float32).to(cd).item()
    cmin = torch.tensor(CLAMP_MIN_BWD, dtype=torch.float32).to(cd).item()
    da = dell / (aff.clamp(cmin, cmax) - 1)
    da = da * (aff <= cmax)
    dstat = da * pw
    dsrc = (dstat * t3.unsqueeze(-2)).sum(-1) / (3 * s3 * s3)
    ddst = (dstat * s3.unsqueeze(-1)).sum(-2) / (3 * t3 * t3)
    dg = round_in(da * s3.unsqueeze(-1) * t3.unsqueeze(-2))
    dg = dg * (gram.abs() + 1e-9).pow(-1.0 / 3.0) * (2.0 / 3.0) * (gram > 0)
    dk = dk + dg @ kf + dg.transpose(-1, -2) @ kf          # key side and row side of K K^T

    return (dk.reshape(kc.shape).to(kc.dtype), dv.reshape(vc.shape).to(vc.dtype),
            dq.reshape(xq.shape).to(xq.dtype), dsrc.reshape(static_src.shape).to(static_src.dtype),
            ddst.reshape(static_dest.shape).to(static_dest.dtype))


def merge_forward(mat, vec):
    """``SMVecMatMul.forward``: softmax over the key-chunk axis of ``vec`` weights
    the last axis of ``mat``.  universal_attention_autograd.py:280-283."""
    w = vec.float().softmax(dim=-1).to(mat.dtype)
    return (mat * w.unsqueeze(-2)).sum(-1)


def merge_backward(mat, vec, g):
    """``SMVecMatMul.backward``.  universal_attention_autograd.py:291-297."""
    w = vec.softmax(dim=-1)
    d_mat = g.unsqueeze(-1) * w.unsqueeze(-2)
    d_vec = (g.unsqueeze(-1) * mat).sum(-2)
    d_vec = (d_vec - (d_vec * w).sum(-1, keepdim=True)) * w
    return d_mat, d_vec


def driver_step(kc, vc, xq, static_src, static_dest, compute_dtype=torch.float32):
    """One forward+backward of the reference driver's flow (``main.py:55-62``):
    operator -> merge -> ``loss = merged.pow(2).sum()`` -> gradients.
    Returns ``(loss, merged, out, denom, grads)``."""
    out, denom, _ = ua_forward(kc, vc, xq, static_src, static_dest, compute_dtype)
    merged = merge_forward(out, denom)
    loss = merged.float().pow(2).sum()
    g = 2 * merged
    d_mat, d_vec = merge_backward(out, denom, g)
    grads = ua_backward(kc, vc, xq, static_src, static_dest, d_mat, d_vec, compute_dtype)
    return loss, merged, out, denom, grads


def make_inputs(B, H, R, L, chunk, D, dtype=torch.float32, seed=0, qkv_std=1.0,
                gate_mean=0.0, gate_std=1.0, two_d=False):
    """Seeded synthetic inputs: fp32 normals drawn on the CPU generator in the
    order xq, kc, vc, src_logits, dest_logits; gates are ``sigmoid(logit)`` (the
    operator needs gates in (0, 1): ``pow(1/3)`` of a negative number is NaN,
    universal_attention_autograd.py:15-16)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    n = L // chunk
    xq = torch.randn(B, H, R, L, D, generator=g) * qkv_std
    kc = torch.randn(B, H, n, chunk, D, generator=g) * qkv_std
    vc = torch.randn(B, H, n, chunk, D, generator=g) * qkv_std
    ss = (torch.randn(B, H, n, chunk, generator=g) * gate_std + gate_mean).sigmoid()
    sd = (torch.randn(B, H, L, generator=g) * gate_std + gate_mean).sigmoid()
    if two_d:
        xq = xq.view(B, H, R, n, chunk, D)
        sd = sd.view(B, H, n, chunk)
    return tuple(x.to(dtype) for x in (kc, vc, xq, ss, sd))
