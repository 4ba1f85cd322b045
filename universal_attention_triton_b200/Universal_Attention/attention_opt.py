"""``attention(q, k, v, causal, sm_scale, static_src, static_dest, ...)`` with the signature of the reference's
flash-style entry point (``Universal_Attention/triton/universal_attention_kernel_opt.py:433-583``,
``attention = _attention.apply``), on top of ``UniversalAttentionMerged``.

That entry point returns the softmax over ALL keys of ``q k^T + decay`` times ``v`` -- the merged output of the
chunked operator -- for
    q (b, n_heads, s, d),  k, v (b, n_kv_heads, s, d),  static_src, static_dest (b, n_kv_heads, s)
with query head ``h`` reading kv head ``h % n_kv_heads`` (``off_h % KV_H``, ``:142``), ``s`` a multiple of 128
(``:439``), head dims outside {16, 32, 64, 128, 256} zero-padded (``:445-453``) and ``sm_scale`` accepted but not
applied to the scores (``:84-85``: ``qk = tl.dot(q, k); qk += aff``).  The same holds here.  Differences, all on the
side of accuracy: the decay prefix stays in fp32 (the reference stores its affinity matrix in the input dtype, ``:53``),
and rows are masked with -1e12 instead of -1e8.  ``warp_specialize`` and ``ac`` (recompute the affinity matrix in the
backward) have no meaning here: nothing of size s x s is ever stored.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..universal_attention_autograd import UniversalAttentionMerged

CHUNK = 128


def attention(q, k, v, causal=True, sm_scale=None, static_src=None, static_dest=None, warp_specialize=True, ac=False):
    assert causal, "currently, only support causal-autoregressive style generation only."
    assert static_src is not None and static_dest is not None
    b, n_heads, s, d = q.shape
    n_kv = k.shape[1]
    assert s % CHUNK == 0, "Only works for multiples of 128!"
    assert k.shape == (b, n_kv, s, d) and v.shape == (b, n_kv, s, d) and n_heads % n_kv == 0
    assert static_src.shape == (b, n_kv, s) and static_dest.shape == (b, n_kv, s)
    rep = n_heads // n_kv
    # head dims the tensor-core kernels do not take are zero-padded: zero columns change neither k.k, q.k nor the
    # leading d columns of the output
    dp = 64 if d <= 64 else (128 if d <= 128 else d)
    if dp != d:
        q, k, v = (F.pad(t, (0, dp - d)) for t in (q, k, v))
    n = s // CHUNK
    xq = q.view(b, rep, n_kv, s, dp).transpose(1, 2)          # query head r * n_kv + kv reads kv head kv
    kc = k.reshape(b, n_kv, n, CHUNK, dp)
    vc = v.reshape(b, n_kv, n, CHUNK, dp)
    merged = UniversalAttentionMerged.apply(kc, vc, xq.contiguous(), static_src.reshape(b, n_kv, n, CHUNK), static_dest)
    o = merged.view(b, n_kv, rep, s, dp).transpose(1, 2).reshape(b, n_heads, s, dp)
    return o[..., :d]
