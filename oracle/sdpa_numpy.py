"""Independent numpy f64 restatement of the attention semantics — TEST
INFRASTRUCTURE ONLY (second opinion on the C oracle and source of the committed
golden fixtures).

Written mask-first and vectorised, on purpose unlike the loop form of
``sdpa_oracle.c``: a dense visibility matrix, then a masked softmax.
Semantics: packages/runntime/test/core/kernels/attention/checkSdpa.ts:58-108
and the visibility rule documented at
packages/runntime/src/core/graph/ops/attention.ts:14-27.
"""
from __future__ import annotations

import math

import numpy as np


def visibility(qLen, kvLen, windowLeft=math.inf, windowRight=math.inf, qPosOffset=0, segs=None):
    """Boolean [qLen, kvLen]: key j visible to row i."""
    i = np.arange(qLen, dtype=np.float64)[:, None] + qPosOffset
    j = np.arange(kvLen, dtype=np.float64)[None, :]
    vis = (j >= i - windowLeft) & (j <= i + windowRight)
    if segs is not None:
        segs = np.asarray(segs, dtype=np.float64)
        vis &= (j >= segs[:, 0:1]) & (j < segs[:, 1:2])
    return vis


def sdpa_numpy(q, k, v, *, qHeads, kvHeads, headDim, windowLeft=math.inf, windowRight=math.inf,
               qPosOffset=0, sinks=None, segs=None, keyBias=None):
    q = np.asarray(q, dtype=np.float64)
    k = np.asarray(k, dtype=np.float64)
    v = np.asarray(v, dtype=np.float64)
    qLen, kvLen, hd = q.shape[0], k.shape[0], headDim
    vis = visibility(qLen, kvLen, windowLeft, windowRight, qPosOffset, segs)
    out = np.zeros((qLen, qHeads * hd))
    group = qHeads // kvHeads
    bias = np.zeros(kvLen)
    if keyBias is not None:
        bias[keyBias[0]:keyBias[1]] = keyBias[2]
    for h in range(qHeads):
        g = h // group
        s = q[:, h * hd:(h + 1) * hd] @ k[:, g * hd:(g + 1) * hd].T + bias[None, :]
        s = np.where(vis, s, -np.inf)
        sink = -np.inf if sinks is None else float(sinks[h]) * math.log(2.0)
        m = np.maximum(s.max(axis=1, initial=-np.inf), sink)
        live = np.isfinite(m)
        ms = np.where(live, m, 0.0)
        p = np.exp(s - ms[:, None])
        den = p.sum(axis=1) + np.exp(sink - ms)
        o = (p @ v[:, g * hd:(g + 1) * hd]) / np.where(den > 0, den, 1.0)[:, None]
        out[:, h * hd:(h + 1) * hd] = np.where(live[:, None], o, 0.0)
    return out
