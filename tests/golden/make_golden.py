"""Generates tests/golden/sdpa_golden.npz.

The reference stores no golden vectors for attention and its TypeScript
oracle cannot be executed where this repository is built (no Node), so the
fixtures come from an independent numpy f64 restatement
(``oracle/sdpa_numpy.py``) driven by a pure-Python copy of the reference
tests' input generator (packages/runntime/test/gpu.ts:114-130,
checkSdpa.ts:142-161).  Neither shares code with ``oracle/sdpa_oracle.c``,
which the fixtures are then used to pin.

Run from the repository root:  python tests/golden/make_golden.py
"""
from __future__ import annotations

import json
import math
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from oracle.sdpa_numpy import sdpa_numpy  # noqa: E402
import cases  # noqa: E402


def lcg(n: int, seed: int) -> np.ndarray:
    """s = s*1664525 + 1013904223 mod 2^32; value s / 2^31 - 1, stored as f32."""
    out = np.empty(n, dtype=np.float32)
    s = seed & 0xFFFFFFFF
    for i in range(n):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = s / 2 ** 31 - 1
    return out


def inputs(c, dtype):
    rnd = (lambda a: a.astype(np.float16).astype(np.float32)) if dtype == "f16" else (lambda a: a)
    hd = c.headDim
    q = rnd((lcg(c.qLen * c.qHeads * hd, 1).astype(np.float64) * (2 / math.sqrt(hd)))
            .astype(np.float32)).reshape(c.qLen, -1)
    k = rnd(lcg(c.kvLen * c.kvHeads * hd, 2)).reshape(c.kvLen, -1)
    v = rnd(lcg(c.kvLen * c.kvHeads * hd, 3)).reshape(c.kvLen, -1)
    sinks = (2 * lcg(c.qHeads, 4)).astype(np.float32) if c.sinks else None
    segs = None
    if c.segments:
        segs = np.empty((c.qLen, 2), dtype=np.float32)
        qh, kh = c.qLen // 2, c.kvLen // 2
        segs[:qh] = (0, kh)
        segs[qh:] = (kh, c.kvLen)
    kb = (c.kvLen // 4, c.kvLen // 2, 2.0) if c.keyBias else None
    return q, k, v, sinks, segs, kb


def golden_cases():
    out = []
    for dtype in ("f32", "f16"):
        for name, c in cases.option_cases(37, 16):
            out.append((f"opt-{dtype}-{name}", dtype, c))
    small = {"hd1", "qposoffset_small", "empty_rows_sinks_small", "empty_rows_sinks_40x20",
             "segments_maxseg_32", "qposoffset_50"}
    for name, c in cases.PREFILL_SHAPES:
        if name in small:
            out.append((f"shape-f32-{name}", "f32", c))
    for name, c in cases.DECODE_CASES:
        if c.kvLen <= 300:
            out.append((f"decode-f32-{name}", "f32", c))
            out.append((f"decode-f16-{name}", "f16", c))
    return out


def main():
    arrays, meta = {}, {}
    for name, dtype, c in golden_cases():
        q, k, v, sinks, segs, kb = inputs(c, dtype)
        arrays[name] = sdpa_numpy(q, k, v, qHeads=c.qHeads, kvHeads=c.kvHeads,
                                  headDim=c.headDim, windowLeft=c.windowLeft,
                                  windowRight=c.windowRight, qPosOffset=c.qPosOffset,
                                  sinks=sinks, segs=segs, keyBias=kb)
        d = dict(c.__dict__)
        for key in ("windowLeft", "windowRight"):
            if d[key] == math.inf:
                d[key] = "inf"
        meta[name] = dict(dtype=dtype, case=d)
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "sdpa_golden.npz"), **arrays)
    with open(os.path.join(here, "sdpa_golden.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)
    print(f"wrote {len(arrays)} cases")


if __name__ == "__main__":
    main()
