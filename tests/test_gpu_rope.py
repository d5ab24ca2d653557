"""Rotary embedding on the GPU: the reference suite's cases
(packages/runntime/test/core/kernels/attention/rope.gpu.test.ts:51-123) — including
its hand-worked vector, the one numeric known answer the reference stores for
this path — and the decoder's chain rope -> writeRows -> sdpa."""
import math

import numpy as np
import pytest

import oracle
from gpu_harness import ex  # noqa: F401

pytestmark = pytest.mark.gpu


def rope_tables(rows, headDim):
    """angle t * 10000^(-2i/headDim) for pair i at position t, pair-duplicated."""
    t = np.arange(rows, dtype=np.float64)[:, None]
    i = np.arange(headDim // 2, dtype=np.float64)[None, :]
    ang = t * 10000.0 ** (-2 * i / headDim)
    cos = np.repeat(np.cos(ang), 2, axis=1).astype(np.float32)
    sin = np.repeat(np.sin(ang), 2, axis=1).astype(np.float32)
    return cos, sin


CASES = [
    ("one_pair", dict(rows=1, cols=2, headDim=2)),
    ("one_head", dict(rows=5, cols=64, headDim=64)),
    ("several_heads_odd_rows", dict(rows=7, cols=60, headDim=10)),
    ("pairs_not_multiple_of_block", dict(rows=3, cols=4 * 34, headDim=34)),
    ("slice_of_slab", dict(rows=9, cols=8 * 16, headDim=16, srcStart=4 * 16, width=2 * 16)),
    ("last_head_of_slab", dict(rows=3, cols=48, headDim=16, srcStart=32, width=16)),
    ("moonshine_tiny_qkv", dict(rows=200, cols=3 * 288, headDim=36, srcStart=288, width=288)),
]


def _check(ex, c, dtype):
    import runntime_b200 as rt
    rows, cols, hd = c["rows"], c["cols"], c["headDim"]
    x = oracle.random_f32(rows * cols, 1)
    if dtype == "f16":
        x = oracle.round_f16(x)
    x = x.reshape(rows, cols)
    cos, sin = rope_tables(rows, hd)
    opts = dict(headDim=hd, srcStart=c.get("srcStart"), width=c.get("width"))
    got = rt.toArray(rt.rope(ex.upload(x, [rows, cols], dtype), ex.upload(cos, [rows, hd]),
                             ex.upload(sin, [rows, hd]), opts), ex)
    want = oracle.rope_ref(x, cos, sin, headDim=hd, srcStart=c.get("srcStart", 0) or 0,
                           width=c.get("width"))
    tol = dict(atol=1e-3, rtol=1e-3) if dtype == "f16" else dict(atol=1e-6, rtol=1e-6)
    assert np.all(np.abs(got - want.reshape(-1)) <= tol["atol"] + tol["rtol"] * np.abs(want.reshape(-1)))


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("name,c", CASES, ids=[n for n, _ in CASES])
def test_rope_cases(ex, dtype, name, c):
    _check(ex, c, dtype)


def test_rotates_by_the_angle_worked_out_by_hand(ex):
    # Position 1, headDim 2: angle 1, so (1, 0) turns to (cos 1, sin 1) and (0, 1)
    # to (-sin 1, cos 1).  (The reference's known-answer vector, rope.gpu.test.ts:110-116.)
    import runntime_b200 as rt
    x = ex.upload(np.array([1, 0, 0, 1], np.float32), [2, 2])
    cos = ex.upload(np.array([1, 1, math.cos(1), math.cos(1)], np.float32), [2, 2])
    sin = ex.upload(np.array([0, 0, math.sin(1), math.sin(1)], np.float32), [2, 2])
    got = rt.toArray(rt.rope(x, cos, sin, dict(headDim=2)), ex)
    want = np.array([1, 0, -math.sin(1), math.cos(1)])
    assert np.all(np.abs(got - want) <= 1e-7 + 1e-6 * np.abs(want))


def test_runs_past_2p24_elements(ex):
    _check(ex, dict(rows=4100, cols=4096, headDim=64), "f32")


def test_decoder_chain_rope_append_attend(ex):
    """q and kNew roped out of one fused qkv row, appended and attended (the decoder
    layer's step, packages/runntime/src/zoo/moonshine/decoder.ts:58-76)."""
    import runntime_b200 as rt
    heads, hd, t, rows = 8, 36, 57, 194
    w = heads * hd
    rnd = oracle.round_f16
    qkv = rnd(oracle.random_f32(3 * w, 21)).reshape(1, 3 * w)
    kc = rnd(oracle.random_f32(rows * w, 22)).reshape(rows, w)
    vc = rnd(oracle.random_f32(rows * w, 23)).reshape(rows, w)
    cos_all, sin_all = rope_tables(rows, hd)
    cos_all, sin_all = cos_all * hd ** -0.25, sin_all * hd ** -0.25  # score scale folded in
    cos, sin = cos_all[t:t + 1].copy(), sin_all[t:t + 1].copy()
    X = ex.upload(qkv, [1, 3 * w], "f16")
    C, S = ex.upload(cos, [1, hd]), ex.upload(sin, [1, hd])
    kcache, vcache = ex.upload(kc, [rows, w], "f16"), ex.upload(vc, [rows, w], "f16")
    q = rt.rope(X, C, S, dict(headDim=hd, srcStart=0, width=w))
    kNew = rt.rope(X, C, S, dict(headDim=hd, srcStart=w, width=w))
    vNew = ex.upload(qkv[:, 2 * w:], [1, w], "f16")
    k = rt.writeRows(kcache, kNew, t)
    v = rt.writeRows(vcache, vNew, t)
    mha = rt.MultiHeadAttention(dict(qHeads=heads, kvHeads=heads, headDim=hd,
                                     windowLeft=math.inf, windowRight=0))
    got = rt.toArray(mha.forward(q, k, v, dict(qPosOffset=t)), ex)
    q_ref = rnd(oracle.rope_ref(qkv, cos, sin, headDim=hd, srcStart=0, width=w).astype(np.float32))
    k_ref = rnd(oracle.rope_ref(qkv, cos, sin, headDim=hd, srcStart=w, width=w).astype(np.float32))
    kc[t], vc[t] = k_ref[0], qkv[0, 2 * w:]
    want = oracle.sdpa_ref(q_ref, kc[:t + 1], vc[:t + 1], qHeads=heads, kvHeads=heads, headDim=hd,
                           windowRight=0, qPosOffset=t)
    oracle.assert_close(got, want, "f16")
    got_k = ex.readback(kcache.buffer, kcache.shape).reshape(rows, w)
    assert np.array_equal(np.delete(got_k, t, 0), np.delete(kc, t, 0))
    assert np.all(np.abs(got_k[t] - kc[t]) <= 1e-3 + 1e-3 * np.abs(kc[t]))
