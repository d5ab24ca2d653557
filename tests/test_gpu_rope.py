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


def _decoder_step_inputs(dtype, heads, kvHeads, hd, rows, seed):
    rnd = oracle.round_f16 if dtype == "f16" else (lambda a: a)
    qw, kvw = heads * hd, kvHeads * hd
    qkv = rnd(oracle.random_f32(qw + 2 * kvw, seed)).reshape(1, -1)
    qkv[:, :qw] *= 0.5
    kc = rnd(oracle.random_f32(rows * kvw, seed + 1)).reshape(rows, kvw)
    vc = rnd(oracle.random_f32(rows * kvw, seed + 2)).reshape(rows, kvw)
    cos_all, sin_all = rope_tables(rows, hd)
    s = hd ** -0.25  # the score scale, folded into the tables as the reference does
    return qkv, kc, vc, cos_all * s, sin_all * s


def _decoder_step(ex, dtype, heads, kvHeads, hd, rows, t, *, fused, seed=21):
    """q and kNew roped out of one fused qkv row, vNew sliced out of it, appended
    and attended (packages/runntime/src/zoo/moonshine/decoder.ts:58-76).  Returns
    (out, kCache, vCache, inputs, dispatches)."""
    import runntime_b200 as rt
    qw, kvw = heads * hd, kvHeads * hd
    qkv, kc, vc, cos_all, sin_all = _decoder_step_inputs(dtype, heads, kvHeads, hd, rows, seed)
    cos, sin = cos_all[t:t + 1].copy(), sin_all[t:t + 1].copy()
    X = ex.upload(qkv, [1, qw + 2 * kvw], dtype)
    C, S = ex.upload(cos, [1, hd]), ex.upload(sin, [1, hd])
    kcache, vcache = ex.upload(kc, [rows, kvw], dtype), ex.upload(vc, [rows, kvw], dtype)
    q = rt.rope(X, C, S, dict(headDim=hd, srcStart=0, width=qw))
    kNew = rt.rope(X, C, S, dict(headDim=hd, srcStart=qw, width=kvw))
    vNew = rt.slice(X, 1, qw + kvw, qw + 2 * kvw)
    k = rt.writeRows(kcache, kNew, t)
    v = rt.writeRows(vcache, vNew, t)
    mha = rt.MultiHeadAttention(dict(qHeads=heads, kvHeads=kvHeads, headDim=hd,
                                     windowLeft=math.inf, windowRight=0))
    y = mha.forward(q, k, v, dict(qPosOffset=t))
    del ex.dispatches[:]
    if fused:
        rt.evalValues([y], ex)
    else:
        rt.evalValues([y, q, kNew, vNew, k, v], ex)  # all wanted by the caller: no fusion
    out = ex.readback(y.buffer, y.shape)
    return (out, ex.readback(kcache.buffer, kcache.shape).reshape(rows, kvw),
            ex.readback(vcache.buffer, vcache.shape).reshape(rows, kvw),
            (qkv, kc, vc, cos, sin), list(ex.dispatches))


@pytest.mark.parametrize("dtype,heads,kvHeads,hd,rows,t", [
    ("f16", 8, 8, 36, 194, 57),     # Moonshine tiny
    ("f16", 8, 8, 52, 194, 193),    # Moonshine base, last position
    ("f16", 8, 8, 36, 194, 0),      # first token: only the appended row
    ("f32", 8, 8, 36, 448, 300),    # split route
    ("f16", 14, 2, 64, 600, 511),   # GQA
    ("f32", 4, 4, 38, 64, 9),       # head width off the vector paths
    ("f16", 8, 8, 128, 300, 299),
    ("f32", 8, 8, 128, 200, 150),    # four threads per (key, head) pair, f32 rows
    ("f32", 4, 4, 64, 333, 332),     # two threads per pair
    ("f16", 32, 32, 128, 700, 650),  # a wide model: two keys of all heads per tile
    ("f16", 32, 8, 128, 300, 0),     # first token, grouped heads
])
def test_decoder_layer_step_in_one_launch(ex, dtype, heads, kvHeads, hd, rows, t):
    qw, kvw = heads * hd, kvHeads * hd
    got, gk, gv, (qkv, kc, vc, cos, sin), log = _decoder_step(
        ex, dtype, heads, kvHeads, hd, rows, t, fused=True)
    assert log == ["decode+rope+append"]
    rnd = oracle.round_f16 if dtype == "f16" else (lambda a: a.astype(np.float32))
    q_ref = rnd(oracle.rope_ref(qkv, cos, sin, headDim=hd, srcStart=0, width=qw).astype(np.float32))
    k_ref = rnd(oracle.rope_ref(qkv, cos, sin, headDim=hd, srcStart=qw, width=kvw).astype(np.float32))
    kc2, vc2 = kc.copy(), vc.copy()
    kc2[t], vc2[t] = k_ref[0], qkv[0, qw + kvw:]
    want = oracle.sdpa_ref(q_ref, kc2[:t + 1], vc2[:t + 1], qHeads=heads, kvHeads=kvHeads,
                           headDim=hd, windowRight=0, qPosOffset=t)
    oracle.assert_close(got, want, dtype)
    # the append: row t holds the rotated k and the v slice, every other row is untouched
    assert np.array_equal(np.delete(gk, t, 0), np.delete(kc, t, 0))
    assert np.array_equal(gv, vc2)
    tol = 1e-3 if dtype == "f16" else 1e-6
    assert np.all(np.abs(gk[t] - kc2[t]) <= tol + tol * np.abs(kc2[t]))
    # and the six separate dispatches of the reference leave the same bits in the caches
    # (the output may differ in its last place: the new row is then one more cache key and
    # is summed in another order)
    got2, gk2, gv2, _, log2 = _decoder_step(ex, dtype, heads, kvHeads, hd, rows, t, fused=False)
    assert sorted(log2) == sorted(["rope", "rope", "sliceCols", "writeRows", "writeRows", "decode"])
    assert np.array_equal(gk, gk2) and np.array_equal(gv, gv2)
    oracle.assert_close(got, got2, dtype)


def test_batched_steps_from_the_fused_projection(ex):
    """KvCacheEngine.stepQkv: every sequence at its own position, one table for the model."""
    import torch
    from runntime_b200.engine import KvCacheEngine
    batch, heads, hd, maxPos, steps = 5, 8, 36, 96, 12
    w = heads * hd
    eng = KvCacheEngine(ex, batch=batch, maxPositions=maxPos, qHeads=heads, kvHeads=heads,
                        headDim=hd, dtype="f16")
    dev = eng.k.device
    cos, sin = rope_tables(maxPos, hd)
    cos, sin = cos * hd ** -0.25, sin * hd ** -0.25
    eng.setRope(torch.from_numpy(cos).to(dev), torch.from_numpy(sin).to(dev))
    start = [0, 3, 17, 40, 80]           # ragged: sequences already hold this many rows
    g = torch.Generator().manual_seed(11)
    k0 = torch.randn(batch, maxPos, w, generator=g).half()
    v0 = torch.randn(batch, maxPos, w, generator=g).half()
    eng.k.copy_(k0)
    eng.v.copy_(v0)
    eng.lens.copy_(torch.tensor(start, dtype=torch.int32))
    eng.maxLen = max(start)
    kRef, vRef = k0.float().numpy().copy(), v0.float().numpy().copy()
    out = torch.empty(batch, w, dtype=torch.float16, device=dev)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        for step in range(steps):
            qkv = torch.randn(batch, 3 * w, generator=g).half()
            eng.stepQkv(qkv.to(dev), out)
            ex.sync()
            got = out.float().cpu().numpy()
            x = qkv.float().numpy()
            for b in range(batch):
                t = start[b] + step
                c, s = cos[t:t + 1], sin[t:t + 1]
                rnd = oracle.round_f16
                qr = rnd(oracle.rope_ref(x[b:b + 1], c, s, headDim=hd, srcStart=0, width=w)
                         .astype(np.float32))
                kr = rnd(oracle.rope_ref(x[b:b + 1], c, s, headDim=hd, srcStart=w, width=w)
                         .astype(np.float32))
                kRef[b, t], vRef[b, t] = kr[0], x[b, 2 * w:]
                want = oracle.sdpa_ref(qr, kRef[b, :t + 1], vRef[b, :t + 1], qHeads=heads,
                                       kvHeads=heads, headDim=hd, windowRight=0, qPosOffset=t)
                oracle.assert_close(got[b], want.reshape(-1), "f16", f"step {step} seq {b}")
    finally:
        ex.setStream(None)
    gk = eng.k.float().cpu().numpy()
    assert np.all(np.abs(gk - kRef) <= 1e-3 + 1e-3 * np.abs(kRef))
    assert np.array_equal(eng.v.float().cpu().numpy(), vRef)


@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_slice_and_chunk(ex, dtype):
    import runntime_b200 as rt
    rows, cols = 37, 3 * 52
    x = oracle.random_f32(rows * cols, 9)
    x = (oracle.round_f16(x) if dtype == "f16" else x).reshape(rows, cols)
    X = ex.upload(x, [rows, cols], dtype)
    assert np.array_equal(rt.toArray(rt.slice(X, 1, 52, 130), ex).reshape(rows, -1), x[:, 52:130])
    assert np.array_equal(rt.toArray(rt.slice(X, 1, 1, 2), ex).reshape(rows, -1), x[:, 1:2])
    assert np.array_equal(rt.toArray(rt.slice(X, 0, 5, 30), ex).reshape(-1, cols), x[5:30])
    parts = rt.chunk(X, 3, 1)
    rt.evalValues(parts, ex)
    for i, p in enumerate(parts):
        assert np.array_equal(ex.readback(p.buffer, p.shape).reshape(rows, -1),
                              x[:, i * 52:(i + 1) * 52])
