"""Pins the CPU oracle: analytic known answers, the committed golden fixtures
(made by an independent numpy restatement) and the shader-order f32 variant."""
import json
import math
import os

import numpy as np
import pytest

import cases
import oracle
from oracle import SdpaCase, make_inputs, sdpa_ref, sdpa_ref_inputs, sdpa_rows
from oracle.sdpa_numpy import sdpa_numpy

GOLDEN_DIR = os.path.join(os.path.dirname(__file__), "golden")


def _golden():
    with open(os.path.join(GOLDEN_DIR, "sdpa_golden.json")) as f:
        meta = json.load(f)
    data = np.load(os.path.join(GOLDEN_DIR, "sdpa_golden.npz"))
    return meta, data


def _case_from_meta(d):
    d = dict(d)
    for k in ("windowLeft", "windowRight"):
        if d[k] == "inf":
            d[k] = math.inf
    return SdpaCase(**d)


def test_generator_matches_lcg_definition():
    got = oracle.random_f32(5, 1)
    s, want = 1, []
    for _ in range(5):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        want.append(np.float32(s / 2 ** 31 - 1))
    assert np.array_equal(got, np.array(want, dtype=np.float32))
    assert (oracle.random_f32(1000, 7) >= -1).all() and (oracle.random_f32(1000, 7) < 1).all()


def test_round_f16_is_nearest_even():
    x = np.array([1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 65519.0, 1e-8], dtype=np.float32)
    got = oracle.round_f16(x)
    assert got[0] == 1.0 and got[1] == np.float32(1.0 + 2 ** -9) and got[2] == 65504.0
    assert got[3] == 0.0


def test_one_key_returns_v():
    q = np.ones((3, 8), np.float32)
    k = np.full((1, 4), 0.3, np.float32)
    v = np.arange(4, dtype=np.float32).reshape(1, 4)
    out = sdpa_ref(q, k, v, qHeads=2, kvHeads=1, headDim=4)
    assert np.allclose(out, np.tile(v, (3, 2)))


def test_uniform_scores_average_v():
    q = np.zeros((2, 4), np.float32)
    k = oracle.random_f32(5 * 4, 2).reshape(5, 4)
    v = oracle.random_f32(5 * 4, 3).reshape(5, 4)
    out = sdpa_ref(q, k, v, qHeads=1, kvHeads=1, headDim=4)
    assert np.allclose(out, np.tile(v.astype(np.float64).mean(0), (2, 1)))


def test_hand_worked_2x2():
    # scores row0 = [ln 1, ln 3] -> p = [1/4, 3/4]; row1 causal at qPos 0 sees key 0 only
    q = np.array([[1.0], [1.0]], np.float32)
    k = np.array([[0.0], [math.log(3.0)]], np.float32)
    v = np.array([[4.0], [8.0]], np.float32)
    out = sdpa_ref(q, k, v, qHeads=1, kvHeads=1, headDim=1)
    assert np.allclose(out[:, 0], [7.0, 7.0], rtol=1e-6)
    out = sdpa_ref(q, k, v, qHeads=1, kvHeads=1, headDim=1, windowRight=0)
    assert np.allclose(out[:, 0], [4.0, 7.0], rtol=1e-6)


def test_sink_only_and_empty_band_are_zero():
    q = np.ones((2, 2), np.float32)
    k = np.ones((2, 2), np.float32)
    v = np.ones((2, 2), np.float32)
    sinks = np.array([0.5], np.float32)
    out = sdpa_ref(q, k, v, qHeads=1, kvHeads=1, headDim=2, windowLeft=0, qPosOffset=5,
                   sinks=sinks)
    assert (out == 0).all()
    out = sdpa_ref(q, k, v, qHeads=1, kvHeads=1, headDim=2, windowLeft=0, qPosOffset=5)
    assert (out == 0).all()


def test_sink_enters_denominator_only():
    q = np.zeros((1, 1), np.float32)
    k = np.zeros((1, 1), np.float32)
    v = np.array([[6.0]], np.float32)
    sinks = np.array([1.0], np.float32)  # exp(1*ln2) = 2 -> out = 6 * 1/(1+2)
    out = sdpa_ref(q, k, v, qHeads=1, kvHeads=1, headDim=1, sinks=sinks)
    assert np.allclose(out, 2.0)


def test_oracle_matches_golden_fixtures():
    meta, data = _golden()
    assert len(meta) >= 60
    for name, m in meta.items():
        c = _case_from_meta(m["case"])
        got = sdpa_ref_inputs(make_inputs(c, m["dtype"]))
        assert np.allclose(got, data[name], rtol=1e-11, atol=1e-13), name


@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_oracle_matches_numpy_on_shapes(dtype):
    picks = [c for n, c in cases.PREFILL_SHAPES if c.qLen * c.kvLen <= 200 * 200]
    picks += [c for _, c in cases.flash_cases() if c.headDim <= 128]
    picks += [c for _, c in cases.option_cases(37, 40)]
    for c in picks:
        x = make_inputs(c, dtype)
        want = sdpa_numpy(x.q, x.k, x.v, qHeads=c.qHeads, kvHeads=c.kvHeads, headDim=c.headDim,
                          windowLeft=c.windowLeft, windowRight=c.windowRight,
                          qPosOffset=c.qPosOffset, sinks=x.sinks, segs=x.segs, keyBias=x.keyBias)
        assert np.allclose(sdpa_ref_inputs(x), want, rtol=1e-11, atol=1e-13), c


@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_shader_order_variant_within_reference_tolerance(dtype):
    for _, c in cases.option_cases(37, 40) + cases.option_cases(200, 16):
        x = make_inputs(c, dtype)
        npdt = np.float32 if dtype == "f32" else np.float16
        kw = dict(qHeads=c.qHeads, kvHeads=c.kvHeads, headDim=c.headDim,
                  windowLeft=c.windowLeft, windowRight=c.windowRight, qPosOffset=c.qPosOffset,
                  sinks=x.sinks, segs=x.segs, keyBias=x.keyBias)
        if c.packed:
            got = sdpa_rows(None, None, None, packed=x.packed_qkv.astype(npdt), **kw)
        else:
            got = sdpa_rows(x.q.astype(npdt), x.k.astype(npdt), x.v.astype(npdt), **kw)
        oracle.assert_close(got, sdpa_ref_inputs(x), dtype, str(c))


def test_merge_partials_equals_unsplit_attention():
    c = SdpaCase(qLen=1, kvLen=300, qHeads=4, kvHeads=2, headDim=16, qPosOffset=299,
                 windowRight=0)
    x = make_inputs(c, "f32")
    want = sdpa_ref_inputs(x)
    parts = []
    for lo, hi in ((0, 100), (100, 101), (101, 300)):
        rows = []
        for h in range(4):
            g = h // 2
            s = x.k[lo:hi, g * 16:(g + 1) * 16].astype(np.float64) @ x.q[0, h * 16:(h + 1) * 16]
            m = s.max()
            p = np.exp(s - m)
            rows.append(np.concatenate([[m, p.sum()], p @ x.v[lo:hi, g * 16:(g + 1) * 16]]))
        parts.append(rows)
    parts.append([[-1e30, 0.0] + [0.0] * 16 for _ in range(4)])  # an empty shard
    got = oracle.merge_partials(np.array(parts, dtype=np.float32))
    assert np.allclose(got.reshape(-1), want.reshape(-1), rtol=1e-5, atol=1e-6)


def test_write_rows_appends_in_place():
    dst = np.zeros((6, 4), np.float16)
    src = np.arange(8, dtype=np.float16).reshape(2, 4)
    view = oracle.write_rows(dst, src, 3)
    assert view.shape == (5, 4) and np.array_equal(dst[3:5], src) and (dst[:3] == 0).all()
    assert (dst[5] == 0).all()


# ---- rope -------------------------------------------------------------------------

def test_rope_hand_worked_vector():
    # packages/runntime/test/core/kernels/attention/rope.gpu.test.ts:110-116: position 1,
    # headDim 2, angle 1 turns (1, 0) to (cos 1, sin 1) and (0, 1) to (-sin 1, cos 1).
    x = np.array([[1, 0], [0, 1]], np.float32)
    cos = np.array([[1, 1], [math.cos(1)] * 2], np.float32)
    sin = np.array([[0, 0], [math.sin(1)] * 2], np.float32)
    got = oracle.rope_ref(x, cos, sin, headDim=2)
    want = np.array([[1, 0], [-np.float32(math.sin(1)), np.float32(math.cos(1))]], np.float64)
    assert np.allclose(got, want, rtol=0, atol=1e-12)


@pytest.mark.parametrize("rows,cols,hd,start,width", [
    (7, 60, 10, 0, None), (9, 128, 16, 64, 32), (3, 48, 16, 32, 16), (3, 136, 34, 0, None)])
def test_rope_against_numpy(rows, cols, hd, start, width):
    x = oracle.random_f32(rows * cols, 5).reshape(rows, cols)
    cos = oracle.random_f32(rows * hd, 6).reshape(rows, hd)
    sin = oracle.random_f32(rows * hd, 7).reshape(rows, hd)
    w = cols if width is None else width  # tables need not be pair-duplicated: entry 2p is read
    xs = x[:, start:start + w].astype(np.float64).reshape(rows, w // hd, hd // 2, 2)
    c = cos.astype(np.float64).reshape(rows, 1, hd // 2, 2)
    s = sin.astype(np.float64).reshape(rows, 1, hd // 2, 2)
    want = np.stack([xs[..., 0] * c[..., 0] - xs[..., 1] * s[..., 0],
                     xs[..., 1] * c[..., 0] + xs[..., 0] * s[..., 0]], -1).reshape(rows, w)
    got = oracle.rope_ref(x, cos, sin, headDim=hd, srcStart=start, width=width)
    assert np.allclose(got, want, rtol=1e-14, atol=1e-14)


# ---- softmax ----------------------------------------------------------------------

def test_softmax_matches_the_reference_known_answers():
    # packages/runntime/test/core/kernels/reduce/softmax.gpu.test.ts:100-122:
    # [1, 2, 3] -> e^[0, 1, 2] / (1 + e + e^2), the same as torch.softmax; 1000 more
    # only shifts the max.
    want = [0.09003057, 0.24472847, 0.66524096]
    got = oracle.softmax_ref(np.array([[1, 2, 3]], np.float32))
    assert np.allclose(got[0], want, rtol=1e-6, atol=1e-7)
    got = oracle.softmax_ref(np.array([[1001, 1002, 1003, -1000]], np.float32))
    assert np.allclose(got[0], want + [0], rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("n,wl,wr", [(12, math.inf, math.inf), (9, math.inf, 0), (136, 2, 1),
                                     (12, 0, 0)])
def test_masked_softmax_against_numpy(n, wl, wr):
    x = (8 * oracle.random_f32(n * n, 2)).reshape(n, n)
    half = n // 2
    segs = np.array([[0, half] if r < half else [half, n] for r in range(n)], np.float32)
    r, j = np.arange(n)[:, None], np.arange(n)[None, :]
    keep = (j >= segs[:, :1]) & (j < segs[:, 1:]) & (j >= r - wl) & (j <= r + wr)
    xs = np.where(keep, x.astype(np.float64), -np.inf)
    e = np.exp(xs - xs.max(axis=1, keepdims=True))
    want = e / e.sum(axis=1, keepdims=True)
    got = oracle.softmax_ref(x, segs, wl, wr)
    assert np.allclose(got, want, rtol=1e-13, atol=1e-15)
    assert (got[~keep] == 0).all()


# ---- localAttention -----------------------------------------------------------------

def _local_numpy(qkv, rel, qScale, heads, hd, window, kScale, softcap):
    """Independent numpy restatement: banded scores from full matrices."""
    rows, width = qkv.shape[0], heads * hd
    x = qkv.astype(np.float64)
    out = np.zeros((rows, width))
    for h in range(heads):
        q = x[:, h * hd:(h + 1) * hd] * qScale.astype(np.float64)
        k = x[:, width + h * hd:width + (h + 1) * hd] * kScale
        v = x[:, 2 * width + h * hd:2 * width + (h + 1) * hd]
        s = np.full((rows, rows), -np.inf)
        for j in range(window):
            r = rel[j, h * hd:(h + 1) * hd].astype(np.float64)
            t = np.arange(j, rows)
            s[t, t - j] = np.einsum("td,td->t", q[t], k[t - j] + r)
        s = softcap * np.tanh(s / softcap)
        s[np.isnan(s)] = -np.inf
        band = np.tril(np.ones((rows, rows), bool)) & ~np.tril(np.ones((rows, rows), bool), -window)
        s = np.where(band, s, -np.inf)
        e = np.exp(s - s.max(axis=1, keepdims=True))
        out[:, h * hd:(h + 1) * hd] = (e / e.sum(axis=1, keepdims=True)) @ v
    return out


@pytest.mark.parametrize("rows,heads,hd,window,kScale,softcap", [
    (50, 8, 128, 12, math.log1p(math.e) / math.log(2), 50), (6, 2, 8, 1, 1, 50),
    (40, 2, 16, 32, 1, 50), (3, 2, 8, 12, 1, 50), (16, 2, 32, 6, 4, 0.5), (10, 2, 8, 3, -1.5, 50)])
def test_local_attention_against_numpy(rows, heads, hd, window, kScale, softcap):
    width = heads * hd
    qkv = oracle.random_f32(rows * 3 * width, 1).reshape(rows, 3 * width)
    rel = oracle.random_f32(window * width, 2).reshape(window, width)
    qScale = oracle.random_f32(hd, 3)
    got = oracle.local_attention_ref(qkv, rel, qScale, heads=heads, headDim=hd, window=window,
                                     kScale=kScale, softcap=softcap)
    want = _local_numpy(qkv, rel, qScale, heads, hd, window, kScale, softcap)
    assert np.allclose(got, want, rtol=1e-11, atol=1e-13)


def test_local_attention_window_one_returns_v():
    rows, heads, hd = 6, 2, 8
    width = heads * hd
    qkv = oracle.random_f32(rows * 3 * width, 1).reshape(rows, 3 * width)
    got = oracle.local_attention_ref(qkv, np.zeros((1, width), np.float32),
                                     np.ones(hd, np.float32), heads=heads, headDim=hd, window=1)
    assert np.array_equal(got, qkv[:, 2 * width:].astype(np.float64))
