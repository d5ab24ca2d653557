"""Row softmax on the GPU against the f64 oracle: the reference suite's shapes,
known answers and masks
(packages/runntime/test/core/kernels/reduce/softmax.gpu.test.ts:57-170)."""
import math

import numpy as np
import pytest

import oracle
from gpu_harness import ex  # noqa: F401

pytestmark = pytest.mark.gpu
INF = math.inf

# f32: exp and the division are a few ulp each; f16 output adds 2^-11 relative.
TOLERANCE = {"f32": dict(atol=1e-7, rtol=1e-5), "f16": dict(atol=1e-5, rtol=2e-3)}


def close(got, want, dtype):
    t = TOLERANCE[dtype]
    want = np.asarray(want, np.float64).reshape(-1)
    bad = np.abs(got - want) > t["atol"] + t["rtol"] * np.abs(want)
    assert not bad.any(), f"{bad.sum()} of {bad.size} off, worst {np.abs(got - want).max()}"


SHAPES = [(3, 4), (5, 128), (2, 260), (1, 32768), (70000, 4), (1, 1), (3, 7), (4, 65),
          (37, 1001), (70000, 3), (9, 2048), (3, 2052), (2, 4099)]


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("rows,cols", SHAPES)
def test_softmax_shapes(ex, dtype, rows, cols):
    import runntime_b200 as rt
    # Scaled so a row spans e^+-8 and the running max has to rescale the sum.
    x = 8 * oracle.random_f32(rows * cols, 1)
    x = (oracle.round_f16(x) if dtype == "f16" else x).reshape(rows, cols)
    got = rt.toArray(rt.softmax(ex.upload(x, [rows, cols], dtype)), ex)
    close(got, oracle.softmax_ref(x), dtype)


@pytest.mark.parametrize("x,want", [
    ([1, 2, 3], [0.09003057, 0.24472847, 0.66524096]),
    ([1001, 1002, 1003, -1000], [0.09003057, 0.24472847, 0.66524096, 0]),
])
def test_softmax_matches_torch_known_answers(ex, x, want):
    import runntime_b200 as rt
    got = rt.toArray(rt.softmax(ex.upload(np.array(x, np.float32), [1, len(x)])), ex)
    assert np.all(np.abs(got - want) <= 1e-7 + 1e-6 * np.abs(want))


MASKS = [(INF, INF), (INF, 0), (2, 1), (0, 0)]


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("n", [12, 9, 136, 1000])
@pytest.mark.parametrize("wl,wr", MASKS)
def test_masked_softmax(ex, dtype, n, wl, wr):
    import runntime_b200 as rt
    half = n // 2
    x = 8 * oracle.random_f32(n * n, 2)
    x = (oracle.round_f16(x) if dtype == "f16" else x).reshape(n, n)
    segs = np.array([[0, half] if r < half else [half, n] for r in range(n)], np.float32)
    got = rt.toArray(rt.softmax(ex.upload(x, [n, n], dtype),
                                dict(segments=ex.upload(segs, [n, 2]), windowLeft=wl,
                                     windowRight=wr)), ex)
    close(got, oracle.softmax_ref(x, segs, wl, wr), dtype)


def test_a_row_that_keeps_nothing_is_zero(ex):
    import runntime_b200 as rt
    n = 8
    x = oracle.random_f32(n * n, 3).reshape(n, n)
    segs = np.array([[0, n]] * n, np.float32)
    segs[3] = (5, 5)       # empty range
    segs[6] = (0, 2)       # range that the causal window never reaches... it does: keeps 0, 1
    got = rt.toArray(rt.softmax(ex.upload(x, [n, n]), dict(segments=ex.upload(segs, [n, 2]),
                                                          windowLeft=1, windowRight=0)), ex)
    got = got.reshape(n, n)
    assert (got[3] == 0).all() and (got[6] == 0).all()   # row 6 sees keys 5..6, range is [0, 2)
    assert abs(got[2].sum() - 1) < 1e-6


def test_softmax_runs_past_2p24_elements(ex):
    import runntime_b200 as rt
    rows, cols = 4100, 4096
    x = oracle.random_f32(rows * cols, 3).reshape(rows, cols)
    got = rt.toArray(rt.softmax(ex.upload(x, [rows, cols])), ex)
    close(got, oracle.softmax_ref(x), "f32")


def test_matmul_attention_path_agrees_with_the_fused_op(ex):
    """softmax(q k^T) v with the masked softmax equals sdpaPacked's answer: the
    equivalence the reference keeps both paths for
    (packages/runntime/src/core/kernels/reduce/softmax.ts:128-133)."""
    import runntime_b200 as rt
    t, heads, hd = 96, 1, 32
    q = oracle.random_f32(t * hd, 1).reshape(t, hd) * hd ** -0.5 * 2
    k = oracle.random_f32(t * hd, 2).reshape(t, hd)
    v = oracle.random_f32(t * hd, 3).reshape(t, hd)
    segs = np.array([[0, 40]] * 40 + [[40, 96]] * 56, np.float32)
    scores = (q.astype(np.float64) @ k.astype(np.float64).T).astype(np.float32)
    S = ex.upload(segs, [t, 2])
    probs = rt.toArray(rt.softmax(ex.upload(scores, [t, t]),
                                  dict(segments=S, windowLeft=8, windowRight=8)), ex).reshape(t, t)
    viaMatmul = probs.astype(np.float64) @ v.astype(np.float64)
    fused = rt.toArray(rt.sdpa(ex.upload(q, [t, hd]), ex.upload(k, [t, hd]), ex.upload(v, [t, hd]),
                               dict(qHeads=heads, kvHeads=heads, headDim=hd, windowLeft=8,
                                    windowRight=8, segments=S)), ex).reshape(t, hd)
    assert np.all(np.abs(fused - viaMatmul) <= 2e-5 + 1e-4 * np.abs(viaMatmul))
