"""The projections either side of attention on the GPU against numpy f64:
matmul with its bias / activation / addend epilogue, the baseRow view, and
argmaxDot (shapes after packages/runntime/test/core/kernels/matmul/*.gpu.test.ts
and the decoder layer's projections)."""
import math

import numpy as np
import pytest

import oracle
from gpu_harness import ex  # noqa: F401

pytestmark = pytest.mark.gpu


def act_ref(x, name):
    if name is None:
        return x
    if name == "tanh":
        return np.tanh(x)
    if name == "gelu":
        from math import erf
        return 0.5 * x * (1 + np.vectorize(erf)(x / math.sqrt(2)))
    if name == "silu":
        return x / (1 + np.exp(-x))
    if name == "relu":
        return np.maximum(x, 0)
    if name == "geluTanh":
        return 0.5 * x * (1 + np.tanh(math.sqrt(2 / math.pi) * (x + 0.044715 * x ** 3)))
    if name == "elu":
        return np.where(x > 0, x, np.exp(np.minimum(x, 0)) - 1)
    raise AssertionError(name)


def check(ex, m, k, n, dtype, *, bias=False, addend=False, act=None, baseRow=None, extra=0):
    import runntime_b200 as rt
    rnd = oracle.round_f16 if dtype == "f16" else (lambda a: a)
    a = rnd(oracle.random_f32(m * k, 1)).reshape(m, k)
    bRows = k + extra
    b = rnd(oracle.random_f32(bRows * n, 2) * (2 / math.sqrt(k))).reshape(bRows, n)
    opts = {}
    base = 0 if baseRow is None else baseRow
    want = a.astype(np.float64) @ b[base:base + k].astype(np.float64)
    if bias:
        bv = rnd(oracle.random_f32(n, 3))
        opts["bias"] = ex.upload(bv, [n], dtype)
        want = want + bv
    want = act_ref(want, act)
    if act:
        opts["activation"] = act
    if addend:
        av = rnd(oracle.random_f32(m * n, 4)).reshape(m, n)
        opts["addend"] = ex.upload(av, [m, n], dtype)
        want = want + av
    if baseRow is not None:
        opts["baseRow"] = baseRow
    got = rt.toArray(rt.matmul(ex.upload(a, [m, k], dtype), ex.upload(b, [bRows, n], dtype), opts),
                     ex).reshape(m, n)
    # f32: sums of k products in f32; f16: output rounding 2^-11 (and f16 inputs are exact)
    atol, rtol = (2e-3, 4e-3) if dtype == "f16" else (1e-5 * math.sqrt(k), 1e-4)
    bad = np.abs(got - want) > atol + rtol * np.abs(want)
    assert not bad.any(), f"{bad.sum()} of {bad.size} off, worst {np.abs(got - want).max()}"


SHAPES = [(1, 288, 864), (1, 416, 1248), (1, 288, 288), (8, 288, 864), (13, 416, 1248),
          (16, 64, 136), (1, 1, 1), (2, 3, 5), (4, 3, 1), (1, 300, 52), (17, 288, 864),
          (200, 288, 864), (130, 77, 100), (64, 416, 416)]


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("m,k,n", SHAPES)
def test_matmul_shapes(ex, dtype, m, k, n):
    check(ex, m, k, n, dtype)


TC_SHAPES = [(128, 64, 128), (129, 64, 64), (1000, 1024, 1536), (300, 520, 72), (2048, 288, 864),
             (17, 4096, 128), (256, 200, 1000)]


@pytest.mark.parametrize("m,k,n", TC_SHAPES)
def test_matmul_on_the_tensor_cores(ex, m, k, n):
    """f16, more than 16 rows, 16-byte row pitches: the tcgen05 kernel; the same shapes
    through the FP32-pipe kernel (option off) agree with it."""
    import runntime_b200 as rt
    from runntime_b200._lib import OPT_PREFILL_TC
    check(ex, m, k, n, "f16", bias=True, addend=True, act="silu")
    check(ex, m, k, n, "f16")
    ex.setOption(OPT_PREFILL_TC, 0)
    try:
        check(ex, m, k, n, "f16")
    finally:
        ex.setOption(OPT_PREFILL_TC, 1)


# (m, k, n): one to eight K slices per column tile, ragged last K step and column tile,
# a K that leaves the last slice empty (k = 576: nine steps over four slices of three).
SKINNY_TC_SHAPES = [(1, 64, 128), (8, 4096, 12288), (9, 1024, 4096), (16, 4096, 1024), (3, 200, 136),
                    (8, 576, 2048), (5, 8192, 128), (16, 72, 40000), (2, 2048, 6144)]


@pytest.mark.parametrize("m,k,n", SKINNY_TC_SHAPES)
def test_decode_step_matmul_on_the_tensor_cores(ex, m, k, n):
    """f16, up to 16 rows, at least 128 columns: the cluster kernel (K slices reduced
    through distributed shared memory); the FP32-pipe kernel (option off) agrees."""
    from runntime_b200._lib import OPT_PREFILL_TC
    check(ex, m, k, n, "f16", bias=True, addend=True, act="gelu")
    check(ex, m, k, n, "f16")
    ex.setOption(OPT_PREFILL_TC, 0)
    try:
        check(ex, m, k, n, "f16")
    finally:
        ex.setOption(OPT_PREFILL_TC, 1)


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("m", [1, 5, 40])
@pytest.mark.parametrize("act", [None, "tanh", "gelu", "silu", "relu", "geluTanh", "elu"])
def test_matmul_epilogue(ex, dtype, m, act):
    check(ex, m, 96, 264, dtype, bias=True, addend=True, act=act)


@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_matmul_views_rows_of_a_taller_weight(ex, dtype):
    check(ex, 3, 64, 128, dtype, baseRow=64, extra=128, bias=True)
    check(ex, 33, 64, 128, dtype, baseRow=128, extra=128)


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("rows,cols", [(50000, 16), (32768, 288), (7, 5), (1, 1), (1000, 417)])
def test_argmax_dot(ex, dtype, rows, cols):
    import runntime_b200 as rt
    rnd = oracle.round_f16 if dtype == "f16" else (lambda a: a)
    w = rnd(oracle.random_f32(rows * cols, 5)).reshape(rows, cols)
    x = rnd(oracle.random_f32(cols, 6)).reshape(1, cols)
    got = rt.toArray(rt.argmaxDot(ex.upload(w, [rows, cols], dtype), ex.upload(x, [1, cols], dtype)), ex)
    logits = w.astype(np.float64) @ x[0].astype(np.float64)
    best = int(got[0])
    # the winner's logit is the maximum up to f32 summation error
    assert logits[best] >= logits.max() - 1e-4 * math.sqrt(cols)


def test_argmax_dot_takes_the_lowest_index_on_ties(ex):
    import runntime_b200 as rt
    w = np.zeros((4096, 8), np.float32)
    w[[77, 1500, 4000]] = 1.0
    x = np.ones((1, 8), np.float32)
    got = rt.toArray(rt.argmaxDot(ex.upload(w, [4096, 8]), ex.upload(x, [1, 8])), ex)
    assert int(got[0]) == 77
