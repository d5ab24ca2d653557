"""localAttention on the GPU against the f64 oracle: the reference suite's cases
(packages/runntime/test/core/kernels/attention/attnLocal.gpu.test.ts:100-178)."""
import math

import numpy as np
import pytest

import oracle
from gpu_harness import ex  # noqa: F401

pytestmark = pytest.mark.gpu

GEMMA_K_SCALE = math.log1p(math.e) / math.log(2)   # k's scale in the EmbeddingGemma 2 audio tower

CASES = [
    ("gemma_audio_layer", dict(rows=50, heads=8, headDim=128, window=12, kScale=GEMMA_K_SCALE)),
    ("window_1", dict(rows=6, heads=2, headDim=8, window=1)),
    ("largest_window", dict(rows=40, heads=2, headDim=16, window=32)),
    ("fewer_rows_than_window", dict(rows=3, heads=2, headDim=8, window=12)),
    ("one_row", dict(rows=1, heads=1, headDim=8, window=12)),
    ("head_of_4", dict(rows=9, heads=3, headDim=4, window=5)),
    ("head_wider_than_128", dict(rows=7, heads=1, headDim=136, window=4)),
    ("head_wider_than_512", dict(rows=37, heads=2, headDim=640, window=7)),
    ("saturating_softcap", dict(rows=16, heads=2, headDim=32, window=6, kScale=4, softcap=0.5)),
    ("negative_kscale", dict(rows=10, heads=2, headDim=8, window=3, kScale=-1.5)),
    ("many_groups", dict(rows=8200, heads=8, headDim=4, window=3)),
    ("gemma_audio_30s", dict(rows=750, heads=8, headDim=128, window=12, kScale=GEMMA_K_SCALE)),
]


def check(ex, c, dtype):
    import runntime_b200 as rt
    rows, heads, hd, window = c["rows"], c["heads"], c["headDim"], c["window"]
    kScale, softcap = c.get("kScale", 1), c.get("softcap", 50)
    width = heads * hd
    # The oracle sees the f16-rounded qkv the kernel reads; rel and qScale are f32 in both.
    qkv = oracle.random_f32(rows * 3 * width, 1)
    qkv = (oracle.round_f16(qkv) if dtype == "f16" else qkv).reshape(rows, 3 * width)
    rel = oracle.random_f32(window * width, 2).reshape(window, width)
    qScale = oracle.random_f32(hd, 3)
    got = rt.toArray(rt.localAttention(
        ex.upload(qkv, [rows, 3 * width], dtype), ex.upload(rel, [window, width]),
        ex.upload(qScale, [1, hd]),
        dict(heads=heads, headDim=hd, window=window, kScale=kScale, softcap=softcap)), ex)
    want = oracle.local_attention_ref(qkv, rel, qScale, heads=heads, headDim=hd, window=window,
                                      kScale=kScale, softcap=softcap).reshape(-1)
    # f16 output adds 2^-11 relative.
    atol, rtol = (1e-3, 2e-3) if dtype == "f16" else (1e-5, 1e-4)
    bad = np.abs(got - want) > atol + rtol * np.abs(want)
    assert not bad.any(), f"{bad.sum()} of {bad.size} off, worst {np.abs(got - want).max()}"


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("name,c", CASES, ids=[n for n, _ in CASES])
def test_local_attention(ex, dtype, name, c):
    check(ex, c, dtype)


def test_qkv_past_2p24_elements(ex):
    check(ex, dict(rows=5462, heads=8, headDim=128, window=12, kScale=GEMMA_K_SCALE), "f32")
