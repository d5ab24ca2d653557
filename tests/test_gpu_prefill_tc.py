"""The tensor-core prefill kernel (f16, head sizes 64/128/256): multi-tile
shapes, every mask family, GQA, sinks, key bias, packed qkv and the padded-batch
form, against the f64 oracle (f16 tolerance: atol 2e-3 + rtol 4e-3) and against
the FP32-pipe kernel on the same inputs."""
import math

import numpy as np
import pytest

import cases
import oracle
from gpu_harness import check_sdpa, ex, run_sdpa  # noqa: F401
from oracle import SdpaCase, make_inputs

pytestmark = pytest.mark.gpu
INF = math.inf


def _c(**kw):
    return SdpaCase(**kw)


TC_CASES = [
    ("one_tile_exact", _c(qLen=128, kvLen=128, qHeads=2, kvHeads=2, headDim=128)),
    ("two_rows", _c(qLen=2, kvLen=2, qHeads=1, kvHeads=1, headDim=64)),
    ("causal_1000", _c(qLen=1000, kvLen=1000, qHeads=2, kvHeads=1, headDim=128, windowRight=0)),
    ("causal_1000_hd64", _c(qLen=1000, kvLen=1000, qHeads=4, kvHeads=2, headDim=64,
                            windowRight=0)),
    ("causal_700_hd256", _c(qLen=700, kvLen=700, qHeads=3, kvHeads=1, headDim=256,
                            windowRight=0)),
    ("sliding_both_hd256", _c(qLen=900, kvLen=900, qHeads=3, kvHeads=1, headDim=256,
                              windowLeft=200, windowRight=200)),
    ("sliding_left_300", _c(qLen=1500, kvLen=1500, qHeads=2, kvHeads=2, headDim=128,
                            windowLeft=300, windowRight=0)),
    ("cross_300x2000", _c(qLen=300, kvLen=2000, qHeads=2, kvHeads=1, headDim=128)),
    ("qposoffset_into_cache", _c(qLen=200, kvLen=900, qHeads=2, kvHeads=1, headDim=64,
                                 windowRight=0, qPosOffset=700)),
    ("segments_two_halves", _c(qLen=1000, kvLen=1000, qHeads=2, kvHeads=2, headDim=128,
                               segments=True)),
    ("segments_causal_sinks", _c(qLen=777, kvLen=777, qHeads=4, kvHeads=2, headDim=64,
                                 segments=True, windowRight=0, sinks=True)),
    ("packed_causal", _c(qLen=600, kvLen=600, qHeads=4, kvHeads=2, headDim=64, packed=True,
                         windowRight=0)),
    ("packed_segments_sinks_hd128", _c(qLen=520, kvLen=520, qHeads=2, kvHeads=1, headDim=128,
                                       packed=True, segments=True, sinks=True)),
    ("keybias_reverb", _c(qLen=335, kvLen=640, qHeads=12, kvHeads=6, headDim=128, keyBias=True)),
    ("keybias_sinks_segments", _c(qLen=400, kvLen=400, qHeads=2, kvHeads=1, headDim=64,
                                  keyBias=True, sinks=True, segments=True)),
    ("rows_see_no_key", _c(qLen=300, kvLen=150, qHeads=2, kvHeads=1, headDim=64, windowLeft=0,
                           sinks=True)),
    ("long_keys_many_tiles", _c(qLen=130, kvLen=5000, qHeads=1, kvHeads=1, headDim=128)),
    ("window_narrower_than_tile", _c(qLen=1024, kvLen=1024, qHeads=1, kvHeads=1, headDim=128,
                                     windowLeft=5, windowRight=3)),
]


@pytest.fixture
def one_tile(ex):
    """The kernel with one 128-row query tile per thread block, for every shape."""
    from runntime_b200._lib import OPT_PREFILL_TC
    ex.setOption(OPT_PREFILL_TC, 2)
    yield ex
    ex.setOption(OPT_PREFILL_TC, 1)


@pytest.mark.parametrize("name,c", TC_CASES, ids=[n for n, _ in TC_CASES])
def test_tensor_core_prefill_against_oracle(one_tile, name, c):
    check_sdpa(one_tile, c, "f16", route="prefill_tc")


def test_default_routing_among_the_tensor_core_kernels(ex):
    """Every head size the tensor-core kernels take goes to the alternating-warpgroup kernel,
    whatever the grid."""
    small = _c(qLen=1000, kvLen=1000, qHeads=2, kvHeads=1, headDim=128, windowRight=0)
    check_sdpa(ex, small, "f16", route="prefill_tc3")
    big = _c(qLen=2304, kvLen=2304, qHeads=128, kvHeads=8, headDim=64, windowLeft=64, windowRight=0)
    check_sdpa(ex, big, "f16", route="prefill_tc3")
    check_sdpa(ex, big.with_(headDim=256, qHeads=32, kvHeads=8, qLen=512, kvLen=512), "f16",
               route="prefill_tc3")


@pytest.mark.parametrize("hd", [64, 128, 256])
def test_every_option_takes_the_tensor_core_route(one_tile, hd):
    for name, c in cases.option_cases(300, hd):
        if c.packed and hd > 128:
            continue
        check_sdpa(one_tile, c, "f16", route="prefill_tc")


def test_matches_the_fp32_pipe_kernel(ex):
    from runntime_b200._lib import OPT_PREFILL_TC
    c = _c(qLen=900, kvLen=900, qHeads=4, kvHeads=2, headDim=128, windowLeft=400, windowRight=0,
           sinks=True)
    x = make_inputs(c, "f16")
    ex.setOption(OPT_PREFILL_TC, 2)
    tc = run_sdpa(ex, x)
    assert ex.dispatches[-1] == "prefill_tc"
    ex.setOption(OPT_PREFILL_TC, 3)
    try:
        two = run_sdpa(ex, x)
        assert ex.dispatches[-1] == "prefill_tc2"
    finally:
        ex.setOption(OPT_PREFILL_TC, 1)
    assert np.abs(tc - two).max() < 1e-3
    ex.setOption(OPT_PREFILL_TC, 0)
    try:
        simt = run_sdpa(ex, x)
        assert ex.dispatches[-1] == "prefill_simt"
    finally:
        ex.setOption(OPT_PREFILL_TC, 1)
    assert np.abs(tc - simt).max() < 2e-3


@pytest.mark.parametrize("mode,route", [(2, "prefill_tc"), (3, "prefill_tc2")])
def test_large_scores_need_the_rescale_path(ex, mode, route):
    """Scores that keep growing along the keys force repeated accumulator rescales
    (in the two-tile kernel: every tile's first half is computed twice)."""
    import runntime_b200 as rt
    from runntime_b200._lib import OPT_PREFILL_TC
    T, hd = 640, 64
    rng = np.random.default_rng(1)
    q = np.ones((T, hd), np.float32) * 0.25
    k = (np.arange(T, dtype=np.float32)[:, None] / 16.0 * np.ones((1, hd), np.float32)) / 4
    k = oracle.round_f16(k.astype(np.float32))
    v = oracle.round_f16(rng.standard_normal((T, hd)).astype(np.float32))
    opts = dict(qHeads=1, kvHeads=1, headDim=hd, windowLeft=INF, windowRight=INF)
    ex.setOption(OPT_PREFILL_TC, mode)
    try:
        out = rt.toArray(rt.sdpa(ex.upload(q, [T, hd], "f16"), ex.upload(k, [T, hd], "f16"),
                                 ex.upload(v, [T, hd], "f16"), opts), ex)
    finally:
        ex.setOption(OPT_PREFILL_TC, 1)
    assert ex.dispatches[-1] == route
    want = oracle.sdpa_ref(q, k, v, qHeads=1, kvHeads=1, headDim=hd)
    oracle.assert_close(out, want, "f16")


def test_n_of_1_inputs_at_long_sequence_keep_the_tolerance(ex):
    """N(0,1) values at head size 128 over 4096 keys: P rounded to f16 for the
    second product must still meet 2e-3 absolute."""
    import runntime_b200 as rt
    T, hd = 4096, 128
    rng = np.random.default_rng(2)
    f = hd ** -0.25
    q = oracle.round_f16((rng.standard_normal((256, hd)) * f).astype(np.float32))
    k = oracle.round_f16((rng.standard_normal((T, hd)) * f).astype(np.float32))
    v = oracle.round_f16(rng.standard_normal((T, hd)).astype(np.float32))
    opts = dict(qHeads=1, kvHeads=1, headDim=hd, windowLeft=INF, windowRight=0,
                qPosOffset=T - 256)
    out = rt.toArray(rt.sdpa(ex.upload(q, [256, hd], "f16"), ex.upload(k, [T, hd], "f16"),
                             ex.upload(v, [T, hd], "f16"), opts), ex)
    want = oracle.sdpa_ref(q, k, v, qHeads=1, kvHeads=1, headDim=hd, windowRight=0,
                           qPosOffset=T - 256)
    assert np.abs(out.reshape(want.shape) - want).max() <= 2e-3


@pytest.mark.parametrize("hd,heads,kvHeads,wl,wr,packed", [
    (256, 3, 1, 512, 512, False),    # EmbeddingGemma sliding layer
    (256, 3, 1, INF, INF, False),    # EmbeddingGemma global layer
    (64, 4, 4, INF, INF, True),      # a packed bidirectional encoder batch
    (128, 8, 8, INF, 0, True),
])
def test_greedy_packed_batch_of_ragged_sequences(ex, hd, heads, kvHeads, wl, wr, packed):
    """Sequences of unequal length packed back to back, a [start, end) range per
    row, T rounded up with rows that keep nothing — the batch the embedders build
    (packages/runntime/src/zoo/embeddinggemma2/embedCore.ts:43-73,131-134) — on
    the tensor-core kernel: row tiles straddle several sequences."""
    lens = [37, 300, 5, 130, 1, 263, 128, 129]
    T = (sum(lens) + 3) // 4 * 4 + 4          # padded rows at the end
    c = _c(qLen=T, kvLen=T, qHeads=heads, kvHeads=kvHeads, headDim=hd, windowLeft=wl,
           windowRight=wr, segments=True, packed=packed, maxSegment=max(lens))
    x = make_inputs(c, "f16")
    segs = np.zeros((T, 2), np.float32)
    at = 0
    for n in lens:
        segs[at:at + n] = (at, at + n)
        at += n
    x.segs = segs
    got = run_sdpa(ex, x)
    assert ex.dispatches[-1] == "prefill_tc3"      # the library's own choice at every head size
    want = oracle.sdpa_ref_inputs(x)
    oracle.assert_close(got, want, "f16")
    assert (got.reshape(T, -1)[at:] == 0).all()


# ---- two query tiles per thread block (head sizes 64 and 128) ----------------------

@pytest.fixture
def two_tiles(ex):
    from runntime_b200._lib import OPT_PREFILL_TC
    ex.setOption(OPT_PREFILL_TC, 3)
    yield ex
    ex.setOption(OPT_PREFILL_TC, 1)


def _two_tile_ok(c):
    return c.headDim in (64, 128) and c.qLen > 128


TWO_TILE_CASES = [(n, c) for n, c in TC_CASES if _two_tile_ok(c)] + [
    ("causal_odd_rows", _c(qLen=1000, kvLen=1000, qHeads=2, kvHeads=1, headDim=128, windowRight=0)),
    ("second_tile_partly_past_the_end", _c(qLen=300, kvLen=300, qHeads=1, kvHeads=1, headDim=64,
                                           windowRight=0)),
    ("second_tile_empty_band", _c(qLen=256, kvLen=100, qHeads=1, kvHeads=1, headDim=64,
                                  windowLeft=0, windowRight=INF, qPosOffset=0)),
    ("cross_long_keys", _c(qLen=257, kvLen=3000, qHeads=4, kvHeads=2, headDim=128)),
    ("sliding_window_gqa_sinks", _c(qLen=1500, kvLen=1500, qHeads=6, kvHeads=2, headDim=64,
                                    windowLeft=200, windowRight=0, sinks=True)),
    ("decode_chunk_offset", _c(qLen=384, kvLen=2048, qHeads=2, kvHeads=2, headDim=128,
                               windowRight=0, qPosOffset=1664)),
]


@pytest.mark.parametrize("name,c", TWO_TILE_CASES, ids=[n for n, _ in TWO_TILE_CASES])
def test_two_tile_kernel_against_oracle(two_tiles, name, c):
    check_sdpa(two_tiles, c, "f16", route="prefill_tc2")


@pytest.mark.parametrize("hd", [64, 128])
def test_every_option_on_the_two_tile_kernel(two_tiles, hd):
    for name, c in cases.option_cases(300, hd):
        check_sdpa(two_tiles, c, "f16", route="prefill_tc2")
