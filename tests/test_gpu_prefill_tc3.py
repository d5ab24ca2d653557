"""The tensor-core prefill kernel with two softmax warpgroups on alternate key tiles
(f16; head sizes 64/128/256 and the narrow heads 32/36/52 padded inside the tile):
every case of the other tensor-core kernels, the shared running maximum's rescale
path, and the zoo shapes with narrow heads, against the f64 oracle (f16 tolerance:
atol 2e-3 + rtol 4e-3)."""
import math

import numpy as np
import pytest

import cases
import oracle
from gpu_harness import check_sdpa, ex, run_sdpa  # noqa: F401
from oracle import SdpaCase, make_inputs
from test_gpu_prefill_tc import TC_CASES, TWO_TILE_CASES

pytestmark = pytest.mark.gpu
INF = math.inf


def _c(**kw):
    return SdpaCase(**kw)


@pytest.fixture
def alt(ex):
    """Routes every eligible shape to the alternating-warpgroup kernel."""
    from runntime_b200._lib import OPT_PREFILL_TC
    ex.setOption(OPT_PREFILL_TC, 4)
    yield ex
    ex.setOption(OPT_PREFILL_TC, 1)


ALL = {n: c for n, c in TC_CASES + TWO_TILE_CASES}


@pytest.mark.parametrize("name", sorted(ALL))
def test_alternating_warpgroups_against_oracle(alt, name):
    check_sdpa(alt, ALL[name], "f16", route="prefill_tc3")


@pytest.mark.parametrize("hd", [64, 128, 256])
def test_every_option(alt, hd):
    for name, c in cases.option_cases(300, hd):
        if c.packed and hd > 128:
            continue
        check_sdpa(alt, c, "f16", route="prefill_tc3")


# K and V rows must have a pitch that is a multiple of 16 bytes for the bulk tensor copies
# (kvHeads * headDim a multiple of 8 halves); other shapes stay on the FP32 pipes.
NARROW = [
    ("minilm_hd32_packed_segments", _c(qLen=512, kvLen=512, qHeads=12, kvHeads=12, headDim=32,
                                       packed=True, segments=True)),
    ("moonshine_tiny_encoder_hd36", _c(qLen=200, kvLen=200, qHeads=8, kvHeads=8, headDim=36)),
    ("moonshine_base_encoder_hd52", _c(qLen=200, kvLen=200, qHeads=8, kvHeads=8, headDim=52)),
    ("hd36_causal_1000", _c(qLen=1000, kvLen=1000, qHeads=8, kvHeads=8, headDim=36,
                            windowRight=0)),
    ("hd52_gqa_odd_kv_head_sliding", _c(qLen=700, kvLen=700, qHeads=8, kvHeads=4, headDim=52,
                                        windowLeft=100, windowRight=20, sinks=True)),
    ("hd36_gqa_3to1_cross", _c(qLen=150, kvLen=900, qHeads=12, kvHeads=4, headDim=36)),
    ("hd52_keybias_segments", _c(qLen=400, kvLen=400, qHeads=4, kvHeads=2, headDim=52,
                                 keyBias=True, segments=True, sinks=True)),
    ("hd48_full", _c(qLen=128, kvLen=128, qHeads=6, kvHeads=6, headDim=48)),
    ("hd16_two_rows", _c(qLen=2, kvLen=2, qHeads=2, kvHeads=1, headDim=16, windowRight=0)),
    ("hd4_last_head_reads_past_the_columns", _c(qLen=130, kvLen=130, qHeads=6, kvHeads=6,
                                               headDim=4)),
    ("hd60_rows_see_no_key", _c(qLen=300, kvLen=150, qHeads=4, kvHeads=2, headDim=60,
                                windowLeft=0, sinks=True)),
    ("hd36_packed_causal", _c(qLen=600, kvLen=600, qHeads=4, kvHeads=2, headDim=36, packed=True,
                              windowRight=0)),
]


def _pitch_ok(c):
    kv = c.kvHeads * c.headDim
    stride = (c.qHeads + 2 * c.kvHeads) * c.headDim if c.packed else kv
    base_ok = (c.qHeads * c.headDim) % 8 == 0 and kv % 8 == 0 if c.packed else True
    return stride % 8 == 0 and base_ok


@pytest.mark.parametrize("name,c", NARROW, ids=[n for n, _ in NARROW])
def test_narrow_heads_take_the_tensor_cores_by_default(ex, name, c):
    check_sdpa(ex, c, "f16", route="prefill_tc3")


@pytest.mark.parametrize("hd", [32, 36, 52])
def test_every_option_on_narrow_heads(ex, hd):
    routed = 0
    for name, c in cases.option_cases(300, hd):
        ok = _pitch_ok(c)
        check_sdpa(ex, c, "f16", route="prefill_tc3" if ok else "prefill_simt")
        routed += ok
    assert routed >= 10


def test_zoo_shapes_with_narrow_heads_route_to_the_tensor_cores(ex):
    wanted = {"moonshine_tiny_encoder_f16", "minilm_bucket_512"}
    seen = set()
    for name, dtype, c in cases.ZOO_SHAPES:
        if name in wanted:
            check_sdpa(ex, c, dtype, route="prefill_tc3")
            seen.add(name)
    assert seen == wanted


@pytest.mark.parametrize("hd", [64, 40])
def test_growing_scores_move_the_shared_reference_point(alt, hd):
    """Scores that keep growing along the keys move the rows' reference point in tile
    after tile, alternately from either warpgroup: every move rescales the accumulator
    once and both warpgroups' row sums."""
    import runntime_b200 as rt
    T = 1100
    rng = np.random.default_rng(1)
    q = np.ones((T, hd), np.float32) * 0.25
    k = (np.arange(T, dtype=np.float32)[:, None] / 16.0 * np.ones((1, hd), np.float32)) / 4
    k = oracle.round_f16(k.astype(np.float32))
    v = oracle.round_f16(rng.standard_normal((T, hd)).astype(np.float32))
    opts = dict(qHeads=1, kvHeads=1, headDim=hd, windowLeft=INF, windowRight=INF)
    out = rt.toArray(rt.sdpa(alt.upload(q, [T, hd], "f16"), alt.upload(k, [T, hd], "f16"),
                             alt.upload(v, [T, hd], "f16"), opts), alt)
    assert alt.dispatches[-1] == "prefill_tc3"
    want = oracle.sdpa_ref(q, k, v, qHeads=1, kvHeads=1, headDim=hd)
    oracle.assert_close(out, want, "f16")


def test_scores_that_shrink_then_jump(alt):
    """A late key tile whose scores tower over everything before it: the reference
    point jumps once, far, in a tile of the second warpgroup."""
    import runntime_b200 as rt
    T, hd = 900, 128
    rng = np.random.default_rng(3)
    q = oracle.round_f16((rng.standard_normal((T, hd)) * 0.2).astype(np.float32))
    k = oracle.round_f16((rng.standard_normal((T, hd)) * 0.2).astype(np.float32))
    k[5 * 128 + 7] = oracle.round_f16(q[300] * 12.0)      # one key aligned with row 300
    v = oracle.round_f16(rng.standard_normal((T, hd)).astype(np.float32))
    opts = dict(qHeads=1, kvHeads=1, headDim=hd, windowLeft=INF, windowRight=INF)
    out = rt.toArray(rt.sdpa(alt.upload(q, [T, hd], "f16"), alt.upload(k, [T, hd], "f16"),
                             alt.upload(v, [T, hd], "f16"), opts), alt)
    want = oracle.sdpa_ref(q, k, v, qHeads=1, kvHeads=1, headDim=hd)
    oracle.assert_close(out, want, "f16")


def test_matches_the_other_kernels(alt):
    from runntime_b200._lib import OPT_PREFILL_TC
    c = _c(qLen=900, kvLen=900, qHeads=4, kvHeads=2, headDim=128, windowLeft=400, windowRight=0,
           sinks=True)
    x = make_inputs(c, "f16")
    three = run_sdpa(alt, x)
    assert alt.dispatches[-1] == "prefill_tc3"
    for mode, route in ((2, "prefill_tc"), (0, "prefill_simt")):
        alt.setOption(OPT_PREFILL_TC, mode)
        other = run_sdpa(alt, x)
        assert alt.dispatches[-1] == route
        assert np.abs(three - other).max() < 2e-3


@pytest.mark.parametrize("hd,heads,kvHeads,wl,wr,packed", [
    (256, 3, 1, 512, 512, False),    # EmbeddingGemma sliding layer
    (256, 3, 1, INF, INF, False),    # EmbeddingGemma global layer
    (32, 12, 12, INF, INF, True),    # MiniLM, f16
    (128, 8, 8, INF, 0, True),
])
def test_greedy_packed_batch_of_ragged_sequences(alt, hd, heads, kvHeads, wl, wr, packed):
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
    got = run_sdpa(alt, x)
    assert alt.dispatches[-1] == "prefill_tc3"
    want = oracle.sdpa_ref_inputs(x)
    oracle.assert_close(got, want, "f16")
    assert (got.reshape(T, -1)[at:] == 0).all()


# ---- pairs of CTAs sharing every K/V tile (head sizes 128 and 256) -------------------

@pytest.fixture
def pair(ex):
    from runntime_b200._lib import OPT_PREFILL_TC
    ex.setOption(OPT_PREFILL_TC, 5)
    yield ex
    ex.setOption(OPT_PREFILL_TC, 1)


def _pair_ok(c):
    return c.headDim in (128, 256) and c.qLen > 128


PAIRED = {n: c for n, c in ALL.items() if _pair_ok(c)}
PAIRED.update({
    "odd_number_of_row_tiles": _c(qLen=640, kvLen=640, qHeads=2, kvHeads=1, headDim=128,
                                  windowRight=0),
    "second_tile_of_the_pair_is_empty": _c(qLen=256, kvLen=100, qHeads=1, kvHeads=1, headDim=128,
                                           windowLeft=0, windowRight=INF),
    "gqa_3to1_hd256_sliding_2048": _c(qLen=2048, kvLen=2048, qHeads=3, kvHeads=1, headDim=256,
                                      windowLeft=512, windowRight=512),
    "causal_3000_hd128_gqa": _c(qLen=3000, kvLen=3000, qHeads=4, kvHeads=2, headDim=128,
                                windowRight=0, sinks=True),
})


@pytest.mark.parametrize("name", sorted(PAIRED))
def test_pairs_against_oracle(pair, name):
    check_sdpa(pair, PAIRED[name], "f16", route="prefill_tc3_pair")


@pytest.mark.parametrize("hd", [128, 256])
def test_every_option_in_pairs(pair, hd):
    for name, c in cases.option_cases(300, hd):
        if c.packed and hd > 128:
            continue
        check_sdpa(pair, c, "f16", route="prefill_tc3_pair")


def test_growing_scores_in_pairs(pair):
    import runntime_b200 as rt
    T, hd = 1100, 128
    rng = np.random.default_rng(1)
    q = np.ones((T, hd), np.float32) * 0.125
    k = (np.arange(T, dtype=np.float32)[:, None] / 16.0 * np.ones((1, hd), np.float32)) / 4
    k = oracle.round_f16(k.astype(np.float32))
    v = oracle.round_f16(rng.standard_normal((T, hd)).astype(np.float32))
    opts = dict(qHeads=1, kvHeads=1, headDim=hd, windowLeft=INF, windowRight=INF)
    out = rt.toArray(rt.sdpa(pair.upload(q, [T, hd], "f16"), pair.upload(k, [T, hd], "f16"),
                             pair.upload(v, [T, hd], "f16"), opts), pair)
    assert pair.dispatches[-1] == "prefill_tc3_pair"
    want = oracle.sdpa_ref(q, k, v, qHeads=1, kvHeads=1, headDim=hd)
    oracle.assert_close(out, want, "f16")
