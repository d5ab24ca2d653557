"""The persistent tensor-core prefill kernel (one thread block per SM walking a queue of
query tiles whose pipelines overlap; f16, head sizes 64/128/256): every case of the other
tensor-core kernels, ragged batches whose units have one, two or no key tiles, more units
than SMs, and two launches in a row (the work counter rewinds itself), against the f64
oracle (f16 tolerance: atol 2e-3 + rtol 4e-3)."""
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
def persistent(ex):
    """Routes every eligible shape to the persistent kernel."""
    from runntime_b200._lib import OPT_PREFILL_TC
    ex.setOption(OPT_PREFILL_TC, 6)
    yield ex
    ex.setOption(OPT_PREFILL_TC, 1)


ALL = {n: c for n, c in TC_CASES + TWO_TILE_CASES}


@pytest.mark.parametrize("name", sorted(ALL))
def test_persistent_against_oracle(persistent, name):
    check_sdpa(persistent, ALL[name], "f16", route="prefill_tc4")


@pytest.mark.parametrize("hd", [64, 128, 256])
def test_every_option(persistent, hd):
    for name, c in cases.option_cases(300, hd):
        if c.packed and hd > 128:
            continue
        check_sdpa(persistent, c, "f16", route="prefill_tc4")


MANY = [
    # more units than SMs: every block takes several, of different lengths
    ("causal_4000_hd128_8_heads", _c(qLen=4000, kvLen=4000, qHeads=8, kvHeads=8, headDim=128,
                                     windowRight=0)),
    ("sliding_3000_hd256_gqa", _c(qLen=3000, kvLen=3000, qHeads=6, kvHeads=2, headDim=256,
                                  windowLeft=200, windowRight=200)),
    ("sliding_one_tile_units_hd64", _c(qLen=5000, kvLen=5000, qHeads=4, kvHeads=4, headDim=64,
                                       windowLeft=20, windowRight=20, sinks=True)),
    ("cross_rows_see_no_key_hd128", _c(qLen=3000, kvLen=700, qHeads=4, kvHeads=2, headDim=128,
                                       windowLeft=0, windowRight=INF, sinks=True)),
    ("segments_hd256", _c(qLen=2500, kvLen=2500, qHeads=3, kvHeads=1, headDim=256, segments=True)),
    ("keybias_causal_hd64", _c(qLen=3000, kvLen=3000, qHeads=8, kvHeads=2, headDim=64,
                               windowRight=0, keyBias=True)),
]


@pytest.mark.parametrize("name,c", MANY, ids=[n for n, _ in MANY])
def test_more_units_than_blocks(persistent, name, c):
    check_sdpa(persistent, c, "f16", route="prefill_tc4")


def test_two_launches_in_a_row_give_the_same_rows(persistent):
    c = _c(qLen=2000, kvLen=2000, qHeads=4, kvHeads=4, headDim=128, windowRight=0)
    x = make_inputs(c, "f16")
    a = run_sdpa(persistent, x)
    b = run_sdpa(persistent, x)
    assert persistent.dispatches[-1] == "prefill_tc4"
    assert np.array_equal(a, b)
    oracle.assert_close(a, oracle.sdpa_ref_inputs(x), "f16")


@pytest.mark.parametrize("hd,heads,kvHeads,wl,wr", [
    (256, 3, 1, 512, 512),      # EmbeddingGemma sliding layer
    (256, 3, 1, INF, INF),      # EmbeddingGemma global layer
    (128, 8, 8, INF, 0),
    (64, 4, 2, 100, 0),
])
def test_padded_batch_of_ragged_sequences(persistent, hd, heads, kvHeads, wl, wr):
    """Sequences of different lengths at a common stride: units past a sequence's end see no
    key (written as zeros by the scheduler warp), units at its end see a tile or two."""
    import torch
    from runntime_b200.engine import prefill_batched
    S = 1024
    lens = [37, 1024, 5, 130, 1, 700, 128, 129, 900, 513]
    batch = len(lens)
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(77)
    f = hd ** -0.25
    q = (torch.randn(batch * S, heads * hd, generator=g, device=dev) * f).half()
    k = (torch.randn(batch * S, kvHeads * hd, generator=g, device=dev) * f).half()
    v = torch.randn(batch * S, kvHeads * hd, generator=g, device=dev).half()
    out = torch.full_like(q, 3.0)
    ld = torch.tensor(lens, dtype=torch.int32, device=dev)
    persistent.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        prefill_batched(persistent, q, k, v, out, dtype="f16", batch=batch, seqStride=S, seqLens=ld,
                        qHeads=heads, kvHeads=kvHeads, headDim=hd,
                        windowLeft=None if wl == INF else wl, windowRight=None if wr == INF else wr)
        persistent.sync()
    finally:
        persistent.setStream(None)
    got = out.float().cpu().numpy()
    for b, L in enumerate(lens):
        qb, kb, vb = (t[b * S:b * S + L].float().cpu().numpy() for t in (q, k, v))
        want = oracle.sdpa_ref(qb, kb, vb, qHeads=heads, kvHeads=kvHeads, headDim=hd,
                               windowLeft=wl, windowRight=wr)
        oracle.assert_close(got[b * S:b * S + L], want.reshape(L, -1), "f16", f"seq {b}")
        assert (got[b * S + L:(b + 1) * S] == 0).all()     # rows past the length
