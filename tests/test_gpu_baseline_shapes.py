"""Parity at the benchmark's own shapes (the five configurations the headline numbers
are quoted on), through the same batched entry points bench.py times, against the f64
oracle.  Where a full f64 pass over the shape would take minutes the oracle runs on a
stated sample of query rows (a row's output depends on nothing but that row's q, so a
sample is exact for the rows it covers).  Tolerances: f16 atol 2e-3 + rtol 4e-3, f32
atol 2e-5 + rtol 1e-4 (the reference's, packages/runntime/test/core/kernels/attention/
checkSdpa.ts:127), plus the benchmark contract's own bars."""
import math

import numpy as np
import pytest

import oracle
from gpu_harness import ex  # noqa: F401
from oracle import sdpa_ref

pytestmark = pytest.mark.gpu
INF = math.inf


@pytest.mark.parametrize("mode,route", [(3, "prefill_tc2"), (4, "prefill_tc3"), (2, "prefill_tc")])
def test_c5_causal_prefill_one_full_sequence(ex, mode, route):
    """8192 rows x 8 heads x 128, causal, two sequences through the padded-batch form:
    every 128-row tile boundary, the first and last rows and a spread in between
    (96 rows per sequence, all heads)."""
    import torch
    from runntime_b200._lib import OPT_PREFILL_TC
    from runntime_b200.engine import prefill_batched
    S, heads, hd, batch = 8192, 8, 128, 2
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(1000)
    f = hd ** -0.25
    q = (torch.randn(batch * S, heads * hd, generator=g, device=dev) * f).half()
    k = (torch.randn(batch * S, heads * hd, generator=g, device=dev) * f).half()
    v = torch.randn(batch * S, heads * hd, generator=g, device=dev).half()
    out = torch.empty_like(q)
    lens = torch.full((batch,), S, dtype=torch.int32, device=dev)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    ex.setOption(OPT_PREFILL_TC, mode)
    try:
        before = ex.launchCount()
        prefill_batched(ex, q, k, v, out, dtype="f16", batch=batch, seqStride=S, seqLens=lens,
                        qHeads=heads, kvHeads=heads, headDim=hd, windowLeft=None, windowRight=0)
        ex.sync()
        assert ex.launchCount() == before + 1
    finally:
        ex.setOption(OPT_PREFILL_TC, 1)
        ex.setStream(None)
    rows = sorted({0, 1, 127, 128, 129, 255, 256, 4095, 4096, 8063, 8064, 8190, 8191}
                  | set(range(383, S, 128)) | set(range(640, S, 400)))
    got = out.float().cpu().numpy()
    worst = 0.0
    for b in range(batch):
        qb, kb, vb = (t[b * S:(b + 1) * S].float().cpu().numpy() for t in (q, k, v))
        for r in rows:
            want = sdpa_ref(qb[r:r + 1], kb[:r + 1], vb[:r + 1], qHeads=heads, kvHeads=heads,
                            headDim=hd, windowRight=0, qPosOffset=r).reshape(-1)
            oracle.assert_close(got[b * S + r], want, "f16", f"{route} seq {b} row {r}")
            worst = max(worst, float(np.abs(got[b * S + r] - want).max()))
    assert worst <= 2e-3          # the benchmark contract's bar for f16: max absolute error


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("wl,wr", [(512, 512), (None, None)])
def test_c3_gqa_prefill_full_sequence_with_padded_neighbours(ex, mode, wl, wr):
    """2048 rows, 3 query heads on 1 kv head of 256, f16, N(0, 0.5): a full-length
    sequence between two padded ones (lengths 700, 2048, 1301), the sliding (+-512) and
    the global layer.  Oracle rows: tile and window edges plus a spread."""
    import torch
    from runntime_b200._lib import OPT_PREFILL_TC
    from runntime_b200.engine import prefill_batched
    S, heads, hd = 2048, 3, 256
    lens = [700, 2048, 1301]
    batch = len(lens)
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(3000)
    q = (torch.randn(batch * S, heads * hd, generator=g, device=dev) * 0.5).half()
    k = (torch.randn(batch * S, hd, generator=g, device=dev) * 0.5).half()
    v = (torch.randn(batch * S, hd, generator=g, device=dev) * 0.5).half()
    out = torch.full_like(q, 3.0)
    ld = torch.tensor(lens, dtype=torch.int32, device=dev)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    ex.setOption(OPT_PREFILL_TC, mode)
    try:
        prefill_batched(ex, q, k, v, out, dtype="f16", batch=batch, seqStride=S, seqLens=ld,
                        qHeads=heads, kvHeads=1, headDim=hd, windowLeft=wl, windowRight=wr)
        ex.sync()
    finally:
        ex.setOption(OPT_PREFILL_TC, 1)
        ex.setStream(None)
    got = out.float().cpu().numpy()
    for b, L in enumerate(lens):
        qb, kb, vb = (t[b * S:b * S + L].float().cpu().numpy() for t in (q, k, v))
        rows = sorted({0, 1, 127, 128, 511, 512, 513, L - 513, L - 512, L - 129, L - 2, L - 1}
                      | set(range(77, L, 211)))
        rows = [r for r in rows if 0 <= r < L]
        for r in rows:
            want = sdpa_ref(qb[r:r + 1], kb, vb, qHeads=heads, kvHeads=1, headDim=hd,
                            windowLeft=INF if wl is None else wl,
                            windowRight=INF if wr is None else wr, qPosOffset=r).reshape(-1)
            oracle.assert_close(got[b * S + r], want, "f16", f"seq {b} row {r}")
        assert (got[b * S + L:(b + 1) * S] == 0).all()     # rows past the length


def test_c1_eight_packed_sequences_f32(ex):
    """MiniLM shape: 12 heads of 32, f32, eight sequences of 16..128 rows packed back to
    back with a [start, end) range per row (the reference's own form), 6 layers of
    independent inputs; every row against the oracle."""
    import runntime_b200 as rt
    rng = np.random.default_rng(1001)
    heads, hd = 12, 32
    for layer in range(6):
        lens = rng.integers(16, 129, size=8).tolist()
        T = sum(lens)
        f = hd ** -0.25
        qkv = rng.standard_normal((T, 3 * heads * hd)).astype(np.float32)
        qkv[:, :2 * heads * hd] *= f
        segs = np.zeros((T, 2), np.float32)
        at = 0
        for n in lens:
            segs[at:at + n] = (at, at + n)
            at += n
        opts = dict(qHeads=heads, kvHeads=heads, headDim=hd, windowLeft=INF, windowRight=INF,
                    segments=ex.upload(segs, [T, 2]), maxSegment=max(lens))
        out = rt.toArray(rt.sdpaPacked(ex.upload(qkv, [T, 3 * heads * hd]), opts), ex)
        want = sdpa_ref(None, None, None, qHeads=heads, kvHeads=heads, headDim=hd, segs=segs,
                        packed=qkv)
        oracle.assert_close(out, want, "f32", f"layer {layer}")
        rel = np.abs(out.reshape(want.shape) - want) / np.maximum(np.abs(want), 0.2 * np.sqrt((want ** 2).mean()))
        assert rel.max() <= 1e-4      # the benchmark contract's bar for f32 inputs


def test_c2_decode_step_batch_64_self_and_cross(ex):
    """Moonshine-tiny step: 8 heads of 36, f16, batch 64, self caches of 1..448 visible
    rows (the appended one included) and cross-attention over 200 encoder rows; every
    sequence against the oracle, and the caches after the append."""
    import torch
    from runntime_b200.engine import decode_batched
    batch, heads, hd, rows, cross = 64, 8, 36, 448, 200
    w = heads * hd
    g = torch.Generator().manual_seed(2000)
    lens = torch.randint(1, rows + 1, (batch,), generator=g)
    lens[0], lens[1] = 1, rows
    kc = torch.randn(batch, rows, w, generator=g).half()
    vc = torch.randn(batch, rows, w, generator=g).half()
    kn = torch.randn(batch, w, generator=g).half()
    vn = torch.randn(batch, w, generator=g).half()
    ck = torch.randn(batch, cross, w, generator=g).half()
    cv = torch.randn(batch, cross, w, generator=g).half()
    q = (torch.randn(batch, w, generator=g) / 6).half()
    dev = torch.device("cuda", 0)
    kcd, vcd = kc.to(dev), vc.to(dev)
    out = torch.empty(batch, w, dtype=torch.float16, device=dev)
    out2 = torch.empty_like(out)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        decode_batched(ex, q.to(dev), out, kcd, vcd, dtype="f16", batch=batch, cacheRows=rows,
                       qHeads=heads, kvHeads=heads, headDim=hd, kvLen=int(lens.max()),
                       kvLens=lens.to(torch.int32).to(dev), kNew=kn.to(dev), vNew=vn.to(dev))
        decode_batched(ex, q.to(dev), out2, ck.to(dev), cv.to(dev), dtype="f16", batch=batch,
                       cacheRows=cross, qHeads=heads, kvHeads=heads, headDim=hd, kvLen=cross)
        ex.sync()
    finally:
        ex.setStream(None)
    kc2, vc2 = kc.clone(), vc.clone()
    for b, L in enumerate(lens.tolist()):
        kc2[b, L - 1], vc2[b, L - 1] = kn[b], vn[b]
        want = sdpa_ref(q[b:b + 1].float().numpy(), kc2[b, :L].float().numpy(),
                        vc2[b, :L].float().numpy(), qHeads=heads, kvHeads=heads, headDim=hd,
                        windowRight=0, qPosOffset=L - 1)
        oracle.assert_close(out[b].float().cpu().numpy(), want, "f16", f"self seq {b} len {L}")
        want = sdpa_ref(q[b:b + 1].float().numpy(), ck[b].float().numpy(), cv[b].float().numpy(),
                        qHeads=heads, kvHeads=heads, headDim=hd)
        oracle.assert_close(out2[b].float().cpu().numpy(), want, "f16", f"cross seq {b}")
    assert torch.equal(kcd.cpu(), kc2) and torch.equal(vcd.cpu(), vc2)


def test_c4_long_decode_batch_at_8192_rows(ex):
    """Moonshine-base long decode: 8 heads of 52, f16, six sequences over full 8192-row
    caches (each cache is 6.8 MB, as in the benchmark), the library's own split choice
    and a forced split; every sequence against the oracle."""
    import torch
    from runntime_b200.engine import decode_batched
    batch, heads, hd, rows = 6, 8, 52, 8192
    w = heads * hd
    g = torch.Generator().manual_seed(4000)
    kc = torch.randn(batch, rows, w, generator=g).half()
    vc = torch.randn(batch, rows, w, generator=g).half()
    q = (torch.randn(batch, w, generator=g) * hd ** -0.5).half()
    dev = torch.device("cuda", 0)
    kcd, vcd, qd = kc.to(dev), vc.to(dev), q.to(dev)
    out = torch.empty(batch, w, dtype=torch.float16, device=dev)
    refs = [sdpa_ref(q[b:b + 1].float().numpy(), kc[b].float().numpy(), vc[b].float().numpy(),
                     qHeads=heads, kvHeads=heads, headDim=hd) for b in range(batch)]
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        for splits in (0, 1, 5):
            out.fill_(9.0)
            decode_batched(ex, qd, out, kcd, vcd, dtype="f16", batch=batch, cacheRows=rows,
                           qHeads=heads, kvHeads=heads, headDim=hd, kvLen=rows, splits=splits)
            ex.sync()
            for b in range(batch):
                got = out[b].float().cpu().numpy()
                oracle.assert_close(got, refs[b], "f16", f"seq {b} splits {splits}")
                assert np.abs(got - refs[b].reshape(-1)).max() <= 2e-3
    finally:
        ex.setStream(None)
