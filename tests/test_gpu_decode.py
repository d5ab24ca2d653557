"""Decode parity on the GPU: the reference's decode suite
(packages/runntime/test/core/kernels/attention/attnDecode.gpu.test.ts:38-115),
the fused KV-cache append, batched caches, partials + merge."""
import ctypes as C
import math

import numpy as np
import pytest

import cases
import oracle
from gpu_harness import check_sdpa, ex  # noqa: F401
from oracle import SdpaCase, make_inputs, sdpa_ref

pytestmark = pytest.mark.gpu

INF = math.inf


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("name,c", cases.DECODE_CASES, ids=[n for n, _ in cases.DECODE_CASES])
def test_decode_cases(ex, dtype, name, c):
    check_sdpa(ex, c, dtype, route="decode")


@pytest.mark.parametrize("name,dtype,c", [z for z in cases.ZOO_SHAPES if z[2].qLen == 1],
                         ids=[z[0] for z in cases.ZOO_SHAPES if z[2].qLen == 1])
def test_zoo_decode_shapes(ex, name, dtype, c):
    check_sdpa(ex, c, dtype, route="decode")


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("hd,heads", [(36, 8), (52, 8), (64, 4), (128, 2), (16, 4), (37, 3)])
def test_model_head_sizes_long_cache(ex, dtype, hd, heads):
    for kv in (1, 33, 448, 3000):
        check_sdpa(ex, cases.decode(kv, qHeads=heads, kvHeads=heads, headDim=hd), dtype,
                   route="decode")


def test_two_chained_calls_share_the_split_scratch(ex):
    import runntime_b200 as rt
    opts = dict(qHeads=4, kvHeads=4, headDim=16, windowLeft=INF, windowRight=0, qPosOffset=599)
    q = oracle.random_f32(64, 1)
    k = oracle.random_f32(600 * 64, 2).reshape(600, 64)
    v = oracle.random_f32(600 * 64, 3).reshape(600, 64)
    ku, vu = ex.upload(k, [600, 64]), ex.upload(v, [600, 64])
    first = rt.sdpa(ex.upload(q, [1, 64]), ku, vu, opts)
    got = rt.toArray(rt.sdpa(first, vu, ku, opts), ex)
    kw = dict(qHeads=4, kvHeads=4, headDim=16, windowRight=0, qPosOffset=599)
    first_want = sdpa_ref(q.reshape(1, 64), k, v, **kw).astype(np.float32)
    oracle.assert_close(got, sdpa_ref(first_want, v, k, **kw), "f32")


def _decode_step_through_ops(ex, dtype, t, hd=36, heads=8, cacheRows=194):
    """The decoder's step: writeRows K and V at t, causal sdpa with qPosOffset t."""
    import runntime_b200 as rt
    w = heads * hd
    rnd = oracle.round_f16 if dtype == "f16" else (lambda a: a)
    kc = rnd(oracle.random_f32(cacheRows * w, 5)).reshape(cacheRows, w)
    vc = rnd(oracle.random_f32(cacheRows * w, 6)).reshape(cacheRows, w)
    kn = rnd(oracle.random_f32(w, 7)).reshape(1, w)
    vn = rnd(oracle.random_f32(w, 8)).reshape(1, w)
    q = rnd(oracle.random_f32(w, 9) * np.float32(2 / math.sqrt(hd))).reshape(1, w)
    kcache, vcache = ex.upload(kc, [cacheRows, w], dtype), ex.upload(vc, [cacheRows, w], dtype)
    k = rt.writeRows(kcache, ex.upload(kn, [1, w], dtype), t)
    v = rt.writeRows(vcache, ex.upload(vn, [1, w], dtype), t)
    mha = rt.MultiHeadAttention(dict(qHeads=heads, kvHeads=heads, headDim=hd, windowLeft=INF,
                                     windowRight=0))
    before = len(ex.dispatches)
    out = rt.toArray(mha.forward(ex.upload(q, [1, w], dtype), k, v, dict(qPosOffset=t)), ex)
    routes = ex.dispatches[before:]
    kc2, vc2 = kc.copy(), vc.copy()
    kc2[t], vc2[t] = kn[0], vn[0]
    want = sdpa_ref(q, kc2[: t + 1], vc2[: t + 1], qHeads=heads, kvHeads=heads, headDim=hd,
                    windowRight=0, qPosOffset=t)
    oracle.assert_close(out, want, dtype, f"decode step t={t}")
    # the cache holds the new row exactly, the rest is untouched
    assert np.array_equal(ex.readback(kcache.buffer, kcache.shape).reshape(cacheRows, w), kc2)
    assert np.array_equal(ex.readback(vcache.buffer, vcache.shape).reshape(cacheRows, w), vc2)
    return routes


@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("t", [0, 1, 31, 32, 100, 193])
def test_decoder_step_append_then_attend(ex, dtype, t):
    assert _decode_step_through_ops(ex, dtype, t) == ["decode+append"]


def test_decoder_step_generic_head_size(ex):
    assert _decode_step_through_ops(ex, "f16", 50, hd=37, heads=3, cacheRows=64) == ["decode+append"]
    assert _decode_step_through_ops(ex, "f32", 50, hd=20, heads=5, cacheRows=64) == ["decode+append"]


def _batched_inputs(batch, cacheRows, heads, kvHeads, hd, dtype, lens, seed=11):
    torch = pytest.importorskip("torch")
    g = torch.Generator().manual_seed(seed)
    tdt = torch.float16 if dtype == "f16" else torch.float32
    w, qw = kvHeads * hd, heads * hd
    kc = torch.randn(batch, cacheRows, w, generator=g).to(tdt)
    vc = torch.randn(batch, cacheRows, w, generator=g).to(tdt)
    kn = torch.randn(batch, w, generator=g).to(tdt)
    vn = torch.randn(batch, w, generator=g).to(tdt)
    q = (torch.randn(batch, qw, generator=g) / math.sqrt(hd)).to(tdt)
    return q, kc, vc, kn, vn, torch.tensor(lens, dtype=torch.int32)


@pytest.mark.parametrize("dtype", ["f16", "f32"])
# the last three: wide models, where a tile holds only a few keys of all the heads
@pytest.mark.parametrize("heads,kvHeads,hd", [(8, 8, 36), (8, 8, 52), (6, 2, 64), (4, 4, 20),
                                              (32, 32, 128), (32, 8, 128), (16, 16, 64)])
def test_batched_decode_with_append_matches_per_sequence_oracle(ex, dtype, heads, kvHeads, hd):
    import torch
    from runntime_b200.engine import decode_batched
    batch, cacheRows = 9, 448
    lens = [1, 2, 31, 32, 33, 200, 257, 447, 448]
    q, kc, vc, kn, vn, lt = _batched_inputs(batch, cacheRows, heads, kvHeads, hd, dtype, lens)
    dev = torch.device("cuda", 0)
    qd, kcd, vcd, knd, vnd, ld = (t.to(dev) for t in (q, kc, vc, kn, vn, lt))
    out = torch.full((batch, heads * hd), 7.0, dtype=qd.dtype, device=dev)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        for splits in (0, 1, 3):
            kcd.copy_(kc)
            vcd.copy_(vc)
            decode_batched(ex, qd, out, kcd, vcd, dtype=dtype, batch=batch, cacheRows=cacheRows,
                           qHeads=heads, kvHeads=kvHeads, headDim=hd, kvLen=max(lens), kvLens=ld,
                           kNew=knd, vNew=vnd, splits=splits)
            ex.sync()
            got = out.float().cpu().numpy()
            kc2, vc2 = kc.clone(), vc.clone()
            for b, L in enumerate(lens):
                kc2[b, L - 1], vc2[b, L - 1] = kn[b], vn[b]
                want = sdpa_ref(q[b:b + 1].float().numpy(), kc2[b, :L].float().numpy(),
                                vc2[b, :L].float().numpy(), qHeads=heads, kvHeads=kvHeads,
                                headDim=hd, windowRight=0, qPosOffset=L - 1)
                oracle.assert_close(got[b], want, dtype, f"seq {b} len {L} splits {splits}")
            assert torch.equal(kcd.cpu(), kc2) and torch.equal(vcd.cpu(), vc2)
    finally:
        ex.setStream(None)


@pytest.mark.parametrize("heads,hd", [(8, 52), (32, 128)])
def test_device_side_length_past_the_cache_is_refused_not_written(ex, heads, hd):
    """kvLens lives on the device, so the host cannot check it: an entry one past
    cacheRows must not append (writeRows: 'rows exceed dst capacity') nor read past the
    cache.  The sequence comes out as zeros, the rows after its cache keep their
    contents, the other sequences are computed, and rt_sync reports it."""
    import torch
    import runntime_b200 as rt
    from runntime_b200.engine import decode_batched
    batch, cacheRows, alloc = 3, 100, 104      # four guard rows behind each cache
    lens = [100, 101, 37]
    q, kc, vc, kn, vn, lt = _batched_inputs(batch, alloc, heads, heads, hd, "f16", lens)
    dev = torch.device("cuda", 0)
    qd, kcd, vcd, knd, vnd, ld = (t.to(dev) for t in (q, kc, vc, kn, vn, lt))
    out = torch.full((batch, heads * hd), 7.0, dtype=qd.dtype, device=dev)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        for splits in (1, 3):
            kcd.copy_(kc)
            vcd.copy_(vc)
            decode_batched(ex, qd, out, kcd, vcd, dtype="f16", batch=batch, cacheRows=cacheRows,
                           cacheSeqStride=alloc * heads * hd, qHeads=heads, kvHeads=heads,
                           headDim=hd, kvLen=cacheRows, kvLens=ld, kNew=knd, vNew=vnd,
                           splits=splits)
            with pytest.raises(rt.RunntimeError, match="kvLens entry past cacheRows") as e:
                ex.sync()
            assert e.value.code == "EXECUTION_FAILED"
            got = out.float().cpu().numpy()
            assert (got[1] == 0).all()
            kc2, vc2 = kc.clone(), vc.clone()
            for b in (0, 2):
                L = lens[b]
                kc2[b, L - 1], vc2[b, L - 1] = kn[b], vn[b]
                want = sdpa_ref(q[b:b + 1].float().numpy(), kc2[b, :L].float().numpy(),
                                vc2[b, :L].float().numpy(), qHeads=heads, kvHeads=heads,
                                headDim=hd, windowRight=0, qPosOffset=L - 1)
                oracle.assert_close(got[b], want, "f16", f"seq {b} splits {splits}")
            assert torch.equal(kcd.cpu(), kc2) and torch.equal(vcd.cpu(), vc2)   # guard rows too
            ex.sync()     # the report cleared the status word
    finally:
        ex.setStream(None)


@pytest.mark.parametrize("dtype,heads,kvHeads,hd", [("f16", 8, 8, 36), ("f16", 32, 8, 128),
                                                     ("f32", 4, 4, 20)])
def test_self_and_cross_attention_in_one_launch(ex, dtype, heads, kvHeads, hd):
    """A decoder layer's two attentions — the step over the self cache with the append,
    and the cross-attention over the encoder states with a query of its own — from one
    kernel launch, for every split choice."""
    import torch
    from runntime_b200.engine import decode_batched, second_attention
    batch, cacheRows, cross = 9, 448, 200
    lens = [1, 2, 31, 32, 33, 200, 257, 447, 448]
    q, kc, vc, kn, vn, lt = _batched_inputs(batch, cacheRows, heads, kvHeads, hd, dtype, lens)
    q2, ck, cv, _, _, _ = _batched_inputs(batch, cross, heads, kvHeads, hd, dtype, [cross] * batch,
                                          seed=12)
    dev = torch.device("cuda", 0)
    qd, kcd, vcd, knd, vnd, ld, q2d, ckd, cvd = (t.to(dev) for t in (q, kc, vc, kn, vn, lt, q2, ck, cv))
    out = torch.full((batch, heads * hd), 7.0, dtype=qd.dtype, device=dev)
    out2 = torch.full_like(out, 7.0)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        for splits in (0, 1, 3):
            kcd.copy_(kc)
            vcd.copy_(vc)
            sec = second_attention(q2d, out2, ckd, cvd, cacheRows=cross, qHeads=heads,
                                   kvHeads=kvHeads, headDim=hd, kvLen=cross)
            before = ex.launchCount()
            decode_batched(ex, qd, out, kcd, vcd, dtype=dtype, batch=batch, cacheRows=cacheRows,
                           qHeads=heads, kvHeads=kvHeads, headDim=hd, kvLen=max(lens), kvLens=ld,
                           kNew=knd, vNew=vnd, splits=splits, second=sec)
            ex.sync()
            assert ex.launchCount() == before + 1
            got, got2 = out.float().cpu().numpy(), out2.float().cpu().numpy()
            kc2, vc2 = kc.clone(), vc.clone()
            for b, L in enumerate(lens):
                kc2[b, L - 1], vc2[b, L - 1] = kn[b], vn[b]
                want = sdpa_ref(q[b:b + 1].float().numpy(), kc2[b, :L].float().numpy(),
                                vc2[b, :L].float().numpy(), qHeads=heads, kvHeads=kvHeads,
                                headDim=hd, windowRight=0, qPosOffset=L - 1)
                oracle.assert_close(got[b], want, dtype, f"self seq {b} splits {splits}")
                want = sdpa_ref(q2[b:b + 1].float().numpy(), ck[b].float().numpy(),
                                cv[b].float().numpy(), qHeads=heads, kvHeads=kvHeads, headDim=hd)
                oracle.assert_close(got2[b], want, dtype, f"cross seq {b} splits {splits}")
            assert torch.equal(kcd.cpu(), kc2) and torch.equal(vcd.cpu(), vc2)
            assert torch.equal(ckd.cpu(), ck)
    finally:
        ex.setStream(None)


@pytest.mark.parametrize("heads,hd", [(8, 52), (32, 128), (3, 37)])
def test_caches_allocated_one_by_one(ex, heads, hd):
    """Every sequence's K and V cache is its own allocation (as the reference's per-layer,
    per-sequence cache tensors are), handed over as arrays of pointers."""
    import torch
    import runntime_b200 as rt
    from runntime_b200.engine import decode_batched
    batch, cacheRows = 5, 300
    lens = [300, 1, 77, 256, 129]
    q, kc, vc, kn, vn, lt = _batched_inputs(batch, cacheRows, heads, heads, hd, "f16", lens)
    dev = torch.device("cuda", 0)
    ks = [kc[b].clone().to(dev) for b in range(batch)]
    vs = [vc[b].clone().to(dev) for b in range(batch)]
    kp = torch.tensor([t.data_ptr() for t in ks], dtype=torch.int64, device=dev)
    vp = torch.tensor([t.data_ptr() for t in vs], dtype=torch.int64, device=dev)
    qd, knd, vnd, ld = q.to(dev), kn.to(dev), vn.to(dev), lt.to(dev)
    out = torch.full((batch, heads * hd), 7.0, dtype=qd.dtype, device=dev)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        decode_batched(ex, qd, out, None, None, dtype="f16", batch=batch, cacheRows=cacheRows,
                       qHeads=heads, kvHeads=heads, headDim=hd, kvLen=max(lens), kvLens=ld, kNew=knd,
                       vNew=vnd, kCachePtrs=kp, vCachePtrs=vp)
        ex.sync()
        got = out.float().cpu().numpy()
        for b, L in enumerate(lens):
            kb, vb = kc[b, :L].clone(), vc[b, :L].clone()
            kb[L - 1], vb[L - 1] = kn[b], vn[b]
            want = sdpa_ref(q[b:b + 1].float().numpy(), kb.float().numpy(), vb.float().numpy(),
                            qHeads=heads, kvHeads=heads, headDim=hd, windowRight=0, qPosOffset=L - 1)
            oracle.assert_close(got[b], want, "f16", f"seq {b}")
            assert torch.equal(ks[b][:L].cpu(), kb) and torch.equal(ks[b][L:].cpu(), kc[b, L:])
        if hd % 8 == 4:
            # a cache that starts 8 bytes off a 16-byte boundary cannot take the bulk copies:
            # its sequence comes out as zeros and the status says so; the others are computed
            off = torch.zeros(cacheRows * heads * hd + 4, dtype=torch.float16, device=dev)
            shifted = off[4:]
            shifted.copy_(kc[1].reshape(-1))
            kp2 = kp.clone()
            kp2[1] = shifted.data_ptr()
            out.fill_(7.0)
            decode_batched(ex, qd, out, None, None, dtype="f16", batch=batch, cacheRows=cacheRows,
                           qHeads=heads, kvHeads=heads, headDim=hd, kvLen=max(lens), kvLens=ld,
                           kCachePtrs=kp2, vCachePtrs=vp)
            with pytest.raises(rt.RunntimeError, match="not 16-byte aligned"):
                ex.sync()
            assert (out[1] == 0).all() and not (out[0] == 7.0).any()
    finally:
        ex.setStream(None)


def test_batched_cross_attention_and_window(ex):
    import torch
    from runntime_b200.engine import decode_batched
    batch, rows, heads, hd = 5, 200, 8, 36
    q, kc, vc, _, _, _ = _batched_inputs(batch, rows, heads, heads, hd, "f16", [rows] * batch)
    dev = torch.device("cuda", 0)
    qd, kcd, vcd = q.to(dev), kc.to(dev), vc.to(dev)
    out = torch.empty_like(qd)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        for wl in (None, 10):
            decode_batched(ex, qd, out, kcd, vcd, dtype="f16", batch=batch, cacheRows=rows,
                           qHeads=heads, kvHeads=heads, headDim=hd, kvLen=rows, windowLeft=wl)
            ex.sync()
            for b in range(batch):
                want = sdpa_ref(q[b:b + 1].float().numpy(), kc[b].float().numpy(),
                                vc[b].float().numpy(), qHeads=heads, kvHeads=heads, headDim=hd,
                                windowLeft=INF if wl is None else wl, windowRight=0,
                                qPosOffset=rows - 1)
                oracle.assert_close(out[b].float().cpu().numpy(), want, "f16")
    finally:
        ex.setStream(None)


@pytest.mark.parametrize("parts", [1, 2, 4, 8])
def test_sharded_partials_merge_equals_unsharded(ex, parts):
    """KV sequence cut into `parts` shards: per-shard partials + merge == whole."""
    import torch
    from runntime_b200.engine import decode_batched, merge_partials, shard_rows
    batch, rows, heads, hd = 6, 1000, 8, 52
    q, kc, vc, _, _, _ = _batched_inputs(batch, rows, heads, heads, hd, "f16", [rows] * batch)
    dev = torch.device("cuda", 0)
    qd = q.to(dev)
    partials = torch.zeros(parts, batch, heads, 2 + hd, dtype=torch.float32, device=dev)
    out = torch.empty_like(qd)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        for r in range(parts):
            s, e = shard_rows(rows, parts, r)
            ks = kc[:, s:e].contiguous().to(dev)
            vs = vc[:, s:e].contiguous().to(dev)
            decode_batched(ex, qd, None, ks, vs, dtype="f16", batch=batch, cacheRows=e - s,
                           qHeads=heads, kvHeads=heads, headDim=hd, kvLen=e - s,
                           partialsOut=partials[r], splits=0 if r % 2 else 2)
            ex.sync()
        merge_partials(ex, partials, parts, batch * heads, hd, out, "f16")
        ex.sync()
    finally:
        ex.setStream(None)
    # GPU merge == oracle merge of the same partials == unsharded attention
    host = partials.cpu().numpy().reshape(parts, batch * heads, 2 + hd)
    oracle.assert_close(out.float().cpu().numpy(), oracle.merge_partials(host), "f16")
    for b in range(batch):
        want = sdpa_ref(q[b:b + 1].float().numpy(), kc[b].float().numpy(), vc[b].float().numpy(),
                        qHeads=heads, kvHeads=heads, headDim=hd)
        oracle.assert_close(out[b].float().cpu().numpy(), want, "f16")


def test_write_rows_standalone(ex):
    import runntime_b200 as rt
    dst = np.arange(8 * 6, dtype=np.float32).reshape(8, 6)
    src = -np.arange(2 * 6, dtype=np.float32).reshape(2, 6) - 1
    for dtype in ("f32", "f16"):
        d = ex.upload(dst, [8, 6], dtype)
        view = rt.writeRows(d, ex.upload(src, [2, 6], dtype), 3)
        got = rt.toArray(view, ex).reshape(5, 6)
        want = dst.copy()
        oracle.write_rows(want, src, 3)
        assert np.array_equal(got, want[:5])
        assert np.array_equal(ex.readback(d.buffer, d.shape).reshape(8, 6), want)
        assert view.buffer is d.buffer
