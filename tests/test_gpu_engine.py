"""Batched prefill, the KV-cache engine and context lifetime on the GPU."""
import ctypes as C
import math

import numpy as np
import pytest

import oracle
from gpu_harness import ex  # noqa: F401
from oracle import sdpa_ref

pytestmark = pytest.mark.gpu
INF = math.inf


def _padded_batch_reference(q, k, v, lens, S, **kw):
    """Oracle for the padded-batch form: segments derived from the lengths."""
    T = q.shape[0]
    segs = np.zeros((T, 2), np.float32)
    for b, L in enumerate(lens):
        segs[b * S:b * S + L] = (b * S, b * S + L)
    return sdpa_ref(q, k, v, segs=segs, **kw)


@pytest.mark.parametrize("dtype,heads,kvHeads,hd,wl,wr", [
    ("f32", 12, 12, 32, INF, INF),     # MiniLM shape, bidirectional
    ("f16", 3, 1, 256, 64, 64),        # EmbeddingGemma shape, sliding
    ("f16", 3, 1, 256, INF, INF),      # EmbeddingGemma shape, global
    ("f16", 8, 8, 128, INF, 0),        # causal
    ("f16", 4, 2, 64, 20, 0),
])
def test_padded_batch_prefill(ex, dtype, heads, kvHeads, hd, wl, wr):
    import torch
    from runntime_b200.engine import prefill_batched
    batch, S = 4, 160
    lens = [160, 16, 1, 97]
    g = torch.Generator().manual_seed(3)
    tdt = torch.float16 if dtype == "f16" else torch.float32
    q = (torch.randn(batch * S, heads * hd, generator=g) * hd ** -0.25).to(tdt)
    k = (torch.randn(batch * S, kvHeads * hd, generator=g) * hd ** -0.25).to(tdt)
    v = torch.randn(batch * S, kvHeads * hd, generator=g).to(tdt)
    dev = torch.device("cuda", 0)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    out = torch.full_like(qd, 5.0)
    ld = torch.tensor(lens, dtype=torch.int32, device=dev)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        prefill_batched(ex, qd, kd, vd, out, dtype=dtype, batch=batch, seqStride=S, seqLens=ld,
                        qHeads=heads, kvHeads=kvHeads, headDim=hd, windowLeft=wl, windowRight=wr)
        ex.sync()
    finally:
        ex.setStream(None)
    want = _padded_batch_reference(q.float().numpy(), k.float().numpy(), v.float().numpy(), lens, S,
                                   qHeads=heads, kvHeads=kvHeads, headDim=hd, windowLeft=wl,
                                   windowRight=wr)
    got = out.float().cpu().numpy()
    oracle.assert_close(got, want, dtype)
    for b, L in enumerate(lens):  # rows past a sequence's length are zero
        assert (got[b * S + L:(b + 1) * S] == 0).all()


def test_kv_cache_engine_steps_like_the_decoder_loop(ex):
    import torch
    from runntime_b200.engine import KvCacheEngine
    batch, heads, hd, steps, crossRows = 3, 8, 36, 40, 200
    eng = KvCacheEngine(ex, batch=batch, maxPositions=64, qHeads=heads, kvHeads=heads, headDim=hd,
                        dtype="f16")
    dev = eng.k.device
    g = torch.Generator().manual_seed(5)
    w = heads * hd
    ks = torch.randn(steps, batch, w, generator=g).half()
    vs = torch.randn(steps, batch, w, generator=g).half()
    qs = (torch.randn(steps, batch, w, generator=g) / 6).half()
    ck = torch.randn(batch, crossRows, w, generator=g).half()
    cv = torch.randn(batch, crossRows, w, generator=g).half()
    ckd, cvd = ck.to(dev), cv.to(dev)
    eng.setCross(ckd, cvd, crossRows)
    out = torch.empty(batch, w, dtype=torch.float16, device=dev)
    out2 = torch.empty_like(out)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        for t in range(steps):
            eng.step(qs[t].to(dev), ks[t].to(dev), vs[t].to(dev), out)
            eng.crossAttend(qs[t].to(dev), out2)
            ex.sync()
            if t in (0, 1, 17, 39):
                for b in range(batch):
                    want = sdpa_ref(qs[t, b:b + 1].float().numpy(), ks[:t + 1, b].float().numpy(),
                                    vs[:t + 1, b].float().numpy(), qHeads=heads, kvHeads=heads,
                                    headDim=hd, windowRight=0, qPosOffset=t)
                    oracle.assert_close(out[b].float().cpu().numpy(), want, "f16", f"self t={t}")
                    want = sdpa_ref(qs[t, b:b + 1].float().numpy(), ck[b].float().numpy(),
                                    cv[b].float().numpy(), qHeads=heads, kvHeads=heads, headDim=hd)
                    oracle.assert_close(out2[b].float().cpu().numpy(), want, "f16", f"cross t={t}")
        assert torch.equal(eng.k[:, :steps].cpu(), ks.transpose(0, 1))
        assert (eng.k[:, steps:] == 0).all()
        with pytest.raises(ValueError, match="exceed dst capacity 64"):
            for _ in range(30):
                eng.step(qs[0].to(dev), ks[0].to(dev), vs[0].to(dev), out)
    finally:
        ex.setStream(None)


def test_c_abi_argument_errors_carry_codes_and_messages(ex):
    import runntime_b200 as rt
    from runntime_b200._lib import AttnArgs, DecodeArgs, check
    buf = ex.upload(np.zeros(64, np.float32), [4, 16])
    a = AttnArgs()
    a.q = a.k = a.v = a.out = buf.buffer.ptr
    a.dtype, a.qLen, a.kvLen, a.qHeads, a.kvHeads, a.headDim = 0, 4, 4, 3, 2, 8
    a.windowLeft = a.windowRight = rt._lib.WINDOW_INF
    with pytest.raises(rt.RunntimeError, match="qHeads 3 not divisible by kvHeads 2") as e:
        check(ex._lib.rt_attn(ex.ctx, C.byref(a)), ex.ctx)
    assert e.value.code == "INVALID_ARGUMENT"
    a.qHeads, a.kvHeads, a.headDim = 1, 1, 520
    with pytest.raises(rt.RunntimeError, match=r"headDim 520 exceeds the kernel's max \(512\)"):
        check(ex._lib.rt_attn(ex.ctx, C.byref(a)), ex.ctx)
    a.headDim, a.windowRight, a.kvLen = 8, 0, 3
    with pytest.raises(rt.RunntimeError, match=r"qPosOffset\+qLen 4 exceeds key rows kvLen 3"):
        check(ex._lib.rt_attn(ex.ctx, C.byref(a)), ex.ctx)
    a.qLen, a.kvLen, a.headDim = 1, 4, 130
    with pytest.raises(rt.RunntimeError, match=r"headDim 130 exceeds the kernel's max \(128\)"):
        check(ex._lib.rt_attn(ex.ctx, C.byref(a)), ex.ctx)
    with pytest.raises(rt.RunntimeError, match="exceed dst capacity 4") as e:
        check(ex._lib.rt_kv_append(ex.ctx, buf.buffer.ptr, buf.buffer.ptr, 3, 2, 16, 4, 0), ex.ctx)
    assert e.value.code == "INVALID_ARGUMENT"
    with pytest.raises(rt.RunntimeError) as e:
        ex.upload(np.zeros(0, np.float32), [0, 8])
    assert e.value.code == "INVALID_ARGUMENT"
    d = DecodeArgs()
    with pytest.raises(rt.RunntimeError) as e:
        check(ex._lib.rt_attn_decode(ex.ctx, C.byref(d)), ex.ctx)
    assert e.value.code == "INVALID_ARGUMENT"
    ex.destroy(buf)


def test_dispose_frees_everything_and_later_use_fails(ex):
    import runntime_b200 as rt
    e2 = rt.CudaExecutor(0)
    x = e2.upload(np.ones(32, np.float32), [4, 8])
    y = rt.sdpa(x, x, x, dict(qHeads=1, kvHeads=1, headDim=8, windowLeft=INF, windowRight=INF))
    assert rt.toArray(y, e2).shape == (32,)
    assert e2.launchCount() == 1
    handle = e2._ctx
    e2.dispose()
    with pytest.raises(rt.RunntimeError) as err:
        e2.sync()
    assert err.value.code == "RESOURCE_DISPOSED"
    assert e2._lib.rt_sync(handle) == 7  # the C ABI recognises the dead handle too


def test_no_buffer_leak_across_evals(ex):
    import runntime_b200 as rt
    base = ex.liveBuffers()
    x = ex.upload(oracle.random_f32(64 * 32, 1), [64, 32])
    for _ in range(5):
        y = rt.sdpa(x, x, x, dict(qHeads=2, kvHeads=2, headDim=16, windowLeft=INF, windowRight=0))
        z = rt.sdpa(y, x, x, dict(qHeads=2, kvHeads=2, headDim=16, windowLeft=INF, windowRight=0))
        rt.toArray(z, ex)
        ex.releaseValues([z])
    assert ex.liveBuffers() == base + 1
    ex.destroy(x)
    assert ex.liveBuffers() == base


@pytest.mark.parametrize("world,splits,dtype", [(1, 0, "f16"), (2, 0, "f16"), (4, 3, "f16"),
                                                (8, 0, "f16"), (3, 2, "f32")])
def test_peer_exchange_of_partials_emulated_on_one_gpu(ex, world, splits, dtype):
    """The cross-GPU exchange with every "rank" on this GPU: the ranks' decode
    launches run one after the other (each writes its rows into all the buffers and
    signals), then each rank's merge finds all arrival words already set.  Three
    steps, so that both halves of the buffers and the step counters are exercised."""
    import torch
    from runntime_b200.engine import decode_batched, exchange_words, make_exchange, shard_rows
    batch, heads, kvHeads, hd, rows = 5, 8, 4, 64, 700
    dev = torch.device("cuda", 0)
    tdt = torch.float16 if dtype == "f16" else torch.float32
    g = torch.Generator().manual_seed(9)
    units = batch * heads
    nfloat, nword = exchange_words(world, units, hd)
    partials = [torch.zeros(nfloat, dtype=torch.float32, device=dev) for _ in range(world)]
    control = [torch.zeros(nword, dtype=torch.int32, device=dev) for _ in range(world)]
    xs = [make_exchange(world, r, partials, control) for r in range(world)]
    outs = [torch.empty(batch, heads * hd, dtype=tdt, device=dev) for _ in range(world)]
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        for step in range(3):
            k = torch.randn(batch, rows, kvHeads * hd, generator=g).to(tdt)
            v = torch.randn(batch, rows, kvHeads * hd, generator=g).to(tdt)
            q = (torch.randn(batch, heads * hd, generator=g) / 8).to(tdt)
            qd = q.to(dev)
            shards = []
            for r in range(world):
                s, e = shard_rows(rows, world, r)
                shards.append((k[:, s:e].contiguous().to(dev), v[:, s:e].contiguous().to(dev), e - s))
            # decode kernels of all ranks first, their merges after: nothing waits on a later launch
            from runntime_b200._lib import DecodeArgs, DTYPE_CODE, check
            import ctypes as C
            for r in range(world):
                ks, vs, n = shards[r]
                d = DecodeArgs()
                d.q, d.out = qd.data_ptr(), outs[r].data_ptr()
                d.kCache, d.vCache = ks.data_ptr(), vs.data_ptr()
                d.cacheSeqStride = n * kvHeads * hd
                d.dtype = DTYPE_CODE[dtype]
                d.batch, d.cacheRows, d.kvLen = batch, n, n
                d.qHeads, d.kvHeads, d.headDim = heads, kvHeads, hd
                d.windowLeft, d.splits = 0x3fffffff, splits
                d.exchange = C.pointer(xs[r])
                shards[r] = shards[r] + (d,)
            for phase in (1, 2):   # 1: attend and send, 2: wait and merge
                for r in range(world):
                    xs[r].phases = phase
                    check(ex._lib.rt_attn_decode(ex.ctx, C.byref(shards[r][3])), ex.ctx)
            ex.sync()
            for b in range(batch):
                ref = oracle.sdpa_ref(q[b:b + 1].float().numpy(), k[b].float().numpy(),
                                      v[b].float().numpy(), qHeads=heads, kvHeads=kvHeads,
                                      headDim=hd)
                for r in range(world):
                    oracle.assert_close(outs[r][b].float().cpu().numpy(), ref.reshape(-1), dtype,
                                        f"step {step} rank {r} seq {b}")
            assert all(int(c[world].item()) == step + 1 for c in control)      # step counters
            assert all((c[:world] == step + 1).all().item() for c in control)  # arrival words
    finally:
        ex.setStream(None)
