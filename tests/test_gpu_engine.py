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
        # one more token with the layer's two attentions in one launch: the self step (append
        # + attend) and the cross-attention, whose query is another projection
        kn, vn = torch.randn(batch, w, generator=g).half(), torch.randn(batch, w, generator=g).half()
        qa, qb = (torch.randn(batch, w, generator=g) / 6).half(), (torch.randn(batch, w, generator=g) / 6).half()
        before = ex.launchCount()
        eng.stepWithCross(qa.to(dev), kn.to(dev), vn.to(dev), out, qb.to(dev), out2)
        ex.sync()
        assert ex.launchCount() == before + 1
        for b in range(batch):
            kb = torch.cat([ks[:, b], kn[b:b + 1]]).float().numpy()
            vb = torch.cat([vs[:, b], vn[b:b + 1]]).float().numpy()
            want = sdpa_ref(qa[b:b + 1].float().numpy(), kb, vb, qHeads=heads, kvHeads=heads,
                            headDim=hd, windowRight=0, qPosOffset=steps)
            oracle.assert_close(out[b].float().cpu().numpy(), want, "f16", "self, one launch")
            want = sdpa_ref(qb[b:b + 1].float().numpy(), ck[b].float().numpy(), cv[b].float().numpy(),
                            qHeads=heads, kvHeads=heads, headDim=hd)
            oracle.assert_close(out2[b].float().cpu().numpy(), want, "f16", "cross, one launch")
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


def _emulated_world(world, batch, heads, hd, dev):
    """Exchange structures for `world` ranks that all live on this GPU (plain torch
    allocations stand where the peers' mapped blocks would)."""
    import torch
    from runntime_b200.engine import exchange_sizes, make_exchange
    nfloat, nword, nstage = exchange_sizes(world, batch, heads, hd)
    partials = [torch.zeros(nfloat, dtype=torch.float32, device=dev) for _ in range(world)]
    control = [torch.zeros(nword, dtype=torch.int32, device=dev) for _ in range(world)]
    stage = [torch.zeros(nstage, dtype=torch.float32, device=dev) for _ in range(world)]
    xs = [make_exchange(world, r, partials, control, stage[r]) for r in range(world)]
    return xs, control, (partials, stage)


@pytest.mark.parametrize("world,splits,dtype", [(1, 0, "f16"), (2, 0, "f16"), (4, 3, "f16"),
                                                (8, 0, "f16"), (3, 2, "f32")])
def test_peer_exchange_of_partials_emulated_on_one_gpu(ex, world, splits, dtype):
    """The cross-GPU exchange with every "rank" on this GPU: the ranks' decode
    launches run one after the other (each sends every sequence's rows to the rank
    that owns the sequence and signals it), then each rank's merge finds all arrival
    words already set and writes its own sequences.  Three steps, so that both halves
    of the buffers and the step counters are exercised.  Nine sequences: the ranks
    own unequal numbers of them."""
    import torch
    from runntime_b200.engine import owned_sequences, shard_rows
    batch, heads, kvHeads, hd, rows = 9, 8, 4, 64, 700
    dev = torch.device("cuda", 0)
    tdt = torch.float16 if dtype == "f16" else torch.float32
    g = torch.Generator().manual_seed(9)
    xs, control, keep = _emulated_world(world, batch, heads, hd, dev)
    outs = [torch.full((batch, heads * hd), 7.0, dtype=tdt, device=dev) for _ in range(world)]
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
            for r in range(world):
                first, n = owned_sequences(batch, world, r)
                got = outs[r].float().cpu().numpy()
                for b in range(batch):
                    if first <= b < first + n:
                        ref = oracle.sdpa_ref(q[b:b + 1].float().numpy(), k[b].float().numpy(),
                                              v[b].float().numpy(), qHeads=heads, kvHeads=kvHeads,
                                              headDim=hd)
                        oracle.assert_close(got[b], ref.reshape(-1), dtype,
                                            f"step {step} rank {r} seq {b}")
                    else:
                        assert (got[b] == 7.0).all()       # another rank's sequence: untouched
            for r, c in enumerate(control):
                c = c.cpu()
                assert int(c[world]) == step + 1                       # the rank's step counter
                assert (c[world + 2:] == 0).all()                      # arrival counters back at zero
                assert (c[:world] == step + 1).all()                   # every rank's arrival word
    finally:
        ex.setStream(None)


def test_merge_gives_up_when_a_rank_never_signals(ex):
    """A bounded wait that runs out: two ranks emulated on this GPU, rank 0 runs its
    whole step, rank 1 never launches — rank 0's merge polls rank 1's arrival word a
    (shortened) bounded number of times, writes zeros and records the failure, which
    rt_sync turns into EXECUTION_FAILED.  Nothing spins without a bound."""
    import torch
    import runntime_b200 as rt
    from runntime_b200._lib import OPT_WAIT_POLLS
    from runntime_b200.engine import decode_batched
    batch, heads, hd, rows = 4, 8, 52, 300
    dev = torch.device("cuda", 0)
    g = torch.Generator().manual_seed(2)
    xs, control, keep = _emulated_world(2, batch, heads, hd, dev)
    k = torch.randn(batch, rows, heads * hd, generator=g).half().to(dev)
    v = torch.randn(batch, rows, heads * hd, generator=g).half().to(dev)
    q = (torch.randn(batch, heads * hd, generator=g) / 7).half().to(dev)
    out = torch.full((batch, heads * hd), 3.0, dtype=torch.float16, device=dev)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    ex.setOption(OPT_WAIT_POLLS, 2000)      # a couple of milliseconds
    try:
        decode_batched(ex, q, out, k, v, dtype="f16", batch=batch, cacheRows=rows, qHeads=heads,
                       kvHeads=heads, headDim=hd, kvLen=rows, exchange=xs[0])
        with pytest.raises(rt.RunntimeError, match="bounded device-side wait ran out") as e:
            ex.sync()
        assert e.value.code == "EXECUTION_FAILED"
        got = out.float().cpu().numpy()
        assert (got[:2] == 0).all() and (got[2:] == 3.0).all()   # rank 0 merges sequences 0 and 1
        ex.sync()                                                # the status word was cleared
    finally:
        ex.setOption(OPT_WAIT_POLLS, 1 << 20)
        ex.setStream(None)


@pytest.mark.parametrize("world", [1, 2, 3])
def test_sharded_kv_cache_engine_appends_on_the_owning_rank(ex, world):
    """Caches split by position over `world` ranks (all emulated on this GPU): each
    step's new K/V row lands in the shard that owns the position and nowhere else,
    the ranks' partials merge to the attention over the whole sequence, and stepping
    walks across the shard boundaries."""
    import torch
    from runntime_b200.engine import ShardedKvCacheEngine, owned_sequences, shard_of_position
    batch, heads, hd, maxPositions, steps = 3, 8, 36, 40, 31
    dev = torch.device("cuda", 0)
    xs, control, keep = _emulated_world(world, batch, heads, hd, dev)
    engines = [ShardedKvCacheEngine(ex, xs[r], batch=batch, maxPositions=maxPositions, qHeads=heads,
                                    kvHeads=heads, headDim=hd, dtype="f16", device=dev)
               for r in range(world)]
    g = torch.Generator().manual_seed(5)
    w = heads * hd
    ks = torch.randn(steps, batch, w, generator=g).half()
    vs = torch.randn(steps, batch, w, generator=g).half()
    qs = (torch.randn(steps, batch, w, generator=g) / 6).half()
    outs = [torch.empty(batch, w, dtype=torch.float16, device=dev) for _ in range(world)]
    try:
        for t in range(steps):
            qd, kd, vd = qs[t].to(dev), ks[t].to(dev), vs[t].to(dev)
            for phase in (1, 2):
                for r in range(world):
                    engines[r].step(qd, kd, vd, outs[r], phases=phase)
            ex.sync()
            if t in (0, 1, 12, 13, 14, 20, 27, 30):
                for r in range(world):
                    first, n = owned_sequences(batch, world, r)
                    for b in range(first, first + n):
                        want = sdpa_ref(qs[t, b:b + 1].float().numpy(), ks[:t + 1, b].float().numpy(),
                                        vs[:t + 1, b].float().numpy(), qHeads=heads, kvHeads=heads,
                                        headDim=hd, windowRight=0, qPosOffset=t)
                        oracle.assert_close(outs[r][b].float().cpu().numpy(), want, "f16",
                                            f"t={t} rank {r} seq {b}")
        shardRows = engines[0].shardRows
        for r in range(world):
            kc = engines[r].k.cpu()
            for row in range(shardRows):
                t = r * shardRows + row
                if t < steps:
                    owner, local = shard_of_position(t, shardRows)
                    assert (owner, local) == (r, row)
                    assert torch.equal(kc[:, row], ks[t])
                else:
                    assert (kc[:, row] == 0).all()
    finally:
        ex.setStream(None)


def test_exchange_blocks_from_the_c_abi_on_one_gpu(ex):
    """rt_xmem_*: two ranks that live in one process attach each other's blocks (the
    one-process-several-devices form; here both on this GPU) and run a step."""
    import torch
    from runntime_b200.engine import ExchangeMemory, decode_batched, owned_sequences, shard_rows
    import runntime_b200 as rt
    batch, heads, hd, rows, world = 6, 8, 52, 500, 2
    dev = torch.device("cuda", 0)
    mems = [ExchangeMemory(0, world, r, batch, heads, hd) for r in range(world)]
    with pytest.raises(rt.RunntimeError, match="rank 1 has not been imported or attached") as e:
        mems[0].exchange()
    assert e.value.code == "NOT_INITIALIZED"
    handle = mems[0].export()
    assert len(handle) == 64
    mems[0].attach(1, mems[1])
    mems[1].attach(0, mems[0])
    with pytest.raises(rt.RunntimeError, match="already mapped"):
        mems[1].attach(0, mems[0])
    xs = [m.exchange() for m in mems]
    g = torch.Generator().manual_seed(8)
    k = torch.randn(batch, rows, heads * hd, generator=g).half()
    v = torch.randn(batch, rows, heads * hd, generator=g).half()
    q = (torch.randn(batch, heads * hd, generator=g) / 7).half()
    outs = [torch.empty(batch, heads * hd, dtype=torch.float16, device=dev) for _ in range(world)]
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    try:
        shards = []
        for r in range(world):
            s, e_ = shard_rows(rows, world, r)
            shards.append((k[:, s:e_].contiguous().to(dev), v[:, s:e_].contiguous().to(dev), e_ - s))
        for phase in (1, 2):
            for r in range(world):
                xs[r].phases = phase
                ks_, vs_, n = shards[r]
                decode_batched(ex, q.to(dev), outs[r], ks_, vs_, dtype="f16", batch=batch,
                               cacheRows=n, qHeads=heads, kvHeads=heads, headDim=hd, kvLen=n,
                               exchange=xs[r])
        ex.sync()
        for r in range(world):
            first, n = owned_sequences(batch, world, r)
            for b in range(first, first + n):
                ref = oracle.sdpa_ref(q[b:b + 1].float().numpy(), k[b].float().numpy(),
                                      v[b].float().numpy(), qHeads=heads, kvHeads=heads, headDim=hd)
                oracle.assert_close(outs[r][b].float().cpu().numpy(), ref.reshape(-1), "f16")
    finally:
        ex.setStream(None)
        for m in mems:
            m.destroy()
