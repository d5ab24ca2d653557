"""rt_attn_decode_noalloc: the decode entry point for callers that cannot
allocate device memory — a loop whose memory budget was fixed before the model
started, a plugin living inside another framework's pool, code that holds the
allocator lock.  It takes no context; its split scratch is a fixed array inside
the library.

The tests drive it through the C ABI and check it, on two calls in a row — the
second call meets the first one's leftovers in the shared array — against the f64
oracle per sequence (appended row included) and against rt_attn_decode (the
context-owning entry point), within the f16 / f32 tolerance the other decode
tests use: the whole-row path with key splits (which needs the scratch), the
sub-row path of wide heads, f32, and the split counts that need no scratch.  They
also check the refusals of requests larger than the fixed scratch and the status
reader.  This file is named to be collected last so that a failure here cannot
hide the rest of the suite."""
import ctypes as C

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def _args(L, q, out, k, v, kn, vn, lens, *, dtype, batch, rows, heads, hd, kvLen, splits):
    a = L.DecodeArgs()
    a.q, a.out, a.kCache, a.vCache = q.data_ptr(), out.data_ptr(), k.data_ptr(), v.data_ptr()
    a.kNew, a.vNew, a.kvLens = kn.data_ptr(), vn.data_ptr(), lens.data_ptr()
    a.cacheSeqStride = rows * heads * hd
    a.dtype, a.batch, a.cacheRows, a.kvLen = L.DTYPE_CODE[dtype], batch, rows, kvLen
    a.qHeads, a.kvHeads, a.headDim = heads, heads, hd
    a.windowLeft, a.splits = L.WINDOW_INF, splits
    return a


@pytest.mark.parametrize("dtype,heads,hd,splits", [
    ("f16", 8, 52, (3, 4)),      # whole-row bulk path, key splits through the fixed scratch
    ("f16", 32, 128, (2, 5)),    # sub-row path of wide heads
    ("f32", 8, 36, (3, 2)),
    ("f16", 8, 52, (0, 1)),      # the library's own choice, and one split: no scratch needed
])
def test_decode_without_allocation(dtype, heads, hd, splits):
    import torch
    import runntime_b200 as rt
    import runntime_b200._lib as L
    lib = L.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    batch, rows = 7, 1200
    tdt = torch.float16 if dtype == "f16" else torch.float32
    g = torch.Generator().manual_seed(21)
    w = heads * hd
    kc = torch.randn(batch, rows, w, generator=g).to(tdt)
    vc = torch.randn(batch, rows, w, generator=g).to(tdt)
    lens = torch.tensor([1200, 1, 2, 640, 999, 33, 1187], dtype=torch.int32)
    stream = torch.cuda.current_stream().cuda_stream
    ex = rt.CudaExecutor(0)
    ex.setStream(stream)
    try:
        for call in range(2):  # the second call sees the first call's scratch contents
            q = (torch.randn(batch, w, generator=g) / hd ** 0.5).to(tdt)
            kn = torch.randn(batch, w, generator=g).to(tdt)
            vn = torch.randn(batch, w, generator=g).to(tdt)
            qd, knd, vnd = q.to(dev), kn.to(dev), vn.to(dev)
            ld = lens.to(dev)
            k1, v1, k2, v2 = kc.to(dev), vc.to(dev), kc.to(dev), vc.to(dev)
            want = torch.zeros(batch, w, dtype=tdt, device=dev)
            got = torch.full_like(want, 9.0)
            kw = dict(dtype=dtype, batch=batch, rows=rows, heads=heads, hd=hd, kvLen=1200,
                      splits=splits[call])
            L.check(lib.rt_attn_decode(ex.ctx, C.byref(_args(L, qd, want, k1, v1, knd, vnd, ld, **kw))),
                    ex.ctx)
            ex.sync()
            L.check(lib.rt_attn_decode_noalloc(C.byref(_args(L, qd, got, k2, v2, knd, vnd, ld, **kw)),
                                               C.c_void_p(stream)))
            L.check(lib.rt_attn_decode_noalloc_status(C.c_void_p(stream)))
            g_np = got.float().cpu().numpy()
            oracle.assert_close(g_np, want.float().cpu().numpy(), dtype, f"call {call} vs rt_attn_decode")
            for b, n in enumerate(lens.tolist()):
                kb, vb = kc[b, :n].clone(), vc[b, :n].clone()
                kb[n - 1], vb[n - 1] = kn[b], vn[b]
                ref = oracle.sdpa_ref(q[b:b + 1].float().numpy(), kb.float().numpy(),
                                      vb.float().numpy(), qHeads=heads, kvHeads=heads, headDim=hd,
                                      windowRight=0, qPosOffset=n - 1)
                oracle.assert_close(g_np[b], ref, dtype, f"call {call} seq {b} vs oracle")
            assert torch.equal(k1, k2) and torch.equal(v1, v2)  # the fused append too
    finally:
        ex.setStream(None)
        ex.dispose()


def test_requests_past_the_fixed_scratch_are_refused():
    import torch
    import runntime_b200._lib as L
    lib = L.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    t = torch.zeros(64, dtype=torch.float16, device=dev)
    lens = torch.ones(1, dtype=torch.int32, device=dev)
    # nothing is launched: the pointers are never followed
    big = _args(L, t, t, t, t, t, t, lens, dtype="f16", batch=60000, rows=1200, heads=8, hd=52,
                kvLen=1200, splits=8)
    assert lib.rt_attn_decode_noalloc(C.byref(big), C.c_void_p(stream)) == 6  # INVALID_ARGUMENT
    msg = lib.rt_last_error(None).decode()
    assert "exceeds the fixed scratch" in msg and "1048576" in msg
    # few floats but more (sequence, head block) counters than the array holds:
    # 5000 sequences x 2 splits x 1 head x (2 + 4) floats = 60000 floats, 5000 counters
    many = _args(L, t, t, t, t, t, t, lens, dtype="f16", batch=5000, rows=64, heads=1, hd=4,
                 kvLen=64, splits=2)
    assert lib.rt_attn_decode_noalloc(C.byref(many), C.c_void_p(stream)) == 6
    msg = lib.rt_last_error(None).decode()
    assert "5000 counters (limit 4096)" in msg
    assert lib.rt_attn_decode_noalloc_status(C.c_void_p(stream)) == 0


def test_status_reader_reports_a_length_past_the_cache():
    import torch
    import runntime_b200._lib as L
    lib = L.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    stream = torch.cuda.current_stream().cuda_stream
    batch, rows, heads, hd = 2, 64, 8, 52
    w = heads * hd
    g = torch.Generator().manual_seed(3)
    k = torch.randn(batch, rows, w, generator=g).half().to(dev)
    v = torch.randn(batch, rows, w, generator=g).half().to(dev)
    q = torch.randn(batch, w, generator=g).half().to(dev)
    lens = torch.tensor([64, 65], dtype=torch.int32, device=dev)
    out = torch.full((batch, w), 5.0, dtype=torch.float16, device=dev)
    a = _args(L, q, out, k, v, q, q, lens, dtype="f16", batch=batch, rows=rows, heads=heads, hd=hd,
              kvLen=64, splits=1)
    a.kNew = a.vNew = None
    L.check(lib.rt_attn_decode_noalloc(C.byref(a), C.c_void_p(stream)))
    assert lib.rt_attn_decode_noalloc_status(C.c_void_p(stream)) == 5       # EXECUTION_FAILED
    assert "kvLens entry exceeds cacheRows" in lib.rt_last_error(None).decode()
    assert lib.rt_attn_decode_noalloc_status(C.c_void_p(stream)) == 0       # reported once
    assert (out[1] == 0).all() and not (out[0] == 5.0).any()
