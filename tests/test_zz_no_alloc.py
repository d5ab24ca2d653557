"""rt_attn_decode_noalloc: the decode entry point for callers that cannot
allocate device memory — a loop whose memory budget was fixed before the model
started, a plugin living inside another framework's pool, code that holds the
allocator lock.  It takes no context; its split scratch is a fixed array inside
the library.

The test drives it through the C ABI with a split count that needs the scratch
and checks it against rt_attn_decode (the context-owning entry point) on two
calls in a row — the second call meets the first one's leftovers in the shared
array — within the f16 tolerance the other decode tests use.  It also checks the
refusal of a request larger than the fixed scratch.  This file is named to be
collected last so that a failure here cannot hide the rest of the suite."""
import ctypes as C

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


def _args(L, q, out, k, v, kn, vn, lens, *, batch, rows, heads, hd, kvLen, splits):
    a = L.DecodeArgs()
    a.q, a.out, a.kCache, a.vCache = q.data_ptr(), out.data_ptr(), k.data_ptr(), v.data_ptr()
    a.kNew, a.vNew, a.kvLens = kn.data_ptr(), vn.data_ptr(), lens.data_ptr()
    a.cacheSeqStride = rows * heads * hd
    a.dtype, a.batch, a.cacheRows, a.kvLen = L.RT_F16, batch, rows, kvLen
    a.qHeads, a.kvHeads, a.headDim = heads, heads, hd
    a.windowLeft, a.splits = L.WINDOW_INF, splits
    return a


def test_decode_without_allocation_matches_the_context_entry_point():
    import torch
    import runntime_b200 as rt
    import runntime_b200._lib as L
    lib = L.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    batch, rows, heads, hd = 7, 1200, 8, 52
    g = torch.Generator().manual_seed(21)
    w = heads * hd
    kc = torch.randn(batch, rows, w, generator=g).half()
    vc = torch.randn(batch, rows, w, generator=g).half()
    lens = torch.tensor([1200, 1, 2, 640, 999, 33, 1187], dtype=torch.int32)
    stream = torch.cuda.current_stream().cuda_stream
    ex = rt.CudaExecutor(0)
    ex.setStream(stream)
    try:
        for call in range(2):  # the second call sees the first call's scratch contents
            q = (torch.randn(batch, w, generator=g) / hd ** 0.5).half().to(dev)
            kn = torch.randn(batch, w, generator=g).half().to(dev)
            vn = torch.randn(batch, w, generator=g).half().to(dev)
            ld = lens.to(dev)
            k1, v1, k2, v2 = kc.to(dev), vc.to(dev), kc.to(dev), vc.to(dev)
            want = torch.zeros(batch, w, dtype=torch.float16, device=dev)
            got = torch.full_like(want, 9.0)
            kw = dict(batch=batch, rows=rows, heads=heads, hd=hd, kvLen=1200, splits=3 + call)
            L.check(lib.rt_attn_decode(ex.ctx, C.byref(_args(L, q, want, k1, v1, kn, vn, ld, **kw))),
                    ex.ctx)
            ex.sync()
            L.check(lib.rt_attn_decode_noalloc(C.byref(_args(L, q, got, k2, v2, kn, vn, ld, **kw)),
                                               C.c_void_p(stream)))
            torch.cuda.synchronize()
            oracle.assert_close(got.float().cpu().numpy(), want.float().cpu().numpy(), "f16",
                                f"call {call}")
            assert torch.equal(k1, k2) and torch.equal(v1, v2)  # the fused append too
        # a request past the fixed scratch is refused before anything is enqueued
        big = _args(L, q, got, k2, v2, kn, vn, ld, batch=batch, rows=rows, heads=heads, hd=hd,
                    kvLen=1200, splits=3)
        big.batch, big.splits = 60000, 8
        status = lib.rt_attn_decode_noalloc(C.byref(big), C.c_void_p(stream))
        assert status == 6  # INVALID_ARGUMENT
        msg = lib.rt_last_error(None).decode()
        assert "exceeds the fixed scratch" in msg and "1048576" in msg
    finally:
        ex.setStream(None)
        ex.dispose()
