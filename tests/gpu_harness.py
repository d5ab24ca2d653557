"""Shared by the GPU suites: runs one sdpa through the operator API (which calls
the C ABI) and checks it against the CPU oracle — the counterpart of the
reference's checkSdpa (packages/runntime/test/core/kernels/attention/
checkSdpa.ts:130-227)."""
from __future__ import annotations

import numpy as np
import pytest

import oracle
from oracle import SdpaCase, make_inputs, sdpa_ref_inputs


def have_gpu() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


@pytest.fixture(scope="session")
def ex():
    """One executor (context) for the whole GPU session."""
    import runntime_b200 as rt
    e = rt.CudaExecutor(0)
    yield e
    e.dispose()


def run_sdpa(ex, x: oracle.SdpaInputs):
    """Uploads the inputs, builds the op the way a model would, reads it back."""
    import runntime_b200 as rt
    c, dtype = x.case, x.dtype
    held = []

    def up(a, shape, dt="f32"):
        v = ex.upload(a, shape, dt)
        held.append(v)
        return v

    opts = dict(qHeads=c.qHeads, kvHeads=c.kvHeads, headDim=c.headDim, windowLeft=c.windowLeft,
                windowRight=c.windowRight, qPosOffset=c.qPosOffset,
                sinks=up(x.sinks, [1, c.qHeads]) if x.sinks is not None else None,
                segments=up(x.segs, [c.qLen, 2]) if x.segs is not None else None,
                maxSegment=c.maxSegment)
    if c.packed:
        w = (c.qHeads + 2 * c.kvHeads) * c.headDim
        out = rt.sdpaPacked(up(x.packed_qkv, [c.qLen, w], dtype), opts)
    else:
        if x.keyBias is not None:
            opts["keyBias"] = dict(start=x.keyBias[0], end=x.keyBias[1], value=x.keyBias[2])
        out = rt.sdpa(up(x.q, [c.qLen, c.qHeads * c.headDim], dtype),
                      up(x.k, [c.kvLen, c.kvHeads * c.headDim], dtype),
                      up(x.v, [c.kvLen, c.kvHeads * c.headDim], dtype), opts)
    got = rt.toArray(out, ex)
    ex.releaseValues([out])
    for v in held:
        ex.destroy(v)
    return got


def check_sdpa(ex, c: SdpaCase, dtype: str = "f32", route: str | None = None):
    x = make_inputs(c, dtype)
    before = len(ex.dispatches)
    got = run_sdpa(ex, x)
    if route is not None:
        assert ex.dispatches[before:] == [route], ex.dispatches[before:]
    want = sdpa_ref_inputs(x)
    oracle.assert_close(got, want, dtype, f"{c} [{dtype}]")
    return got, want
