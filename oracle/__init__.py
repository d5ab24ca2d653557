"""CPU oracle for the attention hot path — TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import
this package.  The product (``runntime_b200``) never does.

``liboracle.so`` is built from ``sdpa_oracle.c`` by ``make -C oracle``; this
module is the ctypes face of it plus the test-input builder that mirrors the
reference's ``checkSdpa`` harness
(packages/runntime/test/core/kernels/attention/checkSdpa.ts:130-161).
"""
from __future__ import annotations

import ctypes as C
import math
import os
import subprocess
from dataclasses import dataclass, field
from typing import Optional

import numpy as np

WINDOW_INF = 0x3FFFFFFF
_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")


class _Dims(C.Structure):
    _fields_ = [
        ("qLen", C.c_int64), ("kvLen", C.c_int64),
        ("qHeads", C.c_int32), ("kvHeads", C.c_int32), ("headDim", C.c_int32),
        ("windowLeft", C.c_int64), ("windowRight", C.c_int64),
        ("qPosOffset", C.c_int64),
        ("packed", C.c_int32), ("hasKeyBias", C.c_int32),
        ("biasStart", C.c_int64), ("biasEnd", C.c_int64),
        ("biasValue", C.c_double),
    ]


def build(force: bool = False) -> str:
    """Compile liboracle.so if it is missing or older than its source (or ``force``)."""
    src = os.path.join(_HERE, "sdpa_oracle.c")
    stale = not os.path.exists(_LIB_PATH) or os.path.getmtime(src) > os.path.getmtime(_LIB_PATH)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-B" if force else "-s", "liboracle.so"])
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _win(w) -> int:
    if w is None or w == math.inf:
        return WINDOW_INF
    return min(int(w), WINDOW_INF)


@dataclass
class SdpaCase:
    """One attention call, with the reference harness's option names."""
    qLen: int
    kvLen: int
    qHeads: int
    kvHeads: int
    headDim: int
    windowLeft: float = math.inf
    windowRight: float = math.inf
    qPosOffset: int = 0
    sinks: bool = False
    segments: bool = False
    maxSegment: Optional[int] = None
    packed: bool = False
    keyBias: bool = False

    def with_(self, **kw) -> "SdpaCase":
        d = dict(self.__dict__)
        d.update(kw)
        return SdpaCase(**d)


@dataclass
class SdpaInputs:
    case: SdpaCase
    dtype: str
    q: np.ndarray  # f32 [qLen, qHeads*hd], f16-rounded when dtype == 'f16'
    k: np.ndarray
    v: np.ndarray
    sinks: Optional[np.ndarray] = None
    segs: Optional[np.ndarray] = None
    keyBias: Optional[tuple] = None  # (start, end, value)
    packed_qkv: Optional[np.ndarray] = field(default=None)


def random_f32(n: int, seed: int = 1) -> np.ndarray:
    """The reference tests' LCG (packages/runntime/test/gpu.ts:114-123)."""
    out = np.empty(n, dtype=np.float32)
    lib().oracle_random_f32(_p(out), C.c_int64(n), C.c_uint32(seed & 0xFFFFFFFF))
    return out


def round_f16(x: np.ndarray) -> np.ndarray:
    return x.astype(np.float16).astype(np.float32)


def make_inputs(c: SdpaCase, dtype: str = "f32") -> SdpaInputs:
    """Inputs exactly as the reference harness builds them: q = seed 1 scaled
    by 2/sqrt(hd), k = seed 2, v = seed 3, sinks = 2 * seed 4, segments = two
    halves, keyBias = +2 on [kvLen/4, kvLen/2)."""
    rnd = round_f16 if dtype == "f16" else (lambda a: a)
    hd = c.headDim
    scale = np.float64(2.0) / np.sqrt(np.float64(hd))
    q = rnd((random_f32(c.qLen * c.qHeads * hd, 1).astype(np.float64) * scale).astype(np.float32))
    k = rnd(random_f32(c.kvLen * c.kvHeads * hd, 2))
    v = rnd(random_f32(c.kvLen * c.kvHeads * hd, 3))
    q = q.reshape(c.qLen, c.qHeads * hd)
    k = k.reshape(c.kvLen, c.kvHeads * hd)
    v = v.reshape(c.kvLen, c.kvHeads * hd)
    sinks = (2 * random_f32(c.qHeads, 4)).astype(np.float32) if c.sinks else None
    segs = None
    if c.segments:
        segs = np.empty((c.qLen, 2), dtype=np.float32)
        qh, kh = c.qLen // 2, c.kvLen // 2
        segs[:qh, 0], segs[:qh, 1] = 0, kh
        segs[qh:, 0], segs[qh:, 1] = kh, c.kvLen
    kb = (c.kvLen // 4, c.kvLen // 2, 2.0) if c.keyBias else None
    packed = np.ascontiguousarray(np.concatenate([q, k, v], axis=1)) if c.packed else None
    return SdpaInputs(c, dtype, q, k, v, sinks, segs, kb, packed)


def _dims(qLen, kvLen, qHeads, kvHeads, headDim, windowLeft, windowRight, qPosOffset, packed,
          keyBias) -> _Dims:
    d = _Dims()
    d.qLen, d.kvLen = qLen, kvLen
    d.qHeads, d.kvHeads, d.headDim = qHeads, kvHeads, headDim
    d.windowLeft, d.windowRight = _win(windowLeft), _win(windowRight)
    d.qPosOffset = qPosOffset
    d.packed = 1 if packed else 0
    if keyBias is not None:
        d.hasKeyBias, d.biasStart, d.biasEnd, d.biasValue = 1, keyBias[0], keyBias[1], keyBias[2]
    return d


def sdpa_ref(q, k, v, *, qHeads, kvHeads, headDim, windowLeft=math.inf, windowRight=math.inf,
             qPosOffset=0, sinks=None, segs=None, keyBias=None, packed=None) -> np.ndarray:
    """f64 two-pass oracle.  q/k/v are f32 arrays; with ``packed`` (an f32
    [T, (qH+2kvH)*hd] array) they are ignored and read from its column blocks."""
    if packed is not None:
        packed = np.ascontiguousarray(packed, dtype=np.float32)
        qLen = kvLen = packed.shape[0]
        q = k = v = packed
    else:
        q = np.ascontiguousarray(q, dtype=np.float32)
        k = np.ascontiguousarray(k, dtype=np.float32)
        v = np.ascontiguousarray(v, dtype=np.float32)
        qLen, kvLen = q.shape[0], k.shape[0]
    sinks = None if sinks is None else np.ascontiguousarray(sinks, dtype=np.float32)
    segs = None if segs is None else np.ascontiguousarray(segs, dtype=np.float32)
    d = _dims(qLen, kvLen, qHeads, kvHeads, headDim, windowLeft, windowRight, qPosOffset,
              packed is not None, keyBias)
    out = np.empty((qLen, qHeads * headDim), dtype=np.float64)
    lib().oracle_sdpa_f64(_p(q), _p(k), _p(v), _p(sinks), _p(segs), C.byref(d), _p(out))
    return out


def sdpa_ref_inputs(x: SdpaInputs) -> np.ndarray:
    c = x.case
    return sdpa_ref(x.q, x.k, x.v, qHeads=c.qHeads, kvHeads=c.kvHeads, headDim=c.headDim,
                    windowLeft=c.windowLeft, windowRight=c.windowRight, qPosOffset=c.qPosOffset,
                    sinks=x.sinks, segs=x.segs, keyBias=x.keyBias, packed=x.packed_qkv)


def sdpa_rows(q, k, v, *, qHeads, kvHeads, headDim, windowLeft=math.inf, windowRight=math.inf,
              qPosOffset=0, sinks=None, segs=None, keyBias=None, packed=None) -> np.ndarray:
    """Shader-order online softmax in f32 on all host threads; storage dtype
    follows the inputs (float32 or float16).  This is the timed CPU baseline."""
    src = packed if packed is not None else q
    dt = src.dtype
    assert dt in (np.float32, np.float16)
    if packed is not None:
        packed = np.ascontiguousarray(packed)
        qLen = kvLen = packed.shape[0]
        q = k = v = packed
    else:
        q, k, v = (np.ascontiguousarray(a) for a in (q, k, v))
        assert k.dtype == dt and v.dtype == dt
        qLen, kvLen = q.shape[0], k.shape[0]
    sinks = None if sinks is None else np.ascontiguousarray(sinks, dtype=np.float32)
    segs = None if segs is None else np.ascontiguousarray(segs, dtype=np.float32)
    d = _dims(qLen, kvLen, qHeads, kvHeads, headDim, windowLeft, windowRight, qPosOffset,
              packed is not None, keyBias)
    out = np.empty((qLen, qHeads * headDim), dtype=dt)
    fn = lib().oracle_sdpa_rows_f32 if dt == np.float32 else lib().oracle_sdpa_rows_f16
    fn(_p(q), _p(k), _p(v), _p(sinks), _p(segs), C.byref(d), _p(out))
    return out


def write_rows(dst: np.ndarray, src: np.ndarray, startRow: int) -> np.ndarray:
    """In-place append; returns the [startRow+r, cols] view, like writeRows."""
    assert dst.dtype == src.dtype and dst.shape[1] == src.shape[1]
    assert dst.flags.c_contiguous and src.flags.c_contiguous
    assert 0 <= startRow and startRow + src.shape[0] <= dst.shape[0]
    lib().oracle_write_rows(_p(dst), _p(src), C.c_int64(startRow), C.c_int64(src.shape[0]),
                            C.c_int64(src.shape[1]), C.c_int32(dst.itemsize))
    return dst[: startRow + src.shape[0]]


def merge_partials(partials: np.ndarray) -> np.ndarray:
    """partials f32 [parts, units, 2+hd] -> f64 [units, hd]."""
    partials = np.ascontiguousarray(partials, dtype=np.float32)
    parts, units, w = partials.shape
    out = np.empty((units, w - 2), dtype=np.float64)
    lib().oracle_merge_partials(_p(partials), C.c_int32(parts), C.c_int64(units),
                                C.c_int32(w - 2), _p(out))
    return out


def rope_ref(x, cos, sin, *, headDim, srcStart=0, width=None) -> np.ndarray:
    """f64 rotary embedding of a column window of x [rows, cols] (f32 values)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    cos = np.ascontiguousarray(cos, dtype=np.float32)
    sin = np.ascontiguousarray(sin, dtype=np.float32)
    rows, cols = x.shape
    width = cols if width is None else width
    out = np.empty((rows, width), dtype=np.float64)
    lib().oracle_rope_f64(_p(x), _p(cos), _p(sin), C.c_int64(rows), C.c_int64(cols),
                          C.c_int32(headDim), C.c_int64(srcStart), C.c_int64(width), _p(out))
    return out


def local_attention_ref(qkv, rel, qScale, *, heads, headDim, window, kScale=1.0,
                        softcap=50.0) -> np.ndarray:
    """f64 local attention over qkv [rows, 3*heads*headDim] (f32 values)."""
    qkv = np.ascontiguousarray(qkv, dtype=np.float32)
    rel = np.ascontiguousarray(rel, dtype=np.float32)
    qScale = np.ascontiguousarray(qScale, dtype=np.float32)
    rows = qkv.shape[0]
    out = np.empty((rows, heads * headDim), dtype=np.float64)
    lib().oracle_local_attention_f64(_p(qkv), _p(rel), _p(qScale), C.c_int64(rows),
                                     C.c_int32(heads), C.c_int32(headDim), C.c_int32(window),
                                     C.c_double(kScale), C.c_double(softcap), _p(out))
    return out


def softmax_ref(x, segs=None, windowLeft=math.inf, windowRight=math.inf) -> np.ndarray:
    """f64 row softmax of x [rows, cols] (f32 values), masked when ``segs`` is given."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, cols = x.shape
    out = np.empty((rows, cols), dtype=np.float64)
    sp = None
    if segs is not None:
        segs = np.ascontiguousarray(segs, dtype=np.float32)
        sp = _p(segs)
    lib().oracle_softmax_f64(_p(x), sp, C.c_int64(rows), C.c_int64(cols),
                             C.c_int64(_win(windowLeft)), C.c_int64(_win(windowRight)), _p(out))
    return out


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    """Host threads for the parallel loops (a launcher such as torchrun sets
    OMP_NUM_THREADS=1 for its workers; the CPU baseline wants all cores)."""
    lib().oracle_set_num_threads(C.c_int(int(n)))


# Tolerances of the reference's own comparison (checkSdpa.ts:127):
# |got - want| <= atol + rtol * |want|.
TOLERANCE = {"f32": dict(atol=2e-5, rtol=1e-4), "f16": dict(atol=2e-3, rtol=4e-3)}


def assert_close(got, want, dtype: str, what: str = "") -> None:
    got = np.asarray(got, dtype=np.float64).reshape(-1)
    want = np.asarray(want, dtype=np.float64).reshape(-1)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    tol = TOLERANCE[dtype]
    err = np.abs(got - want)
    bad = ~(err <= tol["atol"] + tol["rtol"] * np.abs(want))  # NaN fails
    if bad.any():
        i = int(np.argmax(bad))
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{got.size} elements off; first at {i}: got {got[i]}, "
            f"want {want[i]} (atol {tol['atol']}, rtol {tol['rtol']}); max abs err {np.nanmax(err)}")
