"""Operator constructors of the attention path: ``sdpa``, ``sdpaPacked``, ``rope`` and
``writeRows`` with the reference's names, option names, defaults, synchronous
validation and error texts
(packages/runntime/src/core/graph/ops/attention.ts:28-212,
packages/runntime/src/core/graph/ops/shape.ts:236-259).  They only build a
pending node; ``evalValues``/``toArray`` run it on the GPU."""
from __future__ import annotations

import json
import math
from typing import Optional, Sequence

from ._lib import WINDOW_INF
from .value import Value, ValueMeta, pending

FLOAT_DTYPES = ("f32", "f16")
MAX_HEAD_DIM = 512          # widest head with more than one query row
MAX_DECODE_HEAD_DIM = 128   # widest head with one query row


def _js(x) -> str:
    """A number as JavaScript's template literals print it."""
    if isinstance(x, bool):
        return "true" if x else "false"
    if isinstance(x, float):
        if math.isinf(x):
            return "Infinity" if x > 0 else "-Infinity"
        if math.isnan(x):
            return "NaN"
        if x.is_integer():
            return str(int(x))
        return repr(x)
    return str(x)


def _is_int(x) -> bool:
    if isinstance(x, bool):
        return False
    if isinstance(x, int):
        return True
    return isinstance(x, float) and math.isfinite(x) and x.is_integer()


def want2d(name: str, x: Value, allow: Sequence[str]):
    """[rows, cols, dtype] of a 2-D row-major tensor whose dtype is allowed
    (packages/runntime/src/core/graph/ops/shared.ts:46-75)."""
    dims, dtype = x.shape.dims, x.shape.dtype
    if dims is None or len(dims) != 2 or dtype not in allow:
        got = "undefined" if dims is None else json.dumps(list(dims), separators=(",", ":"))
        raise ValueError(
            f"{name}: expected a 2D {' or '.join(allow)} tensor, got dims={got} dtype={dtype}")
    return dims[0], dims[1], dtype


def _lower_window(op: str, name: str, w) -> int:
    if w == math.inf:
        return WINDOW_INF
    if not _is_int(w) or w < 0:
        raise ValueError(f"{op}: {name} {_js(w)} must be a non-negative integer or Infinity")
    return min(int(w), WINDOW_INF)


def sdpa(q: Value, k: Value, v: Value, opts: dict) -> Value:
    """The reference's ``sdpa`` (packages/runntime/src/core/graph/ops/attention.ts:28-141):
    checks the arguments now, with the reference's messages, and returns a pending
    'attn' node whose attrs vector has the reference's layout; nothing runs until the
    value is evaluated.

    What the node computes, for ``q [qLen, qHeads*headDim]`` against
    ``k, v [kvLen, kvHeads*headDim]``: every query head attends to the kv head of its group
    (grouped-query attention); row i stands at position ``qPosOffset + i`` and sees the
    keys from ``windowLeft`` before that position to ``windowRight`` after it (``math.inf``
    = no limit on that side); with ``segments`` a row is further confined to its own
    ``[start, end)`` of keys; ``keyBias`` raises the scores of one key range by a constant;
    ``sinks`` gives every head an extra term in the softmax denominator.  Scores are used
    as they come: callers fold 1/sqrt(headDim) into q or k."""
    qHeads, kvHeads, headDim = opts["qHeads"], opts["kvHeads"], opts["headDim"]
    sinks: Optional[Value] = opts.get("sinks")
    segments: Optional[Value] = opts.get("segments")
    keyBias = opts.get("keyBias")
    qPosOffset = opts.get("qPosOffset")
    qPosOffset = 0 if qPosOffset is None else qPosOffset
    qLen, qw, dtype = want2d("sdpa", q, FLOAT_DTYPES)
    if qw != qHeads * headDim:
        raise ValueError(f"sdpa: q cols {qw} != qHeads*headDim {qHeads * headDim}")
    if kvHeads <= 0 or qHeads % kvHeads != 0:
        raise ValueError(f"sdpa: qHeads {qHeads} not divisible by kvHeads {kvHeads}")
    maxHeadDim = MAX_DECODE_HEAD_DIM if qLen == 1 else MAX_HEAD_DIM
    if headDim > maxHeadDim:
        raise ValueError(f"sdpa: headDim {headDim} exceeds the kernel's max ({maxHeadDim})")
    wl = _lower_window("sdpa", "windowLeft", opts["windowLeft"])
    wr = _lower_window("sdpa", "windowRight", opts["windowRight"])
    if not _is_int(qPosOffset) or qPosOffset < 0:
        raise ValueError(f"sdpa: qPosOffset {_js(qPosOffset)} must be a non-negative integer")
    qPosOffset = int(qPosOffset)
    kvw = kvHeads * headDim
    kvLen, kw, kDtype = want2d("sdpa.k", k, FLOAT_DTYPES)
    if kw != kvw:
        raise ValueError(f"sdpa: k cols {kw} != kvHeads*headDim {kvw}")
    vt, vw, vDtype = want2d("sdpa.v", v, FLOAT_DTYPES)
    if kDtype != dtype or vDtype != dtype:
        raise ValueError(f"sdpa: q, k and v must share a dtype, got {dtype}/{kDtype}/{vDtype}")
    if vt != kvLen:
        raise ValueError(f"sdpa: v rows {vt} != k rows {kvLen}")
    if vw != kvw:
        raise ValueError(f"sdpa: v cols {vw} != kvHeads*headDim {kvw}")
    if wr != WINDOW_INF and qPosOffset + qLen > kvLen:
        raise ValueError(
            f"sdpa: qPosOffset+qLen {qPosOffset + qLen} exceeds key rows kvLen {kvLen}")
    if sinks is not None and (sinks.shape.dtype != "f32" or sinks.shape.elems != qHeads):
        raise ValueError(f"sdpa: sinks must be f32 with {qHeads} elems, got {sinks.shape.elems}")
    if segments is not None:
        if segments.shape.dtype != "f32" or segments.shape.elems != 2 * qLen:
            raise ValueError(
                f"sdpa: segments must be f32 [qLen, 2] = {2 * qLen} elems, got "
                f"({segments.shape.elems},{segments.shape.dtype})")
        if qLen == 1:
            raise ValueError("sdpa: segments need qLen > 1 (decode has no segment route)")
    maxSegment = opts.get("maxSegment")
    maxSegment = 0 if maxSegment is None else maxSegment
    if maxSegment != 0:
        if segments is None:
            raise ValueError("sdpa: maxSegment needs segments")
        if not _is_int(maxSegment) or maxSegment < 1:
            raise ValueError(f"sdpa: maxSegment {_js(maxSegment)} must be a positive integer")
    bias_attrs = []
    if keyBias:
        start, end, value = keyBias["start"], keyBias["end"], keyBias["value"]
        if (not _is_int(start) or not _is_int(end) or start < 0 or start > end or end > kvLen):
            raise ValueError(
                f"sdpa: keyBias keys [{_js(start)}, {_js(end)}) must lie within the {kvLen} keys")
        if not math.isfinite(value):
            raise ValueError(f"sdpa: keyBias value {_js(value)} must be finite")
        if qLen == 1:
            raise ValueError("sdpa: keyBias needs qLen > 1 (decode has no key bias route)")
        bias_attrs = [1, int(start), int(end), value]
    inputs = [q, k, v] + ([sinks] if sinks is not None else []) + (
        [segments] if segments is not None else [])
    attrs = [qHeads, kvHeads, headDim, wl, wr, qPosOffset, 1 if sinks is not None else 0,
             1 if segments is not None else 0, int(maxSegment), 0, *bias_attrs]
    return pending(ValueMeta(qLen * qw, dtype, (qLen, qw)), "attn", inputs, None, attrs)


def sdpaPacked(qkv: Value, opts: dict) -> Value:
    """The reference's ``sdpaPacked`` (ops/attention.ts:146-212): self-attention whose
    q, k and v are the three column blocks of ONE tensor ``qkv [T, (qHeads +
    2*kvHeads)*headDim]`` — the fused projection's output is attended to where it lies, no
    slicing.  More than one row, heads up to 128 wide, no key bias; otherwise ``sdpa``."""
    qHeads, kvHeads, headDim = opts["qHeads"], opts["kvHeads"], opts["headDim"]
    sinks: Optional[Value] = opts.get("sinks")
    segments: Optional[Value] = opts.get("segments")
    qPosOffset = opts.get("qPosOffset")
    qPosOffset = 0 if qPosOffset is None else qPosOffset
    t, w, dtype = want2d("sdpaPacked", qkv, FLOAT_DTYPES)
    qw = qHeads * headDim
    packedW = (qHeads + 2 * kvHeads) * headDim
    if w != packedW:
        raise ValueError(f"sdpaPacked: qkv cols {w} != (qHeads + 2*kvHeads)*headDim = {packedW}")
    if kvHeads <= 0 or qHeads % kvHeads != 0:
        raise ValueError(f"sdpaPacked: qHeads {qHeads} not divisible by kvHeads {kvHeads}")
    if headDim > 128:
        raise ValueError(f"sdpaPacked: headDim {headDim} exceeds the kernel's max (128)")
    if t == 1:
        raise ValueError("sdpaPacked: qLen must be > 1 (decode has no packed route)")
    wl = _lower_window("sdpaPacked", "windowLeft", opts["windowLeft"])
    wr = _lower_window("sdpaPacked", "windowRight", opts["windowRight"])
    if not _is_int(qPosOffset) or qPosOffset < 0:
        raise ValueError(f"sdpaPacked: qPosOffset {_js(qPosOffset)} must be a non-negative integer")
    qPosOffset = int(qPosOffset)
    if wr != WINDOW_INF and qPosOffset + t > t:
        raise ValueError(f"sdpaPacked: qPosOffset+qLen {qPosOffset + t} exceeds key rows kvLen {t}")
    if sinks is not None and (sinks.shape.dtype != "f32" or sinks.shape.elems != qHeads):
        raise ValueError(
            f"sdpaPacked: sinks must be f32 with {qHeads} elems, got {sinks.shape.elems}")
    if segments is not None and (segments.shape.dtype != "f32" or segments.shape.elems != 2 * t):
        raise ValueError(
            f"sdpaPacked: segments must be f32 [qLen, 2] = {2 * t} elems, got "
            f"({segments.shape.elems},{segments.shape.dtype})")
    maxSegment = opts.get("maxSegment")
    maxSegment = 0 if maxSegment is None else maxSegment
    if maxSegment != 0:
        if segments is None:
            raise ValueError("sdpaPacked: maxSegment needs segments")
        if not _is_int(maxSegment) or maxSegment < 1:
            raise ValueError(f"sdpaPacked: maxSegment {_js(maxSegment)} must be a positive integer")
    inputs = [qkv] + ([sinks] if sinks is not None else []) + (
        [segments] if segments is not None else [])
    attrs = [qHeads, kvHeads, headDim, wl, wr, qPosOffset, 1 if sinks is not None else 0,
             1 if segments is not None else 0, int(maxSegment), 1]
    return pending(ValueMeta(t * qw, dtype, (t, qw)), "attn", inputs, None, attrs)


def rope(x: Value, cos: Value, sin: Value, opts: dict) -> Value:
    """The reference's ``rope`` (ops/attention.ts:214-252): rotates each adjacent
    pair of columns (2i, 2i+1) of every head of ``x [T, W]`` by the row's angle, taken
    from f32 tables ``cos, sin [T, headDim]`` that hold each pair's value twice and may
    carry a scale.  ``srcStart``/``width`` pick a column window of a wider row — the q
    or the k part of a fused qkv projection — so that no slice is needed first."""
    headDim = opts["headDim"]
    t, xw, dtype = want2d("rope", x, FLOAT_DTYPES)
    srcStart = opts.get("srcStart")
    srcStart = 0 if srcStart is None else srcStart
    w = opts.get("width")
    w = xw if w is None else w
    if not _is_int(headDim) or headDim <= 0 or headDim % 2 != 0:
        raise ValueError(f"rope: headDim {_js(headDim)} must be a positive even integer")
    if not _is_int(srcStart) or srcStart < 0 or srcStart % 2 != 0:
        raise ValueError(f"rope: srcStart {_js(srcStart)} must be a non-negative even integer")
    if not _is_int(w) or w <= 0 or srcStart + w > xw:
        raise ValueError(
            f"rope: window [{_js(srcStart)}, {_js(srcStart + w)}) exceeds {xw} input cols")
    if w % headDim != 0:
        raise ValueError(f"rope: width {_js(w)} must be a multiple of headDim {headDim}")
    for name, v in (("cos", cos), ("sin", sin)):
        if v.shape.dtype != "f32" or v.shape.elems != t * headDim:
            raise ValueError(
                f"rope: {name} must be f32 [T,headDim] = {t * headDim} elems, got {v.shape.elems}")
    return pending(ValueMeta(t * int(w), dtype, (t, int(w))), "rope", [x, cos, sin], None,
                   [int(headDim), int(srcStart), int(w)])


ACT_CODE = {"none": 0, "tanh": 1, "gelu": 2, "silu": 3, "relu": 4, "geluTanh": 5, "elu": 6}


def matmul(a: Value, b: Value, opts: Optional[dict] = None) -> Value:
    """2D matrix multiply, a [M,K] x b [K,N] to [M,N], with the fused bias,
    activation and addend epilogue: act(a·b + bias) + addend.  ``baseRow`` views K
    rows of a taller fused b.  Plain f32/f16 weights only (quantized weights are
    not built).  packages/runntime/src/core/graph/ops/matmul.ts:28-99."""
    opts = opts or {}
    if any(opts.get(k) for k in ("scales", "bits", "groupSize")) or b.shape.dtype == "quantW":
        raise ValueError("matmul: quantW weights are not supported by this build")
    ad, bd = a.shape.dims, b.shape.dims
    if ad is None or len(ad) != 2 or bd is None or len(bd) != 2:
        raise ValueError("matmul: both inputs must be 2D matrices (use matrix())")
    if a.shape.dtype != b.shape.dtype or a.shape.dtype not in FLOAT_DTYPES:
        raise ValueError("matmul: both inputs must be f32 or both f16, got "
                         f"{a.shape.dtype} and {b.shape.dtype}")
    dtype = a.shape.dtype
    m, k = ad
    rows, n = bd
    baseRow = opts.get("baseRow")
    base = 0 if baseRow is None else baseRow
    if not _is_int(base) or base < 0 or base + k > rows:
        raise ValueError(f"matmul: bad baseRow {_js(base)} — need integer >= 0 with baseRow+K "
                         f"({k}) <= rows ({rows})")
    if baseRow is None and k != rows:
        raise ValueError(f"matmul: inner dims disagree — a=[{m},{k}] b=[{rows},{n}]")
    bias, addend = opts.get("bias"), opts.get("addend")
    if bias is not None and (bias.shape.dtype != dtype or bias.shape.elems != n):
        raise ValueError(f"matmul: bias must be {dtype} [N] = {n} elems, got "
                         f"({bias.shape.elems},{bias.shape.dtype})")
    if addend is not None and (addend.shape.dtype != dtype or addend.shape.elems != m * n):
        raise ValueError(f"matmul: addend must be {dtype} [M,N] = {m * n} elems, got "
                         f"({addend.shape.elems},{addend.shape.dtype})")
    act = opts.get("activation")
    if act is not None and act not in ACT_CODE:
        raise ValueError(f"matmul: unknown activation {act}")
    inputs = [a, b] + ([bias] if bias is not None else []) + ([addend] if addend is not None else [])
    return pending(ValueMeta(m * n, dtype, (m, n)), "matmul", inputs, None,
                   [1 if bias is not None else 0, 1 if addend is not None else 0,
                    ACT_CODE[act] if act else 0, int(base), 0 if baseRow is None else 1])


def argmaxDot(w: Value, x: Value) -> Value:
    """Fused gemv and argmax for greedy decoding: w [V,N] · x [1,N] to the argmax
    row index, lowest on ties; always f32
    (packages/runntime/src/core/graph/ops/matmul.ts:316-333)."""
    _, n, wDtype = want2d("argmaxDot.w", w, FLOAT_DTYPES)
    xr, xn, xDtype = want2d("argmaxDot.x", x, FLOAT_DTYPES)
    if xr != 1:
        raise ValueError(f"argmaxDot: x must be a single row, got {xr}")
    if xn != n:
        raise ValueError(f"argmaxDot: x cols {xn} != w cols {n}")
    if wDtype != xDtype:
        raise ValueError(f"argmaxDot: w dtype {wDtype} must match x's {xDtype}")
    return pending(ValueMeta(1, "f32", (1, 1)), "argmaxDot", [w, x])


ATTN_LOCAL_MAX_WINDOW = 32  # most keys a query of localAttention sees


def localAttention(qkv: Value, rel: Value, qScale: Value, opts: dict) -> Value:
    """Local attention over a fused qkv slab [T, 3*heads*headDim]: row t sees keys
    t - window + 1 .. t.  The score of the key j rows back is
    cap * tanh((q * qScale) . (k * kScale + rel[j]) / cap), with rel
    [window, heads*headDim] one f32 bias row per distance and qScale [headDim]
    f32 per column of q.  Returns [T, heads*headDim]
    (packages/runntime/src/core/graph/ops/attention.ts:255-300)."""
    heads, headDim, window = opts["heads"], opts["headDim"], opts["window"]
    kScale, softcap = opts["kScale"], opts["softcap"]
    t, w, dtype = want2d("localAttention", qkv, FLOAT_DTYPES)
    if not _is_int(heads) or heads < 1 or not _is_int(headDim) or headDim % 4 != 0:
        raise ValueError(f"localAttention: heads {_js(heads)} must be a positive integer and "
                         f"headDim {_js(headDim)} a multiple of 4")
    heads, headDim = int(heads), int(headDim)
    width = heads * headDim
    if w != 3 * width:
        raise ValueError(
            f"localAttention: qkv must have 3·heads·headDim = {3 * width} cols, got {w}")
    if not _is_int(window) or window < 1 or window > ATTN_LOCAL_MAX_WINDOW:
        raise ValueError(f"localAttention: window {_js(window)} must be an integer from 1 to "
                         f"{ATTN_LOCAL_MAX_WINDOW}")
    window = int(window)
    if rel.shape.dtype != "f32" or rel.shape.elems != window * width:
        raise ValueError(f"localAttention: rel must be f32 [{window}, {width}]")
    if qScale.shape.dtype != "f32" or qScale.shape.elems != headDim:
        raise ValueError(f"localAttention: qScale must be f32 [{headDim}]")
    if not (softcap > 0) or not math.isfinite(kScale):
        raise ValueError("localAttention: softcap must be positive and kScale finite, got "
                         f"{_js(softcap)}, {_js(kScale)}")
    return pending(ValueMeta(t * width, dtype, (t, width)), "localAttention", [qkv, rel, qScale],
                   None, [heads, headDim, window, kScale, softcap])


def softmax(x: Value, opts: Optional[dict] = None) -> Value:
    """Row-wise softmax over the last dim.  With ``segments`` ([M, 2] f32, a
    [start, end) range per row) x is MxM attention scores: row r keeps the keys in
    its range and window, r included, and the rest come out 0.  Windows default to
    Infinity (packages/runntime/src/core/graph/ops/reduce.ts:12-39)."""
    opts = opts or {}
    m, n, dtype = want2d("softmax", x, FLOAT_DTYPES)
    shape = ValueMeta(m * n, dtype, (m, n))
    segments = opts.get("segments")
    if segments is None:
        return pending(shape, "softmax", [x], None, [0, 0, 0])
    if m != n:
        raise ValueError(f"softmax: a masked softmax needs square scores, got [{m}, {n}]")
    if segments.shape.dtype != "f32" or segments.shape.elems != 2 * m:
        raise ValueError(f"softmax: segments must be f32 [{m}, 2]")

    def lower(name: str, w) -> int:
        w = math.inf if w is None else w
        if w == math.inf:
            return WINDOW_INF
        if not _is_int(w) or w < 0:
            raise ValueError(
                f"softmax: {name} must be a non-negative integer or Infinity, got {_js(w)}")
        return min(int(w), WINDOW_INF)

    wl = lower("windowLeft", opts.get("windowLeft"))
    wr = lower("windowRight", opts.get("windowRight"))
    return pending(shape, "softmax", [x, segments], None, [1, wl, wr])


def _norm_dim(op: str, dim, rank: int) -> int:
    """packages/runntime/src/core/graph/ops/shared.ts:102-109."""
    if not _is_int(dim):
        raise ValueError(f"{op}: dim must be an integer, got {_js(dim)}")
    d = int(dim) + rank if dim < 0 else int(dim)
    if d < 0 or d >= rank:
        raise ValueError(f"{op}: dim {_js(dim)} out of range for a rank-{rank} operand")
    return d


def slice(x: Value, dim, start, end) -> Value:  # noqa: A001 - the reference's name
    """Narrows a 2-D x to [start, end) along dim, like torch's narrow: how v is
    cut out of a fused qkv row and k | v out of the fused cross projection
    (packages/runntime/src/core/graph/ops/shape.ts:69-135)."""
    dims = x.shape.dims
    if dims is None or len(dims) != 2:
        got = "undefined" if dims is None else ",".join(str(d) for d in dims)
        raise ValueError(f"slice: needs a 2D or 3D operand, got dims {got}")
    d = _norm_dim("slice", dim, 2)
    m, n, dtype = want2d("slice", x, FLOAT_DTYPES)
    size, what = (m, "rows") if d == 0 else (n, "cols")
    if not _is_int(start) or not _is_int(end) or start < 0 or end > size or start >= end:
        raise ValueError(f"slice: bad range [{_js(start)}, {_js(end)}) for {size} {what}")
    start, end = int(start), int(end)
    if d == 0:
        return pending(ValueMeta((end - start) * n, dtype, (end - start, n)), "sliceRows", [x],
                       None, [start, end])
    return pending(ValueMeta(m * (end - start), dtype, (m, end - start)), "sliceCols", [x], None,
                   [start, end])


def chunk(x: Value, n, dim) -> list:
    """Splits x into n equal parts along dim, like torch.chunk; exact division only
    (packages/runntime/src/core/graph/ops/shape.ts:83-96)."""
    rank = len(x.shape.dims) if x.shape.dims is not None else 0
    d = _norm_dim("chunk", dim, rank)
    size = x.shape.dims[d]
    if not _is_int(n) or n < 1:
        raise ValueError(f"chunk: n must be a positive integer, got {_js(n)}")
    if size % n != 0:
        raise ValueError(f"chunk: dim {_js(dim)} size {size} does not divide into {_js(n)} equal parts")
    step = size // int(n)
    return [slice(x, d, i * step, (i + 1) * step) for i in range(int(n))]


def writeRows(dst: Value, src: Value, startRow) -> Value:
    """In-place row write: copies src into rows [startRow, startRow + r) of the
    caller-owned buffer behind dst and returns a [startRow + r, cols] view of
    that same buffer.  Built for KV-cache appends: rows past the view keep
    whatever they held."""
    dstRows, dstCols, dtype = want2d("writeRows.dst", dst, FLOAT_DTYPES)
    srcRows, srcCols, srcDtype = want2d("writeRows.src", src, FLOAT_DTYPES)
    if srcDtype != dtype:
        raise ValueError(f"writeRows: dtype mismatch — dst is {dtype}, src is {srcDtype}")
    if dst.state != "materialized":
        raise ValueError("writeRows: dst must be a materialized (caller-owned) buffer")
    if srcCols != dstCols:
        raise ValueError(f"writeRows: col mismatch — dst has {dstCols}, src has {srcCols}")
    if not _is_int(startRow) or startRow < 0 or startRow + srcRows > dstRows:
        end = startRow + srcRows if isinstance(startRow, (int, float)) else "NaN"
        raise ValueError(
            f"writeRows: rows [{_js(startRow)}, {_js(end)}) exceed dst capacity {dstRows}")
    viewRows = int(startRow) + srcRows
    return pending(ValueMeta(viewRows * dstCols, dtype, (viewRows, dstCols)), "writeRows",
                   [dst, src], None, [int(startRow)])
