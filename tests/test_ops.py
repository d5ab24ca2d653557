"""The operator boundary: shapes, attrs layout and every refusal of ``sdpa``,
``sdpaPacked`` and ``writeRows``.  The cases and error texts are the ones the
reference pins (packages/runntime/test/core/graph/ops/attention.test.ts:23-231,
packages/runntime/test/core/graph/ops/shape.test.ts:232-280,
packages/runntime/test/core/nn/layers.test.ts:1112-1131)."""
import math
import re

import pytest

from runntime_b200 import MultiHeadAttention, sdpa, sdpaPacked, writeRows
from runntime_b200.value import DeviceBuffer, ValueMeta, materialized, pending

INF = math.inf
QH, KVH, HD = 4, 2, 8
heads = dict(qHeads=QH, kvHeads=KVH, headDim=HD)
causal = dict(heads, windowLeft=INF, windowRight=0)
full = dict(heads, windowLeft=INF, windowRight=INF)


def meta(dims, dtype="f32"):
    n = 1
    for d in dims:
        n *= d
    return ValueMeta(n, dtype, tuple(dims))


def input_(dims, dtype="f32"):
    """A pending value of the given shape (an op input not yet computed)."""
    return pending(meta(dims, dtype), "reshape", [])


def materialized_input(dims, dtype="f32"):
    m = meta(dims, dtype)
    return materialized(m, DeviceBuffer(0xDEAD0000, m.elems * 4, owned=False))


def qkv(qLen, kvLen):
    return input_([qLen, QH * HD]), input_([kvLen, KVH * HD]), input_([kvLen, KVH * HD])


def test_sdpa_gives_one_output_row_per_query_row():
    q, k, v = qkv(5, 7)
    c = sdpa(q, k, v, causal)
    assert c.shape == meta([5, QH * HD])
    assert c.pending.op == "attn"
    assert list(c.pending.attrs[:3]) == [QH, KVH, HD]


def test_unbounded_window_is_a_large_finite_number():
    q, k, v = qkv(5, 7)
    attrs = sdpa(q, k, v, causal).pending.attrs
    assert math.isfinite(attrs[3]) and attrs[3] > 1e9 and attrs[4] == 0


@pytest.mark.parametrize("qLen,kvLen,opts", [
    (1, 7, dict(causal, qPosOffset=6)),
    (5, 3, full),
    (5, 5, dict(heads, windowLeft=2, windowRight=0)),
    (5, 5, dict(causal, kvHeads=1)),
])
def test_sdpa_accepts(qLen, kvLen, opts):
    q = input_([qLen, QH * HD])
    kv = input_([kvLen, opts["kvHeads"] * HD])
    assert sdpa(q, kv, kv, opts).shape == meta([qLen, QH * HD])


def test_sinks_and_segments_are_extra_inputs():
    q, k, v = qkv(5, 5)
    sinks, segments = input_([QH]), input_([5, 2])
    c = sdpa(q, k, v, dict(causal, sinks=sinks, segments=segments, maxSegment=3))
    assert list(c.pending.inputs) == [q, k, v, sinks, segments]
    assert list(c.pending.attrs[6:10]) == [1, 1, 3, 0]


def test_key_bias_is_attrs_not_an_input():
    q, k, v = qkv(5, 7)
    c = sdpa(q, k, v, dict(causal, keyBias=dict(start=2, end=7, value=-1.5)))
    assert list(c.pending.inputs) == [q, k, v]
    assert list(c.pending.attrs[10:]) == [1, 2, 7, -1.5]


@pytest.mark.parametrize("repl,error", [
    (dict(q=[5, 30]), r"q cols 30 != qHeads\*headDim 32"),
    (dict(k=[7, 8]), r"k cols 8 != kvHeads\*headDim 16"),
    (dict(v=[6, 16]), r"v rows 6 != k rows 7"),
    (dict(v=[7, 8]), r"v cols 8 != kvHeads\*headDim 16"),
    (dict(v=([7, 16], "f16")), r"must share a dtype, got f32/f32/f16"),
])
def test_sdpa_rejects_shapes(repl, error):
    base = dict(zip("qkv", qkv(5, 7)))
    for name, spec in repl.items():
        base[name] = input_(*spec) if isinstance(spec, tuple) else input_(spec)
    with pytest.raises(ValueError, match=error):
        sdpa(base["q"], base["k"], base["v"], causal)


@pytest.mark.parametrize("opts,error", [
    (dict(causal, kvHeads=3), r"qHeads 4 not divisible by kvHeads 3"),
    (dict(causal, kvHeads=0), r"not divisible by kvHeads 0"),
    (dict(causal, windowLeft=-1), r"windowLeft -1 must be a non-negative integer"),
    (dict(causal, windowRight=0.5), r"windowRight 0.5 must be"),
    (dict(causal, windowLeft=1.5), r"windowLeft 1.5 must be a non-negative integer or Infinity"),
    (dict(causal, qPosOffset=-1), r"qPosOffset -1 must be a non-negative integer"),
    (dict(causal, qPosOffset=3), r"qPosOffset\+qLen 8 exceeds key rows kvLen 7"),
    (dict(causal, sinks=input_([2])), r"sinks must be f32 with 4 elems"),
    (dict(causal, segments=input_([5])), r"segments must be f32 \[qLen, 2\] = 10 elems"),
    (dict(causal, maxSegment=3), r"maxSegment needs segments"),
    (dict(causal, segments=input_([5, 2]), maxSegment=1.5),
     r"maxSegment 1.5 must be a positive integer"),
    (dict(causal, keyBias=dict(start=3, end=8, value=1)),
     r"keyBias keys \[3, 8\) must lie within the 7 keys"),
    (dict(causal, keyBias=dict(start=4, end=2, value=1)), r"keyBias keys \[4, 2\)"),
    (dict(causal, keyBias=dict(start=0.5, end=2, value=1)), r"keyBias keys \[0.5, 2\)"),
    (dict(causal, keyBias=dict(start=0, end=2, value=math.nan)),
     r"keyBias value NaN must be finite"),
])
def test_sdpa_rejects_options(opts, error):
    q, k, v = qkv(5, 7)
    if opts["kvHeads"] not in (KVH,):
        pass
    with pytest.raises(ValueError, match=error):
        sdpa(q, k, v, opts)


def test_sdpa_rejects_segments_and_key_bias_on_decode():
    q, k, v = qkv(1, 7)
    with pytest.raises(ValueError, match=r"segments need qLen > 1"):
        sdpa(q, k, v, dict(causal, qPosOffset=6, segments=input_([1, 2])))
    with pytest.raises(ValueError, match=r"keyBias needs qLen > 1"):
        sdpa(q, k, v, dict(causal, qPosOffset=6, keyBias=dict(start=0, end=2, value=1)))


def test_head_size_limits():
    x = input_([2, 512])
    assert sdpa(x, x, x, dict(full, qHeads=1, kvHeads=1, headDim=512)).shape == meta([2, 512])
    for qLen, hd, mx in ((1, 160, 128), (2, 640, 512)):
        x = input_([qLen, hd])
        with pytest.raises(ValueError, match=re.escape(f"headDim {hd} exceeds the kernel's max ({mx})")):
            sdpa(x, x, x, dict(full, qHeads=1, kvHeads=1, headDim=hd))


def test_queries_past_keys_under_bounded_right_window():
    q = input_([4, 16])
    kv = input_([3, 8])
    with pytest.raises(ValueError, match=r"qPosOffset\+qLen 4 exceeds key rows kvLen 3"):
        sdpa(q, kv, kv, dict(qHeads=2, kvHeads=1, headDim=8, windowLeft=INF, windowRight=0))


def test_want2d_message():
    with pytest.raises(ValueError, match=r"sdpa: expected a 2D f32 or f16 tensor, got dims=\[5\] dtype=f32"):
        sdpa(input_([5]), input_([5, 16]), input_([5, 16]), causal)


def packed(t):
    return input_([t, (QH + 2 * KVH) * HD])


def test_sdpa_packed_reads_one_tensor():
    c = sdpaPacked(packed(5), causal)
    assert c.shape == meta([5, QH * HD])
    assert c.pending.attrs[-1] == 1 and len(c.pending.attrs) == 10
    assert len(c.pending.inputs) == 1


@pytest.mark.parametrize("x,opts,error", [
    (input_([5, 60]), causal, r"qkv cols 60 != \(qHeads \+ 2\*kvHeads\)\*headDim = 64"),
    (packed(1), causal, r"qLen must be > 1"),
    (packed(5), dict(causal, qPosOffset=1), r"exceeds key rows"),
    (input_([5, 3 * 130]), dict(qHeads=1, kvHeads=1, headDim=130, windowLeft=INF, windowRight=0),
     r"headDim 130 exceeds the kernel's max \(128\)"),
])
def test_sdpa_packed_rejects(x, opts, error):
    with pytest.raises(ValueError, match=error):
        sdpaPacked(x, opts)


def test_sdpa_packed_allows_offset_with_unbounded_right():
    assert sdpaPacked(packed(5), dict(full, qPosOffset=1)).shape == meta([5, QH * HD])


cache = materialized_input([8, 4])


def test_write_rows_returns_view_up_to_last_written_row():
    c = writeRows(cache, input_([2, 4]), 3)
    assert c.shape == meta([5, 4]) and list(c.pending.attrs) == [3]
    assert c.pending.op == "writeRows"
    assert writeRows(cache, input_([2, 4]), 6).shape == meta([8, 4])


@pytest.mark.parametrize("dst,src,start,error", [
    (input_([8, 4]), input_([2, 4]), 0, r"dst must be a materialized"),
    (cache, input_([2, 4]), 7, r"rows \[7, 9\) exceed dst capacity 8"),
    (cache, input_([2, 4]), -1, r"exceed dst capacity"),
    (cache, input_([2, 5]), 0, r"col mismatch"),
    (cache, input_([2, 4], "f16"), 0, r"dtype mismatch"),
])
def test_write_rows_rejects(dst, src, start, error):
    with pytest.raises(ValueError, match=error):
        writeRows(dst, src, start)


def test_multi_head_attention_module():
    mha = MultiHeadAttention(dict(causal, sinks=True))
    assert list(mha.parameters()) == ["sinks"]
    assert mha.sinks.shape == ValueMeta(QH, "f32", (QH,)) and mha.sinks.pinned
    with pytest.raises(RuntimeError):
        mha.forward(*qkv(5, 5))
    mha.sinks.set(input_([QH]))
    q, k, v = qkv(5, 7)
    c = mha.forward(q, k, v, dict(qPosOffset=2))
    assert c.pending.attrs[5] == 2 and c.pending.attrs[6] == 1
    assert MultiHeadAttention(causal).parameters() == {}
    c = MultiHeadAttention(causal).forwardPacked(packed(5))
    assert c.pending.attrs[9] == 1


# ---- rope (packages/runntime/test/core/graph/ops/attention.test.ts:232-283) ----

from runntime_b200 import rope  # noqa: E402


def _tables(t, headDim=HD):
    return input_([t, headDim]), input_([t, headDim])


def test_rope_rotates_every_head_or_a_slice():
    cos, sin = _tables(5)
    c = rope(input_([5, 32], "f16"), cos, sin, dict(headDim=HD))
    assert c.shape == meta([5, 32], "f16") and list(c.pending.attrs) == [HD, 0, 32]
    assert c.pending.op == "rope"
    c = rope(input_([5, 64]), cos, sin, dict(headDim=HD, srcStart=32, width=16))
    assert c.shape == meta([5, 16]) and list(c.pending.attrs) == [HD, 32, 16]


@pytest.mark.parametrize("opts,error", [
    (dict(headDim=7), r"headDim 7 must be a positive even integer"),
    (dict(headDim=HD, srcStart=3, width=8), r"srcStart 3 must be a non-negative even integer"),
    (dict(headDim=HD, srcStart=24, width=16), r"window \[24, 40\) exceeds 32 input cols"),
    (dict(headDim=HD, width=12), r"width 12 must be a multiple of headDim 8"),
])
def test_rope_rejects_options(opts, error):
    cos, sin = _tables(5)
    with pytest.raises(ValueError, match=error):
        rope(input_([5, 32]), cos, sin, opts)


def test_rope_rejects_tables():
    with pytest.raises(ValueError, match=r"cos must be f32 \[T,headDim\] = 40 elems, got 32"):
        rope(input_([5, 32]), input_([4, HD]), input_([5, HD]), dict(headDim=HD))
    with pytest.raises(ValueError, match=r"cos must be f32"):
        rope(input_([5, 32]), input_([5, HD], "f16"), input_([5, HD]), dict(headDim=HD))


# ---- slice / chunk (packages/runntime/src/core/graph/ops/shape.ts:69-135) --------

from runntime_b200 import chunk, slice as slice_  # noqa: E402


def test_slice_columns_and_rows():
    c = slice_(input_([3, 24], "f16"), 1, 16, 24)
    assert c.shape == meta([3, 8], "f16") and c.pending.op == "sliceCols"
    assert list(c.pending.attrs) == [16, 24]
    r = slice_(input_([6, 4]), 0, 2, 5)
    assert r.shape == meta([3, 4]) and r.pending.op == "sliceRows"
    assert slice_(input_([6, 4]), -1, 0, 2).pending.op == "sliceCols"


def test_slice_rejects_bad_ranges():
    with pytest.raises(ValueError, match=r"slice: bad range \[4, 4\) for 8 cols"):
        slice_(input_([2, 8]), 1, 4, 4)
    with pytest.raises(ValueError, match=r"slice: bad range \[0, 9\) for 8 cols"):
        slice_(input_([2, 8]), 1, 0, 9)
    with pytest.raises(ValueError, match=r"slice: bad range \[-1, 1\) for 2 rows"):
        slice_(input_([2, 8]), 0, -1, 1)
    with pytest.raises(ValueError, match=r"slice: dim 2 out of range for a rank-2 operand"):
        slice_(input_([2, 8]), 2, 0, 1)


def test_chunk_splits_k_and_v_of_a_fused_projection():
    k, v = chunk(input_([200, 576], "f16"), 2, 1)
    assert k.shape == meta([200, 288], "f16") and list(v.pending.attrs) == [288, 576]
    with pytest.raises(ValueError, match=r"chunk: dim 1 size 576 does not divide into 5 equal parts"):
        chunk(input_([200, 576]), 5, 1)
    with pytest.raises(ValueError, match=r"chunk: n must be a positive integer, got 0"):
        chunk(input_([200, 576]), 0, 1)


# ---- softmax (packages/runntime/test/core/graph/ops/reduce.test.ts:17-78) ----------

from runntime_b200 import softmax  # noqa: E402


def test_softmax_keeps_the_shape_and_runs_unmasked_without_segments():
    c = softmax(input_([4, 8], "f16"))
    assert c.shape == meta([4, 8], "f16") and list(c.pending.attrs) == [0, 0, 0]
    with pytest.raises(ValueError, match=r"expected a 2D"):
        softmax(input_([8]))


def test_masked_softmax_takes_segments_as_a_second_input():
    x, segments = input_([5, 5]), input_([5, 2])
    c = softmax(x, dict(segments=segments, windowLeft=2, windowRight=0))
    assert c.shape == meta([5, 5]) and list(c.pending.inputs) == [x, segments]
    assert list(c.pending.attrs) == [1, 2, 0]
    _, left, right = softmax(x, dict(segments=segments)).pending.attrs
    assert math.isfinite(left) and left > 1e9 and right == left


@pytest.mark.parametrize("x,segments,opts,error", [
    ([4, 8], ([4, 2], "f32"), {}, r"needs square scores, got \[4, 8\]"),
    ([5, 5], ([5], "f32"), {}, r"segments must be f32 \[5, 2\]"),
    ([5, 5], ([5, 2], "f16"), {}, r"segments must be f32"),
    ([5, 5], ([5, 2], "f32"), dict(windowLeft=-1),
     r"windowLeft must be a non-negative integer or Infinity, got -1"),
    ([5, 5], ([5, 2], "f32"), dict(windowRight=0.5),
     r"windowRight must be a non-negative integer or Infinity, got 0.5"),
])
def test_masked_softmax_rejects(x, segments, opts, error):
    with pytest.raises(ValueError, match=error):
        softmax(input_(x), dict(segments=input_(*segments), **opts))


# ---- localAttention (packages/runntime/test/core/graph/ops/attention.test.ts:291-332) ----

from runntime_b200 import localAttention  # noqa: E402

LOCAL = dict(heads=2, headDim=HD, window=3, kScale=1, softcap=50)


def test_local_attention_gives_one_row_of_heads_times_head_dim():
    c = localAttention(input_([5, 48]), input_([3, 16]), input_([HD]), LOCAL)
    assert c.shape == meta([5, 16]) and c.pending.op == "localAttention"
    assert list(c.pending.attrs) == [2, HD, 3, 1, 50]


@pytest.mark.parametrize("over,error", [
    (dict(qkv=([5, 40],)), r"48 cols, got 40"),
    (dict(rel=([4, 16],)), r"rel must be f32 \[3, 16\]"),
    (dict(rel=([3, 16], "f16")), r"rel must be f32"),
    (dict(qScale=([4],)), r"qScale must be f32 \[8\]"),
    (dict(opts=dict(window=33)), r"window 33 must be an integer from 1 to 32"),
    (dict(opts=dict(headDim=6)), r"headDim 6 a multiple of 4"),
    (dict(opts=dict(softcap=0)), r"softcap must be positive"),
])
def test_local_attention_rejects(over, error):
    qkv = input_(*over.get("qkv", ([5, 48],)))
    rel = input_(*over.get("rel", ([3, 16],)))
    qScale = input_(*over.get("qScale", ([HD],)))
    with pytest.raises(ValueError, match=error):
        localAttention(qkv, rel, qScale, dict(LOCAL, **over.get("opts", {})))


# ---- matmul / argmaxDot (packages/runntime/test/core/graph/ops/matmul.test.ts) -------

from runntime_b200 import ACT_CODE, argmaxDot, matmul  # noqa: E402


@pytest.mark.parametrize("a,b,out", [([2, 3], [3, 5], [2, 5]), ([1, 288], [288, 864], [1, 864]),
                                     ([4, 3], [3, 1], [4, 1]), ([1, 1], [1, 1], [1, 1])])
def test_matmul_shapes(a, b, out):
    c = matmul(input_(a), input_(b))
    assert c.shape == meta(out) and c.pending.op == "matmul"
    assert matmul(input_([2, 3], "f16"), input_([3, 5], "f16")).shape == meta([2, 5], "f16")


def test_matmul_epilogue_inputs_and_attrs():
    a, b, bias, addend = input_([2, 3]), input_([3, 5]), input_([5]), input_([2, 5])
    c = matmul(a, b, dict(bias=bias, addend=addend, activation="gelu"))
    assert list(c.pending.inputs) == [a, b, bias, addend]
    assert list(c.pending.attrs) == [1, 1, ACT_CODE["gelu"], 0, 0]   # hasBias, hasAddend, act, baseRow, hasBaseRow
    assert list(matmul(a, b, dict(activation="geluTanh")).pending.attrs) == [0, 0, 5, 0, 0]
    assert list(matmul(a, input_([9, 5]), dict(baseRow=6)).pending.attrs) == [0, 0, 0, 6, 1]


@pytest.mark.parametrize("a,b,opts,error", [
    ([2, 3], ([4, 5],), {}, r"inner dims disagree — a=\[2,3\] b=\[4,5\]"),
    ([6], ([6, 2],), {}, r"must be 2D"),
    ([2, 3], ([3, 5], "f16"), {}, r"must be f32 or both f16, got f32 and f16"),
    ([2, 3], ([3, 5],), dict(bias=([3],)), r"bias must be f32 \[N\] = 5 elems"),
    ([2, 3], ([3, 5],), dict(bias=([5], "f16")), r"bias must be f32"),
    ([2, 3], ([3, 5],), dict(addend=([5],)), r"addend must be f32 \[M,N\] = 10 elems"),
    ([2, 3], ([9, 5],), dict(baseRow=7), r"bad baseRow 7"),
])
def test_matmul_rejects(a, b, opts, error):
    o = {k: (input_(*v) if isinstance(v, tuple) else v) for k, v in opts.items()}
    with pytest.raises(ValueError, match=error):
        matmul(input_(a), input_(*b), o)


def test_argmax_dot_gives_one_f32_index():
    assert argmaxDot(input_([50000, 16], "f16"), input_([1, 16], "f16")).shape == meta([1, 1])
    for x, error in ((input_([2, 16]), r"must be a single row, got 2"),
                     (input_([1, 8]), r"x cols 8 != w cols 16"),
                     (input_([1, 16], "f16"), r"must match x's f16")):
        with pytest.raises(ValueError, match=error):
            argmaxDot(input_([100, 16]), x)
