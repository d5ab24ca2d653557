"""The eval driver against a recording fake backend (no GPU): dispatch order,
buffer lifetime, the in-place rule for writeRows and the append+attend fusion.
Mirrors the reference's fake-executor suite
(packages/runntime/test/core/graph/evalCore.test.ts:7-56,115-133)."""
import math

import pytest

from runntime_b200 import sdpa, writeRows
from runntime_b200.executor import _fusable_appends, evalValues
from runntime_b200.value import DeviceBuffer, ValueMeta, materialized

INF = math.inf


def mat(rows, cols, dtype="f32", name="buf"):
    m = ValueMeta(rows * cols, dtype, (rows, cols))
    b = DeviceBuffer(0x1000, m.elems * 4, owned=False)
    return materialized(m, b)


class Recorder:
    def __init__(self, names):
        self.node_name = {id(v): n for n, v in names.items()}
        self.buf_name = {id(v.buffer): n for n, v in names.items() if v.state == "materialized"}
        self.log, self.held, self.released, self.n = [], set(), set(), 0

    def acquireOutput(self, shape):
        b = DeviceBuffer(0, 0, owned=True)
        self.buf_name[id(b)] = f"#{self.n}"
        self.n += 1
        self.held.add(id(b))
        return b

    def releaseOutput(self, buf, shape):
        if id(buf) not in self.held:
            raise AssertionError(f"release of {self.buf_name.get(id(buf))}, which is not held")
        self.held.discard(id(buf))
        self.released.add(id(buf))
        self.log.append(f"release {self.buf_name[id(buf)]}")

    def dispatch(self, node, inputs, out, extras=None):
        for b in inputs:
            if b is None:
                continue  # computed inside the fused kernel
            assert id(b) not in self.released, "reads a released buffer"
        line = f"{self.node_name[id(node)]} -> {self.buf_name[id(out)]}"
        if extras and "fusedAppend" in extras:
            f = extras["fusedAppend"]
            line += f" +append({self.buf_name[id(f['kNew'])]},{self.buf_name[id(f['vNew'])]})"
            if "ropeCos" in f:
                line += (f" +rope({self.buf_name[id(f['q'])]}@{f['qOffset']},"
                         f"k@{f['kNewOffset']},v@{f['vNewOffset']})")
        self.log.append(line)

    def submit(self):
        self.log.append("submit")


heads = dict(qHeads=2, kvHeads=1, headDim=4, windowLeft=INF)


def test_each_node_once_after_inputs_freed_after_last_reader():
    q, k, v = mat(3, 8), mat(3, 4), mat(3, 4)
    a = sdpa(q, k, v, dict(heads, windowRight=0))
    b = sdpa(a, k, v, dict(heads, windowRight=0))
    c = sdpa(a, v, k, dict(heads, windowRight=0))
    d = sdpa(b, k, v, dict(heads, windowRight=0))
    rec = Recorder(dict(q=q, k=k, v=v, a=a, b=b, c=c, d=d))
    evalValues([d, c], rec)
    assert rec.log == ["a -> #0", "b -> #1", "d -> #2", "release #1", "c -> #3", "release #0",
                       "submit"]
    assert a.state == "released" and b.state == "released"
    assert c.state == "materialized" and d.state == "materialized"
    with pytest.raises(RuntimeError, match="buffer was recycled by eval"):
        evalValues([sdpa(a, k, v, dict(heads, windowRight=0))], Recorder({}))


def test_write_rows_writes_caller_owned_buffer_and_is_never_freed():
    cache = mat(8, 4)
    q, k0, v0 = mat(2, 4), mat(2, 4), mat(2, 4)
    kNew = sdpa(q, k0, v0, dict(qHeads=1, kvHeads=1, headDim=4, windowLeft=INF, windowRight=0))
    k = writeRows(cache, kNew, 3)
    y = sdpa(mat(5, 8), k, k, dict(heads, windowRight=0))
    rec = Recorder(dict(cache=cache, kNew=kNew, k=k, y=y))
    evalValues([y], rec)
    assert rec.log == ["kNew -> #0", "k -> cache", "release #0", "y -> #1", "submit"]
    assert k.buffer is cache.buffer


def _decode_step(t, cacheRows=8, wr=0, kRows=1):
    kc, vc = mat(cacheRows, 4), mat(cacheRows, 4)
    kNew, vNew, q = mat(kRows, 4), mat(kRows, 4), mat(1, 8)
    k = writeRows(kc, kNew, t)
    v = writeRows(vc, vNew, t)
    y = sdpa(q, k, v, dict(heads, windowRight=wr, qPosOffset=t + kRows - 1))
    return dict(kc=kc, vc=vc, kNew=kNew, vNew=vNew, q=q, k=k, v=v, y=y)


def test_decode_step_fuses_append_into_attention():
    n = _decode_step(3)
    rec = Recorder(n)
    evalValues([n["y"]], rec)
    assert rec.log == ["y -> #0 +append(kNew,vNew)", "submit"]
    assert n["k"].buffer is n["kc"].buffer and n["v"].buffer is n["vc"].buffer


def test_no_fusion_when_the_view_is_also_a_target_or_not_a_single_row():
    n = _decode_step(3)
    rec = Recorder(n)
    evalValues([n["y"], n["k"]], rec)
    assert rec.log == ["k -> kc", "v -> vc", "y -> #0", "submit"]
    n = _decode_step(2, kRows=2)
    rec = Recorder(n)
    evalValues([n["y"]], rec)
    assert rec.log[:2] == ["k -> kc", "v -> vc"]
    n = _decode_step(3, wr=INF)  # cross-style window: not the causal decode step
    assert _fusable_appends([n["k"], n["v"], n["y"]], [n["y"]]) == {}


def _decoder_layer_step(t, *, share_tables=True, slice_v=True):
    """q and kNew roped out of one fused qkv row, vNew sliced out of it
    (packages/runntime/src/zoo/moonshine/decoder.ts:58-76)."""
    from runntime_b200 import rope, slice as slice_
    w = 8  # qHeads 2 x headDim 4; kvHeads 2 for this one
    hd = 4
    qkv = mat(1, 3 * w, name="qkv")
    cos, sin, cos2 = mat(1, hd), mat(1, hd), mat(1, hd)
    kc, vc = mat(16, w), mat(16, w)
    q = rope(qkv, cos, sin, dict(headDim=hd, srcStart=0, width=w))
    kNew = rope(qkv, cos if share_tables else cos2, sin, dict(headDim=hd, srcStart=w, width=w))
    vNew = slice_(qkv, 1, 2 * w, 3 * w) if slice_v else mat(1, w)
    k, v = writeRows(kc, kNew, t), writeRows(vc, vNew, t)
    y = sdpa(q, k, v, dict(qHeads=2, kvHeads=2, headDim=hd, windowLeft=INF, windowRight=0,
                           qPosOffset=t))
    return dict(qkv=qkv, cos=cos, sin=sin, cos2=cos2, kc=kc, vc=vc, q=q, kNew=kNew, vNew=vNew,
                k=k, v=v, y=y)


def test_decoder_layer_step_is_one_dispatch():
    n = _decoder_layer_step(5)
    rec = Recorder(n)
    evalValues([n["y"]], rec)
    assert rec.log == ["y -> #0 +append(qkv,qkv) +rope(qkv@0,k@32,v@64)", "submit"]
    # the absorbed nodes were never dispatched and own no buffer
    for name in ("q", "kNew", "vNew"):
        assert n[name].state == "pending"
    assert n["k"].buffer is n["kc"].buffer


def test_rope_is_not_absorbed_over_different_tables_or_when_kept():
    n = _decoder_layer_step(5, share_tables=False)
    rec = Recorder(n)
    evalValues([n["y"]], rec)
    assert rec.log[:2] == ["q -> #0", "kNew -> #1"]
    assert rec.log[2] == "y -> #2 +append(#1,qkv)"   # append still fused, v still sliced in place
    n = _decoder_layer_step(5)
    rec = Recorder(n)
    evalValues([n["y"], n["q"]], rec)                # q is wanted by the caller: dispatched
    assert "q -> #0" in rec.log and not any("+rope" in line for line in rec.log)


def test_new_v_row_may_be_a_tensor_of_its_own():
    n = _decoder_layer_step(5, slice_v=False)
    rec = Recorder(n)
    evalValues([n["y"]], rec)
    assert rec.log == ["y -> #0 +append(qkv,vNew) +rope(qkv@0,k@32,v@0)", "submit"]
