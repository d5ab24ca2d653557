"""The CUDA backend behind the operator API: the counterpart of the reference's
WebGPU executor (packages/runntime/src/core/gpu/eval.ts:135-320) and of the
device-agnostic eval driver above it
(packages/runntime/src/core/graph/evalCore.ts:14-43,63-267).

Buffers are CUDA device pointers owned by the C library instead of GPUBuffer
handles; ``submit()`` has nothing to do because work is already enqueued on the
context's stream in dispatch order; ``readback`` is a device-to-host copy plus
a stream sync.  Outputs come from a pool keyed by (dtype, elems) and return to
it after their last consumer; in-place ops (writeRows) write caller-owned
buffers that are never pooled or freed here.

One fusion the reference does not have: a decode-step ``attn`` node whose k and
v are single-row ``writeRows`` appends at the query's position runs as one
kernel that appends and attends (rt_attn_decode).  When, as in a decoder
layer's step (packages/runntime/src/zoo/moonshine/decoder.ts:58-76), q and the
new k row are ``rope`` windows of one fused qkv row over the same tables and
the new v row is a column ``slice`` (or any other row), those nodes run inside
the same kernel too: six dispatches become one.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import AttnArgs, DecodeArgs, DTYPE_CODE, WINDOW_INF, check
from .errors import RunntimeError
from .value import DeviceBuffer, Value, ValueMeta, elemBytes, matrix, materialized

IN_PLACE_OPS = {"writeRows"}


class CudaExecutor:
    """One context on one GPU: stream, scratch, buffer pool."""

    def __init__(self, device: int = 0):
        self._lib = _lib.load()
        ctx = C.c_void_p()
        check(self._lib.rt_ctx_create(device, C.byref(ctx)))
        self._ctx = ctx
        self.device = device
        self._pool: Dict[tuple, List[DeviceBuffer]] = {}
        self._live: set = set()
        self._disposed = False
        self.dispatches: List[str] = []   # op routes since the last submit(), for tests/perf

    # -- context ---------------------------------------------------------------
    @property
    def ctx(self):
        if self._disposed:
            raise RunntimeError("RESOURCE_DISPOSED", "executor was disposed")
        return self._ctx

    def setStream(self, cuda_stream: Optional[int]) -> None:
        """Enqueue on the caller's stream (a cudaStream_t handle as an int; 0 is
        the legacy default stream); None goes back to the context's own."""
        check(self._lib.rt_ctx_set_stream(self.ctx, C.c_void_p(cuda_stream or 0),
                                          0 if cuda_stream is None else 1), self.ctx)

    def setOption(self, option: int, value: int) -> None:
        check(self._lib.rt_ctx_set_option(self.ctx, option, value), self.ctx)

    def sync(self) -> None:
        check(self._lib.rt_sync(self.ctx), self.ctx)

    def launchCount(self) -> int:
        return int(self._lib.rt_launch_count(self.ctx))

    def dispose(self) -> None:
        if self._disposed:
            return
        for b in list(self._live):
            self._free(b)
        for bucket in self._pool.values():
            for b in bucket:
                self._lib.rt_buf_free(self._ctx, C.c_void_p(b.ptr))
        self._pool.clear()
        check(self._lib.rt_ctx_destroy(self._ctx))
        self._disposed = True

    # -- buffers ---------------------------------------------------------------
    def _alloc(self, nbytes: int) -> DeviceBuffer:
        p = C.c_void_p()
        check(self._lib.rt_buf_alloc(self.ctx, nbytes, C.byref(p)), self.ctx)
        b = DeviceBuffer(p.value, nbytes, owned=True)
        self._live.add(b)
        return b

    def _free(self, b: DeviceBuffer) -> None:
        if b in self._live:
            self._live.discard(b)
            check(self._lib.rt_buf_free(self._ctx, C.c_void_p(b.ptr)), self._ctx)

    def liveBuffers(self) -> int:
        """Caller-visible allocations not yet destroyed (leak checks)."""
        return len(self._live)

    def upload(self, data, shape=None, dtype: Optional[str] = None) -> Value:
        """A materialized Value holding ``data`` (f32 values; stored as f16 raw
        halfwords when the dtype is 'f16').  ``shape`` is [rows, cols], a flat
        [n], or a ValueMeta.  Mirrors tensor()/upload of the reference
        (packages/runntime/src/core/gpu/buffers.ts:83-121)."""
        arr = np.ascontiguousarray(np.asarray(data, dtype=np.float32)).reshape(-1)
        if isinstance(shape, ValueMeta):
            meta = shape if dtype is None else ValueMeta(shape.elems, dtype, shape.dims)
        else:
            dims = tuple(int(d) for d in (shape if shape is not None else [arr.size]))
            meta = ValueMeta(int(np.prod(dims)) if dims else 0, dtype or "f32", dims)
        if meta.elems == 0 or arr.size == 0:
            raise RunntimeError("INVALID_ARGUMENT", "upload: empty tensor")
        if arr.size != meta.elems:
            raise ValueError(f"upload: data has {arr.size} elems, shape wants {meta.elems}")
        host = arr.astype(np.float16) if meta.dtype == "f16" else arr
        buf = self._alloc(host.nbytes)
        check(self._lib.rt_buf_upload(self.ctx, C.c_void_p(buf.ptr), 0,
                                      host.ctypes.data_as(C.c_void_p), host.nbytes), self.ctx)
        self.sync()  # the host array may go away after this call
        return materialized(meta, buf)

    def zeros(self, shape, dtype: str = "f32") -> Value:
        dims = tuple(int(d) for d in shape)
        return self.upload(np.zeros(int(np.prod(dims)), np.float32), dims, dtype)

    def wrap(self, ptr: int, shape, dtype: str, keepalive=None) -> Value:
        """A materialized Value over device memory someone else owns (for
        example a torch tensor's ``data_ptr()``)."""
        dims = tuple(int(d) for d in shape)
        elems = int(np.prod(dims))
        return materialized(ValueMeta(elems, dtype, dims),
                            DeviceBuffer(ptr, elems * elemBytes(dtype), owned=False,
                                         keepalive=keepalive))

    def destroy(self, value: Value) -> None:
        """Frees a caller-owned upload."""
        b = value.buffer
        if b.owned:
            self._free(b)
        value.markReleased("buffer was destroyed by its owner")

    # -- Executor interface ------------------------------------------------------
    def acquireOutput(self, shape: ValueMeta) -> DeviceBuffer:
        key = (shape.dtype, shape.elems)
        bucket = self._pool.get(key)
        if bucket:
            b = bucket.pop()
            self._live.add(b)
            return b
        return self._alloc(shape.elems * elemBytes(shape.dtype))

    def releaseOutput(self, buffer: DeviceBuffer, shape: ValueMeta) -> None:
        if not buffer.owned:
            return
        self._live.discard(buffer)
        self._pool.setdefault((shape.dtype, shape.elems), []).append(buffer)

    def dispatch(self, node: Value, inputs: Sequence[DeviceBuffer], out: DeviceBuffer,
                 extras: Optional[dict] = None) -> None:
        op = node.pending.op
        if op == "attn":
            self._dispatch_attn(node, inputs, out, extras)
        elif op == "writeRows":
            self._dispatch_write_rows(node, inputs)
        elif op == "rope":
            self._dispatch_rope(node, inputs, out)
        elif op in ("sliceRows", "sliceCols"):
            self._dispatch_slice(node, inputs, out)
        elif op == "softmax":
            self._dispatch_softmax(node, inputs, out)
        elif op == "matmul":
            hasBias, hasAddend, act, baseRow, _ = (int(v) for v in node.pending.attrs)
            ins = node.pending.inputs
            m, k = ins[0].shape.dims
            bRows, n = ins[1].shape.dims
            nxt = 2
            bias = addend = None
            if hasBias:
                bias = C.c_void_p(inputs[nxt].ptr)
                nxt += 1
            if hasAddend:
                addend = C.c_void_p(inputs[nxt].ptr)
            check(self._lib.rt_matmul(self.ctx, C.c_void_p(inputs[0].ptr), C.c_void_p(inputs[1].ptr),
                                      bias, addend, C.c_void_p(out.ptr), m, k, n, bRows, baseRow,
                                      act, DTYPE_CODE[node.shape.dtype]), self.ctx)
            self.dispatches.append("matmul")
        elif op == "argmaxDot":
            wV = node.pending.inputs[0]
            rows, cols = wV.shape.dims
            check(self._lib.rt_argmax_dot(self.ctx, C.c_void_p(inputs[0].ptr),
                                          C.c_void_p(inputs[1].ptr), C.c_void_p(out.ptr), rows,
                                          cols, DTYPE_CODE[wV.shape.dtype]), self.ctx)
            self.dispatches.append("argmaxDot")
        elif op == "localAttention":
            heads, hd, window, kScale, softcap = node.pending.attrs
            check(self._lib.rt_local_attention(
                self.ctx, C.c_void_p(inputs[0].ptr), C.c_void_p(inputs[1].ptr),
                C.c_void_p(inputs[2].ptr), C.c_void_p(out.ptr), node.shape.dims[0], int(heads),
                int(hd), int(window), float(kScale), float(softcap),
                DTYPE_CODE[node.shape.dtype]), self.ctx)
            self.dispatches.append("localAttention")
        else:
            raise RunntimeError("INVALID_ARGUMENT", f"dispatch: no kernel for op '{op}'")

    def submit(self) -> None:
        """Work is already on the stream; kept for the Executor interface."""

    def readback(self, buffer: DeviceBuffer, shape: ValueMeta) -> np.ndarray:
        host = np.empty(shape.elems, np.float16 if shape.dtype == "f16" else np.float32)
        check(self._lib.rt_buf_download(self.ctx, C.c_void_p(buffer.ptr), 0,
                                        host.ctypes.data_as(C.c_void_p), host.nbytes), self.ctx)
        return host.astype(np.float32)

    def releaseValues(self, values: Sequence[Value]) -> None:
        for v in values:
            if v.state == "materialized" and v.pending is not None \
                    and v.pending.op not in IN_PLACE_OPS:
                self.releaseOutput(v.buffer, v.shape)
                v.markReleased("released by releaseValues")

    # -- per-op encoders -----------------------------------------------------------
    def _dispatch_attn(self, node, inputs, out, extras):
        a = node.pending.attrs
        qHeads, kvHeads, hd, wl, wr, qPosOffset, hasSinks, hasSegs, maxSegment, packed = (
            int(x) for x in a[:10])
        ins = list(node.pending.inputs)
        bufs = list(inputs)
        if packed:
            qv = ins[0]
            q = k = v = bufs[0]
            rest = 1
            qLen = kvLen = qv.shape.dims[0]
        else:
            q, k, v = bufs[0], bufs[1], bufs[2]
            rest = 3
            qLen, kvLen = ins[0].shape.dims[0], ins[1].shape.dims[0]
        sinks = segs = None
        if hasSinks:
            sinks = bufs[rest]
            rest += 1
        if hasSegs:
            segs = bufs[rest]
        fused = (extras or {}).get("fusedAppend")
        if fused is not None:
            d = DecodeArgs()
            d.q = fused["q"].ptr + fused["qOffset"] if "q" in fused else q.ptr
            d.out = out.ptr
            d.kCache, d.vCache = fused["kCache"].ptr, fused["vCache"].ptr
            d.kNew = fused["kNew"].ptr + fused["kNewOffset"]
            d.vNew = fused["vNew"].ptr + fused["vNewOffset"]
            if "ropeCos" in fused:
                d.ropeCos, d.ropeSin = fused["ropeCos"].ptr, fused["ropeSin"].ptr
            d.sinks = sinks.ptr if sinks else None
            d.cacheSeqStride = 0
            d.dtype = DTYPE_CODE[node.shape.dtype]
            d.batch, d.cacheRows, d.kvLen = 1, fused["cacheRows"], kvLen
            d.qHeads, d.kvHeads, d.headDim = qHeads, kvHeads, hd
            d.windowLeft, d.splits = wl, 0
            check(self._lib.rt_attn_decode(self.ctx, C.byref(d)), self.ctx)
            self.dispatches.append("decode+rope+append" if "ropeCos" in fused else "decode+append")
            return
        args = AttnArgs()
        args.q, args.k, args.v, args.out = q.ptr, k.ptr, v.ptr, out.ptr
        args.sinks = sinks.ptr if sinks else None
        args.segments = segs.ptr if segs else None
        args.dtype = DTYPE_CODE[node.shape.dtype]
        args.qkvPacked = packed
        args.qLen, args.kvLen = qLen, kvLen
        args.qHeads, args.kvHeads, args.headDim = qHeads, kvHeads, hd
        args.windowLeft, args.windowRight, args.maxSegment = wl, wr, maxSegment
        args.qPosOffset = qPosOffset
        if len(a) > 10 and a[10]:
            args.hasKeyBias, args.biasStart, args.biasEnd = 1, int(a[11]), int(a[12])
            args.biasValue = float(a[13])
        route = C.c_char_p()
        check(self._lib.rt_attn_route(self.ctx, C.byref(args), C.byref(route)), self.ctx)
        check(self._lib.rt_attn(self.ctx, C.byref(args)), self.ctx)
        self.dispatches.append(route.value.decode())

    def _dispatch_rope(self, node, inputs, out):
        xV = node.pending.inputs[0]
        headDim, srcStart, width = (int(a) for a in node.pending.attrs)
        rows, cols = xV.shape.dims
        check(self._lib.rt_rope(self.ctx, C.c_void_p(inputs[0].ptr), C.c_void_p(inputs[1].ptr),
                                C.c_void_p(inputs[2].ptr), C.c_void_p(out.ptr), rows, cols,
                                headDim, srcStart, width, DTYPE_CODE[xV.shape.dtype]), self.ctx)
        self.dispatches.append("rope")

    def _dispatch_softmax(self, node, inputs, out):
        a = node.pending.attrs
        if a is None or len(a) < 3:
            raise RunntimeError("INVALID_ARGUMENT",
                                "dispatch: softmax attrs need [masked, windowLeft, windowRight]")
        rows, cols = node.shape.dims
        segs = C.c_void_p(inputs[1].ptr) if int(a[0]) else None
        check(self._lib.rt_softmax(self.ctx, C.c_void_p(inputs[0].ptr), C.c_void_p(out.ptr), segs,
                                   rows, cols, int(a[1]), int(a[2]), DTYPE_CODE[node.shape.dtype]),
              self.ctx)
        self.dispatches.append("softmax")

    def _dispatch_slice(self, node, inputs, out):
        xV = node.pending.inputs[0]
        rows, cols = xV.shape.dims
        start, end = (int(a) for a in node.pending.attrs)
        box = (start, end, 0, cols) if node.pending.op == "sliceRows" else (0, rows, start, end)
        check(self._lib.rt_slice(self.ctx, C.c_void_p(inputs[0].ptr), C.c_void_p(out.ptr), rows,
                                 cols, *box, DTYPE_CODE[xV.shape.dtype]), self.ctx)
        self.dispatches.append(node.pending.op)

    def _dispatch_write_rows(self, node, inputs):
        dstV, srcV = node.pending.inputs
        startRow = int(node.pending.attrs[0])
        rows, cols = srcV.shape.dims
        check(self._lib.rt_kv_append(self.ctx, C.c_void_p(inputs[0].ptr), C.c_void_p(inputs[1].ptr),
                                     startRow, rows, cols, dstV.shape.dims[0],
                                     DTYPE_CODE[dstV.shape.dtype]), self.ctx)
        self.dispatches.append("writeRows")


gpuExecutor = CudaExecutor


def _collect_pending(targets: Sequence[Value]) -> List[Value]:
    order: List[Value] = []
    seen = set()

    def visit(v: Value) -> None:
        if v.state == "released":
            op = v.pending.op if v.pending else "upload"
            raise RuntimeError(f"evalValues: '{op}': {v.releasedReason}")
        if v.state == "materialized" or id(v) in seen:
            return
        seen.add(id(v))
        for i in v.pending.inputs:
            visit(i)
        order.append(v)

    for t in targets:
        visit(t)
    return order


def _fusable_appends(order: List[Value], targets: Sequence[Value]) -> Dict[int, dict]:
    """attn nodes (by id) that can run as one append+attend kernel: one query
    row at the last position, causal, with k and v being single-row writeRows
    appends at that position used by nothing else in this evaluation.  The plan
    also names the rope / slice nodes feeding q and the new rows that the kernel
    can absorb ("elided": used once, not targets, rope over the same tables)."""
    uses: Dict[int, int] = {}
    for n in order:
        for i in n.pending.inputs:
            uses[id(i)] = uses.get(id(i), 0) + 1
    target_ids = {id(t) for t in targets}
    pending_ids = {id(n) for n in order}

    def private(v: Value, op: str) -> bool:
        return (id(v) in pending_ids and v.pending.op == op and uses.get(id(v), 0) == 1
                and id(v) not in target_ids)

    plan: Dict[int, dict] = {}
    for n in order:
        if n.pending.op != "attn":
            continue
        a = n.pending.attrs
        ins = n.pending.inputs
        if int(a[9]) or len(ins) < 3 or ins[0].shape.dims[0] != 1 or int(a[4]) != 0:
            continue
        q, k, v = ins[0], ins[1], ins[2]
        ok = True
        for w in (k, v):
            ok &= (private(w, "writeRows")
                   and w.pending.inputs[1].shape.dims[0] == 1
                   and int(w.pending.attrs[0]) == int(a[5])
                   and w.shape.dims[0] == int(a[5]) + 1)
        if not ok or k is v:
            continue
        entry = {"k": k, "v": v, "elided": []}
        kNew, vNew = k.pending.inputs[1], v.pending.inputs[1]
        hd = int(a[2])
        if (private(q, "rope") and private(kNew, "rope")
                and q.pending.inputs[1] is kNew.pending.inputs[1]
                and q.pending.inputs[2] is kNew.pending.inputs[2]
                and int(q.pending.attrs[0]) == hd and int(kNew.pending.attrs[0]) == hd
                and q.pending.inputs[0].shape.dims[0] == 1
                and kNew.pending.inputs[0].shape.dims[0] == 1):
            entry["rope"] = (q, kNew)
            entry["elided"] += [q, kNew]
        if private(vNew, "sliceCols") and vNew.pending.inputs[0].shape.dims[0] == 1:
            entry["vSlice"] = vNew
            entry["elided"].append(vNew)
        plan[id(n)] = entry
    return plan


def _window(node: Value, startCol: int):
    """(buffer, byte offset) of column ``startCol`` of the single row ``node`` reads."""
    x = node.pending.inputs[0]
    return x.buffer, startCol * elemBytes(x.shape.dtype)


def _fused_extras(f: dict) -> dict:
    """Buffers (and byte offsets into them) the fused decode step reads."""
    k, v = f["k"], f["v"]
    kNew, vNew = k.pending.inputs[1], v.pending.inputs[1]
    ex = {"kCache": k.pending.inputs[0].buffer, "vCache": v.pending.inputs[0].buffer,
          "cacheRows": k.pending.inputs[0].shape.dims[0]}
    if "rope" in f:
        q = f["rope"][0]
        ex["q"], ex["qOffset"] = _window(q, int(q.pending.attrs[1]))
        ex["kNew"], ex["kNewOffset"] = _window(kNew, int(kNew.pending.attrs[1]))
        ex["ropeCos"], ex["ropeSin"] = q.pending.inputs[1].buffer, q.pending.inputs[2].buffer
    else:
        ex["kNew"], ex["kNewOffset"] = kNew.buffer, 0
    if "vSlice" in f:
        ex["vNew"], ex["vNewOffset"] = _window(vNew, int(vNew.pending.attrs[0]))
    else:
        ex["vNew"], ex["vNewOffset"] = vNew.buffer, 0
    return ex


def evalValues(targets: Sequence[Value], ex: CudaExecutor) -> None:
    """Dispatches every pending node the targets depend on, once, in dependency
    order; intermediates go back to the pool after their last consumer."""
    order = _collect_pending(targets)
    produced = {id(v) for v in order}
    target_ids = {id(t) for t in targets}
    fuse = _fusable_appends(order, targets)
    skipped = {id(w) for f in fuse.values() for w in (f["k"], f["v"])}
    # Nodes a fused kernel computes on the fly: never dispatched, they stay pending.
    elided = {id(w) for f in fuse.values() for w in f["elided"]}
    remaining: Dict[int, int] = {}
    for n in order:
        for i in set(n.pending.inputs):
            remaining[id(i)] = remaining.get(id(i), 0) + 1
    aliased = set()
    for node in order:
        if id(node) in elided:
            continue
        p = node.pending
        ins = [None if id(i) in elided else i.buffer for i in p.inputs]
        if p.op in IN_PLACE_OPS:
            out = ins[0]
            aliased.add(id(node))
            if id(node) not in skipped:
                ex.dispatch(node, ins, out)
        else:
            out = ex.acquireOutput(node.shape)
            extras = None
            if id(node) in fuse:
                extras = {"fusedAppend": _fused_extras(fuse[id(node)])}
            ex.dispatch(node, ins, out, extras)
        node.setMaterialized(out)
        if id(node) in skipped:
            continue  # its inputs are read by the fused kernel: released after that one
        consumed = [p.inputs]
        if id(node) in fuse:
            f = fuse[id(node)]
            consumed += [f["k"].pending.inputs, f["v"].pending.inputs]
            consumed += [w.pending.inputs for w in f["elided"]]
        for group in consumed:
            for i in set(group):
                remaining[id(i)] -= 1
                if (remaining[id(i)] == 0 and id(i) in produced and id(i) not in target_ids):
                    if id(i) in aliased or id(i) in elided:
                        continue  # a view of a caller-owned buffer / never materialized
                    ex.releaseOutput(i.buffer, i.shape)
                    i.markReleased()
    ex.submit()


def toArray(value: Value, ex: CudaExecutor) -> np.ndarray:
    """Evaluates ``value`` and reads it back as float32."""
    if value.state == "pending":
        evalValues([value], ex)
    return ex.readback(value.buffer, value.shape)
