"""Batched entry points over the C ABI, for callers that hold many sequences:

- ``prefill_batched``: padded-batch prefill (``batch`` sequences of
  ``seqStride`` rows, per-sequence lengths) — the packed-segments form of the
  reference (packages/runntime/src/zoo/minilm/model.ts:167-185) computed on the
  fly from the lengths.
- ``decode_batched``: one decode step for ``batch`` KV caches with the append
  fused — the step of packages/runntime/src/zoo/moonshine/decoder.ts:58-76 for
  many sequences at once; ``KvCacheEngine`` keeps the caches and lengths like
  the transcriber does (transcriber.ts:111-118,161-203).
- ``ShardedDecode``: long-context decode with the KV sequence split across
  ranks; each rank attends to its rows, the (m, l, acc) partials are
  all-gathered and merged (algebra of attnDecode.ts:405-422).

Tensors are passed as device pointers (ints) or as anything with
``data_ptr()`` (torch tensors).  torch is used only for device memory and
``torch.distributed``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

from ._lib import AttnArgs, DecodeArgs, DTYPE_CODE, Exchange, WINDOW_INF, check
from .executor import CudaExecutor


def _ptr(x) -> Optional[int]:
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return int(x.data_ptr())


def _win(w) -> int:
    if w is None or w == float("inf"):
        return WINDOW_INF
    return min(int(w), WINDOW_INF)


def prefill_batched(ex: CudaExecutor, q, k, v, out, *, dtype: str, batch: int, seqStride: int,
                    seqLens, qHeads: int, kvHeads: int, headDim: int, windowLeft=None,
                    windowRight=None, sinks=None) -> None:
    """q/out: [batch*seqStride, qHeads*headDim]; k/v: [batch*seqStride,
    kvHeads*headDim]; seqLens: device int32 [batch].  Row r of sequence b sees
    keys of sequence b only, inside the window, below seqLens[b]; rows at or
    past seqLens[b] come out zero."""
    a = AttnArgs()
    a.q, a.k, a.v, a.out = _ptr(q), _ptr(k), _ptr(v), _ptr(out)
    a.sinks = _ptr(sinks)
    a.dtype = DTYPE_CODE[dtype]
    a.qLen = a.kvLen = batch * seqStride
    a.qHeads, a.kvHeads, a.headDim = qHeads, kvHeads, headDim
    a.windowLeft, a.windowRight = _win(windowLeft), _win(windowRight)
    a.seqStride, a.seqLens = seqStride, _ptr(seqLens)
    check(ex._lib.rt_attn(ex.ctx, C.byref(a)), ex.ctx)


def decode_batched(ex: CudaExecutor, q, out, kCache, vCache, *, dtype: str, batch: int,
                   cacheRows: int, qHeads: int, kvHeads: int, headDim: int, kvLen: int = 0,
                   kvLens=None, kNew=None, vNew=None, cacheSeqStride: Optional[int] = None,
                   windowLeft=None, sinks=None, partialsOut=None, splits: int = 0,
                   ropeCos=None, ropeSin=None, ropeByPosition: bool = False, qRowStride: int = 0,
                   kNewRowStride: int = 0, vNewRowStride: int = 0, exchange=None) -> None:
    """One decode step for ``batch`` sequences; see rt_attn_decode in
    include/rt_attn.h.  ``kvLen`` is the (maximum) visible length including the
    appended row; ``kvLens`` gives it per sequence.  With ``ropeCos``/``ropeSin``
    q and kNew are un-rotated rows (for example windows of the fused qkv
    projection, ``*RowStride`` apart) and the kernel rotates them."""
    d = DecodeArgs()
    d.q, d.out = _ptr(q), _ptr(out)
    d.kCache, d.vCache = _ptr(kCache), _ptr(vCache)
    d.kNew, d.vNew = _ptr(kNew), _ptr(vNew)
    d.kvLens, d.sinks, d.partialsOut = _ptr(kvLens), _ptr(sinks), _ptr(partialsOut)
    d.cacheSeqStride = (cacheRows * kvHeads * headDim) if cacheSeqStride is None else cacheSeqStride
    d.dtype = DTYPE_CODE[dtype]
    d.batch, d.cacheRows, d.kvLen = batch, cacheRows, kvLen
    d.qHeads, d.kvHeads, d.headDim = qHeads, kvHeads, headDim
    d.windowLeft, d.splits = _win(windowLeft), splits
    d.ropeCos, d.ropeSin, d.ropeByPosition = _ptr(ropeCos), _ptr(ropeSin), int(ropeByPosition)
    d.qRowStride, d.kNewRowStride, d.vNewRowStride = qRowStride, kNewRowStride, vNewRowStride
    if exchange is not None:
        d.exchange = C.pointer(exchange)
    check(ex._lib.rt_attn_decode(ex.ctx, C.byref(d)), ex.ctx)


def merge_partials(ex: CudaExecutor, partials, parts: int, units: int, headDim: int, out,
                   dtype: str) -> None:
    check(ex._lib.rt_attn_merge_partials(ex.ctx, C.c_void_p(_ptr(partials)), parts, units,
                                         headDim, C.c_void_p(_ptr(out)), DTYPE_CODE[dtype]),
          ex.ctx)


class KvCacheEngine:
    """Preallocated self-attention caches for ``batch`` sequences plus their
    lengths, stepped one token at a time: append + causal attend in one kernel.
    Optionally a fixed cross-attention K/V (encoder states) per sequence."""

    def __init__(self, ex: CudaExecutor, *, batch: int, maxPositions: int, qHeads: int,
                 kvHeads: int, headDim: int, dtype: str = "f16", windowLeft=None, device=None):
        import torch
        self.ex, self.batch, self.maxPositions = ex, batch, maxPositions
        self.qHeads, self.kvHeads, self.headDim, self.dtype = qHeads, kvHeads, headDim, dtype
        self.windowLeft = windowLeft
        dev = device if device is not None else torch.device("cuda", ex.device)
        tdt = torch.float16 if dtype == "f16" else torch.float32
        kvw = kvHeads * headDim
        self.k = torch.zeros(batch, maxPositions, kvw, dtype=tdt, device=dev)
        self.v = torch.zeros(batch, maxPositions, kvw, dtype=tdt, device=dev)
        self.lens = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.maxLen = 0
        self.cross: Optional[Tuple[object, object, int]] = None
        self.rope = None

    def setCross(self, k, v, rows: int) -> None:
        """Precomputed cross-attention K/V [batch, rows, kvHeads*headDim]."""
        self.cross = (k, v, rows)

    def setRope(self, cos, sin) -> None:
        """Pair-duplicated f32 tables [maxPositions, headDim] (any scale folded in,
        packages/runntime/src/zoo/moonshine/rope.ts:18-50); stepQkv then rotates."""
        self.rope = (cos, sin)

    def stepQkv(self, qkv, out) -> None:
        """One decoder-layer step from the fused projection's rows
        qkv [batch, (qHeads + 2*kvHeads)*headDim] (columns q|k|v, un-rotated): rope
        on q and k at each sequence's position, append, causal attend — the six
        dispatches of packages/runntime/src/zoo/moonshine/decoder.ts:66-76 in one launch."""
        qw, kvw = self.qHeads * self.headDim, self.kvHeads * self.headDim
        es = qkv.element_size()
        base = qkv.data_ptr()
        cos, sin = self.rope
        self._advance()
        decode_batched(self.ex, base, out, self.k, self.v, dtype=self.dtype, batch=self.batch,
                       cacheRows=self.maxPositions, qHeads=self.qHeads, kvHeads=self.kvHeads,
                       headDim=self.headDim, kvLen=self.maxLen, kvLens=self.lens,
                       kNew=base + qw * es, vNew=base + (qw + kvw) * es,
                       windowLeft=self.windowLeft, ropeCos=cos, ropeSin=sin, ropeByPosition=True,
                       qRowStride=qw + 2 * kvw, kNewRowStride=qw + 2 * kvw,
                       vNewRowStride=qw + 2 * kvw)

    def _advance(self) -> None:
        if self.maxLen + 1 > self.maxPositions:
            raise ValueError(
                f"writeRows: rows [{self.maxLen}, {self.maxLen + 1}) exceed dst capacity "
                f"{self.maxPositions}")
        self.lens.add_(1)
        self.maxLen += 1

    def step(self, q, kNew, vNew, out) -> None:
        """Appends kNew/vNew at each sequence's end and attends causally."""
        self._advance()
        decode_batched(self.ex, q, out, self.k, self.v, dtype=self.dtype, batch=self.batch,
                       cacheRows=self.maxPositions, qHeads=self.qHeads, kvHeads=self.kvHeads,
                       headDim=self.headDim, kvLen=self.maxLen, kvLens=self.lens, kNew=kNew,
                       vNew=vNew, windowLeft=self.windowLeft)

    def crossAttend(self, q, out) -> None:
        k, v, rows = self.cross
        decode_batched(self.ex, q, out, k, v, dtype=self.dtype, batch=self.batch, cacheRows=rows,
                       qHeads=self.qHeads, kvHeads=self.kvHeads, headDim=self.headDim, kvLen=rows)


def shard_rows(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows [start, end) of a ``total``-row KV sequence that live on ``rank``:
    contiguous, balanced to within one row."""
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def exchange_words(world: int, units: int, headDim: int) -> Tuple[int, int]:
    """(floats of one rank's partials buffer, 32-bit words of its control block)
    for the cross-GPU exchange: two halves of [world, units, 2+headDim] partials;
    [world] arrival words + step counter."""
    return 2 * world * units * (2 + headDim), world + 1


def make_exchange(world: int, rank: int, partialPtrs, controlPtrs) -> Exchange:
    """rt_exchange over every rank's partials buffer and control block as mapped in
    this process (``controlPtrs[r]``: rank r's [world] arrival words, then its step
    counter, all zero at the start)."""
    x = Exchange()
    x.world, x.rank = world, rank
    for r in range(world):
        x.partials[r] = _ptr(partialPtrs[r])
        x.flags[r] = _ptr(controlPtrs[r])
    x.step = _ptr(controlPtrs[rank]) + 4 * world
    return x


class PeerExchangeDecode:
    """KV-sequence-sharded decode whose ranks trade partials through peer memory:
    the decode kernel stores this rank's (m, l, acc) rows into every peer's buffer
    and signals them, a merge kernel waits for all ranks' rows of the step and
    merges — no library collective on the step.  The buffers come from torch's
    symmetric memory (one process per GPU, NVLink peers)."""

    def __init__(self, *, units: int, headDim: int, device, group=None):
        import os
        import torch
        import torch.distributed as dist
        # plain peer mappings only: no NVLink multicast object is bound to these buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        nfloat, nword = exchange_words(self.world, units, headDim)
        group_name = (group or dist.group.WORLD).group_name
        self.partials = symm.empty(nfloat, dtype=torch.float32, device=device)
        self.control = symm.empty(nword, dtype=torch.int32, device=device)
        self.partials.zero_()
        self.control.zero_()
        hp = symm.rendezvous(self.partials, group_name)
        hc = symm.rendezvous(self.control, group_name)
        torch.cuda.synchronize(device)
        dist.barrier(group)           # everybody's words are zero before anybody signals
        self.exchange = make_exchange(self.world, self.rank, [int(p) for p in hp.buffer_ptrs],
                                      [int(p) for p in hc.buffer_ptrs])
        self._handles = (hp, hc)

    def step(self, ex: CudaExecutor, q, kShard, vShard, out, *, dtype: str, batch: int,
             shardRows: int, qHeads: int, kvHeads: int, headDim: int, kvLens=None,
             splits: int = 0):
        decode_batched(ex, q, out, kShard, vShard, dtype=dtype, batch=batch, cacheRows=shardRows,
                       qHeads=qHeads, kvHeads=kvHeads, headDim=headDim, kvLen=shardRows,
                       kvLens=kvLens, splits=splits, exchange=self.exchange)
        return out


class ShardedDecode:
    """KV-sequence-sharded decode.  ``partial_fn(out_partials)`` computes this
    rank's (m, l, acc) partials into a [units, 2+hd] f32 tensor; ``merge_fn
    (gathered, out)`` merges [world, units, 2+hd].  The exchange is one
    all-gather of ``units * (2+hd)`` floats per rank."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self._gathered = None

    def gather(self, partials):
        """All-gathers the ranks' partial tensors into [world, units, 2+hd]."""
        import torch
        if self._gathered is None or self._gathered.shape[1:] != partials.shape \
                or self._gathered.device != partials.device:
            self._gathered = torch.empty((self.world, *partials.shape), dtype=partials.dtype,
                                         device=partials.device)
        if self.world == 1:
            self._gathered[0].copy_(partials)
        else:
            # concatenation along dim 0 is the layout every backend accepts
            flat = self._gathered.view(self.world * partials.shape[0], *partials.shape[1:])
            self.dist.all_gather_into_tensor(flat, partials.contiguous(), group=self.group)
        return self._gathered

    def step(self, ex: CudaExecutor, q, kShard, vShard, out, *, dtype: str, batch: int,
             shardRows: int, qHeads: int, kvHeads: int, headDim: int, partials, kvLens=None,
             splits: int = 0):
        """Attends to this rank's rows, exchanges partials, merges into ``out``."""
        decode_batched(ex, q, None, kShard, vShard, dtype=dtype, batch=batch,
                       cacheRows=shardRows, qHeads=qHeads, kvHeads=kvHeads, headDim=headDim,
                       kvLen=shardRows, kvLens=kvLens, partialsOut=partials, splits=splits)
        gathered = self.gather(partials)
        merge_partials(ex, gathered, self.world, batch * qHeads, headDim, out, dtype)
        return out
