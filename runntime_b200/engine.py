"""Batched entry points over the C ABI, for callers that hold many sequences:

- ``prefill_batched``: padded-batch prefill (``batch`` sequences of
  ``seqStride`` rows, per-sequence lengths) — the packed-segments form of the
  reference (packages/runntime/src/zoo/minilm/model.ts:167-185) computed on the
  fly from the lengths.
- ``decode_batched``: one decode step for ``batch`` KV caches with the append
  fused — the step of packages/runntime/src/zoo/moonshine/decoder.ts:58-76 for
  many sequences at once; ``KvCacheEngine`` keeps the caches and lengths like
  the transcriber does (transcriber.ts:111-118,161-203).
- ``PeerExchangeDecode`` / ``ShardedDecode``: long-context decode with the KV
  sequence split across ranks; each rank attends to its rows, the (m, l, acc)
  partials go to the rank that merges the sequence through peer memory, or are
  all-gathered by NCCL, and are merged (algebra of attnDecode.ts:405-422).
  ``ShardedKvCacheEngine`` is the KV-cache engine over caches sharded by position,
  ``ExchangeMemory`` the set-up of the peer buffers through the C ABI.

Tensors are passed as device pointers (ints) or as anything with
``data_ptr()`` (torch tensors).  torch is used only for device memory and
``torch.distributed``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

from ._lib import AttnArgs, DecodeArgs, DecodeSecond, DTYPE_CODE, Exchange, WINDOW_INF, check
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
                   kNewRowStride: int = 0, vNewRowStride: int = 0, exchange=None,
                   kvSharded: bool = False, shardStart: int = 0, kCachePtrs=None, vCachePtrs=None,
                   second=None) -> None:
    """One decode step for ``batch`` sequences; see rt_attn_decode in
    include/rt_attn.h.  ``kvLen`` is the (maximum) visible length including the
    appended row; ``kvLens`` gives it per sequence.  With ``ropeCos``/``ropeSin``
    q and kNew are un-rotated rows (for example windows of the fused qkv
    projection, ``*RowStride`` apart) and the kernel rotates them.
    ``kCachePtrs``/``vCachePtrs``: device int64 arrays [batch] of cache addresses, for
    caches allocated one by one (``kCache``/``vCache`` may then be None).  ``second``
    (from ``second_attention``): a cross-attention computed by the same launch."""
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
    d.kvSharded, d.shardStart = int(kvSharded), shardStart
    d.kCachePtrs, d.vCachePtrs = _ptr(kCachePtrs), _ptr(vCachePtrs)
    if second is not None:
        d.second = C.pointer(second)
    check(ex._lib.rt_attn_decode(ex.ctx, C.byref(d)), ex.ctx)


def second_attention(q, out, kCache, vCache, *, cacheRows: int, qHeads: int, kvHeads: int,
                     headDim: int, kvLen: int = 0, kvLens=None, windowLeft=None,
                     cacheSeqStride: Optional[int] = None, qRowStride: int = 0, kCachePtrs=None,
                     vCachePtrs=None) -> DecodeSecond:
    """The ``second`` argument of decode_batched: a cross-attention (no append, no rope)
    that shares the launch of a self-attention step — the two attentions of a decoder
    layer (packages/runntime/src/zoo/moonshine/decoder.ts:58-76, 105-109) in one kernel."""
    x = DecodeSecond()
    x.q, x.out = _ptr(q), _ptr(out)
    x.kCache, x.vCache = _ptr(kCache), _ptr(vCache)
    x.kCachePtrs, x.vCachePtrs = _ptr(kCachePtrs), _ptr(vCachePtrs)
    x.kvLens = _ptr(kvLens)
    x.cacheSeqStride = (cacheRows * kvHeads * headDim) if cacheSeqStride is None else cacheSeqStride
    x.qRowStride = qRowStride
    x.cacheRows, x.kvLen, x.windowLeft = cacheRows, (kvLen or cacheRows), _win(windowLeft)
    return x


def merge_partials(ex: CudaExecutor, partials, parts: int, units: int, headDim: int, out,
                   dtype: str) -> None:
    check(ex._lib.rt_attn_merge_partials(ex.ctx, C.c_void_p(_ptr(partials)), parts, units,
                                         headDim, C.c_void_p(_ptr(out)), DTYPE_CODE[dtype]),
          ex.ctx)


class KvCacheEngine:
    """Preallocated self-attention caches for ``batch`` sequences plus their
    lengths, stepped one token at a time: append + causal attend in one kernel.
    Optionally a fixed cross-attention K/V (encoder states) per sequence.  The
    lengths are advanced by torch and read by the library's kernels, so every
    step binds the executor to torch's current stream first."""

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
        _bind_to_torch_stream(self.ex)
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
        _bind_to_torch_stream(self.ex)
        self._advance()
        decode_batched(self.ex, q, out, self.k, self.v, dtype=self.dtype, batch=self.batch,
                       cacheRows=self.maxPositions, qHeads=self.qHeads, kvHeads=self.kvHeads,
                       headDim=self.headDim, kvLen=self.maxLen, kvLens=self.lens, kNew=kNew,
                       vNew=vNew, windowLeft=self.windowLeft)

    def stepWithCross(self, q, kNew, vNew, out, qCross, outCross) -> None:
        """The self-attention step (append + causal attend) and the cross-attention over
        the encoder states set by setCross, in one launch."""
        k, v, rows = self.cross
        _bind_to_torch_stream(self.ex)
        self._advance()
        sec = second_attention(qCross, outCross, k, v, cacheRows=rows, qHeads=self.qHeads,
                               kvHeads=self.kvHeads, headDim=self.headDim, kvLen=rows)
        decode_batched(self.ex, q, out, self.k, self.v, dtype=self.dtype, batch=self.batch,
                       cacheRows=self.maxPositions, qHeads=self.qHeads, kvHeads=self.kvHeads,
                       headDim=self.headDim, kvLen=self.maxLen, kvLens=self.lens, kNew=kNew,
                       vNew=vNew, windowLeft=self.windowLeft, second=sec)

    def crossAttend(self, q, out) -> None:
        k, v, rows = self.cross
        _bind_to_torch_stream(self.ex)
        decode_batched(self.ex, q, out, k, v, dtype=self.dtype, batch=self.batch, cacheRows=rows,
                       qHeads=self.qHeads, kvHeads=self.kvHeads, headDim=self.headDim, kvLen=rows)


def shard_rows(total: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows [start, end) of a ``total``-row KV sequence that live on ``rank``:
    contiguous, balanced to within one row."""
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_of_position(position: int, shardRows: int) -> Tuple[int, int]:
    """(rank, local row) of a token position when every rank's cache holds
    ``shardRows`` consecutive positions: position t lives on rank t // shardRows."""
    return position // shardRows, position % shardRows


def owned_sequences(batch: int, world: int, rank: int) -> Tuple[int, int]:
    """(first, count) of the sequences whose partials ``rank`` merges in the cross-GPU
    exchange: contiguous blocks balanced to within one sequence (batch >= world, so
    every rank owns at least one)."""
    first, end = shard_rows(batch, world, rank)
    return first, end - first


def exchange_sizes(world: int, batch: int, qHeads: int, headDim: int) -> Tuple[int, int, int]:
    """(floats of a rank's exchange buffer, 32-bit words of its control block, floats of
    its staging buffer): two halves of [world, per * qHeads, 2+headDim] partials for the
    ``per`` sequences it owns; [world] arrival words + [world + 3] counters; the rank's own
    [batch * qHeads, 2+headDim] rows before they go to their owners."""
    per = -(-batch // world)
    row = 2 + headDim
    return 2 * world * per * qHeads * row, 2 * world + 3, batch * qHeads * row


def make_exchange(world: int, rank: int, partialPtrs, controlPtrs, stagePtr) -> Exchange:
    """rt_exchange over every rank's exchange buffer and control block as mapped in
    this process (``controlPtrs[r]``: rank r's [world] arrival words, then its counters,
    all zero at the start) and this rank's staging buffer."""
    x = Exchange()
    x.world, x.rank = world, rank
    for r in range(world):
        x.partials[r] = _ptr(partialPtrs[r])
        x.flags[r] = _ptr(controlPtrs[r])
    x.step = _ptr(controlPtrs[rank]) + 4 * world
    x.stage = _ptr(stagePtr)
    return x


class ExchangeMemory:
    """A rank's exchange block allocated and mapped through the C ABI (rt_xmem_*):
    what a host without torch.distributed uses.  Processes trade ``export()`` handles
    (64 bytes) and ``importHandle`` them; ranks living in one process ``attach`` each
    other's objects."""

    def __init__(self, device: int, world: int, rank: int, batch: int, qHeads: int,
                 headDim: int):
        from . import _lib
        self._lib = _lib.load()
        h = C.c_void_p()
        check(self._lib.rt_xmem_create(device, world, rank, batch, qHeads, headDim, C.byref(h)))
        self._h, self.world, self.rank = h, world, rank

    def export(self) -> bytes:
        from ._lib import XMEM_HANDLE_BYTES
        buf = C.create_string_buffer(XMEM_HANDLE_BYTES)
        check(self._lib.rt_xmem_export(self._h, buf))
        return buf.raw

    def importHandle(self, peer: int, handle: bytes) -> None:
        check(self._lib.rt_xmem_import(self._h, peer, C.create_string_buffer(handle, len(handle))))

    def attach(self, peer: int, other: "ExchangeMemory") -> None:
        check(self._lib.rt_xmem_attach(self._h, peer, other._h))

    def exchange(self) -> Exchange:
        x = Exchange()
        check(self._lib.rt_xmem_exchange(self._h, C.byref(x)))
        return x

    def destroy(self) -> None:
        if self._h is not None:
            check(self._lib.rt_xmem_destroy(self._h))
            self._h = None


def _bind_to_torch_stream(ex: CudaExecutor) -> None:
    """The engines mix torch work (length updates, collectives) with the library's
    kernels: both must be on one stream, so the executor is bound to torch's current
    stream before every step (a context's own stream is non-blocking and would not be
    ordered with torch's)."""
    import torch
    ex.setStream(torch.cuda.current_stream().cuda_stream)


class PeerExchangeDecode:
    """KV-sequence-sharded decode whose ranks trade partials through peer memory:
    the decode kernel sends each sequence's (m, l, acc) rows to the rank that owns the
    sequence and signals it; that rank's merge kernel waits for all ranks' rows of the
    step and merges — no library collective on the step.  ``out`` receives the rows of
    this rank's own sequences (``self.first``, ``self.owned``).  One process per GPU;
    the buffers come from torch's symmetric memory (``transport="symm"``) or from the
    library's own CUDA-IPC set-up (``transport="ipc"``, handles carried by
    ``all_gather_object``).  Kernels run on torch's current stream."""

    def __init__(self, *, batch: int, qHeads: int, headDim: int, device, group=None,
                 transport: str = "symm"):
        import os
        import torch
        import torch.distributed as dist
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.first, self.owned = owned_sequences(batch, self.world, self.rank)
        self.transport = transport
        if transport == "ipc":
            index = device.index if device.index is not None else torch.cuda.current_device()
            self.mem = ExchangeMemory(index, self.world, self.rank, batch, qHeads, headDim)
            handles = [None] * self.world
            dist.all_gather_object(handles, self.mem.export(), group=group)
            for r, h in enumerate(handles):
                if r != self.rank:
                    self.mem.importHandle(r, h)
            self.exchange = self.mem.exchange()
            dist.barrier(group)       # every block is mapped (and zero) before anybody signals
            return
        # plain peer mappings only: no NVLink multicast object is bound to these buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm
        nfloat, nword, nstage = exchange_sizes(self.world, batch, qHeads, headDim)
        group_name = (group or dist.group.WORLD).group_name
        self.partials = symm.empty(nfloat, dtype=torch.float32, device=device)
        self.control = symm.empty(nword, dtype=torch.int32, device=device)
        self.stage = torch.zeros(nstage, dtype=torch.float32, device=device)
        self.partials.zero_()
        self.control.zero_()
        hp = symm.rendezvous(self.partials, group_name)
        hc = symm.rendezvous(self.control, group_name)
        torch.cuda.synchronize(device)
        dist.barrier(group)           # everybody's words are zero before anybody signals
        self.exchange = make_exchange(self.world, self.rank, [int(p) for p in hp.buffer_ptrs],
                                      [int(p) for p in hc.buffer_ptrs], self.stage)
        self._handles = (hp, hc)

    def step(self, ex: CudaExecutor, q, kShard, vShard, out, *, dtype: str, batch: int,
             shardRows: int, qHeads: int, kvHeads: int, headDim: int, kvLens=None,
             kvLen: Optional[int] = None, kNew=None, vNew=None, shardStart: Optional[int] = None,
             splits: int = 0):
        """One step over this rank's rows.  Without ``shardStart`` the shard is a static
        slab of ``shardRows`` visible rows (``kvLens``: local lengths).  With it the caches
        are sharded by position — this rank holds global rows [shardStart, shardStart +
        shardRows) — ``kvLen``/``kvLens`` are global lengths and ``kNew``/``vNew`` are
        appended by the rank that owns the new position."""
        _bind_to_torch_stream(ex)
        sharded = shardStart is not None
        decode_batched(ex, q, out, kShard, vShard, dtype=dtype, batch=batch, cacheRows=shardRows,
                       qHeads=qHeads, kvHeads=kvHeads, headDim=headDim,
                       kvLen=(kvLen if kvLen is not None else shardRows), kvLens=kvLens,
                       kNew=kNew, vNew=vNew, splits=splits, exchange=self.exchange,
                       kvSharded=sharded, shardStart=shardStart or 0)
        return out


class ShardedKvCacheEngine:
    """The KV-cache engine with every sequence's cache split by position over the ranks
    of an exchange: rank r keeps positions [r*shardRows, (r+1)*shardRows) of all
    ``batch`` sequences (shardRows = ceil(maxPositions / world)).  A step appends the
    new token's K/V row on the rank that owns its position — the others attend without
    it — and merges the ranks' partials; ``out`` receives this rank's own sequences.
    The decoder loop it serves: packages/runntime/src/zoo/moonshine/transcriber.ts:
    111-118,161-203 (caches preallocated per layer, one writeRows + attention per step).
    Kernels run on torch's current stream."""

    def __init__(self, ex: CudaExecutor, exchange: Exchange, *, batch: int, maxPositions: int,
                 qHeads: int, kvHeads: int, headDim: int, dtype: str = "f16", device=None):
        import torch
        self.ex, self.exchange, self.batch = ex, exchange, batch
        self.world, self.rank = exchange.world, exchange.rank
        self.maxPositions = maxPositions
        self.shardRows = -(-maxPositions // self.world)
        self.shardStart = self.rank * self.shardRows
        self.qHeads, self.kvHeads, self.headDim, self.dtype = qHeads, kvHeads, headDim, dtype
        dev = device if device is not None else torch.device("cuda", ex.device)
        tdt = torch.float16 if dtype == "f16" else torch.float32
        kvw = kvHeads * headDim
        self.k = torch.zeros(batch, self.shardRows, kvw, dtype=tdt, device=dev)
        self.v = torch.zeros(batch, self.shardRows, kvw, dtype=tdt, device=dev)
        self.lens = torch.zeros(batch, dtype=torch.int32, device=dev)   # global lengths
        self.maxLen = 0
        self.first, self.owned = owned_sequences(batch, self.world, self.rank)

    def step(self, q, kNew, vNew, out, *, phases: int = 0) -> None:
        """Appends kNew/vNew [batch, kvHeads*headDim] at each sequence's end (on the rank
        that owns that position) and attends causally over all ranks' rows."""
        _bind_to_torch_stream(self.ex)
        if phases in (0, 1, 3):
            if self.maxLen + 1 > self.maxPositions:
                raise ValueError(
                    f"writeRows: rows [{self.maxLen}, {self.maxLen + 1}) exceed dst capacity "
                    f"{self.maxPositions}")
            self.lens.add_(1)
            self.maxLen += 1
        self.exchange.phases = phases
        decode_batched(self.ex, q, out, self.k, self.v, dtype=self.dtype, batch=self.batch,
                       cacheRows=self.shardRows, qHeads=self.qHeads, kvHeads=self.kvHeads,
                       headDim=self.headDim, kvLen=self.maxLen, kvLens=self.lens, kNew=kNew,
                       vNew=vNew, exchange=self.exchange, kvSharded=True,
                       shardStart=self.shardStart)


class ShardedDecode:
    """KV-sequence-sharded decode.  ``partial_fn(out_partials)`` computes this
    rank's (m, l, acc) partials into a [units, 2+hd] f32 tensor; ``merge_fn
    (gathered, out)`` merges [world, units, 2+hd].  The exchange is one
    all-gather of ``units * (2+hd)`` floats per rank.  The library's kernels and
    the collective run on torch's current stream."""

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
             kvLen: Optional[int] = None, kNew=None, vNew=None, shardStart: Optional[int] = None,
             splits: int = 0):
        """Attends to this rank's rows, exchanges partials, merges into ``out`` (every
        rank gets every sequence).  ``shardStart``/``kvLen``/``kNew``/``vNew``: the
        position-sharded form with append, as in PeerExchangeDecode.step."""
        _bind_to_torch_stream(ex)
        sharded = shardStart is not None
        decode_batched(ex, q, None, kShard, vShard, dtype=dtype, batch=batch,
                       cacheRows=shardRows, qHeads=qHeads, kvHeads=kvHeads, headDim=headDim,
                       kvLen=(kvLen if kvLen is not None else shardRows), kvLens=kvLens, kNew=kNew,
                       vNew=vNew, partialsOut=partials, splits=splits, kvSharded=sharded,
                       shardStart=shardStart or 0)
        gathered = self.gather(partials)
        merge_partials(ex, gathered, self.world, batch * qHeads, headDim, out, dtype)
        return out
