"""Host side of KV-sequence-sharded decode on CPU ranks (gloo, world size 2 and
3): the shard plan covers the sequence, the exchange is one all-gather of
(m, l, acc) partials, and merging them equals unsharded attention.  The
per-shard partials here come from plain numpy: only the plumbing is under
test, the kernels have their own GPU suite."""
import math
import os
import socket

import numpy as np
import pytest

import oracle
from runntime_b200.engine import shard_rows


def test_shard_rows_partition_the_sequence():
    for total in (1, 7, 8192, 8193):
        for world in (1, 2, 3, 8):
            spans = [shard_rows(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1


def _partials(q, k, v, heads, hd):
    """(m, l, acc) per head over the given rows, natural-log domain."""
    out = np.zeros((heads, 2 + hd), np.float32)
    for h in range(heads):
        if k.shape[0] == 0:
            out[h, 0] = -1e30
            continue
        s = k[:, h * hd:(h + 1) * hd].astype(np.float64) @ q[h * hd:(h + 1) * hd].astype(np.float64)
        m = s.max()
        p = np.exp(s - m)
        out[h, 0], out[h, 1] = m, p.sum()
        out[h, 2:] = p @ v[:, h * hd:(h + 1) * hd].astype(np.float64)
    return out


def _worker(rank, world, port, rows, result):
    import torch
    import torch.distributed as dist
    from runntime_b200.engine import ShardedDecode
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        batch, heads, hd = 3, 4, 8
        rng = np.random.default_rng(0)
        q = rng.standard_normal((batch, heads * hd)).astype(np.float32)
        k = rng.standard_normal((batch, rows, heads * hd)).astype(np.float32)
        v = rng.standard_normal((batch, rows, heads * hd)).astype(np.float32)
        sd = ShardedDecode()
        assert (sd.world, sd.rank) == (world, rank)
        s, e = shard_rows(rows, world, rank)
        mine = np.stack([_partials(q[b], k[b, s:e], v[b, s:e], heads, hd) for b in range(batch)])
        gathered = sd.gather(torch.from_numpy(mine.reshape(batch * heads, 2 + hd)))
        assert tuple(gathered.shape) == (world, batch * heads, 2 + hd)
        assert np.array_equal(gathered[rank].numpy(), mine.reshape(batch * heads, 2 + hd))
        got = oracle.merge_partials(gathered.numpy())
        for b in range(batch):
            want = oracle.sdpa_ref(q[b:b + 1], k[b], v[b], qHeads=heads, kvHeads=heads, headDim=hd)
            assert np.allclose(got.reshape(batch, -1)[b], want.reshape(-1), rtol=1e-5, atol=1e-6)
        result[rank] = 1
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,rows", [(2, 64), (3, 2)])
def test_sharded_decode_exchange_on_cpu_ranks(world, rows):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    result = ctx.Array("i", world)
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, rows, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert list(result) == [1] * world


def test_exchange_layout_of_buffers_and_control_words():
    """Sizes and addresses of the cross-GPU exchange (host arithmetic only)."""
    from runntime_b200.engine import exchange_sizes, make_exchange, owned_sequences
    world, batch, heads, hd = 4, 512, 8, 52
    nfloat, nword, nstage = exchange_sizes(world, batch, heads, hd)
    # a rank's buffer holds the rows of the 128 sequences it merges, from every rank, twice
    assert nfloat == 2 * world * 128 * heads * 54 and nword == 2 * world + 3
    assert nstage == batch * heads * 54
    bufs = [0x10000000 + r * 0x1000000 for r in range(world)]
    ctl = [0x90000000 + r * 0x100 for r in range(world)]
    x = make_exchange(world, 2, bufs, ctl, 0xA0000000)
    assert (x.world, x.rank) == (4, 2)
    assert [x.partials[r] for r in range(world)] == bufs and x.partials[4] is None
    assert [x.flags[r] for r in range(world)] == ctl
    assert x.step == ctl[2] + 4 * world and x.stage == 0xA0000000
    # every sequence has exactly one owner and every rank owns one (batch >= world)
    for batch, world in ((512, 8), (6, 4), (8, 8), (7, 3), (5, 5), (9, 8)):
        spans = [owned_sequences(batch, world, r) for r in range(world)]
        covered = [b for first, n in spans for b in range(first, first + n)]
        assert covered == list(range(batch)), (batch, world, spans)
        assert min(n for _, n in spans) >= 1 and max(n for _, n in spans) <= -(-batch // world)
    assert owned_sequences(6, 4, 3) == (5, 1)


def test_positions_map_to_one_rank_and_row():
    from runntime_b200.engine import shard_of_position
    for maxPositions, world in ((448, 2), (8192, 8), (194, 4), (7, 3)):
        shardRows = -(-maxPositions // world)
        seen = set()
        for t in range(maxPositions):
            r, row = shard_of_position(t, shardRows)
            assert 0 <= r < world and 0 <= row < shardRows and r * shardRows + row == t
            seen.add((r, row))
        assert len(seen) == maxPositions


def _append_worker(rank, world, port, result):
    """Each CPU rank keeps its shard of the caches as numpy arrays and appends the new
    token's row only when the position is its own — the host-side rule of
    ShardedKvCacheEngine; an all-gather of the shards must reproduce the whole cache."""
    import torch
    import torch.distributed as dist
    from runntime_b200.engine import shard_of_position
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        maxPositions, width, steps = 23, 6, 23
        shardRows = -(-maxPositions // world)
        shard = np.zeros((shardRows, width), np.float32)
        rng = np.random.default_rng(1)       # the same rows on every rank
        rows = rng.standard_normal((steps, width)).astype(np.float32)
        for t in range(steps):
            r, local = shard_of_position(t, shardRows)
            if r == rank:
                shard[local] = rows[t]
        gathered = [torch.zeros(shardRows, width) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(shard))
        whole = torch.cat(gathered).numpy()[:maxPositions]
        assert np.array_equal(whole, rows)
        result[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_append_ownership_on_cpu_ranks(world):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    result = ctx.Array("i", world)
    port = _free_port()
    procs = [ctx.Process(target=_append_worker, args=(r, world, port, result)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert list(result) == [1] * world
