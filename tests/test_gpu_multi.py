"""KV-sequence-sharded decode on two real GPUs (skipped on a one-GPU box): the
exchange of partials through peer memory against the NCCL all-gather form and
against the oracle over the whole, unsharded cache.  One process per GPU."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _gpus() -> int:
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0


def _worker(rank, world, port, result):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    os.environ.setdefault("NCCL_DEBUG", "WARN")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import oracle
    import runntime_b200 as rt
    from runntime_b200.engine import PeerExchangeDecode, ShardedDecode, shard_rows
    ex = rt.CudaExecutor(rank)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    batch, heads, kvHeads, hd, rows = 6, 8, 8, 52, 1500
    peer = PeerExchangeDecode(units=batch * heads, headDim=hd, device=dev)
    nccl = ShardedDecode()
    g = torch.Generator().manual_seed(4)          # same numbers on every rank
    worst_vs_nccl, worst_ok = 0.0, True
    try:
        for step in range(4):
            k = torch.randn(batch, rows, kvHeads * hd, generator=g).half()
            v = torch.randn(batch, rows, kvHeads * hd, generator=g).half()
            q = (torch.randn(batch, heads * hd, generator=g) / 7).half()
            s, e = shard_rows(rows, world, rank)
            ks, vs, qd = k[:, s:e].contiguous().to(dev), v[:, s:e].contiguous().to(dev), q.to(dev)
            out_p = torch.empty(batch, heads * hd, dtype=torch.float16, device=dev)
            out_n = torch.empty_like(out_p)
            part = torch.empty(batch * heads, 2 + hd, dtype=torch.float32, device=dev)
            common = dict(dtype="f16", batch=batch, shardRows=e - s, qHeads=heads, kvHeads=kvHeads,
                          headDim=hd)
            peer.step(ex, qd, ks, vs, out_p, **common)
            nccl.step(ex, qd, ks, vs, out_n, partials=part, **common)
            ex.sync()
            worst_vs_nccl = max(worst_vs_nccl, float((out_p.float() - out_n.float()).abs().max()))
            if rank == 0:
                for b in range(batch):
                    ref = oracle.sdpa_ref(q[b:b + 1].float().numpy(), k[b].float().numpy(),
                                          v[b].float().numpy(), qHeads=heads, kvHeads=kvHeads,
                                          headDim=hd).reshape(-1)
                    got = out_p[b].float().cpu().numpy()
                    worst_ok &= bool(np.all(np.abs(got - ref) <= 2e-3 + 4e-3 * np.abs(ref)))
        result[rank] = (worst_vs_nccl, worst_ok)
    finally:
        ex.setStream(None)
        ex.dispose()
        dist.barrier()
        dist.destroy_process_group()


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_peer_exchange_matches_nccl_and_oracle_on_two_gpus():
    import torch.multiprocessing as mp
    world = 2
    with mp.Manager() as m:
        result = m.dict()
        mp.spawn(_worker, args=(world, 29533, result), nprocs=world, join=True)
        assert len(result) == world
        for rank in range(world):
            diff, ok = result[rank]
            assert diff <= 1e-3, (rank, diff)     # same partials, merged in another order
            assert ok, rank
