#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5|c4|c3|c2|c1]
    python bench.py --workload rope|softmax|local|step|layer|gemv|gemm|argmax   # the operators beside attention
    python bench.py --impl reference ...        # the CPU restatement, host cores

One JSON line on stdout (rank 0).  The default workload is the large causal
prefill (batch 64 x seq 8192 x 8 heads x 128, f16), reported as TFLOP/s against
the measured tensor-core peak; the long-context decode (batch 512, KV 8192,
8 x 52, f16) rides along under "decode" as HBM GB/s against the measured copy
bandwidth.  Work is counted algorithmically: 4*hd FLOPs per visible
(query, key) pair per query head for prefill; visible K and V rows + q + out for
decode.  Inputs are seeded synthetic tensors of the named shapes.

With N > 1 (torchrun, one rank per GPU) the total work is fixed and sharded:
prefill by sequences with no collective; decode by KV rows with one NCCL
all-gather of (m, l, acc) partials and a merge.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p["bf16_tflops"],
                    tflops_sustained=p.get("bf16_tflops_sustained"), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


def load_traffic():
    """Per-launch DRAM traffic figures taken from committed ncu captures."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    return json.load(open(path)) if os.path.exists(path) else {}


# ----------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------

CONFIGS = {
    "c1": dict(kind="prefill", name="minilm_bidirectional_f32", dtype="f32", batch=8, seq=128,
               qHeads=12, kvHeads=12, hd=32, lens=(16, 128), wl=None, wr=None, sigma=1.0,
               fold=32 ** -0.25, layers=6),
    "c3": dict(kind="prefill", name="embeddinggemma_gqa_prefill_f16", dtype="f16", batch=32,
               seq=2048, qHeads=3, kvHeads=1, hd=256, lens=(512, 2048), wl=512, wr=512, sigma=0.5,
               fold=1.0, layers=6),
    "c5": dict(kind="prefill", name="causal_prefill_f16_b64_s8192_h8_d128", dtype="f16", batch=64,
               seq=8192, qHeads=8, kvHeads=8, hd=128, lens=None, wl=None, wr=0, sigma=1.0,
               fold=128 ** -0.25, layers=1),
    "c2": dict(kind="decode", name="moonshine_tiny_decode_step_f16", dtype="f16", batch=64,
               cacheRows=448, qHeads=8, kvHeads=8, hd=36, lens=(1, 448), cross=200),
    "c4": dict(kind="decode", name="moonshine_base_long_decode_f16_b512_kv8192", dtype="f16",
               batch=512, cacheRows=8192, qHeads=8, kvHeads=8, hd=52, lens=None, cross=0),
}


def visible_pairs(L, wl, wr):
    """Visible (query, key) pairs of one sequence of length L under a window."""
    if wl is None and wr is None:
        return L * L
    total = 0
    lo_w = L if wl is None else wl
    hi_w = L if wr is None else wr
    # sum over i of (min(i+hi_w, L-1) - max(i-lo_w, 0) + 1), closed form by loop (L <= 8192)
    for i in range(L):
        total += min(i + hi_w, L - 1) - max(i - lo_w, 0) + 1
    return total


class Prefill:
    def __init__(self, cfg, rank, world, ex, layer=0):
        import torch
        self.cfg, self.ex, self.torch = cfg, ex, torch
        b = cfg["batch"]
        per = b // world if b % world == 0 else -(-b // world)
        self.b0, self.b1 = min(rank * per, b), min((rank + 1) * per, b)
        self.nb = self.b1 - self.b0
        S, hd = cfg["seq"], cfg["hd"]
        dev = torch.device("cuda", torch.cuda.current_device())
        tdt = torch.float16 if cfg["dtype"] == "f16" else torch.float32
        gl = torch.Generator(device="cpu").manual_seed(4242 + layer)
        if cfg["lens"]:
            lens = torch.randint(cfg["lens"][0], cfg["lens"][1] + 1, (b,), generator=gl)
        else:
            lens = torch.full((b,), S, dtype=torch.int64)
        self.lens_all = lens.tolist()
        self.lens = lens[self.b0:self.b1].to(torch.int32).to(dev)
        gd = torch.Generator(device=dev).manual_seed(1000 + 17 * rank + layer)
        rows = max(self.nb, 1) * S
        f = cfg["fold"] * cfg["sigma"]
        self.q = (torch.randn(rows, cfg["qHeads"] * hd, generator=gd, device=dev) * f).to(tdt)
        self.k = (torch.randn(rows, cfg["kvHeads"] * hd, generator=gd, device=dev) * f).to(tdt)
        self.v = (torch.randn(rows, cfg["kvHeads"] * hd, generator=gd, device=dev)
                  * cfg["sigma"]).to(tdt)
        self.out = torch.empty_like(self.q)
        self.layers = cfg["layers"]

    def windows(self, layer):
        c = self.cfg
        if c["name"].startswith("embeddinggemma") and layer % 6 == 5:
            return None, None  # every sixth layer is global
        return c["wl"], c["wr"]

    def flops(self, layer=0, all_ranks=True):
        c = self.cfg
        wl, wr = self.windows(layer)
        lens = self.lens_all if all_ranks else self.lens_all[self.b0:self.b1]
        cache = {}
        pairs = 0
        for L in lens:
            if L not in cache:
                cache[L] = visible_pairs(L, wl, wr)
            pairs += cache[L]
        return 4.0 * c["hd"] * pairs * c["qHeads"]

    def step(self, layer=0):
        from runntime_b200.engine import prefill_batched
        c = self.cfg
        if self.nb == 0:
            return
        self.ex.setStream(self.torch.cuda.current_stream().cuda_stream)
        wl, wr = self.windows(layer)
        prefill_batched(self.ex, self.q, self.k, self.v, self.out, dtype=c["dtype"], batch=self.nb,
                        seqStride=c["seq"], seqLens=self.lens, qHeads=c["qHeads"],
                        kvHeads=c["kvHeads"], headDim=c["hd"], windowLeft=wl, windowRight=wr)

    def io_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.q, self.k, self.v)), \
            self.out.numel() * self.out.element_size()

    def verify(self):
        """Runs every distinct layer once and checks a sample of output rows of this rank's
        first and last sequences against the f64 oracle (a row's output depends only on that
        row's q, so the sample is exact for the rows it covers).  Returns (worst absolute
        error, rows checked, all within tolerance)."""
        import numpy as np
        import oracle
        c, S, t = self.cfg, self.cfg["seq"], self.torch
        if self.nb == 0:
            return 0.0, 0, True
        worst, nrows, ok = 0.0, 0, True
        tol = oracle.TOLERANCE[c["dtype"]]
        layers = sorted({0, self.layers - 1})
        for layer in layers:
            self.out.fill_(7.0)
            self.step(layer)
            t.cuda.synchronize()
            wl, wr = self.windows(layer)
            for b in sorted({0, self.nb - 1}):
                L = int(self.lens_all[self.b0 + b])
                q, k, v = (x[b * S:b * S + L].float().cpu().numpy() for x in (self.q, self.k, self.v))
                got = self.out[b * S:(b + 1) * S].float().cpu().numpy()
                rows = sorted({0, 1, L // 3, L // 2, L - 129 if L > 129 else 0, L - 2 if L > 1 else 0, L - 1}
                              | {r for r in (127, 128, 255, 256, 511, 512, 513) if r < L})
                for r in rows:
                    hi = L if wr is None else min(L, r + wr + 1)   # keys past the band are never read
                    want = oracle.sdpa_ref(q[r:r + 1], k[:hi], v[:hi], qHeads=c["qHeads"],
                                           kvHeads=c["kvHeads"], headDim=c["hd"],
                                           windowLeft=math.inf if wl is None else wl,
                                           windowRight=math.inf if wr is None else wr,
                                           qPosOffset=r).reshape(-1)
                    err = np.abs(got[r] - want)
                    worst = max(worst, float(err.max()))
                    ok &= bool(np.all(err <= tol["atol"] + tol["rtol"] * np.abs(want)))
                    nrows += 1
                ok &= bool((got[L:] == 0).all())     # rows past the length are zeros
        return worst, nrows, ok

    def make_host(self):
        t = self.torch
        self.hq, self.hk, self.hv = (x.cpu().pin_memory() for x in (self.q, self.k, self.v))
        self.hout = t.empty(self.out.shape, dtype=self.out.dtype).pin_memory()

    def e2e_step(self, layer=0):
        """Host buffers in, host buffer out, pipelined over groups of sequences: the
        upload of group g+1, the attention of group g and the download of group g-1 run
        on three streams (the two PCIe directions and the SMs work at the same time)."""
        from runntime_b200.engine import prefill_batched
        t, c = self.torch, self.cfg
        if self.nb == 0:
            return
        per = 8 if self.nb >= 16 else self.nb        # sequences per group
        if not hasattr(self, "_streams"):
            self._streams = (t.cuda.Stream(), t.cuda.Stream(), t.cuda.Stream())
        up, run, down = self._streams
        main = t.cuda.current_stream()
        for st in self._streams:
            st.wait_stream(main)
        wl, wr = self.windows(layer)
        S = c["seq"]
        for b0 in range(0, self.nb, per):
            b1 = min(b0 + per, self.nb)
            r0, r1 = b0 * S, b1 * S
            with t.cuda.stream(up):
                self.q[r0:r1].copy_(self.hq[r0:r1], non_blocking=True)
                self.k[r0:r1].copy_(self.hk[r0:r1], non_blocking=True)
                self.v[r0:r1].copy_(self.hv[r0:r1], non_blocking=True)
            run.wait_stream(up)
            with t.cuda.stream(run):
                self.ex.setStream(run.cuda_stream)
                prefill_batched(self.ex, self.q[r0:r1], self.k[r0:r1], self.v[r0:r1], self.out[r0:r1],
                                dtype=c["dtype"], batch=b1 - b0, seqStride=S,
                                seqLens=self.lens[b0:b1], qHeads=c["qHeads"],
                                kvHeads=c["kvHeads"], headDim=c["hd"], windowLeft=wl,
                                windowRight=wr)
            down.wait_stream(run)
            with t.cuda.stream(down):
                self.hout[r0:r1].copy_(self.out[r0:r1], non_blocking=True)
        self.ex.setStream(main.cuda_stream)
        main.wait_stream(down)


class Decode:
    def __init__(self, cfg, rank, world, ex):
        import torch
        from runntime_b200.engine import ShardedDecode
        self.cfg, self.ex, self.torch, self.world, self.rank = cfg, ex, torch, world, rank
        dev = torch.device("cuda", torch.cuda.current_device())
        self.dev = dev
        b, hd, H = cfg["batch"], cfg["hd"], cfg["kvHeads"]
        w = H * hd
        self.shard_kv = cfg["lens"] is None  # long-context: split KV rows across ranks
        gl = torch.Generator(device="cpu").manual_seed(77)
        self.b0 = 0
        if self.shard_kv:
            # every rank holds positions [rank*rows, (rank+1)*rows) of every sequence
            self.rows = -(-cfg["cacheRows"] // world)
            self.shardStart = rank * self.rows
            self.b = b
            self.lens_all = [cfg["cacheRows"]] * b
            self.lens = torch.full((b,), cfg["cacheRows"], dtype=torch.int32, device=dev)
        else:
            per = -(-b // world)
            b0, b1 = min(rank * per, b), min((rank + 1) * per, b)
            self.b0, self.b = b0, b1 - b0
            lens = torch.randint(cfg["lens"][0], cfg["lens"][1] + 1, (b,), generator=gl)
            self.lens_all = lens.tolist()
            self.lens_mine = self.lens_all[b0:b1]
            self.lens = lens[b0:b1].to(torch.int32).to(dev)
            self.rows = cfg["cacheRows"]
            self.shardStart = 0
        gd = torch.Generator(device=dev).manual_seed(2000 + rank)
        nb = max(self.b, 1)
        self.k = torch.randn(nb, self.rows, w, generator=gd, device=dev, dtype=torch.float16)
        self.v = torch.randn(nb, self.rows, w, generator=gd, device=dev, dtype=torch.float16)
        gq = torch.Generator(device=dev).manual_seed(3000)  # q and the new row: the same on every rank
        self.q = (torch.randn(cfg["batch"], cfg["qHeads"] * hd, generator=gq, device=dev)
                  * hd ** -0.5).to(torch.float16)[self.b0:self.b0 + nb].contiguous()
        self.kNew = torch.randn(cfg["batch"], w, generator=gq, device=dev,
                                dtype=torch.float16)[self.b0:self.b0 + nb].contiguous()
        self.vNew = torch.randn(cfg["batch"], w, generator=gq, device=dev,
                                dtype=torch.float16)[self.b0:self.b0 + nb].contiguous()
        self.out = torch.zeros_like(self.q)
        if cfg["cross"]:
            self.ck = torch.randn(nb, cfg["cross"], w, generator=gd, device=dev, dtype=torch.float16)
            self.cv = torch.randn(nb, cfg["cross"], w, generator=gd, device=dev, dtype=torch.float16)
            self.q2 = (torch.randn(nb, cfg["qHeads"] * hd, generator=gd, device=dev)
                       * hd ** -0.5).to(torch.float16)      # the cross-attention's own projection
            self.out2 = torch.empty_like(self.q)
        # KV rows split over ranks: the partials are traded through peer memory by the decode
        # kernel itself (--exchange peer, the default; the peers' blocks mapped through the
        # library's own CUDA-IPC set-up, or torch's symmetric memory if that fails) or by one
        # NCCL all-gather (--exchange nccl, also the last fallback).
        self.sharded = self.peer = None
        self.exchange = "none"
        if self.shard_kv and world > 1:
            if cfg.get("exchange", "peer") == "peer":
                from runntime_b200.engine import PeerExchangeDecode
                import torch.distributed as dist
                for transport in ("ipc", "symm"):
                    try:
                        peer = PeerExchangeDecode(batch=nb, qHeads=cfg["qHeads"], headDim=hd,
                                                  device=dev, transport=transport)
                    except Exception as e:  # noqa: BLE001 - any set-up failure: next transport
                        sys.stderr.write(f"rank {rank}: peer exchange over {transport} unavailable "
                                         f"({type(e).__name__}: {e})\n")
                        peer = None
                    agreed = torch.tensor([1 if peer is not None else 0], device=dev)
                    dist.all_reduce(agreed, op=dist.ReduceOp.MIN)     # all ranks or none
                    if int(agreed.item()):
                        self.peer = peer
                        self.exchange = ("peer memory (CUDA IPC), rows sent by the decode kernel to "
                                         "the rank that merges the sequence" if transport == "ipc" else
                                         "peer memory (torch symmetric memory), rows sent by the decode "
                                         "kernel to the rank that merges the sequence")
                        break
            if self.peer is None:
                self.sharded = ShardedDecode()
                self.exchange = "one NCCL all-gather"
        self.partials = (torch.empty(nb * cfg["qHeads"], 2 + hd, dtype=torch.float32, device=dev)
                         if self.sharded else None)

    def bytes(self, all_ranks=True):
        c = self.cfg
        es = 2
        w = c["kvHeads"] * c["hd"]
        qo = 2 * c["qHeads"] * c["hd"] * es
        lens = self.lens_all if (all_ranks or self.shard_kv) else self.lens_mine
        total = 0
        for L in lens:
            total += 2 * L * w * es + qo
            total += 2 * w * es          # appended K/V row write
            if c["cross"]:
                total += 2 * c["cross"] * w * es + qo
        if self.shard_kv and not all_ranks:
            total = total * self.rows / c["cacheRows"]
        return float(total)


    def step(self, layer=0):
        from runntime_b200.engine import decode_batched
        c = self.cfg
        if self.b == 0:
            return
        self.ex.setStream(self.torch.cuda.current_stream().cuda_stream)   # also inside a graph capture
        common = dict(dtype="f16", batch=self.b, qHeads=c["qHeads"], kvHeads=c["kvHeads"],
                      headDim=c["hd"])
        if self.peer:
            self.peer.step(self.ex, self.q, self.k, self.v, self.out, shardRows=self.rows,
                           kvLens=self.lens, kvLen=c["cacheRows"], kNew=self.kNew, vNew=self.vNew,
                           shardStart=self.shardStart, **common)
            return
        if self.sharded:
            self.sharded.step(self.ex, self.q, self.k, self.v, self.out, shardRows=self.rows,
                              partials=self.partials, kvLens=self.lens, kvLen=c["cacheRows"],
                              kNew=self.kNew, vNew=self.vNew, shardStart=self.shardStart, **common)
            return
        # self-attention with the append and, where the step has one, the cross-attention
        # over the encoder states: one launch
        second = None
        if c["cross"]:
            from runntime_b200.engine import second_attention
            second = second_attention(self.q2, self.out2, self.ck, self.cv, cacheRows=c["cross"],
                                      qHeads=c["qHeads"], kvHeads=c["kvHeads"], headDim=c["hd"],
                                      kvLen=c["cross"])
        decode_batched(self.ex, self.q, self.out, self.k, self.v, cacheRows=self.rows,
                       kvLen=max(self.lens_all), kvLens=self.lens, kNew=self.kNew, vNew=self.vNew,
                       splits=int(os.environ.get("RT_BENCH_SPLITS", "0")), second=second, **common)

    def verify(self):
        """One step, then a few sequences against the f64 oracle over their whole caches
        (gathered from the ranks when the KV rows are sharded; the appended row included).
        Each rank checks sequences whose output it holds.  Returns (worst absolute error,
        sequences checked, all within tolerance) over this rank."""
        import numpy as np
        import oracle
        t, c = self.torch, self.cfg
        if self.b == 0:
            return 0.0, 0, True
        self.out.fill_(7.0)
        self.step()
        t.cuda.synchronize()
        H, hd = c["qHeads"], c["hd"]
        tol = oracle.TOLERANCE["f16"]
        sample = sorted({0, self.b // 2, self.b - 1})
        if self.shard_kv and self.world > 1:
            import torch.distributed as dist
            idx = t.tensor(sample, device=self.dev)
            parts_k = [t.empty(len(sample), self.rows, self.k.shape[2], dtype=self.k.dtype, device=self.dev)
                       for _ in range(self.world)]
            parts_v = [t.empty_like(parts_k[0]) for _ in range(self.world)]
            dist.all_gather(parts_k, self.k[idx].contiguous())
            dist.all_gather(parts_v, self.v[idx].contiguous())
            kk = t.cat(parts_k, dim=1)[:, :c["cacheRows"]]
            vv = t.cat(parts_v, dim=1)[:, :c["cacheRows"]]
        else:
            kk, vv = self.k[sample], self.v[sample]
        if self.peer:
            mine = range(self.peer.first, self.peer.first + self.peer.owned)
        else:
            mine = range(self.b)
        worst, n, ok = 0.0, 0, True
        for i, b in enumerate(sample):
            L = int(self.lens_all[self.b0 + b]) if not self.shard_kv else c["cacheRows"]
            kb, vb = kk[i, :L].float().cpu().numpy(), vv[i, :L].float().cpu().numpy()
            # the step appended this sequence's new row at position L-1
            ok &= bool(np.array_equal(kb[L - 1], self.kNew[b].float().cpu().numpy()))
            if b not in mine:
                continue
            want = oracle.sdpa_ref(self.q[b:b + 1].float().cpu().numpy(), kb, vb, qHeads=H,
                                   kvHeads=c["kvHeads"], headDim=hd).reshape(-1)
            err = np.abs(self.out[b].float().cpu().numpy() - want)
            worst = max(worst, float(err.max()))
            ok &= bool(np.all(err <= tol["atol"] + tol["rtol"] * np.abs(want)))
            n += 1
            if c["cross"]:
                want = oracle.sdpa_ref(self.q2[b:b + 1].float().cpu().numpy(),
                                       self.ck[b].float().cpu().numpy(), self.cv[b].float().cpu().numpy(),
                                       qHeads=H, kvHeads=c["kvHeads"], headDim=hd).reshape(-1)
                err = np.abs(self.out2[b].float().cpu().numpy() - want)
                worst = max(worst, float(err.max()))
                ok &= bool(np.all(err <= tol["atol"] + tol["rtol"] * np.abs(want)))
        return worst, n, ok

    def io_bytes(self):
        n = self.q.numel() * 2
        if self.kNew is not None:
            n += 2 * self.kNew.numel() * 2
        return n, self.out.numel() * 2

    def make_host(self):
        # A decode step's inputs are the new token's q and K/V row; the cache is
        # device-resident state, as it is in the reference's decoder loop.
        self.hq = self.q.cpu().pin_memory()
        self.hout = self.torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory()
        self.hkn, self.hvn = self.kNew.cpu().pin_memory(), self.vNew.cpu().pin_memory()

    def e2e_step(self, layer=0):
        self.q.copy_(self.hq, non_blocking=True)
        self.kNew.copy_(self.hkn, non_blocking=True)
        self.vNew.copy_(self.hvn, non_blocking=True)
        self.step(layer)
        self.hout.copy_(self.out, non_blocking=True)


# ----------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------

class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
                power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------
# CPU baseline (the oracle's shader-order f32 loop on the host cores)
# ----------------------------------------------------------------------------

def cpu_sample(key, budget_s=12.0):
    """Times the CPU restatement on a bounded slice of the workload and returns
    (metric value, cores, description).  This is the one place the benchmark
    executes oracle code, and only as the reported CPU baseline."""
    import numpy as np
    import oracle
    cfg = CONFIGS[key]
    rng = np.random.default_rng(5)
    cores = oracle.num_threads()
    if cfg["kind"] == "prefill":
        hd = cfg["hd"]
        npdt = np.float16 if cfg["dtype"] == "f16" else np.float32
        if key == "c5":
            S, heads = 2048, 1
            sample = "1 sequence x 1 head, causal, first 2048 positions of 8192"
        elif key == "c3":
            S, heads = 2048, 3
            sample = "1 sequence of 2048 x 3 q heads, window +-512"
        else:
            S, heads = cfg["seq"], cfg["qHeads"]
            sample = f"1 sequence of {S} x {heads} heads"
        kvh = max(1, heads * cfg["kvHeads"] // cfg["qHeads"])
        q = (rng.standard_normal((S, heads * hd)) * cfg["fold"]).astype(npdt)
        k = (rng.standard_normal((S, kvh * hd)) * cfg["fold"]).astype(npdt)
        v = rng.standard_normal((S, kvh * hd)).astype(npdt)
        kw = dict(qHeads=heads, kvHeads=kvh, headDim=hd,
                  windowLeft=math.inf if cfg["wl"] is None else cfg["wl"],
                  windowRight=math.inf if cfg["wr"] is None else cfg["wr"])
        flops = 4.0 * hd * visible_pairs(S, cfg["wl"], cfg["wr"]) * heads
        oracle.sdpa_rows(q[:64], k[:64], v[:64], **kw)  # warm the thread pool
        n, t0 = 0, time.perf_counter()
        while True:
            oracle.sdpa_rows(q, k, v, **kw)
            n += 1
            if time.perf_counter() - t0 > budget_s or n >= 50:
                break
        dt = (time.perf_counter() - t0) / n
        return flops / dt / 1e12, cores, f"{sample}; {n} passes of {dt * 1e3:.1f} ms", dt * 1e3
    # decode: a few sequences, each a 1-row attention over its cache
    hd, H = cfg["hd"], cfg["qHeads"]
    nseq = 8 if key == "c4" else 64
    L = cfg["cacheRows"]
    q = (rng.standard_normal((nseq, 1, H * hd)) / math.sqrt(hd)).astype(np.float16)
    k = rng.standard_normal((nseq, L, H * hd)).astype(np.float16)
    v = rng.standard_normal((nseq, L, H * hd)).astype(np.float16)
    kw = dict(qHeads=H, kvHeads=H, headDim=hd, windowRight=0, qPosOffset=L - 1)
    nbytes = nseq * (2 * L * H * hd * 2 + 2 * H * hd * 2)
    n, t0 = 0, time.perf_counter()
    while True:
        for s in range(nseq):
            oracle.sdpa_rows(q[s], k[s], v[s], **kw)
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= 200:
            break
    dt = (time.perf_counter() - t0) / n
    return (nbytes / dt / 1e9, cores, f"{nseq} of {cfg['batch']} sequences, full {L}-row caches; "
            f"{n} passes of {dt * 1e3:.1f} ms", dt * 1e3)


def run_reference(args):
    """--impl reference: the CPU restatement of the reference's shader math on
    the host cores (the reference's own WebGPU path cannot run here)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun starts its workers with OMP_NUM_THREADS=1: the CPU arm uses every host core
    # at every N, so that its number is the same beside each of the GPU arm's.
    import oracle
    oracle.set_num_threads(os.cpu_count() or 1)
    key = args.workload
    cfg = CONFIGS[key]
    vals, mss = [], []
    desc, cores = "", 1
    for i in range(args.warmup + args.steps):
        val, cores, desc, ms = cpu_sample(key, budget_s=max(2.0, 60.0 / (args.warmup + args.steps)))
        if i >= args.warmup:
            vals.append(val)
            mss.append(ms)
    value = statistics.mean(vals)
    unit = "TFLOP/s" if cfg["kind"] == "prefill" else "GB/s"
    line = {
        "impl": "reference", "metric": metric_name(cfg), "value": value, "unit": unit,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": statistics.mean(mss),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": cfg["dtype"], "data": "synthetic",
        "config": {"workload": cfg["name"], "note": "CPU restatement of the reference's shader "
                   "math (oracle port) on host cores; each step is a bounded sample"},
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port",
                         "sample": desc},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def metric_name(cfg):
    return "prefill_attn_tflops" if cfg["kind"] == "prefill" else "decode_attn_hbm_gbs"


# ----------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------

def timed(torch, dist, world, fn, steps, warmup, flush=None, min_warm_s=0.0, min_timed_s=0.0):
    """Warm-up, then the timed steps bracketed by barrier + sync; returns (max over ranks of
    the device time in ms, timed steps, warm-up steps), timed with CUDA events on the launch
    stream.  At least `warmup` warm-up steps and `steps` timed steps; with min_warm_s /
    min_timed_s both are extended — by the same counts on every rank, from the slowest
    rank's estimate of a step — so that the timed region is long enough to be measured at
    the clocks a sustained load settles at (a region of a few milliseconds sees boost
    clocks that a one-second region does not: the two cannot be compared).  With `flush`
    every step is timed on its own, with the L2 flushed before it."""
    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run(n, first=0):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            fn(first + i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    fn(0)                       # first call: lazy set-up (function attributes, tensor maps)
    barrier()
    est = run(max(warmup, 1), 1) / max(warmup, 1)      # ms per step, this rank
    if world > 1:
        t = torch.tensor([est], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        est = float(t.item())
    est = max(est, 1e-3)
    warm = max(warmup, 1)
    extra = int(math.ceil(min_warm_s * 1e3 / est)) - warm
    if extra > 0:
        done = 0
        while done < extra:                 # in slices, so the launch queue stays short
            n = min(extra - done, 256)
            run(n, warm + done)
            done += n
        warm += extra
    total_steps = steps
    if flush is None and min_timed_s > 0:
        total_steps = max(steps, int(math.ceil(min_timed_s * 1e3 / est / steps)) * steps)
    barrier()
    total = 0.0
    if flush is None:
        total = run(total_steps)
    else:
        for i in range(total_steps):
            flush()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn(i)
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
    if world > 1:
        dist.barrier()
        t = torch.tensor([total], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total = float(t.item())
    return total, total_steps, warm


def bind_to_gpu_numa_node(index):
    """Runs this rank on the host cores next to its GPU (as the driver's topology reports
    them), before any pinned host buffer is allocated: with several ranks streaming inputs
    from host memory at once, buffers that the first-touch policy placed on the other
    socket halve the host-to-device rate.  Only reads the topology; changes nothing on the
    GPU.  Any failure leaves the process where it was."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * w + b for w, mask in enumerate(words) for b in range(64) if (mask >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception as e:  # noqa: BLE001 - placement is an optimisation only
        sys.stderr.write(f"no NUMA placement for GPU {index}: {type(e).__name__}: {e}\n")


def run_gpu(args):
    import torch
    import torch.distributed as dist
    import runntime_b200 as rt

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    # This program's stdout is one JSON line.  Libraries that write banners to file
    # descriptor 1 (NCCL's version line) get stderr instead; the line goes to the real one.
    sys.stdout.flush()
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        bind_to_gpu_numa_node(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ex = rt.CudaExecutor(local)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    if args.tc_mode is not None:
        from runntime_b200._lib import OPT_PREFILL_TC
        ex.setOption(OPT_PREFILL_TC, args.tc_mode)
    peaks = load_peaks()
    traffic = load_traffic()

    def verify(wl):
        """Output check before anything is timed: a sample against the f64 oracle on every
        rank; a miss anywhere ends the run with a non-zero exit code."""
        worst, n, ok = wl.verify()
        if world > 1:
            t = torch.tensor([worst, -float(ok), float(n)], device="cuda", dtype=torch.float64)
            mx = t.clone()
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            sm = t.clone()
            dist.all_reduce(sm, op=dist.ReduceOp.SUM)
            worst, ok, n = float(mx[0].item()), mx[1].item() == -1.0, int(sm[2].item())
        return {"max_abs_err": worst, "rows": n, "against": "f64 oracle, same inputs", "ok": bool(ok)}

    def measure(key, steps, warmup, with_e2e, sized=True):
        cfg = dict(CONFIGS[key])
        cfg["exchange"] = args.exchange
        if args.batch and key == args.workload:
            cfg["batch"] = args.batch
            cfg["name"] += f"_batch{args.batch}"
        if args.rows and key == args.workload:
            cfg["cacheRows" if cfg["kind"] == "decode" else "seq"] = args.rows
            cfg["name"] += f"_rows{args.rows}"
        wl = (Prefill if cfg["kind"] == "prefill" else Decode)(cfg, rank, world, ex)
        layers = cfg.get("layers", 1)
        verified = None
        if not args.no_verify:
            verified = verify(wl)
            if not verified["ok"]:
                if rank == 0:
                    sys.stderr.write(f"bench.py: {cfg['name']}: output differs from the oracle "
                                     f"({json.dumps(verified)}); nothing was timed\n")
                raise SystemExit(3)
        small = key in ("c1", "c2")
        # Flush by READING 256 MB: a written buffer leaves the L2 full of dirty lines and the
        # timed kernel then pays for their write-back (measured: +18 us on a 100 MB stream).
        flushbuf = torch.zeros(64 << 20, dtype=torch.int32, device="cuda") if small else None
        flush = (lambda: flushbuf.sum()) if small else None
        sampler = ClockSampler(local) if (rank == 0 and not args.no_clocks) else None
        step_fn = lambda i: wl.step(i % layers)
        graphed, graph_steps = False, 1
        n1 = ex.launchCount()
        for i in range(3):
            wl.step(i % layers)
        per_step = (ex.launchCount() - n1) / 3.0          # kernels of this library per step
        torch.cuda.synchronize()
        if cfg["kind"] == "decode" and not args.no_graph:
            # A decode step is a few short launches (kernel, merge): capture it once in a
            # CUDA graph so that the device is not left waiting for the host.
            # Where steps run back to back (no L2 flush between them) the graph holds several:
            # inside a graph a kernel is launched as a programmatic dependent of the one
            # before it, as it is in a decoder's graph of a whole token, which single-kernel
            # graphs replayed one after the other cannot show.
            graph_steps = max(1, args.graph_steps) if flush is None else 1
            graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
            with torch.cuda.graph(graph, stream=side):
                for g in range(graph_steps):
                    wl.step(g % layers)
            ex.setStream(torch.cuda.current_stream().cuda_stream)
            step_fn = lambda i: graph.replay()
            graphed = True
        if sampler:
            sampler.start()
        # Time-sized: at least 1.5 s of warm-up and a timed region of at least 1 s (whole
        # multiples of --steps), so that every N is measured at sustained clocks.
        ms, timed_steps, warm_steps = timed(torch, dist, world, step_fn, steps, warmup, flush,
                                            min_warm_s=1.5 if (sized and not args.short) else 0.0,
                                            min_timed_s=1.0 if (sized and not args.short) else 0.0)
        clocks = sampler.stop() if sampler else None
        ex.sync()
        timed_steps, warm_steps = timed_steps * graph_steps, warm_steps * graph_steps
        launches = int(round(per_step * timed_steps))
        resample = clocks is not None and (clocks.get("samples") or 0) < 3
        if world > 1:      # rank 0 holds the sampler; every rank must take the same path
            flag = torch.tensor([1 if resample else 0], device="cuda")
            dist.broadcast(flag, 0)
            resample = bool(flag.item())
        if resample:
            # The timed region was shorter than the sampler's period: repeat the same
            # steps untimed for about 1.5 s with the sampler on and report that.  Every
            # rank runs the same number of steps (the ranks of a sharded decode wait for
            # one another), counted from the measured step time.
            sampler = ClockSampler(local) if rank == 0 else None
            if sampler:
                sampler.start()
            n_rep = max(8, int(1500.0 / max(ms / timed_steps * graph_steps, 1e-3)))
            n_rep = min(n_rep, 200000)
            for i in range(n_rep):
                step_fn(i)
                if i % 64 == 63:
                    torch.cuda.synchronize()
            torch.cuda.synchronize()
            if sampler:
                clocks = sampler.stop()
                clocks["sampled"] = "1.5 s untimed repeat of the timed loop (timed region < sampler period)"
        ex.sync()
        long_region = ms >= 900.0 and flush is None
        if cfg["kind"] == "prefill":
            work = sum(wl.flops(i % layers) for i in range(timed_steps))
            value, unit = work / (ms * 1e-3) / 1e12, "TFLOP/s"
            # burst figure for a kernel timed alone, sustained one for a second-long region
            peak = peaks["tflops_sustained"] if (long_region and peaks.get("tflops_sustained")) else peaks["tflops"]
            bound = "tensor"
            per_launch_local = sum(wl.flops(i % layers, all_ranks=False) for i in range(timed_steps)) / timed_steps
        else:
            work = wl.bytes() * timed_steps
            value, unit = work / (ms * 1e-3) / 1e9, "GB/s"
            peak, bound = peaks["hbm_gbs"], "hbm"
            per_launch_local = wl.bytes(all_ranks=False)
        # roofline of the dominant kernel on this rank: its algorithmic work / its launch time
        achieved = per_launch_local / (ms / timed_steps * 1e-3) / (1e12 if bound == "tensor" else 1e9)
        roof = {"bound": bound, "achieved": achieved, "peak": peak,
                "unit": "TFLOP/s" if bound == "tensor" else "GB/s",
                "frac": achieved / peak, "traffic": traffic.get(key),
                "peak_source": peaks["source"] + (
                    "" if bound != "tensor" else
                    " (sustained: the timed region is a second of back-to-back launches)"
                    if peak != peaks["tflops"] else " (burst)")}
        if bound == "tensor":
            roof["frac_of_burst"] = achieved / peaks["tflops"]
        res = {
            "exchange": getattr(wl, "exchange", None),
            "metric": metric_name(cfg), "value": value, "unit": unit, "ms_per_step": ms / timed_steps,
            "dtype": cfg["dtype"], "workload": cfg["name"], "timed_steps": timed_steps,
            "warmup_steps": warm_steps, "roofline": roof,
            "clocks": clocks, "gpu_launches": launches, "verified": verified,
            "l2": "256 MB read between timed steps" if small else "inputs larger than L2",
            "launch": (f"CUDA graph replay of {graph_steps} step{'s' if graph_steps > 1 else ''}"
                       if graphed else "direct launches"),
        }
        if with_e2e and not args.no_e2e:
            wl.make_host()
            h2d, d2h = wl.io_bytes()
            e_steps = max(2, min(steps, 3)) if not small else steps
            ems, e_steps, _ = timed(torch, dist, world, lambda i: wl.e2e_step(i % layers), e_steps, 1)
            if cfg["kind"] == "prefill":
                ework = sum(wl.flops(i % layers) for i in range(e_steps))
                evalue = ework / (ems * 1e-3) / 1e12
            else:
                evalue = wl.bytes() * e_steps / (ems * 1e-3) / 1e9
            res["e2e"] = {"value": evalue, "unit": unit, "h2d_bytes_per_step": h2d,
                          "d2h_bytes_per_step": d2h, "ms_per_step": ems / e_steps}
        del wl
        torch.cuda.empty_cache()
        return res

    key = args.workload
    cfg = CONFIGS[key]
    main = measure(key, args.steps, args.warmup, True)
    cfg = dict(cfg, name=main["workload"])
    riders = {}
    if key == "c5" and not args.no_decode:
        riders["decode"] = measure("c4", max(args.steps, 5), max(args.warmup, 3), True)
    if key == "c5" and not args.no_riders:
        # the other three configurations: milliseconds each, so every configuration the
        # headline table names is in the one line the driver records
        for rk in ("c3", "c1", "c2"):
            riders[rk] = measure(rk, max(args.steps, 5), max(args.warmup, 3), rk == "c3", sized=(rk == "c3"))

    if rank == 0:
        line = {
            "metric": main["metric"], "value": main["value"], "unit": main["unit"],
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": main["dtype"], "data": "synthetic",
            "timed_steps": main["timed_steps"], "warmup_steps": main["warmup_steps"],
            "config": {"workload": cfg["name"], "l2": main["l2"], "launch": main["launch"],
                       "timing": "the timed region is --steps repeated to at least 1 s after at "
                                 "least 1.5 s of warm-up (timed_steps, warmup_steps)",
                       "parallelism": ("sequences sharded over ranks, no collective"
                                       if cfg["kind"] == "prefill" else
                                       "KV rows sharded over ranks, partials exchanged by "
                                       + str(main.get("exchange"))
                                       if cfg.get("lens") is None else "sequences sharded over ranks")},
            "roofline": main["roofline"], "clocks": main["clocks"],
            "e2e": main.get("e2e"), "gpu_launches": main["gpu_launches"],
            "verified": main["verified"],
        }
        if world == 1 and not args.no_cpu:
            v, cores, desc, _ = cpu_sample(key)
            line["cpu_baseline"] = {"value": v, "unit": main["unit"], "cores": cores,
                                    "kind": "port", "sample": desc}
        for name, extra in riders.items():
            line[name] = {k: extra.get(k) for k in ("metric", "value", "unit", "ms_per_step",
                                                    "workload", "roofline", "e2e", "timed_steps",
                                                    "gpu_launches", "clocks", "launch", "l2",
                                                    "exchange", "verified")}
            if name == "decode" and world == 1 and not args.no_cpu:
                v, cores, desc, _ = cpu_sample("c4", budget_s=6.0)
                line["decode"]["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": cores,
                                                  "kind": "port", "sample": desc}
        real_stdout.write(json.dumps(line) + "\n")
        real_stdout.flush()
    ex.dispose()
    if world > 1:
        dist.destroy_process_group()


# ----------------------------------------------------------------------------
# the operators either side of attention: rope, masked softmax, localAttention and the
# fused decoder-layer step (HBM- or latency-bound; one GPU, replicas if more)
# ----------------------------------------------------------------------------

AUX = {
    "rope": dict(name="rope_f16_65536x4096_hd128", rows=65536, cols=4096, hd=128),
    "softmax": dict(name="masked_softmax_f16_16384x16384_causal_2_segments", n=16384),
    "local": dict(name="local_attention_f16_T262144_8x128_window12", rows=262144, heads=8, hd=128,
                  window=12),
    "gemv": dict(name="decode_projection_f16_m8_k4096_n12288_bias_addend", m=8, k=4096, n=12288),
    "gemm": dict(name="prefill_projection_f16_m32768_k1024_n3072_bias", m=32768, k=1024, n=3072),
    "argmax": dict(name="greedy_head_argmaxdot_f16_v262144_n2048", rows=262144, cols=2048),
    "step": dict(name="moonshine_tiny_decoder_layer_step_f16_batch64_rope_append_attend",
                 batch=64, heads=8, hd=36, maxPos=448),
    "layer": dict(name="decoder_layer_attention_block_f16_b8_dim4096_h32x128_kv4096_qkv_rope_append_attend_oproj",
                  batch=8, heads=32, hd=128, maxPos=4096, layers=4),
}


def run_aux(args):
    import ctypes as C
    import numpy as np
    import torch
    import oracle
    import runntime_b200 as rt
    from runntime_b200._lib import DTYPE_CODE, check
    if int(os.environ.get("RANK", "0")) != 0:
        return  # these operators do not shard: other ranks would only be replicas
    key, cfg = args.workload, AUX[args.workload]
    rotating = None   # set by a workload that defeats the L2 by walking through several inputs
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    ex = rt.CudaExecutor(0)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    lib, peaks = ex._lib, load_peaks()
    g = torch.Generator(device=dev).manual_seed(11)
    f16 = DTYPE_CODE["f16"]
    ptr = lambda t: C.c_void_p(t.data_ptr())
    cores = oracle.num_threads()
    unit = "GB/s"
    if key == "rope":
        R, W, hd = cfg["rows"], cfg["cols"], cfg["hd"]
        x = torch.randn(R, W, generator=g, device=dev, dtype=torch.float16)
        ang = torch.rand(R, hd // 2, generator=g, device=dev) * 6.28
        cos, sin = (t.repeat_interleave(2, dim=1).contiguous() for t in (ang.cos(), ang.sin()))
        out = torch.empty_like(x)
        step = lambda i: check(lib.rt_rope(ex.ctx, ptr(x), ptr(cos), ptr(sin), ptr(out), R, W, hd,
                                           0, W, f16), ex.ctx)
        work = 2 * x.numel() * 2 + 2 * cos.numel() * 4
        host_in, host_out = [x], out
        n = 2048  # CPU sample rows
        xs = np.random.default_rng(1).standard_normal((n, W)).astype(np.float32)
        cs = np.ones((n, hd), np.float32)
        cpu = lambda: oracle.rope_ref(xs, cs, cs, headDim=hd)
        cpu_work, sample = 2 * n * W * 2 + 2 * n * hd * 4, f"{n} of {R} rows (f64 restatement)"
    elif key == "softmax":
        n = cfg["n"]
        x = (torch.randn(n, n, generator=g, device=dev) * 3).to(torch.float16)
        segs = torch.empty(n, 2, device=dev)
        segs[: n // 2] = torch.tensor([0.0, n // 2], device=dev)
        segs[n // 2:] = torch.tensor([n // 2, float(n)], device=dev)
        out = torch.empty_like(x)
        step = lambda i: check(lib.rt_softmax(ex.ctx, ptr(x), ptr(out), ptr(segs), n, n,
                                              rt._lib.WINDOW_INF, 0, f16), ex.ctx)
        # a causal row r of segment [s, e) reads r - s + 1 scores; every row writes n
        half = n // 2
        kept = 2 * (half * (half + 1) // 2)
        work = kept * 2 + n * n * 2
        host_in, host_out = [x], out
        m = 2048
        xs = np.random.default_rng(1).standard_normal((m, m)).astype(np.float32)
        sg = np.array([[0, m]] * m, np.float32)
        cpu = lambda: oracle.softmax_ref(xs, sg, math.inf, 0)
        cpu_work, sample = (m * (m + 1) // 2) * 2 + m * m * 2, f"{m} x {m} causal (f64 restatement)"
    elif key == "local":
        R, H, hd, wn = cfg["rows"], cfg["heads"], cfg["hd"], cfg["window"]
        w = H * hd
        qkv = torch.randn(R, 3 * w, generator=g, device=dev, dtype=torch.float16)
        rel = torch.randn(wn, w, generator=g, device=dev)
        qs = torch.rand(hd, generator=g, device=dev)
        out = torch.empty(R, w, device=dev, dtype=torch.float16)
        step = lambda i: check(lib.rt_local_attention(ex.ctx, ptr(qkv), ptr(rel), ptr(qs), ptr(out),
                                                      R, H, hd, wn, 1.0, 50.0, f16), ex.ctx)
        work = qkv.numel() * 2 + out.numel() * 2
        host_in, host_out = [qkv], out
        m = 1024
        xs = np.random.default_rng(1).standard_normal((m, 3 * w)).astype(np.float32)
        rl, q1 = rel.cpu().numpy(), qs.cpu().numpy()
        cpu = lambda: oracle.local_attention_ref(xs, rl, q1, heads=H, headDim=hd, window=wn)
        cpu_work, sample = m * 4 * w * 2, f"{m} of {R} rows (f64 restatement)"
    elif key == "gemm":
        M, K, N = cfg["m"], cfg["k"], cfg["n"]
        a = torch.randn(M, K, generator=g, device=dev, dtype=torch.float16)
        b = (torch.randn(K, N, generator=g, device=dev) / 32).to(torch.float16)
        bias = torch.randn(N, generator=g, device=dev, dtype=torch.float16)
        out = torch.empty(M, N, device=dev, dtype=torch.float16)
        step = lambda i: check(lib.rt_matmul(ex.ctx, ptr(a), ptr(b), ptr(bias), None, ptr(out),
                                             M, K, N, K, 0, 0, f16), ex.ctx)
        work = 2.0 * M * K * N          # FLOPs: this one is measured against the tensor peak
        unit = "TFLOP/s"
        host_in, host_out = [a], out
        mm = 2048
        a1 = np.random.default_rng(1).standard_normal((mm, K)).astype(np.float32)
        b1 = np.random.default_rng(2).standard_normal((K, N)).astype(np.float32)
        cpu = lambda: a1 @ b1
        cpu_work, sample = 2.0 * mm * K * N, f"[{mm},{K}] x [{K},{N}] numpy f32 (BLAS)"
    elif key == "gemv":
        M, K, N = cfg["m"], cfg["k"], cfg["n"]
        a = torch.randn(M, K, generator=g, device=dev, dtype=torch.float16)
        # One weight matrix (101 MB) would stay in the L2 from step to step; the steps walk
        # through four of them, as the layers of a decoder do (403 MB between two uses of one).
        bs = [(torch.randn(K, N, generator=g, device=dev) / 64).to(torch.float16) for _ in range(4)]
        b = bs[0]
        bias = torch.randn(N, generator=g, device=dev, dtype=torch.float16)
        add = torch.randn(M, N, generator=g, device=dev, dtype=torch.float16)
        out = torch.empty(M, N, device=dev, dtype=torch.float16)
        step = lambda i: check(lib.rt_matmul(ex.ctx, ptr(a), ptr(bs[i % 4]), ptr(bias), ptr(add),
                                             ptr(out), M, K, N, K, 0, 0, f16), ex.ctx)
        work = (K * N + M * K + N + 2 * M * N) * 2     # the weight, read once, dominates
        rotating = "four weight matrices in rotation, 403 MB, larger than L2"
        host_in, host_out = [a], out
        kk, nn = 1024, 3072
        a1 = np.random.default_rng(1).standard_normal((M, kk)).astype(np.float32)
        b1 = np.random.default_rng(2).standard_normal((kk, nn)).astype(np.float32)
        cpu = lambda: a1 @ b1
        cpu_work, sample = (kk * nn + M * kk + M * nn) * 2, f"[{M},{kk}] x [{kk},{nn}] numpy f32 (BLAS)"
    elif key == "argmax":
        R, W = cfg["rows"], cfg["cols"]
        w = torch.randn(R, W, generator=g, device=dev, dtype=torch.float16)
        x = torch.randn(1, W, generator=g, device=dev, dtype=torch.float16)
        out = torch.empty(1, device=dev, dtype=torch.float32)
        step = lambda i: check(lib.rt_argmax_dot(ex.ctx, ptr(w), ptr(x), ptr(out), R, W, f16), ex.ctx)
        work = (R * W + W) * 2 + 4
        host_in, host_out = [x], out
        r1 = 16384
        w1 = np.random.default_rng(1).standard_normal((r1, W)).astype(np.float32)
        x1 = np.random.default_rng(2).standard_normal(W).astype(np.float32)
        cpu = lambda: int(np.argmax(w1 @ x1))
        cpu_work, sample = r1 * W * 2, f"{r1} of {R} rows, numpy f32 gemv + argmax"
    elif key == "layer":
        # The attention block of a decoder layer for one new token per sequence, on device from
        # the hidden state to the residual sum: fused qkv projection (+ bias), rope of q and k
        # + append + attention in one launch, output projection with the residual as addend.
        # Three launches per layer; the steps walk through `layers` sets of weights and caches.
        from runntime_b200.engine import decode_batched
        B, H, hd, P, NL = cfg["batch"], cfg["heads"], cfg["hd"], cfg["maxPos"], cfg["layers"]
        D = H * hd
        x = torch.randn(B, D, generator=g, device=dev, dtype=torch.float16)
        wqkv = [(torch.randn(D, 3 * D, generator=g, device=dev) / 64).to(torch.float16) for _ in range(NL)]
        bqkv = torch.randn(3 * D, generator=g, device=dev, dtype=torch.float16)
        wo = [(torch.randn(D, D, generator=g, device=dev) / 64).to(torch.float16) for _ in range(NL)]
        kc = [torch.randn(B, P, D, generator=g, device=dev, dtype=torch.float16) for _ in range(NL)]
        vc = [torch.randn(B, P, D, generator=g, device=dev, dtype=torch.float16) for _ in range(NL)]
        kvLens = torch.full((B,), P, dtype=torch.int32, device=dev)   # the appended row is the last
        tab = torch.rand(P, hd // 2, generator=g, device=dev) * 6.28
        cos = (tab.cos().repeat_interleave(2, 1) * hd ** -0.25).contiguous()
        sin = (tab.sin().repeat_interleave(2, 1) * hd ** -0.25).contiguous()
        qkv = torch.empty(B, 3 * D, device=dev, dtype=torch.float16)
        att = torch.empty(B, D, device=dev, dtype=torch.float16)
        out = torch.empty(B, D, device=dev, dtype=torch.float16)
        base = qkv.data_ptr()

        def step(i):
            L = i % NL
            check(lib.rt_matmul(ex.ctx, ptr(x), ptr(wqkv[L]), ptr(bqkv), None, ptr(qkv), B, D, 3 * D,
                                D, 0, 0, f16), ex.ctx)
            decode_batched(ex, base, att, kc[L], vc[L], dtype="f16", batch=B, cacheRows=P, qHeads=H,
                           kvHeads=H, headDim=hd, kvLen=P, kvLens=kvLens, kNew=base + D * 2,
                           vNew=base + 2 * D * 2, ropeCos=cos, ropeSin=sin, ropeByPosition=True,
                           qRowStride=3 * D, kNewRowStride=3 * D, vNewRowStride=3 * D)
            check(lib.rt_matmul(ex.ctx, ptr(att), ptr(wo[L]), None, ptr(x), ptr(out), B, D, D,
                                D, 0, 0, f16), ex.ctx)
        # weights and the visible cache rows read once; activations are noise beside them
        work = (D * 3 * D + D * D + 2 * B * P * D) * 2 + (B * D * 4 + B * 3 * D * 2 + 3 * D) * 2
        rotating = f"{NL} layers' weights and caches in rotation ({NL * (4 * D * D + 2 * B * P * D) * 2 >> 20} MB), larger than L2"
        host_in, host_out = [x], out
        cpu, cpu_work, sample = None, 0, ""
    else:  # step: rope x2 + slice + writeRows x2 + attention of one decoder layer, batch of sequences
        from runntime_b200.engine import decode_batched
        B, H, hd, P = cfg["batch"], cfg["heads"], cfg["hd"], cfg["maxPos"]
        w = H * hd
        kc = torch.randn(B, P, w, generator=g, device=dev, dtype=torch.float16)
        vc = torch.randn(B, P, w, generator=g, device=dev, dtype=torch.float16)
        lens = torch.randint(1, P - 8, (B,), generator=torch.Generator().manual_seed(3))
        kvLens = (lens + 1).to(torch.int32).to(dev)   # visible rows including the appended one
        tab = torch.rand(P, hd // 2, generator=g, device=dev) * 6.28
        cos = (tab.cos().repeat_interleave(2, 1) * hd ** -0.25).contiguous()
        sin = (tab.sin().repeat_interleave(2, 1) * hd ** -0.25).contiguous()
        qkv = torch.randn(B, 3 * w, generator=g, device=dev, dtype=torch.float16)
        out = torch.empty(B, w, device=dev, dtype=torch.float16)
        base, maxLen = qkv.data_ptr(), int(lens.max()) + 1

        def step(i):  # the same positions every step: the append rewrites the same rows
            decode_batched(ex, base, out, kc, vc, dtype="f16", batch=B, cacheRows=P, qHeads=H,
                           kvHeads=H, headDim=hd, kvLen=maxLen, kvLens=kvLens, kNew=base + w * 2,
                           vNew=base + 2 * w * 2, ropeCos=cos, ropeSin=sin, ropeByPosition=True,
                           qRowStride=3 * w, kNewRowStride=3 * w, vNewRowStride=3 * w)
        work = sum(2 * (int(L) + 1) * w * 2 for L in lens) + B * (3 * w + w + 2 * w) * 2
        host_in, host_out = [qkv], out
        cpu, cpu_work, sample = None, 0, ""
    flushbuf = torch.zeros(64 << 20, dtype=torch.int32, device=dev)   # read, not written: see Prefill
    small = work < (512 << 20) and not rotating   # less than about four times the L2: flush it between timed steps
    n0 = ex.launchCount()
    sampler = ClockSampler(0) if not args.no_clocks else None
    if sampler:
        sampler.start()
    ms, _, _ = timed(torch, None, 1, step, args.steps, args.warmup, (lambda: flushbuf.sum()) if small else None)
    clocks = sampler.stop() if sampler else None
    launches = (ex.launchCount() - n0) * args.steps // (args.steps + max(args.warmup, 1) + 1)
    tensor = unit == "TFLOP/s"
    scale = 1e12 if tensor else 1e9
    value = work * args.steps / (ms * 1e-3) / scale
    peak = peaks["tflops"] if tensor else peaks["hbm_gbs"]
    line = {
        "metric": f"{key}_tflops" if tensor else f"{key}_hbm_gbs", "value": value, "unit": unit, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": cfg["name"],
                   "l2": rotating or ("256 MB read between timed steps" if small else "inputs larger than L2"),
                   "parallelism": "replicas only"},
        "roofline": {"bound": "tensor" if tensor else "hbm", "achieved": value, "peak": peak,
                     "unit": unit, "frac": value / peak, "traffic": load_traffic().get(key),
                     "peak_source": peaks["source"] + (" (burst)" if tensor else "")},
        "clocks": clocks, "gpu_launches": launches,
    }
    if not args.no_e2e:
        hin = [t.cpu().pin_memory() for t in host_in]
        hout = torch.empty(host_out.shape, dtype=host_out.dtype).pin_memory()

        def e2e(i):
            for d, h in zip(host_in, hin):
                d.copy_(h, non_blocking=True)
            step(i)
            hout.copy_(host_out, non_blocking=True)
        ems, esteps, _ = timed(torch, None, 1, e2e, max(2, min(args.steps, 3)), 1)
        line["e2e"] = {"value": work * esteps / (ems * 1e-3) / scale, "unit": unit,
                       "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host_in),
                       "d2h_bytes_per_step": host_out.numel() * host_out.element_size(),
                       "ms_per_step": ems / esteps}
    if cpu is not None and not args.no_cpu:
        cpu()
        n, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < 5.0 and n < 50:
            cpu()
            n += 1
        dt = (time.perf_counter() - t0) / n
        line["cpu_baseline"] = {"value": cpu_work / dt / scale, "unit": unit, "cores": cores,
                                "kind": "port", "sample": f"{sample}; {n} passes of {dt * 1e3:.1f} ms"}
    print(json.dumps(line), flush=True)
    ex.dispose()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c5", choices=sorted(CONFIGS) + sorted(AUX))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-decode", action="store_true", help="skip the decode rider of c5")
    ap.add_argument("--no-riders", action="store_true", help="skip the c1/c2/c3 riders of c5")
    ap.add_argument("--no-verify", action="store_true", help="skip the oracle check before timing")
    ap.add_argument("--short", action="store_true",
                    help="time exactly --steps after --warmup (small cases for profiler captures)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer (e2e) leg")
    ap.add_argument("--no-clocks", action="store_true", help="do not sample nvidia-smi clocks")
    ap.add_argument("--graph-steps", type=int, default=8,
                    help="decode steps captured in one CUDA graph (back-to-back workloads)")
    ap.add_argument("--no-graph", action="store_true",
                    help="launch decode steps directly instead of replaying a CUDA graph")
    ap.add_argument("--tc-mode", type=int, default=None,
                    help="RT_OPT_PREFILL_TC value (0: FP32-pipe kernel, 1: tensor-core kernel)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="how KV-sharded decode trades partials between ranks")
    ap.add_argument("--rows", type=int, default=0,
                    help="override the workload's sequence / cache length (small cases)")
    ap.add_argument("--batch", type=int, default=0,
                    help="override the workload's batch (small cases for profiler captures)")
    args = ap.parse_args()
    if args.workload in AUX:
        if args.impl == "reference":
            print(json.dumps({"impl": "reference", "unavailable":
                              "the reference arm covers the attention workloads c1..c5 only"}))
        else:
            run_aux(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
