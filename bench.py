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
        wl, wr = self.windows(layer)
        prefill_batched(self.ex, self.q, self.k, self.v, self.out, dtype=c["dtype"], batch=self.nb,
                        seqStride=c["seq"], seqLens=self.lens, qHeads=c["qHeads"],
                        kvHeads=c["kvHeads"], headDim=c["hd"], windowLeft=wl, windowRight=wr)

    def io_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.q, self.k, self.v)), \
            self.out.numel() * self.out.element_size()

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
        from runntime_b200.engine import ShardedDecode, shard_rows
        self.cfg, self.ex, self.torch, self.world, self.rank = cfg, ex, torch, world, rank
        dev = torch.device("cuda", torch.cuda.current_device())
        b, hd, H = cfg["batch"], cfg["hd"], cfg["kvHeads"]
        w = H * hd
        self.shard_kv = cfg["lens"] is None  # long-context: split KV rows across ranks
        gl = torch.Generator(device="cpu").manual_seed(77)
        if self.shard_kv:
            s, e = shard_rows(cfg["cacheRows"], world, rank)
            self.rows = e - s
            self.b = b
            self.lens_all = [cfg["cacheRows"]] * b
            self.lens = None
        else:
            per = -(-b // world)
            b0, b1 = min(rank * per, b), min((rank + 1) * per, b)
            self.b = b1 - b0
            lens = torch.randint(cfg["lens"][0], cfg["lens"][1] + 1, (b,), generator=gl)
            self.lens_all = lens.tolist()
            self.lens_mine = self.lens_all[b0:b1]
            self.lens = lens[b0:b1].to(torch.int32).to(dev)
            self.rows = cfg["cacheRows"]
        gd = torch.Generator(device=dev).manual_seed(2000 + rank)
        nb = max(self.b, 1)
        self.k = torch.randn(nb, self.rows, w, generator=gd, device=dev, dtype=torch.float16)
        self.v = torch.randn(nb, self.rows, w, generator=gd, device=dev, dtype=torch.float16)
        gq = torch.Generator(device=dev).manual_seed(3000)  # q is the same on every rank
        self.q = (torch.randn(nb, cfg["qHeads"] * hd, generator=gq, device=dev)
                  * hd ** -0.5).to(torch.float16)
        self.out = torch.empty_like(self.q)
        self.kNew = self.vNew = None
        if not self.shard_kv:
            self.kNew = torch.randn(nb, w, generator=gd, device=dev, dtype=torch.float16)
            self.vNew = torch.randn(nb, w, generator=gd, device=dev, dtype=torch.float16)
        if cfg["cross"]:
            self.ck = torch.randn(nb, cfg["cross"], w, generator=gd, device=dev, dtype=torch.float16)
            self.cv = torch.randn(nb, cfg["cross"], w, generator=gd, device=dev, dtype=torch.float16)
            self.out2 = torch.empty_like(self.q)
        # KV rows split over ranks: the partials are traded through peer memory by the decode
        # kernel itself (--exchange peer, the default) or by one NCCL all-gather (--exchange nccl,
        # also the fallback when symmetric memory cannot be set up).
        self.sharded = self.peer = None
        self.exchange = "none"
        if self.shard_kv and world > 1:
            if cfg.get("exchange", "peer") == "peer":
                try:
                    from runntime_b200.engine import PeerExchangeDecode
                    self.peer = PeerExchangeDecode(units=nb * cfg["qHeads"], headDim=hd, device=dev)
                    self.exchange = "peer memory, in the decode kernel"
                except Exception as e:  # noqa: BLE001 - any set-up failure means: use NCCL
                    sys.stderr.write(f"peer exchange unavailable ({type(e).__name__}: {e}); using NCCL\n")
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
            if not self.shard_kv:
                total += 2 * w * es          # appended K/V row write
            if c["cross"]:
                total += 2 * c["cross"] * w * es + qo
        if self.shard_kv and not all_ranks:
            total = total * self.rows / c["cacheRows"]
        return float(total)

    def launches_per_step(self):
        n = 1 + (1 if self.cfg["cross"] else 0)
        return n + (1 if (self.sharded or self.peer) else 0)

    def step(self, layer=0):
        from runntime_b200.engine import decode_batched
        c = self.cfg
        if self.b == 0:
            return
        common = dict(dtype="f16", batch=self.b, qHeads=c["qHeads"], kvHeads=c["kvHeads"],
                      headDim=c["hd"])
        if self.peer:
            self.peer.step(self.ex, self.q, self.k, self.v, self.out, shardRows=self.rows, **common)
            return
        if self.sharded:
            self.sharded.step(self.ex, self.q, self.k, self.v, self.out, shardRows=self.rows,
                              partials=self.partials, **common)
            return
        decode_batched(self.ex, self.q, self.out, self.k, self.v, cacheRows=self.rows,
                       kvLen=max(self.lens_all) if self.lens is not None else self.rows,
                       kvLens=self.lens, kNew=self.kNew, vNew=self.vNew,
                       splits=int(os.environ.get("RT_BENCH_SPLITS", "0")), **common)
        if c["cross"]:
            decode_batched(self.ex, self.q, self.out2, self.ck, self.cv, cacheRows=c["cross"],
                           kvLen=c["cross"], **common)

    def io_bytes(self):
        n = self.q.numel() * 2
        if self.kNew is not None:
            n += 2 * self.kNew.numel() * 2
        return n, self.out.numel() * 2

    def make_host(self):
        # A decode step's inputs are the new token's q (and K/V row); the cache is
        # device-resident state, as it is in the reference's decoder loop.
        self.hq = self.q.cpu().pin_memory()
        self.hout = self.torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory()
        if self.kNew is not None:
            self.hkn, self.hvn = self.kNew.cpu().pin_memory(), self.vNew.cpu().pin_memory()

    def e2e_step(self, layer=0):
        self.q.copy_(self.hq, non_blocking=True)
        if self.kNew is not None:
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

def timed(torch, dist, world, fn, steps, warmup, flush=None):
    """W warm-ups, then K timed steps bracketed by barrier + sync; returns the
    max over ranks of the device time in ms (CUDA events on the launch stream)."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    total = 0.0
    if flush is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        torch.cuda.synchronize()
        total = e0.elapsed_time(e1)
    else:
        for i in range(steps):
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
    return total


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
    if world > 1:
        # NCCL's version banner goes to stdout; this program's stdout is one JSON line.
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ex = rt.CudaExecutor(local)
    ex.setStream(torch.cuda.current_stream().cuda_stream)
    if args.tc_mode is not None:
        from runntime_b200._lib import OPT_PREFILL_TC
        ex.setOption(OPT_PREFILL_TC, args.tc_mode)
    peaks = load_peaks()
    traffic = load_traffic()

    def measure(key, steps, warmup, with_e2e):
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
        small = key in ("c1", "c2")
        # Flush by READING 256 MB: a written buffer leaves the L2 full of dirty lines and the
        # timed kernel then pays for their write-back (measured: +18 us on a 100 MB stream).
        flushbuf = torch.zeros(64 << 20, dtype=torch.int32, device="cuda") if small else None
        flush = (lambda: flushbuf.sum()) if small else None
        sampler = ClockSampler(local) if (rank == 0 and not args.no_clocks) else None
        step_fn = lambda i: wl.step(i % layers)
        graphed = False
        if cfg["kind"] == "decode" and not args.no_graph:
            # A decode step is a few short launches (kernel, all-gather, merge): capture
            # it once in a CUDA graph so that the device is not left waiting for the host.
            n1 = ex.launchCount()
            for i in range(3):
                wl.step(0)
            per_step = (ex.launchCount() - n1) // 3
            torch.cuda.synchronize()
            graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
            with torch.cuda.graph(graph, stream=side):
                ex.setStream(torch.cuda.current_stream().cuda_stream)
                wl.step(0)
            ex.setStream(torch.cuda.current_stream().cuda_stream)
            step_fn = lambda i: graph.replay()
            graphed = True
        n0 = ex.launchCount()
        if sampler:
            sampler.start()
        ms = timed(torch, dist, world, step_fn, steps, warmup, flush)
        clocks = sampler.stop() if sampler else None
        ex.sync()
        launches = (per_step * steps) if graphed else \
            (ex.launchCount() - n0) * steps // (steps + warmup)
        if world == 1 and clocks is not None and (clocks.get("samples") or 0) < 3:
            # The timed region was shorter than the sampler's period: repeat the same
            # steps untimed for about 1.5 s with the sampler on and report that.
            sampler = ClockSampler(local)
            sampler.start()
            t_end = time.perf_counter() + 1.5
            i = 0
            while time.perf_counter() < t_end:
                step_fn(i)
                i += 1
                if i % 8 == 0:
                    torch.cuda.synchronize()
            torch.cuda.synchronize()
            clocks = sampler.stop()
            clocks["sampled"] = "1.5 s untimed repeat of the timed loop (timed region < sampler period)"
        ex.sync()
        if cfg["kind"] == "prefill":
            work = sum(wl.flops(i % layers) for i in range(steps))
            value, unit = work / (ms * 1e-3) / 1e12, "TFLOP/s"
            peak, bound = peaks["tflops"], "tensor"
            per_launch_local = sum(wl.flops(i % layers, all_ranks=False) for i in range(steps)) / steps
        else:
            work = wl.bytes() * steps
            value, unit = work / (ms * 1e-3) / 1e9, "GB/s"
            peak, bound = peaks["hbm_gbs"], "hbm"
            per_launch_local = wl.bytes(all_ranks=False)
        # roofline of the dominant kernel on this rank: its algorithmic work / its launch time
        achieved = per_launch_local / (ms / steps * 1e-3) / (1e12 if bound == "tensor" else 1e9)
        res = {
            "exchange": getattr(wl, "exchange", None),
            "metric": metric_name(cfg), "value": value, "unit": unit, "ms_per_step": ms / steps,
            "dtype": cfg["dtype"], "workload": cfg["name"],
            "roofline": {"bound": bound, "achieved": achieved, "peak": peak,
                         "unit": "TFLOP/s" if bound == "tensor" else "GB/s",
                         "frac": achieved / peak, "traffic": traffic.get(key),
                         "peak_source": peaks["source"] + (" (burst)" if bound == "tensor" else "")},
            "clocks": clocks, "gpu_launches": launches,
            "l2": "256 MB read between timed steps" if small else "inputs larger than L2",
            "launch": "CUDA graph replay of one step" if graphed else "direct launches",
        }
        if with_e2e and not args.no_e2e:
            wl.make_host()
            h2d, d2h = wl.io_bytes()
            e_steps = max(2, min(steps, 3)) if not small else steps
            ems = timed(torch, dist, world, lambda i: wl.e2e_step(i % layers), e_steps, 1)
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
    extra = None
    if key == "c5" and not args.no_decode:
        extra = measure("c4", max(args.steps, 5), max(args.warmup, 3), True)

    if rank == 0:
        line = {
            "metric": main["metric"], "value": main["value"], "unit": main["unit"],
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": main["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": main["dtype"], "data": "synthetic",
            "config": {"workload": cfg["name"], "l2": main["l2"], "launch": main["launch"],
                       "parallelism": ("sequences sharded over ranks, no collective"
                                       if cfg["kind"] == "prefill" else
                                       "KV rows sharded over ranks, partials exchanged by "
                                       + str(main.get("exchange"))
                                       if cfg.get("lens") is None else "sequences sharded over ranks")},
            "roofline": main["roofline"], "clocks": main["clocks"],
            "e2e": main.get("e2e"), "gpu_launches": main["gpu_launches"],
        }
        if world == 1 and not args.no_cpu:
            v, cores, desc, _ = cpu_sample(key)
            line["cpu_baseline"] = {"value": v, "unit": main["unit"], "cores": cores,
                                    "kind": "port", "sample": desc}
        if extra:
            line["decode"] = {k: extra.get(k) for k in ("metric", "value", "unit", "ms_per_step",
                                                        "workload", "roofline", "e2e",
                                                        "gpu_launches", "clocks", "launch",
                                                        "exchange")}
            if world == 1 and not args.no_cpu:
                v, cores, desc, _ = cpu_sample("c4", budget_s=6.0)
                line["decode"]["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": cores,
                                                  "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
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
    ms = timed(torch, None, 1, step, args.steps, args.warmup, (lambda: flushbuf.sum()) if small else None)
    clocks = sampler.stop() if sampler else None
    launches = (ex.launchCount() - n0) * args.steps // (args.steps + args.warmup)
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
        ems = timed(torch, None, 1, e2e, max(2, min(args.steps, 3)), 1)
        esteps = max(2, min(args.steps, 3))
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
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer (e2e) leg")
    ap.add_argument("--no-clocks", action="store_true", help="do not sample nvidia-smi clocks")
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
