#!/usr/bin/env python
"""Benchmark of the Forgetting Attention hot path (fwd + bwd) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg3] [--impl ours|reference]

One "step" is one forward + backward pass of the operator over one synthetic batch of
the named workload.  With N > 1 (launched by torch.distributed.run, one rank per GPU)
every rank runs its own batch of the same shape -- the (batch, head) units are
independent, there is no collective on the data path -- so the job is N times larger
("scaling": "weak") and `value` is the whole-job rate: FLOPs of all ranks / max-over-ranks
device time.  FLOPs are the algorithmic count 14 * D * H * sum_b n_b (n_b + 1) / 2 with
n_b = T - seq_start_b (4 forward + 10 backward per query/key pair and head-dim element).

Prints ONE JSON line (rank 0).  `--impl reference` times the upstream project's own CPU
formulation of the operator (the dense PyTorch math, restated in oracle/) on the host
cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "fwd+bwd Forgetting Attention TFLOP/s"
UNIT = "TFLOP/s"

# name: (B, T, H, D, gate-logit mean, gate-logit std, has seq_start, adaptive_threshold, per-head input scale)
WORKLOADS = {
    "cfg2": dict(B=4, T=512, H=12, D=64, mu=0.0, sigma=1.0, seq=False, thr=None, head_scale=False, seed=1002),
    "cfg3": dict(B=2, T=16384, H=24, D=64, mu=4.0, sigma=1.0, seq=True, thr=None, head_scale=False, seed=1003),
    "cfg4": dict(B=4, T=16384, H=16, D=128, mu=-1.0, sigma=1.5, seq=False, thr=None, head_scale=True, seed=1004),
    "cfg4_acp": dict(B=4, T=16384, H=16, D=128, mu=-1.0, sigma=1.5, seq=False, thr="auto", head_scale=True, seed=1004),
    # attention of the FoX-Pro block shape; at N > 1 GPUs the sequence is split (context parallel, strong scaling)
    "cfg5_attn": dict(B=1, T=65536, H=24, D=64, mu=5.0, sigma=1.0, seq=False, thr=None, head_scale=False, seed=1005,
                      context_parallel=True),
    # small cases for profiler captures: inputs (4 x 34 / 67 MB) exceed the 126 MB L2, kernels last a few ms
    "prof_d64": dict(B=2, T=8192, H=16, D=64, mu=4.0, sigma=1.0, seq=True, thr=None, head_scale=False, seed=1005),
    "prof_d128": dict(B=2, T=8192, H=16, D=128, mu=-1.0, sigma=1.5, seq=False, thr=None, head_scale=True, seed=1006),
}
DESCR = {
    "cfg2": "kernel-level op B4 T512 H12 D64 bf16",
    "cfg3": "long-context FoX-760M layer shape B2 T16384 H24 D64 bf16, gate logits N(4,1), seq_start U[0,2048)",
    "cfg4": "ACP stress shape B4 T16384 H16 D128 bf16, gate logits N(-1,1.5), pruning off",
    "cfg4_acp": "ACP stress shape B4 T16384 H16 D128 bf16, gate logits N(-1,1.5), adaptive_threshold=auto",
    "cfg5_attn": "attention of the FoX-Pro block shape B1 T65536 H24 D64 bf16, gate logits N(5,1); N>1: context parallel",
    "prof_d64": "profiler-sized case B2 T8192 H16 D64 bf16 (cfg3 distributions)",
    "prof_d128": "profiler-sized case B2 T8192 H16 D128 bf16 (cfg4 distributions, pruning off)",
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def make_inputs(w, rank, pin=False):
    """Seeded synthetic inputs on the CPU generator (device independent bits): q, k, v,
    gate logits, dout, then config-specific extras, in that order.  Every rank draws the same
    batch: the units are independent, and equal work per rank (same seq_start draws) makes the
    max-over-ranks time a statement about the hardware, not about the luck of the draw."""
    del rank
    g = torch.Generator().manual_seed(w["seed"])
    B, T, H, D = w["B"], w["T"], w["H"], w["D"]
    q = torch.randn(B, H, T, D, generator=g)
    k = torch.randn(B, H, T, D, generator=g)
    v = torch.randn(B, H, T, D, generator=g)
    logit = torch.randn(B, H, T, generator=g) * w["sigma"] + w["mu"]
    dout = torch.randn(B, H, T, D, generator=g)
    seq = torch.randint(0, 2048, (B,), generator=g) if w["seq"] else None
    if w["head_scale"]:
        s = (torch.rand(H, generator=g) * 1.5 + 0.5).view(1, H, 1, 1)
        q, k, v = q * s, k * s, v * s
    q, k, v, dout = [t.to(torch.bfloat16) for t in (q, k, v, dout)]
    log_fgate = torch.nn.functional.logsigmoid(logit.float())
    ts = dict(q=q, k=k, v=v, log_fgate=log_fgate, dout=dout)
    if pin:
        ts = {n: t.pin_memory() for n, t in ts.items()}
    ts["seq_start"] = seq
    return ts


def flops_of(w, seq):
    n = torch.full((w["B"],), float(w["T"]), dtype=torch.float64)
    if seq is not None:
        n = n - seq.double()
    pairs = float((n * (n + 1) / 2).sum()) * w["H"]
    return 14.0 * w["D"] * pairs, pairs


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        clocks, mx, reasons = [], None, set()
        for line in out.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                clocks.append(float(f[1]))
                mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": mx, "reasons": ["no samples"]}
        top = max(clocks)
        loaded = [c for c in clocks if c >= 0.5 * top] or clocks
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks)}


# --------------------------------------------------------------------------- CPU arm
def cpu_sample(w, threads, rows=None):
    """The upstream dense formulation (oracle) on the host: ONE (batch, head) unit of the
    workload at full key length, fwd + autograd bwd, evaluated over query-row chunks so the
    T x T matrices stay bounded.  rows=None: every query row; rows=r: only the last r query
    rows (a smaller sample of the same unit).  Returns (seconds, flops, description)."""
    from oracle import fox_oracle as orc
    torch.set_num_threads(threads)
    T, D = w["T"], w["D"]
    g = torch.Generator().manual_seed(w["seed"])
    q, k, v, dout = [torch.randn(1, 1, T, D, generator=g) for _ in range(4)]
    lf = torch.nn.functional.logsigmoid(torch.randn(1, 1, T, generator=g) * w["sigma"] + w["mu"])
    chunk = min(T, 2048)
    first = 0 if rows is None else max(T - rows, 0)
    t0 = time.perf_counter()
    kk, vv, ll = [t.clone().requires_grad_() for t in (k, v, lf)]
    for r0 in range(first, T, chunk):
        r1 = min(T, r0 + chunk)
        qq = q[:, :, r0:r1].clone().requires_grad_()
        out = orc.dense_forgetting_attention(qq, kk[:, :, :r1], vv[:, :, :r1], ll[:, :, :r1], None, None)
        out.backward(dout[:, :, r0:r1])
    dt = time.perf_counter() - t0
    pairs = T * (T + 1) / 2 - first * (first + 1) / 2
    flops = 14.0 * D * pairs
    what = "every query row" if rows is None else f"the last {T - first} query rows"
    return dt, flops, (f"1 of {w['B'] * w['H']} (batch, head) units, {what} against keys [0, T={T}), fp32 dense "
                       f"PyTorch fwd+autograd bwd in {chunk}-row chunks")


def cpu_rows(w):
    """Query rows of the CPU sample: every row of the unit up to T = 16384 (seconds per sample), the last 4096
    beyond.  The reference arm and the cpu_baseline leg of the GPU arm time the same sample."""
    return None if w["T"] <= 16384 else 4096


def run_reference(args, w, wname):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows = cpu_rows(w)
    for _ in range(args.warmup):
        cpu_sample(w, threads, rows)
    times = []
    flops = 0.0
    desc = ""
    for _ in range(args.steps):
        dt, flops, desc = cpu_sample(w, threads, rows)
        times.append(dt)
    mean = sum(times) / len(times)
    val = flops / mean / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": mean * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wname, "description": DESCR[wname], "step": "bounded CPU sample: " + desc},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    _emit(line)


def context_parallel_leg(world, rank, dev, steps=5, warmup=3):
    """cfg5's attention (B1 T65536 H24 D64), context parallel over all ranks (strong scaling: one sequence),
    next to the same sequence on rank 0 alone in the same run.  Device-timed, max over ranks.  Returns the
    record for the JSON line (rank 0) or None."""
    import torch.distributed as dist
    import forgetting_transformer_b200 as fox
    from forgetting_transformer_b200 import _lib, sharding
    w = WORKLOADS["cfg5_attn"]
    host = make_inputs(w, rank)
    flops, _ = flops_of(w, None)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(step_fn, n_warm, n):
        for _ in range(n_warm):
            step_fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(n):
            step_fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    one_gpu_ms = None
    if rank == 0:      # the whole sequence on one GPU; the other ranks wait at the barrier inside their first timed()
        full = {n: host[n].to(dev) for n in ("q", "k", "v", "log_fgate", "dout")}
        fq, fk, fv, fl = [full[n].requires_grad_() for n in ("q", "k", "v", "log_fgate")]

        def one_step():
            fq.grad = fk.grad = fv.grad = fl.grad = None
            fox.forgetting_attention(fq, fk, fv, fl, head_first=True).backward(full["dout"])

        for _ in range(2):
            one_step()
        torch.cuda.synchronize()
        e0.record()
        for _ in range(3):
            one_step()
        e1.record()
        torch.cuda.synchronize()
        one_gpu_ms = e0.elapsed_time(e1) / 3
        del full, fq, fk, fv, fl
        torch.cuda.empty_cache()
    tc = w["T"] // (2 * world)
    c0, c1 = sharding.zigzag_chunks(world, rank)
    loc = {n: torch.cat([host[n][:, :, c0 * tc:(c0 + 1) * tc], host[n][:, :, c1 * tc:(c1 + 1) * tc]], dim=2).to(dev)
           for n in ("q", "k", "v", "log_fgate", "dout")}
    q, k, v, lf = [loc[n].requires_grad_() for n in ("q", "k", "v", "log_fgate")]

    # How the upper halves travel, the priority of the NCCL stream and the number of head groups (each a complete
    # step on its own CUDA stream, so that one group's exposed collectives run under the other's kernels) are tuned
    # here, in the run itself: every candidate is timed for a few steps and the fastest one measured (all reported).
    # (two head groups measured 2 % slower on 2 GPUs and 7 % slower on 4: not among the candidates)
    candidates = [("p2p", True, 1), ("collective", True, 1), ("collective", False, 1)]
    groups = {True: sharding.context_parallel_group(high_priority=True),
              False: sharding.context_parallel_group(high_priority=False)}
    state = {"group": None, "head_groups": 1}

    def cp_step():
        q.grad = k.grad = v.grad = lf.grad = None
        sharding.context_parallel_attention(q, k, v, lf, group=state["group"],
                                            head_groups=state["head_groups"]).backward(loc["dout"])

    trial = {}
    for mode, hp, hg in candidates:
        sharding.UPPER_EXCHANGE, state["group"], state["head_groups"] = mode, groups[hp], hg
        t_ = torch.tensor([timed(cp_step, 2, 3)], dtype=torch.float64, device=dev)
        dist.all_reduce(t_, op=dist.ReduceOp.MAX)
        trial[f"{mode}, {'high' if hp else 'default'}-priority stream, {hg} head group{'s' if hg > 1 else ''}"] = float(t_.item())
    best = min(trial, key=trial.get)              # (the same on every rank: the times were max-reduced)
    mode, hp, hg = candidates[list(trial).index(best)]
    sharding.UPPER_EXCHANGE, state["group"], state["head_groups"] = mode, groups[hp], hg
    ms = timed(cp_step, warmup, steps)
    sharding.UPPER_EXCHANGE = None
    _lib.check_status()
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    if rank != 0:
        return None
    return {"workload": "cfg5_attn", "description": DESCR["cfg5_attn"], "scaling": "strong", "n_gpus": world,
            "ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12, "one_gpu_ms": one_gpu_ms,
            "one_gpu_tflops": flops / (one_gpu_ms * 1e-3) / 1e12, "speedup": one_gpu_ms / ms,
            "efficiency": one_gpu_ms / (world * ms), "steps": steps, "warmup": warmup,
            "upper_half_exchange": best, "ms_per_step_by_exchange_3_steps": trial,
            "exchange": "lower halves of K, V (chunk j on rank j) by NCCL all-gather into sequence-major staging, "
                        "their gradients by reduce-scatter; upper halves point to point (causal subset, slabs "
                        "straight into place, under the first chunk's forward) or by collectives, whichever "
                        "measured faster in this run; no collective inside the kernels"}


# --------------------------------------------------------------------------- upstream's Triton operator
# Block configurations tried for upstream's three kernels, (BLOCK_M, BLOCK_N, num_stages, num_warps) as
# (forward, key side of the backward, query side of the backward) by head dim.  Upstream's own table stops at
# sm_90 and raises on sm_100; its config functions are documented as overridable
# (src/forgetting_transformer/ops/forgetting_attention.py:459, 799).  First row: upstream's H100 entries
# (lines 467-472, 855-859, 882-886).
UPSTREAM_CONFIGS = {
    64: [("h100_rows", (128, 64, 3, 8), (128, 64, 3, 4), (128, 128, 4, 8)),
         ("all_128x128", (128, 128, 2, 8), (128, 128, 2, 8), (128, 128, 2, 8)),
         ("narrow_kv", (128, 64, 3, 4), (64, 64, 3, 4), (128, 64, 3, 4))],
    128: [("h100_rows", (128, 128, 2, 8), (64, 64, 2, 4), (128, 128, 2, 8)),
          ("all_128x128", (128, 128, 2, 8), (128, 128, 2, 8), (128, 128, 2, 8)),
          ("narrow_kv", (128, 64, 2, 8), (64, 128, 2, 8), (128, 64, 2, 8))],
}


def find_upstream():
    """Upstream's operator module, from $FOX_REFERENCE_SRC (directory holding its ``forgetting_transformer``
    package) or ``baseline/_ref`` of this checkout (pip install --target; git-ignored); None when absent."""
    import importlib
    for cand in (os.environ.get("FOX_REFERENCE_SRC"), os.path.join(ROOT, "baseline", "_ref")):
        if cand and os.path.isdir(os.path.join(cand, "forgetting_transformer")):
            if cand not in sys.path:
                sys.path.insert(0, cand)
            sys.dont_write_bytecode = True
            return importlib.import_module("forgetting_transformer.ops.forgetting_attention")
    return None


def time_upstream_triton(q, k, v, lf, dout, seq_d, thr, flops, n_configs, steps):
    """fwd + bwd of upstream's Triton operator on the same device tensors, CUDA-event timed like our own step,
    for the first ``n_configs`` rows of UPSTREAM_CONFIGS; returns the record for the JSON line (the best row's
    ms per step and TFLOP/s, every row's time, or the reason it could not run)."""
    try:
        up = find_upstream()
        if up is None:
            return {"unavailable": "no copy of the upstream package (FOX_REFERENCE_SRC or baseline/_ref)"}
        D = q.shape[-1]
        rows = {}
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for name, fwd, kv, qs in UPSTREAM_CONFIGS[D][:n_configs]:
            up.get_fwd_config = lambda *a, _c=fwd: _c
            up.get_bwd_kv_config = lambda *a, _c=kv: _c
            up.get_bwd_q_config = lambda *a, _c=qs: _c
            try:
                def ustep():
                    q.grad = k.grad = v.grad = lf.grad = None
                    up.forgetting_attention(q, k, v, lf, head_first=True, seq_start=seq_d,
                                            adaptive_threshold=thr).backward(dout)
                for _ in range(2):
                    ustep()
                torch.cuda.synchronize()
                e0.record()
                for _ in range(steps):
                    ustep()
                e1.record()
                torch.cuda.synchronize()
                rows[name] = e0.elapsed_time(e1) / steps
            except Exception as exc:  # a configuration that does not fit (shared memory) or does not compile
                rows[name] = f"{type(exc).__name__}: {str(exc)[:200]}"
        q.grad = k.grad = v.grad = lf.grad = None
        timed = {n: t for n, t in rows.items() if isinstance(t, float)}
        if not timed:
            return {"unavailable": "no block configuration ran", "configs": rows}
        best = min(timed, key=timed.get)
        import triton
        return {"ms_per_step": timed[best], "tflops": flops / (timed[best] * 1e-3) / 1e12, "best_config": best,
                "config_table": {n: dict(zip(("fwd", "bwd_kv", "bwd_q"), c)) for n, *c in UPSTREAM_CONFIGS[D][:n_configs]},
                "ms_per_step_by_config": rows, "steps": steps, "triton": triton.__version__,
                "note": "upstream's Triton kernels, block-size hooks overridden (they raise on sm_100), same tensors"}
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}


# --------------------------------------------------------------------------- GPU arm
def run_ours(args, w, wname):
    import torch.distributed as dist
    import forgetting_transformer_b200 as fox
    from forgetting_transformer_b200 import _lib, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (sm_100a); the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.load()

    host = make_inputs(w, rank, pin=True)
    seq = host["seq_start"]
    flops, pairs = flops_of(w, seq)
    cp = bool(w.get("context_parallel")) and world > 1
    if cp:
        # strong scaling: one sequence, every rank keeps its two zig-zag chunks; per-rank share of the FLOPs
        from forgetting_transformer_b200 import sharding
        tc = w["T"] // (2 * world)
        c0, c1 = sharding.zigzag_chunks(world, rank)
        for n_ in ("q", "k", "v", "log_fgate", "dout"):
            t_ = host[n_]
            host[n_] = torch.cat([t_[:, :, c0 * tc:(c0 + 1) * tc], t_[:, :, c1 * tc:(c1 + 1) * tc]], dim=2).pin_memory()
        flops = flops / world
    seq_d = None if seq is None else seq.to(dev)
    d = {n: host[n].to(dev, non_blocking=True) for n in ("q", "k", "v", "log_fgate", "dout")}
    q, k, v, lf = [d[n].requires_grad_() for n in ("q", "k", "v", "log_fgate")]
    dout = d["dout"]
    thr = w["thr"]

    cp_group = sharding.context_parallel_group() if cp else None

    def attention(q_, k_, v_, lf_):
        if cp:
            return sharding.context_parallel_attention(q_, k_, v_, lf_, group=cp_group, adaptive_threshold=thr)
        return fox.forgetting_attention(q_, k_, v_, lf_, head_first=True, seq_start=seq_d, adaptive_threshold=thr)

    def step():
        q.grad = k.grad = v.grad = lf.grad = None
        out = attention(q, k, v, lf)
        out.backward(dout)
        return out

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup if args.no_e2e else max(args.warmup, 3)):
        step()
    barrier()
    _lib.check_status()

    # ---- timed region: K steps, device-timed, inputs resident in HBM ----
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ops.KernelTimer() as timer:
        barrier()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier()
    clocks = sampler.stop() if rank == 0 else None
    _lib.check_status()
    ms = e0.elapsed_time(e1)
    kern = timer.summary()
    launches = sum(n for n, _ in kern.values())
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())
    ms_per_step = ms_max / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the public API with host buffers ----
    # Every step copies its inputs from pinned host memory and its results (out + four gradients) back;
    # HostStreamedAttention overlaps the copies of neighbouring steps with the kernels (three streams,
    # two buffer sets), so the timed region holds K complete host-to-host steps.
    from forgetting_transformer_b200.host_pipeline import HostStreamedAttention
    h2d = sum(host[n].numel() * host[n].element_size() for n in ("q", "k", "v", "log_fgate", "dout"))
    e2e_val, d2h, n_e2e = None, 0, 0
    if not args.no_e2e:
        pipe = HostStreamedAttention(dev, seq_start=seq_d, adaptive_threshold=thr,
                                     attention=(lambda q_, k_, v_, lf_: attention(q_, k_, v_, lf_)) if cp else None)
        for _ in range(args.e2e_warmup):
            pipe.submit(host)
        pipe.finish()
        barrier()
        d2h = pipe.d2h_bytes
        n_e2e = max(6, min(args.steps, 20))
        barrier()
        e0.record()
        for _ in range(n_e2e):
            pipe.submit(host)
        pipe.finish()            # the last step's results are on the host
        e1.record()
        barrier()
        t2 = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t2, op=dist.ReduceOp.MAX)
        e2e_val = world * flops / (float(t2.item()) / n_e2e * 1e-3) / 1e12
        del pipe

    # ---- launch-bound shapes: the same step replayed from CUDA graphs (forward graph + backward graph) ----
    graphed = None
    if world == 1 and ms_per_step < 1.0 and not args.no_e2e:
        gq, gk, gv, gl = [t.detach().clone().requires_grad_() for t in (q, k, v, lf)]
        gf = fox.make_graphed(gq, gk, gv, gl, head_first=True, seq_start=seq_d, adaptive_threshold=thr)

        def gstep():
            gq.grad = gk.grad = gv.grad = gl.grad = None
            gf(gq, gk, gv, gl).backward(dout)

        for _ in range(5):
            gstep()
        barrier()
        n_g = max(args.steps, 50)
        e0.record()
        for _ in range(n_g):
            gstep()
        e1.record()
        barrier()
        ms_g = e0.elapsed_time(e1) / n_g
        graphed = {"ms_per_step": ms_g, "value": flops / (ms_g * 1e-3) / 1e12, "unit": UNIT, "steps": n_g,
                   "speedup_over_eager_launches": ms_per_step / ms_g}

    # ---- the context-parallel configuration (cfg5's attention) beside the sharded one, whenever N > 1 ----
    cp_leg = None
    if world > 1 and not cp and not args.no_cp:
        cp_leg = context_parallel_leg(world, rank, dev)

    # ---- upstream's Triton operator on the same tensors (single GPU, not context parallel) ----
    upstream = None
    if world == 1 and not cp and args.upstream_configs > 0:
        upstream = time_upstream_triton(q, k, v, lf, dout, seq_d, thr, flops, args.upstream_configs,
                                        max(3, min(args.steps, 5)))
        if "ms_per_step" in upstream:
            upstream["speedup_vs_upstream_triton"] = upstream["ms_per_step"] / ms_per_step

    # ---- pruning statistics and dense comparison (ACP workloads) ----
    acp = None
    if thr is not None:
        with torch.no_grad():
            _, _, si = ops.ForgettingAttention.apply(q, k, v, lf, seq_d, True, None, thr, False, True, None, False, False)
        T = w["T"]
        nmb = si.shape[-1]
        hi = torch.clamp((torch.arange(nmb, device=dev) + 1) * 128, max=T)
        skipped = (torch.minimum(si, hi[None, None, :]) // 128).sum().item()
        total = float(torch.ceil(hi / 128).sum().item()) * si.shape[0] * si.shape[1]
        pfrac = skipped / total
        n_off = max(3, min(args.steps, 5))

        def step_off():
            q.grad = k.grad = v.grad = lf.grad = None
            out = fox.forgetting_attention(q, k, v, lf, head_first=True, seq_start=seq_d, adaptive_threshold=None)
            out.backward(dout)

        step_off()
        barrier()
        e0.record()
        for _ in range(n_off):
            step_off()
        e1.record()
        barrier()
        ms_off = e0.elapsed_time(e1) / n_off
        acp = {"pruned_tile_fraction": pfrac, "ms_per_step_pruning_off": ms_off, "speedup": ms_off / ms_per_step,
               "speedup_predicted_by_pruned_fraction": 1.0 / max(1.0 - pfrac, 1e-9),
               "executed_tflops": value * (1.0 - pfrac)}

    # ---- HBM-bound kernels: fused per-head RMSNorm + gate at the FoX-Pro layer shape ----
    normgate = None
    if world == 1 and not args.no_e2e:
        tokens, G, Dh = 65536, 24, 64
        m = fox.FusedGroupNormGated(G, G * Dh, is_rms_norm=True, eps=1e-6, activation="sigmoid").to(dev)
        x = torch.randn(1, tokens, G * Dh, device=dev, dtype=torch.bfloat16).requires_grad_()
        gate = torch.randn(1, tokens, G * Dh, device=dev, dtype=torch.bfloat16).requires_grad_()
        dy = torch.randn(1, tokens, G * Dh, device=dev, dtype=torch.bfloat16)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]

        def timed(fwd_fn, grad, leaves, n_it=10):
            """Mean device time of n_it forwards queued back to back, then of their n_it backwards (queued, so
            that the host's launch latency is not inside the timed intervals of these 0.1-0.4 ms kernels)."""
            for _ in range(3):
                fwd_fn().backward(grad)
            outs = [fwd_fn() for _ in range(n_it)]   # untimed: lets the caching allocator grow to n_it live outputs
            del outs
            torch.cuda.synchronize()
            ev[0].record()
            outs = [fwd_fn() for _ in range(n_it)]
            ev[1].record()
            for o_ in outs:
                for leaf in leaves:        # no gradient accumulation kernels inside the timed interval
                    leaf.grad = None
                o_.backward(grad)
            ev[2].record()
            torch.cuda.synchronize()
            return ev[0].elapsed_time(ev[1]) / n_it, ev[1].elapsed_time(ev[2]) / n_it

        tf, tb = timed(lambda: m(x, gate), dy, (x, gate, m.weight))
        n_el = tokens * G * Dh
        normgate = {"shape": "tokens 65536 x 24 heads x 64", "fwd_ms": tf, "bwd_ms": tb,
                    "fwd_gbs": (6 * n_el + 4 * tokens * G) / (tf * 1e-3) / 1e9,
                    "bwd_gbs_incl_host_dw_sum": (10 * n_el + 4 * tokens * G) / (tb * 1e-3) / 1e9}
        # the other two HBM-bound operators of the FoX-Pro layer: per-head RMSNorm of q / k, token shift of k / v
        qkn = fox.GroupNorm(G, G * Dh, is_rms_norm=True).to(dev)
        f_ms, b_ms = timed(lambda: qkn(x), dy, (x, qkn.weight))
        normgate["qk_norm"] = {"fwd_ms": f_ms, "bwd_ms": b_ms,
                               "fwd_gbs": (4 * n_el + 4 * tokens * G) / (f_ms * 1e-3) / 1e9,
                               "bwd_gbs_incl_host_dw_sum": (6 * n_el + 4 * tokens * G) / (b_ms * 1e-3) / 1e9}
        x4 = x.detach().view(1, tokens, G, Dh).requires_grad_()
        alpha = torch.rand(1, tokens, G, device=dev).requires_grad_()
        f_ms, b_ms = timed(lambda: fox.token_shift(x4, alpha, 1.0 - alpha), dy.view(1, tokens, G, Dh), (x4, alpha))
        # the block's input norm (row RMSNorm, hidden 1536) and the MLP's SwiGLU (65536 x 4096 per half)
        rn = fox.RMSNorm(G * Dh, eps=1e-6).to(dev)
        f2, b2 = timed(lambda: rn(x), dy, (x, rn.weight))
        normgate["row_rms_norm"] = {"fwd_ms": f2, "bwd_ms": b2, "fwd_gbs": 4 * n_el / (f2 * 1e-3) / 1e9,
                                    "bwd_gbs_incl_host_dw_sum": 6 * n_el / (b2 * 1e-3) / 1e9}
        gx = torch.randn(tokens, 4096, device=dev, dtype=torch.bfloat16).requires_grad_()
        gy = torch.randn(tokens, 4096, device=dev, dtype=torch.bfloat16).requires_grad_()
        gdz = torch.randn(tokens, 4096, device=dev, dtype=torch.bfloat16)
        f3, b3 = timed(lambda: fox.swiglu(gx, gy), gdz, (gx, gy))
        n_g = tokens * 4096
        normgate["swiglu"] = {"fwd_ms": f3, "bwd_ms": b3, "fwd_gbs": 6 * n_g / (f3 * 1e-3) / 1e9,
                              "bwd_gbs": 10 * n_g / (b3 * 1e-3) / 1e9}
        del gx, gy, gdz
        normgate["token_shift"] = {"fwd_ms_incl_1_minus_alpha": f_ms, "bwd_ms": b_ms,
                                   "fwd_gbs": (4 * n_el + 8 * tokens * G) / (f_ms * 1e-3) / 1e9,
                                   "bwd_gbs": (6 * n_el + 16 * tokens * G) / (b_ms * 1e-3) / 1e9}

    # ---- the FoX-Pro block of config 5 around the attention (single GPU): Linear layers are cuBLAS, the rest
    #      this library's kernels; reported beside the attention-only numbers, not as the metric ----
    block = None
    if world == 1 and wname == "cfg5_attn" and not args.no_e2e:
        hidden, inter = w["H"] * w["D"], 4096
        blk = fox.FoxProBlock(hidden, w["H"], inter, fgate_bias=5.0).to(dev).to(torch.bfloat16)
        xb = torch.randn(w["B"], w["T"], hidden, device=dev, dtype=torch.bfloat16).requires_grad_()
        dyb = torch.randn(w["B"], w["T"], hidden, device=dev, dtype=torch.bfloat16)
        for _ in range(2):
            blk(xb).backward(dyb)
        torch.cuda.synchronize()
        n_blk = 3
        with ops.KernelTimer() as btimer:
            e0.record()
            for _ in range(n_blk):
                blk(xb).backward(dyb)
            e1.record()
            torch.cuda.synchronize()
        bk = btimer.summary()
        ms_blk = e0.elapsed_time(e1) / n_blk
        tokens_b = w["B"] * w["T"]
        lin_flops = 6.0 * tokens_b * (5 * hidden * hidden + 3 * hidden * inter + 3 * hidden * w["H"])
        block = {"shape": f"B{w['B']} T{w['T']} hidden {hidden}, {w['H']} heads, SwiGLU {inter}, bf16 weights",
                 "ms_per_step": ms_blk,
                 "attention_kernels_ms": sum(v_[1] * v_[0] / n_blk for k_, v_ in bk.items()),
                 "attention_flops": flops, "linear_flops": lin_flops,
                 "tflops_total": (flops + lin_flops) / (ms_blk * 1e-3) / 1e12}
        del blk, xb, dyb
        # generation step on the same cache: one query row against all N keys (split-KV decode kernels), beside
        # the same call through the general forward kernel (what a call with gradients enabled takes)
        q1 = q.detach()[:, :, -1:, :].contiguous()
        def dec_step(grad):
            with torch.set_grad_enabled(grad):
                qq_ = q1.requires_grad_(grad)
                return fox.forgetting_attention(qq_, k.detach(), v.detach(), lf.detach(), head_first=True)
        times = {}
        for name_, grad in (("decode_kernels_ms", False), ("general_kernel_ms", True)):
            for _ in range(3):
                dec_step(grad)
            e0.record()
            for _ in range(20):
                dec_step(grad)
            e1.record()
            torch.cuda.synchronize()
            times[name_] = e0.elapsed_time(e1) / 20
        kv_bytes = 2 * k.numel() * k.element_size()
        block["decode_step"] = dict(times, keys=w["T"], kv_gbs_decode_incl_prefix_sum=kv_bytes / (times["decode_kernels_ms"] * 1e-3) / 1e9)

    if rank == 0:
        peaks = load_peaks()
        bwd_n, bwd_ms = kern.get("fox_attn_bwd", (0, float("nan")))
        fwd_n, fwd_ms = kern.get("fox_attn_fwd", (0, float("nan")))
        # executed FLOPs of the dominant kernel (backward: 10 of the 14 per pair)
        # (a context-parallel step launches each kernel once per local chunk: FLOPs per step over launches per step)
        bwd_tf = (10.0 / 14.0) * flops / (bwd_ms * max(bwd_n // args.steps, 1) * 1e-3) / 1e12
        fwd_tf = (4.0 / 14.0) * flops / (fwd_ms * max(fwd_n // args.steps, 1) * 1e-3) / 1e12
        dq_n, dq_ms = kern.get("fox_attn_bwd_dq", (0, float("nan")))
        two_kernel = dq_n > 0
        bwd_kernel_name = "fox_attn_bwd_kernel"
        if two_kernel:
            # head dim 128: the backward is a key-side kernel (S^T, dP^T, dV, dK: 8 of the 14 FLOPs per pair) and a
            # query-side kernel (S and dP recomputed, dQ: 6 per pair executed, 2 of them algorithmic). The roofline
            # entry is the longer of the two with the FLOPs it executes; the pair's algorithmic rate is beside it.
            per = max(bwd_n // args.steps, 1)
            key_tf = (8.0 / 14.0) * flops / (bwd_ms * per * 1e-3) / 1e12
            qry_tf = (6.0 / 14.0) * flops / (dq_ms * max(dq_n // args.steps, 1) * 1e-3) / 1e12
            pair_tf = (10.0 / 14.0) * flops / ((bwd_ms + dq_ms) * per * 1e-3) / 1e12
            two = {"key_side": {"kernel": "fox_attn_bwd_kv_kernel", "ms_per_launch": bwd_ms, "executed_tflops": key_tf,
                                "frac": key_tf / peaks["bf16"], "frac_of_sustained_peak": key_tf / peaks["bf16_sustained"]},
                   "query_side": {"kernel": "fox_attn_bwd_dq2_kernel", "ms_per_launch": dq_ms, "executed_tflops": qry_tf,
                                  "frac": qry_tf / peaks["bf16"], "frac_of_sustained_peak": qry_tf / peaks["bf16_sustained"]},
                   "algorithmic_tflops_of_the_pair": pair_tf,
                   "algorithmic_frac_of_the_pair": pair_tf / peaks["bf16"]}
            if dq_ms > bwd_ms:
                bwd_kernel_name, bwd_tf, bwd_ms, bwd_n = "fox_attn_bwd_dq2_kernel", qry_tf, dq_ms, dq_n
            else:
                bwd_kernel_name, bwd_tf = "fox_attn_bwd_kv_kernel", key_tf
        roof = {
            "kernel": bwd_kernel_name, "bound": "tensor", "achieved": bwd_tf,
            "peak": peaks["bf16"], "unit": "TFLOP/s", "frac": bwd_tf / peaks["bf16"],
            "peak_kind": (f"bf16_tflops (burst) of {peaks['source']}: the timed region lasts a fraction of a second at "
                          "full clocks; the sustained figure is beside it"),
            "frac_of_sustained_peak": bwd_tf / peaks["bf16_sustained"],
            "traffic": TRAFFIC_BYTES_PER_LAUNCH.get((wname, bwd_kernel_name), TRAFFIC_BYTES_PER_LAUNCH.get(wname)),
            "ms_per_launch": bwd_ms, "launches": bwd_n,
            "fwd_kernel": {"achieved": fwd_tf, "frac": fwd_tf / peaks["bf16"],
                           "frac_of_sustained_peak": fwd_tf / peaks["bf16_sustained"], "ms_per_launch": fwd_ms},
            "all_kernels_ms": {k_: round(v_[1], 4) for k_, v_ in kern.items()},
        }
        if two_kernel:
            roof["backward_two_kernels"] = two
        if thr is None and not cp and not two_kernel:
            # what actually bounds the one-pass backward: every (KV tile, query tile) pair add-reduces a 128 x D
            # fp32 dQ partial into L2, whose reduction rate is chip-wide (~1.54 KB/clk = 3.03 TB/s at 1965 MHz,
            # measured with a stand-alone probe on this pool; not part of MEASURED_PEAKS.json)
            nT = (w["T"] + 127) // 128
            pairs_t = 0
            for b_ in range(w["B"]):
                s0 = 0 if seq is None else int(seq[b_])
                j0 = max((s0 - 1) // 128, 0) if s0 > 0 else 0
                pairs_t += sum(nT - j for j in range(j0, nT))
            red_bytes = float(pairs_t) * w["H"] * 128 * w["D"] * 4
            roof["l2_reduction"] = {"bytes_per_launch": red_bytes, "achieved_gbs": red_bytes / (bwd_ms * 1e-3) / 1e9,
                                    "probe_peak_gbs": 3030.0,
                                    "frac": red_bytes / (bwd_ms * 1e-3) / 1e9 / 3030.0}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong" if cp else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": wname, "description": DESCR[wname], "per_gpu_batch": w["B"],
                       "global_batch": w["B"] * (1 if cp else world), "seq_len": w["T"], "heads": w["H"],
                       "head_dim": w["D"],
                       "sharding": ("context parallel: zig-zag sequence chunks, batched NCCL point-to-point transfers of "
                                    "K, V and log-gate chunk slabs, partial gradients summed by the owner") if cp else
                                   "independent (batch, head) units per rank, no collective",
                       "l2": "inputs (>=400 MB per step) larger than the 126 MB L2; no explicit flush",
                       "algorithmic_flops_per_step_per_gpu": flops,
                       "frac_of_bf16_peak": value / world / peaks["bf16"],
                       "frac_of_nominal_2250": value / world / 2250.0},
            "roofline": roof,
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": n_e2e},
            "gpu_launches": launches,
            "clocks": clocks,
        }
        if cp_leg is not None:
            line["context_parallel"] = cp_leg
        if upstream is not None:
            line["upstream_triton"] = upstream
        if graphed is not None:
            line["cuda_graph"] = graphed
        if acp is not None:
            line["acp"] = acp
        if block is not None:
            line["fox_pro_block"] = block
        if normgate is not None:
            normgate["frac_of_hbm_peak_fwd"] = normgate["fwd_gbs"] / peaks["hbm_gbs"]
            line["normgate"] = normgate
        n_vec = w["B"] * w["H"] * w["T"]
        aux = {}
        for name, bytes_ in (("fox_cumsum_fwd", 8 * n_vec), ("fox_revcumsum", 12 * n_vec),
                             ("fox_bwd_delta", 2 * 2 * n_vec * w["D"] + 4 * n_vec),
                             ("fox_dq_convert", 6 * n_vec * w["D"])):
            if name in kern:
                aux[name] = {"ms": kern[name][1], "gbs": bytes_ / (kern[name][1] * 1e-3) / 1e9}
        line["hbm_kernels"] = aux
        if world == 1 and not args.no_cpu:
            dt, fl, desc = cpu_sample(w, os.cpu_count() or 1, cpu_rows(w))
            line["cpu_baseline"] = {"value": fl / dt / 1e12, "unit": UNIT, "cores": os.cpu_count() or 1,
                                    "kind": "port", "sample": desc, "seconds": dt}
        _emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# DRAM bytes (read + write) of one backward-kernel launch from an ncu capture of the profiler-sized cases,
# per workload (None = not captured).
TRAFFIC_BYTES_PER_LAUNCH = {
    # backward kernel: 264.4 MB measured on prof_d64; the traffic is per-row (inputs once, outputs once, dQ
    # workspace once), cfg3 has 3x the rows
    "cfg3": 3 * 264.4e6,
    "prof_d64": 264.4e6,
    # head dim 128, one-pass kernel (FOX_B200_ONE_PASS_BWD=1)
    "prof_d128": 632.8e6,
    "cfg4": 4 * 632.8e6,
    # head dim 128, the kernel pair; cfg4 has 4x the rows of prof_d128
    ("prof_d128", "fox_attn_bwd_kv_kernel"): 380.1e6,
    ("prof_d128", "fox_attn_bwd_dq2_kernel"): 325.3e6,
    ("cfg4", "fox_attn_bwd_kv_kernel"): 4 * 380.1e6,
    ("cfg4", "fox_attn_bwd_dq2_kernel"): 4 * 325.3e6,
}


def _emit(line: dict) -> None:
    """Write the one JSON line to the real stdout (see main: fd 1 is pointed at stderr while the
    benchmark runs so that library banners, e.g. NCCL's version line, cannot land next to it)."""
    data = (json.dumps(line) + "\n").encode()
    os.write(_REAL_STDOUT if _REAL_STDOUT is not None else 1, data)


_REAL_STDOUT = None


def main():
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiler runs)")
    ap.add_argument("--e2e-warmup", type=int, default=3, help="untimed host-to-host steps before the end-to-end leg")
    ap.add_argument("--no-cp", action="store_true", help="N > 1: skip the context-parallel leg (cfg5's attention)")
    ap.add_argument("--upstream-configs", type=int, default=2,
                    help="rows of UPSTREAM_CONFIGS to time upstream's Triton operator with (0: skip that leg)")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, w, args.workload)
    else:
        run_ours(args, w, args.workload)


if __name__ == "__main__":
    main()
