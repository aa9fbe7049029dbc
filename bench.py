#!/usr/bin/env python
"""Benchmark of the compiled MLP training step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4] [--impl b200|reference]

One "step" is one full training step (forward, MSE, backward, optimizer update) on one
batch of seeded synthetic input.  Prints ONE JSON line:
  value       whole-job samples/s with inputs resident in HBM, timed with CUDA events on the
              library's own stream, max over ranks
  e2e         the same metric through the C-ABI step call with pinned HOST inputs (host->device
              copy of X and Y and a device->host read of the loss inside the timed region)
  roofline    the dominant kernel against the measured tensor / HBM peak (TF32 dense peak measured
              in this run the way the bf16 denominator was: a cuBLAS GEMM, burst and sustained)
  cpu_baseline  the reference's CPU path (its gemm_shim.c, compiled unmodified, under the
              restated step) timed on this host's cores (N = 1 only): the small configurations with
              the reference's own protocol, the large ones on bounded samples, one process per core
  config      names the workload; also carries the final loss (the same at every GPU count to
              rounding), a repeat-run bit-identity check, and - in the default run - configuration 5
              (4096-16384-16384-4096-1, Adam, batch 131072) timed the same way
`--impl reference` times only the CPU path and prints the same line shape.
Under torchrun (N > 1) the global batch is sharded over the ranks (strong scaling).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

L2_BYTES = 126e6


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# DRAM traffic (ncu: dram__bytes_read.sum + dram__bytes_write.sum) per batch row of one launch of the
# CTA-pair GEMM at configuration 4's widths, captured at batch 8192; the traffic of these GEMMs grows
# in proportion to the batch, so a full launch is rows x this figure.
NCU_TRAFFIC_PER_ROW = {
    "fwd_gemm_nn_Bx4096x4096": (620.370688e6 + 246.531584e6) / 8192,
    "fwd_gemm_nn_Bx1024x4096": (200.767232e6 + 44.852224e6) / 8192,
    "dX_gemm_nt_Bx4096x4096": (754.393088e6 + 131.598336e6) / 8192,
    "dW_gemm_tn_4096x4096xB": (615.041280e6 + 130.149376e6) / 8192,   # K split in two: two slabs written
}


def ncu_traffic_bytes(kernel_name: str, rows: int):
    import re
    m = re.match(r"(fwd|dW|dX)\d+_gemm_(nn|nt|tn)_(\d+)x(\d+)x(\d+)", kernel_name)
    if not m:
        return None
    fam, lay, a, b, c = m.group(1), m.group(2), int(m.group(3)), int(m.group(4)), int(m.group(5))
    key = "%s_gemm_%s_Bx%dx%d" % (fam, lay, b, c) if fam != "dW" else "%s_gemm_%s_%dx%dxB" % (fam, lay, a, b)
    per_row = NCU_TRAFFIC_PER_ROW.get(key)
    return per_row * rows if per_row else None


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU every 200 ms while running."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.stop_flag, self.sm, self.reasons, self.sm_max, self.power = index, False, [], set(), None, []
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def run(self):
        while not self.stop_flag and self.nv is not None:
            try:
                self.sm.append(int(self.nv.nvmlDeviceGetClockInfo(self.dev, self.nv.NVML_CLOCK_SM)))
                self.power.append(self.nv.nvmlDeviceGetPowerUsage(self.dev) / 1000.0)
                mask = int(self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.dev))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.2)

    def summary(self):
        if not self.sm:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(self.sm)), "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons),
                "samples": len(self.sm), "power_w_max": max(self.power) if self.power else None}


# ------------------------------------------------------------------------------ CPU arm
def _oracle_with_reference_gemm(cfg, B, layers=None, optimizer=None):
    from oracle.oracle import Oracle
    o = Oracle(layers or list(cfg.layers), cfg.activation, optimizer or cfg.optimizer, B)
    flavour = o.use_reference_gemm()
    return o, flavour


def cpu_protocol_run(cfg, inputs: str, warm: int = 10, inner: int = 7, optimizer=None, steps=None):
    """The reference's own measurement protocol (docs/BENCHMARKS.md:11-26) on one configuration, in full: `warm`
    untimed steps, then `inner` runs of the configuration's step count each, per-step time of every run; the
    median, minimum and maximum over the runs.  inputs = "seeded" (the configuration's seeded tensors and
    Kaiming weights) or "closed_form" (the reference's X[i] = (i%17)*0.01-0.08, Y[i] = (i%7)*0.1 with its default
    LCG-Xavier weights).  One core: the reference's GEMM shim is not re-entrant."""
    from volta_b200 import synth
    layers, B = list(cfg.layers), cfg.batch
    steps = steps or cfg.steps
    o, flavour = _oracle_with_reference_gemm(cfg, B, optimizer=optimizer)
    if inputs == "seeded":
        for i, (w, b) in enumerate(zip(*synth.kaiming_uniform_weights(layers, 42))):
            o.set_params(i, w, b)
        x = synth.rows(cfg.x_dist, 1234, 0, B, layers[0])
        y = synth.rows(cfg.y_dist, 4321, 0, B, layers[-1])
    else:
        x = ((np.arange(B * layers[0]) % 17) * 0.01 - 0.08).astype(np.float32).reshape(B, layers[0])
        y = ((np.arange(B * layers[-1]) % 7) * 0.1).astype(np.float32).reshape(B, layers[-1])
    for _ in range(warm):
        o.step(x, y, cfg.lr)
    runs = []
    for _ in range(inner):
        t0 = time.perf_counter()
        for _ in range(steps):
            o.step(x, y, cfg.lr)
        runs.append((time.perf_counter() - t0) / steps * 1e3)
    med = float(np.median(runs))
    out = {"ms_per_step_median": med, "ms_per_step_min": float(min(runs)), "ms_per_step_max": float(max(runs)),
           "samples_per_s": B / (med * 1e-3), "batch": B, "optimizer": optimizer or cfg.optimizer, "inputs": inputs,
           "protocol": "%d warm-up steps, %d runs x %d steps" % (warm, inner, steps), "cores": 1,
           "gemm": flavour or "oracle loops", "loss": o.loss()}
    o.free()
    return out


def _cpu_shard_worker(rank, world, port, cfg_name, B_global, steps, warm, out_path):
    """One CPU process of the many-core baseline: the reference GEMM shim under the restated step on this
    process's row shard, gradients summed over the processes (gloo), the same update everywhere."""
    import torch
    import torch.distributed as dist
    torch.set_num_threads(1)
    os.environ.setdefault("OMP_NUM_THREADS", "1")
    from volta_b200 import CONFIGS, synth
    cfg = CONFIGS[cfg_name]
    layers = list(cfg.layers)
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    B = B_global // world
    o, flavour = _oracle_with_reference_gemm(cfg, B)
    o.set_global_batch(B_global)
    for i, (w, b) in enumerate(zip(*synth.kaiming_uniform_weights(layers, 42))):
        o.set_params(i, w, b)
    x = synth.rows(cfg.x_dist, 1234, rank * B, B, layers[0])
    y = synth.rows(cfg.y_dist, 4321, rank * B, B, layers[-1])
    gw, gb = o.grad_views()
    flat = [torch.from_numpy(g) for g in gw + gb]
    times = []
    for it in range(warm + steps):
        dist.barrier()
        t0 = time.perf_counter()
        o.grad_step(x, y)
        for t in flat:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        o.update(cfg.lr)
        dist.barrier()
        if it >= warm:
            times.append(time.perf_counter() - t0)
    loss = torch.tensor([o.loss()], dtype=torch.float64)
    dist.all_reduce(loss, op=dist.ReduceOp.SUM)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump({"ms_per_step": float(np.median(times)) * 1e3, "loss": float(loss.item()), "gemm": flavour}, f)
    dist.destroy_process_group()


def cpu_many_core_run(cfg, B_global: int, procs: int, steps: int = 2, warm: int = 1):
    """The reference's CPU path on `procs` cores: one process per core, each with its rows of the batch."""
    import socket
    import tempfile
    import torch.multiprocessing as mp
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    out = os.path.join(tempfile.mkdtemp(), "r.json")
    mp.spawn(_cpu_shard_worker, args=(procs, port, cfg.name, B_global, steps, warm, out), nprocs=procs, join=True)
    with open(out) as f:
        r = json.load(f)
    ms = r["ms_per_step"]
    return {"batch": B_global, "processes": procs, "rows_per_process": B_global // procs, "ms_per_step": ms,
            "samples_per_s": B_global / (ms * 1e-3), "gflops": cfg.flops_per_step(B_global) / (ms * 1e-3) / 1e9,
            "steps": steps, "warmup": warm, "loss": r["loss"], "gemm": r["gemm"]}


def usable_cores() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return max(1, os.cpu_count() or 1)


def cpu_reference_arm(cfg, quick: bool = False):
    """The CPU baseline of one configuration.  Small configurations (one step well under a second) are timed
    in full with the reference's protocol on one core.  Large ones are timed on two reduced batches, one
    process per core on its row shard; the per-sample time must agree between the two (the step is linear in
    the batch) and is what the full batch is extrapolated with.  Returns the cpu_baseline object."""
    cores = usable_cores()
    procs = 1
    while procs * 2 <= cores:
        procs *= 2
    if cfg.flops_per_step() < 5e9:
        r = cpu_protocol_run(cfg, "seeded", warm=10, inner=3 if quick else 7)
        return {"value": r["samples_per_s"], "unit": "samples/s", "cores": 1, "kind": "reference" if r["gemm"] != "oracle loops" else "port",
                "sample": "workload %s in full, the reference's protocol (%s), median; its gemm_shim.c (%s build, one core: "
                          "the shim is not re-entrant) under the restated step" % (cfg.name, r["protocol"], r["gemm"]),
                "ms_per_step": r["ms_per_step_median"], "detail": r, "host_cpus": os.cpu_count()}
    batches = [b for b in (1024, 4096) if b <= cfg.batch and b % procs == 0]
    if quick or cfg.flops_per_step(4096) > 3e12:
        batches = batches[:1] if cfg.flops_per_step(4096) <= 3e12 else [max(procs * 16, 256)]
    points = [cpu_many_core_run(cfg, b, procs, steps=2, warm=1) for b in batches]
    per_sample = [p["ms_per_step"] / p["batch"] for p in points]
    best = points[-1]
    value = best["samples_per_s"]
    return {"value": value, "unit": "samples/s", "cores": procs, "kind": "reference" if best["gemm"] else "port",
            "sample": "workload %s at batch %s of %d (the step is linear in the batch: %s ms per sample), %d warm-up + %d "
                      "timed steps each, median; %d processes, one per core, each running the reference's gemm_shim.c (%s "
                      "build, not re-entrant, hence processes) under the restated step on its rows, gradients summed "
                      "over the processes" % (cfg.name, " and ".join(str(b) for b in batches), cfg.batch,
                                              " / ".join("%.4f" % v for v in per_sample), 1, 2, procs, best["gemm"]),
            "ms_per_step_extrapolated_full_batch": cfg.batch / value * 1e3, "points": points,
            "linearity": (max(per_sample) / min(per_sample) if len(per_sample) > 1 else None),
            "gflops": best["gflops"], "host_cpus": os.cpu_count()}


def torch_cpu_run(cfg, B: int, steps: int = 3):
    """Second CPU line: PyTorch eager on all host cores, as examples/bench_pytorch.py does."""
    import torch
    torch.set_num_threads(usable_cores())
    layers = list(cfg.layers)
    acts = {"relu": torch.relu, "silu": torch.nn.functional.silu, "sigmoid": torch.sigmoid, "tanh": torch.tanh,
            "leaky_relu": lambda t: torch.nn.functional.leaky_relu(t, 0.01),
            "gelu": lambda t: torch.nn.functional.gelu(t, approximate="tanh")}
    ws = [torch.randn(r, c, requires_grad=True) for r, c in zip(layers[:-1], layers[1:])]
    bs = [torch.zeros(c, requires_grad=True) for c in layers[1:]]
    opt = {"sgd": lambda p: torch.optim.SGD(p, lr=cfg.lr), "sgd_momentum": lambda p: torch.optim.SGD(p, lr=cfg.lr, momentum=0.9),
           "adam": lambda p: torch.optim.Adam(p, lr=cfg.lr), "adamw": lambda p: torch.optim.AdamW(p, lr=cfg.lr),
           "adagrad": lambda p: torch.optim.Adagrad(p, lr=cfg.lr)}[cfg.optimizer](ws + bs)
    x, y = torch.randn(B, layers[0]), torch.randn(B, layers[-1])
    times = []
    for it in range(steps + 1):
        t0 = time.perf_counter()
        h = x
        for i, (w, b) in enumerate(zip(ws, bs)):
            h = h @ w + b
            if i < len(ws) - 1:
                h = acts[cfg.activation](h)
        loss = torch.mean((h - y) ** 2)
        opt.zero_grad()
        loss.backward()
        opt.step()
        if it:
            times.append(time.perf_counter() - t0)
    med = float(np.median(times))
    return {"value": B / med, "unit": "samples/s", "cores": usable_cores(), "batch": B, "ms_per_step": med * 1e3}


# ------------------------------------------------------------------------------ GPU arm
def measure_tf32_peak(seconds: float = 3.0):
    """Dense TF32 throughput of this GPU measured the way MEASURED_PEAKS.json measured bf16: torch.matmul (cuBLAS)
    on 8192^3 fp32 operands with TF32 allowed, best of 10 (burst) and back to back for a few seconds (sustained)."""
    import torch
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        c = torch.empty(n, n, device="cuda")
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch.matmul(a, b, out=c)
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        flops = 2.0 * n ** 3
        reps = max(10, int(seconds / (best * 1e-3)))
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch.matmul(a, b, out=c)
        e1.record()
        torch.cuda.synchronize()
        sustained = flops * reps / (e0.elapsed_time(e1) * 1e-3) / 1e12
        return {"tf32_tflops": flops / (best * 1e-3) / 1e12, "tf32_tflops_sustained": sustained,
                "how": "torch.matmul fp32 with allow_tf32, 8192^3: best of 10 (burst) and %d back to back (sustained)" % reps}
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


class Job:
    """torch.distributed plumbing shared by the workloads of one bench run."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
        torch.cuda.set_device(self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local_rank))

    def unique_id(self):
        from volta_b200.train import dp_unique_id
        if self.world == 1:
            return None
        box = [dp_unique_id() if self.rank == 0 else None]
        self.dist.broadcast_object_list(box, src=0)
        return box[0]

    def max_over_ranks(self, v: float) -> float:
        if self.world == 1:
            return v
        t = self.torch.tensor([v], device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def close(self):
        if self.world > 1:
            self.dist.destroy_process_group()


def run_workload(job: Job, cfg, args, steps: int, warmup: int, device_data: bool, profile: bool, e2e_steps=None):
    """Times one configuration on the job's GPUs.  Returns a dict of results (every rank computes it; the values
    that are maxima over ranks are the same everywhere)."""
    torch, dist, world, rank = job.torch, job.dist, job.world, job.rank
    from volta_b200 import TrainHandle, synth
    assert cfg.batch % world == 0
    B = cfg.batch // world
    layers = list(cfg.layers)
    lr = cfg.lr

    def make_handle():
        h = TrainHandle(layers, cfg.activation, cfg.optimizer, B, global_batch=cfg.batch, world_size=world, rank=rank,
                        unique_id=job.unique_id(), gemm_path=args.gemm_path,
                        fuse_sgd=(cfg.optimizer == "sgd" and world == 1),
                        dp_exchange="peer_copy" if (world > 1 and args.dp_mode == "copy") else "nccl")
        if world > 1 and args.dp_mode in ("fused", "copy"):
            handles = [None] * world
            dist.all_gather_object(handles, h.ipc_handle())
            h.attach_peers(handles)
        return h

    if device_data:
        weights = synth.kaiming_uniform_weights_cuda(layers, 42)
        x_dev = synth.rows_cuda(cfg.x_dist, 1234, rank * B, B, layers[0])
        y_dev = synth.rows_cuda(cfg.y_dist, 4321, rank * B, B, layers[-1])
        x_host = y_host = None
    else:
        weights = synth.kaiming_uniform_weights(layers, 42)
        x_host = torch.from_numpy(synth.rows(cfg.x_dist, 1234, rank * B, B, layers[0])).pin_memory()
        y_host = torch.from_numpy(synth.rows(cfg.y_dist, 4321, rank * B, B, layers[-1])).pin_memory()
        x_dev, y_dev = x_host.cuda(), y_host.cuda()

    def load(h):
        for i, (w, b) in enumerate(zip(*weights)):
            h.set_params(i, w, b)

    h = make_handle()
    load(h)
    stream = torch.cuda.ExternalStream(h.stream)

    def barrier():
        h.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    working_set = h.arena_bytes
    flush_needed = working_set < 2 * L2_BYTES
    flush_buf = torch.empty(int(256e6) // 4, device="cuda") if flush_needed else None

    for _ in range(warmup):
        h.step(x_dev, y_dev, lr)
    barrier()
    sampler = ClockSampler(job.local_rank)
    sampler.start()
    # ---- device-resident timing
    if flush_needed:
        per = []
        for _ in range(steps):
            with torch.cuda.stream(stream):
                flush_buf.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            h.step(x_dev, y_dev, lr)
            e1.record(stream)
            per.append((e0, e1))
        barrier()
        ms_total = sum(a.elapsed_time(b) for a, b in per)
    else:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            h.step(x_dev, y_dev, lr)
        e1.record(stream)
        barrier()
        ms_total = e0.elapsed_time(e1)
    ms_per_step = job.max_over_ranks(ms_total) / steps
    loss_dev = h.loss()
    steps_taken = warmup + steps

    # ---- end to end through the host-pointer step call
    e2e = None
    es = steps if e2e_steps is None else e2e_steps
    if es > 0:
        if x_host is None:
            x_host, y_host = x_dev.cpu().pin_memory(), y_dev.cpu().pin_memory()
        for _ in range(min(warmup, 2)):
            h.step(x_host, y_host, lr)
            h.loss()
        barrier()
        t0 = time.perf_counter()
        for _ in range(es):
            if flush_needed:
                with torch.cuda.stream(stream):
                    flush_buf.zero_()
            h.step(x_host, y_host, lr)
            h.loss()
        h.synchronize()
        e2e_s = job.max_over_ranks(time.perf_counter() - t0)
        barrier()
        e2e = {"value": cfg.batch / (e2e_s / es), "unit": "samples/s", "ms_per_step": e2e_s / es * 1e3,
               "h2d_bytes_per_step": int(world * 4 * B * (layers[0] + layers[-1])), "d2h_bytes_per_step": int(world * 8),
               "steps": es, "timer": "host wall clock, max over ranks", "includes_l2_flush": bool(flush_needed)}
    sampler.stop_flag = True
    sampler.join(timeout=2)

    # ---- per-kernel times (single GPU only; plain launches, event pairs)
    kernel_table, agg = None, None
    if profile and (world == 1 or args.dp_mode in ("nccl", "copy")):
        agg = {}
        reps = 3
        for _ in range(reps):
            for name, ms, fl, by in h.profile_step(x_dev, y_dev, lr):
                a = agg.setdefault(name, [0.0, fl, by])
                a[0] += ms / reps
        tot = sum(v[0] for v in agg.values())
        kernel_table = [{"kernel": k, "ms": round(v[0], 5), "share": round(v[0] / tot, 4),
                         "tflops": round(v[1] / v[0] / 1e9, 2) if v[1] else None,
                         "gbs": round(v[2] / v[0] / 1e6, 1)} for k, v in sorted(agg.items(), key=lambda kv: -kv[1][0])]
    kernels_per_step, arena = h.kernels_per_step, h.arena_bytes
    h.free()

    # ---- determinism: two fresh handles, the same few steps, the same bits (and the same on every rank)
    def short_run(nsteps=3 if cfg.flops_per_step() < 1e14 else 2):
        g = make_handle()
        load(g)
        for _ in range(nsteps):
            g.step(x_dev, y_dev, lr)
        bits = int(np.float32(g.loss()).view(np.uint32))
        g.free()
        return bits
    if args.lean:
        a_bits = b_bits = 0
    else:
        a_bits, b_bits = short_run(), short_run()
    same = a_bits == b_bits
    if world > 1:
        t = torch.tensor([a_bits, b_bits], device="cuda", dtype=torch.int64)
        lo, hi = t.clone(), t.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        same = same and bool((lo == hi).all().item())
    return {"ms_per_step": ms_per_step, "value": cfg.batch / (ms_per_step * 1e-3), "loss": loss_dev, "steps_taken": steps_taken,
            "e2e": e2e, "clocks": sampler.summary(), "kernels_per_step": kernels_per_step, "arena_bytes": arena,
            "flush_needed": flush_needed, "kernel_table": kernel_table, "agg": agg, "per_gpu_batch": B,
            "repeat_bit_identical": same, "loss_bits_after_3_steps": "0x%08x" % a_bits,
            "tflops_logical_fp32": cfg.flops_per_step() / (ms_per_step * 1e-3) / 1e12}


def roofline_of(res, cfg, peaks, tf32):
    """The dominant kernel of a profiled single-GPU run against its bound."""
    agg = res["agg"]
    if not agg:
        return None
    top, tv = max(agg.items(), key=lambda kv: kv[1][0])
    if tf32:
        tensor_peak = tf32["tf32_tflops_sustained"] / 3.0
        basis = "TF32 dense measured in this run (%s): %.1f TFLOP/s burst, %.1f sustained; / 3 for the three MMAs of a " \
                "3xTF32 product; achieved counts logical fp32 flops" % (tf32["how"], tf32["tf32_tflops"], tf32["tf32_tflops_sustained"])
    else:
        tensor_peak = peaks["bf16_tflops_sustained"] / 6.0
        basis = "%s bf16 sustained %.1f TFLOP/s / 6" % (peaks["source"], peaks["bf16_tflops_sustained"])
    if "gemm" in top and tv[1] / max(tv[2], 1) > 50:
        ach = tv[1] / tv[0] / 1e9
        roof = {"kernel": top, "bound": "tensor", "achieved": ach, "peak": tensor_peak, "unit": "TFLOP/s",
                "frac": ach / tensor_peak, "traffic": ncu_traffic_bytes(top, res["per_gpu_batch"]), "peak_basis": basis,
                "frac_of_bf16_sustained_over_6": ach / (peaks["bf16_tflops_sustained"] / 6.0)}
    else:
        ach = tv[2] / tv[0] / 1e6
        roof = {"kernel": top, "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": ach / peaks["hbm_gbs"], "traffic": None, "peak_basis": "%s STREAM-style copy" % peaks["source"]}
    gemm_ms = sum(v[0] for k, v in agg.items() if "gemm" in k)
    gemm_fl = sum(v[1] for k, v in agg.items() if "gemm" in k)
    roof["all_gemms_tflops"] = gemm_fl / gemm_ms / 1e9 if gemm_ms else None
    roof["all_gemms_frac"] = roof["all_gemms_tflops"] / tensor_peak if gemm_ms else None
    roof["whole_step_tflops"] = res["tflops_logical_fp32"]
    roof["whole_step_frac"] = res["tflops_logical_fp32"] / tensor_peak
    roof["gemms_below_0.60"] = [k for k, v in agg.items() if "gemm" in k and v[1] / max(v[2], 1) > 50 and v[1] / v[0] / 1e9 < 0.6 * tensor_peak]
    opt = agg.get("optimizer")
    if opt:
        roof["optimizer_gbs"] = opt[2] / opt[0] / 1e6
        roof["optimizer_frac_of_hbm"] = opt[2] / opt[0] / 1e6 / peaks["hbm_gbs"]
    if tf32:
        roof["tf32_measured"] = tf32
    return roof


def side_table(job: Job, args, flush_buf):
    """The single-GPU configurations, the reference's option examples and its inference protocol, briefly
    (device-resident inputs, L2 flushed between steps)."""
    torch = job.torch
    from volta_b200 import CONFIGS, TrainHandle, synth
    others = {}

    def timed(oh, ox, oy, lr, nsteps):
        ostream = torch.cuda.ExternalStream(oh.stream)
        for _ in range(5):
            oh.step(ox, oy, lr)
        oh.synchronize()
        pairs = []
        for _ in range(nsteps):
            with torch.cuda.stream(ostream):
                flush_buf.zero_()
            a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(ostream)
            oh.step(ox, oy, lr)
            b2.record(ostream)
            pairs.append((a, b2))
        oh.synchronize()
        torch.cuda.synchronize()
        ms = sorted(x.elapsed_time(y2) for x, y2 in pairs)
        return ms[len(ms) // 2]

    for name in ("c1", "c2", "c3_b64", "c3_b1024"):
        if name == args.workload:
            continue
        oc = CONFIGS[name]
        ol = list(oc.layers)
        oh = TrainHandle(ol, oc.activation, oc.optimizer, oc.batch, gemm_path=args.gemm_path, fuse_sgd=(oc.optimizer == "sgd"))
        for i, (w, b) in enumerate(zip(*synth.kaiming_uniform_weights(ol, 42))):
            oh.set_params(i, w, b)
        ox = torch.from_numpy(synth.rows(oc.x_dist, 1234, 0, oc.batch, ol[0])).cuda()
        oy = torch.from_numpy(synth.rows(oc.y_dist, 4321, 0, oc.batch, ol[-1])).cuda()
        med = timed(oh, ox, oy, oc.lr, oc.steps)
        opt_bytes = oc.optimizer_bytes_per_param() * oc.n_params
        others[name] = {"ms_per_step": med, "samples_per_s": oc.batch / (med * 1e-3), "steps": oc.steps,
                        "kernels_per_step": oh.kernels_per_step, "loss": oh.loss(),
                        "one_persistent_kernel": oh.kernels_per_step == 1,
                        "hbm_bound_ms": opt_bytes / (measured_peaks()["hbm_gbs"] * 1e9) * 1e3,
                        "workload": "MLP %s, %s, %s, B=%d" % ("->".join(map(str, ol)), oc.activation, oc.optimizer, oc.batch)}
        oh.free()
    # the reference's option examples (examples/bench_dropout.vt, bench_layernorm.vt, bench_softmax.vt):
    # the c2 topology with one optional stage each, SGD lr 0.01, batch 64
    c2 = CONFIGS["c2"]
    for name, act, kw in (("c2_dropout", "relu", {"dropout_p": 0.2}), ("c2_layernorm", "relu", {"use_layernorm": True}),
                          ("c2_softmax", "softmax", {})):
        ol = list(c2.layers)
        # weights: the handle's default, the reference's LCG-Xavier stream (with the Kaiming weights of the
        # main configurations the dropout example diverges at this learning rate, on the CPU oracle too)
        oh = TrainHandle(ol, act, "sgd", c2.batch, gemm_path=args.gemm_path, **kw)
        ox = torch.from_numpy(synth.rows(c2.x_dist, 1234, 0, c2.batch, ol[0])).cuda()
        oy = torch.from_numpy(synth.rows(c2.y_dist, 4321, 0, c2.batch, ol[-1])).cuda()
        med = timed(oh, ox, oy, 0.01, 50)
        others[name] = {"ms_per_step": med, "steps": 50, "kernels_per_step": oh.kernels_per_step, "loss": oh.loss(),
                        "workload": "MLP %s, %s, sgd, B=%d, %s" % ("->".join(map(str, ol)), act, c2.batch, kw or "softmax hidden activation")}
        oh.free()
    # inference through host buffers, the protocol of the reference's examples/bench_infer.c:
    # c2 topology, 10 000 calls of one row and 1 000 calls of 64 rows, wall clock per call
    ol = list(c2.layers)
    oh = TrainHandle(ol, c2.activation, "sgd", 64, gemm_path=args.gemm_path)
    for i, (w, b) in enumerate(zip(*synth.kaiming_uniform_weights(ol, 42))):
        oh.set_params(i, w, b)
    for rows, warm, calls in ((1, 200, 10000), (64, 20, 1000)):
        xin = synth.rows(c2.x_dist, 1234, 0, rows, ol[0])
        out = np.empty((rows, ol[-1]), np.float32)
        fn, hh, n_in = oh.lib.volta_b200_infer, oh.h, xin.size
        pin, pout = xin.ctypes.data, out.ctypes.data
        for _ in range(warm):
            fn(hh, pin, n_in, pout, out.size)
        t0 = time.perf_counter()
        for _ in range(calls):
            fn(hh, pin, n_in, pout, out.size)
        dt = time.perf_counter() - t0
        others["infer_c2_b%d" % rows] = {"us_per_call": dt / calls * 1e6, "calls": calls, "rows": rows,
                                         "workload": "volta_infer protocol, host buffers, wall clock"}
    oh.free()
    return others


def workload_desc(cfg, world, dp_mode):
    return {"workload": "%s: MLP %s, %s, MSE, %s lr=%g, fp32, global batch %d" % (
        cfg.name, "->".join(map(str, cfg.layers)), cfg.activation, cfg.optimizer, cfg.lr, cfg.batch),
        "global_batch": cfg.batch, "x_dist": cfg.x_dist, "y_dist": cfg.y_dist,
        "weights": "Kaiming-uniform, seed 42", "parallelism": "dp%d" % world, "dp_mode": dp_mode if world > 1 else None,
        "note": cfg.note}


# ------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=None, help="default: c4 as the headline plus c5 inside config")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--gemm-path", default="auto", choices=["auto", "ffma", "tensor", "tensor_pair"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-workloads", action="store_true")
    ap.add_argument("--no-c5", action="store_true")
    ap.add_argument("--lean", action="store_true",
                    help="for profiler captures: no TF32 peak measurement, no per-kernel profile, no repeat-run check")
    ap.add_argument("--dp-mode", default="nccl", choices=["nccl", "fused", "copy"],
                    help="gradient exchange under data parallelism: bucketed NCCL all-reduce + optimizer, the fused "
                         "peer-memory reduce + update kernels, or copy-engine pushes into per-rank receive slots + a local "
                         "ordered sum and update")
    ap.add_argument("--batch", type=int, default=None,
                    help="override the workload's global batch (for small profiler captures; not a headline number)")
    args = ap.parse_args()

    from volta_b200 import CONFIGS
    default_run = args.workload is None and not args.batch
    args.workload = args.workload or "c4"
    cfg = CONFIGS[args.workload]
    if args.batch:
        cfg = dataclasses.replace(cfg, batch=args.batch, note=(cfg.note + "; batch overridden to %d" % args.batch).strip("; "))
    steps = args.steps if args.steps is not None else (10 if cfg.batch > 4096 else cfg.steps)
    warmup = max(args.warmup, 0)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        if rank != 0:
            return
        base = cpu_reference_arm(cfg)
        line = {"impl": "reference", "metric": "train_samples_per_s", "value": base["value"], "unit": "samples/s",
                "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
                "steps_run": "see cpu_baseline.sample: the CPU arm runs its own bounded protocol, not --steps/--warmup",
                "ms_per_step": cfg.batch / base["value"] * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": workload_desc(cfg, world, args.dp_mode), "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    job = Job()
    torch = job.torch
    peaks = measured_peaks()
    tf32 = None
    if world == 1 and not args.lean:
        try:
            tf32 = measure_tf32_peak()
        except Exception as exc:  # the bf16-derived denominator is then used and said so
            tf32 = None
            print("TF32 peak measurement failed: %s" % exc, file=sys.stderr)

    res = run_workload(job, cfg, args, steps, warmup, device_data=cfg.batch * cfg.layers[0] > 3e8, profile=not args.lean,
                       e2e_steps=0 if args.lean else None)
    roofline = roofline_of(res, cfg, peaks, tf32) if (world == 1 and res["agg"]) else None
    if world > 1 and res["agg"]:
        # per-phase view of rank 0's step under data parallelism (plain launches, the exchange overlapped as in
        # the graph): where the time beyond global-batch / N goes
        agg = res["agg"]
        gemm = sum(v[0] for k, v in agg.items() if "gemm" in k)
        roofline = {"kernel": "per-phase times of rank 0, ms", "bound": "tensor", "achieved": None, "peak": None, "unit": "TFLOP/s",
                    "frac": None, "traffic": None,
                    "phases_ms": {"gemms": gemm, "exposed_gradient_exchange": agg.get("wait_for_gradient_exchange", [0.0])[0],
                                  "optimizer": agg.get("optimizer", [0.0])[0],
                                  "other_kernels": sum(v[0] for k, v in agg.items() if "gemm" not in k and k not in ("optimizer", "wait_for_gradient_exchange")),
                                  "sum": sum(v[0] for v in agg.values()), "graph_step": res["ms_per_step"]},
                    "gemm_tflops_per_gpu": sum(v[1] for k, v in agg.items() if "gemm" in k) / gemm / 1e9 if gemm else None}

    desc = dict(workload_desc(cfg, world, args.dp_mode), per_gpu_batch=res["per_gpu_batch"], gemm_path=args.gemm_path,
                l2="inputs larger than L2" if not res["flush_needed"] else "L2 flushed between steps",
                arena_gb=round(res["arena_bytes"] / 1e9, 3), final_loss=res["loss"], steps_before_final_loss=res["steps_taken"],
                repeat_bit_identical=res["repeat_bit_identical"], loss_bits_after_3_steps=res["loss_bits_after_3_steps"])

    # ---- configuration 5 in the same run (sharded like the headline)
    if default_run and not args.no_c5:
        c5 = CONFIGS["c5"]
        r5 = run_workload(job, c5, args, c5.steps, 2, device_data=True, profile=True, e2e_steps=2)
        block = {"workload": workload_desc(c5, world, args.dp_mode)["workload"], "ms_per_step": r5["ms_per_step"],
                 "samples_per_s": r5["value"], "steps": c5.steps, "warmup": 2, "per_gpu_batch": r5["per_gpu_batch"],
                 "tflops_logical_fp32": r5["tflops_logical_fp32"], "arena_gb": round(r5["arena_bytes"] / 1e9, 3),
                 "final_loss": r5["loss"], "repeat_bit_identical": r5["repeat_bit_identical"],
                 "e2e_samples_per_s": r5["e2e"]["value"] if r5["e2e"] else None,
                 "inputs": "generated on the GPU (seeded per block of 4096 rows), N(0,1); weights Kaiming-uniform on the GPU",
                 "clocks": r5["clocks"]}
        if r5["agg"]:
            roof5 = roofline_of(r5, c5, peaks, tf32)
            block.update({"gemm_tflops": roof5["all_gemms_tflops"], "gemm_frac": roof5["all_gemms_frac"],
                          "whole_step_frac": roof5["whole_step_frac"], "optimizer_gbs": roof5.get("optimizer_gbs"),
                          "optimizer_frac_of_hbm": roof5.get("optimizer_frac_of_hbm"),
                          "kernels": r5["kernel_table"][:12]})
            if roofline is not None:
                roofline["c5"] = {k: block[k] for k in ("gemm_tflops", "gemm_frac", "whole_step_frac", "optimizer_gbs", "optimizer_frac_of_hbm")}
        desc["c5"] = block

    cpu_baseline = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        cpu_baseline = cpu_reference_arm(cfg)
        per_config = {}
        # the reference's protocol is 10 warm-up steps and 7 runs of 50 steps; the heavier configurations
        # take fewer or shorter runs here so that the whole benchmark stays within minutes (each entry
        # states what it ran)
        for name, (inner_a, steps_a), (inner_b, steps_b) in (("c1", (7, 50), (7, 50)), ("c2", (7, 50), (3, 50)),
                                                              ("c3_b64", (7, 10), (3, 10))):
            oc = CONFIGS[name]
            per_config[name] = {"seeded": cpu_protocol_run(oc, "seeded", inner=inner_a, steps=steps_a),
                                "closed_form_sgd": cpu_protocol_run(dataclasses.replace(oc, lr=0.01), "closed_form",
                                                                    optimizer="sgd", inner=inner_b, steps=steps_b)}
        per_config["c3_b1024"] = cpu_reference_arm(CONFIGS["c3_b1024"], quick=True)
        cpu_baseline["per_config"] = per_config
        try:
            tb = cpu_baseline["points"][-1]["batch"] if "points" in cpu_baseline else cfg.batch
            te = torch_cpu_run(cfg, tb)
            cpu_baseline["torch_cpu_eager"] = te
            cpu_baseline["sample"] += "; beside it PyTorch eager on %d cores at the same batch: %.0f samples/s" % (te["cores"], te["value"])
        except Exception as exc:  # secondary line only
            cpu_baseline["torch_cpu_eager"] = {"error": str(exc)}

    others = None
    if world == 1 and not args.batch and not args.no_other_workloads:
        others = side_table(job, args, torch.empty(int(256e6) // 4, device="cuda"))

    if rank == 0:
        line = {"metric": "train_samples_per_s", "value": res["value"], "unit": "samples/s", "n_gpus": world, "steps": steps,
                "warmup": warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": desc,
                "tflops_logical_fp32": res["tflops_logical_fp32"], "loss": res["loss"], "e2e": res["e2e"],
                "gpu_launches": res["kernels_per_step"] * steps, "kernels_per_step": res["kernels_per_step"],
                "clocks": res["clocks"], "roofline": roofline, "cpu_baseline": cpu_baseline, "other_workloads": others,
                "kernels": res["kernel_table"]}
        print(json.dumps(line))
    job.close()


if __name__ == "__main__":
    # Libraries loaded along the way (NCCL prints its version banner) write to stdout; the
    # contract is ONE JSON line there.  Point fd 1 at stderr while running and print the line
    # to the real stdout.
    sys.stdout.flush()
    _real_stdout = os.dup(1)
    os.dup2(2, 1)
    _out = os.fdopen(_real_stdout, "w")
    _print = print

    def print(*a, **k):  # noqa: A001  (only the JSON line goes through here)
        k.setdefault("file", _out)
        _print(*a, **k)
        _out.flush()

    main()
