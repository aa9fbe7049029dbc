#!/usr/bin/env python
"""Benchmark of the compiled MLP training step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4] [--impl b200|reference]

One "step" is one full training step (forward, MSE, backward, optimizer update) on one
batch of seeded synthetic input.  Prints ONE JSON line:
  value       whole-job samples/s with inputs resident in HBM, timed with CUDA events on the
              library's own stream, max over ranks
  e2e         the same metric through the C-ABI step call with pinned HOST inputs (host->device
              copy of X and Y and a device->host read of the loss inside the timed region)
  roofline    the dominant kernel against the measured tensor / HBM peak
  cpu_baseline  the reference's CPU path (its gemm_shim.c, compiled unmodified, under the
              restated step) timed on this host's cores on a bounded sample (N = 1 only)
`--impl reference` times only that CPU path and prints the same line shape.
Under torchrun (N > 1) the global batch is sharded over the ranks (strong scaling).
"""
from __future__ import annotations

import argparse
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


# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per batch row of one launch, from
# the ncu capture summarised in profiles/gemm_tc3_pair_c4_batch8192.md (taken at batch 8192; traffic
# of these GEMMs grows in proportion to the batch, so a full launch is rows x this figure).
NCU_TRAFFIC_PER_ROW = {
    "fwd_gemm_nn_Bx4096x4096": (620.196096e6 + 245.701376e6) / 8192,
    "fwd_gemm_nn_Bx1024x4096": (200.767232e6 + 44.852224e6) / 8192,
    "dX_gemm_nt_Bx4096x4096": (754.354176e6 + 131.911168e6) / 8192,
    "dW_gemm_tn_4096x4096xB": (628.525824e6 + 67.879424e6) / 8192,
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
def cpu_reference_run(cfg, steps: int, warmup: int, sample_batch: int | None = None):
    """Times the reference's CPU implementation of the step on a bounded sample of the
    workload.  Returns the cpu_baseline object and ms/step of the sample."""
    from oracle.oracle import Oracle
    from volta_b200 import synth

    layers = list(cfg.layers)
    # ~10-30 s of CPU work: the shim sustains roughly 10-15 GFLOP/s on one core
    budget_flops = 2.0e11
    B = sample_batch or cfg.batch
    per_step = cfg.flops_per_step(B)
    while sample_batch is None and B > 64 and per_step * (steps + warmup) > budget_flops:
        B //= 2
        per_step = cfg.flops_per_step(B)
    o = Oracle(layers, cfg.activation, cfg.optimizer, B)
    flavour = o.use_reference_gemm()
    kind = "reference" if flavour else "port"
    ws, bs = synth.kaiming_uniform_weights(layers, 42)
    for i, (w, b) in enumerate(zip(ws, bs)):
        o.set_params(i, w, b)
    x = synth.rows(cfg.x_dist, 1234, 0, B, layers[0])
    y = synth.rows(cfg.y_dist, 4321, 0, B, layers[-1])
    for _ in range(warmup):
        o.step(x, y, cfg.lr)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        o.step(x, y, cfg.lr)
        times.append(time.perf_counter() - t0)
    med = float(np.median(times))
    sample = "workload %s at batch %d of %d, %d warm-up + %d timed steps, median; GEMMs through the reference's " \
             "gemm_shim.c (%s build, single thread: its OpenMP branch is not thread-safe), step restated in C" % (
                 cfg.name, B, cfg.batch, warmup, steps, flavour or "none; oracle loops")
    base = {"value": B / med, "unit": "samples/s", "cores": 1, "kind": kind, "sample": sample,
            "ms_per_step_sample": med * 1e3, "sample_batch": B, "gflops": cfg.flops_per_step(B) / med / 1e9,
            "host_cpus": os.cpu_count(), "loss": o.loss()}
    o.free()
    return base, med * 1e3


def torch_cpu_run(cfg, B: int, steps: int = 3):
    """Second CPU line: PyTorch eager on all host cores, as examples/bench_pytorch.py does."""
    import torch
    torch.set_num_threads(os.cpu_count() or 1)
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
    return {"value": B / med, "unit": "samples/s", "cores": os.cpu_count(), "batch": B, "ms_per_step": med * 1e3}


# ------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="c4")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--gemm-path", default="auto", choices=["auto", "ffma", "tensor", "tensor_pair"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-other-workloads", action="store_true")
    ap.add_argument("--dp-mode", default="nccl", choices=["nccl", "fused"],
                    help="gradient exchange under data parallelism: bucketed NCCL all-reduce + optimizer, or the fused "
                         "peer-memory reduce + update kernels")
    ap.add_argument("--batch", type=int, default=None,
                    help="override the workload's global batch (for small profiler captures; not a headline number)")
    args = ap.parse_args()

    from volta_b200 import CONFIGS
    cfg = CONFIGS[args.workload]
    if args.batch:
        import dataclasses
        cfg = dataclasses.replace(cfg, batch=args.batch, note=(cfg.note + "; batch overridden to %d" % args.batch).strip("; "))
    steps = args.steps if args.steps is not None else (10 if cfg.batch > 4096 else cfg.steps)
    warmup = max(args.warmup, 0)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    workload_desc = {"workload": "%s: MLP %s, %s, MSE, %s lr=%g, fp32, global batch %d" % (
        cfg.name, "->".join(map(str, cfg.layers)), cfg.activation, cfg.optimizer, cfg.lr, cfg.batch),
        "global_batch": cfg.batch, "x_dist": cfg.x_dist, "y_dist": cfg.y_dist,
        "weights": "Kaiming-uniform, seed 42", "parallelism": "dp%d" % world, "dp_mode": args.dp_mode if world > 1 else None, "note": cfg.note}

    if args.impl == "reference":
        if rank != 0:
            return
        base, ms = cpu_reference_run(cfg, max(1, min(steps, 5)), min(warmup, 1))
        line = {"impl": "reference", "metric": "train_samples_per_s", "value": base["value"], "unit": "samples/s",
                "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": cfg.batch / base["value"] * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": workload_desc, "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist

    from volta_b200 import TrainHandle, synth
    from volta_b200.train import dp_unique_id

    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local_rank)
    uid = None
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        box = [dp_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        uid = box[0]
    assert cfg.batch % world == 0
    B = cfg.batch // world
    layers = list(cfg.layers)

    h = TrainHandle(layers, cfg.activation, cfg.optimizer, B, global_batch=cfg.batch, world_size=world, rank=rank,
                    unique_id=uid, gemm_path=args.gemm_path, fuse_sgd=(cfg.optimizer == "sgd" and world == 1))
    if world > 1 and args.dp_mode == "fused":
        handles = [None] * world
        dist.all_gather_object(handles, h.ipc_handle())
        h.attach_peers(handles)
    ws, bs = synth.kaiming_uniform_weights(layers, 42)
    for i, (w, b) in enumerate(zip(ws, bs)):
        h.set_params(i, w, b)
    del ws, bs
    x_host = torch.from_numpy(synth.rows(cfg.x_dist, 1234, rank * B, B, layers[0])).pin_memory()
    y_host = torch.from_numpy(synth.rows(cfg.y_dist, 4321, rank * B, B, layers[-1])).pin_memory()
    x_dev, y_dev = x_host.cuda(), y_host.cuda()
    stream = torch.cuda.ExternalStream(h.stream)

    def barrier():
        h.synchronize()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    working_set = h.arena_bytes
    flush_needed = working_set < 2 * L2_BYTES
    flush_buf = torch.empty(int(256e6) // 4, device="cuda") if flush_needed else None

    for _ in range(warmup):
        h.step(x_dev, y_dev, cfg.lr)
    barrier()

    sampler = ClockSampler(local_rank)
    sampler.start()
    # ---- device-resident timing
    if flush_needed:
        per = []
        for _ in range(steps):
            with torch.cuda.stream(stream):
                flush_buf.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            h.step(x_dev, y_dev, cfg.lr)
            e1.record(stream)
            per.append((e0, e1))
        barrier()
        ms_total = sum(a.elapsed_time(b) for a, b in per)
    else:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            h.step(x_dev, y_dev, cfg.lr)
        e1.record(stream)
        barrier()
        ms_total = e0.elapsed_time(e1)
    ms_total = max_over_ranks(ms_total)
    ms_per_step = ms_total / steps
    value = cfg.batch / (ms_per_step * 1e-3)
    loss_dev = h.loss()

    # ---- end to end through the host-pointer step call
    for _ in range(min(warmup, 2)):
        h.step(x_host, y_host, cfg.lr)
        h.loss()
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        if flush_needed:
            with torch.cuda.stream(stream):
                flush_buf.zero_()
        h.step(x_host, y_host, cfg.lr)
        last = h.loss()
    h.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    sampler.stop_flag = True
    sampler.join(timeout=2)
    e2e = {"value": cfg.batch / (e2e_s / steps), "unit": "samples/s", "ms_per_step": e2e_s / steps * 1e3,
           "h2d_bytes_per_step": int(world * 4 * B * (layers[0] + layers[-1])), "d2h_bytes_per_step": int(world * 8),
           "timer": "host wall clock, max over ranks", "includes_l2_flush": bool(flush_needed)}

    # ---- per-kernel times for the roofline (single GPU only; plain launches, event pairs)
    peaks = measured_peaks()
    roofline, kernel_table = None, None
    if world == 1:
        agg = {}
        reps = 3
        for _ in range(reps):
            for name, ms, fl, by in h.profile_step(x_dev, y_dev, cfg.lr):
                a = agg.setdefault(name, [0.0, fl, by])
                a[0] += ms / reps
        tot = sum(v[0] for v in agg.values())
        kernel_table = [{"kernel": k, "ms": round(v[0], 5), "share": round(v[0] / tot, 4),
                         "tflops": round(v[1] / v[0] / 1e9, 2) if v[1] else None,
                         "gbs": round(v[2] / v[0] / 1e6, 1)} for k, v in sorted(agg.items(), key=lambda kv: -kv[1][0])]
        top, tv = max(agg.items(), key=lambda kv: kv[1][0])
        if "gemm" in top and tv[1] / max(tv[2], 1) > 50:
            peak = peaks["bf16_tflops_sustained"] / 6.0
            ach = tv[1] / tv[0] / 1e9
            roofline = {"kernel": top, "bound": "tensor", "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                        "frac": ach / peak, "traffic": ncu_traffic_bytes(top, B),
                        "peak_basis": "%s bf16 sustained %.1f TFLOP/s / 6 (TF32 runs at half the bf16 rate and a "
                                      "3xTF32 product issues three MMAs); achieved counts logical fp32 flops" % (
                                          peaks["source"], peaks["bf16_tflops_sustained"])}
        else:
            ach = tv[2] / tv[0] / 1e6
            roofline = {"kernel": top, "bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                        "frac": ach / peaks["hbm_gbs"], "traffic": None,
                        "peak_basis": "%s STREAM-style copy" % peaks["source"]}
        gemm_ms = sum(v[0] for k, v in agg.items() if "gemm" in k)
        gemm_fl = sum(v[1] for k, v in agg.items() if "gemm" in k)
        roofline["all_gemms_tflops"] = gemm_fl / gemm_ms / 1e9 if gemm_ms else None
        opt = agg.get("optimizer")
        if opt:
            roofline["optimizer_gbs"] = opt[2] / opt[0] / 1e6
            roofline["optimizer_frac_of_hbm"] = opt[2] / opt[0] / 1e6 / peaks["hbm_gbs"]

    cpu_baseline = None
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        cpu_baseline, _ = cpu_reference_run(cfg, 3, 1)
        try:
            cpu_baseline["torch_cpu_eager"] = torch_cpu_run(cfg, cpu_baseline["sample_batch"])
        except Exception as exc:  # secondary line only
            cpu_baseline["torch_cpu_eager"] = {"error": str(exc)}

    # ---- the single-GPU configurations, briefly (device-resident inputs, L2 flushed between steps)
    others = None
    if world == 1 and not args.batch and not args.no_other_workloads:
        others = {}
        for name in ("c1", "c2", "c3_b64", "c3_b1024"):
            if name == args.workload:
                continue
            oc = CONFIGS[name]
            ol = list(oc.layers)
            oh = TrainHandle(ol, oc.activation, oc.optimizer, oc.batch, gemm_path=args.gemm_path,
                             fuse_sgd=(oc.optimizer == "sgd"))
            for i, (w, b) in enumerate(zip(*synth.kaiming_uniform_weights(ol, 42))):
                oh.set_params(i, w, b)
            ox = torch.from_numpy(synth.rows(oc.x_dist, 1234, 0, oc.batch, ol[0])).cuda()
            oy = torch.from_numpy(synth.rows(oc.y_dist, 4321, 0, oc.batch, ol[-1])).cuda()
            ostream = torch.cuda.ExternalStream(oh.stream)
            if flush_buf is None:
                flush_buf = torch.empty(int(256e6) // 4, device="cuda")
            for _ in range(5):
                oh.step(ox, oy, oc.lr)
            oh.synchronize()
            pairs = []
            for _ in range(oc.steps):
                with torch.cuda.stream(ostream):
                    flush_buf.zero_()
                a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(ostream)
                oh.step(ox, oy, oc.lr)
                b2.record(ostream)
                pairs.append((a, b2))
            oh.synchronize()
            torch.cuda.synchronize()
            ms = sorted(x.elapsed_time(y2) for x, y2 in pairs)
            med = ms[len(ms) // 2]
            others[name] = {"ms_per_step": med, "samples_per_s": oc.batch / (med * 1e-3), "steps": oc.steps,
                            "kernels_per_step": oh.kernels_per_step, "loss": oh.loss(),
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
            ostream = torch.cuda.ExternalStream(oh.stream)
            for _ in range(5):
                oh.step(ox, oy, 0.01)
            oh.synchronize()
            pairs = []
            for _ in range(50):
                with torch.cuda.stream(ostream):
                    flush_buf.zero_()
                a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(ostream)
                oh.step(ox, oy, 0.01)
                b2.record(ostream)
                pairs.append((a, b2))
            oh.synchronize()
            torch.cuda.synchronize()
            ms = sorted(x.elapsed_time(y2) for x, y2 in pairs)
            others[name] = {"ms_per_step": ms[len(ms) // 2], "steps": 50, "kernels_per_step": oh.kernels_per_step,
                            "loss": oh.loss(), "workload": "MLP %s, %s, sgd, B=%d, %s" % (
                                "->".join(map(str, ol)), act, c2.batch, kw or "softmax hidden activation")}
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

    if rank == 0:
        line = {"metric": "train_samples_per_s", "value": value, "unit": "samples/s", "n_gpus": world, "steps": steps,
                "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": dict(workload_desc, per_gpu_batch=B, gemm_path=args.gemm_path,
                               l2="inputs larger than L2" if not flush_needed else "L2 flushed between steps",
                               arena_gb=round(working_set / 1e9, 3)),
                "tflops_logical_fp32": cfg.flops_per_step() / (ms_per_step * 1e-3) / 1e12,
                "loss": loss_dev, "loss_e2e": last, "e2e": e2e, "gpu_launches": h.kernels_per_step * steps,
                "kernels_per_step": h.kernels_per_step, "clocks": sampler.summary(), "roofline": roofline,
                "cpu_baseline": cpu_baseline, "other_workloads": others, "kernels": kernel_table}
        print(json.dumps(line))
    h.free()
    if world > 1:
        dist.destroy_process_group()


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
