#!/usr/bin/env python
"""Benchmark of the hot path: compile the five benchmark comprehensions and run them on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload suite|tensordot|batchmatmul|tmm|group_conv|mlp3|sum1d|sum2d|colsum]
    python bench.py --impl reference ...        # the CPU reference arm (ATen on the host cores)

A "step" is one pass over the selected comprehensions (default: all five, "tc5_suite") on one
batch of seeded synthetic inputs that are already resident in HBM.  One JSON line is printed by
rank 0.  `value` is the whole-job algorithmic TFLOP/s over all ranks; `per_config` carries the
per-comprehension kernel time, GB/s, TFLOP/s and roofline fraction; `e2e` is the same step driven
from pinned host buffers (host->device copies of every input and device->host copies of every
output inside the timed region).

Multi-GPU (torchrun, one rank per GPU): every comprehension shards along an output index that also
indexes its large operand, no reduction crosses GPUs, so there is no data-path collective; each
rank runs a full-size shard (weak scaling) and timing is the max over ranks of device time.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "tc5_suite_throughput"
UNIT = "TFLOP/s"

# DRAM traffic per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum from the
# ncu captures summarised under profiles/), keyed by workload.  mlp3: the first (largest) of its three
# launches, [16384x2048]x[1024x2048]; algorithmic bytes of that launch are 209.7 MB, the 67 MB output
# is only partly written back to DRAM before the kernel ends (it stays in the 126 MB L2).
NCU_TRAFFIC_BYTES = {"mlp3": 142808576 + 46954240, "tmm": 271044608 + 5323008,
                     "tensordot": 413891584 + 84587008, "sum1d": 268450560 + 4871936}


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "tf32_tflops": d["bf16_tflops_sustained"] / 2.0,
                "tf32_tflops_burst": d["bf16_tflops"] / 2.0, "source": "measured"}
    # fallback figures of the pool (6.65 TB/s, 1.59 PFLOP/s bf16 burst, ~1.4 sustained)
    return {"hbm_gbs": 6650.0, "tf32_tflops": 700.0, "tf32_tflops_burst": 795.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks/throttle reasons every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
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
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # the median over the samples taken under load (the top half of the samples)
        load = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# The product arm
# ------------------------------------------------------------------------------------------------

class Program:
    """One comprehension compiled for its shapes: device buffers, plans, launch."""

    def __init__(self, w, dev, seed, rotate_bytes, tune=False):
        import torch
        from tensorcomprehensions_b200 import workloads as wl
        from tensorcomprehensions_b200 import runtime
        self.w, self.dev = w, dev
        self.host_inputs = [t.pin_memory() for t in wl.make_inputs(w, seed=seed)]
        self.exe = runtime.compile_workload(w, dev, tune=tune)
        # rotating sets: a small problem is timed over enough copies of its buffers to exceed L2
        per_set = w.bytes
        self.sets = max(1, -(-rotate_bytes // per_set)) if per_set < rotate_bytes else 1
        self.inputs = [[t.to(dev) for t in self.host_inputs] for _ in range(self.sets)]
        self.outputs = [self.exe.prepare_outputs() for _ in range(self.sets)]
        self.host_outputs = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in self.outputs[0]]
        self.cursor = 0
        self.staged = None
        self.launches_per_run = self.exe.launches

    def run(self):
        i = self.cursor
        self.cursor = (i + 1) % self.sets
        self.exe.run(self.inputs[i], self.outputs[i])

    def run_e2e(self):
        """Host buffers in, host buffers out through the public HostStagedExecutor: H2D of every input,
        launch, D2H of every output; copies of consecutive calls overlap (three streams, two buffer sets)."""
        if self.staged is None:
            self.staged = self.exe.host_staged(depth=2)
        self.staged.submit(self.host_inputs, self.host_outputs)

    def h2d_bytes(self):
        return sum(t.numel() * 4 for t in self.host_inputs)

    def d2h_bytes(self):
        return sum(t.numel() * 4 for t in self.host_outputs)


def window_times_us(prog, n_windows=20, min_window_us=200.0):
    """Per-launch device time of one comprehension: windows of R graph-replayed runs over the rotating sets."""
    import torch
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        est = []
        for _ in range(3):   # warm-up on this stream and a first estimate
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            prog.run()
            e1.record()
            e1.synchronize()
            est.append(e0.elapsed_time(e1) * 1e3)
        passes = max(1, int(-(-min_window_us // (min(est) * prog.sets))))
        runs = passes * prog.sets
        graph = torch.cuda.CUDAGraph()
        # thread-local capture mode: other threads of the process (NCCL's watchdog at N > 1) keep their CUDA calls
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            for _ in range(runs):
                prog.run()
        for _ in range(2):
            graph.replay()
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_windows)]
        for a, b in ev:
            a.record()
            graph.replay()
            b.record()
        stream.synchronize()
    t = sorted(a.elapsed_time(b) * 1e3 / runs for a, b in ev)
    return {"min": round(t[0], 2), "p50": round(t[len(t) // 2], 2), "p90": round(t[(len(t) * 9) // 10], 2),
            "runs_per_window": runs}


def roofline_time_us(w, peaks, split):
    """max(bytes / BW_hbm, k * flops / P_tf32); k = 3 under the 3xTF32 split; no tensor term for SIMT kernels."""
    t_mem = w.bytes / (peaks["hbm_gbs"] * 1e3)
    if split == 0:
        return t_mem
    return max(t_mem, split * w.flops / (peaks["tf32_tflops"] * 1e6))


def run_product(args):
    import torch
    import torch.distributed as dist
    from tensorcomprehensions_b200 import workloads as wl

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (the product path has no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # NCCL_DEBUG=VERSION makes NCCL print its version banner on stdout, ahead of the JSON line
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()

    names = list(wl.ALL) if args.workload == "suite" else [args.workload]
    progs = [Program(wl.BY_NAME[n](), dev, seed=20240 + wl.BY_NAME[n]().index + 1000 * rank,
                     rotate_bytes=192 << 20, tune=args.tune) for n in names]
    launches_per_step = sum(p.launches_per_run for p in progs)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- timed region 1: device-resident inputs ----------------------------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()   # sampled from the warm-up to the end of the host-buffer region
    for _ in range(args.warmup):
        for p in progs:
            p.run()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(progs) + 1)] for _ in range(args.steps)]
    barrier()
    for s in range(args.steps):
        ev[s][0].record()
        for i, p in enumerate(progs):
            p.run()
            ev[s][i + 1].record()
    barrier()
    total_ms = ev[0][0].elapsed_time(ev[-1][-1])
    per_prog_us = [statistics.mean(ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(args.steps)) * 1e3
                   for i in range(len(progs))]
    total_ms = max_over_ranks(total_ms)
    ms_per_step = total_ms / args.steps

    # ---- per-config windows: R back-to-back launches over the rotating sets in ONE event pair --------
    # (the reference's benchmark fixture times a kernel this way; a CUDA graph replays the launches so
    # that the window holds device time, not the host's launch rate: the two smallest kernels run
    # 7-30 us, the order of a launch through Python).  min / p50 / p90 over the windows.
    windows = [window_times_us(p) for p in progs]

    # ---- timed region 2: host buffers (e2e) -----------------------------------------------------
    for _ in range(min(args.warmup, 3)):
        for p in progs:
            p.run_e2e()
    for p in progs:
        p.staged.synchronize()
    barrier()
    e2e_steps = max(1, min(args.steps, 10))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for p in progs:   # the staging streams start after e0
        for st in (p.staged.h2d, p.staged.compute, p.staged.d2h):
            st.wait_event(e0)
    for _ in range(e2e_steps):
        for p in progs:
            p.run_e2e()
    for p in progs:   # e1 after every copy and kernel of the region
        p.staged.join()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / e2e_steps
    clocks = sampler.stop() if rank == 0 else None

    flops_step = sum(p.w.flops for p in progs) * world
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    per_config = []
    for p, us, win in zip(progs, per_prog_us, windows):
        split = p.exe.split_tf32
        troof = roofline_time_us(p.w, peaks, split)
        per_config.append({
            "workload": p.w.name, "kernel_us": round(us, 2), "launches": p.launches_per_run,
            "gbs": round(p.w.bytes / us / 1e3, 1), "tflops": round(p.w.flops / us / 1e6, 2),
            "roofline_us": round(troof, 2), "roofline_frac": round(troof / us, 3),
            "window_us": win, "roofline_frac_window": round(troof / win["p50"], 3),
            "bound": "tensor" if split and split * p.w.flops / (peaks["tf32_tflops"] * 1e6) >
            p.w.bytes / (peaks["hbm_gbs"] * 1e3) else "hbm",
            "kernel": p.exe.describe(), "rotating_sets": p.sets})
    # dominant kernel = largest share of the step
    dom = max(range(len(progs)), key=lambda i: per_prog_us[i])
    dp, dus, dc = progs[dom], per_prog_us[dom], per_config[dom]
    if dc["bound"] == "tensor":
        split = dp.exe.split_tf32
        roof = {"bound": "tensor", "achieved": round(split * dp.w.flops / dus / 1e6, 1),
                "peak": round(peaks["tf32_tflops"], 1), "unit": "TFLOP/s",
                "frac": round(split * dp.w.flops / dus / 1e6 / peaks["tf32_tflops"], 3),
                "note": "tensor-pipe flops issued = %d x algorithmic (3xTF32 split); peak = bf16_tflops_sustained/2 "
                        "(%s); algorithmic %.1f TFLOP/s" % (split, peaks["source"], dp.w.flops / dus / 1e6)}
    else:
        roof = {"bound": "hbm", "achieved": round(dp.w.bytes / dus / 1e3, 1), "peak": peaks["hbm_gbs"],
                "unit": "GB/s", "frac": round(dp.w.bytes / dus / 1e3 / peaks["hbm_gbs"], 3),
                "note": "of %s" % peaks["source"]}
    roof["kernel"] = dp.w.name
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(dp.w.name)
    if dp.w.name == "mlp3":
        roof["traffic_note"] = ("ncu capture of the first of the three launches (layer 1: 209.7 MB algorithmic, "
                                "76 % of the flops); achieved/frac cover all three")

    cpu = cpu_baseline(names, budget_s=args.cpu_seconds) if world == 1 and not args.no_cpu else None

    line = {
        "metric": METRIC, "value": round(flops_step / (ms_per_step * 1e-3) / 1e12, 3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": "tc5_suite" if args.workload == "suite" else args.workload,
                   "configs": names, "tiles": "autotuned" if args.tune else "family default",
                   "shard": "one full-size instance of every comprehension per GPU",
                   "l2": "inputs larger than L2 (suite streams 1.2 GB per step; small problems rotate over "
                         ">=192 MB of buffer sets)"},
        "e2e": {"value": round(flops_step / (e2e_ms * 1e-3) / 1e12, 3), "unit": UNIT,
                "ms_per_step": round(e2e_ms, 3),
                "h2d_bytes_per_step": sum(p.h2d_bytes() for p in progs),
                "d2h_bytes_per_step": sum(p.d2h_bytes() for p in progs)},
        "gpu_launches": launches_per_step * args.steps,
        "clocks": clocks, "roofline": roof, "per_config": per_config,
    }
    if cpu:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# The CPU arm: the reference's own CPU-side comparator (ATen on the host cores)
# ------------------------------------------------------------------------------------------------

def cpu_suite(names):
    import torch
    from oracle import oracle as orc
    from tensorcomprehensions_b200 import workloads as wl
    ws = [wl.BY_NAME[n]() for n in names]
    inputs = [wl.make_inputs(w) for w in ws]

    def step():
        for w, ins in zip(ws, inputs):
            orc.ATEN[w.name](*ins)
    return ws, step, torch.get_num_threads()


def cpu_baseline(names, budget_s=20.0):
    """ATen-CPU evaluation of the same step on the host cores; bounded sample of whole steps."""
    ws, step, threads = cpu_suite(names)
    step()  # warm-up
    times, t_start = [], time.perf_counter()
    while len(times) < 5 and (time.perf_counter() - t_start < budget_s or not times):
        t0 = time.perf_counter()
        step()
        times.append(time.perf_counter() - t0)
    best = min(times)
    flops = sum(w.flops for w in ws)
    return {"value": round(flops / best / 1e12, 4), "unit": UNIT, "cores": threads, "kind": "port",
            "sample": "%d whole steps of the same suite through ATen-CPU (best of them, %.3f s)" % (len(times), best),
            "ms_per_step": round(best * 1e3, 2)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from tensorcomprehensions_b200 import workloads as wl
    names = list(wl.ALL) if args.workload == "suite" else [args.workload]
    ws, step, threads = cpu_suite(names)
    for _ in range(min(args.warmup, 2)):
        step()
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    ms = (time.perf_counter() - t0) / steps * 1e3
    flops = sum(w.flops for w in ws)
    v = round(flops / (ms * 1e-3) / 1e12, 4)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT,
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": min(args.warmup, 2),
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "tc5_suite" if args.workload == "suite" else args.workload, "configs": names},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "whole steps of the suite through ATen-CPU, the comparator the reference's own "
                                   "harness uses (its CPU executor is a stub and its JIT needs Halide/isl/LLVM)"},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="suite",
                    choices=["suite", "tensordot", "batchmatmul", "tmm", "group_conv", "mlp3", "sum1d", "sum2d", "colsum"])
    ap.add_argument("--cpu-seconds", type=float, default=20.0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--tune", action="store_true",
                    help="pick each comprehension's tile with the autotuner's sweep instead of the family default")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_product(args)


if __name__ == "__main__":
    main()
