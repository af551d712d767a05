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

Multi-GPU (torchrun, one rank per GPU): every comprehension is split along an output index that also
indexes its large operand (tensordot, group convolution: n; batchmatmul: b; transposed matmul: the rows of
B = the columns of C; MLP3: the batch), each rank compiles and runs its shard, no reduction crosses
GPUs, so computing needs no collective.  The total work is the same at every N (strong scaling); time
is the max over ranks of device time.  At N > 1 the opt-in exchange that assembles the full outputs (an
all-gather over NCCL) is timed separately per comprehension and reported beside the kernel-only time.
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
NCU_TRAFFIC_BYTES = {"mlp3": 142796544 + 46067712, "tmm": 270619392 + 5780480,
                     "tensordot": 413908992 + 83188736, "sum1d": 268450304 + 4541184}


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

EXECUTION_ORDER = ["tensordot", "batchmatmul", "group_conv", "mlp3", "tmm"]

SHARD_NOTE = ("strong scaling: every comprehension split across the GPUs along one output index "
              "(tensordot n, batchmatmul b, tmm the rows of B = columns of C, group_conv n, mlp3 the batch), "
              "remainders on the first ranks; replicated operands (A of tmm, filters, MLP weights) on every GPU; "
              "no data-path collective")


def make_config(args):
    """The `config` object of the JSON line: the same for both arms at the same arguments."""
    names = suite_names(args)
    return {"workload": "tc5_suite" if args.workload == "suite" else args.workload, "configs": names,
            "tiles": "autotuned" if args.tune else "family default", "shard": SHARD_NOTE,
            "l2": "inputs larger than L2: every comprehension rotates over buffer sets that total >= 192 MB",
            "launch": "the K timed steps are one CUDA-graph replay (device time); per_config.kernel_us comes from "
                      "the same steps launched one by one with an event after each comprehension",
            "order": [n for n in EXECUTION_ORDER if n in names] + [n for n in names if n not in EXECUTION_ORDER]}


def suite_names(args):
    from tensorcomprehensions_b200 import workloads as wl
    return list(wl.ALL) if args.workload == "suite" else [args.workload]


class Program:
    """One rank's shard of one comprehension, compiled for its shapes: device buffers, plans, launch."""

    def __init__(self, name, world, rank, dev, rotate_bytes, tune=False):
        import torch
        from tensorcomprehensions_b200 import workloads as wl
        from tensorcomprehensions_b200 import runtime
        self.name, self.dev, self.world = name, dev, world
        self.full = wl.BY_NAME[name]()
        if name in wl.ALL:
            self.w, draws = wl.make_shard_inputs(name, world, rank)
        else:  # the extra single-GPU workloads are not sharded
            self.w, draws = self.full, wl.make_inputs(self.full)
        self.host_inputs = [t.pin_memory() for t in draws]
        self.exe = runtime.compile_workload(self.w, dev, tune=tune)
        # rotating sets: the comprehension is timed over enough copies of its buffers to exceed L2
        per_set = self.w.bytes
        self.sets = max(1, -(-rotate_bytes // per_set)) if per_set < rotate_bytes else 1
        self.inputs = [[t.to(dev) for t in self.host_inputs] for _ in range(self.sets)]
        self.outputs = [self.exe.prepare_outputs() for _ in range(self.sets)]
        self.host_outputs = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in self.outputs[0]]
        self.cursor = 0
        self.staged = None
        self.gatherers = None
        self.launches_per_run = self.exe.launches

    def run(self):
        i = self.cursor
        self.cursor = (i + 1) % self.sets
        self.exe.run(self.inputs[i], self.outputs[i])
        return self.outputs[i]

    def run_gathered(self):
        """The shard's launch followed by the all-gather of every output (NCCL) and its assembly."""
        from tensorcomprehensions_b200 import sharding
        outs = self.run()
        if self.gatherers is None:
            self.gatherers = [sharding.Gatherer(tuple(o.shape), d, full_shape[d], self.dev)
                              for o, d, full_shape in zip(outs, self.w.shard_outputs, self.full_output_shapes())]
        return [g.gather(o) for g, o in zip(self.gatherers, outs)]

    def full_output_shapes(self):
        """Unsharded output shapes: the shard's with the sharded dimension at its full extent."""
        dim = next(d for d in self.full.shard_inputs if d is not None)
        total = next(s for s, d in zip(self.full.shapes, self.full.shard_inputs) if d is not None)[dim]
        shapes = []
        for o, d in zip(self.outputs[0], self.w.shard_outputs):
            s = list(o.shape)
            s[d] = total
            shapes.append(tuple(s))
        return shapes

    def gathered_bytes(self):
        n = 0
        for s in self.full_output_shapes():
            k = 4
            for x in s:
                k *= x
            n += k
        return n

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


def window_times_us(run, sets, n_windows=20, min_window_us=200.0):
    """Per-launch device time of one comprehension: windows of R graph-replayed runs over the rotating sets."""
    import torch
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        est = []
        for _ in range(3):   # warm-up on this stream and a first estimate
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run()
            e1.record()
            e1.synchronize()
            est.append(e0.elapsed_time(e1) * 1e3)
        passes = max(1, int(-(-min_window_us // (min(est) * sets))))
        runs = passes * sets
        graph = torch.cuda.CUDAGraph()
        # thread-local capture mode: other threads of the process (NCCL's watchdog at N > 1) keep their CUDA calls
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            for _ in range(runs):
                run()
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


def roofline_time_us(w, peaks, split, gpus=1, burst=False):
    """max(bytes / BW_hbm, k * flops / P_tf32) over `gpus` GPUs; k = 3 under the 3xTF32 split; no tensor term for
    SIMT kernels."""
    t_mem = w.bytes / (peaks["hbm_gbs"] * 1e3 * gpus)
    if split == 0:
        return t_mem
    p = peaks["tf32_tflops_burst"] if burst else peaks["tf32_tflops"]
    return max(t_mem, split * w.flops / (p * 1e6 * gpus))


# fp32 FMA rate of the part, measured with a register-resident FMA loop (both the scalar and the packed
# fp32x2 form): 36.9 T fused multiply-adds per second.  The group convolution at C = F = 16 is bound by it
# (464 M multiply-adds), not by HBM.
FMA_PEAK_TFMA = 36.9


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
    # stdout carries the one JSON line and nothing else.  Libraries print there too (NCCL writes its version
    # banner to stdout when a communicator comes up, at a moment of its choosing): file descriptor 1 points at
    # stderr for the whole run and the line is written to the saved descriptor at the end.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()

    names = suite_names(args)
    if world > 1 and any(n not in wl.ALL for n in names):
        raise SystemExit("bench.py: %s is a single-GPU workload" % args.workload)
    # --shard-of W (one GPU only): run rank 0's shard of a W-GPU run, e.g. to profile the kernels a shard uses
    shard_world = args.shard_of if (world == 1 and args.shard_of > 1) else world
    # Order inside a step: the transposed matmul (tensor-bound, 3 TB/s of HBM traffic) runs right after MLP3, so that
    # the write-back of MLP3's 117 MB of outputs from L2 lands under a kernel that leaves HBM bandwidth free, not under
    # the tensordot, which needs all of it (80.6 us alone, 90 us when it follows MLP3).
    run_order = [n for n in EXECUTION_ORDER if n in names] + [n for n in names if n not in EXECUTION_ORDER]
    progs = [Program(n, shard_world, rank, dev, rotate_bytes=192 << 20, tune=args.tune) for n in run_order]
    if shard_world != world:
        for p in progs:
            p.full = p.w   # the shard is the whole job of this run
    launches_per_step = sum(p.launches_per_run for p in progs)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def over_ranks(values, op):
        if world == 1:
            return list(values)
        t = torch.tensor(list(values), dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=op)
        return [float(x) for x in t.tolist()]

    def max_over_ranks(values):
        return over_ranks(values, dist.ReduceOp.MAX if world > 1 else None)

    def sum_over_ranks(values):
        return over_ranks(values, dist.ReduceOp.SUM if world > 1 else None)

    # ---- timed region 1: device-resident inputs ----------------------------------------------
    # The K timed steps are ONE CUDA-graph replay: the launches of K consecutive steps (each step takes the next
    # buffer set of every comprehension) are captured once and replayed, so that the step time is device time.
    # Launched one by one through Python the small shards of a multi-GPU run (kernels of 4-15 us) would be
    # timed at the host's launch rate.  A first replay is the warm-up of the graph itself.
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()   # sampled from the warm-up to the end of the host-buffer region
    for _ in range(args.warmup):
        for p in progs:
            p.run()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for p in progs:
            p.cursor = 0
        graph = torch.cuda.CUDAGraph()
        # thread-local capture mode: other threads of the process (NCCL's watchdog at N > 1) keep their CUDA calls
        with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
            for _ in range(args.steps):
                for p in progs:
                    p.run()
        graph.replay()
        stream.synchronize()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        graph.replay()
        g1.record()
        stream.synchronize()
        barrier()
    total_ms = max_over_ranks([g0.elapsed_time(g1)])[0]
    ms_per_step = total_ms / args.steps
    del graph

    # ---- the same steps launched one by one, with an event after every comprehension: the per-comprehension
    # split of a step (inflated by the host's launch rate where a kernel is shorter than a launch) ----------
    eager_steps = max(3, min(args.steps, 20))
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(len(progs) + 1)] for _ in range(eager_steps)]
    barrier()
    for s in range(eager_steps):
        ev[s][0].record()
        for i, p in enumerate(progs):
            p.run()
            ev[s][i + 1].record()
    barrier()
    eager_ms_per_step = max_over_ranks([ev[0][0].elapsed_time(ev[-1][-1]) / eager_steps])[0]
    per_prog_us = [statistics.mean(ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(eager_steps)) * 1e3
                   for i in range(len(progs))]
    per_prog_us = max_over_ranks(per_prog_us)

    # ---- per-config windows: R back-to-back launches over the rotating sets in ONE event pair --------
    # (the reference's benchmark fixture times a kernel this way; a CUDA graph replays the launches so
    # that the window holds device time, not the host's launch rate: the smallest kernels run a few
    # microseconds, the order of a launch through Python).  min / p50 / p90 over the windows, each the max
    # over ranks.
    windows = []
    for p in progs:
        win = window_times_us(p.run, p.sets)
        m = max_over_ranks([win["min"], win["p50"], win["p90"]])
        win.update({"min": round(m[0], 2), "p50": round(m[1], 2), "p90": round(m[2], 2)})
        windows.append(win)

    # ---- the opt-in exchange: shard launch + all-gather of every output over NCCL, per comprehension ----
    gather = [None] * len(progs)
    if world > 1:
        reps = 10
        for i, p in enumerate(progs):
            for _ in range(3):
                p.run_gathered()
            barrier()
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            e0.record()
            for _ in range(reps):
                p.run()
            e1.record()
            for _ in range(reps):
                p.run_gathered()
            e2.record()
            barrier()
            k_us, kg_us = max_over_ranks([e0.elapsed_time(e1) * 1e3 / reps, e1.elapsed_time(e2) * 1e3 / reps])
            gather[i] = {"kernel_us": round(k_us, 2), "kernel_plus_gather_us": round(kg_us, 2),
                         "gathered_bytes": p.gathered_bytes(),
                         "how": "%d back-to-back calls each, host-launched; all_gather_into_tensor (NCCL) of "
                                "equal padded shards + assembly kernel where the split is uneven or not on "
                                "dimension 0" % reps}

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
    e2e_ms = max_over_ranks([e0.elapsed_time(e1)])[0] / e2e_steps
    h2d, d2h, launches = sum_over_ranks([sum(p.h2d_bytes() for p in progs), sum(p.d2h_bytes() for p in progs),
                                         launches_per_step])
    clocks = sampler.stop() if rank == 0 else None

    # the three reductions of the fourth kernel family, alone, on one GPU (not part of the suite's value)
    reductions = None
    if world == 1 and args.workload == "suite" and not args.no_reductions:
        reductions = []
        for n in wl.EXTRA:
            rp = Program(n, 1, 0, dev, rotate_bytes=0)
            win = window_times_us(rp.run, rp.sets)
            reductions.append({"workload": n, "window_us": win, "gbs": round(rp.w.bytes / win["p50"] / 1e3, 1),
                               "roofline_frac_window": round(rp.w.bytes / win["p50"] / 1e3 / peaks["hbm_gbs"], 3),
                               "kernel": rp.exe.describe()})
            del rp
            torch.cuda.empty_cache()

    flops_step = sum(p.full.flops for p in progs)   # the whole job: the shards of all ranks add up to this
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # the timed region is a burst (milliseconds to a second) unless many steps are asked for: the tensor peak
    # it is compared with is the burst figure then, the sustained one for regions of a second and more
    burst = total_ms < 1000.0
    per_config = []
    for p, us, win, ga in zip(progs, per_prog_us, windows, gather):
        split = p.exe.split_tf32
        troof = roofline_time_us(p.full, peaks, split, world, burst)
        t_tensor = split * p.full.flops / ((peaks["tf32_tflops_burst"] if burst else peaks["tf32_tflops"]) * 1e6 * world)
        t_hbm = p.full.bytes / (peaks["hbm_gbs"] * 1e3 * world)
        entry = {
            "workload": p.name, "kernel_us": round(us, 2), "launches": p.launches_per_run,
            "gbs": round(p.full.bytes / us / 1e3, 1), "tflops": round(p.full.flops / us / 1e6, 2),
            "roofline_us": round(troof, 2), "roofline_frac": round(troof / us, 3),
            "window_us": win, "roofline_frac_window": round(troof / win["p50"], 3),
            "bound": "tensor" if split and t_tensor > t_hbm else "hbm",
            "kernel": p.exe.describe(), "rotating_sets": p.sets, "shard_shapes": [list(s) for s in p.w.shapes]}
        if p.name == "group_conv" and not split:
            # the fp32 kernels of this family are bound by the FMA pipe, not by HBM
            fma_us = (p.full.flops / 2.0) / (FMA_PEAK_TFMA * 1e6 * world)
            entry.update({"bound": "fma", "fma_floor_us": round(fma_us, 2),
                          "fma_frac": round(fma_us / us, 3), "fma_frac_window": round(fma_us / win["p50"], 3)})
        elif p.name == "group_conv":
            # Tensor-core kernel with the filter rows as accumulator rows: KH * F = 48 of an MMA's 128 rows carry work
            # and all H * W pixels of an item are computed for its OH * OW outputs, so the tensor pipe ISSUES
            # 3 (3xTF32) x 128/48 x 256/196 x the algorithmic flops; at the pipe's measured 4096 flop per clock and SM
            # that is the floor this formulation can reach.
            (_, _, _, H, W), (_, F, _, KH, KW) = p.full.shapes[0], p.full.shapes[1]
            factor = 3.0 * 128.0 / (KH * F) * (H * W) / ((H - KH + 1) * (W - KW + 1))
            pipe_us = p.full.flops * factor / (4096.0 * 148 * 1965.0 * world)
            entry.update({"pipe_floor_us": round(pipe_us, 2), "pipe_frac_window": round(pipe_us / win["p50"], 3),
                          "pipe_note": "MMA flops issued = %.2f x algorithmic; 4096 flop/clk/SM at 1965 MHz" % factor})
        if ga:
            entry["gather"] = ga
        per_config.append(entry)
    per_config.sort(key=lambda e: names.index(e["workload"]))   # reported in the order the configurations are listed
    # dominant kernel = largest share of the step at the device's pace: the graph-replayed windows (the one-by-one
    # event times of the smallest kernels hold the host's launch rate, above all on the shards of a multi-GPU run)
    dom = max(range(len(progs)), key=lambda i: windows[i]["p50"])
    dp, dus = progs[dom], windows[dom]["p50"]
    dc = next(e for e in per_config if e["workload"] == dp.name)
    if dc["bound"] == "tensor":
        split = dp.exe.split_tf32
        peak = (peaks["tf32_tflops_burst"] if burst else peaks["tf32_tflops"]) * world
        roof = {"bound": "tensor", "achieved": round(split * dp.full.flops / dus / 1e6, 1),
                "peak": round(peak, 1), "unit": "TFLOP/s",
                "frac": round(split * dp.full.flops / dus / 1e6 / peak, 3),
                "note": "tensor-pipe flops issued = %d x algorithmic (3xTF32 split); peak = %d x %s / 2 (%s; the "
                        "timed region lasted %.1f ms); algorithmic %.1f TFLOP/s" %
                        (split, world, "bf16_tflops (burst)" if burst else "bf16_tflops_sustained",
                         peaks["source"], total_ms, dp.full.flops / dus / 1e6)}
    else:
        roof = {"bound": "hbm", "achieved": round(dp.full.bytes / dus / 1e3, 1), "peak": peaks["hbm_gbs"] * world,
                "unit": "GB/s", "frac": round(dp.full.bytes / dus / 1e3 / (peaks["hbm_gbs"] * world), 3),
                "note": "of %s" % peaks["source"]}
    roof["kernel"] = dp.name
    roof["timed"] = "p50 of %d windows of graph-replayed launches, CUDA events on the launching stream" % 20
    roof["traffic"] = NCU_TRAFFIC_BYTES.get(dp.name) if world == 1 else None
    if dp.name == "mlp3" and world == 1:
        roof["traffic_note"] = ("ncu capture of the first of the three launches (layer 1: 209.7 MB algorithmic, "
                                "76 % of the flops); achieved/frac cover all three")

    cpu = cpu_baseline(names, budget_s=args.cpu_seconds) if world == 1 and not args.no_cpu else None

    line = {
        "metric": METRIC, "value": round(flops_step / (ms_per_step * 1e-3) / 1e12, 3), "unit": UNIT,
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "ms_per_step_launched_one_by_one": round(eager_ms_per_step, 4),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": dict(make_config(args), **({"shard_of": shard_world} if shard_world != world else {})),
        "e2e": {"value": round(flops_step / (e2e_ms * 1e-3) / 1e12, 3), "unit": UNIT,
                "ms_per_step": round(e2e_ms, 3),
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h)},
        "gpu_launches": int(launches) * args.steps,
        "clocks": clocks, "roofline": roof, "per_config": per_config,
    }
    if reductions:
        line["reductions"] = reductions
    if cpu:
        line["cpu_baseline"] = cpu
    os.write(json_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# The CPU arm: the reference's own CPU-side comparator (ATen on the host cores)
# ------------------------------------------------------------------------------------------------

def host_threads():
    """Host cores this process may use.  torchrun exports OMP_NUM_THREADS=1 to its workers, which would leave
    ATen on one thread: the CPU arm sets its thread count from the affinity mask instead."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_suite(names):
    import torch
    from oracle import oracle as orc
    from tensorcomprehensions_b200 import workloads as wl
    torch.set_num_threads(host_threads())
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
    """The CPU arm: the whole (unsharded) suite through ATen on all the host cores this process may use, with
    exactly the steps and warm-up asked for.  Under torchrun rank 0 alone runs it; the total work per step is
    the same as the product arm's at every N (the product arm splits it, this arm has one host)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    names = suite_names(args)
    ws, step, threads = cpu_suite(names)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    ms = (time.perf_counter() - t0) / args.steps * 1e3
    flops = sum(w.flops for w in ws)
    v = round(flops / (ms * 1e-3) / 1e12, 4)
    line = {
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT,
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": make_config(args),
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
    ap.add_argument("--shard-of", type=int, default=1,
                    help="on one GPU: run rank 0's shard of a run on this many GPUs (profiling aid; not a bench line)")
    ap.add_argument("--no-reductions", action="store_true",
                    help="skip the stand-alone timing of the three reduction workloads (one GPU, suite only)")
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
