#!/usr/bin/env python
"""Benchmark of the small-batch matmul hot path (one JSON line on stdout, rank 0).

Workload "bt_sweep" (default): one step = five calls of edgemm_m8n128k64x4_bt,
M in {1,2,4,8,16}, K = N = 8192 per GPU, fp16, weight stored NxK; each call streams a
different one of four weight copies (537 MB, larger than the 126 MB L2).  With N GPUs every
rank holds its own 8192-row shard of an (8192*N) x 8192 weight ("weak" scaling): the ranks
compute their output slices independently and the slices are assembled with one NCCL
all-gather per call.  `value` is the whole job's effective HBM bandwidth (algorithmic bytes
of all ranks / time, gather included at N > 1); `no_gather` reports the same without it.

  value     inputs resident in HBM, step replayed from a CUDA graph (N = 1) or launched on
            a stream (N > 1), timed with CUDA events on the launching stream
  e2e       the same step through the public operator (fastgate_b200.edgemm_m8n128k64x4_bt)
            with the step's activations copied from pinned host memory and its results
            copied back to pinned host memory every step, two steps in flight (copies on side
            streams; the host waits for step k-1 while step k runs); the weight stays resident,
            as at the reference's call sites
  roofline  algorithmic bytes per launch / average launch duration, against the measured
            copy bandwidth of this pool's B200s
  cpu_baseline  the CPU oracle (a port of the reference's arithmetic, OpenMP) on this box's
            host cores, for one step

`--impl reference` times the reference's own kernels, rebuilt unmodified for sm_100a
(oracle/_ref), on the same workload through the reference's operator; when that build is
not available it falls back to the CPU oracle port.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0   # earlier measurement on this pool, used only without MEASURED_PEAKS.json
N_WEIGHT_COPIES = 4
# dram__bytes_read.sum + dram__bytes_write.sum per launch, mean over the five launches of one
# step, from the ncu capture summarised in profiles/bt_sweep__ncu_full.md
NCU_TRAFFIC_BYTES_PER_LAUNCH = 138.3e6


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=("bt_sweep", "cfg1", "cfg3", "cfg4", "w4", "dit"), default="bt_sweep",
                    help="bt_sweep (default, config 2) | cfg1 edgemm_m8n128k64x4 | cfg3 fastgemv | cfg4 fastgemv_int8 | "
                         "dit: the 40-layer DiT linear stack, N-sharded over the GPUs (strong scaling)")
    ap.add_argument("--layers", type=int, default=40, help="dit: number of layers")
    ap.add_argument("--no-graph", action="store_true", help="launch on a stream instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-push", action="store_true", help="N > 1: assemble outputs with NCCL only")
    ap.add_argument("--reference-arm", choices=("auto", "gpu", "cpu"), default="auto")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples of one GPU during the timed region."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.strip().splitlines():
            f = [v.strip() for v in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def hold_load(step_fn, stream, seconds: float = 0.5) -> None:
    """Keeps replaying the step (untimed, uncounted) so that the clock sampler, which ticks every
    100 ms, sees the GPU under the load of the timed region, which lasts only a few milliseconds."""
    import torch

    t_end = time.perf_counter() + seconds
    with torch.cuda.stream(stream):
        while time.perf_counter() < t_end:
            for _ in range(20):
                step_fn()
            stream.synchronize()


def dist_setup(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("bench.py --gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("NCCL_DEBUG", "WARN")  # keep NCCL's version banner off stdout
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def barrier_sync(world):
    import torch
    import torch.distributed as dist

    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms: float, world: int) -> float:
    import torch
    import torch.distributed as dist

    if world == 1:
        return ms
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(step_fn, steps: int, warmup: int, world: int, stream, graph=None) -> float:
    """ms for exactly `steps` steps, device-timed on `stream`, max over ranks."""
    import torch

    with torch.cuda.stream(stream):
        for _ in range(warmup):
            graph.replay() if graph is not None else step_fn()
        barrier_sync(world)
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.replay() if graph is not None else step_fn()
        e1.record(stream)
        barrier_sync(world)
    return max_over_ranks(e0.elapsed_time(e1), world)


def pipelined_e2e(compute, x_all_host, n_rows: int, n_cols: int, dev, stream, steps: int, warmup: int) -> float:
    """ms for `steps` end-to-end steps on one GPU, two steps deep.

    Every step copies its activations from pinned host memory (side stream), runs
    `compute(x_dev, out_dev)` on `stream` and copies the results back to pinned host memory
    (another side stream); the host waits for the results of step k-1 while step k is in
    flight, as a serving loop does.  All copies of all timed steps lie inside the timed
    region, which ends when the last step's results are in host memory."""
    import torch

    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    x_dev = [torch.empty_like(x_all_host, device=dev) for _ in range(2)]
    out_dev = [torch.zeros(n_rows, n_cols, dtype=torch.float16, device=dev) for _ in range(2)]
    out_host = [torch.empty(n_rows, n_cols, dtype=torch.float16).pin_memory() for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def run(n: int) -> int:
        last = 0
        for k in range(n):
            b = k & 1
            with torch.cuda.stream(s_in):  # x_dev[b] was last read by step k-2, whose results the host already has
                x_dev[b].copy_(x_all_host, non_blocking=True)
                ev_in[b].record(s_in)
            stream.wait_event(ev_in[b])
            compute(x_dev[b], out_dev[b])
            ev_comp[b].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_comp[b])
                out_host[b].copy_(out_dev[b], non_blocking=True)
                ev_out[b].record(s_out)
            if k >= 1:
                ev_out[1 - b].synchronize()  # the caller has the previous step's results
            last = b
        ev_out[last].synchronize()
        return last

    with torch.cuda.stream(stream):
        run(max(2, warmup))
        torch.cuda.synchronize(dev)
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        s_in.wait_event(e0)
        last = run(steps)
        stream.wait_event(ev_out[last])
        stream.wait_event(ev_out[1 - last])
        e1.record(stream)
        torch.cuda.synchronize(dev)
    return e0.elapsed_time(e1)


def cpu_baseline_leg(cases, sample_reps: int = 3) -> dict:
    """The CPU oracle (port of the reference's arithmetic) on one full step, host cores."""
    import numpy as np

    from oracle import oracle

    rng = np.random.default_rng(0)
    W = (rng.standard_normal((8192, 8192)) / 90.5).astype(np.float16)
    xs = [rng.standard_normal((c.M, c.K)).astype(np.float16) for c in cases]
    oracle.gemm_nk(xs[0], W)  # warm-up, builds the library if needed
    times = []
    for _ in range(sample_reps):
        t0 = time.perf_counter()
        for x in xs:
            oracle.gemm_nk(x, W)
        times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    bytes_step = sum(c.algorithmic_bytes for c in cases)
    return {"value": bytes_step / sec / 1e9, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
            "sample": f"one full step (5 calls, M=1,2,4,8,16, K=N=8192), median of {sample_reps}",
            "ms_per_step": sec * 1e3}


def run_ours(args):
    import torch

    import fastgate_b200 as fg
    from fastgate_b200 import shard, workloads as wl

    world, rank, local = dist_setup(args)
    dev = torch.device("cuda", local)
    cases = wl.cfg2()
    bytes_step_rank = sum(c.algorithmic_bytes for c in cases)

    # this rank's shard of the (8192*world) x 8192 weight, four seeded copies
    weights = []
    for i in range(N_WEIGHT_COPIES):
        g = torch.Generator(device="cpu").manual_seed(2000 + 97 * rank + i)
        weights.append((torch.randn(8192, 8192, generator=g) / 8192 ** 0.5).to(torch.float16).to(dev))
    xs_host = [wl.make_activation(c).pin_memory() for c in cases]
    xs = [x.to(dev) for x in xs_host]
    layers = [shard.ShardedLinear(w, 8192 * world) for w in weights]

    stream = torch.cuda.Stream(device=dev)
    state = {"i": 0}

    def step_local():
        for ci in range(len(cases)):
            layers[(state["i"] + ci) % N_WEIGHT_COPIES].forward_local(xs[ci])
        state["i"] += 1

    def step_gather():
        for ci in range(len(cases)):
            layers[(state["i"] + ci) % N_WEIGHT_COPIES].forward(xs[ci])
        state["i"] += 1

    def step_push():
        # The five calls are chained the way the layers of a model are: call i+1 reads its
        # activations only after every rank's tiles of call i have landed here (a wait inside
        # the kernel, after its first weight tiles are already on their way); one wait kernel
        # closes the step, so all five outputs are complete on every rank when the step ends.
        prev = None
        for ci in range(len(cases)):
            lay = layers[(state["i"] + ci) % N_WEIGHT_COPIES]
            lay.forward_push(xs[ci], wait=False, after=prev)
            prev = lay.last_push(cases[ci].M)
        lay.push_wait(prev)
        state["i"] += 1

    # ---- device-resident timing -------------------------------------------------------
    graph = None
    use_graph = (not args.no_graph) and world == 1
    with torch.cuda.stream(stream):
        for _ in range(3):
            step_local()
        torch.cuda.synchronize()
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(N_WEIGHT_COPIES):  # every rotation of the copies
                    step_local()

    launches0 = fg.launch_count()
    sampler = ClockSampler(local) if rank == 0 else None
    if graph is not None:
        # one replay = N_WEIGHT_COPIES steps
        reps = max(1, -(-args.steps // N_WEIGHT_COPIES))
        wreps = max(1, -(-args.warmup // N_WEIGHT_COPIES))
        ms_local = time_steps(None, reps, wreps, world, stream, graph=graph) * args.steps / (reps * N_WEIGHT_COPIES)
        launches = reps * N_WEIGHT_COPIES * len(cases)
    else:
        ms_local = time_steps(step_local, args.steps, args.warmup, world, stream)
        launches = fg.launch_count() - launches0 - args.warmup * len(cases)
    ms_nccl = None
    gather_kind = "none (single GPU)"
    if world > 1:
        ms_nccl = time_steps(step_gather, args.steps, args.warmup, world, stream)
        ms_full, gather_kind = ms_nccl, "NCCL all_gather_into_tensor + [g,M,N/g]->[M,N] copy per call"
        if not args.no_push:
            try:
                with torch.cuda.stream(stream):
                    step_push()  # collective: allocates and exchanges the symmetric outputs
                    torch.cuda.synchronize()
                ms_full = time_steps(step_push, args.steps, args.warmup, world, stream)
                gather_kind = "fused: epilogue stores tiles into every rank's C over NVLink + bounded flag wait"
            except Exception as e:  # symmetric memory unavailable: keep the NCCL number
                sys.stderr.write(f"rank {rank}: fused all-gather unavailable ({e}); reporting the NCCL path\n")
    else:
        ms_full = ms_local
    if world == 1:
        hold_load(graph.replay if graph is not None else step_local, stream)
    clocks = sampler.stop() if sampler else None
    if clocks is not None and world == 1:
        clocks["window"] = "the timed region and 0.5 s more of the same step, replayed untimed"

    # per-M device time (graph of 20 calls on rotating copies), for the breakdown
    per_call = {}
    if world == 1:
        with torch.cuda.stream(stream):
            for ci, c in enumerate(cases):
                gg = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gg, stream=stream):
                    for r in range(20):
                        layers[r % N_WEIGHT_COPIES].forward_local(xs[ci])
                gg.replay()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(5):
                    gg.replay()
                e1.record(stream)
                torch.cuda.synchronize()
                us = e0.elapsed_time(e1) * 1e3 / 100
                per_call[f"M{c.M}"] = {"us": round(us, 2), "GBps": round(c.algorithmic_bytes / us / 1e3, 1)}

    # the same 20 calls (five M values x four weight copies) as ONE grouped launch: what the
    # per-call fixed cost (launch, prologue, tail of split tiles) amounts to
    grouped = None
    if world == 1:
        try:
            from fastgate_b200.group import LinearGroup

            g_xs = [xs[ci] for _ in range(N_WEIGHT_COPIES) for ci in range(len(cases))]
            g_ws = [weights[w] for w in range(N_WEIGHT_COPIES) for _ in range(len(cases))]
            g_cs = [torch.empty(x.shape[0], 8192, dtype=torch.float16, device=dev) for x in g_xs]
            grp = LinearGroup(g_xs, g_ws, g_cs)
            with torch.cuda.stream(stream):
                for _ in range(3):
                    grp.run()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(10):
                    grp.run()
                e1.record(stream)
                torch.cuda.synchronize()
            ms_g = e0.elapsed_time(e1) / 10 / N_WEIGHT_COPIES  # per step of five calls
            grouped = {"value": bytes_step_rank / ms_g / 1e6, "unit": "GB/s", "ms_per_step": ms_g,
                       "note": "20 calls as one grouped launch (fg_group_run); not the headline: one launch per call is"}
            del grp, g_cs
        except Exception as e:
            sys.stderr.write(f"grouped launch unavailable ({e})\n")

    # ---- end to end through the operator, host activations in, host result out -----------
    e2e = None
    if not args.no_e2e:
        outs_host = [torch.empty(c.M, c.N, dtype=torch.float16).pin_memory() for c in cases]
        x_stage = [torch.empty_like(x) for x in xs]

        use_push = world > 1 and gather_kind.startswith("fused")

        # single GPU: the step's five activations travel as one pinned block, the five
        # results come back as one block (one copy each way per step)
        rows = [0]
        for c in cases:
            rows.append(rows[-1] + c.M)
        x_all_host = torch.cat(xs_host).pin_memory()
        x_all_dev = torch.empty_like(x_all_host, device=dev)
        out_all_dev = torch.empty(rows[-1], cases[0].N, dtype=torch.float16, device=dev)
        out_all_host = torch.empty(rows[-1], cases[0].N, dtype=torch.float16).pin_memory()

        def step_e2e():
            if world == 1:
                x_all_dev.copy_(x_all_host, non_blocking=True)
                for ci in range(len(cases)):
                    fg.edgemm_m8n128k64x4_bt(x_all_dev[rows[ci]:rows[ci + 1]], weights[(state["i"] + ci) % N_WEIGHT_COPIES],
                                             out_all_dev[rows[ci]:rows[ci + 1]])
                out_all_host.copy_(out_all_dev, non_blocking=True)
            else:
                for ci in range(len(cases)):
                    x_stage[ci].copy_(xs_host[ci], non_blocking=True)
                for ci in range(len(cases)):
                    lay = layers[(state["i"] + ci) % N_WEIGHT_COPIES]
                    res = lay.forward_push(x_stage[ci]) if use_push else lay.forward(x_stage[ci])
                    # the next call may reuse the layer's output buffer: read it out now
                    outs_host[ci].copy_(res[:, :cases[ci].N], non_blocking=True)
            state["i"] += 1
            torch.cuda.current_stream().synchronize()  # the caller has its results

        if world == 1:
            def compute_e2e(x_dev, out_dev):
                for ci in range(len(cases)):
                    fg.edgemm_m8n128k64x4_bt(x_dev[rows[ci]:rows[ci + 1]], weights[(state["i"] + ci) % N_WEIGHT_COPIES],
                                             out_dev[rows[ci]:rows[ci + 1]])
                state["i"] += 1

            ms_e2e = pipelined_e2e(compute_e2e, x_all_host, rows[-1], cases[0].N, dev, stream, args.steps, args.warmup)
        else:
            ms_e2e = time_steps(step_e2e, args.steps, args.warmup, world, stream)
        e2e = {"value": bytes_step_rank * world / (ms_e2e / args.steps) / 1e6, "unit": "GB/s",
               "ms_per_step": ms_e2e / args.steps,
               "how": ("two steps in flight: copies on side streams, the host waits for step k-1 while step k runs"
                       if world == 1 else "one step at a time, stream synchronised per step"),
               "h2d_bytes_per_step": sum(x.numel() * 2 for x in xs_host),
               "d2h_bytes_per_step": sum(o.numel() * 2 for o in outs_host)}

    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    ms_step = ms_full / args.steps
    ms_step_local = ms_local / args.steps
    avg_launch_s = ms_step_local / 1e3 / len(cases)
    avg_bytes = bytes_step_rank / len(cases)
    achieved = avg_bytes / avg_launch_s / 1e9
    line = {
        "metric": "effective HBM GB/s of M<=16 fp16 GEMM-GEMV (edgemm_m8n128k64x4_bt, K=N=8192)",
        "value": bytes_step_rank * world / ms_step / 1e6, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": "bt_sweep: edgemm_m8n128k64x4_bt, M in {1,2,4,8,16}, K=N=8192 per GPU, weight NxK fp16",
                   "calls_per_step": len(cases), "l2": f"{N_WEIGHT_COPIES} rotating weight copies (537 MB) > 126 MB L2",
                   "launch": "cuda graph replay" if graph is not None else "stream launches",
                   "sharding": f"N-sharded, {world} x 8192 columns; gather: {gather_kind}" if world > 1 else "single GPU"},
        "us_per_call": ms_step * 1e3 / len(cases),
        "per_call": per_call,
        "no_gather": {"value": bytes_step_rank * world / ms_step_local / 1e6, "unit": "GB/s", "ms_per_step": ms_step_local},
        "nccl_gather": None if ms_nccl is None else {"value": bytes_step_rank * world / (ms_nccl / args.steps) / 1e6,
                                                     "unit": "GB/s", "ms_per_step": ms_nccl / args.steps},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_8000": achieved / 8000.0,
                     "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "kernel": "fg::fg_umma_kernel<1,16>",
                     "algorithmic_bytes_per_launch": avg_bytes},
        "clocks": clocks, "gpu_launches": int(launches), "e2e": e2e, "grouped": grouped,
    }
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline_leg(cases)
    return line


def _graph_time(step_fn, steps, warmup, world, stream, use_graph):
    import torch

    graph = None
    with torch.cuda.stream(stream):
        for _ in range(2):
            step_fn()
        torch.cuda.synchronize()
        if use_graph:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                step_fn()
    return time_steps(step_fn, steps, warmup, world, stream, graph=graph), graph is not None


def run_other_workload(args):
    """Configs 1, 3, 4 (single GPU) and 5 (the DiT stack, N-sharded over the ranks)."""
    import torch

    import fastgate_b200 as fg
    from fastgate_b200 import shard, workloads as wl

    world, rank, local = dist_setup(args)
    dev = torch.device("cuda", local)
    stream = torch.cuda.Stream(device=dev)
    peak, peak_kind = measured_peak()
    name = args.workload
    extra = {}
    if name != "dit":
        if world != 1:
            raise SystemExit(f"--workload {name} is a single-GPU workload")
        cases = {"cfg1": wl.cfg1, "cfg3": wl.cfg3, "cfg4": wl.cfg4, "w4": wl.w4}[name]()
        copies = []  # per case: rotating weight copies beyond the L2 size
        for c in cases:
            n_rot = max(2, -(-600 * 2 ** 20 // c.weight_bytes))
            w0 = wl.make_weight(c).to(dev)
            copies.append([w0] + [w0.clone() for _ in range(n_rot - 1)])
        xs = [wl.make_activation(c).to(dev) for c in cases]
        scs = [wl.make_scales(c) for c in cases]
        scs = [t.to(dev) if t is not None else None for t in scs]
        outs = [torch.zeros(c.M, c.N, dtype=torch.float16, device=dev) for c in cases]
        state = {"i": 0}

        def call(ci, w):
            c = cases[ci]
            if c.op == wl.OP_KN:
                fg.edgemm_m8n128k64x4(xs[ci], w, outs[ci])
            elif c.op == wl.OP_NK:
                fg.fastgemv(w, xs[ci], outs[ci])
            elif c.op == wl.OP_W8:
                fg.fastgemv_int8(w, xs[ci], outs[ci], scs[ci])
            else:
                fg.fastgemv_int4(w, xs[ci], outs[ci], scs[ci])

        n_rot_all = max(len(c) for c in copies)

        def step_once():
            for ci in range(len(cases)):
                call(ci, copies[ci][state["i"] % len(copies[ci])])
            state["i"] += 1

        def step():  # one graph = every rotation, so that a replay never re-reads a cached weight
            for _ in range(n_rot_all):
                step_once()

        n0 = fg.launch_count()
        sampler = ClockSampler(local)
        reps = max(1, -(-args.steps // n_rot_all))
        ms, graphed = _graph_time(step, reps, max(1, -(-args.warmup // n_rot_all)), 1, stream, not args.no_graph)
        hold_load(step_once, stream)
        clocks = sampler.stop()
        clocks["window"] = "the timed region and 0.5 s more of the same calls, untimed"
        steps_done = reps * n_rot_all
        ms_step = ms / steps_done
        bytes_step = sum(c.algorithmic_bytes for c in cases)
        launches = steps_done * len(cases)
        workload = {"cfg1": "edgemm_m8n128k64x4: M=8, K=N=4096, weight KxN fp16",
                    "cfg3": "fastgemv: M=1, weight 11008x4096 and 4096x11008 fp16 (NxK)",
                    "cfg4": "fastgemv_int8: M in {1,8}, weight int8 28672x8192 + fp16 scale per output channel",
                    "w4": "fastgemv_int4: M in {1,8,16}, weight 28672x8192 packed 4-bit + fp16 scale per 128 k"}[name]
        sharding = "single GPU"
        scaling = "weak"
        metric = "effective HBM GB/s of M<=16 fp16/int8 GEMM-GEMV"
        n_calls = len(cases)
    else:
        cases_all = wl.cfg5(args.layers)
        g = torch.Generator(device=dev).manual_seed(5000 + rank)
        layers, xs = [], []
        for c in cases_all:  # this rank's rows of every weight (seeded on the device: 9 GB in total)
            n_loc = c.N // world
            w = (torch.randn(n_loc, c.K, device=dev, generator=g, dtype=torch.float32) / c.K ** 0.5).to(torch.float16)
            layers.append(shard.ShardedLinear(w, c.N))
        for j in range(4):
            xs.append(torch.randn(16, wl.DIT_LINEARS[j][2], device=dev, generator=g).to(torch.float16))
        state = {"i": 0}

        def step_local():
            for i, lay in enumerate(layers):
                lay.forward_local(xs[i % 4])

        def step_nccl():
            for i, lay in enumerate(layers):
                lay.forward(xs[i % 4])

        def step_push():
            prev = None
            for i, lay in enumerate(layers):
                lay.forward_push(xs[i % 4], wait=False, after=prev)
                prev = lay.last_push(16)
            lay.push_wait(prev)

        n0 = fg.launch_count()
        sampler = ClockSampler(local) if rank == 0 else None
        ms_local, graphed = _graph_time(step_local, args.steps, args.warmup, world, stream, (not args.no_graph) and world == 1)
        ms, gather_kind = ms_local, "none (single GPU)"
        if world > 1:
            ms_nccl, _ = _graph_time(step_nccl, args.steps, args.warmup, world, stream, False)
            ms, gather_kind = ms_nccl, "NCCL all_gather_into_tensor + copy per linear"
            extra["nccl_gather"] = {"ms_per_step": ms_nccl / args.steps}
            if not args.no_push:
                try:
                    ms_push, _ = _graph_time(step_push, args.steps, args.warmup, world, stream, False)
                    ms, gather_kind = ms_push, "fused: tiles pushed into every rank's output + in-kernel dependency wait"
                except Exception as e:
                    sys.stderr.write(f"rank {rank}: fused all-gather unavailable ({e})\n")
        extra["per_layer_launches"] = {"ms_per_step": ms / args.steps, "gather": gather_kind}
        # The config gives every projection its own input, so the whole stack can also run as ONE
        # grouped launch (at N > 1 with the tiles pushed into every rank's outputs and a single
        # bounded wait at the end of the pass).
        try:
            from fastgate_b200.group import LinearGroup

            g_xs = [xs[i % 4] for i in range(len(layers))]
            g_ws = [lay.w for lay in layers]
            if world == 1:
                g_cs = [torch.empty(16, lay.n_total, dtype=torch.float16, device=dev) for lay in layers]
                grp = LinearGroup(g_xs, g_ws, g_cs)

                def step_group():
                    grp.run()
            else:
                pbs = [lay.push_buffers(16, dev) for lay in layers]
                gflag = shard.PushBuffers(16, 128, dev)
                grp = LinearGroup(g_xs, g_ws, None, peer_C_ptrs=[pb.c_ptrs for pb in pbs], flag_ptrs=gflag.flag_ptrs,
                                  rank=rank, n_totals=[lay.n_total for lay in layers],
                                  mc_C_ptrs=[pb.mc_out for pb in pbs], mc_flag_ptr=gflag.mc_flag)

                def step_group():
                    grp.run()
                    gflag.target += grp.tiles
                    fg.push_wait(gflag.flag_ptrs[rank], world, gflag.target, local)
            ms_group, g_graphed = _graph_time(step_group, args.steps, args.warmup, world, stream,
                                              (not args.no_graph) and world == 1)
            extra["per_layer_launches"]["value"] = sum(c.algorithmic_bytes for c in cases_all) / (ms / args.steps) / 1e6
            ms, graphed = ms_group, g_graphed
            ms_local = min(ms_local, ms_group) if world == 1 else ms_local
            gather_kind = "one grouped launch per pass" + (", tiles pushed into every rank's outputs, one wait" if world > 1 else "")
            extra["grouped"] = True
        except Exception as e:
            sys.stderr.write(f"rank {rank}: grouped launch unavailable ({e})\n")
        # The same weights wired as a stack whose layers DO feed each other (qkv -> out + residual
        # -> up + bias, gelu -> down + residual, block after block; the attention between qkv and
        # out is left out, out reads the first 3072 columns of qkv): one cooperative launch per
        # pass, to set beside per_layer_launches, which is what such a stack costs call by call.
        if world == 1:
            try:
                from fastgate_b200.chain import LayerChain

                h = xs[0].clone()
                c_bias = (torch.randn(12288, device=dev, generator=g) * 0.1).to(torch.float16)
                c_res = xs[1].clone()  # a fixed residual keeps the magnitudes of 160 chained layers bounded
                spec, prev = [], -1
                for b in range(len(layers) // 4):
                    wq, wo, wu, wd = (layers[4 * b + j].w for j in range(4))
                    qkv = torch.empty(16, 9216, dtype=torch.float16, device=dev)
                    h1 = torch.empty(16, 3072, dtype=torch.float16, device=dev)
                    up = torch.empty(16, 12288, dtype=torch.float16, device=dev)
                    h2 = torch.empty(16, 3072, dtype=torch.float16, device=dev)
                    base = len(spec)
                    spec += [dict(x=h, W=wq, C=qkv, dep=prev),
                             dict(x=qkv[:, :3072], W=wo, C=h1, dep=base, residual=c_res),
                             dict(x=h1, W=wu, C=up, dep=base + 1, bias=c_bias, act="gelu_tanh"),
                             dict(x=up, W=wd, C=h2, dep=base + 2, residual=c_res)]
                    h, prev = h2, base + 3
                chain = LayerChain(spec)
                ms_chain, _ = _graph_time(chain.run, args.steps, args.warmup, world, stream, not args.no_graph)
                if chain.status() != 0:
                    raise RuntimeError("chain kernel reported a timeout")
                extra["dependent_chain"] = {
                    "ms_per_step": ms_chain / args.steps, "unit": "GB/s",
                    "value": sum(c.algorithmic_bytes for c in cases_all) / (ms_chain / args.steps) / 1e6,
                    "us_per_layer": ms_chain / args.steps * 1e3 / len(spec),
                    "what": "every layer reads the previous layer's output; one cooperative launch per pass"}
            except Exception as e:
                sys.stderr.write(f"dependent chain unavailable ({e})\n")
        clocks = sampler.stop() if sampler else None
        steps_done = args.steps
        ms_step = ms / steps_done
        bytes_step = sum(c.algorithmic_bytes for c in cases_all)  # whole model, whatever the number of ranks
        extra["no_gather"] = {"value": bytes_step / (ms_local / steps_done) / 1e6, "unit": "GB/s",
                              "ms_per_step": ms_local / steps_done}
        if "nccl_gather" in extra:
            extra["nccl_gather"]["value"] = bytes_step / extra["nccl_gather"]["ms_per_step"] / 1e6
            extra["nccl_gather"]["unit"] = "GB/s"
        # one grouped launch per pass (plus the wait kernel at N > 1), else one launch per projection
        launches = steps_done * ((2 if world > 1 else 1) if extra.get("grouped") else len(cases_all))
        workload = (f"dit: {args.layers} layers x (3072->9216, 3072->3072, 3072->12288, 12288->3072), M=16, fp16, "
                    f"weights NxK, {sum(c.weight_bytes for c in cases_all) / 1e9:.2f} GB")
        sharding = f"N-sharded over {world} GPUs; {gather_kind}" if world > 1 else f"single GPU; {gather_kind}"
        scaling = "strong"
        metric = "effective HBM GB/s of the DiT linear stack (M=16 fp16 GEMM, N-sharded)"
        n_calls = len(cases_all)
        ms_step_local = ms_local / steps_done
    if rank != 0:
        return None
    if name != "dit":
        ms_step_local = ms_step
    per_rank_bytes = bytes_step / (world if name == "dit" else 1)
    achieved = per_rank_bytes / n_calls / (ms_step_local / 1e3 / n_calls) / 1e9
    line = {
        "metric": metric, "value": bytes_step / ms_step / 1e6, "unit": "GB/s", "n_gpus": world, "steps": steps_done,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
        "dtype": {"cfg4": "int8 weights, f16 activations (fp32 accumulate)",
                  "w4": "int4 weights, f16 activations (fp32 accumulate)"}.get(name, "f16 (fp32 accumulate)"),
        "data": "synthetic",
        "config": {"workload": workload, "calls_per_step": n_calls, "sharding": sharding,
                   "l2": "weights rotate over more than 600 MB" if name != "dit" else "9 GB of distinct weights per pass",
                   "launch": "cuda graph replay" if graphed else "stream launches"},
        "us_per_call": ms_step * 1e3 / n_calls,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_8000": achieved / 8000.0, "traffic": None,
                     "kernel": "fg::fg_streamk_kernel / fg::fg_umma_kernel"},
        "clocks": clocks, "gpu_launches": int(launches), "e2e": None,
    }
    line.update(extra)
    return line


def run_reference(args):
    """The reference's own implementation of the path: its kernels rebuilt for sm_100a when
    available (and a GPU is present), else the CPU oracle port on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    from fastgate_b200 import workloads as wl

    cases = wl.cfg2()
    bytes_step = sum(c.algorithmic_bytes for c in cases)
    cpu = cpu_baseline_leg(cases)
    want_gpu = args.reference_arm in ("auto", "gpu")
    ref = None
    if want_gpu:
        try:
            import torch

            from oracle import ref_gpu
            if torch.cuda.is_available():
                ref = ref_gpu.load()
        except Exception as e:  # unloadable build: fall back to the port
            ref = None
            sys.stderr.write(f"reference kernels unavailable: {e}\n")
    base = {
        "impl": "reference",
        "metric": "effective HBM GB/s of M<=16 fp16 GEMM-GEMV (edgemm_m8n128k64x4_bt, K=N=8192)",
        "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "data": "synthetic",
        "config": {"workload": "bt_sweep: edgemm_m8n128k64x4_bt, M in {1,2,4,8,16}, K=N=8192 per GPU, weight NxK fp16",
                   "calls_per_step": len(cases)},
        "cpu_baseline": cpu,
    }
    if ref is None:
        sec = cpu["ms_per_step"] / 1e3
        base.update({"value": bytes_step / sec / 1e9, "ms_per_step": sec * 1e3, "dtype": "f32 accumulate (CPU port)",
                     "reference_kind": "cpu oracle port (reference kernels not built or no GPU)",
                     "e2e": {"value": bytes_step / sec / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
        return base

    import torch

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    weights = []
    for i in range(N_WEIGHT_COPIES):
        g = torch.Generator(device="cpu").manual_seed(2000 + i)
        weights.append((torch.randn(8192, 8192, generator=g) / 8192 ** 0.5).to(torch.float16).to(dev))
    xs_host = [wl.make_activation(c).pin_memory() for c in cases]
    xs = [x.to(dev) for x in xs_host]
    outs = [torch.zeros(c.M, c.N, dtype=torch.float16, device=dev) for c in cases]
    outs_host = [torch.empty(c.M, c.N, dtype=torch.float16).pin_memory() for c in cases]
    x_stage = [torch.empty_like(x) for x in xs]
    state = {"i": 0}
    # the reference launches on the legacy default stream (hk/edgemm.cu:319), so time there
    stream = torch.cuda.default_stream(dev)

    def step():
        for ci in range(len(cases)):
            ref.edgemm_m8n128k64x4_bt(xs[ci], weights[(state["i"] + ci) % N_WEIGHT_COPIES], outs[ci])
        state["i"] += 1

    rows = [0]
    for c in cases:
        rows.append(rows[-1] + c.M)
    x_all_host = torch.cat(xs_host).pin_memory()
    sampler = ClockSampler(0)
    ms = time_steps(step, args.steps, args.warmup, 1, stream)
    hold_load(step, stream)
    clocks = sampler.stop()
    clocks["window"] = "the timed region and 0.5 s more of the same step, untimed"
    def compute_e2e(x_dev, out_dev):  # same shape as our arm: one block in, five operator calls, one block out
        for ci in range(len(cases)):
            ref.edgemm_m8n128k64x4_bt(x_dev[rows[ci]:rows[ci + 1]], weights[(state["i"] + ci) % N_WEIGHT_COPIES],
                                      out_dev[rows[ci]:rows[ci + 1]])
        state["i"] += 1

    ms_e2e = pipelined_e2e(compute_e2e, x_all_host, rows[-1], cases[0].N, dev, stream, args.steps, args.warmup)
    base.update({
        "value": bytes_step / (ms / args.steps) / 1e6, "ms_per_step": ms / args.steps,
        "dtype": "f16 (fp16 accumulate)", "clocks": clocks,
        "reference_kind": "reference kernels (hk/edgemm.cu:274-324) rebuilt unmodified for sm_100a, same B200",
        "e2e": {"value": bytes_step / (ms_e2e / args.steps) / 1e6, "unit": "GB/s", "ms_per_step": ms_e2e / args.steps,
                "how": "two steps in flight: copies on side streams, the host waits for step k-1 while step k runs",
                "h2d_bytes_per_step": sum(x.numel() * 2 for x in xs_host),
                "d2h_bytes_per_step": sum(o.numel() * 2 for o in outs_host)},
    })
    return base


def main():
    args = parse_args()
    if args.impl == "reference":
        line = run_reference(args)
    elif args.workload == "bt_sweep":
        line = run_ours(args)
    else:
        line = run_other_workload(args)
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
    except Exception:
        pass
    if line is not None:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
