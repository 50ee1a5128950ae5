#!/usr/bin/env python
"""Benchmark of the small-batch matmul hot path (one JSON line on stdout, rank 0).

Headline workload "bt_sweep" (config 2): one step = five calls of edgemm_m8n128k64x4_bt,
M in {1,2,4,8,16}, K = N = 8192 per GPU, fp16, weight stored NxK; each call streams a
different one of four weight copies (537 MB, larger than the 126 MB L2).  With N GPUs every
rank holds its own 8192-row shard of an (8192*N) x 8192 weight ("weak" scaling) and the
output slices are assembled on every rank.

  value     inputs resident in HBM, step replayed from a CUDA graph (N = 1) or launched on
            a stream (N > 1), timed with CUDA events on the launching stream: the median of
            five batches of exactly --steps steps (all batches are listed)
  e2e       the same step through the public operator with the step's activations copied
            from pinned host memory and its results copied back every step, two steps in
            flight (copies on side streams; the host waits for step k-1 while step k runs);
            the weight stays resident, as at the reference's call sites
  roofline  algorithmic bytes per launch / average launch duration, against the measured
            copy bandwidth of this pool's B200s
  configs   the other configurations of the metric, each timed the same way (graph replay over
            rotating weight copies, median of five): config 1 (edgemm_m8n128k64x4), 3a / 3b
            (fastgemv), 4 (fastgemv_int8, M = 1 and 8), 5 (the DiT linear stack: one launch per
            linear, one grouped launch, one dependent chain), with cuBLAS through torch.matmul
            in the same harness beside them
  dit       N > 1: config 5 N-sharded over the ranks (strong scaling): shards only, NCCL
            all-gather per linear, fused push per linear, one grouped launch with fused push
  cpu_baseline  the CPU oracle (a port of the reference's arithmetic, OpenMP) and torch.matmul
            fp32 on this box's host cores, for one step

`--impl reference` times the reference's own kernels, rebuilt unmodified for sm_100a
(oracle/_ref), on the same workloads through the reference's operators; when that build is
not available it falls back to the CPU oracle port.
"""
from __future__ import annotations

import argparse
import importlib.util
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
N_BATCHES = 5
# dram__bytes_read.sum + dram__bytes_write.sum per launch from one ncu capture of the named kernel
# on an 8192 x 8192 weight (see the profile summaries that ship with the repository)
NCU_TRAFFIC = {"kernel": "fg::fg_umma_kernel<1,16>", "bytes_per_launch": 138.0e6}
METRIC = "effective HBM GB/s of M<=16 fp16 GEMM-GEMV (edgemm_m8n128k64x4_bt, K=N=8192)"
WORKLOAD = "bt_sweep: edgemm_m8n128k64x4_bt, M in {1,2,4,8,16}, K=N=8192 per GPU, weight NxK fp16"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--workload", choices=("bt_sweep", "cfg1", "cfg3", "cfg4", "w4", "dit"), default="bt_sweep",
                    help="bt_sweep (default: config 2 as the headline plus every other config) | one config alone")
    ap.add_argument("--layers", type=int, default=40, help="dit: number of layers")
    ap.add_argument("--no-graph", action="store_true", help="launch on a stream instead of replaying a CUDA graph")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline only: skip the other configurations")
    ap.add_argument("--no-push", action="store_true", help="N > 1: assemble outputs with NCCL only")
    ap.add_argument("--reference-arm", choices=("auto", "gpu", "cpu"), default="auto")
    return ap.parse_args()


def load_workloads():
    """fastgate_b200/workloads.py as a stand-alone module: the reference arm must not import the
    package (whose __init__ loads the native extension)."""
    spec = importlib.util.spec_from_file_location("fg_workloads", os.path.join(ROOT, "fastgate_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules["fg_workloads"] = mod
    spec.loader.exec_module(mod)
    return mod


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


def time_batches(step_fn, steps: int, warmup: int, world: int, stream, graph=None, batches: int = N_BATCHES) -> list:
    """`batches` timed regions of exactly `steps` steps each (the first one after `warmup` warm-up
    steps): ms per region."""
    out = [time_steps(step_fn, steps, warmup, world, stream, graph=graph)]
    for _ in range(batches - 1):
        out.append(time_steps(step_fn, steps, 0, world, stream, graph=graph))
    return out


def spread(ms_list, per: float) -> dict:
    """Median / min / max of the batches, in ms per `per` steps."""
    v = sorted(m / per for m in ms_list)
    return {"n": len(v), "median": statistics.median(v), "min": v[0], "max": v[-1]}


def pipelined_e2e(compute, x_all_host, n_rows: int, n_cols: int, dev, stream, steps: int, warmup: int, world: int = 1,
                  read_out=None, prepare=None) -> float:
    """ms for `steps` end-to-end steps on this rank's GPU, two steps deep, max over ranks.

    Every step copies its activations from pinned host memory (side stream), runs
    `compute(x_dev, out_dev, k)` on `stream` and copies the results back to pinned host memory
    (another side stream); the host waits for the results of step k-1 while step k is in
    flight, as a serving loop does.  All copies of all timed steps lie inside the timed
    region, which ends when the last step's results are in host memory.  `read_out(out_dev, k)`
    (optional) moves a step's results into out_dev on `stream` when `compute` leaves them
    elsewhere.  `prepare(x_dev, out_dev)` (optional) sees the two sets of device buffers before the
    first step (to capture graphs over them)."""
    import torch

    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    x_dev = [torch.empty_like(x_all_host, device=dev) for _ in range(2)]
    out_dev = [torch.zeros(n_rows, n_cols, dtype=torch.float16, device=dev) for _ in range(2)]
    out_host = [torch.empty(n_rows, n_cols, dtype=torch.float16).pin_memory() for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]
    counter = {"k": 0}
    if prepare is not None:
        prepare(x_dev, out_dev)

    def run(n: int) -> int:
        last = 0
        for _ in range(n):
            k = counter["k"]
            counter["k"] += 1
            b = k & 1
            with torch.cuda.stream(s_in):  # x_dev[b] was last read by step k-2, whose results the host already has
                x_dev[b].copy_(x_all_host, non_blocking=True)
                ev_in[b].record(s_in)
            stream.wait_event(ev_in[b])
            compute(x_dev[b], out_dev[b], k)
            if read_out is not None:
                read_out(out_dev[b], k)
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
        barrier_sync(world)
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        s_in.wait_event(e0)
        last = run(steps)
        stream.wait_event(ev_out[last])
        stream.wait_event(ev_out[1 - last])
        e1.record(stream)
        barrier_sync(world)
    return max_over_ranks(e0.elapsed_time(e1), world)


def cpu_baseline_leg(cases, sample_reps: int = 3) -> dict:
    """One full step on this box's host cores: the CPU oracle (a port of the reference's
    arithmetic, OpenMP) and, beside it, torch.matmul in fp32 (weights converted outside the
    timed region: fp16 CPU matmul would be a strawman)."""
    import numpy as np
    import torch

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
    out = {"value": bytes_step / sec / 1e9, "unit": "GB/s", "cores": oracle.num_threads(), "kind": "port",
           "sample": f"one full step (5 calls, M=1,2,4,8,16, K=N=8192), median of {sample_reps}",
           "ms_per_step": sec * 1e3}
    try:
        Wt = torch.from_numpy(W).float().t().contiguous()
        xt = [torch.from_numpy(x).float() for x in xs]
        torch.matmul(xt[0], Wt)
        tt = []
        for _ in range(5):
            t0 = time.perf_counter()
            for x in xt:
                torch.matmul(x, Wt)
            tt.append(time.perf_counter() - t0)
        sec_t = statistics.median(tt)
        out["torch_matmul"] = {"value": bytes_step / sec_t / 1e9, "unit": "GB/s (fp16 algorithmic bytes / time)",
                               "ms_per_step": sec_t * 1e3, "threads": torch.get_num_threads(), "cpu_count": os.cpu_count(),
                               "sample": "the same step with fp32 weights (converted outside the timed region), median of 5"}
    except Exception as e:  # pragma: no cover
        out["torch_matmul"] = {"unavailable": str(e)}
    return out


def graph_of(step_fn, stream, use_graph: bool, warm: int = 2):
    """Warm up `step_fn` and capture it once (or return None)."""
    import torch

    with torch.cuda.stream(stream):
        for _ in range(warm):
            step_fn()
        torch.cuda.synchronize()
        if not use_graph:
            return None
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
            step_fn()
    return g


def us_per_call(step_fn, calls_per_step: int, stream, use_graph: bool = True, reps: int = 4, warm_reps: int = 2) -> dict:
    """Median / min / max us per call of `step_fn` (which makes `calls_per_step` launches), graph
    replayed `reps` times per batch, five batches."""
    g = graph_of(step_fn, stream, use_graph)
    ms = time_batches(step_fn, reps, warm_reps, 1, stream, graph=g)
    s = spread(ms, reps * calls_per_step)
    return {"us": s["median"] * 1e3, "us_min": s["min"] * 1e3, "us_max": s["max"] * 1e3}


# ---- the other configurations, single GPU -------------------------------------------------------
def other_configs(dev, stream, peak: float, layers: int = 40) -> dict:
    """Configs 1, 3a, 3b, 4 (M = 1, 8) and 5 on one GPU: our operator and cuBLAS (torch.matmul) in
    the same harness.  Every call of a graph streams another weight copy (more than 600 MB in
    rotation), so nothing is served from L2."""
    import torch

    import fastgate_b200 as fg
    from fastgate_b200 import workloads as wl

    out = {}

    def entry(bytes_call, t, cublas=None, **extra):
        e = {"us_per_call": round(t["us"], 3), "us_min": round(t["us_min"], 3), "us_max": round(t["us_max"], 3),
             "GBps": round(bytes_call / t["us"] / 1e3, 1), "frac": round(bytes_call / t["us"] / 1e3 / peak, 4),
             "frac_of_8000": round(bytes_call / t["us"] / 1e3 / 8000.0, 4)}
        if cublas is not None:
            e["cublas_us"] = round(cublas["us"], 3)
        e.update(extra)
        return e

    singles = [("cfg1", wl.cfg1()[0], "edgemm_m8n128k64x4 M=8 K=N=4096 (KxN)"),
               ("cfg3a", wl.cfg3()[0], "fastgemv M=1 N=11008 K=4096"),
               ("cfg3b", wl.cfg3()[1], "fastgemv M=1 N=4096 K=11008"),
               ("cfg4_M1", wl.cfg4()[0], "fastgemv_int8 M=1 N=28672 K=8192, fp16 scale per channel"),
               ("cfg4_M8", wl.cfg4()[1], "fastgemv_int8 M=8 N=28672 K=8192, fp16 scale per channel")]
    for key, c, what in singles:
        n_rot = max(2, -(-600 * 2 ** 20 // c.weight_bytes))
        w0 = wl.make_weight(c).to(dev)
        ws = [w0] + [w0.clone() for _ in range(n_rot - 1)]
        x = wl.make_activation(c).to(dev)
        s = wl.make_scales(c)
        s = s.to(dev) if s is not None else None
        C = torch.zeros(c.M, c.N, dtype=torch.float16, device=dev)

        def ours():
            for w in ws:
                if c.op == wl.OP_KN:
                    fg.edgemm_m8n128k64x4(x, w, C)
                elif c.op == wl.OP_NK:
                    fg.fastgemv(w, x, C)
                else:
                    fg.fastgemv_int8(w, x, C, s)

        t = us_per_call(ours, n_rot, stream)
        cub = None
        if c.op != wl.OP_W8:  # cuBLAS has no fp16 x int8-weight GEMV
            wv = ws if c.op == wl.OP_KN else [w.t() for w in ws]

            def lib():
                for w in wv:
                    torch.matmul(x, w, out=C)

            cub = us_per_call(lib, n_rot, stream)
        out[key] = entry(c.algorithmic_bytes, t, cub, what=what)
        del ws, w0

    # config 5 on one GPU
    try:
        from fastgate_b200.chain import LayerChain
        from fastgate_b200.group import LinearGroup

        cases = wl.cfg5(layers)
        g = torch.Generator(device=dev).manual_seed(5000)
        ws = [(torch.randn(c.N, c.K, device=dev, generator=g, dtype=torch.float32) / c.K ** 0.5).to(torch.float16) for c in cases]
        xs = [torch.randn(16, wl.DIT_LINEARS[j][2], device=dev, generator=g).to(torch.float16) for j in range(4)]
        Cs = [torch.empty(16, c.N, dtype=torch.float16, device=dev) for c in cases]
        bytes_pass = sum(c.algorithmic_bytes for c in cases)
        n = len(cases)

        def per_linear():
            for i in range(n):
                fg.edgemm_m8n128k64x4_bt(xs[i % 4], ws[i], Cs[i])

        def lib():
            for i in range(n):
                torch.matmul(xs[i % 4], ws[i].t(), out=Cs[i])

        t = us_per_call(per_linear, n, stream, reps=2, warm_reps=1)
        cub = us_per_call(lib, n, stream, reps=2, warm_reps=1)
        out["cfg5_per_linear"] = entry(bytes_pass / n, t, cub, what=f"DiT stack, {layers} layers x 4 linears, M=16, one launch per linear",
                                       ms_per_pass=round(t["us"] * n / 1e3, 4))
        grp = LinearGroup([xs[i % 4] for i in range(n)], ws, Cs)
        t = us_per_call(grp.run, n, stream, reps=2, warm_reps=1)
        out["cfg5_grouped"] = entry(bytes_pass / n, t, None, what="the same stack as ONE grouped launch per pass (the config gives every "
                                    "projection its own input)", ms_per_pass=round(t["us"] * n / 1e3, 4))
        del grp
        # the same weights wired as a stack whose layers DO feed each other
        h = xs[0].clone()
        c_bias = (torch.randn(12288, device=dev, generator=g) * 0.1).to(torch.float16)
        c_res = xs[1].clone()
        spec, prev = [], -1
        for b in range(n // 4):
            wq, wo, wu, wd = (ws[4 * b + j] for j in range(4))
            qkv = torch.empty(16, 9216, dtype=torch.float16, device=dev)
            h1 = torch.empty(16, 3072, dtype=torch.float16, device=dev)
            up = torch.empty(16, 12288, dtype=torch.float16, device=dev)
            h2 = torch.empty(16, 3072, dtype=torch.float16, device=dev)
            base = len(spec)
            spec += [dict(x=h, W=wq, C=qkv, dep=prev), dict(x=qkv[:, :3072], W=wo, C=h1, dep=base, residual=c_res),
                     dict(x=h1, W=wu, C=up, dep=base + 1, bias=c_bias, act="gelu_tanh"),
                     dict(x=up, W=wd, C=h2, dep=base + 2, residual=c_res)]
            h, prev = h2, base + 3
        chain = LayerChain(spec)
        t = us_per_call(chain.run, n, stream, reps=2, warm_reps=1)
        if chain.status() != 0:
            raise RuntimeError("chain kernel reported a timeout")
        out["cfg5_chain"] = entry(bytes_pass / n, t, None, what="the same weights as a stack whose layers feed each other (fused bias, "
                                  "GELU, residuals), one cooperative launch per pass", ms_per_pass=round(t["us"] * n / 1e3, 4))
        del chain, spec, ws, Cs
    except Exception as e:
        out["cfg5_error"] = str(e)
    torch.cuda.empty_cache()
    return out


# ---- config 5 N-sharded over the ranks (strong scaling) ------------------------------------------
def dit_sharded(args, world: int, rank: int, local: int, dev, stream) -> dict:
    import torch

    import fastgate_b200 as fg
    from fastgate_b200 import shard, workloads as wl

    cases_all = wl.cfg5(args.layers)
    g = torch.Generator(device=dev).manual_seed(5000 + rank)
    layers = []
    for c in cases_all:  # this rank's rows of every weight (seeded on the device: 9 GB in total)
        w = (torch.randn(c.N // world, c.K, device=dev, generator=g, dtype=torch.float32) / c.K ** 0.5).to(torch.float16)
        layers.append(shard.ShardedLinear(w, c.N))
    xs = [torch.randn(16, wl.DIT_LINEARS[j][2], device=dev, generator=g).to(torch.float16) for j in range(4)]
    bytes_pass = sum(c.algorithmic_bytes for c in cases_all)  # the whole model, whatever the number of ranks
    steps, warm = max(2, min(args.steps, 10)), max(1, min(args.warmup, 3))
    res = {"workload": f"dit: {args.layers} layers x (3072->9216, 3072->3072, 3072->12288, 12288->3072), M=16, fp16, weights NxK, "
                       f"{sum(c.weight_bytes for c in cases_all) / 1e9:.2f} GB, N-sharded over {world} GPUs", "scaling": "strong",
           "steps": steps}

    def leg(name, fn, what, graphed=True):
        # Legs made of this library's kernels only are captured once (one pass) and replayed, as the
        # single-GPU configurations are; the NCCL leg is launched from the host call by call.
        try:
            graph = None
            with torch.cuda.stream(stream):
                fn()
                torch.cuda.synchronize()
                if graphed and not args.no_graph:
                    barrier_sync(world)
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(graph, stream=stream, capture_error_mode="thread_local"):
                        fn()
            ms = time_batches(fn, steps, warm, world, stream, graph=graph, batches=3)
            s = spread(ms, steps)
            res[name] = {"ms_per_pass": s["median"], "ms_min": s["min"], "ms_max": s["max"],
                         "value": bytes_pass / s["median"] / 1e6, "unit": "GB/s", "what": what,
                         "launch": "cuda graph replay" if graph is not None else "stream launches"}
            del graph
        except Exception as e:
            res[name] = {"unavailable": str(e)}

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

    leg("no_gather", step_local, "every rank computes its output slices, nothing is assembled")
    leg("nccl_gather", step_nccl, "all_gather_into_tensor + [g,M,N/g]->[M,N] copy after every linear", graphed=False)
    if not args.no_push:
        leg("push_per_linear", step_push, "tiles stored into every rank's output from the kernel's epilogue; each linear waits "
                                          "in-kernel for the previous one's tiles from all ranks")
        try:
            from fastgate_b200.group import LinearGroup

            pbs = [lay.push_buffers(16, dev) for lay in layers]
            gflag = shard.PushBuffers(16, 128, dev)
            grp = LinearGroup([xs[i % 4] for i in range(len(layers))], [lay.w for lay in layers], None,
                              peer_C_ptrs=[pb.c_ptrs for pb in pbs], flag_ptrs=gflag.flag_ptrs, rank=rank,
                              n_totals=[lay.n_total for lay in layers], mc_C_ptrs=[pb.mc_out for pb in pbs],
                              mc_flag_ptr=gflag.mc_flag, target_dev_ptr=gflag.target_ptr)

            def step_group():
                grp.run()
                fg.push_wait_dev(gflag.flag_ptrs[rank], world, gflag.target_ptr, local)

            leg("push_grouped", step_group, "the whole stack as one grouped launch per pass, tiles pushed into every rank's "
                                            "outputs, one wait" + (", multimem" if gflag.mc_flag else ""))
        except Exception as e:
            res["push_grouped"] = {"unavailable": str(e)}
    return res


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

    push_sets = {}  # slot -> one symmetric output + counters per call of a step

    def push_set(slot):
        # collective: every rank creates its sets in the same order
        if slot not in push_sets:
            push_sets[slot] = [shard.PushBuffers(16, 8192 * world, dev) for _ in cases]
        return push_sets[slot]

    def step_push(slot=0, inputs=None, sink=None, chained=False):
        # Five calls whose tiles go straight into every rank's output; wait kernels close the step, so
        # all five outputs are complete on every rank when the step ends.  As at N = 1 the calls do not
        # read each other's results, so a call only follows its predecessor in stream order.
        # chained=True: the calls are tied the way the layers of a model are: call i+1 reads its
        # activations only after every rank's tiles of call i have landed here (a wait inside the
        # kernel, after its first weight tiles are already on their way).
        # Each call of a step pushes into buffers of its own, each step in flight into a set of its own.
        bufs = push_set(slot)
        prev = None
        for ci in range(len(cases)):
            lay = layers[(state["i"] + ci) % N_WEIGHT_COPIES]
            res = lay.forward_push((inputs or xs)[ci], wait=False, after=prev if chained else None, into=bufs[ci])
            prev = bufs[ci]
            if sink is not None:
                sink.append((ci, res, prev))
        if chained:
            lay.push_wait(prev)  # the last call's counters imply the earlier ones'
        else:
            shard.push_wait_all(bufs)  # one wait kernel for the five outputs
        state["i"] += 1

    # ---- device-resident timing -------------------------------------------------------
    use_graph = not args.no_graph
    # one replay = N_WEIGHT_COPIES steps (every rotation of the weight copies)
    reps = max(1, -(-args.steps // N_WEIGHT_COPIES))
    wreps = max(1, -(-args.warmup // N_WEIGHT_COPIES))

    def timed(step_fn):
        """(ms per `args.steps` steps for each batch, the graph or None, steps actually run per batch).
        Legs made of this library's kernels only are captured once and replayed at every N (the fused
        path keeps its tile totals on the device, so nothing in a launch changes between replays)."""
        with torch.cuda.stream(stream):
            for _ in range(3):
                step_fn()
            torch.cuda.synchronize()
            if not use_graph:
                return time_batches(step_fn, args.steps, args.warmup, world, stream), None, args.steps
            barrier_sync(world)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                for _ in range(N_WEIGHT_COPIES):
                    step_fn()
        ran = reps * N_WEIGHT_COPIES
        return [ms * args.steps / ran for ms in time_batches(None, reps, wreps, world, stream, graph=g)], g, ran

    sampler = ClockSampler(local) if rank == 0 else None
    batches_local, graph, ran_steps = timed(step_local)
    launches = N_BATCHES * ran_steps * len(cases)
    ms_local = statistics.median(batches_local)
    batches_full, batches_nccl, batches_chained = batches_local, None, None
    gather_kind = "none (single GPU)"
    push_checked = None
    if world > 1:
        batches_nccl = time_batches(step_gather, args.steps, args.warmup, world, stream)
        batches_full, gather_kind = batches_nccl, "NCCL all_gather_into_tensor + [g,M,N/g]->[M,N] copy per call"
        if not args.no_push:
            try:
                import torch.distributed as dist

                # the fused path against the NCCL path on the same inputs, bit for bit, before anything is timed
                with torch.cuda.stream(stream):
                    for slot in range(4):  # collective: allocates and exchanges the symmetric outputs
                        push_set(slot)
                    got = []
                    i0 = state["i"]
                    step_push(sink=got)
                    torch.cuda.synchronize()
                    ok = True
                    for ci, res, _ in got:
                        want = layers[(i0 + ci) % N_WEIGHT_COPIES].forward(xs[ci])
                        if cases[ci].M > 2:
                            ok = ok and bool(torch.equal(res.view(torch.int16), want.view(torch.int16)))
                        else:  # the unfused path runs the row-split GEMV kernel there: another summation order
                            ok = ok and float((res.float() - want.float()).abs().max()) <= 2e-2
                    ok = ok and fg.workspace_status(local) == 0
                    t = torch.tensor([1 if ok else 0], device=dev)
                    dist.all_reduce(t, op=dist.ReduceOp.MIN)
                    push_checked = bool(t.item())
                    torch.cuda.synchronize()
                batches_full, graph_push, ran_steps = timed(step_push)
                launches = N_BATCHES * ran_steps * (len(cases) + 1)  # five compute kernels and one wait kernel
                gather_kind = ("fused: the epilogue stores every tile into every rank's C over NVLink; bounded waits on the "
                               "arrival counters close the step")
                batches_chained, graph_chained, _ = timed(lambda: step_push(chained=True))
                with torch.cuda.stream(stream):
                    torch.cuda.synchronize()
                    ok = fg.workspace_status(local) == 0  # no wait of the replayed steps gave up
                    t = torch.tensor([1 if ok else 0], device=dev)
                    dist.all_reduce(t, op=dist.ReduceOp.MIN)
                    push_checked = push_checked and bool(t.item())
                    torch.cuda.synchronize()
            except Exception as e:  # symmetric memory unavailable: keep the NCCL number
                sys.stderr.write(f"rank {rank}: fused all-gather unavailable ({e}); reporting the NCCL path\n")
    ms_full = statistics.median(batches_full)
    if world == 1:
        hold_load(graph.replay if graph is not None else step_local, stream)
    clocks = sampler.stop() if sampler else None
    if clocks is not None and world == 1:
        clocks["window"] = "the timed region and 0.5 s more of the same step, replayed untimed"

    # per-M device time (graph of 20 calls on rotating copies), for the breakdown
    per_call = {}
    if world == 1:
        for ci, c in enumerate(cases):
            def calls():
                for r in range(20):
                    layers[r % N_WEIGHT_COPIES].forward_local(xs[ci])

            t = us_per_call(calls, 20, stream, reps=3, warm_reps=1)
            plan = fg_plan_name(c.M)
            per_call[f"M{c.M}"] = {"us": round(t["us"], 2), "us_min": round(t["us_min"], 2), "us_max": round(t["us_max"], 2),
                                   "GBps": round(c.algorithmic_bytes / t["us"] / 1e3, 1), "kernel": plan}

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
            ms_g = statistics.median(time_batches(grp.run, 10, 3, 1, stream)) / 10 / N_WEIGHT_COPIES  # per step of five calls
            grouped = {"value": bytes_step_rank / ms_g / 1e6, "unit": "GB/s", "ms_per_step": ms_g,
                       "note": "20 calls as one grouped launch (fg_group_run); not the headline: one launch per call is"}
            del grp, g_cs
        except Exception as e:
            sys.stderr.write(f"grouped launch unavailable ({e})\n")

    # ---- end to end through the operator, host activations in, host result out -----------
    e2e = None
    if not args.no_e2e:
        use_push = world > 1 and gather_kind.startswith("fused")
        rows = [0]
        for c in cases:
            rows.append(rows[-1] + c.M)
        n_cols = cases[0].N * world
        # the step's five activations travel as one pinned block, the five results come back as one block
        x_all_host = torch.cat(xs_host).pin_memory()

        def compute_e2e(x_dev, out_dev, k):
            if world == 1:
                for ci in range(len(cases)):
                    fg.edgemm_m8n128k64x4_bt(x_dev[rows[ci]:rows[ci + 1]], weights[(state["i"] + ci) % N_WEIGHT_COPIES],
                                             out_dev[rows[ci]:rows[ci + 1]])
                state["i"] += 1
            elif use_push:
                # Three sets of push buffers in rotation: a set is pushed into again three steps later, and
                # no rank can get there before every rank's host has seen the results of the step that used
                # it last (the waits that close a step need all ranks' tiles of that step, and a host
                # issues step k+2 only after it holds step k's results).
                if e2e_graphs:
                    e2e_graphs[k % len(e2e_graphs)].replay()
                else:
                    push_step_e2e(x_dev, out_dev, k)
            else:
                for ci in range(len(cases)):
                    res = layers[(state["i"] + ci) % N_WEIGHT_COPIES].forward(x_dev[rows[ci]:rows[ci + 1]])
                    out_dev[rows[ci]:rows[ci + 1]].copy_(res)
                state["i"] += 1

        def push_step_e2e(x_dev, out_dev, k):
            state["i"] = k
            got = []
            step_push(slot=1 + k % 3, inputs=[x_dev[rows[ci]:rows[ci + 1]] for ci in range(len(cases))], sink=got)
            for ci, res, _ in got:
                out_dev[rows[ci]:rows[ci + 1]].copy_(res)

        e2e_graphs = []

        def prepare_e2e(x_devs, out_devs):
            # The fused path's step (five pushing calls, five waits, five copies into the result block) is
            # captured once per combination of input block (2), push-buffer set (3) and weight copy (4):
            # twelve graphs, replayed in turn.
            if not (use_push and use_graph):
                return
            with torch.cuda.stream(stream):
                for key in range(12):
                    push_step_e2e(x_devs[key & 1], out_devs[key & 1], key)
                torch.cuda.synchronize()
                barrier_sync(world)
                for key in range(12):
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream, capture_error_mode="thread_local"):
                        push_step_e2e(x_devs[key & 1], out_devs[key & 1], key)
                    e2e_graphs.append(g)

        ms_e2e = pipelined_e2e(compute_e2e, x_all_host, rows[-1], n_cols, dev, stream, args.steps,
                               args.warmup if world == 1 else max(3, args.warmup), world, prepare=prepare_e2e)
        e2e = {"value": bytes_step_rank * world / (ms_e2e / args.steps) / 1e6, "unit": "GB/s",
               "ms_per_step": ms_e2e / args.steps,
               "how": "two steps in flight: copies on side streams, the host waits for step k-1 while step k runs"
                      + ("; every rank copies in the step's activations and copies out the full assembled outputs" if world > 1 else "")
                      + ("; a step's calls are replayed from a graph captured over the operator calls" if e2e_graphs else ""),
               "h2d_bytes_per_step": x_all_host.numel() * 2,
               "d2h_bytes_per_step": rows[-1] * n_cols * 2}

    # ---- config 5 N-sharded, and the other single-GPU configs -----------------------------
    dit = None
    configs = None
    if not args.no_extras:
        if world > 1:
            dit = dit_sharded(args, world, rank, local, dev, stream)
        else:
            peak0, _ = measured_peak()
            configs = other_configs(dev, stream, peak0, args.layers)

    if rank != 0:
        return None
    peak, peak_kind = measured_peak()
    ms_step = ms_full / args.steps
    ms_step_local = ms_local / args.steps
    avg_launch_s = ms_step_local / 1e3 / len(cases)
    avg_bytes = bytes_step_rank / len(cases)
    achieved = avg_bytes / avg_launch_s / 1e9
    roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "peak_kind": f"of {peak_kind}", "frac_of_8000": achieved / 8000.0,
            "traffic": NCU_TRAFFIC["bytes_per_launch"], "traffic_kernel": NCU_TRAFFIC["kernel"],
            "kernel": "fg::fg_umma_kernel<1,16> (M = 2, 4, 8, 16) and fg::fg_gemv_kernel<1,2> (M = 1): average over the step's five launches",
            "algorithmic_bytes_per_launch": avg_bytes}
    if per_call:
        umma = [c for c in cases if "fg_umma" in per_call[f"M{c.M}"]["kernel"]]
        t_umma = sum(per_call[f"M{c.M}"]["us"] for c in umma) / len(umma)
        b_umma = sum(c.algorithmic_bytes for c in umma) / len(umma)
        roof["dominant_kernel"] = {"kernel": "fg::fg_umma_kernel<1,16>", "us_per_launch": t_umma, "achieved": b_umma / t_umma / 1e3,
                                   "frac": b_umma / t_umma / 1e3 / peak}
    line = {
        "metric": METRIC, "value": bytes_step_rank * world / ms_step / 1e6, "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "calls_per_step": len(cases),
                   "l2": f"{N_WEIGHT_COPIES} rotating weight copies (537 MB) > 126 MB L2",
                   "launch": ("cuda graph replay" if graph is not None else "stream launches")
                             + ("; the NCCL leg is launched call by call" if world > 1 else ""),
                   "sharding": f"N-sharded, {world} x 8192 columns; gather: {gather_kind}" if world > 1 else "single GPU"},
        "batches": {"what": f"{N_BATCHES} timed regions of {args.steps} steps each; value is their median",
                    "ms_per_step": [round(b / args.steps, 6) for b in batches_full]},
        "us_per_call": ms_step * 1e3 / len(cases),
        "per_call": per_call,
        "no_gather": {"value": bytes_step_rank * world / ms_step_local / 1e6, "unit": "GB/s", "ms_per_step": ms_step_local},
        "nccl_gather": None if batches_nccl is None else {
            "value": bytes_step_rank * world / (statistics.median(batches_nccl) / args.steps) / 1e6, "unit": "GB/s",
            "ms_per_step": statistics.median(batches_nccl) / args.steps},
        "roofline": roof,
        "clocks": clocks, "gpu_launches": int(launches), "e2e": e2e, "grouped": grouped,
    }
    if world > 1:
        line["push_checked"] = push_checked
        if batches_chained is not None:
            ms_c = statistics.median(batches_chained) / args.steps
            line["push_chained"] = {"value": bytes_step_rank * world / ms_c / 1e6, "unit": "GB/s", "ms_per_step": ms_c,
                                    "what": "the five calls tied like dependent layers: each reads its activations only after "
                                            "every rank's tiles of the previous call have arrived (in-kernel wait)"}
    if configs is not None:
        line["configs"] = configs
    if dit is not None:
        line["dit"] = dit
    if not args.no_cpu_baseline and world == 1:
        line["cpu_baseline"] = cpu_baseline_leg(cases)
    return line


def fg_plan_name(M: int) -> str:
    from fastgate_b200 import capi

    p = capi.plan(capi.FG_OP_F16_NK, M, 8192, 8192)
    return {4: f"fg::fg_gemv_kernel<{M},2>", 2: f"fg::fg_umma_kernel<1,{p.m_tile}>", 0: f"fg::fg_streamk_kernel<1,{p.m_tile}>"}[p.math]


def run_other_workload(args):
    """One of configs 1, 3, 4, the int4 sibling (single GPU) or 5 (the DiT stack, N-sharded) alone."""
    import torch

    import fastgate_b200 as fg
    from fastgate_b200 import workloads as wl

    world, rank, local = dist_setup(args)
    dev = torch.device("cuda", local)
    stream = torch.cuda.Stream(device=dev)
    peak, peak_kind = measured_peak()
    name = args.workload
    if name == "dit":
        sampler = ClockSampler(local) if rank == 0 else None
        if world == 1:
            res = {k: v for k, v in other_configs(dev, stream, peak, args.layers).items() if k.startswith("cfg5")}
        else:
            res = dit_sharded(args, world, rank, local, dev, stream)
        clocks = sampler.stop() if sampler else None
        if rank != 0:
            return None
        cases_all = wl.cfg5(args.layers)
        bytes_pass = sum(c.algorithmic_bytes for c in cases_all)
        if world == 1:
            best = res.get("cfg5_grouped") or res.get("cfg5_per_linear")
            ms_pass = best["ms_per_pass"]
        else:
            best = next((res[k] for k in ("push_grouped", "push_per_linear", "nccl_gather") if "ms_per_pass" in res.get(k, {})), None)
            ms_pass = best["ms_per_pass"]
        return {"metric": "effective HBM GB/s of the DiT linear stack (M=16 fp16 GEMM, N-sharded)", "value": bytes_pass / ms_pass / 1e6,
                "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_pass,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16 (fp32 accumulate)",
                "data": "synthetic", "config": {"workload": f"dit: {args.layers} layers, M=16, fp16, weights NxK"},
                "legs": res, "clocks": clocks, "e2e": None, "gpu_launches": None,
                "roofline": {"bound": "hbm", "achieved": bytes_pass / world / ms_pass / 1e6, "peak": peak, "unit": "GB/s",
                             "frac": bytes_pass / world / ms_pass / 1e6 / peak, "peak_kind": f"of {peak_kind}", "traffic": None}}
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

    sampler = ClockSampler(local)
    reps = max(1, -(-args.steps // n_rot_all))
    g = graph_of(step, stream, not args.no_graph)
    ms_b = time_batches(step, reps, max(1, -(-args.warmup // n_rot_all)), 1, stream, graph=g)
    hold_load(step_once, stream)
    clocks = sampler.stop()
    clocks["window"] = "the timed region and 0.5 s more of the same calls, untimed"
    steps_done = reps * n_rot_all
    ms_step = statistics.median(ms_b) / steps_done
    bytes_step = sum(c.algorithmic_bytes for c in cases)
    workload = {"cfg1": "edgemm_m8n128k64x4: M=8, K=N=4096, weight KxN fp16",
                "cfg3": "fastgemv: M=1, weight 11008x4096 and 4096x11008 fp16 (NxK)",
                "cfg4": "fastgemv_int8: M in {1,8}, weight int8 28672x8192 + fp16 scale per output channel",
                "w4": "fastgemv_int4: M in {1,8,16}, weight 28672x8192 packed 4-bit + fp16 scale per 128 k"}[name]
    achieved = bytes_step / ms_step / 1e6
    return {
        "metric": "effective HBM GB/s of M<=16 fp16/int8 GEMM-GEMV", "value": achieved, "unit": "GB/s", "n_gpus": 1,
        "steps": steps_done, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None,
        "dtype": {"cfg4": "int8 weights, f16 activations (fp32 accumulate)",
                  "w4": "int4 weights, f16 activations (fp32 accumulate)"}.get(name, "f16 (fp32 accumulate)"),
        "data": "synthetic",
        "config": {"workload": workload, "calls_per_step": len(cases), "sharding": "single GPU",
                   "l2": "weights rotate over more than 600 MB", "launch": "cuda graph replay" if g is not None else "stream launches"},
        "batches": {"ms_per_step": [round(b / steps_done, 6) for b in ms_b]},
        "us_per_call": ms_step * 1e3 / len(cases),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "peak_kind": f"of {peak_kind}", "frac_of_8000": achieved / 8000.0, "traffic": None},
        "clocks": clocks, "gpu_launches": int(N_BATCHES * steps_done * len(cases)), "e2e": None,
    }


def run_reference(args):
    """The reference's own implementation of the path: its kernels rebuilt for sm_100a when
    available (and a GPU is present), else the CPU oracle port on the host cores.  Nothing of the
    fastgate_b200 package is imported here: only the reference build under oracle/_ref runs."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return None
    wl = load_workloads()

    cases = wl.cfg2()
    bytes_step = sum(c.algorithmic_bytes for c in cases)
    # the CPU leg only where it has the host's cores to itself (a torchrun launch pins OpenMP to one thread)
    cpu = cpu_baseline_leg(cases) if world == 1 else None
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
        "impl": "reference", "metric": METRIC, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
        "config": {"workload": WORKLOAD, "calls_per_step": len(cases)},
    }
    if cpu is not None:
        base["cpu_baseline"] = cpu
    if ref is None:
        if cpu is None:
            cpu = cpu_baseline_leg(cases)
            base["cpu_baseline"] = cpu
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
    ms_b = time_batches(step, args.steps, args.warmup, 1, stream)
    ms = statistics.median(ms_b)
    hold_load(step, stream)
    clocks = sampler.stop()
    clocks["window"] = "the timed region and 0.5 s more of the same step, untimed"

    def compute_e2e(x_dev, out_dev, k):  # same shape as our arm: one block in, five operator calls, one block out
        for ci in range(len(cases)):
            ref.edgemm_m8n128k64x4_bt(x_dev[rows[ci]:rows[ci + 1]], weights[(state["i"] + ci) % N_WEIGHT_COPIES],
                                      out_dev[rows[ci]:rows[ci + 1]])
        state["i"] += 1

    ms_e2e = pipelined_e2e(compute_e2e, x_all_host, rows[-1], cases[0].N, dev, stream, args.steps, args.warmup)
    base.update({
        "value": bytes_step / (ms / args.steps) / 1e6, "ms_per_step": ms / args.steps,
        "batches": {"ms_per_step": [round(b / args.steps, 6) for b in ms_b]},
        "dtype": "f16 (fp16 accumulate)", "clocks": clocks,
        "reference_kind": "reference kernels (hk/edgemm.cu:274-324) rebuilt unmodified for sm_100a, same B200",
        "e2e": {"value": bytes_step / (ms_e2e / args.steps) / 1e6, "unit": "GB/s", "ms_per_step": ms_e2e / args.steps,
                "how": "two steps in flight: copies on side streams, the host waits for step k-1 while step k runs",
                "h2d_bytes_per_step": x_all_host.numel() * 2,
                "d2h_bytes_per_step": rows[-1] * cases[0].N * 2},
    })
    if not args.no_extras:
        base["configs"] = reference_other_configs(ref, wl, dev, stream)
    del weights
    return base


def reference_other_configs(ref, wl, dev, stream) -> dict:
    """The reference's own operators on configs 1, 3a, 3b and 4 (M = 1; its int8 GEMV takes one row
    and no scales), stream-launched on its default stream over rotating weight copies, including
    the C.zero_() its split-K kernels need (hk/edgemm.cu:138-142; the GEMV ops overwrite)."""
    import torch

    out = {}
    todo = [("cfg1", wl.cfg1()[0], "edgemm_m8n128k64x4 (hk/edgemm.cu:102)"),
            ("cfg3a", wl.cfg3()[0], "fastgemv (hk/fastgemv.cu:12)"), ("cfg3b", wl.cfg3()[1], "fastgemv (hk/fastgemv.cu:12)"),
            ("cfg4_M1", wl.cfg4()[0], "fastgemv_int8 (hk/fastgemv.cu:35), no scales")]
    for key, c, what in todo:
        try:
            n_rot = max(2, -(-600 * 2 ** 20 // c.weight_bytes))
            w0 = wl.make_weight(c).to(dev)
            ws = [w0] + [w0.clone() for _ in range(n_rot - 1)]
            x = wl.make_activation(c).to(dev)
            C = torch.zeros(c.M, c.N, dtype=torch.float16, device=dev)

            def step():
                for w in ws:
                    if c.op == wl.OP_KN:
                        ref.edgemm_m8n128k64x4(x, w, C)
                    elif c.op == wl.OP_NK:
                        ref.fastgemv(w, x, C)
                    else:
                        ref.fastgemv_int8(w, x, C)

            ms = time_batches(step, 4, 2, 1, stream)
            s = spread(ms, 4 * n_rot)
            out[key] = {"us_per_call": round(s["median"] * 1e3, 3), "us_min": round(s["min"] * 1e3, 3), "us_max": round(s["max"] * 1e3, 3),
                        "GBps": round(c.algorithmic_bytes / s["median"] / 1e6, 1), "what": what}
            del ws, w0
        except Exception as e:
            out[key] = {"unavailable": str(e)}
    return out


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
