"""Front end of the built-in tracer: per-CTA timeline of one launch.

    python -m fastgate_b200.trace --op nk --M 16 --N 8192 --K 8192 [--pdl 0]

Prints, relative to the earliest CTA start, the minimum / median / maximum over the CTAs of:
CTA start, first copy issued, first stage landed, last copy issued, end of the tensor-core
work of the last segment (warp 0 / all warps), end of the finisher warp.  Times come from
%globaltimer (a few hundred ns of granularity).
"""
from __future__ import annotations

import argparse
import ctypes

import numpy as np
import torch

from . import capi

OPS = {"kn": capi.FG_OP_F16_KN, "nk": capi.FG_OP_F16_NK, "w8": capi.FG_OP_W8A16_NK, "w4": capi.FG_OP_W4A16_NK}


def timeline(op: int, M: int, N: int, K: int, pdl: int = 0, copies: int = 3, math: int = -1, chunks: int = 0,
             stages: int = 0):
    dev = torch.device("cuda", torch.cuda.current_device())
    L = capi.lib
    ws_bytes = capi.workspace_bytes(N)
    ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    x = torch.randn(M, K, device=dev).half()
    if op == capi.FG_OP_W8A16_NK:
        Ws = [torch.randint(-127, 128, (N, K), dtype=torch.int8, device=dev) for _ in range(copies)]
    elif op == capi.FG_OP_W4A16_NK:
        Ws = [torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev) for _ in range(copies)]
    elif op == capi.FG_OP_F16_KN:
        Ws = [(torch.randn(K, N, device=dev) / K ** 0.5).half() for _ in range(copies)]
    else:
        Ws = [(torch.randn(N, K, device=dev) / K ** 0.5).half() for _ in range(copies)]
    C = torch.zeros(M, N, dtype=torch.half, device=dev)
    props = torch.cuda.get_device_properties(dev)
    p = capi.plan(op, M, N, K, props.multi_processor_count, 0)
    p.pdl = pdl
    if math == 2 or (math == -1 and p.math == 2 and (chunks or stages)):
        ck = chunks or p.k_per_stage // 64
        p.math, p.m_tile, p.consumer_warps = 2, 16, 4
        p.k_per_stage = ck * 64
        p.k_blocks = -(-K // p.k_per_stage)
        p.grid = min(props.multi_processor_count, p.tiles * p.k_blocks)
        p.stages = stages or min(24, (232448 - 1024 - 64) // (ck * 18432 + 16))
        p.smem_bytes = 1024 + p.stages * (ck * 18432 + 16) + 64

    def run(W):
        st = L.fg_gemm_planned(ctypes.byref(p), x.data_ptr(), W.data_ptr(), None, C.data_ptr(), M, N, K,
                               ws.data_ptr(), ws_bytes, stream)
        assert st == capi.FG_OK, capi.status_str(st)

    for W in Ws[:-1]:
        run(W)
    torch.cuda.synchronize()
    buf = (ctypes.c_ulonglong * (16 * p.grid))()
    L.fg_trace_enable(1)
    try:
        assert L.fg_trace_read(ws.data_ptr(), buf, p.grid, stream) == capi.FG_OK  # clear
        run(Ws[-1])
        assert L.fg_trace_read(ws.data_ptr(), buf, p.grid, stream) == capi.FG_OK
    finally:
        L.fg_trace_enable(0)
    t = np.array(list(buf), dtype=np.float64).reshape(p.grid, 16)
    t[:, 5] = np.maximum(t[:, 5], t[:, 13])  # the later of the two finisher teams
    return p, t


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=sorted(OPS), default="nk")
    ap.add_argument("--M", type=int, default=16)
    ap.add_argument("--N", type=int, default=8192)
    ap.add_argument("--K", type=int, default=8192)
    ap.add_argument("--pdl", type=int, default=0)
    ap.add_argument("--math", type=int, default=-1, help="-1: the planner's choice; 0 mma.sync; 2 tcgen05")
    ap.add_argument("--chunks", type=int, default=0, help="weight chunks per stage (0: the planner's choice)")
    ap.add_argument("--stages", type=int, default=0)
    a = ap.parse_args()
    p, t = timeline(OPS[a.op], a.M, a.N, a.K, a.pdl, math=a.math, chunks=a.chunks, stages=a.stages)
    t0 = t[:, 0].min()
    print(f"op={a.op} M={a.M} N={a.N} K={a.K} plan={p.as_dict()}")
    print(f"stages per CTA {p.tiles * p.k_blocks / p.grid:.1f}; segments per CTA {int(t[:, 6].min())}..{int(t[:, 6].max())}")
    for col, lab in [(0, "CTA start"), (1, "first copy issued"), (3, "first stage landed"), (2, "last copy issued"),
                     (4, "warp 0 math done"), (7, "all warps math done"), (5, "finisher done")]:
        if t[:, col].max() <= 0:  # a stamp this kernel does not take
            continue
        v = (t[:, col] - t0) / 1e3
        print(f"  {lab:22s} min {v.min():7.2f}  med {np.median(v):7.2f}  max {v.max():7.2f} us")
    for col, lab in [(9, "math: waiting for a stage"), (10, "math: issuing"),
                     (11, "epilogue: waiting for an accumulator")]:
        v = t[:, col] / 1e3
        if v.max() > 0:
            print(f"  total {lab:38s} min {v.min():7.2f}  med {np.median(v):7.2f}  max {v.max():7.2f} us")


if __name__ == "__main__":
    main()
