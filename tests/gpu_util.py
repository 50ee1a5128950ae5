"""Helpers of the GPU tests: C-ABI calls on torch device buffers, canary-padded outputs."""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from fastgate_b200 import capi, workloads as wl

L = capi.lib
CANARY = 0x7BCD  # fp16 bit pattern written around every output buffer


class Workspace:
    def __init__(self, device, n_max: int = 65536):
        self.bytes = capi.workspace_bytes(n_max)
        self.buf = torch.empty(self.bytes, dtype=torch.uint8, device=device)
        st = L.fg_workspace_init(self.buf.data_ptr(), self.bytes, stream())
        assert st == capi.FG_OK, capi.status_str(st)

    @property
    def ptr(self):
        return self.buf.data_ptr()

    def status(self) -> int:
        v = ctypes.c_int(-1)
        st = L.fg_workspace_status(self.ptr, ctypes.byref(v), stream())
        assert st == capi.FG_OK, capi.status_str(st)
        return v.value


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class GuardedOut:
    """An M x N fp16 output with 4 KB of canary halves on both sides."""

    PAD = 2048

    def __init__(self, M: int, N: int, device):
        self.M, self.N = M, N
        self.raw = torch.full((self.PAD * 2 + M * N,), CANARY, dtype=torch.int16, device=device)
        self.out = self.raw[self.PAD:self.PAD + M * N].view(torch.float16).view(M, N)
        self.out.fill_(float("nan"))

    def check_canaries(self):
        assert bool((self.raw[:self.PAD] == CANARY).all()), "write before the output buffer"
        assert bool((self.raw[self.PAD + self.M * self.N:] == CANARY).all()), "write past the output buffer"


def call(case_op: int, x, W, scales, out, M, N, K, ws: Workspace, plan=None) -> int:
    sp = scales.data_ptr() if scales is not None else None
    if plan is not None:
        return L.fg_gemm_planned(ctypes.byref(plan), x.data_ptr(), W.data_ptr(), sp, out.data_ptr(), M, N, K,
                                 ws.ptr, ws.bytes, stream())
    if case_op == wl.OP_KN:
        return L.fg_gemm_f16_kn(x.data_ptr(), W.data_ptr(), out.data_ptr(), M, N, K, ws.ptr, ws.bytes, stream())
    if case_op == wl.OP_NK:
        return L.fg_gemm_f16_nk(x.data_ptr(), W.data_ptr(), out.data_ptr(), M, N, K, ws.ptr, ws.bytes, stream())
    return L.fg_gemm_w8a16_nk(x.data_ptr(), W.data_ptr(), sp, out.data_ptr(), M, N, K, ws.ptr, ws.bytes, stream())


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()
