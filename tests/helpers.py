"""Shared helpers of the test-suite: seeded inputs and the CPU oracle (test-only)."""
from __future__ import annotations

import numpy as np
import torch

from fastgate_b200 import workloads as wl
from oracle import oracle


def np16(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().contiguous().numpy()


def oracle_ref32(case: wl.Case, x: torch.Tensor, W: torch.Tensor, scales) -> np.ndarray:
    """fp32-accumulated reference C32[M,N] of `case` on CPU tensors."""
    if case.op == wl.OP_KN:
        return oracle.gemm_kn(np16(x), np16(W))
    if case.op == wl.OP_NK:
        return oracle.gemm_nk(np16(x), np16(W))
    return oracle.gemm_w8a16_nk(np16(x), np16(W), None if scales is None else np16(scales))


def inputs(case: wl.Case):
    return wl.make_activation(case), wl.make_weight(case), wl.make_scales(case)
