"""Seeded random shapes through the C ABI against the CPU oracle.

The planner switches kernels and grids with the shape (row-split kernel for one or two rows,
tile-aligned grids for small problems, stream-K on all SMs otherwise, one to three passes for
M > 64): a sweep over shapes nobody picked by hand, every one with the checks of the parity tests
(status, no device-side timeout, canaries, tolerance, bit-identical second run)."""
import numpy as np
import pytest
import torch

from fastgate_b200 import capi, workloads as wl

from . import gpu_util as gu
from .test_gpu_parity import run_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a B200"
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def ws(dev):
    return gu.Workspace(dev)


def _cases():
    rng = np.random.default_rng(20240607)
    out = []
    for i in range(72):
        op = (wl.OP_NK, wl.OP_KN, wl.OP_W8)[i % 3]
        M = int(rng.choice([1, 2, 3, 4, 5, 7, 8, 9, 12, 16, 17, 20, 33, 64, 70], p=[.14, .1, .07, .07, .06, .06, .1, .05, .05, .1, .04, .04, .04, .04, .04]))
        if op == wl.OP_W8 and M > 40:
            M = 16
        N = 128 * int(rng.integers(1, 41))
        K = 128 * int(rng.integers(1, 49))
        out.append(wl.Case(f"fuzz{i}_op{op}_M{M}_N{N}_K{K}", op, M, N, K, 12000 + i))
    return out


@pytest.mark.parametrize("case", _cases(), ids=lambda c: c.name)
def test_random_shapes(case, dev, ws):
    p = capi.plan(case.op, case.M, case.N, case.K, 148, 232448)
    assert p.math in (0, 2, 4)
    run_case(case, dev, ws)


@pytest.mark.parametrize("M", [1, 3, 8])
@pytest.mark.parametrize("N,K", [(8192, 4096), (5120, 5120), (4096, 8192)])
def test_large_kn_weights_with_few_rows_run_the_tcgen05_kernel(M, N, K, dev, ws):
    """KxN weights above 40 MB leave the mma.sync kernel also for M <= 8 (rows beyond M are zero-filled)."""
    assert capi.plan(wl.OP_KN, M, N, K, 148, 232448).math == 2
    assert capi.plan(wl.OP_KN, M, 4096, 4096, 148, 232448).math == 0
    run_case(wl.Case(f"kn_large_M{M}_N{N}_K{K}", wl.OP_KN, M, N, K, 13000 + M + N), dev, ws)
