"""More than 16 token rows: up to 64 rows ride along with one pass over an fp16 weight
(tcgen05 kernel with 32 or 64 accumulator columns); beyond that, passes of 64."""
import numpy as np
import pytest
import torch

import fastgate_b200 as fg
from fastgate_b200 import capi, workloads as wl
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "needs a B200"
    return torch.device("cuda:0")


@pytest.mark.parametrize("layout", ["nk", "kn"])
@pytest.mark.parametrize("M", [17, 24, 32, 33, 48, 64, 65, 100, 130])
@pytest.mark.parametrize("N,K", [(1152, 2304), (4096, 4096), (128, 128)])
def test_parity(M, N, K, layout, dev):
    case = wl.Case("tall", wl.OP_NK, M, N, K, 600 + M)
    x, W = wl.make_activation(case), wl.make_weight(case)
    ref = oracle.gemm_nk(x.numpy(), W.numpy())
    C = torch.full((M, N), float("nan"), dtype=torch.half, device=dev)
    if layout == "nk":
        fg.edgemm_m8n128k64x4_bt(x.to(dev), W.to(dev), C)
    else:
        fg.edgemm_m8n128k64x4(x.to(dev), W.t().contiguous().to(dev), C)
    oracle.check_tolerance(C.cpu().numpy(), ref, f"M={M} N={N} K={K} {layout}")


def test_plan_takes_one_pass_up_to_64_rows():
    for M, tile, passes in [(16, 16, 1), (17, 32, 1), (32, 32, 1), (33, 64, 1), (64, 64, 1), (65, 64, 2), (200, 64, 4)]:
        p = capi.plan(capi.FG_OP_F16_NK, M, 8192, 8192, 148, 232448)
        assert (p.m_tile, p.passes, p.math) == (tile, passes, 2), (M, p.as_dict())
    # quantized weights stay at 16 rows per pass
    p = capi.plan(capi.FG_OP_W8A16_NK, 40, 4096, 4096, 148, 232448)
    assert (p.m_tile, p.passes) == (16, 3)


def test_rows_do_not_depend_on_their_neighbours(dev):
    """Row m of a 64-row call equals the same row computed in a 16-row call within one rounding
    step (different tile heights cut the fp32 sums differently), and twice the same call is bitwise equal."""
    case = wl.Case("tall", wl.OP_NK, 64, 2048, 4096, 77)
    x, W = wl.make_activation(case).to(dev), wl.make_weight(case).to(dev)
    C64 = torch.zeros(64, 2048, dtype=torch.half, device=dev)
    again = torch.zeros_like(C64)
    fg.edgemm_m8n128k64x4_bt(x, W, C64)
    fg.edgemm_m8n128k64x4_bt(x, W, again)
    assert torch.equal(C64.view(torch.int16), again.view(torch.int16))
    for m0 in (0, 16, 48):
        C16 = torch.zeros(16, 2048, dtype=torch.half, device=dev)
        fg.edgemm_m8n128k64x4_bt(x[m0:m0 + 16].contiguous(), W, C16)
        assert oracle.tolerance_excess(C64[m0:m0 + 16].cpu().numpy(), C16.float().cpu().numpy()) <= 0.1


def test_fused_epilogue_on_a_tall_call(dev):
    M, N, K = 40, 1152, 2304
    case = wl.Case("tall", wl.OP_NK, M, N, K, 88)
    x, W = wl.make_activation(case), wl.make_weight(case)
    g = torch.Generator().manual_seed(2)
    bias, res = torch.randn(N, generator=g).half(), torch.randn(M, N, generator=g).half()
    ref = oracle.epilogue(oracle.gemm_nk(x.numpy(), W.numpy()), bias.numpy(), res.numpy(), 3)
    C = torch.zeros(M, N, dtype=torch.half, device=dev)
    fg.linear_fused(x.to(dev), W.to(dev), C, bias=bias.to(dev), residual=res.to(dev), act="silu")
    oracle.check_tolerance(C.cpu().numpy(), ref, "tall fused")
