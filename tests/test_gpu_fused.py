"""Fused epilogue: C = act(x . W^T * scales + bias) + residual, against the CPU oracle."""
import numpy as np
import pytest
import torch

import fastgate_b200 as fg
from fastgate_b200 import workloads as wl
from oracle import oracle

pytestmark = pytest.mark.gpu
ACTS = {"none": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3}


@pytest.mark.parametrize("act", list(ACTS))
@pytest.mark.parametrize("M,layout", [(1, "nk"), (8, "kn"), (16, "nk"), (16, "kn"), (21, "nk")])
def test_fp16_fused(act, M, layout):
    dev = torch.device("cuda:0")
    N, K = 1152, 2304
    case = wl.Case("f", wl.OP_NK, M, N, K, 40 + M)
    x, W = wl.make_activation(case), wl.make_weight(case)
    g = torch.Generator().manual_seed(M)
    bias = torch.randn(N, generator=g).half()
    res = torch.randn(M, N, generator=g).half()
    ref = oracle.epilogue(oracle.gemm_nk(x.numpy(), W.numpy()), bias.numpy(), res.numpy(), ACTS[act])
    Wd = (W if layout == "nk" else W.t().contiguous()).to(dev)
    C = torch.full((M, N), float("nan"), dtype=torch.half, device=dev)
    fg.linear_fused(x.to(dev), Wd, C, bias=bias.to(dev), residual=res.to(dev), act=act, layout=layout)
    oracle.check_tolerance(C.cpu().numpy(), ref, f"{act} M={M} {layout}")
    # each piece on its own
    C2 = torch.zeros_like(C)
    fg.linear_fused(x.to(dev), Wd, C2, bias=bias.to(dev), layout=layout)
    oracle.check_tolerance(C2.cpu().numpy(), oracle.epilogue(oracle.gemm_nk(x.numpy(), W.numpy()), bias.numpy()), "bias only")
    # no epilogue at all equals the plain operator bit for bit
    C3, C4 = torch.zeros_like(C), torch.zeros_like(C)
    fg.linear_fused(x.to(dev), Wd, C3, layout=layout)
    (fg.edgemm_m8n128k64x4_bt if layout == "nk" else fg.edgemm_m8n128k64x4)(x.to(dev), Wd, C4)
    assert torch.equal(C3.view(torch.int16), C4.view(torch.int16))


def test_int8_fused_in_place_residual():
    dev = torch.device("cuda:0")
    case = wl.Case("f8", wl.OP_W8, 8, 1024, 2048, 9)
    x, W8, s = wl.make_activation(case), wl.make_weight(case), wl.make_scales(case)
    g = torch.Generator().manual_seed(1)
    bias = torch.randn(1024, generator=g).half()
    h = torch.randn(8, 1024, generator=g).half()
    ref = oracle.epilogue(oracle.gemm_w8a16_nk(x.numpy(), W8.numpy(), s.numpy()), bias.numpy(), h.numpy(), 3)
    C = h.clone().to(dev)  # residual stream updated in place: C = silu(x W^T s + b) + C
    fg.linear_fused(x.to(dev), W8.to(dev), C, scales=s.to(dev), bias=bias.to(dev), residual=C, act="silu")
    oracle.check_tolerance(C.cpu().numpy(), ref, "int8 fused")


def test_fused_argument_checks():
    dev = torch.device("cuda:0")
    x = torch.zeros(4, 128, dtype=torch.half, device=dev)
    W = torch.zeros(128, 128, dtype=torch.half, device=dev)
    C = torch.zeros(4, 128, dtype=torch.half, device=dev)
    with pytest.raises(ValueError):
        fg.linear_fused(x, W, C, act="relu6")
    with pytest.raises(RuntimeError, match="bias must hold N"):
        fg.linear_fused(x, W, C, bias=torch.zeros(64, dtype=torch.half, device=dev))
    with pytest.raises(RuntimeError, match="scales only apply"):
        fg.linear_fused(x, W, C, scales=torch.zeros(128, dtype=torch.half, device=dev))
