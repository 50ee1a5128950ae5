"""One-time weight repacks, the SiLU-gated pair of projections and the split (QKV) output.

None of these has a counterpart in the reference; they are checked against numpy restatements in
the CPU oracle module and against the plain operators of this library."""
import ctypes

import numpy as np
import pytest
import torch

import fastgate_b200 as fg
from fastgate_b200 import capi, workloads as wl
from oracle import oracle

from . import gpu_util as gu

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a B200"
    return torch.device("cuda:0")


@pytest.mark.parametrize("N,K", [(64, 64), (128, 4096), (4096, 4096), (1152, 2304), (11008, 4096)])
def test_prepack_kn_to_nk_is_the_transpose(N, K, dev):
    g = torch.Generator().manual_seed(N + K)
    B = torch.randn(K, N, generator=g).half()
    W = fg.prepack_kn_to_nk(B.to(dev))
    assert W.shape == (N, K)
    assert torch.equal(W.cpu(), B.t().contiguous())
    if N % 128 == 0 and K % 128 == 0:
        # the repacked weight through the NxK operator: same product as the KxN operator on the original
        x = torch.randn(8, K, generator=g).half().to(dev)
        a = torch.zeros(8, N, dtype=torch.half, device=dev)
        b = torch.zeros(8, N, dtype=torch.half, device=dev)
        fg.edgemm_m8n128k64x4(x, B.to(dev), a)
        fg.edgemm_m8n128k64x4_bt(x, W, b)
        ref = oracle.gemm_nk(x.cpu().numpy(), W.cpu().numpy())
        oracle.check_tolerance(a.cpu().numpy(), ref, "kn")
        oracle.check_tolerance(b.cpu().numpy(), ref, "nk on the repacked weight")


def test_prepack_argument_checks(dev):
    L = capi.lib
    x = torch.zeros(64, 64, dtype=torch.half, device=dev)
    assert L.fg_prepack_kn_to_nk(x.data_ptr(), x.data_ptr(), 60, 64, gu.stream()) == capi.FG_ERR_SHAPE
    assert L.fg_prepack_kn_to_nk(None, x.data_ptr(), 64, 64, gu.stream()) == capi.FG_ERR_NULL
    assert L.fg_prepack_gate_up(x.data_ptr(), x.data_ptr(), x.data_ptr(), 64, 64, gu.stream()) == capi.FG_ERR_SHAPE  # K % 128
    with pytest.raises(ValueError):
        fg.prepack_gate_up(torch.zeros(64, 128, dtype=torch.half, device=dev), torch.zeros(128, 128, dtype=torch.half, device=dev))


@pytest.mark.parametrize("Nh,K", [(64, 128), (128, 256), (3072, 1024)])
def test_prepack_gate_up_layout(Nh, K, dev):
    g = torch.Generator().manual_seed(Nh)
    Wg, Wu = torch.randn(Nh, K, generator=g).half(), torch.randn(Nh, K, generator=g).half()
    got = fg.prepack_gate_up(Wg.to(dev), Wu.to(dev))
    assert torch.equal(got.cpu(), torch.from_numpy(oracle.interleave_gate_up(Wg.numpy(), Wu.numpy())))


# one whole tile, a few tiles, the LLaMA-7B MLP (172 tiles on 148 CTAs: whole and split tiles), tall tiles, passes
@pytest.mark.parametrize("M,Nh,K", [(1, 64, 128), (16, 64, 128), (5, 512, 1024), (16, 11008, 4096), (2, 11008, 4096),
                                    (21, 1536, 3072), (40, 2048, 2048), (70, 512, 1024), (16, 1536, 12288)])
def test_silu_gate_matches_the_oracle(M, Nh, K, dev):
    g = torch.Generator().manual_seed(M + Nh + K)
    x = torch.randn(M, K, generator=g).half()
    Wg = (torch.randn(Nh, K, generator=g) / K ** 0.5).half()
    Wu = (torch.randn(Nh, K, generator=g) / K ** 0.5).half()
    bias = (torch.randn(2 * Nh, generator=g) * 0.1).half()        # in the order of the packed weight's rows
    res = torch.randn(M, Nh, generator=g).half()
    Wgu = fg.prepack_gate_up(Wg.to(dev), Wu.to(dev))
    b2 = bias.numpy().reshape(Nh // 64, 2, 64)
    ref = oracle.silu_gate(oracle.gemm_nk(x.numpy(), Wg.numpy()), oracle.gemm_nk(x.numpy(), Wu.numpy()),
                           b2[:, 0].reshape(-1), b2[:, 1].reshape(-1), res.numpy())
    C = torch.full((M, Nh), float("nan"), dtype=torch.half, device=dev)
    fg.linear_fused(x.to(dev), Wgu, C, bias=bias.to(dev), residual=res.to(dev), act="silu_gate")
    oracle.check_tolerance(C.cpu().numpy(), ref, f"silu_gate M={M} Nh={Nh} K={K}")
    # without bias and residual, twice: same bits
    ref0 = oracle.silu_gate(oracle.gemm_nk(x.numpy(), Wg.numpy()), oracle.gemm_nk(x.numpy(), Wu.numpy()))
    C0, C1 = torch.zeros_like(C), torch.zeros_like(C)
    fg.linear_fused(x.to(dev), Wgu, C0, act="silu_gate")
    fg.linear_fused(x.to(dev), Wgu, C1, act="silu_gate")
    oracle.check_tolerance(C0.cpu().numpy(), ref0, "plain gate")
    assert torch.equal(C0.view(torch.int16), C1.view(torch.int16))
    assert fg.workspace_status(0) == 0


def test_silu_gate_argument_checks(dev):
    x = torch.zeros(4, 128, dtype=torch.half, device=dev)
    W = torch.zeros(256, 128, dtype=torch.half, device=dev)
    with pytest.raises(RuntimeError):
        fg.linear_fused(x, W, torch.zeros(4, 256, dtype=torch.half, device=dev), act="silu_gate")     # output is [M, N/2]
    with pytest.raises(ValueError):
        fg.linear_fused(x, W.t().contiguous(), torch.zeros(4, 128, dtype=torch.half, device=dev), act="silu_gate", layout="kn")
    C = torch.zeros(4, 128, dtype=torch.half, device=dev)
    with pytest.raises(ValueError):
        fg.linear_fused(x, W, C, act="silu_gate", C2=C)


@pytest.mark.parametrize("layout,M", [("nk", 1), ("nk", 2), ("nk", 8), ("nk", 16), ("nk", 40), ("nk", 70), ("kn", 8), ("kn", 16), ("w8", 8), ("w8", 16)])
def test_split_output_equals_slices_of_the_whole(layout, M, dev):
    """QKV: one projection, three outputs; bitwise the column slices of the unsplit call."""
    N, K = 9216, 3072
    g = torch.Generator().manual_seed(M)
    x = torch.randn(M, K, generator=g).half().to(dev)
    scales = None
    if layout == "w8":
        W = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8).to(dev)
        scales = ((torch.rand(N, generator=g) + 0.5) / 127).half().to(dev)
    else:
        W = (torch.randn(N, K, generator=g) / K ** 0.5).half()
        W = (W if layout == "nk" else W.t().contiguous()).to(dev)
    bias = torch.randn(N, generator=g).half().to(dev)
    lay = "kn" if layout == "kn" else "nk"
    whole = torch.zeros(M, N, dtype=torch.half, device=dev)
    fg.linear_fused(x, W, whole, scales=scales, bias=bias, layout=lay)
    for n1, n2 in [(3072, 6144), (1024, 1152), (9088, 9216), (4608, 9216)]:
        q = torch.full((M, n1), float("nan"), dtype=torch.half, device=dev)
        k = torch.full((M, n2 - n1), float("nan"), dtype=torch.half, device=dev)
        v = torch.full((M, N - n2), float("nan"), dtype=torch.half, device=dev) if n2 < N else None
        fg.linear_fused(x, W, q, scales=scales, bias=bias, layout=lay, C2=k, C3=v)
        assert torch.equal(q.view(torch.int16), whole[:, :n1].contiguous().view(torch.int16)), (n1, n2)
        assert torch.equal(k.view(torch.int16), whole[:, n1:n2].contiguous().view(torch.int16)), (n1, n2)
        if v is not None:
            assert torch.equal(v.view(torch.int16), whole[:, n2:].contiguous().view(torch.int16)), (n1, n2)
    assert fg.workspace_status(0) == 0


def test_split_argument_checks(dev):
    x = torch.zeros(4, 128, dtype=torch.half, device=dev)
    W = torch.zeros(256, 128, dtype=torch.half, device=dev)
    a = torch.zeros(4, 128, dtype=torch.half, device=dev)
    b = torch.zeros(4, 64, dtype=torch.half, device=dev)
    with pytest.raises(RuntimeError, match="add up"):
        fg.linear_fused(x, W, a, C2=b)
    with pytest.raises(ValueError):
        fg.linear_fused(x, W, a, C3=b)
    L = capi.lib
    ws = gu.Workspace(dev)
    ep = capi.Epilogue(None, None, 0, 100, 256, b.data_ptr(), None)   # split1 not a multiple of 8
    assert L.fg_gemm_fused(capi.FG_OP_F16_NK, x.data_ptr(), W.data_ptr(), None, a.data_ptr(), 4, 256, 128, ctypes.byref(ep),
                           ws.ptr, ws.bytes, gu.stream()) == capi.FG_ERR_SHAPE
    ep = capi.Epilogue(None, None, 0, 128, 192, None, None)           # a middle part without a tensor
    assert L.fg_gemm_fused(capi.FG_OP_F16_NK, x.data_ptr(), W.data_ptr(), None, a.data_ptr(), 4, 256, 128, ctypes.byref(ep),
                           ws.ptr, ws.bytes, gu.stream()) == capi.FG_ERR_NULL
