"""The pybind operator surface on a B200: every reference name, its argument order, its
in-place output, its error message."""
import numpy as np
import pytest
import torch

import fastgate_b200 as fg
from fastgate_b200 import workloads as wl
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a B200"
    return torch.device("cuda:0")


def _data(M, N, K, seed, dev):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g).half()
    W = (torch.randn(N, K, generator=g) / K ** 0.5).half()
    ref = oracle.gemm_nk(x.numpy(), W.numpy())
    return x.to(dev), W.to(dev), ref


@pytest.mark.parametrize("name", fg.KN_OPS)
def test_kn_ops(name, dev):
    x, W, ref = _data(8, 1024, 2048, 1, dev)
    B = W.t().contiguous()
    C = torch.full((8, 1024), float("nan"), dtype=torch.half, device=dev)
    op = getattr(fg, name)
    ret = op(x, B, C, 4) if name in fg.BZ_OPS else op(x, B, C)
    assert ret is None
    oracle.check_tolerance(C.cpu().numpy(), ref, name)
    if name in fg.BZ_OPS:  # the split-K hint is optional and does not change the result
        C2 = torch.zeros_like(C)
        op(x, B, C2)
        assert torch.equal(C, C2)


@pytest.mark.parametrize("name", fg.NK_OPS)
def test_nk_ops(name, dev):
    x, W, ref = _data(8, 1024, 2048, 2, dev)
    C = torch.full((8, 1024), float("nan"), dtype=torch.half, device=dev)
    op = getattr(fg, name)
    op(x, W, C, 2) if name in fg.BZ_OPS else op(x, W, C)
    oracle.check_tolerance(C.cpu().numpy(), ref, name)


@pytest.mark.parametrize("name,M", [("fastgemv", 1), ("fastgemv_tuned", 1), ("fastgemm", 1), ("fastgemm", 2),
                                    ("fastgemv_extend", 8), ("fastgemv_extend", 5)])
def test_weight_first_ops(name, M, dev):
    x, W, ref = _data(M, 4096, 4096, 3, dev)
    C = torch.full((M, 4096), float("nan"), dtype=torch.half, device=dev)
    getattr(fg, name)(W, x, C)
    oracle.check_tolerance(C.cpu().numpy(), ref, name)
    if M == 1:  # the reference's scripts pass y as [N], [N,1] or [1,N]; all hold N elements
        y = torch.zeros(4096, dtype=torch.half, device=dev)
        getattr(fg, name)(W, x, y)
        assert torch.equal(y, C[0])


def test_fastgemv_int8_with_and_without_scales(dev):
    case = wl.Case("int8", wl.OP_W8, 8, 2048, 4096, 9)
    x, W8, s = wl.make_activation(case), wl.make_weight(case), wl.make_scales(case)
    C = torch.zeros(8, 2048, dtype=torch.half, device=dev)
    fg.fastgemv_int8(W8.to(dev), x.to(dev), C, s.to(dev))
    oracle.check_tolerance(C.cpu().numpy(), oracle.gemm_w8a16_nk(x.numpy(), W8.numpy(), s.numpy()), "scaled")
    y = torch.zeros(2048, dtype=torch.half, device=dev)
    fg.fastgemv_int8(W8.to(dev), x[:1].to(dev), y)  # the reference's 3-argument form
    oracle.check_tolerance(y.cpu().numpy()[None], oracle.gemm_w8a16_nk(x[:1].numpy(), W8.numpy(), None), "unscaled")


def test_contract_violation_raises_value_error(dev):
    x = torch.zeros(8, 192, dtype=torch.half, device=dev)
    with pytest.raises(ValueError, match="multiple of 128"):
        fg.edgemm_m8n128k64x4(x, torch.zeros(192, 128, dtype=torch.half, device=dev), torch.zeros(8, 128, dtype=torch.half, device=dev))
    with pytest.raises(ValueError, match="transposed output row"):
        fg.edgemm_m8n128k64x4_bt(x, torch.zeros(128, 192, dtype=torch.half, device=dev), torch.zeros(8, 128, dtype=torch.half, device=dev))
    xx = torch.zeros(8, 128, dtype=torch.half, device=dev)
    with pytest.raises(ValueError):
        fg.edgemm_m8n128k64x4(xx, torch.zeros(128, 100, dtype=torch.half, device=dev), torch.zeros(8, 100, dtype=torch.half, device=dev))


def test_type_and_shape_validation(dev):
    x = torch.zeros(8, 128, dtype=torch.half, device=dev)
    W = torch.zeros(128, 128, dtype=torch.half, device=dev)
    C = torch.zeros(8, 128, dtype=torch.half, device=dev)
    with pytest.raises(RuntimeError, match="dtype"):
        fg.edgemm_m8n128k64x4_bt(x.float(), W, C)
    with pytest.raises(RuntimeError, match="contiguous"):
        fg.edgemm_m8n128k64x4_bt(x, W.t(), C)
    with pytest.raises(RuntimeError, match="disagree on K"):
        fg.edgemm_m8n128k64x4_bt(x, torch.zeros(128, 256, dtype=torch.half, device=dev), C)
    with pytest.raises(RuntimeError, match="M\\*N"):
        fg.edgemm_m8n128k64x4_bt(x, W, torch.zeros(4, 128, dtype=torch.half, device=dev))
    with pytest.raises(RuntimeError, match="dtype"):
        fg.fastgemv_int8(W, x, C)  # int8 weight expected


def test_m_above_16_and_other_streams(dev):
    x, W, ref = _data(40, 1024, 1024, 5, dev)
    C = torch.zeros(40, 1024, dtype=torch.half, device=dev)
    fg.edgemm_m8n128k64x4_bt(x, W, C)
    oracle.check_tolerance(C.cpu().numpy(), ref, "M=40")
    s = torch.cuda.Stream()
    C2 = torch.zeros_like(C)
    with torch.cuda.stream(s):
        fg.edgemm_m8n128k64x4_bt(x, W, C2)
    s.synchronize()
    assert torch.equal(C, C2)


def test_cuda_graph_capture(dev):
    """The ops neither synchronise nor allocate once their workspace exists: a captured graph
    replays to the same bits."""
    x, W, ref = _data(16, 2048, 2048, 6, dev)
    C = torch.zeros(16, 2048, dtype=torch.half, device=dev)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        fg.edgemm_m8n128k64x4_bt(x, W, C)  # creates the stream's workspace
        torch.cuda.synchronize()
        eager = C.clone()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for _ in range(3):
                fg.edgemm_m8n128k64x4_bt(x, W, C)
        C.zero_()
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(C, eager)
    oracle.check_tolerance(C.cpu().numpy(), ref, "graph")


def test_comparators(dev):
    x, W, ref = _data(8, 512, 512, 7, dev)
    C = torch.zeros(8, 512, dtype=torch.half, device=dev)
    fg.hgemm_tr(x, W, C)
    oracle.check_tolerance(C.cpu().numpy(), ref, "hgemm_tr")
    fg.hgemm(x, W.t().contiguous(), C)
    oracle.check_tolerance(C.cpu().numpy(), ref, "hgemm")


def test_launches_are_counted(dev):
    x, W, _ = _data(8, 512, 512, 8, dev)
    C = torch.zeros(8, 512, dtype=torch.half, device=dev)
    n0 = fg.launch_count()
    fg.fastgemv_extend(W, x, C)
    fg.fastgemv_extend(W, torch.cat([x] * 3), torch.zeros(24, 512, dtype=torch.half, device=dev))  # 24 rows: one pass
    fg.fastgemv_extend(W, torch.cat([x] * 9), torch.zeros(72, 512, dtype=torch.half, device=dev))  # 72 rows: 64 + 8
    assert fg.launch_count() - n0 == 4
