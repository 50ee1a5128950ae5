"""int4 weight-only GEMV/GEMM (fg_gemm_w4a16_nk / fastgemv_int4) and its quantiser against the CPU oracle."""
import numpy as np
import pytest
import torch

import fastgate_b200 as fg
from fastgate_b200 import workloads as wl
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "needs a B200"
    return torch.device("cuda:0")


def _case(M, N, K, groups, seed):
    c = wl.Case("w4", wl.OP_W4, M, N, K, seed, groups)
    return wl.make_activation(c), wl.make_weight(c), wl.make_scales(c)


@pytest.mark.parametrize("grouped", [False, True])
@pytest.mark.parametrize("M", [1, 3, 8, 13, 16, 21])
@pytest.mark.parametrize("N,K", [(1152, 2304), (128, 128), (256, 384), (4096, 4096)])
def test_parity(M, N, K, grouped, dev):
    """Whole chunks (K % 256 == 0), a ragged last chunk (K = 384), less than one chunk (K = 128);
    tile heights 8 and 16, two passes (M = 21); one scale per channel and one per 128 k."""
    groups = K // 128 if grouped else 1
    x, W4, s = _case(M, N, K, groups, 70 + M)
    ref = oracle.gemm_w4a16_nk(x.numpy(), W4.numpy(), s.numpy(), 8)
    C = torch.full((M, N), float("nan"), dtype=torch.half, device=dev)
    fg.fastgemv_int4(W4.to(dev), x.to(dev), C, s.to(dev))
    oracle.check_tolerance(C.cpu().numpy(), ref, f"int4 M={M} N={N} K={K} groups={groups}")


@pytest.mark.parametrize("zp", [0, 5, 8, 15])
def test_zero_points_and_no_scales(zp, dev):
    x, W4, _ = _case(4, 512, 1024, 1, 90 + zp)
    x = (x / 16).half()  # keep the unscaled sums inside fp16
    ref = oracle.gemm_w4a16_nk(x.numpy(), W4.numpy(), None, zp)
    C = torch.zeros(4, 512, dtype=torch.half, device=dev)
    fg.fastgemv_int4(W4.to(dev), x.to(dev), C, None, zp)
    oracle.check_tolerance(C.cpu().numpy(), ref, f"zero point {zp}")


def test_exact_on_small_integers(dev):
    """Integer activations and weights, sums below 2048: every partial sum is exact in fp32 and
    the result in fp16, so any summation order must give the same bits as the oracle."""
    g = torch.Generator().manual_seed(3)
    N, K = 256, 512
    x = torch.randint(-1, 2, (8, K), generator=g).half()
    W4 = torch.randint(0, 256, (N, K // 2), generator=g, dtype=torch.uint8)
    ref = oracle.gemm_w4a16_nk(x.numpy(), W4.numpy(), None, 8)
    assert np.abs(ref).max() < 2048
    C = torch.zeros(8, N, dtype=torch.half, device=dev)
    fg.fastgemv_int4(W4.to(dev), x.to(dev), C)
    assert np.array_equal(C.cpu().numpy().astype(np.float32), ref)


def test_against_reference_kernel_restatement(dev):
    """M = 1 with the reference's scalar scale and zero point (gemv_quantized_int4,
    hk/fastgemv.cuh:394-495, restated order-exactly on the CPU): same values up to one rounding
    step, since only the summation order differs."""
    N, K = 1024, 4096
    x, W4, _ = _case(1, N, K, 1, 77)
    scale, zp = 0.0625, 8
    y_ref = oracle.gemv_int4_ref(W4.numpy(), x.numpy(), scale, float(zp))
    s = torch.full((N,), scale, dtype=torch.half)
    C = torch.zeros(1, N, dtype=torch.half, device=dev)
    fg.fastgemv_int4(W4.to(dev), x.to(dev), C, s.to(dev), zp)
    assert oracle.tolerance_excess(C.cpu().numpy(), y_ref.astype(np.float32)[None]) <= 0.1


@pytest.mark.parametrize("group_size", [128, 0])
def test_quantiser_matches_oracle_and_roundtrips(group_size, dev):
    N, K = 384, 1024
    g = torch.Generator().manual_seed(11)
    W = (torch.randn(N, K, generator=g) / 32).half()
    W[5] = 0  # an all-zero row: scale 1, every nibble 8
    W4, s = fg.quantize_int4(W.to(dev), group_size)
    groups = K // 128 if group_size else 1
    W4_ref, s_ref = oracle.quantize_rows_w4(W.numpy(), groups)
    assert np.array_equal(W4.cpu().numpy(), W4_ref)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), s_ref.view(np.uint16))
    # the quantised layer stays close to the fp16 one: error bounded by half a step per weight
    x = torch.randn(8, K, generator=g).half()
    C = torch.zeros(8, N, dtype=torch.half, device=dev)
    fg.fastgemv_int4(W4, x.to(dev), C, s)
    oracle.check_tolerance(C.cpu().numpy(), oracle.gemm_w4a16_nk(x.numpy(), W4_ref, s_ref, 8), "quantised layer")
    full = oracle.gemm_nk(x.numpy(), W.numpy())
    step = s_ref.astype(np.float32).max()
    assert np.abs(C.float().cpu().numpy() - full).max() < 0.5 * step * np.abs(x.float().numpy()).sum(axis=1).max()


def test_argument_checks(dev):
    x = torch.zeros(2, 256, dtype=torch.half, device=dev)
    W4 = torch.zeros(128, 128, dtype=torch.uint8, device=dev)
    C = torch.zeros(2, 128, dtype=torch.half, device=dev)
    fg.fastgemv_int4(W4, x, C)
    with pytest.raises(ValueError):
        fg.fastgemv_int4(W4, x, C, None, 16)
    with pytest.raises(RuntimeError, match="scales must hold"):
        fg.fastgemv_int4(W4, x, C, torch.zeros(128 * 3, dtype=torch.half, device=dev))
    with pytest.raises(RuntimeError, match="disagree on K"):
        fg.fastgemv_int4(W4, torch.zeros(2, 128, dtype=torch.half, device=dev), C)
    with pytest.raises(ValueError):
        fg.quantize_int4(torch.zeros(128, 256, dtype=torch.half, device=dev), 64)
