"""The int8 weight producer: bit-exact against the CPU oracle, and usable end to end."""
import numpy as np
import pytest
import torch

import fastgate_b200 as fg
from fastgate_b200 import workloads as wl
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,K", [(128, 128), (1000, 4096), (4096, 11008), (37, 8)])
def test_quantiser_matches_oracle_bitwise(N, K):
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(N + K)
    W = (torch.randn(N, K, generator=g) / K ** 0.5).half()
    W[0] = 0
    W[-1, -1] = 4.0
    q_ref, s_ref = oracle.quantize_rows_w8(W.numpy())
    q, s = fg.quantize_int8(W.to(dev))
    assert q.dtype == torch.int8 and s.dtype == torch.float16 and q.shape == W.shape and s.shape == (N,)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), s_ref.view(np.uint16))
    assert np.array_equal(q.cpu().numpy(), q_ref)


def test_quantise_then_int8_gemv_tracks_fp16():
    """quantize_int8 -> fastgemv_int8 reproduces the fp16 product to quantisation accuracy."""
    dev = torch.device("cuda:0")
    case = wl.Case("q", wl.OP_NK, 8, 4096, 4096, 77)
    x, W = wl.make_activation(case), wl.make_weight(case)
    q, s = fg.quantize_int8(W.to(dev))
    C = torch.zeros(8, 4096, dtype=torch.half, device=dev)
    fg.fastgemv_int8(q, x.to(dev), C, s)
    # exact for the quantised weights ...
    oracle.check_tolerance(C.cpu().numpy(), oracle.gemm_w8a16_nk(x.numpy(), q.cpu().numpy(), s.cpu().numpy()), "w8a16")
    # ... and within int8 quantisation noise of the fp16 product (error ~ |x| * step / sqrt(12) * sqrt(K))
    ref = oracle.gemm_nk(x.numpy(), W.numpy())
    assert np.abs(C.cpu().numpy().astype(np.float32) - ref).max() < 0.05
