"""fg_gemm_f16_nk_noalloc: the entry point for callers that cannot allocate device memory.

Some users of this library are handed device buffers but no allocator (a plugin inside a host
application, code under a fixed memory budget); they cannot create the workspace the normal
entry points need.  This entry point keeps its scratch in a static array inside the library.
The test calls it through the C ABI twice in a row (the array is shared by all calls and keeps
the previous call's contents) and compares each result with the workspace-based entry point
on the same inputs, using the path's tolerance; the two should in fact agree bit for bit,
since the same kernel runs with the same plan.  This file sorts last on purpose: a run that
stops at the first failure has then already run every other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from fastgate_b200 import capi, workloads as wl
from oracle import oracle

pytestmark = pytest.mark.gpu


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("M,N,K", [(16, 4096, 4096), (3, 1152, 2304)])
def test_noalloc_matches_workspace_entry_point_twice(M, N, K):
    assert torch.cuda.is_available(), "needs a B200"
    dev = torch.device("cuda:0")
    L = capi.lib
    ws_bytes = capi.workspace_bytes(N)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    assert L.fg_workspace_init(ws.data_ptr(), ws_bytes, _stream()) == capi.FG_OK
    for round_ in range(2):  # second call finds the scratch as the first one left it
        case = wl.Case("noalloc", wl.OP_NK, M, N, K, 8800 + round_)
        x, W = wl.make_activation(case).to(dev), wl.make_weight(case).to(dev)
        want = torch.zeros(M, N, dtype=torch.float16, device=dev)
        got = torch.full((M, N), float("nan"), dtype=torch.float16, device=dev)
        assert L.fg_gemm_f16_nk(x.data_ptr(), W.data_ptr(), want.data_ptr(), M, N, K, ws.data_ptr(), ws_bytes,
                                _stream()) == capi.FG_OK
        st = L.fg_gemm_f16_nk_noalloc(x.data_ptr(), W.data_ptr(), got.data_ptr(), M, N, K, _stream())
        assert st == capi.FG_OK, capi.status_str(st)
        torch.cuda.synchronize()
        oracle.check_tolerance(got.cpu().numpy(), want.cpu().numpy().astype(np.float32), f"round {round_}")
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"round {round_}: bits differ"
        # and both agree with the CPU oracle
        oracle.check_tolerance(got.cpu().numpy(), oracle.gemm_nk(x.cpu().numpy(), W.cpu().numpy()), "oracle")
        v = ctypes.c_int(-1)
        assert L.fg_noalloc_status(ctypes.byref(v), _stream()) == capi.FG_OK and v.value == capi.FG_OK


def test_noalloc_more_than_16_rows_runs_in_16_row_passes():
    """The built-in scratch holds 16-row partial tiles, so a taller call goes in passes of 16
    (the workspace entry point would take 64 rows at once): same values within one rounding step."""
    assert torch.cuda.is_available(), "needs a B200"
    dev = torch.device("cuda:0")
    M, N, K = 40, 4096, 4096
    case = wl.Case("noalloc_tall", wl.OP_NK, M, N, K, 8810)
    x, W = wl.make_activation(case).to(dev), wl.make_weight(case).to(dev)
    got = torch.full((M, N), float("nan"), dtype=torch.float16, device=dev)
    n0 = capi.launch_count()
    st = capi.lib.fg_gemm_f16_nk_noalloc(x.data_ptr(), W.data_ptr(), got.data_ptr(), M, N, K, _stream())
    assert st == capi.FG_OK, capi.status_str(st)
    torch.cuda.synchronize()
    assert capi.launch_count() - n0 == 3
    oracle.check_tolerance(got.cpu().numpy(), oracle.gemm_nk(x.cpu().numpy(), W.cpu().numpy()), "tall noalloc")


def test_noalloc_rejects_what_does_not_fit():
    assert torch.cuda.is_available(), "needs a B200"
    dev = torch.device("cuda:0")
    L = capi.lib
    x = torch.zeros(1, 128, dtype=torch.float16, device=dev)
    C = torch.zeros(1, 128, dtype=torch.float16, device=dev)
    # N beyond the built-in scratch: refused before anything is launched (pointers are never read)
    assert L.fg_gemm_f16_nk_noalloc(x.data_ptr(), x.data_ptr(), C.data_ptr(), 1, 65536 + 128, 128, _stream()) == capi.FG_ERR_WORKSPACE
    assert L.fg_gemm_f16_nk_noalloc(x.data_ptr(), x.data_ptr(), C.data_ptr(), 1, 100, 128, _stream()) == capi.FG_ERR_SHAPE
    assert L.fg_gemm_f16_nk_noalloc(None, x.data_ptr(), C.data_ptr(), 1, 128, 128, _stream()) == capi.FG_ERR_NULL
