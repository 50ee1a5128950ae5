"""The row-split GEMV kernel (plan.math == 4: NxK fp16 weights, one or two token rows).

Through the C ABI, against the CPU oracle: the shapes of the fastgemv / fastgemm configurations,
every way of dealing the rows (all up front, all on demand, mixed), ring depths and warp counts the
kernel accepts, the fused epilogue, and the bookkeeping the kernel leaves in the workspace
(its row-block counter and exit counter must read zero after every launch)."""
import ctypes

import numpy as np
import pytest
import torch

from fastgate_b200 import capi, workloads as wl
from oracle import oracle

from . import gpu_util as gu

pytestmark = pytest.mark.gpu
L = capi.lib


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a B200"
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def ws(dev):
    return gu.Workspace(dev)


def counters(ws):
    """(row-block counter, exit counter) in the workspace header."""
    torch.cuda.synchronize()
    h = ws.buf[:256].cpu().numpy().view(np.uint32)
    return int(h[16]), int(h[32])


def edited(base, N, K, **kw):
    p = capi.Plan()
    ctypes.memmove(ctypes.byref(p), ctypes.byref(base), ctypes.sizeof(p))
    for k, v in kw.items():
        setattr(p, k, v)
    stage = p.rows_per_stage * K * 2
    p.smem_bytes = 127 + ((p.m_tile * K * 2 + 127) // 128 * 128) + 8 + p.stages * (stage + 24)
    return p if L.fg_plan_validate(ctypes.byref(p), N, K, 232448) == capi.FG_OK else None


def run(case, dev, ws, plan=None, twice=True):
    x, W = wl.make_activation(case), wl.make_weight(case)
    ref = oracle.gemm_nk(x.numpy(), W.numpy())
    xd, Wd = x.to(dev), W.to(dev)
    g = gu.GuardedOut(case.M, case.N, dev)
    st = gu.call(wl.OP_NK, xd, Wd, None, g.out, case.M, case.N, case.K, ws, plan)
    assert st == capi.FG_OK, capi.status_str(st)
    torch.cuda.synchronize()
    assert ws.status() == capi.FG_OK, "device-side wait timed out"
    assert counters(ws) == (0, 0), "the kernel must leave its counters at zero"
    g.check_canaries()
    oracle.check_tolerance(gu.to_np(g.out), ref, case.name)
    if twice:
        g2 = gu.GuardedOut(case.M, case.N, dev)
        assert gu.call(wl.OP_NK, xd, Wd, None, g2.out, case.M, case.N, case.K, ws, plan) == capi.FG_OK
        torch.cuda.synchronize()
        assert torch.equal(g.out.view(torch.int16), g2.out.view(torch.int16)), "two runs differ bitwise"
    return g.out


SHAPES = [(11008, 4096), (4096, 11008), (8192, 8192), (4096, 4096), (128, 1024), (256, 2304), (384, 3072),
          (1152, 2304), (3072, 12288), (640, 16384), (13824, 5120)]


def gemv_plan(M, N, K):
    """The GEMV plan for a shape, also where the planner prefers a tiled kernel (two rows of a large weight)."""
    p = capi.plan(wl.OP_NK, M, N, K, 148, 232448)
    if p.math == 4:
        return p
    one = capi.plan(wl.OP_NK, 1, N, K, 148, 232448)
    assert one.math == 4
    rows = one.rows_per_stage
    while rows * M > 8:
        rows //= 2
    x_bytes = (M * K * 2 + 127) // 128 * 128
    fit = min(24, (232448 - 127 - x_bytes - 8) // (rows * K * 2 + 24))
    def divisor(s):  # the largest warp count up to twelve that divides the ring depth
        return max(w for w in range(1, min(s, 12) + 1) if s % w == 0)

    stages = max(range(max(3, fit - 3), fit + 1), key=lambda s: (divisor(s), s))
    warps = divisor(stages)
    return edited(one, N, K, m_tile=M, rows_per_stage=rows, stages=stages, consumer_warps=warps,
                  static_rows=(N // one.grid) // rows * rows)


@pytest.mark.parametrize("N,K", SHAPES)
@pytest.mark.parametrize("M", [1, 2])
def test_gemv_matches_the_oracle(M, N, K, dev, ws):
    planned = capi.plan(wl.OP_NK, M, N, K, 148, 232448)
    assert (planned.math == 4) == (M == 1 or N * K <= 48 << 20), "one row always, two rows up to 48 Mi weights"
    p = gemv_plan(M, N, K)
    assert p is not None and p.math == 4
    run(wl.Case(f"gemv_M{M}_N{N}_K{K}", wl.OP_NK, M, N, K, 7000 + M + N + K), dev, ws, plan=p)


@pytest.mark.parametrize("M", [1, 2])
def test_every_way_of_dealing_rows_gives_the_same_bits(M, dev, ws):
    """Who computes a row does not enter its sum: all rows up front, all on demand, a mix, fewer
    CTAs, other ring depths and warp counts give bit-identical results."""
    N, K = 1152, 4096
    case = wl.Case(f"gemv_walk_M{M}", wl.OP_NK, M, N, K, 7100 + M)
    base = capi.plan(wl.OP_NK, M, N, K, 148, 232448)
    assert base.math == 4
    want = run(case, dev, ws)
    rb = base.rows_per_stage
    tried = 0
    for kw in [dict(static_rows=0), dict(static_rows=(N // 2 // base.grid) // rb * rb), dict(grid=37, static_rows=0),
               dict(grid=1, static_rows=0), dict(grid=5, static_rows=(N // 5) // rb * rb), dict(stages=4, consumer_warps=4),
               dict(stages=6, consumer_warps=3), dict(stages=3, consumer_warps=1), dict(stages=12, consumer_warps=12),
               dict(rows_per_stage=1, static_rows=0), dict(rows_per_stage=2 * rb if 2 * rb * M <= 8 else rb, static_rows=0), dict(pdl=0)]:
        p = edited(base, N, K, **kw)
        if p is None:
            continue
        got = run(case, dev, ws, plan=p, twice=False)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), kw
        tried += 1
    assert tried >= 9


def test_rows_are_independent_of_m(dev, ws):
    """Row 0 of a two-row call equals the one-row call on the same activations, bit for bit."""
    N, K = 2048, 8192
    case = wl.Case("gemv_rows", wl.OP_NK, 2, N, K, 7200)
    x, W = wl.make_activation(case).to(dev), wl.make_weight(case).to(dev)
    two = torch.zeros(2, N, dtype=torch.float16, device=dev)
    one = torch.zeros(1, N, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, x, W, None, two, 2, N, K, ws) == capi.FG_OK
    assert gu.call(wl.OP_NK, x[:1].contiguous(), W, None, one, 1, N, K, ws) == capi.FG_OK
    torch.cuda.synchronize()
    assert torch.equal(two[:1].view(torch.int16), one.view(torch.int16))


def test_one_hot_activations_select_weight_columns(dev, ws):
    N, K = 256, 2048
    g = torch.Generator().manual_seed(3)
    W = torch.randn(N, K, generator=g).to(torch.float16)
    Wd = W.to(dev)
    for k in (0, 1, 7, 8, 255, 256, 1023, 2047):
        x = torch.zeros(1, K, dtype=torch.float16)
        x[0, k] = 1
        out = torch.zeros(1, N, dtype=torch.float16, device=dev)
        assert gu.call(wl.OP_NK, x.to(dev), Wd, None, out, 1, N, K, ws) == capi.FG_OK
        assert torch.equal(out.cpu()[0], W[:, k]), k


@pytest.mark.parametrize("act", ["none", "gelu", "gelu_tanh", "silu"])
@pytest.mark.parametrize("M", [1, 2])
def test_fused_epilogue(act, M, dev, ws):
    N, K = 1152, 2304
    case = wl.Case("gemv_fused", wl.OP_NK, M, N, K, 7300 + M)
    x, W = wl.make_activation(case), wl.make_weight(case)
    g = torch.Generator().manual_seed(M)
    bias = torch.randn(N, generator=g).half()
    res = torch.randn(M, N, generator=g).half()
    ref = oracle.epilogue(oracle.gemm_nk(x.numpy(), W.numpy()), bias.numpy(), res.numpy(), capi.ACT[act])
    C = torch.full((M, N), float("nan"), dtype=torch.half, device=dev)
    bd, rd = bias.to(dev), res.to(dev)
    ep = capi.Epilogue(bd.data_ptr(), rd.data_ptr(), capi.ACT[act])
    xd, Wd = x.to(dev), W.to(dev)
    st = L.fg_gemm_fused(capi.FG_OP_F16_NK, xd.data_ptr(), Wd.data_ptr(), None, C.data_ptr(), M, N, K, ctypes.byref(ep),
                         ws.ptr, ws.bytes, gu.stream())
    assert st == capi.FG_OK, capi.status_str(st)
    torch.cuda.synchronize()
    oracle.check_tolerance(C.cpu().numpy(), ref, f"{act} M={M}")


def test_the_tiled_kernels_take_what_the_gemv_kernel_cannot(dev, ws):
    """Three rows and more, rows too short or too long for a ring of whole rows, KxN weights, int8 weights with two rows: other plans."""
    for (op, M, N, K) in [(wl.OP_NK, 3, 4096, 4096), (wl.OP_NK, 1, 256, 512), (wl.OP_NK, 1, 256, 32768), (wl.OP_KN, 1, 4096, 4096),
                          (wl.OP_W8, 2, 4096, 4096)]:
        assert capi.plan(op, M, N, K, 148, 232448).math != 4
    for (M, N, K) in [(1, 256, 512), (2, 128, 32768)]:
        case = wl.Case("not_gemv", wl.OP_NK, M, N, K, 7400 + M)
        x, W = wl.make_activation(case), wl.make_weight(case)
        out = torch.zeros(M, N, dtype=torch.float16, device=dev)
        assert gu.call(wl.OP_NK, x.to(dev), W.to(dev), None, out, M, N, K, ws) == capi.FG_OK
        oracle.check_tolerance(out.cpu().numpy(), oracle.gemm_nk(x.numpy(), W.numpy()), case.name)


# ---- int8 weights, one token row --------------------------------------------------------------
W8_SHAPES = [(28672, 8192), (4096, 4096), (128, 2048), (11008, 4096), (384, 16384), (1152, 2304), (256, 32768)]


def _w8_case(N, K, seed):
    case = wl.Case(f"gemv_w8_N{N}_K{K}", wl.OP_W8, 1, N, K, seed)
    return case, wl.make_activation(case), wl.make_weight(case), wl.make_scales(case)


@pytest.mark.parametrize("N,K", W8_SHAPES)
@pytest.mark.parametrize("scaled", [True, False])
def test_int8_gemv_matches_the_oracle(N, K, scaled, dev, ws):
    """fastgemv_int8's shape class on the row-split kernel: exact int8 -> fp16 conversion, fp32 sums, one
    scale per output channel in the epilogue.  Twice, bit for bit; against the tiled kernel within the tolerance."""
    case, x, W, sc = _w8_case(N, K, 7500 + N + K)
    sc = sc if scaled else None
    p = capi.plan(wl.OP_W8, 1, N, K, 148, 232448)
    assert p.math == 4 and p.m_tile == 1 and p.rows_per_stage * K <= 65536, p.as_dict()
    ref = oracle.gemm_w8a16_nk(x.numpy(), W.numpy(), sc.numpy() if scaled else None)
    xd, Wd = x.to(dev), W.to(dev)
    sd = sc.to(dev) if scaled else None
    outs = []
    for _ in range(2):
        g = gu.GuardedOut(1, N, dev)
        st = gu.call(wl.OP_W8, xd, Wd, sd, g.out, 1, N, K, ws)
        assert st == capi.FG_OK, capi.status_str(st)
        torch.cuda.synchronize()
        assert ws.status() == capi.FG_OK and counters(ws) == (0, 0)
        g.check_canaries()
        outs.append(g.out)
    oracle.check_tolerance(gu.to_np(outs[0]), ref, case.name)
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    tiled = capi.Plan()
    assert L.fg_plan_mma_sync(wl.OP_W8, 1, N, K, 148, 232448, ctypes.byref(tiled)) == capi.FG_OK and tiled.math == 0
    t = gu.GuardedOut(1, N, dev)
    assert gu.call(wl.OP_W8, xd, Wd, sd, t.out, 1, N, K, ws, tiled) == capi.FG_OK
    torch.cuda.synchronize()
    oracle.check_tolerance(gu.to_np(t.out), ref, case.name + " tiled")


def test_int8_gemv_extreme_weights_and_one_hot(dev, ws):
    """Every int8 value converts exactly: a one-hot activation reads single weights back, scaled by one."""
    N, K = 256, 2048
    W = (torch.arange(N * K, dtype=torch.int64).reshape(N, K) * 37 % 255 - 127).to(torch.int8)
    W[0, :256] = torch.arange(-128, 128, dtype=torch.int64).to(torch.int8)[:256]
    Wd = W.to(dev)
    for k in (0, 1, 2, 3, 15, 16, 255, 1024, 2047):
        x = torch.zeros(1, K, dtype=torch.float16)
        x[0, k] = 1
        out = torch.zeros(1, N, dtype=torch.float16, device=dev)
        assert gu.call(wl.OP_W8, x.to(dev), Wd, None, out, 1, N, K, ws) == capi.FG_OK
        assert torch.equal(out.cpu()[0], W[:, k].to(torch.float16)), k


def test_int8_gemv_fused_epilogue(dev, ws):
    N, K = 1152, 4096
    case, x, W, sc = _w8_case(N, K, 7600)
    g = torch.Generator().manual_seed(9)
    bias, res = torch.randn(N, generator=g).half(), torch.randn(1, N, generator=g).half()
    ref = oracle.epilogue(oracle.gemm_w8a16_nk(x.numpy(), W.numpy(), sc.numpy()), bias.numpy(), res.numpy(), capi.ACT["silu"])
    xd, Wd, sd, bd, rd = x.to(dev), W.to(dev), sc.to(dev), bias.to(dev), res.to(dev)
    C = torch.full((1, N), float("nan"), dtype=torch.half, device=dev)
    ep = capi.Epilogue(bd.data_ptr(), rd.data_ptr(), capi.ACT["silu"])
    st = L.fg_gemm_fused(capi.FG_OP_W8A16_NK, xd.data_ptr(), Wd.data_ptr(), sd.data_ptr(), C.data_ptr(), 1, N, K, ctypes.byref(ep),
                         ws.ptr, ws.bytes, gu.stream())
    assert st == capi.FG_OK, capi.status_str(st)
    torch.cuda.synchronize()
    oracle.check_tolerance(C.cpu().numpy(), ref, "w8 gemv fused")


def test_int8_rows_too_short_or_too_many_tokens_stay_tiled():
    for (M, N, K) in [(2, 4096, 4096), (8, 28672, 8192), (1, 256, 1024), (1, 128, 65536)]:
        assert capi.plan(wl.OP_W8, M, N, K, 148, 232448).math != 4
