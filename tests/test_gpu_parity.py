"""Parity of the CUDA path with the CPU oracle, through the C ABI, on a B200.

Acceptance rule (fp16 in, fp32 accumulate, fp16 out):  max|out - ref| <= 1e-2 * max(1, |ref|)
elementwise against the fp32-accumulated CPU reference of the same seeded inputs.
Every call is also checked for: status OK, no device-side timeout, no write outside the output
buffer (canaries), and a bit-identical second run (the split-K reduction order is fixed).
"""
import ctypes

import numpy as np
import pytest
import torch

from fastgate_b200 import capi, workloads as wl
from oracle import oracle

from . import gpu_util as gu
from .helpers import inputs, oracle_ref32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a B200"
    return torch.device("cuda:0")


@pytest.fixture(scope="module")
def ws(dev):
    return gu.Workspace(dev)


def run_case(case: wl.Case, dev, ws, plan=None, check_twice=True):
    x, W, s = inputs(case)
    ref = oracle_ref32(case, x, W, s)
    xd, Wd = x.to(dev), W.to(dev)
    sd = s.to(dev) if s is not None else None
    g = gu.GuardedOut(case.M, case.N, dev)
    st = gu.call(case.op, xd, Wd, sd, g.out, case.M, case.N, case.K, ws, plan)
    assert st == capi.FG_OK, capi.status_str(st)
    torch.cuda.synchronize()
    assert ws.status() == capi.FG_OK, "device-side wait timed out"
    g.check_canaries()
    out = gu.to_np(g.out)
    oracle.check_tolerance(out, ref, case.name)
    if check_twice:
        g2 = gu.GuardedOut(case.M, case.N, dev)
        assert gu.call(case.op, xd, Wd, sd, g2.out, case.M, case.N, case.K, ws, plan) == capi.FG_OK
        torch.cuda.synchronize()
        assert torch.equal(g.out.view(torch.int16), g2.out.view(torch.int16)), "two runs differ bitwise"
    return out, ref


# ---- the benchmark configurations at full size ---------------------------------------------
@pytest.mark.parametrize("case", wl.cfg1() + wl.cfg2() + wl.cfg3() + wl.cfg4(), ids=lambda c: c.name)
def test_baseline_configs(case, dev, ws):
    run_case(case, dev, ws)


@pytest.mark.parametrize("j", range(4))
def test_dit_layer_shapes(j, dev, ws):
    """The four projections of one DiT block (M=16), full and as the 1/8 shard of an 8-GPU run."""
    name, n, k = wl.DIT_LINEARS[j]
    run_case(wl.Case(f"dit_{name}", wl.OP_NK, 16, n, k, 5000 + j), dev, ws)
    run_case(wl.Case(f"dit_{name}_shard8", wl.OP_NK, 16, n // 8, k, 5100 + j), dev, ws)


# ---- small and odd shapes, every M, all three layouts -----------------------------------------
SMALL = [(128, 128), (256, 384), (384, 1152), (1152, 256), (128, 4096), (2048, 128)]


@pytest.mark.parametrize("op", [wl.OP_KN, wl.OP_NK, wl.OP_W8])
@pytest.mark.parametrize("N,K", SMALL)
def test_small_shapes_all_m(op, N, K, dev, ws):
    for M in list(range(1, 18)) + [31, 32, 33, 48]:
        run_case(wl.Case(f"op{op}_M{M}_N{N}_K{K}", op, M, N, K, 100 * M + N + K), dev, ws, check_twice=(M in (1, 8, 16, 33)))


@pytest.mark.parametrize("op", [wl.OP_KN, wl.OP_NK, wl.OP_W8])
def test_llm_shapes(op, dev, ws):
    for (N, K) in [(4096, 4096), (5120, 5120), (11008, 4096), (4096, 11008), (13824, 5120)]:
        for M in (1, 8, 16):
            run_case(wl.Case(f"op{op}_M{M}_N{N}_K{K}", op, M, N, K, M + N + K), dev, ws, check_twice=False)


# ---- known answers ------------------------------------------------------------------------
@pytest.mark.parametrize("N,K", [(4096, 4096), (11008, 4096), (4096, 11008), (5120, 13824)])
def test_all_ones_known_answer(N, K, dev, ws):
    """The reference's own check (script/ncu-gemv-test.py:29-47): all-ones operands give K."""
    want = float(np.float16(K))
    x = torch.ones(1, K, dtype=torch.float16, device=dev)
    W = torch.ones(N, K, dtype=torch.float16, device=dev)
    out = torch.zeros(1, N, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, x, W, None, out, 1, N, K, ws) == capi.FG_OK
    assert bool((out.float() == want).all())
    Wt = torch.ones(K, N, dtype=torch.float16, device=dev)
    out.zero_()
    assert gu.call(wl.OP_KN, x, Wt, None, out, 1, N, K, ws) == capi.FG_OK
    assert bool((out.float() == want).all())
    W8 = torch.ones(N, K, dtype=torch.int8, device=dev)
    out.zero_()
    assert gu.call(wl.OP_W8, x, W8, None, out, 1, N, K, ws) == capi.FG_OK
    assert bool((out.float() == want).all())


def test_one_hot_rows_and_columns(dev, ws):
    """x = e_k selects column k of the weight exactly; checks every k-offset inside a tile."""
    N, K = 256, 512
    g = torch.Generator().manual_seed(5)
    W = (torch.randn(N, K, generator=g)).to(torch.float16)
    Wd, Wtd = W.to(dev), W.t().contiguous().to(dev)
    W8 = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    W8d = W8.to(dev)
    ks = list(range(0, 80)) + [127, 128, 255, 256, 511]
    x = torch.zeros(len(ks), K, dtype=torch.float16)
    for i, k in enumerate(ks):
        x[i, k] = 1
    xd = x.to(dev)
    out = torch.zeros(len(ks), N, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, xd, Wd, None, out, len(ks), N, K, ws) == capi.FG_OK
    assert torch.equal(out.cpu(), W[:, ks].t().contiguous())
    out.zero_()
    assert gu.call(wl.OP_KN, xd, Wtd, None, out, len(ks), N, K, ws) == capi.FG_OK
    assert torch.equal(out.cpu(), W[:, ks].t().contiguous())
    out.zero_()
    assert gu.call(wl.OP_W8, xd, W8d, None, out, len(ks), N, K, ws) == capi.FG_OK
    assert torch.equal(out.cpu(), W8[:, ks].t().to(torch.float16).contiguous())


def test_int8_exact_integers(dev, ws):
    """Small-integer activations and int8 weights: every product and sum is exact, so the
    output must equal integer arithmetic bit for bit (also pins the in-register dequantiser,
    including -128 and 127)."""
    N, K, M = 256, 1024, 8
    g = torch.Generator().manual_seed(11)
    W8 = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8)
    W8[0, :4] = torch.tensor([-128, 127, -1, 0], dtype=torch.int8)
    # at most sixteen +-1 entries per row, scattered over the whole K range: |sum| <= 16 * 128 = 2048,
    # and every integer up to 2048 is a half
    x = torch.zeros(M, K, dtype=torch.float16)
    for m in range(M):
        idx = torch.randperm(K, generator=g)[:12]
        x[m, idx] = (torch.randint(0, 2, (12,), generator=g) * 2 - 1).to(torch.float16)
    x[0, :4] = 1  # meets the hand-placed weights -128, 127, -1, 0
    want = (x.double() @ W8.double().t())
    assert want.abs().max() <= 2048  # exactly representable in fp16
    out = torch.zeros(M, N, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_W8, x.to(dev), W8.to(dev), None, out, M, N, K, ws) == capi.FG_OK
    assert torch.equal(out.cpu().double(), want)


def test_int8_unscaled_reference_semantics(dev, ws):
    """fastgemv_int8 as the reference launches it: scale 1, zero-point 0, M = 1
    (hk/fastgemv.cu:50-59); outputs reach several thousand."""
    case = wl.Case("int8_noscale", wl.OP_W8, 1, 28672, 8192, 4321)
    x, W, _ = inputs(case)
    ref = oracle.gemm_w8a16_nk(x.numpy(), W.numpy(), None)
    out = torch.zeros(1, case.N, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_W8, x.to(dev), W.to(dev), None, out, 1, case.N, case.K, ws) == capi.FG_OK
    oracle.check_tolerance(gu.to_np(out), ref, "int8 unscaled")
    # and against the order-exact restatement of the reference kernel
    y_ref = oracle.gemv_int8_ref(W.numpy(), x.numpy())
    oracle.check_tolerance(gu.to_np(out), y_ref[None].astype(np.float32), "vs gemv_quantized_int8 restated")


# ---- properties at full size --------------------------------------------------------------------
def _one_rounding_step_apart(a: torch.Tensor, b: torch.Tensor) -> bool:
    """True if two fp16 results of the same sums differ by no more than a last-place flip of
    a value of magnitude >= 1 (a tenth of the path's tolerance): what a different fp32
    summation order can do, and far less than any dropped or doubled term would."""
    return oracle.tolerance_excess(gu.to_np(a), gu.to_np(b).astype(np.float32)) <= 0.1


def test_linearity_and_row_independence(dev, ws):
    """Rows of x are independent.  With the same accumulator tile height a row's bits do not
    depend on which other rows travel with it or on the pass it lands in; across tile heights
    (another K split over the warps) only the fp32 summation order changes: at most one
    rounding step of the fp16 result."""
    case = wl.Case("rows", wl.OP_NK, 40, 8192, 8192, 77)
    x, W, _ = inputs(case)
    xd, Wd = x.to(dev), W.to(dev)
    full = torch.zeros(40, 8192, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, xd, Wd, None, full, 40, 8192, 8192, ws) == capi.FG_OK
    for (a, b) in [(0, 40), (0, 33), (5, 40), (2, 39)]:  # 64-row tiles, like the full call
        part = torch.zeros(b - a, 8192, dtype=torch.float16, device=dev)
        assert gu.call(wl.OP_NK, xd[a:b].contiguous(), Wd, None, part, b - a, 8192, 8192, ws) == capi.FG_OK
        assert torch.equal(part.view(torch.int16), full[a:b].view(torch.int16)), (a, b)
    sixteen = torch.zeros(16, 8192, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, xd[0:16].contiguous(), Wd, None, sixteen, 16, 8192, 8192, ws) == capi.FG_OK
    assert _one_rounding_step_apart(sixteen, full[0:16])
    for (a, b) in [(3, 19), (7, 16), (0, 9)]:  # 16-row tiles among themselves
        part = torch.zeros(b - a, 8192, dtype=torch.float16, device=dev)
        assert gu.call(wl.OP_NK, xd[a:b].contiguous(), Wd, None, part, b - a, 8192, 8192, ws) == capi.FG_OK
        lo, hi = max(a, 0), min(b, 16)
        assert torch.equal(part[lo - a:hi - a].view(torch.int16), sixteen[lo:hi].view(torch.int16)), (a, b)
    for (a, b) in [(0, 1), (0, 8), (3, 4), (39, 40)]:  # 8-row tiles
        part = torch.zeros(b - a, 8192, dtype=torch.float16, device=dev)
        assert gu.call(wl.OP_NK, xd[a:b].contiguous(), Wd, None, part, b - a, 8192, 8192, ws) == capi.FG_OK
        assert _one_rounding_step_apart(part, full[a:b]), (a, b)
    one = torch.zeros(1, 8192, dtype=torch.float16, device=dev)
    eight = torch.zeros(8, 8192, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, xd[2:3].contiguous(), Wd, None, one, 1, 8192, 8192, ws) == capi.FG_OK
    assert gu.call(wl.OP_NK, xd[0:8].contiguous(), Wd, None, eight, 8, 8192, 8192, ws) == capi.FG_OK
    # one row runs in the row-split GEMV kernel, eight in a tiled one: other summation order
    assert _one_rounding_step_apart(one, eight[2:3])
    # a zero row gives exactly zero, scaling by two is exact in fp16
    z = torch.zeros(2, 8192, dtype=torch.float16, device=dev)
    out = torch.ones(2, 8192, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, z, Wd, None, out, 2, 8192, 8192, ws) == capi.FG_OK
    assert bool((out == 0).all())
    two = torch.zeros(1, 8192, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, (xd[2:3] * 2).contiguous(), Wd, None, two, 1, 8192, 8192, ws) == capi.FG_OK
    assert torch.equal((one.float() * 2).half().view(torch.int16), two.view(torch.int16))


def test_layouts_agree_bitwise(dev, ws):
    """KxN and NxK storage of the same weight give the same bits in the same kernel (same
    summation order): the tcgen05 kernel at 16 rows and, with the tcgen05 plan handed to the KxN
    call, at 8 rows.  The planner's own choice for KxN at 8 rows is the mma.sync kernel, which
    cuts the sums differently: one rounding step apart."""
    case = wl.Case("kn_vs_nk", wl.OP_NK, 16, 4096, 4096, 99)
    x, W, _ = inputs(case)
    a = torch.zeros(16, 4096, dtype=torch.float16, device=dev)
    b = torch.zeros(16, 4096, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, x.to(dev), W.to(dev), None, a, 16, 4096, 4096, ws) == capi.FG_OK
    assert gu.call(wl.OP_KN, x.to(dev), W.t().contiguous().to(dev), None, b, 16, 4096, 4096, ws) == capi.FG_OK
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    a8 = torch.zeros(8, 4096, dtype=torch.float16, device=dev)
    b8 = torch.zeros(8, 4096, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, x[:8].contiguous().to(dev), W.to(dev), None, a8, 8, 4096, 4096, ws) == capi.FG_OK
    umma_kn = capi.plan(wl.OP_KN, 16, 4096, 4096, 148, 232448)  # serves any M <= 16
    assert umma_kn.math == 2
    assert gu.call(wl.OP_KN, x[:8].contiguous().to(dev), W.t().contiguous().to(dev), None, b8, 8, 4096, 4096, ws,
                   plan=umma_kn) == capi.FG_OK
    assert torch.equal(a8.view(torch.int16), b8.view(torch.int16))
    c8 = torch.zeros(8, 4096, dtype=torch.float16, device=dev)
    assert capi.plan(wl.OP_KN, 8, 4096, 4096, 148, 232448).math == 0
    assert gu.call(wl.OP_KN, x[:8].contiguous().to(dev), W.t().contiguous().to(dev), None, c8, 8, 4096, 4096, ws) == capi.FG_OK
    assert _one_rounding_step_apart(c8, a8)


def test_n_shards_concatenate_to_the_full_result(dev, ws):
    """Column-partitioning the weight by N (the multi-GPU scheme) only moves the stream-K cuts,
    i.e. the fp32 summation order: the assembled result is within one rounding step
    of the single-GPU one, and within tolerance of the oracle."""
    case = wl.Case("shards", wl.OP_NK, 16, 9216, 3072, 123)
    x, W, _ = inputs(case)
    xd = x.to(dev)
    full = torch.zeros(16, 9216, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, xd, W.to(dev), None, full, 16, 9216, 3072, ws) == capi.FG_OK
    for world in (2, 4, 8):
        parts = []
        for r in range(world):
            b, e = wl.shard_rows(9216, world, r)
            o = torch.zeros(16, e - b, dtype=torch.float16, device=dev)
            assert gu.call(wl.OP_NK, xd, W[b:e].contiguous().to(dev), None, o, 16, e - b, 3072, ws) == capi.FG_OK
            parts.append(o)
        cat = torch.cat(parts, dim=1)
        assert _one_rounding_step_apart(cat, full), world
        oracle.check_tolerance(gu.to_np(cat), oracle.gemm_nk(x.numpy(), W.numpy()), f"{world} shards")


# ---- every plan shape the kernel accepts ----------------------------------------------------------
def _edited(base, N, K, op, m_tile, chunks, warps, stages, grid, pdl):
    p = capi.Plan()
    ctypes.memmove(ctypes.byref(p), ctypes.byref(base), ctypes.sizeof(p))
    ck = 128 if op == wl.OP_W8 else 64
    p.m_tile = m_tile
    p.math = 0
    p.k_per_stage = chunks * ck
    p.k_blocks = -(-K // p.k_per_stage)
    p.consumer_warps, p.stages, p.pdl = warps, stages, pdl
    p.grid = min(grid, p.tiles * p.k_blocks)
    cb = chunks * (16384 + (2 if op == wl.OP_W8 else 1) * m_tile * 128)
    p.smem_bytes = 1024 + warps * m_tile * 132 * 4 + 32 + stages * (cb + 16)
    return p if capi.lib.fg_plan_validate(ctypes.byref(p), N, K, 232448) == capi.FG_OK else None


@pytest.mark.parametrize("op", [wl.OP_KN, wl.OP_NK, wl.OP_W8])
def test_plan_walk(op, dev, ws):
    """Ring depth, warps, chunks per stage, grid size, tile height and PDL are free parameters
    of the kernel: results must not depend on them beyond summation order."""
    N, K = 1152, 2304
    tried = 0
    for M in (3, 8, 13, 16):
        case = wl.Case(f"walk_op{op}_M{M}", op, M, N, K, 31 + M)
        base = capi.plan(op, M, N, K, 148, 232448)
        for m_tile in ((8, 16) if M <= 8 else (16,)):
            for chunks, warps, stages, grid, pdl in [(1, 1, 2, 148, 0), (1, 2, 2, 7, 1), (2, 4, 4, 148, 1), (4, 2, 2, 37, 0),
                                                    (1, 8, 8, 148, 1), (2, 3, 3, 148, 0), (1, 5, 10, 1, 0), (3, 2, 4, 100, 1),
                                                    (1, 4, 12, 148, 1), (1, 3, 9, 148, 0), (1, 6, 6, 3, 1)]:
                p = _edited(base, N, K, op, m_tile, chunks, warps, stages, grid, pdl)
                if p is None:
                    continue
                run_case(case, dev, ws, plan=p, check_twice=False)
                tried += 1
    assert tried >= 30


def _edited_umma(base, N, K, op, chunks, stages, grid, pdl, m_tile=16):
    p = capi.Plan()
    ctypes.memmove(ctypes.byref(p), ctypes.byref(base), ctypes.sizeof(p))
    p.m_tile, p.math, p.consumer_warps, p.pdl = m_tile, 2, 4, pdl
    p.k_per_stage = chunks * 64
    p.k_blocks = -(-K // p.k_per_stage)
    p.stages = stages
    p.grid = min(grid, p.tiles * p.k_blocks)
    p.smem_bytes = 1024 + stages * (chunks * (16384 + m_tile * 128) + 16) + 64
    return p if capi.lib.fg_plan_validate(ctypes.byref(p), N, K, 232448) == capi.FG_OK else None


@pytest.mark.parametrize("op", [wl.OP_KN, wl.OP_NK])
def test_plan_walk_tcgen05(op, dev, ws):
    """The tcgen05 kernel over ring depths, stage sizes, grid sizes, tile heights, with and
    without PDL, for every M (any tile height serves any smaller M; the planner only picks the
    kernel above 8 rows and the smallest tile that holds the call)."""
    N, K = 1152, 2304
    tried = 0
    for M, m_tile in ((1, 16), (5, 64), (8, 16), (11, 32), (16, 16), (21, 32)):
        case = wl.Case(f"umma_walk_op{op}_M{M}", op, M, N, K, 61 + M)
        base = capi.plan(op, M, N, K, 148, 232448)
        for chunks, stages, grid, pdl in [(1, 2, 148, 0), (1, 12, 148, 1), (2, 6, 148, 1), (4, 3, 148, 0), (3, 4, 17, 1),
                                          (1, 5, 1, 0), (2, 2, 148, 1), (1, 7, 97, 0)]:
            if m_tile > 16 and chunks * (16384 + m_tile * 128) * stages > 220000:
                stages = 2  # the taller activation boxes leave room for fewer of the large stages
            p = _edited_umma(base, N, K, op, chunks, stages, grid, pdl, m_tile)
            assert p is not None, (M, m_tile, chunks, stages)
            run_case(case, dev, ws, plan=p, check_twice=(tried % 5 == 0))
            tried += 1
    assert tried == 48


def test_ragged_last_stage_tcgen05(dev, ws):
    for (op, K) in [(wl.OP_NK, 384), (wl.OP_KN, 640), (wl.OP_NK, 896)]:
        N, M = 256, 13
        base = capi.plan(op, M, N, K, 148, 232448)
        for chunks in (2, 4):
            p = _edited_umma(base, N, K, op, chunks, 3, 148, 1)
            assert p is not None
            run_case(wl.Case(f"umma_ragged_op{op}_K{K}_c{chunks}", op, M, N, K, K + chunks), dev, ws, plan=p)


def test_ragged_last_stage(dev, ws):
    """K that is not a multiple of the stage width: the last stage of a tile is short."""
    for (op, K) in [(wl.OP_NK, 384), (wl.OP_KN, 640), (wl.OP_W8, 384), (wl.OP_W8, 896)]:
        N, M = 256, 5
        base = capi.plan(op, M, N, K, 148, 232448)
        for chunks in (2, 4):
            p = _edited(base, N, K, op, 8, chunks, 2, 2, 148, 1)
            assert p is not None
            run_case(wl.Case(f"ragged_op{op}_K{K}_c{chunks}", op, M, N, K, K + chunks), dev, ws, plan=p)


# ---- error paths on the device ----------------------------------------------------------------------
def test_errors_with_device_present(dev, ws):
    x = torch.zeros(16, 256, dtype=torch.float16, device=dev)
    W = torch.zeros(256, 256, dtype=torch.float16, device=dev)
    out = torch.zeros(16, 256, dtype=torch.float16, device=dev)
    Lc = capi.lib
    assert Lc.fg_gemm_f16_nk(x.data_ptr(), W.data_ptr(), out.data_ptr(), 16, 200, 256, ws.ptr, ws.bytes, gu.stream()) == capi.FG_ERR_SHAPE
    assert Lc.fg_gemm_f16_nk(x.data_ptr() + 2, W.data_ptr(), out.data_ptr(), 1, 256, 256, ws.ptr, ws.bytes, gu.stream()) == capi.FG_ERR_ALIGN
    assert Lc.fg_gemm_f16_nk(x.data_ptr(), W.data_ptr(), out.data_ptr(), 16, 256, 256, ws.ptr, 4096, gu.stream()) == capi.FG_ERR_WORKSPACE
    bad = capi.plan(wl.OP_NK, 16, 256, 256, 148, 232448)
    bad.stages += 1
    assert Lc.fg_gemm_planned(ctypes.byref(bad), x.data_ptr(), W.data_ptr(), None, out.data_ptr(), 16, 256, 256,
                              ws.ptr, ws.bytes, gu.stream()) == capi.FG_ERR_PLAN
    # a plan for 8 rows (KxN weights: the 8-row mma.sync kernel) cannot serve 16
    p8 = capi.plan(wl.OP_KN, 8, 256, 256, 148, 232448)
    assert p8.m_tile == 8
    p8.passes = 1
    assert Lc.fg_gemm_planned(ctypes.byref(p8), x.data_ptr(), W.data_ptr(), None, out.data_ptr(), 16, 256, 256,
                              ws.ptr, ws.bytes, gu.stream()) == capi.FG_ERR_PLAN
    assert ws.status() == capi.FG_OK


def test_linear_host_entry_point(dev, ws):
    """fg_linear_host: host activations in, host result out, weight resident."""
    case = wl.Case("host", wl.OP_NK, 16, 4096, 4096, 5)
    x, W, _ = inputs(case)
    xh = x.pin_memory()
    ch = torch.empty(16, 4096, dtype=torch.float16).pin_memory()
    Wd = W.to(dev)
    xs = torch.empty_like(x, device=dev)
    cs = torch.empty(16, 4096, dtype=torch.float16, device=dev)
    st = capi.lib.fg_linear_host(wl.OP_NK, xh.data_ptr(), Wd.data_ptr(), None, ch.data_ptr(), xs.data_ptr(), cs.data_ptr(),
                                 16, 4096, 4096, ws.ptr, ws.bytes, gu.stream())
    assert st == capi.FG_OK, capi.status_str(st)
    oracle.check_tolerance(ch.numpy(), oracle.gemm_nk(x.numpy(), W.numpy()), "fg_linear_host")


def test_tracer(dev, ws):
    """The built-in tracer records monotone per-CTA timestamps and does not change results."""
    case = wl.Case("trace", wl.OP_NK, 8, 4096, 4096, 6)
    out_plain, _ = run_case(case, dev, ws, check_twice=False)
    capi.lib.fg_trace_enable(1)
    try:
        out_traced, _ = run_case(case, dev, ws, check_twice=False)
        p = capi.plan(case.op, case.M, case.N, case.K, 148, 232448)
        buf = (ctypes.c_ulonglong * (16 * p.grid))()
        assert capi.lib.fg_trace_read(ws.ptr, buf, p.grid, gu.stream()) == capi.FG_OK
    finally:
        capi.lib.fg_trace_enable(0)
    assert np.array_equal(out_plain, out_traced)
    t = np.array(list(buf), dtype=np.uint64).reshape(p.grid, 16)
    assert (t[:, 0] > 0).all() and (t[:, 1] >= t[:, 0]).all() and (t[:, 2] >= t[:, 1]).all()
    assert (t[:, 6] >= 1).all()
    # the next plain call must find the borrowed workspace corner clean and still be right
    run_case(case, dev, ws, check_twice=False)
