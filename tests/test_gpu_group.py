"""Grouped launch (fg_group_*): many independent problems in one persistent kernel."""
import ctypes

import numpy as np
import pytest
import torch

from fastgate_b200 import capi, workloads as wl
from fastgate_b200.group import LinearGroup
from oracle import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "needs a B200"
    return torch.device("cuda:0")


def _problems(shapes, layout, dev, seed0):
    xs, Ws, Cs, refs = [], [], [], []
    for i, (M, N, K) in enumerate(shapes):
        case = wl.Case("g", wl.OP_NK, M, N, K, seed0 + i)
        x, W = wl.make_activation(case), wl.make_weight(case)
        refs.append(oracle.gemm_nk(x.numpy(), W.numpy()))
        xs.append(x.to(dev))
        Ws.append((W if layout == "nk" else W.t().contiguous()).to(dev))
        Cs.append(torch.full((M, N), float("nan"), dtype=torch.float16, device=dev))
    return xs, Ws, Cs, refs


@pytest.mark.parametrize("layout", ["nk", "kn"])
def test_mixed_shapes(layout, dev):
    """Different M, N, K per problem, ragged last stages, problems smaller than one CTA's share."""
    shapes = [(16, 1152, 768), (3, 128, 128), (8, 384, 2304), (1, 256, 384), (16, 3072, 3072), (11, 128, 4096),
              (16, 9216, 3072), (5, 640, 896)]
    xs, Ws, Cs, refs = _problems(shapes, layout, dev, 300)
    grp = LinearGroup(xs, Ws, Cs, weight_layout=layout)
    grp.run()
    torch.cuda.synchronize()
    assert grp.status() == capi.FG_OK
    first = [c.clone() for c in Cs]
    for C, ref, shp in zip(Cs, refs, shapes):
        oracle.check_tolerance(C.cpu().numpy(), ref, f"group {shp}")
    for C in Cs:
        C.fill_(float("nan"))
    grp.run()
    torch.cuda.synchronize()
    for a, b in zip(first, Cs):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16)), "two runs differ bitwise"


def test_dit_block_as_one_launch(dev):
    """Two DiT blocks (eight projections, M = 16) in one launch equal the per-layer operator
    within one rounding step (only the stream-K cuts, i.e. the fp32 summation order, differ)."""
    import fastgate_b200 as fg

    shapes = [(16, n, k) for _ in range(2) for (_, n, k) in wl.DIT_LINEARS]
    xs, Ws, Cs, refs = _problems(shapes, "nk", dev, 500)
    grp = LinearGroup(xs, Ws, Cs)
    n0 = fg.launch_count()
    grp.run()
    assert fg.launch_count() - n0 == 1
    torch.cuda.synchronize()
    for x, W, C, ref in zip(xs, Ws, Cs, refs):
        oracle.check_tolerance(C.cpu().numpy(), ref, "dit group")
        single = torch.zeros_like(C)
        fg.edgemm_m8n128k64x4_bt(x, W, single)
        assert oracle.tolerance_excess(C.cpu().numpy(), single.cpu().numpy().astype(np.float32)) <= 0.1


def test_single_problem_group_and_known_answer(dev):
    x = torch.ones(4, 4096, dtype=torch.float16, device=dev)
    W = torch.ones(512, 4096, dtype=torch.float16, device=dev)
    C = torch.zeros(4, 512, dtype=torch.float16, device=dev)
    grp = LinearGroup([x], [W], [C])
    grp.run()
    torch.cuda.synchronize()
    assert bool((C == 4096).all())


def test_group_pushes_into_peer_outputs(dev):
    """Two ranks emulated back to back on one GPU: each rank's group stores its column slice of
    every problem into both full outputs and bumps its own counter on both flag arrays."""
    world, M = 2, 16
    shapes = [(M, 512, 1024), (M, 256, 384), (M, 1024, 512)]   # N = per-rank columns
    full_refs, xs_host, Ws_host = [], [], []
    for i, (_, n, k) in enumerate(shapes):
        case = wl.Case("gp", wl.OP_NK, M, n * world, k, 700 + i)
        x, W = wl.make_activation(case), wl.make_weight(case)
        xs_host.append(x)
        Ws_host.append(W)
        full_refs.append(oracle.gemm_nk(x.numpy(), W.numpy()))
    outs = [[torch.full((M, n * world), float("nan"), dtype=torch.float16, device=dev) for (_, n, _) in shapes]
            for _ in range(world)]
    flags = [torch.zeros(8, dtype=torch.int64, device=dev) for _ in range(world)]
    groups = []
    for r in range(world):
        xs = [x.to(dev) for x in xs_host]
        Ws = [W[r * n:(r + 1) * n].contiguous().to(dev) for W, (_, n, _) in zip(Ws_host, shapes)]
        peer_ptrs = [[outs[q][i].data_ptr() for q in range(world)] for i in range(len(shapes))]
        groups.append(LinearGroup(xs, Ws, None, peer_C_ptrs=peer_ptrs, flag_ptrs=[f.data_ptr() for f in flags], rank=r,
                                  n_totals=[n * world for (_, n, _) in shapes]))
    for g in groups:
        g.run()
    ws = torch.zeros(capi.workspace_bytes(128), dtype=torch.uint8, device=dev)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for r in range(world):
        assert capi.lib.fg_push_wait(flags[r].data_ptr(), world, groups[0].tiles, ws.data_ptr(), stream) == capi.FG_OK
    torch.cuda.synchronize()
    for r in range(world):
        assert flags[r][:world].tolist() == [groups[0].tiles] * world
        for i, ref in enumerate(full_refs):
            oracle.check_tolerance(outs[r][i].cpu().numpy(), ref, f"rank {r} problem {i}")
    for i in range(len(shapes)):
        assert torch.equal(outs[0][i].view(torch.int16), outs[1][i].view(torch.int16))


def test_group_argument_checks(dev):
    x = torch.zeros(17, 128, dtype=torch.float16, device=dev)
    W = torch.zeros(128, 128, dtype=torch.float16, device=dev)
    with pytest.raises(ValueError):  # more than 16 rows
        LinearGroup([x], [W], [torch.zeros(17, 128, dtype=torch.float16, device=dev)])
    with pytest.raises(ValueError):  # the 128 contract
        LinearGroup([x[:4, :100].contiguous()], [W[:, :100].contiguous()], [torch.zeros(4, 128, dtype=torch.float16, device=dev)])
    L = capi.lib
    h = ctypes.c_void_p()
    assert L.fg_group_create(capi.FG_OP_W8A16_NK, (capi.Problem * 1)(), 1, None, x.data_ptr(), 4096, ctypes.byref(h)) == capi.FG_ERR_PLAN
    assert L.fg_group_create(capi.FG_OP_F16_NK, None, 1, None, x.data_ptr(), 4096, ctypes.byref(h)) == capi.FG_ERR_NULL
    assert L.fg_group_create(capi.FG_OP_F16_NK, (capi.Problem * 1)(), 1, None, x.data_ptr(), 16, ctypes.byref(h)) == capi.FG_ERR_WORKSPACE
    assert L.fg_group_run(None, x.data_ptr(), 1 << 23, None) == capi.FG_ERR_NULL
