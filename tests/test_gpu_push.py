"""The fused all-gather ("push") epilogue.

On one GPU: a single rank pushing into its own buffer, and two ranks emulated back to back
in one process with both full outputs on the same device (the waits come after both pushes
are enqueued, so nothing waits on a kernel that has not been launched).  With two or more
GPUs: real ranks as child processes over torch symmetric memory (skipped on a one-GPU box).
"""
import ctypes
import os
import socket

import numpy as np
import pytest
import torch

from fastgate_b200 import capi, workloads as wl
from oracle import oracle

from . import gpu_util as gu

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "needs a B200"
    return torch.device("cuda:0")


def _peers(world, rank, n_total, outs, flags):
    p = capi.Peers()
    p.world, p.rank, p.n_total = world, rank, n_total
    for q in range(world):
        p.C[q] = outs[q].data_ptr()
        p.flag[q] = flags[q].data_ptr()
    return p


@pytest.mark.parametrize("M,N,K", [(16, 1024, 2048), (5, 384, 1152), (33, 256, 512)])
def test_single_rank_push_equals_plain(M, N, K, dev):
    ws = gu.Workspace(dev)
    case = wl.Case("push1", wl.OP_NK, M, N, K, 700 + M)
    x, W = wl.make_activation(case).to(dev), wl.make_weight(case).to(dev)
    plain = torch.zeros(M, N, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, x, W, None, plain, M, N, K, ws) == capi.FG_OK
    out = torch.full((M, N), float("nan"), dtype=torch.float16, device=dev)
    flag = torch.zeros(8, dtype=torch.int64, device=dev)
    peers = _peers(1, 0, N, [out], [flag])
    L = capi.lib
    for rep in range(2):
        st = L.fg_gemm_f16_nk_push(x.data_ptr(), W.data_ptr(), M, N, K, ctypes.byref(peers), ws.ptr, ws.bytes, gu.stream())
        assert st == capi.FG_OK, capi.status_str(st)
        target = (rep + 1) * (N // 128) * capi.passes(capi.FG_OP_F16_NK, M, N, K)
        assert L.fg_push_wait(flag.data_ptr(), 1, target, ws.ptr, gu.stream()) == capi.FG_OK
        torch.cuda.synchronize()
        assert ws.status() == capi.FG_OK
        assert int(flag[0]) == target
        assert torch.equal(out.view(torch.int16), plain.view(torch.int16))


def test_two_ranks_emulated_on_one_gpu(dev):
    """Each rank's slice lands in both full outputs at its column offset; the counters add up."""
    ws = gu.Workspace(dev)
    M, N_local, K, world = 16, 512, 1024, 2
    case = wl.Case("push2", wl.OP_NK, M, N_local * world, K, 808)
    x, W = wl.make_activation(case), wl.make_weight(case)
    ref = oracle.gemm_nk(x.numpy(), W.numpy())
    xd = x.to(dev)
    outs = [torch.full((M, N_local * world), float("nan"), dtype=torch.float16, device=dev) for _ in range(world)]
    flags = [torch.zeros(8, dtype=torch.int64, device=dev) for _ in range(world)]
    L = capi.lib
    for r in range(world):
        Wr = W[r * N_local:(r + 1) * N_local].contiguous().to(dev)
        peers = _peers(world, r, N_local * world, outs, flags)
        st = L.fg_gemm_f16_nk_push(xd.data_ptr(), Wr.data_ptr(), M, N_local, K, ctypes.byref(peers), ws.ptr, ws.bytes, gu.stream())
        assert st == capi.FG_OK, capi.status_str(st)
    target = N_local // 128  # per source rank
    for r in range(world):
        assert L.fg_push_wait(flags[r].data_ptr(), world, target, ws.ptr, gu.stream()) == capi.FG_OK
    torch.cuda.synchronize()
    assert ws.status() == capi.FG_OK
    for r in range(world):
        assert flags[r][:world].tolist() == [target] * world
        oracle.check_tolerance(outs[r].cpu().numpy(), ref, f"rank {r}")
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))


def test_wait_times_out_without_hanging(dev):
    """A counter nobody bumps: the wait kernel gives up after its budget and reports it in the
    workspace status word; the context stays usable."""
    ws = gu.Workspace(dev)
    flag = torch.zeros(8, dtype=torch.int64, device=dev)
    L = capi.lib
    assert L.fg_push_wait(flag.data_ptr(), 2, 5, ws.ptr, gu.stream()) == capi.FG_OK
    torch.cuda.synchronize()
    assert ws.status() == capi.FG_ERR_TIMEOUT
    assert ws.status() == capi.FG_OK  # reading clears it
    x = torch.ones(1, 128, dtype=torch.float16, device=dev)
    W = torch.ones(128, 128, dtype=torch.float16, device=dev)
    out = torch.zeros(1, 128, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, x, W, None, out, 1, 128, 128, ws) == capi.FG_OK
    assert bool((out == 128).all())


def test_in_kernel_wait_on_an_earlier_layer(dev):
    """Layer B's activations are layer A's pushed output: B is enqueued with A's counters as its
    dependency, reads x only once they have reached the target and gives the chained result.
    With a target nobody will ever reach, B's wait gives up after its budget and says so."""
    ws = gu.Workspace(dev)
    M, N1, K1, N2 = 16, 512, 1024, 256
    ca = wl.Case("A", wl.OP_NK, M, N1, K1, 901)
    cb = wl.Case("B", wl.OP_NK, M, N2, N1, 902)
    x, Wa, Wb = wl.make_activation(ca).to(dev), wl.make_weight(ca).to(dev), wl.make_weight(cb).to(dev)
    ya_plain = torch.zeros(M, N1, dtype=torch.float16, device=dev)
    yb_plain = torch.zeros(M, N2, dtype=torch.float16, device=dev)
    assert gu.call(wl.OP_NK, x, Wa, None, ya_plain, M, N1, K1, ws) == capi.FG_OK
    assert gu.call(wl.OP_NK, ya_plain, Wb, None, yb_plain, M, N2, N1, ws) == capi.FG_OK
    ya = torch.zeros(M, N1, dtype=torch.float16, device=dev)
    yb = torch.zeros(M, N2, dtype=torch.float16, device=dev)
    fa = torch.zeros(8, dtype=torch.int64, device=dev)
    fb = torch.zeros(8, dtype=torch.int64, device=dev)
    L = capi.lib
    pa = _peers(1, 0, N1, [ya], [fa])
    pb = _peers(1, 0, N2, [yb], [fb])
    pb.wait_flags, pb.wait_target = fa.data_ptr(), N1 // 128
    assert L.fg_gemm_f16_nk_push(x.data_ptr(), Wa.data_ptr(), M, N1, K1, ctypes.byref(pa), ws.ptr, ws.bytes, gu.stream()) == capi.FG_OK
    assert L.fg_gemm_f16_nk_push(ya.data_ptr(), Wb.data_ptr(), M, N2, N1, ctypes.byref(pb), ws.ptr, ws.bytes, gu.stream()) == capi.FG_OK
    assert L.fg_push_wait(fb.data_ptr(), 1, N2 // 128, ws.ptr, gu.stream()) == capi.FG_OK
    torch.cuda.synchronize()
    assert ws.status() == capi.FG_OK
    assert torch.equal(yb.view(torch.int16), yb_plain.view(torch.int16))
    # unreachable target: bounded, reported, context intact
    pb.wait_target = 10 ** 9
    assert L.fg_gemm_f16_nk_push(ya.data_ptr(), Wb.data_ptr(), M, N2, N1, ctypes.byref(pb), ws.ptr, ws.bytes, gu.stream()) == capi.FG_OK
    torch.cuda.synchronize()
    assert ws.status() == capi.FG_ERR_TIMEOUT
    assert gu.call(wl.OP_NK, x, Wa, None, ya_plain, M, N1, K1, ws) == capi.FG_OK
    torch.cuda.synchronize()
    assert ws.status() == capi.FG_OK


def test_push_argument_checks(dev):
    ws = gu.Workspace(dev)
    x = torch.zeros(1, 128, dtype=torch.float16, device=dev)
    out = torch.zeros(1, 256, dtype=torch.float16, device=dev)
    flag = torch.zeros(8, dtype=torch.int64, device=dev)
    L = capi.lib
    good = _peers(2, 1, 256, [out, out], [flag, flag])
    assert L.fg_gemm_f16_nk_push(x.data_ptr(), x.data_ptr(), 1, 128, 128, None, ws.ptr, ws.bytes, gu.stream()) == capi.FG_ERR_NULL
    bad = _peers(2, 2, 256, [out, out], [flag, flag])
    assert L.fg_gemm_f16_nk_push(x.data_ptr(), x.data_ptr(), 1, 128, 128, ctypes.byref(bad), ws.ptr, ws.bytes, gu.stream()) == capi.FG_ERR_PLAN
    bad = _peers(2, 1, 384, [out, out], [flag, flag])
    assert L.fg_gemm_f16_nk_push(x.data_ptr(), x.data_ptr(), 1, 128, 128, ctypes.byref(bad), ws.ptr, ws.bytes, gu.stream()) == capi.FG_ERR_SHAPE
    bad = _peers(2, 1, 256, [out, out], [flag, flag])
    bad.flag[0] = None
    assert L.fg_gemm_f16_nk_push(x.data_ptr(), x.data_ptr(), 1, 128, 128, ctypes.byref(bad), ws.ptr, ws.bytes, gu.stream()) == capi.FG_ERR_NULL
    del good


# ---- real ranks ------------------------------------------------------------------------------
def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_main(rank, world, port, q):
    import torch.distributed as dist

    from fastgate_b200 import shard

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        ok = True
        for (M, N, K, seed) in [(16, 2048, 1024, 1), (3, 1024, 2304, 2), (20, 512, 512, 3)]:
            case = wl.Case("ranks", wl.OP_NK, M, N, K, seed)
            x, W = wl.make_activation(case), wl.make_weight(case)
            lin = shard.ShardedLinear(shard.shard_weight(W, world, rank).contiguous().to(dev), N)
            xd = x.to(dev)
            want = lin.forward(xd).clone()          # NCCL all-gather path
            for _ in range(2):
                got = lin.forward_push(xd)
                torch.cuda.synchronize()
                ok = ok and bool(torch.equal(got.view(torch.int16), want.view(torch.int16)))
            ref = oracle.gemm_nk(x.numpy(), W.numpy())
            ok = ok and oracle.tolerance_excess(got.cpu().numpy(), ref) <= 1.0
        # a two-layer chain: the second layer waits inside its kernel for the first one's tiles
        c1, c2 = wl.Case("l1", wl.OP_NK, 16, 1024, 512, 11), wl.Case("l2", wl.OP_NK, 16, 512, 1024, 12)
        x1, W1, W2 = wl.make_activation(c1), wl.make_weight(c1), wl.make_weight(c2)
        l1 = shard.ShardedLinear(shard.shard_weight(W1, world, rank).contiguous().to(dev), 1024)
        l2 = shard.ShardedLinear(shard.shard_weight(W2, world, rank).contiguous().to(dev), 512)
        want2 = l2.forward(l1.forward(x1.to(dev))).clone()
        for _ in range(3):
            y1 = l1.forward_push(x1.to(dev), wait=False)
            y2 = l2.forward_push(y1, wait=True, after=l1.last_push(16))
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(y2.view(torch.int16), want2.view(torch.int16)))
            dist.barrier()  # nobody starts the next round while a slower rank still reads y1
        import fastgate_b200 as fg
        ok = ok and fg.workspace_status(rank) == 0
        dist.barrier()
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_real_ranks_push_equals_nccl_gather(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    res = dict(q.get(timeout=10) for _ in range(world))
    assert res == {r: True for r in range(world)}
