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


@pytest.mark.parametrize("M,N,K", [(16, 1024, 2048), (5, 384, 1152), (33, 256, 512), (20, 512, 1024), (70, 256, 2304), (1, 512, 4096)])
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
        # the contract of the header: a call adds N_local/128 * ceil(M/64) to the rank's counter
        target = (rep + 1) * (N // 128) * -(-M // 64)
        assert L.fg_push_wait(flag.data_ptr(), 1, target, ws.ptr, gu.stream()) == capi.FG_OK
        torch.cuda.synchronize()
        assert ws.status() == capi.FG_OK
        assert int(flag[0]) == target
        if M > 2:  # one or two rows: the plain entry point runs the row-split GEMV kernel, the push a tiled one
            assert torch.equal(out.view(torch.int16), plain.view(torch.int16))
        else:
            assert float((out.float() - plain.float()).abs().max()) <= 2e-2


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


def test_device_resident_targets_replay_in_a_graph(dev):
    """With the running totals kept on the device nothing in a launch changes from call to call: two
    chained layers and the closing wait are captured once and replayed; every replay adds the calls'
    tiles to the totals and leaves the same bits."""
    ws = gu.Workspace(dev)
    M, K1, N1, N2 = 16, 512, 1024, 768
    c1, c2 = wl.Case("gA", wl.OP_NK, M, N1, K1, 901), wl.Case("gB", wl.OP_NK, M, N2, N1, 902)
    x, W1, W2 = wl.make_activation(c1).to(dev), wl.make_weight(c1).to(dev), wl.make_weight(c2).to(dev)
    y1 = torch.zeros(M, N1, dtype=torch.float16, device=dev)
    y2 = torch.zeros(M, N2, dtype=torch.float16, device=dev)
    want1, want2 = torch.zeros_like(y1), torch.zeros_like(y2)
    assert gu.call(wl.OP_NK, x, W1, None, want1, M, N1, K1, ws) == capi.FG_OK
    assert gu.call(wl.OP_NK, want1, W2, None, want2, M, N2, N1, ws) == capi.FG_OK
    f1 = torch.zeros(16, dtype=torch.int64, device=dev)  # counters [0, 8), the running total in word 8
    f2 = torch.zeros(16, dtype=torch.int64, device=dev)
    pa, pb = _peers(1, 0, N1, [y1], [f1]), _peers(1, 0, N2, [y2], [f2])
    pa.target_dev = f1.data_ptr() + 64
    pb.target_dev = f2.data_ptr() + 64
    pb.wait_flags, pb.wait_target_dev = f1.data_ptr(), f1.data_ptr() + 64
    L = capi.lib
    side = torch.cuda.Stream()

    def enqueue():
        s = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert L.fg_gemm_f16_nk_push(x.data_ptr(), W1.data_ptr(), M, N1, K1, ctypes.byref(pa), ws.ptr, ws.bytes, s) == capi.FG_OK
        assert L.fg_gemm_f16_nk_push(y1.data_ptr(), W2.data_ptr(), M, N2, N1, ctypes.byref(pb), ws.ptr, ws.bytes, s) == capi.FG_OK
        assert L.fg_push_wait_dev(f2.data_ptr(), 1, f2.data_ptr() + 64, ws.ptr, s) == capi.FG_OK

    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        enqueue()  # eager
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            enqueue()
            enqueue()
    runs = 1
    for _ in range(3):
        y1.fill_(float("nan"))
        y2.fill_(float("nan"))
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        runs += 2
        assert ws.status() == capi.FG_OK
        assert f1[:9].tolist() == [runs * (N1 // 128)] + [0] * 7 + [runs * (N1 // 128)]
        assert f2[:9].tolist() == [runs * (N2 // 128)] + [0] * 7 + [runs * (N2 // 128)]
        assert torch.equal(y1.view(torch.int16), want1.view(torch.int16))
        assert torch.equal(y2.view(torch.int16), want2.view(torch.int16))
    # both outputs closed by one wait kernel
    fl = (ctypes.c_void_p * 2)(f1.data_ptr(), f2.data_ptr())
    tg = (ctypes.c_void_p * 2)(f1.data_ptr() + 64, f2.data_ptr() + 64)
    assert L.fg_push_wait_dev_many(fl, tg, 2, 1, ws.ptr, gu.stream()) == capi.FG_OK
    torch.cuda.synchronize()
    assert ws.status() == capi.FG_OK
    assert L.fg_push_wait_dev_many(fl, tg, 17, 1, ws.ptr, gu.stream()) == capi.FG_ERR_PLAN
    # a wait on a total nobody will reach gives up and says so
    f2[8] += 1
    assert L.fg_push_wait_dev_many(fl, tg, 2, 1, ws.ptr, gu.stream()) == capi.FG_OK
    torch.cuda.synchronize()
    assert ws.status() == capi.FG_ERR_TIMEOUT
    assert L.fg_push_wait_dev(f2.data_ptr(), 1, f2.data_ptr() + 64, ws.ptr, gu.stream()) == capi.FG_OK
    torch.cuda.synchronize()
    assert ws.status() == capi.FG_ERR_TIMEOUT
    assert L.fg_push_wait_dev(f2.data_ptr(), 1, None, ws.ptr, gu.stream()) == capi.FG_ERR_NULL
    assert L.fg_push_wait_dev(f2.data_ptr(), 1, f2.data_ptr() + 4, ws.ptr, gu.stream()) == capi.FG_ERR_ALIGN


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


def _rank_main(rank, world, port, q, multimem):
    import torch.distributed as dist

    from fastgate_b200 import shard
    from fastgate_b200.group import LinearGroup
    import fastgate_b200 as fg

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    if multimem is not None:
        os.environ["FASTGATE_MULTIMEM"] = multimem  # "0" / "1": one store per rank / multimem.st + multimem.red
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        ok, used_mc = True, False
        # one row to more than one 64-row pass, sizes where a rank's shard is a single tile and many
        for (M, N, K, seed) in [(16, 2048, 1024, 1), (3, 1024, 2304, 2), (20, 1024, 512, 3), (1, 2048, 4096, 4), (70, 1024, 512, 5)]:
            case = wl.Case("ranks", wl.OP_NK, M, N, K, seed)
            x, W = wl.make_activation(case), wl.make_weight(case)
            lin = shard.ShardedLinear(shard.shard_weight(W, world, rank).contiguous().to(dev), N)
            xd = x.to(dev)
            # the NCCL all-gather path runs the row-split GEMV kernel for one or two rows, the push a
            # tiled kernel: bitwise agreement from three rows on, the tolerance below that
            want = lin.forward(xd).clone()
            for _ in range(2):
                got = lin.forward_push(xd)
                torch.cuda.synchronize()
                if M > 2:
                    ok = ok and bool(torch.equal(got.view(torch.int16), want.view(torch.int16)))
                dist.barrier()  # nobody pushes again while a slower rank still reads
            used_mc = used_mc or bool(lin.last_push(M).mc_out)
            ref = oracle.gemm_nk(x.numpy(), W.numpy())
            ok = ok and oracle.tolerance_excess(got.cpu().numpy(), ref) <= 1.0
        # a two-layer chain: the second layer waits inside its kernel for the first one's tiles
        c1, c2 = wl.Case("l1", wl.OP_NK, 16, 1024, 512, 11), wl.Case("l2", wl.OP_NK, 16, 1024, 1024, 12)
        x1, W1, W2 = wl.make_activation(c1), wl.make_weight(c1), wl.make_weight(c2)
        l1 = shard.ShardedLinear(shard.shard_weight(W1, world, rank).contiguous().to(dev), 1024)
        l2 = shard.ShardedLinear(shard.shard_weight(W2, world, rank).contiguous().to(dev), 1024)
        want2 = l2.forward(l1.forward(x1.to(dev))).clone()
        for _ in range(3):
            y1 = l1.forward_push(x1.to(dev), wait=False)
            y2 = l2.forward_push(y1, wait=True, after=l1.last_push(16))
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(y2.view(torch.int16), want2.view(torch.int16)))
            dist.barrier()  # nobody starts the next round while a slower rank still reads y1
        # two independent pushes closed by one wait kernel
        for _ in range(2):
            ya = l1.forward_push(x1.to(dev), wait=False, slot="a")
            yb = l2.forward_push(want2, wait=False, slot="b")
            shard.push_wait_all([l1.last_push(16, "a"), l2.last_push(16, "b")])
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(ya.view(torch.int16), l1.forward(x1.to(dev)).view(torch.int16)))
            ok = ok and bool(torch.equal(yb.view(torch.int16), l2.forward(want2).view(torch.int16)))
            dist.barrier()
        # the same chain captured once per rank and replayed: the tile totals live on the device
        xg = x1.to(dev)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            y1 = l1.forward_push(xg, wait=False, slot="graph")  # eager: allocates this slot's buffers on every rank
            y2 = l2.forward_push(y1, wait=True, after=l1.last_push(16, "graph"), slot="graph")
            torch.cuda.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):  # NCCL's watchdog thread may call into CUDA meanwhile
                y1 = l1.forward_push(xg, wait=False, slot="graph")
                y2 = l2.forward_push(y1, wait=True, after=l1.last_push(16, "graph"), slot="graph")
        for _ in range(3):
            y2.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()  # every rank's copy is blank before anyone replays
            graph.replay()
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(y2.view(torch.int16), want2.view(torch.int16)))
            dist.barrier()
        # a grouped launch that pushes: three independent projections as one kernel per rank
        gcases = [wl.Case("g0", wl.OP_NK, 16, 1024, 512, 21), wl.Case("g1", wl.OP_NK, 5, 2048, 1024, 22), wl.Case("g2", wl.OP_NK, 16, 1024, 2304, 23)]
        gx = [wl.make_activation(c).to(dev) for c in gcases]
        gW = [wl.make_weight(c) for c in gcases]
        glin = [shard.ShardedLinear(shard.shard_weight(W, world, rank).contiguous().to(dev), c.N) for W, c in zip(gW, gcases)]
        gwant = [lin.forward(x).clone() for lin, x in zip(glin, gx)]
        pbs = [lin.push_buffers(16, dev) for lin in glin]
        gflag = shard.PushBuffers(16, 128, dev)
        grp = LinearGroup(gx, [lin.w for lin in glin], None, peer_C_ptrs=[pb.c_ptrs for pb in pbs], flag_ptrs=gflag.flag_ptrs,
                          rank=rank, n_totals=[c.N for c in gcases], mc_C_ptrs=[pb.mc_out for pb in pbs], mc_flag_ptr=gflag.mc_flag,
                          target_dev_ptr=gflag.target_ptr)
        for _ in range(2):
            for pb in pbs:
                pb.out.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            grp.run()
            fg.push_wait_dev(gflag.flag_ptrs[rank], world, gflag.target_ptr, rank)
            torch.cuda.synchronize()
            # the grouped kernel cuts the K sums at other places than the single calls behind `gwant`:
            # one fp16 rounding step apart from them, and bit-identical on every rank
            for pb, want, c in zip(pbs, gwant, gcases):
                got_g = pb.out[:c.M]
                ok = ok and oracle.tolerance_excess(got_g.cpu().numpy(), want.cpu().numpy().astype(np.float32)) <= 0.1
                lo, hi = got_g.view(torch.int16).to(torch.int32), got_g.view(torch.int16).to(torch.int32)  # NCCL has no int16
                dist.all_reduce(lo, op=dist.ReduceOp.MIN)
                dist.all_reduce(hi, op=dist.ReduceOp.MAX)
                ok = ok and bool(torch.equal(lo, hi))
            ok = ok and grp.status() == 0
            dist.barrier()
        ok = ok and fg.workspace_status(rank) == 0
        dist.barrier()
        q.put((rank, ok, used_mc))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,multimem", [(2, "0"), (2, "1"), (4, "0"), (4, "1"), (8, "0"), (8, None)],
                         ids=["2-peer-stores", "2-multimem", "4-peer-stores", "4-multimem", "8-peer-stores", "8-default"])
def test_real_ranks_push_equals_nccl_gather(world, multimem):
    """Real ranks over torch symmetric memory: single calls, a dependent pair, a grouped launch; with one
    store per rank and with multimem (the default wherever the fabric offers multicast mappings).  Every rank leaves through a barrier."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, world, port, q, multimem)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        assert p.exitcode == 0
    res = [q.get(timeout=10) for _ in range(world)]
    assert {r: ok for r, ok, _ in res} == {r: True for r in range(world)}
    if multimem != "0":
        # the fabric may offer no multicast mapping (then the plain path ran and that is what was checked)
        print(f"world {world}: multimem path used: {all(mc for _, _, mc in res)}")
