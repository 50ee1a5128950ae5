"""Host-side logic of the N-sharded path with world_size 2 and 4 on CPU ranks (gloo).

The product has no CPU kernels, so the per-shard product is injected as a torch CPU matmul
here; what is under test is the partitioning, the all-gather and the assembly of C[M,N]."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fastgate_b200 import shard, workloads as wl


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _cpu_compute(x, w, out, scales=None):
    r = x.float() @ w.float().t()
    if scales is not None:
        r = r * scales.float()
    out.copy_(r.half())


def _worker(rank, world, port, N, K, M, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        case = wl.Case("shard", wl.OP_NK, M, N, K, 42)
        W, x = wl.make_weight(case), wl.make_activation(case)  # identical on every rank (seeded)
        lin = shard.ShardedLinear(shard.shard_weight(W, world, rank).contiguous(), N, compute=_cpu_compute)
        full = lin.forward(x)
        want = (x.float() @ W.float().t()).half()
        ok = bool(torch.equal(full, want))
        local = lin.forward_local(x)
        b, e = wl.shard_rows(N, world, rank)
        ok = ok and bool(torch.equal(local, want[:, b:e]))
        # mismatched shard height is refused on the host
        try:
            shard.ShardedLinear(W[: (e - b) // 2].contiguous(), N, compute=_cpu_compute)
            ok = False
        except ValueError:
            pass
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,N", [(2, 1024), (4, 1536)])
def test_sharded_linear_gloo(world, N):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, N, 256, 5, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    res = dict(q.get(timeout=10) for _ in range(world))
    assert res == {r: True for r in range(world)}


def test_shard_rows():
    assert wl.shard_rows(9216, 8, 3) == (3456, 4608)
    assert wl.shard_rows(3072, 8, 7) == (2688, 3072)
    assert wl.shard_rows(12288, 4, 0) == (0, 3072)
    for n, g in [(3072, 16), (1000, 2), (384, 4)]:
        with pytest.raises(ValueError):
            wl.shard_rows(n, g, 0)
    # every DiT projection splits over 1, 2, 4 and 8 GPUs
    for _, n, _k in wl.DIT_LINEARS:
        for g in (1, 2, 4, 8):
            cuts = [wl.shard_rows(n, g, r) for r in range(g)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(cuts, cuts[1:]))
            assert all((e - b) % 128 == 0 for b, e in cuts)


def test_workload_catalogue():
    c1, c2, c3, c4, c5 = wl.cfg1(), wl.cfg2(), wl.cfg3(), wl.cfg4(), wl.cfg5()
    assert c1[0].algorithmic_bytes == 33_685_504
    assert [c.M for c in c2] == [1, 2, 4, 8, 16] and c2[0].algorithmic_bytes == 134_250_496
    assert c2[-1].algorithmic_bytes == 134_742_016
    assert c3[0].algorithmic_bytes == 90_207_744 == c3[1].algorithmic_bytes
    assert c4[0].algorithmic_bytes == 235_012_096 and c4[1].algorithmic_bytes == 235_528_192
    assert len(c5) == 160 and sum(c.weight_bytes for c in c5) == 9_059_696_640
    w = wl.make_weight(c1[0])
    assert w.shape == (4096, 4096) and w.dtype == torch.float16
    w4 = wl.make_weight(wl.Case("t", wl.OP_W8, 1, 256, 128, 1))
    assert w4.dtype == torch.int8 and int(w4.min()) >= -127 and int(w4.max()) <= 127
    s = wl.make_scales(wl.Case("t", wl.OP_W8, 1, 256, 128, 1))
    assert float(s.min()) >= 0.5 / 127 * 0.99 and float(s.max()) <= 1.5 / 127 * 1.01
    # determinism of the generators
    assert torch.equal(wl.make_activation(c2[0]), wl.make_activation(c2[0]))
