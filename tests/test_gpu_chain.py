"""Dependent layer chain (fg_chain_*): a stack of projections that feed each other, one kernel.

Every layer is checked on its own against the CPU oracle, fed with the activations the chain
itself produced for it, so an error in one layer cannot hide behind the next.
"""
import numpy as np
import pytest
import torch

import fastgate_b200 as fg
from fastgate_b200 import capi, workloads as wl
from fastgate_b200.chain import LayerChain
from oracle import oracle

pytestmark = pytest.mark.gpu
ACTS = {"none": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3}


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "needs a B200"
    return torch.device("cuda:0")


def _weight(N, K, seed, layout, dev):
    W = wl.make_weight(wl.Case("c", wl.OP_NK, 1, N, K, seed))
    return W, (W if layout == "nk" else W.t().contiguous()).to(dev)


def _check_layers(layers, host_W, what):
    for i, (l, W) in enumerate(zip(layers, host_W)):
        x = l["x"].cpu().numpy()
        bias = l["bias"].cpu().numpy() if l.get("bias") is not None else None
        res = l["residual_in"].cpu().numpy() if l.get("residual_in") is not None else None
        ref = oracle.epilogue(oracle.gemm_nk(x, W.numpy()), bias, res, ACTS[l.get("act", "none")])
        oracle.check_tolerance(l["C"].cpu().numpy(), ref, f"{what} layer {i}")


def _dit_blocks(dev, M, hidden, blocks, layout, seed):
    """qkv -> out (+residual) -> up (bias, gelu) -> down (+residual), `blocks` times; the
    attention between qkv and out is replaced by taking the first `hidden` columns of qkv."""
    g = torch.Generator().manual_seed(seed)
    h = torch.randn(M, hidden, generator=g).half().to(dev)
    layers, host_W = [], []
    prev = -1
    for b in range(blocks):
        qkv = torch.full((M, 3 * hidden), float("nan"), dtype=torch.half, device=dev)
        h1 = torch.full((M, hidden), float("nan"), dtype=torch.half, device=dev)
        up = torch.full((M, 4 * hidden), float("nan"), dtype=torch.half, device=dev)
        h2 = torch.full((M, hidden), float("nan"), dtype=torch.half, device=dev)
        bias = (torch.randn(4 * hidden, generator=g) * 0.1).half().to(dev)
        shapes = [(3 * hidden, hidden), (hidden, hidden), (4 * hidden, hidden), (hidden, 4 * hidden)]
        Ws = [_weight(n, k, seed + 10 * b + j, layout, dev) for j, (n, k) in enumerate(shapes)]
        host_W += [w[0] for w in Ws]
        base = len(layers)
        layers += [
            dict(x=h, W=Ws[0][1], C=qkv, dep=prev),
            dict(x=qkv[:, :hidden], W=Ws[1][1], C=h1, dep=base, residual=h, residual_in=h),
            dict(x=h1, W=Ws[2][1], C=up, dep=base + 1, bias=bias, act="gelu_tanh"),
            dict(x=up, W=Ws[3][1], C=h2, dep=base + 2, residual=h1, residual_in=h1),
        ]
        h, prev = h2, base + 3
    return layers, host_W


def _strip(layers):
    return [{k: v for k, v in l.items() if k != "residual_in"} for l in layers]


@pytest.mark.parametrize("layout", ["nk", "kn"])
@pytest.mark.parametrize("M", [1, 16])
def test_dit_blocks_chain(layout, M, dev):
    layers, host_W = _dit_blocks(dev, M, 1152, 2, layout, 700 + M)
    chain = LayerChain(_strip(layers), weight_layout=layout)
    chain.run()
    torch.cuda.synchronize()
    assert chain.status() == capi.FG_OK
    _check_layers(layers, host_W, f"chain {layout} M={M}")
    first = [l["C"].clone() for l in layers]
    for l in layers:
        l["C"].fill_(float("nan"))
    chain.run()
    chain.run()  # back to back: the second run starts while nothing is left of the first
    torch.cuda.synchronize()
    assert chain.status() == capi.FG_OK
    for a, l in zip(first, layers):
        assert torch.equal(a.view(torch.int16), l["C"].view(torch.int16)), "two runs differ bitwise"


def test_chain_equals_per_layer_operator(dev):
    """The chain and one fused call per layer agree within one rounding step per layer input
    (only the stream-K cuts differ); checked layer by layer on the chain's own inputs."""
    layers, _ = _dit_blocks(dev, 8, 1024, 1, "nk", 900)
    LayerChain(_strip(layers)).run()
    torch.cuda.synchronize()
    for i, l in enumerate(layers):
        C = torch.empty_like(l["C"])
        fg.linear_fused(l["x"].contiguous(), l["W"], C, bias=l.get("bias"),
                        residual=l["residual_in"] if l.get("residual_in") is not None else None,
                        act=l.get("act", "none"))
        ref = C.float().cpu().numpy()
        assert oracle.tolerance_excess(l["C"].cpu().numpy(), ref) <= 0.1, f"layer {i}"


def test_small_and_ragged_layers(dev):
    """Layers with fewer stages than CTAs, ragged last stages, independent layers mixed in, a
    layer that depends on a layer further back, and a ping-pong buffer that is overwritten."""
    M = 5
    g = torch.Generator().manual_seed(5)
    a = torch.randn(M, 384, generator=g).half().to(dev)
    b = torch.randn(M, 896, generator=g).half().to(dev)
    dims = [(128, 384), (256, 896), (640, 128), (384, 640), (128, 256), (4096, 384)]
    Ws = [_weight(n, k, 40 + i, "nk", dev) for i, (n, k) in enumerate(dims)]
    out = [torch.full((M, n), float("nan"), dtype=torch.half, device=dev) for n, _ in dims]
    layers = [
        dict(x=a, W=Ws[0][1], C=out[0]),                       # 0: a -> 128
        dict(x=b, W=Ws[1][1], C=out[1]),                       # 1: independent
        dict(x=out[0], W=Ws[2][1], C=out[2], dep=0, act="silu"),   # 2: <- 0
        dict(x=out[2], W=Ws[3][1], C=out[3], dep=2),           # 3: <- 2
        dict(x=out[1], W=Ws[4][1], C=out[4], dep=1),           # 4: <- 1 (further back)
        dict(x=out[3], W=Ws[5][1], C=out[5], dep=3),           # 5: wide layer after tiny ones
    ]
    chain = LayerChain(layers)
    chain.run()
    torch.cuda.synchronize()
    assert chain.status() == capi.FG_OK
    _check_layers(layers, [w[0] for w in Ws], "ragged")


def test_chain_argument_checks(dev):
    x = torch.zeros(4, 128, dtype=torch.half, device=dev)
    W = torch.zeros(128, 128, dtype=torch.half, device=dev)
    C = torch.zeros(4, 128, dtype=torch.half, device=dev)
    with pytest.raises(ValueError):
        LayerChain([dict(x=x, W=W, C=C, dep=0)])          # a layer cannot depend on itself
    with pytest.raises(ValueError):
        LayerChain([dict(x=x, W=W, C=C), dict(x=C, W=W, C=x, dep=5)])
    with pytest.raises(ValueError):
        LayerChain([dict(x=torch.zeros(17, 128, dtype=torch.half, device=dev), W=W,
                         C=torch.zeros(17, 128, dtype=torch.half, device=dev))])
    with pytest.raises(ValueError):
        LayerChain([dict(x=x[:, :100], W=W, C=C)])
