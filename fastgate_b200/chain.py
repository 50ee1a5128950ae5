"""Dependent layer chain: a stack of small-batch linears that feed each other, one kernel.

    chain = LayerChain([
        dict(x=h0, W=W_qkv, C=qkv),
        dict(x=qkv[:, :3072], W=W_out, C=h1, dep=0, residual=h0),
        dict(x=h1, W=W_up, C=up, dep=1, bias=b_up, act="gelu_tanh"),
        dict(x=up, W=W_down, C=h2, dep=2, residual=h1),
    ])
    chain.run()        # one cooperative launch on the current stream; repeat at will

Every layer is C = act(x . W^T + bias) + residual with x [M, K] (M <= 16), W [N, K] ("nk") or
[K, N] ("kn").  x, C and residual may be column slices of wider row-major buffers (unit stride in
the last dimension).  `dep` names the earlier layer whose output x reads (-1: ready at launch).
The kernel streams the next layer's weights while the previous layer's last tiles drain; only
the activations wait.  Thin ctypes layer over fg_chain_* of the C ABI.
"""
from __future__ import annotations

import ctypes
from typing import Mapping, Sequence

import torch

from . import capi


def _rows(t: torch.Tensor, what: str):
    if not (t.is_cuda and t.dtype == torch.float16 and t.dim() == 2 and t.stride(1) == 1):
        raise ValueError(f"fastgate_b200: {what} must be a 2-D CUDA fp16 tensor with unit stride in the last dimension")
    return t.stride(0)


class LayerChain:
    def __init__(self, layers: Sequence[Mapping], weight_layout: str = "nk"):
        assert weight_layout in ("nk", "kn")
        n = len(layers)
        if n == 0:
            raise ValueError("fastgate_b200: empty chain")
        self.device = layers[0]["x"].device
        self._keep = [dict(l) for l in layers]
        op = capi.FG_OP_F16_NK if weight_layout == "nk" else capi.FG_OP_F16_KN
        tab = (capi.Layer * n)()
        for i, l in enumerate(layers):
            x, W, C = l["x"], l["W"], l["C"]
            ldx, ldc = _rows(x, "x"), _rows(C, "C")
            if not (W.is_cuda and W.dtype == torch.float16 and W.is_contiguous()):
                raise ValueError("fastgate_b200: W must be a contiguous CUDA fp16 tensor")
            M, K = x.shape
            N = W.shape[0] if weight_layout == "nk" else W.shape[1]
            if (W.shape[1] if weight_layout == "nk" else W.shape[0]) != K or tuple(C.shape) != (M, N):
                raise ValueError("fastgate_b200: chain layer shapes do not agree")
            e = tab[i]
            e.x, e.W, e.C = x.data_ptr(), W.data_ptr(), C.data_ptr()
            e.ldx, e.ldc = ldx, ldc
            e.M, e.N, e.K = M, N, K
            bias, res = l.get("bias"), l.get("residual")
            if bias is not None:
                if not (bias.is_cuda and bias.dtype == torch.float16 and bias.is_contiguous() and bias.numel() == N):
                    raise ValueError("fastgate_b200: bias must be a contiguous CUDA fp16 tensor of N elements")
                e.bias = bias.data_ptr()
            if res is not None:
                e.ldr = _rows(res, "residual")
                if tuple(res.shape) != (M, N):
                    raise ValueError("fastgate_b200: residual must be [M, N]")
                e.residual = res.data_ptr()
            e.act = capi.ACT[l.get("act", "none") or "none"]
            e.dep = int(l.get("dep", -1))
        L = capi.lib
        self._table = torch.empty(int(L.fg_chain_table_bytes(n)), dtype=torch.uint8, device=self.device)
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            st = L.fg_chain_create(op, tab, n, self._table.data_ptr(), self._table.numel(), ctypes.byref(handle))
        if st != capi.FG_OK:
            raise (ValueError if st in (capi.FG_ERR_SHAPE, capi.FG_ERR_PLAN, capi.FG_ERR_ALIGN) else RuntimeError)(
                f"fastgate_b200: {capi.status_str(st)}")
        self._handle = handle
        self._ws_bytes = int(L.fg_chain_workspace_bytes(handle))
        self._ws = torch.zeros(self._ws_bytes, dtype=torch.uint8, device=self.device)

    def run(self) -> None:
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        with torch.cuda.device(self.device):
            st = capi.lib.fg_chain_run(self._handle, self._ws.data_ptr(), self._ws_bytes, stream)
        if st != capi.FG_OK:
            raise RuntimeError(f"fastgate_b200: {capi.status_str(st)}")

    def trace(self) -> torch.Tensor:
        """Trace of the last run made with capi.lib.fg_trace_enable(1): int64 [layers, grid, 8]
        (ns: activations ready, first stage landed, last stage committed, last tile handed on, last
        partial written, its ticket back, its reduction loaded; contributors if this CTA reduced)."""
        L = capi.lib
        grid, off = int(L.fg_chain_grid(self._handle)), int(L.fg_chain_trace_offset(self._handle))
        n = len(self._keep) * grid * 8
        torch.cuda.synchronize(self.device)
        return self._ws[off:off + 8 * n].view(torch.int64).view(len(self._keep), grid, 8).cpu()

    def status(self) -> int:
        v = ctypes.c_int(-1)
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        capi.lib.fg_workspace_status(self._ws.data_ptr(), ctypes.byref(v), stream)
        return v.value

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h:
            capi.lib.fg_chain_destroy(h)
            self._handle = None


def _main() -> None:
    """python -m fastgate_b200.chain [--layers 10 --N 8192 --K 8192 --M 16]: per-layer timeline of a
    stack of dependent square layers (K = N), minimum / median / maximum over the CTAs, in
    microseconds after the layer's activations became readable for the first CTA."""
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=10)
    ap.add_argument("--N", type=int, default=8192)
    ap.add_argument("--M", type=int, default=16)
    ap.add_argument("--show", type=int, default=4, help="layers to print (from the fourth on)")
    a = ap.parse_args()
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(1)
    Ws = [(torch.randn(a.N, a.N, device=dev, generator=g) / a.N ** 0.5).half() for _ in range(a.layers)]
    bufs = [torch.randn(a.M, a.N, device=dev, generator=g).half()]
    bufs += [torch.empty(a.M, a.N, dtype=torch.half, device=dev) for _ in range(a.layers)]
    ch = LayerChain([dict(x=bufs[i], W=Ws[i], C=bufs[i + 1], dep=i - 1) for i in range(a.layers)])
    for _ in range(3):
        ch.run()
    torch.cuda.synchronize()
    capi.lib.fg_trace_enable(1)
    try:
        ch.run()
        t = ch.trace().double()
    finally:
        capi.lib.fg_trace_enable(0)
    names = ["activations ready", "first stage landed", "last stage committed", "last partial written",
             "its ticket back", "reduction loaded", "last tile handed on"]
    cols = [0, 1, 2, 4, 5, 6, 3]
    first = min(3, a.layers - 1)
    for layer in range(first, min(a.layers, first + a.show)):
        t0 = t[layer, :, 0].min()
        print(f"layer {layer} (starts {float(t0 - t[first, :, 0].min()) / 1e3:.2f} us after layer {first}):")
        for name, c in zip(names, cols):
            v = t[layer, :, c]
            v = (v[v > 0] - t0) / 1e3
            if len(v):
                print(f"  {name:22s} min {float(v.min()):6.2f}  med {float(v.median()):6.2f}  max {float(v.max()):6.2f}   ({len(v)} CTAs)")
    if ch.status() != capi.FG_OK:
        raise SystemExit("the chain kernel reported a timeout")


if __name__ == "__main__":
    _main()
