"""Grouped launch: many independent small-batch linears as one persistent kernel.

    grp = LinearGroup(xs, Ws, Cs)      # lists of CUDA fp16 tensors: x[M,K] (M <= 16), W[N,K], C[M,N]
    grp.run()                          # one launch on the current stream; repeat at will

The stages of all problems form one work list that is dealt evenly to the SMs, so launch cost,
DRAM ramp and the tail of split tiles are paid once per group.  Inputs of the grouped problems
must not depend on each other's outputs.  Thin ctypes layer over fg_group_* of the C ABI.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import torch

from . import capi


class LinearGroup:
    def __init__(self, xs: Sequence[torch.Tensor], Ws: Sequence[torch.Tensor], Cs: Optional[Sequence[torch.Tensor]],
                 weight_layout: str = "nk", peer_C_ptrs: Optional[Sequence[Sequence[int]]] = None,
                 flag_ptrs: Optional[Sequence[int]] = None, rank: int = 0, n_totals: Optional[Sequence[int]] = None,
                 mc_C_ptrs: Optional[Sequence[int]] = None, mc_flag_ptr: int = 0, target_dev_ptr: int = 0):
        assert weight_layout in ("nk", "kn")
        n = len(xs)
        assert n == len(Ws) and n > 0
        self.device = xs[0].device
        self._keep = (list(xs), list(Ws), list(Cs) if Cs is not None else None)
        op = capi.FG_OP_F16_NK if weight_layout == "nk" else capi.FG_OP_F16_KN
        probs = (capi.Problem * n)()
        for i, (x, W) in enumerate(zip(xs, Ws)):
            for t in (x, W):
                if not (t.is_cuda and t.dtype == torch.float16 and t.is_contiguous()):
                    raise ValueError("fastgate_b200: grouped operands must be contiguous CUDA fp16 tensors")
            M, K = x.shape
            N = W.shape[0] if weight_layout == "nk" else W.shape[1]
            probs[i].x, probs[i].W = x.data_ptr(), W.data_ptr()
            probs[i].M, probs[i].N, probs[i].K = M, N, K
            if peer_C_ptrs is None:
                C = Cs[i]
                if C.numel() != M * N or C.dtype != torch.float16 or not C.is_contiguous():
                    raise ValueError("fastgate_b200: output must be a contiguous fp16 tensor of M*N elements")
                probs[i].C = C.data_ptr()
            else:
                for r, ptr in enumerate(peer_C_ptrs[i]):
                    probs[i].peer_C[r] = ptr
                probs[i].n_total = n_totals[i]
                if mc_C_ptrs is not None and mc_C_ptrs[i]:
                    probs[i].mc_C = mc_C_ptrs[i]  # multicast mapping of the same outputs
        peers = None
        if peer_C_ptrs is not None:
            peers = capi.Peers()
            peers.world, peers.rank = len(flag_ptrs), rank
            for r, ptr in enumerate(flag_ptrs):
                peers.flag[r] = ptr
            if mc_flag_ptr and mc_C_ptrs is not None:
                peers.mc_flag = mc_flag_ptr
            # this rank's running total of tiles per source (device memory): every run adds self.tiles,
            # so a run followed by push_wait_dev can be captured in a graph and replayed
            peers.target_dev = target_dev_ptr or None
        L = capi.lib
        self._table = torch.empty(int(L.fg_group_table_bytes(n)), dtype=torch.uint8, device=self.device)
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            st = L.fg_group_create(op, probs, n, ctypes.byref(peers) if peers is not None else None,
                                   self._table.data_ptr(), self._table.numel(), ctypes.byref(handle))
        if st != capi.FG_OK:
            raise (ValueError if st == capi.FG_ERR_SHAPE else RuntimeError)(f"fastgate_b200: {capi.status_str(st)}")
        self._handle = handle
        self.tiles = int(L.fg_group_tiles(handle))
        self._ws_bytes = capi.workspace_bytes(128 * self.tiles)
        self._ws = torch.zeros(self._ws_bytes, dtype=torch.uint8, device=self.device)

    def run(self) -> None:
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        with torch.cuda.device(self.device):
            st = capi.lib.fg_group_run(self._handle, self._ws.data_ptr(), self._ws_bytes, stream)
        if st != capi.FG_OK:
            raise RuntimeError(f"fastgate_b200: {capi.status_str(st)}")

    def status(self) -> int:
        v = ctypes.c_int(-1)
        stream = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        capi.lib.fg_workspace_status(self._ws.data_ptr(), ctypes.byref(v), stream)
        return v.value

    def __del__(self):
        h = getattr(self, "_handle", None)
        if h:
            capi.lib.fg_group_destroy(h)
            self._handle = None
