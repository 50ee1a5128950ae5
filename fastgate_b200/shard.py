"""N-sharded linear layers over the GPUs of one box.

The output columns of ``C[M,N] = x[M,K] . W[N,K]^T`` are independent, so a large weight is
column-partitioned by N: rank r of g holds the rows ``W[r*N/g:(r+1)*N/g, :]`` (contiguous in
the NxK storage), receives the full activation, computes its slice ``C_r[M, N/g]`` with the
single-GPU kernels and the slices are assembled with one all-gather over NVLink
(``torch.distributed.all_gather_into_tensor``, NCCL).  The reference has no multi-GPU
path; this is the column-parallel scheme its README's "t2vi inference" linears call for.

Every shard keeps the kernels' contract (N/g % 128 == 0).  The gather delivers
``[g, M, N/g]``; ``assemble`` turns that into row-major ``[M, N]`` with one small copy.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import workloads as wl


def _default_compute(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, scales=None) -> None:
    from . import ops

    if w.dtype == torch.int8:
        ops.fastgemv_int8(w, x, out, scales)
    else:
        ops.edgemm_m8n128k64x4_bt(x, w, out)


class ShardedLinear:
    """One linear layer whose NxK weight is split by rows (output columns) over the ranks
    of `group`.  `weight_shard` is this rank's ``[N/g, K]`` block."""

    def __init__(self, weight_shard: torch.Tensor, n_total: int, group=None,
                 scales_shard: Optional[torch.Tensor] = None,
                 compute: Callable = _default_compute):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n_total = n_total
        b, e = wl.shard_rows(n_total, self.world, self.rank)
        if weight_shard.shape[0] != e - b:
            raise ValueError(f"rank {self.rank} expects {e - b} weight rows, got {weight_shard.shape[0]}")
        self.w = weight_shard
        self.scales = scales_shard
        self.compute = compute
        self._bufs = {}

    def _buffers(self, M: int, device, dtype):
        key = (M, str(device), dtype)
        if key not in self._bufs:
            n_local = self.w.shape[0]
            local = torch.empty(M, n_local, device=device, dtype=dtype)
            gathered = torch.empty(self.world, M, n_local, device=device, dtype=dtype)
            full = torch.empty(M, self.n_total, device=device, dtype=dtype)
            self._bufs[key] = (local, gathered, full)
        return self._bufs[key]

    def forward_local(self, x: torch.Tensor) -> torch.Tensor:
        """This rank's slice C_r[M, N/g] (no communication)."""
        local, _, _ = self._buffers(x.shape[0], x.device, torch.float16)
        self.compute(x, self.w, local, self.scales)
        return local

    def gather(self, local: torch.Tensor) -> torch.Tensor:
        """All-gather of the slices into [g, M, N/g] (rank-major)."""
        _, gathered, _ = self._buffers(local.shape[0], local.device, local.dtype)
        if self.world == 1:
            gathered[0].copy_(local)
        else:
            dist.all_gather_into_tensor(gathered.view(-1), local.view(-1), group=self.group)
        return gathered

    def assemble(self, gathered: torch.Tensor) -> torch.Tensor:
        """[g, M, N/g] -> row-major C[M, N]."""
        _, _, full = self._buffers(gathered.shape[1], gathered.device, gathered.dtype)
        full.view(gathered.shape[1], self.world, -1).copy_(gathered.permute(1, 0, 2))
        return full

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        """Full C[M, N] on every rank."""
        return self.assemble(self.gather(self.forward_local(x)))


def shard_weight(weight: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Rows [r*N/g, (r+1)*N/g) of an NxK weight (a view; call .contiguous() before upload)."""
    b, e = wl.shard_rows(weight.shape[0], world, rank)
    return weight[b:e]
