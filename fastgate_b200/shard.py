"""N-sharded linear layers over the GPUs of one box.

The output columns of ``C[M,N] = x[M,K] . W[N,K]^T`` are independent, so a large weight is
column-partitioned by N: rank r of g holds the rows ``W[r*N/g:(r+1)*N/g, :]`` (contiguous in
the NxK storage), receives the full activation, computes its slice ``C_r[M, N/g]`` with the
single-GPU kernels and the slices are assembled with one all-gather over NVLink
(``torch.distributed.all_gather_into_tensor``, NCCL).  The reference has no multi-GPU
path; this is the column-parallel scheme its README's "t2vi inference" linears call for.

Every shard keeps the kernels' contract (N/g % 128 == 0).  The gather delivers
``[g, M, N/g]``; ``assemble`` turns that into row-major ``[M, N]`` with one small copy.

``forward_push`` is the fused alternative: the kernel's epilogue stores every finished
128-column tile directly into the full ``C[M, N]`` of every rank through NVLink peer
mappings (torch symmetric memory) and bumps each rank's arrival counter; a one-thread wait
kernel then holds the stream until all ranks' tiles have landed.  No NCCL call, no
``[g,M,N/g] -> [M,N]`` copy.  Peer stores and atomics over NVLink mappings, or, where the fabric offers multicast mappings
(``FASTGATE_MULTIMEM=0|1`` overrides), one ``multimem.st`` / ``multimem.red`` per tile that the
NVSwitch replicates to every rank; never a TMA access to peer memory.  The number of tiles a rank
expects is kept on the device next to the counters (pushing kernels add to it, waits read it), so a
sequence of pushes and waits can be captured in a CUDA graph and replayed by every rank.

A layer's push buffers are rewritten by every rank as soon as that rank's next call on the layer
runs: call ``forward_push`` on a layer again only after every rank has consumed the previous
result (a barrier between rounds, or two layers / buffer sets used alternately).
"""
from __future__ import annotations

import os
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


class PushBuffers:
    """The full output ``[m_max, n_total]`` of one layer and an arrival counter, allocated in
    symmetric memory and exchanged with the other ranks of `group` (a collective call: every
    rank must create its PushBuffers in the same order)."""

    def __init__(self, m_max: int, n_total: int, device, group=None):
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = torch.device(device)
        self.n_total = n_total
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem

            grp = group if group is not None else dist.group.WORLD
            self.out = symm_mem.empty((m_max, n_total), dtype=torch.float16, device=self.device)
            self.flag = symm_mem.empty((16,), dtype=torch.int64, device=self.device)
            self.flag.zero_()
            torch.cuda.synchronize(self.device)
            self._h_out = symm_mem.rendezvous(self.out, grp)
            self._h_flag = symm_mem.rendezvous(self.flag, grp)
            self.c_ptrs = [int(p) for p in self._h_out.buffer_ptrs]
            self.flag_ptrs = [int(p) for p in self._h_flag.buffer_ptrs]
            # NVLink multicast mappings of the same allocations (0 where the fabric offers none):
            # with both, a tile is pushed by one multimem store / reduction instead of one per rank
            self.mc_out = int(getattr(self._h_out, "multicast_ptr", 0) or 0)
            self.mc_flag = int(getattr(self._h_flag, "multicast_ptr", 0) or 0)
            # Measured on B200 with 16- and 8-byte multicast stores, multicast against one store per rank:
            # 2 GPUs: 8192 x 8192 sweep, one call per launch, 9.5 against 8.9 TB/s; DiT stack with a push per
            # linear 2.35 against 2.62 ms per pass; as one grouped launch 13.0 against 12.8 TB/s.  4 GPUs (with
            # 4-byte multicast stores): 18.7 against 17.6 TB/s, 2.19 against 2.52 ms, 24.7 against 24.2 TB/s.
            # 8 GPUs (an earlier build): grouped 34.6 against 28.3 TB/s.
            # Default: on wherever the mappings exist; FASTGATE_MULTIMEM=0 / 1 forces it off / on.
            env = os.environ.get("FASTGATE_MULTIMEM")
            want = (env != "0")
            if not (want and self.mc_out and self.mc_flag):
                self.mc_out = self.mc_flag = 0
            dist.barrier(group)  # every counter is zero before anyone pushes
        else:
            self.out = torch.empty(m_max, n_total, dtype=torch.float16, device=self.device)
            self.flag = torch.zeros(16, dtype=torch.int64, device=self.device)
            self.c_ptrs = [self.out.data_ptr()]
            self.flag_ptrs = [self.flag.data_ptr()]
            self.mc_out = self.mc_flag = 0
        # Tiles EACH rank will have delivered to this rank once the calls enqueued so far have run.
        # The total lives on the device (word 8 of this rank's own flag array, which no other rank
        # touches): pushing kernels add to it, waits read it, and nothing in a launch changes from
        # call to call, so pushes and waits can be captured in a CUDA graph and replayed.
        self.target_ptr = self.flag_ptrs[self.rank] + 8 * 8


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

    # ---- fused all-gather -----------------------------------------------------------------
    def push_buffers(self, m_max: int, device, slot=0) -> "PushBuffers":
        """Collective: allocate (once per m_max and slot) a symmetric output of this layer."""
        key = ("push", m_max, slot)
        if key not in self._bufs:
            self._bufs[key] = PushBuffers(m_max, self.n_total, device, self.group)
        return self._bufs[key]

    def forward_push(self, x: torch.Tensor, wait: bool = True, after: Optional["PushBuffers"] = None, slot=0,
                     into: Optional["PushBuffers"] = None) -> torch.Tensor:
        """Full C[M, N] on every rank with the all-gather fused into the kernel's epilogue.

        wait=False: the caller makes sure the result is complete before touching it, either
        with `push_wait` or by handing this layer's buffers as `after=` to the next layer.
        after=: x is the pushed output of that earlier layer; the kernel streams its first
        weight tiles at once and reads x only when every rank's tiles of that layer have landed.
        slot=: which of the layer's output buffer sets to push into (any hashable; every rank must
        use the same sequence).  A set may be pushed into again only when every rank has consumed
        what it held: callers that keep several results alive, or have several steps in flight,
        rotate over slots.
        into=: push into these buffers (made by the caller with PushBuffers(m_max, n_total, device))
        instead of one of the layer's own sets; the same rule applies.
        """
        from . import ops

        if self.w.dtype != torch.float16:
            raise NotImplementedError("the fused all-gather is implemented for fp16 NxK weights")
        M = x.shape[0]
        pb = into if into is not None else self.push_buffers(max(M, 16), x.device, slot)
        if pb.n_total != self.n_total or pb.out.shape[0] < M:
            raise ValueError("fastgate_b200: push buffers do not fit this layer's output")
        wait_ptr, wait_target_ptr = (after.flag_ptrs[after.rank], after.target_ptr) if after is not None else (0, 0)
        # every pass over the weight delivers all of this rank's tiles once and adds them to the
        # buffers' running total on the device
        ops.linear_nk_push(x, self.w, pb.c_ptrs, pb.flag_ptrs, pb.rank, self.n_total, wait_ptr, 0,
                           pb.mc_out, pb.mc_flag, pb.target_ptr, wait_target_ptr)
        if wait:
            self.push_wait(pb)
        return pb.out[:M]

    def last_push(self, M: int, slot=0) -> "PushBuffers":
        """The buffers forward_push with M rows and this slot writes (to hand on as `after=`)."""
        return self._bufs[("push", max(M, 16), slot)]

    def push_wait(self, pb: "PushBuffers") -> None:
        from . import ops

        ops.push_wait_dev(pb.flag_ptrs[pb.rank], pb.world, pb.target_ptr, pb.device.index if pb.device.index is not None else 0)


def push_wait_all(pbs) -> None:
    """One wait kernel for several pushed outputs (up to 16 per launch): the current stream holds until
    every rank's tiles of all of them have landed here."""
    from . import ops

    pbs = list(pbs)
    for i in range(0, len(pbs), 16):
        part = pbs[i:i + 16]
        dev = part[0].device.index if part[0].device.index is not None else 0
        ops.push_wait_dev_many([pb.flag_ptrs[pb.rank] for pb in part], [pb.target_ptr for pb in part], part[0].world, dev)


def shard_weight(weight: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Rows [r*N/g, (r+1)*N/g) of an NxK weight (a view; call .contiguous() before upload)."""
    b, e = wl.shard_rows(weight.shape[0], world, rank)
    return weight[b:e]
