"""Seeded synthetic inputs for the benchmark configurations.

The reference ships no data: its scripts draw random matrices at run time
(script/standard-test.py:122-143, script/benchmark.py:13-14).  These generators fix the
shapes, distributions and seeds so that the CPU oracle, the GPU kernels and the reference
kernels all see identical bits.  Everything is generated on the CPU with a
``torch.Generator`` and copied to the device by the caller.

  weights      N(0, 1/sqrt(K)) -> fp16        seed S
  activations  N(0, 1)         -> fp16        seed S + 100000
  int8 weights uniform integers in [-127, 127]
  int8 scales  uniform [0.5, 1.5] / 127 -> fp16   seed S + 200000
  int4 weights uniform bytes (two nibbles 0..15 each), zero point 8
  int4 scales  uniform [0.5, 1.5] / 8 -> fp16, [N, groups]   seed S + 200000
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

OP_KN, OP_NK, OP_W8, OP_W4 = 0, 1, 2, 3  # FG_OP_F16_KN, FG_OP_F16_NK, FG_OP_W8A16_NK, FG_OP_W4A16_NK


@dataclass(frozen=True)
class Case:
    name: str
    op: int      # OP_*
    M: int
    N: int
    K: int
    seed: int
    groups: int = 1  # int4: scales per weight row (1 or K / 128)

    @property
    def weight_bytes(self) -> int:
        if self.op == OP_W4:
            return self.N * self.K // 2
        return self.N * self.K * (1 if self.op == OP_W8 else 2)

    @property
    def algorithmic_bytes(self) -> int:
        """weight + activations + output (+ per-channel scales): what one call must move."""
        b = self.weight_bytes + 2 * self.M * self.K + 2 * self.M * self.N
        if self.op == OP_W8:
            b += 2 * self.N
        if self.op == OP_W4:
            b += 2 * self.N * self.groups
        return b


def make_weight(case: Case) -> torch.Tensor:
    """The weight in the layout its operator takes: [K,N] for OP_KN, [N,K] otherwise."""
    g = torch.Generator(device="cpu").manual_seed(case.seed)
    if case.op == OP_W8:
        return torch.randint(-127, 128, (case.N, case.K), generator=g, dtype=torch.int8)
    if case.op == OP_W4:
        return torch.randint(0, 256, (case.N, case.K // 2), generator=g, dtype=torch.uint8)
    w = (torch.randn(case.N, case.K, generator=g) / case.K ** 0.5).to(torch.float16)
    return w.t().contiguous() if case.op == OP_KN else w


def make_activation(case: Case) -> torch.Tensor:
    g = torch.Generator(device="cpu").manual_seed(case.seed + 100000)
    return torch.randn(case.M, case.K, generator=g).to(torch.float16)


def make_scales(case: Case):
    if case.op not in (OP_W8, OP_W4):
        return None
    g = torch.Generator(device="cpu").manual_seed(case.seed + 200000)
    if case.op == OP_W4:
        return ((torch.rand(case.N, case.groups, generator=g) + 0.5) / 8.0).to(torch.float16)
    return ((torch.rand(case.N, generator=g) + 0.5) / 127.0).to(torch.float16)


# ---- the five configurations ---------------------------------------------------------------
def cfg1() -> list[Case]:
    """edgemm_m8n128k64x4: M=8, K=N=4096, weight KxN."""
    return [Case("edgemm_m8n128k64x4", OP_KN, 8, 4096, 4096, 1001)]


def cfg2() -> list[Case]:
    """edgemm_m8n128k64x4_bt: M in {1,2,4,8,16}, K=N=8192, weight NxK."""
    return [Case(f"edgemm_m8n128k64x4_bt_M{m}", OP_NK, m, 8192, 8192, 2000 + m) for m in (1, 2, 4, 8, 16)]


def cfg3() -> list[Case]:
    """fastgemv: N=11008,K=4096 and the transposed shape."""
    return [Case("fastgemv_11008x4096", OP_NK, 1, 11008, 4096, 3001),
            Case("fastgemv_4096x11008", OP_NK, 1, 4096, 11008, 3002)]


def cfg4() -> list[Case]:
    """fastgemv_int8 with per-output-channel scales: M in {1,8}, N=28672, K=8192."""
    return [Case(f"fastgemv_int8_M{m}", OP_W8, m, 28672, 8192, 4000 + m) for m in (1, 8)]


def w4() -> list[Case]:
    """fastgemv_int4 with one scale per 128 k: the shape of cfg4 with 4-bit weights, M in {1,8,16}."""
    return [Case(f"fastgemv_int4_M{m}", OP_W4, m, 28672, 8192, 4100 + m, 8192 // 128) for m in (1, 8, 16)]


DIT_LAYERS = 40
DIT_HIDDEN = 3072
# (name, N, K) of the four projections of one block
DIT_LINEARS = (("qkv", 9216, 3072), ("out", 3072, 3072), ("up", 12288, 3072), ("down", 3072, 12288))


def cfg5(layers: int = DIT_LAYERS) -> list[Case]:
    """T2V DiT linear stack: M=16, four projections per layer, weights NxK."""
    out = []
    for layer in range(layers):
        for j, (name, n, k) in enumerate(DIT_LINEARS):
            out.append(Case(f"dit_l{layer}_{name}", OP_NK, 16, n, k, 5000 + layer * 4 + j))
    return out


def shard_rows(N: int, world: int, rank: int) -> tuple[int, int]:
    """Column partition of the output (= row partition of an NxK weight): [begin, end) of
    rank `rank`; every shard keeps the N % 128 == 0 contract."""
    if N % (128 * world):
        raise ValueError(f"N={N} cannot be split into {world} shards that are multiples of 128")
    per = N // world
    return rank * per, (rank + 1) * per
