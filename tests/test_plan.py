"""The launch heuristic and the stream-K work split, on the CPU.

`simulate` mirrors the kernel's index arithmetic (range of each CTA, its segments, who
contributes to a split tile and in which workspace slot) and checks the invariants the
device code relies on."""
import ctypes

import pytest

from fastgate_b200 import capi

B200 = dict(sm_count=148, smem_optin=232448)
CHUNK_K = {0: 64, 1: 64, 2: 128, 3: 256}


def _range_begin(c, total, grid):
    return (c * total) // grid


def _cta_of_unit(u, total, grid):
    c = (u * grid) // total
    while c + 1 < grid and _range_begin(c + 1, total, grid) <= u:
        c += 1
    while c > 0 and _range_begin(c, total, grid) > u:
        c -= 1
    return c


def simulate(tiles, k_blocks, grid):
    total = tiles * k_blocks
    covered = [0] * total
    contrib = {}
    for c in range(grid):
        ub, ue = _range_begin(c, total, grid), _range_begin(c + 1, total, grid)
        assert ue > ub, "every CTA owns at least one unit"
        u, partial_segments = ub, 0
        while u < ue:
            tile, kb0 = divmod(u, k_blocks)
            ln = min(k_blocks - kb0, ue - u)
            for i in range(u, u + ln):
                covered[i] += 1
            if ln != k_blocks:
                partial_segments += 1
                contrib.setdefault(tile, []).append((c, 0 if u == ub else 1))
            u += ln
        assert partial_segments <= 2, "two workspace slots per CTA must suffice"
    assert all(v == 1 for v in covered), "each (tile, k-block) is streamed exactly once"
    for tile, lst in contrib.items():
        first = _cta_of_unit(tile * k_blocks, total, grid)
        last = _cta_of_unit(tile * k_blocks + k_blocks - 1, total, grid)
        want = [(c, 0 if _range_begin(c, total, grid) // k_blocks == tile else 1) for c in range(first, last + 1)]
        assert lst == want, (tile, lst, want)
        assert len(lst) >= 2
    # imbalance: no CTA streams more than one stage more than another
    sizes = [_range_begin(c + 1, total, grid) - _range_begin(c, total, grid) for c in range(grid)]
    assert max(sizes) - min(sizes) <= 1
    return contrib


SHAPES = [(1, 1, 8192, 8192), (1, 2, 8192, 8192), (1, 2, 3072, 12288), (1, 1, 128, 1024), (1, 1, 256, 32768), (1, 2, 128, 128),
          (1, 16, 8192, 8192), (1, 1, 11008, 4096), (1, 1, 4096, 11008), (0, 8, 4096, 4096),
          (2, 1, 28672, 8192), (2, 8, 28672, 8192), (1, 16, 9216, 3072), (1, 16, 3072, 3072),
          (1, 16, 12288, 3072), (1, 16, 3072, 12288), (1, 4, 128, 128), (0, 3, 256, 384),
          (1, 16, 1152, 3072), (1, 16, 384, 3072), (1, 16, 1536, 3072), (1, 33, 4096, 4096),
          (3, 1, 28672, 8192), (3, 16, 28672, 8192), (3, 8, 256, 384), (2, 16, 4096, 4096),
          (1, 17, 8192, 8192), (1, 32, 8192, 8192), (0, 48, 4096, 4096), (1, 64, 8192, 8192), (1, 100, 3072, 3072),
          (2, 40, 4096, 4096)]


def check_gemv_plan(p, M, N, K):
    """Row-split GEMV kernel (math 4): every weight row is streamed exactly once, by one CTA."""
    assert (p.op == 1 and 1 <= M <= 2) or (p.op == 2 and M == 1), "fp16 rows for one or two tokens, int8 rows for one"
    assert p.m_tile == M and p.passes == 1
    assert p.rows_per_stage in (1, 2, 4, 8) and p.rows_per_stage * M <= 8
    assert p.rows_per_stage * K * (1 if p.op == 2 else 2) <= 65536 and p.k_per_stage == K and p.k_blocks == 1
    assert 3 <= p.stages <= 24 and 1 <= p.consumer_warps <= 12 and p.stages % p.consumer_warps == 0
    assert 1 <= p.grid <= 148 and p.smem_bytes <= 232448
    assert p.static_rows % p.rows_per_stage == 0 and p.static_rows * p.grid <= N
    # static shares, then blocks of rows_per_stage rows from the counter, cover [0, N) once
    covered = [0] * N
    for c in range(p.grid):
        for r in range(c * p.static_rows, (c + 1) * p.static_rows):
            covered[r] += 1
    dyn0, j = p.grid * p.static_rows, 0
    while dyn0 + j * p.rows_per_stage < N:
        for r in range(dyn0 + j * p.rows_per_stage, min(N, dyn0 + (j + 1) * p.rows_per_stage)):
            covered[r] += 1
        j += 1
    assert all(v == 1 for v in covered)
    assert j <= 2 * p.grid, "only the remainder is dealt out on demand"


@pytest.mark.parametrize("op,M,N,K", SHAPES)
def test_plan_invariants(op, M, N, K):
    p = capi.plan(op, M, N, K, **B200)
    assert p.op == op and p.tiles == N // 128
    if p.math == 4:
        check_gemv_plan(p, M, N, K)
        assert capi.lib.fg_plan_validate(ctypes.byref(p), N, K, 232448) == capi.FG_OK
        return
    # NxK fp16 weights: one row always runs the GEMV kernel, two rows up to 48 Mi weights
    assert not (op == 1 and 1024 <= K <= 16384 and (M == 1 or (M == 2 and N * K <= 48 << 20))), "this shape belongs to the GEMV kernel"
    assert p.m_tile in (8, 16, 32, 64) and (p.m_tile >= 16 or M <= 8)
    assert p.m_tile >= min(M, 16)
    assert p.m_tile <= 16 or (op in (0, 1) and p.math == 2), "tall tiles: fp16 tcgen05 kernel only"
    assert p.k_per_stage % CHUNK_K[op] == 0
    assert p.k_blocks == -(-K // p.k_per_stage)
    assert 1 <= p.grid <= min(148, p.tiles * p.k_blocks)
    assert p.stages >= 2
    if p.math == 0:
        assert p.stages % p.consumer_warps == 0, "a ring slot must always meet the same warp"
        if op in (2, 3):  # the dequantising kernels: <= 384 threads per CTA
            assert p.consumer_warps <= (3 if p.m_tile == 16 else 6)
    else:
        assert p.math == 2 and p.m_tile >= 16, "tcgen05 kernels: accumulator in tensor memory"
        assert p.stages >= 3 or p.k_per_stage == CHUNK_K[op]
    # NxK fp16 weights always take the tcgen05 kernel, KxN ones above 40 MB, everything else above 8 token rows
    assert (p.math == 2) == (M > 8 or op == 1 or (op == 0 and N * K * 2 > 40 << 20))
    assert p.smem_bytes <= 232448
    rows = 64 if (p.math == 2 and op in (0, 1)) else 16
    assert p.passes == -(-M // rows)
    assert p.m_tile >= min(M, rows) or p.passes > 1
    assert capi.lib.fg_plan_validate(ctypes.byref(p), N, K, 232448) == capi.FG_OK
    simulate(p.tiles, p.k_blocks, p.grid)


@pytest.mark.parametrize("tiles,k_blocks,grid", [(86, 32, 148), (32, 86, 148), (64, 64, 148), (224, 32, 148),
                                                 (1, 2, 2), (1, 1, 1), (3, 7, 5), (24, 48, 148), (9, 24, 148),
                                                 (3, 24, 72), (7, 5, 35), (5, 3, 4), (86, 64, 132)])
def test_streamk_split(tiles, k_blocks, grid):
    simulate(tiles, k_blocks, grid)


@pytest.mark.parametrize("op,M,N,K,grid", [(1, 16, 4096, 4096, 128), (1, 16, 3072, 3072, 96), (0, 8, 4096, 4096, 128), (0, 8, 3072, 3072, 96),
                                            (1, 4, 2048, 8192, 128), (1, 16, 9216, 3072, 144), (1, 16, 3072, 12288, 144),
                                            (0, 8, 1152, 3072, 72), (1, 16, 4096, 2048, 128)])
def test_small_problems_get_tile_aligned_grids(op, M, N, K, grid):
    """Up to 80 MB of fp16 weights: tiles x s CTAs, s a divisor of the stages per tile, so that every CTA
    owns one segment of one tile and every tile is reduced over exactly s contributors."""
    p = capi.plan(op, M, N, K, **B200)
    assert p.math in (0, 2) and p.grid == grid, p.as_dict()
    s = p.grid // p.tiles
    assert p.grid == p.tiles * s and p.k_blocks % s == 0 and s >= 2
    contrib = simulate(p.tiles, p.k_blocks, p.grid)
    total = p.tiles * p.k_blocks
    for t in range(p.tiles):
        assert contrib[t] == [(c, 0) for c in range(t * s, (t + 1) * s)]
    for c in range(p.grid):
        assert _range_begin(c + 1, total, p.grid) - _range_begin(c, total, p.grid) == p.k_blocks // s
    assert capi.lib.fg_plan_validate(ctypes.byref(p), N, K, 232448) == capi.FG_OK


def test_large_or_awkward_problems_keep_all_sms():
    for (op, M, N, K) in [(1, 16, 8192, 8192), (1, 16, 12288, 3072), (0, 8, 8192, 8192), (1, 16, 11008, 4096), (2, 8, 4096, 4096),
                          (1, 16, 1152, 3072)]:
        p = capi.plan(op, M, N, K, **B200)
        assert p.grid == min(148, p.tiles * p.k_blocks), p.as_dict()


def test_plan_rejects_bad_problems():
    p = capi.Plan()
    L = capi.lib
    assert L.fg_plan(1, 1, 100, 128, 0, 0, ctypes.byref(p)) == capi.FG_ERR_SHAPE
    assert L.fg_plan(1, 1, 128, 100, 0, 0, ctypes.byref(p)) == capi.FG_ERR_SHAPE
    assert L.fg_plan(1, 0, 128, 128, 0, 0, ctypes.byref(p)) == capi.FG_ERR_SHAPE
    assert L.fg_plan(9, 1, 128, 128, 0, 0, ctypes.byref(p)) == capi.FG_ERR_PLAN
    assert L.fg_plan(1, 1, 128, 128, 0, 0, None) == capi.FG_ERR_NULL


def test_validate_catches_edited_plans():
    L = capi.lib
    good = capi.plan(0, 8, 4096, 4096, **B200)  # KxN weights at 8 rows, up to 40 MB: the mma.sync kernel
    assert good.math == 0

    def edited(**kw):
        q = capi.Plan()
        ctypes.memmove(ctypes.byref(q), ctypes.byref(good), ctypes.sizeof(q))
        for k, v in kw.items():
            setattr(q, k, v)
        return L.fg_plan_validate(ctypes.byref(q), 4096, 4096, 232448)

    assert edited() == capi.FG_OK
    assert edited(stages=good.stages + 1) == capi.FG_ERR_PLAN      # smem no longer matches / not a multiple
    assert edited(consumer_warps=9) == capi.FG_ERR_PLAN
    assert edited(m_tile=12) == capi.FG_ERR_PLAN
    assert edited(grid=0) == capi.FG_ERR_PLAN
    assert edited(grid=100000) == capi.FG_ERR_PLAN
    assert edited(k_blocks=good.k_blocks + 1) == capi.FG_ERR_PLAN
    assert edited(tiles=good.tiles + 1) == capi.FG_ERR_PLAN
    assert edited(k_per_stage=96) == capi.FG_ERR_PLAN
    assert edited(smem_bytes=good.smem_bytes + 16) == capi.FG_ERR_PLAN
    assert edited(math=1) == capi.FG_ERR_PLAN
    assert edited(math=2) == capi.FG_ERR_PLAN           # the tcgen05 kernel needs the 16-row tile

    umma = capi.plan(1, 16, 8192, 8192, **B200)
    assert umma.math == 2

    def edited2(**kw):
        q = capi.Plan()
        ctypes.memmove(ctypes.byref(q), ctypes.byref(umma), ctypes.sizeof(q))
        for k, v in kw.items():
            setattr(q, k, v)
        return L.fg_plan_validate(ctypes.byref(q), 8192, 8192, 232448)

    assert edited2() == capi.FG_OK
    assert edited2(stages=umma.stages + 1) == capi.FG_ERR_PLAN
    assert edited2(m_tile=8) == capi.FG_ERR_PLAN
    assert edited2(op=2) == capi.FG_ERR_PLAN
    assert edited2(math=0) == capi.FG_ERR_PLAN          # another kernel, another shared-memory layout


def test_validate_catches_edited_gemv_plans():
    L = capi.lib
    good = capi.plan(1, 1, 8192, 8192, **B200)
    assert good.math == 4

    def edited(**kw):
        q = capi.Plan()
        ctypes.memmove(ctypes.byref(q), ctypes.byref(good), ctypes.sizeof(q))
        for k, v in kw.items():
            setattr(q, k, v)
        return L.fg_plan_validate(ctypes.byref(q), 8192, 8192, 232448)

    assert edited() == capi.FG_OK
    assert edited(static_rows=0) == capi.FG_OK                      # everything on demand
    assert edited(static_rows=56) == capi.FG_ERR_PLAN               # 148 x 56 rows > N
    assert edited(rows_per_stage=3) == capi.FG_ERR_PLAN
    assert edited(rows_per_stage=8) == capi.FG_ERR_PLAN             # 128 KB per stage
    assert edited(consumer_warps=5) == capi.FG_ERR_PLAN             # must divide the ring depth
    assert edited(stages=good.stages + 1) == capi.FG_ERR_PLAN       # shared memory no longer matches
    assert edited(m_tile=3) == capi.FG_ERR_PLAN
    assert edited(op=0) == capi.FG_ERR_PLAN                         # KxN weights have no contiguous rows
    assert edited(math=2) == capi.FG_ERR_PLAN


def test_default_device_is_b200():
    a = capi.plan(1, 8, 8192, 8192)          # 0/0 = B200 defaults
    b = capi.plan(1, 8, 8192, 8192, **B200)
    assert a.as_dict() == b.as_dict()
