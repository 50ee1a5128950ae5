"""Pins the CPU oracle to outputs of the reference's own kernels.

tests/golden/reference_b200.npz was written by tests/golden/make_golden.py on a B200 from the
reference's unmodified kernels (rebuilt for sm_100a).  Inputs are regenerated here from the
seeds stored with each case.

* CUDA-core kernels (fastgemv, fastgemm, fastgemv_extend, fastgemv_int8): the order-exact
  restatements in oracle.c must reproduce the GPU output bit for bit.
* Tensor-core kernels (edgemm_m8n128k64x4, _bt): fp16 accumulation in a hardware order, so
  they only have to sit within the path's tolerance of the fp32-accumulated oracle.
"""
import os

import numpy as np
import pytest

from fastgate_b200 import workloads as wl
from oracle import oracle as o

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_b200.npz"))
KEYS = sorted(k for k in GOLD.files if not k.endswith("__meta"))


def _case(key):
    op, M, N, K, seed = (int(v) for v in GOLD[key + "__meta"])
    case = wl.Case(key, op, M, N, K, seed)
    return case, wl.make_activation(case).numpy(), wl.make_weight(case).numpy(), GOLD[key].view(np.float16)


def test_fixture_inventory():
    assert len(KEYS) == 12
    assert sum(k.startswith("fastgemv_int8") for k in KEYS) == 2
    assert sum(k.startswith("edgemm") for k in KEYS) == 3


@pytest.mark.parametrize("key", [k for k in KEYS if not k.startswith("edgemm")])
def test_order_exact_restatement_matches_reference_bits(key):
    case, x, W, gold = _case(key)
    if key.startswith("fastgemv_int8"):
        mine = o.gemv_int8_ref(W, x)[None]
    elif key.startswith("fastgemv_extend"):
        mine = o.gemm_fp16_ref(W, x)
    elif key.startswith("fastgemm_m2"):
        mine = o.gemv_fp16_bs2_ref(W, x)
    else:
        mine = o.gemv_fp16_ref(W, x)[None]
    assert mine.shape == gold.shape
    assert np.array_equal(mine.view(np.uint16), gold.view(np.uint16)), key


@pytest.mark.parametrize("key", KEYS)
def test_fp32_oracle_within_tolerance_of_reference(key):
    case, x, W, gold = _case(key)
    if case.op == wl.OP_W8:
        ref = o.gemm_w8a16_nk(x, W)
    elif case.op == wl.OP_KN:
        ref = o.gemm_kn(x, W)
    else:
        ref = o.gemm_nk(x, W)
    o.check_tolerance(gold, ref, key)


# ---- int4: gemv_quantized_int4 (hk/fastgemv.cuh:394-495) -------------------------------------------
# reference_b200_int4.npz: outputs of the reference's kernel on a B200, launched by
# oracle/ref_int4_launch.cu (the reference has no launcher for it), one scale and zero point
# for the whole matrix.
GOLD4 = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_b200_int4.npz"))
KEYS4 = sorted(k for k in GOLD4.files if "__" not in k)


def _case4(key):
    op, M, N, K, seed, zp = (int(v) for v in GOLD4[key + "__meta"])
    case = wl.Case(key, op, M, N, K, seed)
    scale = float(GOLD4[key + "__scale"][0])
    return wl.make_activation(case).numpy(), wl.make_weight(case).numpy(), scale, zp, GOLD4[key].view(np.float16)


def test_int4_fixture_inventory():
    assert len(KEYS4) == 3 and any(k.endswith("zp5") for k in KEYS4)


@pytest.mark.parametrize("key", KEYS4)
def test_int4_restatement_matches_reference_bits(key):
    x, W4, scale, zp, gold = _case4(key)
    mine = o.gemv_int4_ref(W4, x, scale, float(zp))
    assert np.array_equal(mine.view(np.uint16), gold.view(np.uint16)), key


@pytest.mark.parametrize("key", KEYS4)
def test_int4_fp32_oracle_within_tolerance_of_reference(key):
    x, W4, scale, zp, gold = _case4(key)
    N = W4.shape[0]
    ref = o.gemm_w4a16_nk(x, W4, np.full(N, scale, np.float16), zp)
    o.check_tolerance(gold[None], ref, key)
