"""TEST INFRASTRUCTURE ONLY: loader for the reference's own kernels (oracle/_ref).

`load()` returns the torch extension built by build_ref.py, or None when it has not been
built (the reference checkout is not available on every machine).  Contract notes for
callers, from reading the reference:
  * every op except edgemm_m8n128k64x4 / _bt / flat_gemm_m8n256k32x8_bz1 / _m8n256k32x16 /
    gemm_m8n128k64x4_bt leaves zeroing of C to the caller: pass a zeroed C;
  * edgemm_m8n128k64x4 is only correct for K % 1024 == 0 (fixed split of 8 and a tail that
    assumes an even tile count, backend/cuda/hk/edgemm.cu:115, edgemm.cuh:1823-1833);
  * flat_gemm_* / gemm_*_bt handle M <= 8; fastgemm M <= 2; fastgemv_int8 M = 1.
"""
from __future__ import annotations

import importlib.util
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "_ref", "fastgate_ref.so")
_mod = None


def available() -> bool:
    return os.path.exists(_PATH)


def load():
    global _mod
    if _mod is None and available():
        import torch  # noqa: F401
        spec = importlib.util.spec_from_file_location("fastgate_ref", _PATH)
        _mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(_mod)
    return _mod
