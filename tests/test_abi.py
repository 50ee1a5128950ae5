"""The C ABI on a machine without a GPU: the library loads, exports everything the header
declares, and rejects bad arguments before touching a device."""
import ctypes
import os
import re

import pytest

from fastgate_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "fastgate_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fg_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert _declared_functions() == sorted(capi.EXPORTS)


@pytest.mark.parametrize("name", _declared_functions())
def test_symbol_exported(name):
    assert getattr(capi.lib, name) is not None


def test_version_and_status_strings():
    assert capi.lib.fg_version().decode().startswith("fastgate_b200")
    assert capi.status_str(capi.FG_OK) == "ok"
    # the reference's message for the 128 contract (hk/edgemm.cu:108)
    assert "multiple of 128" in capi.status_str(capi.FG_ERR_SHAPE)
    for st in range(0, 9):
        assert capi.status_str(st) != "unknown status"
    assert capi.status_str(99) == "unknown status"


def test_workspace_size_grows_with_tiles():
    a, b = capi.workspace_bytes(128), capi.workspace_bytes(128 * 4096)
    assert a % 256 == 0 and b % 256 == 0 and b > a > 4 * 2 ** 20


def _call(fn, *args):
    return fn(*args)


def test_argument_checks_need_no_device():
    L = capi.lib
    buf = (ctypes.c_char * 4096)()
    base = ctypes.addressof(buf)
    p16 = (base + 255) // 256 * 256  # 256-byte aligned host address, never dereferenced
    ws_bytes = capi.workspace_bytes(128)
    # null pointers
    assert L.fg_gemm_f16_nk(None, p16, p16, 1, 128, 128, p16, ws_bytes, None) == capi.FG_ERR_NULL
    assert L.fg_gemm_f16_kn(p16, None, p16, 1, 128, 128, p16, ws_bytes, None) == capi.FG_ERR_NULL
    assert L.fg_gemm_w8a16_nk(p16, p16, None, None, 1, 128, 128, p16, ws_bytes, None) == capi.FG_ERR_NULL
    # the K, N % 128 contract and non-positive sizes
    for (M, N, K) in [(1, 100, 128), (1, 128, 192 + 1), (1, 128, 64), (0, 128, 128), (1, 0, 128), (-1, 128, 128)]:
        assert L.fg_gemm_f16_nk(p16, p16, p16, M, N, K, p16, ws_bytes, None) == capi.FG_ERR_SHAPE
        assert L.fg_gemm_f16_kn(p16, p16, p16, M, N, K, p16, ws_bytes, None) == capi.FG_ERR_SHAPE
        assert L.fg_gemm_w8a16_nk(p16, p16, None, p16, M, N, K, p16, ws_bytes, None) == capi.FG_ERR_SHAPE
    # alignment
    assert L.fg_gemm_f16_nk(p16 + 2, p16, p16, 1, 128, 128, p16, ws_bytes, None) == capi.FG_ERR_ALIGN
    assert L.fg_gemm_f16_nk(p16, p16 + 8, p16, 1, 128, 128, p16, ws_bytes, None) == capi.FG_ERR_ALIGN
    # workspace: missing, misaligned, too small
    assert L.fg_gemm_f16_nk(p16, p16, p16, 1, 128, 128, None, ws_bytes, None) == capi.FG_ERR_WORKSPACE
    assert L.fg_gemm_f16_nk(p16, p16, p16, 1, 128, 128, p16 + 16, ws_bytes, None) == capi.FG_ERR_WORKSPACE
    assert L.fg_gemm_f16_nk(p16, p16, p16, 1, 128, 128, p16, 1024, None) == capi.FG_ERR_WORKSPACE
    assert L.fg_workspace_init(None, ws_bytes, None) == capi.FG_ERR_WORKSPACE
    assert L.fg_workspace_init(p16, 16, None) == capi.FG_ERR_WORKSPACE
    assert L.fg_gemm_planned(None, p16, p16, None, p16, 1, 128, 128, p16, ws_bytes, None) == capi.FG_ERR_NULL
    assert L.fg_linear_host(1, None, p16, None, p16, p16, p16, 1, 128, 128, p16, ws_bytes, None) == capi.FG_ERR_NULL
    assert L.fg_linear_host(7, p16, p16, None, p16, p16, p16, 1, 128, 128, p16, ws_bytes, None) == capi.FG_ERR_PLAN


def test_pybind_module_surface():
    """Every host entry point of the reference's hot-path translation units is answered."""
    import fastgate_b200 as fg

    names = """edgemm edgemm_m8n128k128 edgemm_m8n128k64 edgemm_m8n128k64x4 edgemm_m8n128k64x4_amd
    edgemm_m8n128k64x4_bt edgemm_m8n128k64x4_tr_amd edgemm_m8n256k32x8 edgemm_m8n256k64 edgemv_m1n128k64x4
    edgemv_m1n256k64x4 gemm_m8n128k64x4_bt gemm_m8n32k128x8_bt gemm_m8n32k256x8_bt gemm_m8n32k256x8_bt_bz2
    gemm_m8n64k128x8_bt_exp flat_gemm_m8n128k64x4_bz1 flat_gemm_m8n256k32x8_bz1 flat_gemm_m8n256k64x8
    flat_gemm_m8n256k32x16 flat_gemm_m8n512k32x16 flat_gemm_m8n64k128x8 flat_gemm_m8n32k256x8 fastgemv
    fastgemv_int8 fastgemv_tuned fastgemv_extend fastgemm hgemm hgemm_tr""".split()
    assert len(names) == 30
    for n in names:
        assert callable(getattr(fg, n)), n


def test_ops_refuse_cpu_tensors():
    import torch

    import fastgate_b200 as fg

    a = torch.zeros(8, 128, dtype=torch.half)
    w = torch.zeros(128, 128, dtype=torch.half)
    with pytest.raises(RuntimeError, match="no CPU path"):
        fg.edgemm_m8n128k64x4(a, w, torch.zeros(8, 128, dtype=torch.half))
    with pytest.raises(RuntimeError, match="no CPU path"):
        fg.fastgemv(w, a[:1], torch.zeros(128, dtype=torch.half))
