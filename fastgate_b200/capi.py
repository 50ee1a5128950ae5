"""ctypes binding of the C ABI in include/fastgate_b200.h.

This is the route for callers that do not want the pybind module (and the one the parity
tests use): device pointers are passed as integers, e.g. ``tensor.data_ptr()``.
There is no CPU fallback: if libfastgate_b200.so is missing the import fails.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libfastgate_b200.so")

FG_OK, FG_ERR_SHAPE, FG_ERR_ALIGN, FG_ERR_NULL, FG_ERR_WORKSPACE = 0, 1, 2, 3, 4
FG_ERR_CUDA, FG_ERR_TIMEOUT, FG_ERR_PLAN, FG_ERR_NO_DEVICE = 5, 6, 7, 8
FG_OP_F16_KN, FG_OP_F16_NK, FG_OP_W8A16_NK, FG_OP_W4A16_NK = 0, 1, 2, 3

# every symbol include/fastgate_b200.h declares
EXPORTS = (
    "fg_plan", "fg_plan_validate", "fg_workspace_bytes", "fg_workspace_init", "fg_workspace_status",
    "fg_gemm_f16_kn", "fg_gemm_f16_nk", "fg_gemm_w8a16_nk", "fg_gemm_w4a16_nk", "fg_quantize_rows_w4", "fg_gemm_f16_nk_noalloc", "fg_noalloc_status", "fg_gemm_planned",
    "fg_gemm_f16_nk_push", "fg_push_wait", "fg_push_wait_dev", "fg_push_wait_dev_many", "fg_group_table_bytes", "fg_group_create", "fg_group_run",
    "fg_group_tiles", "fg_group_destroy", "fg_chain_table_bytes", "fg_chain_create", "fg_chain_workspace_bytes",
    "fg_chain_run", "fg_chain_grid", "fg_chain_trace_offset", "fg_chain_destroy", "fg_quantize_rows_w8", "fg_gemm_fused", "fg_linear_host",
    "fg_prepack_kn_to_nk", "fg_prepack_gate_up",
    "fg_trace_enable", "fg_trace_read", "fg_status_str", "fg_last_cuda_error", "fg_launch_count", "fg_version",
)


class Plan(ctypes.Structure):
    """Mirror of fg_plan_t."""

    _fields_ = [(n, ctypes.c_int) for n in (
        "op", "m_tile", "k_per_stage", "stages", "consumer_warps", "grid", "tiles", "k_blocks",
        "smem_bytes", "passes", "math", "pdl", "rows_per_stage", "static_rows")]

    def as_dict(self) -> dict:
        return {n: getattr(self, n) for n, _ in self._fields_}


class Peers(ctypes.Structure):
    """Mirror of fg_peers_t."""

    _fields_ = [("world", ctypes.c_int), ("rank", ctypes.c_int), ("n_total", ctypes.c_longlong),
                ("C", ctypes.c_void_p * 8), ("flag", ctypes.c_void_p * 8),
                ("wait_flags", ctypes.c_void_p), ("wait_target", ctypes.c_ulonglong),
                ("mc_C", ctypes.c_void_p), ("mc_flag", ctypes.c_void_p),
                ("target_dev", ctypes.c_void_p), ("wait_target_dev", ctypes.c_void_p)]


class Epilogue(ctypes.Structure):
    """Mirror of fg_epilogue_t."""

    _fields_ = [("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p), ("act", ctypes.c_int),
                ("split1", ctypes.c_int), ("split2", ctypes.c_int), ("C2", ctypes.c_void_p), ("C3", ctypes.c_void_p)]


ACT = {"none": 0, "gelu": 1, "gelu_erf": 1, "gelu_tanh": 2, "silu": 3, "silu_gate": 4}


class Problem(ctypes.Structure):
    """Mirror of fg_problem_t."""

    _fields_ = [("x", ctypes.c_void_p), ("W", ctypes.c_void_p), ("C", ctypes.c_void_p),
                ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("peer_C", ctypes.c_void_p * 8), ("n_total", ctypes.c_longlong), ("mc_C", ctypes.c_void_p)]


class Layer(ctypes.Structure):
    """Mirror of fg_layer_t."""

    _fields_ = [("x", ctypes.c_void_p), ("W", ctypes.c_void_p), ("C", ctypes.c_void_p),
                ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p),
                ("ldx", ctypes.c_longlong), ("ldc", ctypes.c_longlong), ("ldr", ctypes.c_longlong),
                ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("act", ctypes.c_int), ("dep", ctypes.c_int)]


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m fastgate_b200.build` "
            "(fastgate_b200 has no CPU fallback)")
    L = ctypes.CDLL(LIB_PATH)
    vp, sz, i = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int
    L.fg_plan.argtypes = [i, i, i, i, i, i, ctypes.POINTER(Plan)]
    L.fg_plan_validate.argtypes = [ctypes.POINTER(Plan), i, i, i]
    L.fg_plan_tiled.argtypes = [i, i, i, i, i, i, ctypes.POINTER(Plan)]  # internal: never the row-split GEMV plan
    L.fg_workspace_bytes.argtypes = [i]
    L.fg_workspace_bytes.restype = sz
    L.fg_workspace_init.argtypes = [vp, sz, vp]
    L.fg_workspace_status.argtypes = [vp, ctypes.POINTER(i), vp]
    L.fg_gemm_f16_kn.argtypes = [vp, vp, vp, i, i, i, vp, sz, vp]
    L.fg_gemm_f16_nk.argtypes = [vp, vp, vp, i, i, i, vp, sz, vp]
    L.fg_gemm_w8a16_nk.argtypes = [vp, vp, vp, vp, i, i, i, vp, sz, vp]
    L.fg_gemm_w4a16_nk.argtypes = [vp, vp, vp, i, i, vp, i, i, i, vp, sz, vp]
    L.fg_gemm_f16_nk_noalloc.argtypes = [vp, vp, vp, i, i, i, vp]
    L.fg_noalloc_status.argtypes = [ctypes.POINTER(i), vp]
    L.fg_gemm_planned.argtypes = [ctypes.POINTER(Plan), vp, vp, vp, vp, i, i, i, vp, sz, vp]
    L.fg_gemm_f16_nk_push.argtypes = [vp, vp, i, i, i, ctypes.POINTER(Peers), vp, sz, vp]
    L.fg_push_wait.argtypes = [vp, i, ctypes.c_ulonglong, vp, vp]
    L.fg_push_wait_dev.argtypes = [vp, i, vp, vp, vp]
    L.fg_push_wait_dev_many.argtypes = [vp, vp, i, i, vp, vp]
    L.fg_group_table_bytes.argtypes = [i]
    L.fg_group_table_bytes.restype = sz
    L.fg_group_create.argtypes = [i, ctypes.POINTER(Problem), i, ctypes.POINTER(Peers), vp, sz, ctypes.POINTER(vp)]
    L.fg_group_run.argtypes = [vp, vp, sz, vp]
    L.fg_group_tiles.argtypes = [vp]
    L.fg_group_tiles.restype = ctypes.c_ulonglong
    L.fg_group_destroy.argtypes = [vp]
    L.fg_group_destroy.restype = None
    L.fg_chain_table_bytes.argtypes = [i]
    L.fg_chain_table_bytes.restype = sz
    L.fg_chain_create.argtypes = [i, ctypes.POINTER(Layer), i, vp, sz, ctypes.POINTER(vp)]
    L.fg_chain_workspace_bytes.argtypes = [vp]
    L.fg_chain_workspace_bytes.restype = sz
    L.fg_chain_run.argtypes = [vp, vp, sz, vp]
    L.fg_chain_grid.argtypes = [vp]
    L.fg_chain_trace_offset.argtypes = [vp]
    L.fg_chain_trace_offset.restype = sz
    L.fg_chain_destroy.argtypes = [vp]
    L.fg_chain_destroy.restype = None
    L.fg_quantize_rows_w8.argtypes = [vp, vp, vp, i, i, vp]
    L.fg_quantize_rows_w4.argtypes = [vp, vp, vp, i, i, i, vp]
    L.fg_gemm_fused.argtypes = [i, vp, vp, vp, vp, i, i, i, ctypes.POINTER(Epilogue), vp, sz, vp]
    L.fg_prepack_kn_to_nk.argtypes = [vp, vp, i, i, vp]
    L.fg_prepack_gate_up.argtypes = [vp, vp, vp, i, i, vp]
    L.fg_linear_host.argtypes = [i, vp, vp, vp, vp, vp, vp, i, i, i, vp, sz, vp]
    L.fg_trace_enable.argtypes = [i]
    L.fg_trace_read.argtypes = [vp, ctypes.POINTER(ctypes.c_ulonglong), i, vp]
    L.fg_status_str.argtypes = [i]
    L.fg_status_str.restype = ctypes.c_char_p
    L.fg_last_cuda_error.restype = i
    L.fg_launch_count.restype = ctypes.c_ulonglong
    L.fg_version.restype = ctypes.c_char_p
    return L


lib = _load()


def status_str(st: int) -> str:
    return lib.fg_status_str(st).decode()


def plan(op: int, M: int, N: int, K: int, sm_count: int = 0, smem_optin: int = 0) -> Plan:
    p = Plan()
    st = lib.fg_plan(op, M, N, K, sm_count, smem_optin, ctypes.byref(p))
    if st != FG_OK:
        raise ValueError(status_str(st))
    return p


def passes(op: int, M: int, N: int, K: int) -> int:
    """Launches one call makes (a pass covers up to 64 token rows of fp16 weights, 16 otherwise)."""
    return plan(op, M, N, K).passes


def workspace_bytes(N: int) -> int:
    return int(lib.fg_workspace_bytes(N))


def launch_count() -> int:
    return int(lib.fg_launch_count())
