"""ctypes front end of oracle.c — TEST INFRASTRUCTURE ONLY (see oracle.c's header).

All functions take and return numpy arrays; fp16 data travels as numpy float16.
`check_tolerance` is the acceptance rule of the path:  max|out - ref| <= 1e-2 * max(1, |ref|)
elementwise, against the fp32-accumulated reference.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

TOL = 1e-2  # max|d| <= TOL * max(1, |ref|)


def build(force: bool = False) -> str:
    """Compile oracle.c with gcc (a second or two); returns the library path."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-s", "-B", "-C", _HERE, "liboracle.so"], check=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.fgo_num_threads.restype = ctypes.c_int
        _lib.fgo_ref_splitk_bt.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctypes.c_void_p)


def _h(a) -> np.ndarray:
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float16, a.dtype
    return a


def num_threads() -> int:
    return int(lib().fgo_num_threads())


# ---- order-exact restatements of the reference's CUDA-core kernels -----------------------
def gemv_fp16_ref(W, x) -> np.ndarray:
    """fastgemv / fastgemm(M=1): W[N,K], x[1,K] or [K] -> y[N] fp16, bit-exact order."""
    W, x = _h(W), _h(x).reshape(-1)
    N, K = W.shape
    assert x.shape[0] == K
    y = np.empty(N, np.float16)
    lib().fgo_gemv_fp16_ref(_p(W), _p(x), _p(y), N, K)
    return y


def gemv_fp16_bs2_ref(W, x2) -> np.ndarray:
    """fastgemm(M=2): W[N,K], x[2,K] -> C[2,N] fp16."""
    W, x2 = _h(W), _h(x2)
    N, K = W.shape
    assert x2.shape == (2, K)
    C = np.empty((2, N), np.float16)
    lib().fgo_gemv_fp16_bs2_ref(_p(W), _p(x2), _p(C), N, K)
    return C


def gemm_fp16_ref(W, x) -> np.ndarray:
    """fastgemv_extend: W[N,K], x[M,K] (M <= 8) -> C[M,N] fp16."""
    W, x = _h(W), _h(x)
    N, K = W.shape
    M = x.shape[0]
    assert x.shape[1] == K
    C = np.empty((M, N), np.float16)
    lib().fgo_gemm_fp16_ref(_p(W), _p(x), _p(C), M, N, K)
    return C


def gemv_int8_ref(W8, x, scale: float = 1.0, zero_point: float = 0.0) -> np.ndarray:
    """fastgemv_int8 as launched by the reference (scale 1, zero-point 0): y[N] fp16."""
    W8 = np.ascontiguousarray(W8)
    assert W8.dtype == np.int8
    x = _h(x).reshape(-1)
    N, K = W8.shape
    y = np.empty(N, np.float16)
    lib().fgo_gemv_int8_ref(_p(W8), _p(x), _p(y), N, K, ctypes.c_float(scale), ctypes.c_float(zero_point))
    return y


def gemv_int4_ref(W4, x, scale: float = 1.0, zero_point: float = 8.0) -> np.ndarray:
    """gemv_quantized_int4 of the reference, launched 128 x 4 like its int8 sibling: y[N] fp16.
    W4 is [N, K/2] uint8, low nibble = even k."""
    W4 = np.ascontiguousarray(W4)
    assert W4.dtype == np.uint8
    x = _h(x).reshape(-1)
    N, K = W4.shape[0], W4.shape[1] * 2
    assert x.shape[0] == K
    y = np.empty(N, np.float16)
    lib().fgo_gemv_int4_ref(_p(W4), _p(x), _p(y), N, K, ctypes.c_float(scale), ctypes.c_float(zero_point))
    return y


# ---- fp32-accumulated reference ----------------------------------------------------------
def gemm_nk(x, W) -> np.ndarray:
    """C32[M,N] = x[M,K] . W[N,K]^T (double accumulation, fp32 result)."""
    x, W = _h(x), _h(W)
    M, K = x.shape
    N = W.shape[0]
    assert W.shape[1] == K
    C = np.empty((M, N), np.float32)
    lib().fgo_gemm_nk(_p(x), _p(W), _p(C), M, N, K)
    return C


def gemm_nk_f32seq(x, W) -> np.ndarray:
    x, W = _h(x), _h(W)
    M, K = x.shape
    N = W.shape[0]
    C = np.empty((M, N), np.float32)
    lib().fgo_gemm_nk_f32seq(_p(x), _p(W), _p(C), M, N, K)
    return C


def gemm_kn(A, B) -> np.ndarray:
    """C32[M,N] = A[M,K] . B[K,N]."""
    A, B = _h(A), _h(B)
    M, K = A.shape
    N = B.shape[1]
    assert B.shape[0] == K
    C = np.empty((M, N), np.float32)
    lib().fgo_gemm_kn(_p(A), _p(B), _p(C), M, N, K)
    return C


def gemm_w8a16_nk(x, W8, scales=None) -> np.ndarray:
    """C32[M,N] = (x[M,K] . W8[N,K]^T) * scales[N]  (scales None = 1)."""
    x = _h(x)
    W8 = np.ascontiguousarray(W8)
    assert W8.dtype == np.int8
    M, K = x.shape
    N = W8.shape[0]
    C = np.empty((M, N), np.float32)
    sp = None
    if scales is not None:
        scales = _h(scales).reshape(-1)
        assert scales.shape[0] == N
        sp = _p(scales)
    lib().fgo_gemm_w8a16_nk(_p(x), _p(W8), sp, _p(C), M, N, K)
    return C


def epilogue(C32, bias=None, residual=None, act: int = 0) -> np.ndarray:
    """act(C32 + bias) + residual on a copy of C32 (fp32); act: 0 none, 1 gelu-erf, 2 gelu-tanh, 3 silu."""
    out = np.ascontiguousarray(C32, dtype=np.float32).copy()
    M, N = out.shape
    b = _p(_h(bias).reshape(-1)) if bias is not None else None
    r = _p(_h(residual).reshape(M, N)) if residual is not None else None
    lib().fgo_epilogue(_p(out), b, r, int(act), M, N)
    return out


def silu_gate(G32, U32, bias_gate=None, bias_up=None, residual=None) -> np.ndarray:
    """silu(G32 + bias_gate) * (U32 + bias_up) + residual in fp32: the gated-MLP epilogue, which has no
    counterpart in the reference (its operators stop at the matrix product); G32 and U32 are the
    fp32-accumulated products of the gate and the up projection."""
    g = np.asarray(G32, np.float32).copy()
    u = np.asarray(U32, np.float32).copy()
    if bias_gate is not None:
        g += _h(bias_gate).astype(np.float32).reshape(1, -1)
    if bias_up is not None:
        u += _h(bias_up).astype(np.float32).reshape(1, -1)
    out = (g / (np.float32(1) + np.exp(-g, dtype=np.float32))) * u
    if residual is not None:
        out = out + _h(residual).astype(np.float32)
    return out.astype(np.float32)


def interleave_gate_up(Wg, Wu) -> np.ndarray:
    """The weight layout the gated epilogue reads: per 128 rows, 64 gate rows then the matching 64 up rows."""
    Wg, Wu = np.asarray(Wg), np.asarray(Wu)
    n, k = Wg.shape
    assert Wu.shape == (n, k) and n % 64 == 0
    return np.stack([Wg.reshape(n // 64, 64, k), Wu.reshape(n // 64, 64, k)], axis=1).reshape(2 * n, k)


def gemm_w4a16_nk(x, W4, scales=None, zero_point: int = 8) -> np.ndarray:
    """C32[M,N] = sum_g scales[n,g] * sum_{k in g} x[m,k] * (nibble[n,k] - zero_point); scales is
    [N] / [N,1] (per channel), [N, K/128] (group-wise) or None (1)."""
    x = _h(x)
    W4 = np.ascontiguousarray(W4)
    assert W4.dtype == np.uint8
    M, K = x.shape
    N = W4.shape[0]
    assert W4.shape[1] * 2 == K
    C = np.empty((M, N), np.float32)
    sp, groups = None, 1
    if scales is not None:
        scales = _h(scales).reshape(N, -1)
        groups = scales.shape[1]
        assert groups in (1, K // 128)
        sp = _p(scales)
    lib().fgo_gemm_w4a16_nk(_p(x), _p(W4), sp, groups, int(zero_point), _p(C), M, N, K)
    return C


def quantize_rows_w4(W, groups: int = 1):
    """W[N,K] fp16 -> (W4 [N,K/2] uint8, scales [N,groups] fp16), zero point 8."""
    W = _h(W)
    N, K = W.shape
    W4 = np.empty((N, K // 2), np.uint8)
    scales = np.empty((N, groups), np.float16)
    lib().fgo_quantize_rows_w4(_p(W), _p(W4), _p(scales), groups, N, K)
    return W4, scales


def quantize_rows_w8(W):
    """W[N,K] fp16 -> (W8 int8, scales fp16), per-output-channel symmetric."""
    W = _h(W)
    N, K = W.shape
    W8 = np.empty((N, K), np.int8)
    scales = np.empty(N, np.float16)
    lib().fgo_quantize_rows_w8(_p(W), _p(W8), _p(scales), N, K)
    return W8, scales


def ref_splitk_bt(M: int, N: int, K: int) -> int:
    return int(lib().fgo_ref_splitk_bt(M, N, K))


# ---- the acceptance rule --------------------------------------------------------------------
def tolerance_excess(out, ref32) -> float:
    """max over elements of |out-ref| / (TOL*max(1,|ref|)); passes iff <= 1."""
    out = np.asarray(out, dtype=np.float32)
    ref32 = np.asarray(ref32, dtype=np.float32)
    assert out.shape == ref32.shape, (out.shape, ref32.shape)
    if not np.all(np.isfinite(out)):
        return float("inf")
    lim = TOL * np.maximum(1.0, np.abs(ref32))
    return float(np.max(np.abs(out - ref32) / lim)) if out.size else 0.0


def check_tolerance(out, ref32, what: str = "") -> None:
    ex = tolerance_excess(out, ref32)
    assert ex <= 1.0, f"{what}: max|d| is {ex:.3f}x the allowed 1e-2*max(1,|ref|)"
