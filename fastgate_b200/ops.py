"""The reference's operator names, re-exported from the native extension.

Layout classes (the weight is always the large operand):

* ``KN``  ``op(A[M,K], B[K,N], C[M,N])``      edgemm*, edgemv*, flat_gemm_*   (hk/edgemm.h, hk/flatgemm.h)
* ``NK``  ``op(A[M,K], W[N,K], C[M,N])``      edgemm_*_bt, *_tr_amd, gemm_*_bt (hk/edgemm.h, hk/edgemm_tr.h)
* ``WF``  ``op(W[N,K], x[M,K], C[M,N])``      fastgemv*, fastgemm              (hk/fastgemv.h, czn/fastgemm.h)

All write ``C = A.B`` in place (fp32 accumulation, one rounding to fp16) on the current
CUDA stream and raise ``ValueError`` with the reference's message when K or N is not a
multiple of 128 (hk/edgemm.cu:107-109).  Ops that took a split-K hint ``bz`` still accept it.
``fastgemv_int8`` takes an optional 4th tensor ``scales[N]`` (fp16, one per output channel).
``fastgemv_int4(W4[N,K/2] uint8, x, C, scales=None, zero_point=8)`` is the int4 weight-only sibling
(two unsigned 4-bit weights per byte, low nibble first, hk/utility.cuh:13-36; scales [N] or
[N, K/128]); the reference has the kernel (hk/fastgemv.cuh:394-495) but no operator for it.
"""
from . import _C

KN_OPS = (
    "edgemm", "edgemm_m8n256k64", "edgemm_m8n128k64", "edgemm_m8n128k128", "edgemv_m1n128k64x4",
    "edgemm_m8n128k64x4", "edgemv_m1n256k64x4", "edgemm_m8n128k64x4_amd", "edgemm_m8n256k32x8",
    "flat_gemm_m8n128k64x4_bz1", "flat_gemm_m8n256k32x8_bz1", "flat_gemm_m8n256k64x8",
    "flat_gemm_m8n256k32x16", "flat_gemm_m8n512k32x16", "flat_gemm_m8n64k128x8", "flat_gemm_m8n32k256x8",
)
NK_OPS = (
    "edgemm_m8n128k64x4_bt", "edgemm_m8n128k64x4_tr_amd", "gemm_m8n128k64x4_bt", "gemm_m8n32k128x8_bt",
    "gemm_m8n32k256x8_bt", "gemm_m8n32k256x8_bt_bz2", "gemm_m8n64k128x8_bt_exp",
)
WF_OPS = ("fastgemv", "fastgemv_tuned", "fastgemv_extend", "fastgemm", "fastgemv_int8")
BZ_OPS = (
    "flat_gemm_m8n128k64x4_bz1", "flat_gemm_m8n256k64x8", "flat_gemm_m8n512k32x16", "flat_gemm_m8n64k128x8",
    "flat_gemm_m8n32k256x8", "gemm_m8n32k256x8_bt_bz2", "gemm_m8n64k128x8_bt_exp",
)
COMPARATORS = ("hgemm", "hgemm_tr")

EXTRA = ("linear_nk_push", "push_wait", "push_wait_dev", "push_wait_dev_many", "workspace_status", "quantize_int8", "linear_fused", "fastgemv_int4",
         "quantize_int4", "prepack_kn_to_nk", "prepack_gate_up")

__all__ = list(KN_OPS + NK_OPS + WF_OPS + COMPARATORS + EXTRA) + ["launch_count", "version",
                                                         "KN_OPS", "NK_OPS", "WF_OPS", "BZ_OPS"]

for _n in KN_OPS + NK_OPS + WF_OPS + COMPARATORS + EXTRA + ("launch_count", "version"):
    globals()[_n] = getattr(_C, _n)
del _n
