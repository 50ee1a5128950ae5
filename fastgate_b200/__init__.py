"""fastgate_b200 — B200 (sm_100a) small-batch matmul operators.

Drop-in for the operator surface of chanzhennan/Fastgate ("SPEEDGATE"): the same free
functions, positional ``(A, B, C)`` order and in-place output as the reference's host
launchers (backend/cuda/hk/edgemm.h:4-14, edgemm_tr.h:7-11, flatgemm.h:4-10,
fastgemv.h:4-7, backend/cuda/czn/fastgemm.h:4), backed by hand-written sm_100a kernels
behind a C ABI (include/fastgate_b200.h).

There is no CPU path and no fallback: importing this package needs the built extension
(``python -m fastgate_b200.build``) and calling an op needs a B200.
"""
import torch as _torch  # noqa: F401  (loads libtorch before the extension)

__version__ = "0.1"

try:
    from . import _C
    from .ops import *  # noqa: F401,F403
    from .ops import __all__ as _ops_all

    __all__ = list(_ops_all)
except (ImportError, AttributeError) as _e:  # missing or stale build
    _import_error = _e
    __all__ = []

    def __getattr__(name):
        # Submodules that need no native code (build, workloads) stay importable so that the
        # extension can be (re)built; every operator fails loudly.
        if name in ("build", "workloads"):
            import importlib

            return importlib.import_module(f"{__name__}.{name}")
        raise ImportError(
            f"fastgate_b200.{name}: the native extension fastgate_b200/_C.so is missing, unloadable or older than "
            "the Python package; run `python -m fastgate_b200.build` (there is no CPU fallback)") from _import_error
