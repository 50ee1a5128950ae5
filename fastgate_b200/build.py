"""In-tree build of the native parts of fastgate_b200 (sm_100a only).

  libfastgate_b200.so   CUDA kernels + C ABI (nvcc; no PyTorch dependency)
  _C.so                 pybind11/torch extension exposing the reference's operator names,
                        a thin layer over the C ABI (g++, links libfastgate_b200.so)

Both land next to this file so that they travel with the source tree.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libfastgate_b200.so")
EXT = os.path.join(HERE, "_C.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-shared",
]


def _newer(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _sources(exts: tuple[str, ...]) -> list[str]:
    out = [os.path.join(CSRC, f) for f in sorted(os.listdir(CSRC)) if f.endswith(exts)]
    out.append(os.path.join(os.path.dirname(HERE), "include", "fastgate_b200.h"))
    return out


def nvcc_path() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: fastgate_b200 needs the CUDA 12.9 toolkit to build")
    return cand


def build_lib(force: bool = False, verbose: bool = False) -> str:
    deps = _sources((".cu", ".cuh", ".h", ".cpp"))
    if not force and _newer(LIB, deps):
        return LIB
    cmd = [nvcc_path(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", LIB, os.path.join(CSRC, "fg_capi.cu"), os.path.join(CSRC, "fg_plan.cpp")]
    subprocess.run(cmd, check=True, cwd=CSRC)
    return LIB


def build_ext(force: bool = False) -> str:
    """pybind11 torch extension; compiled with g++ against the installed torch headers."""
    build_lib(force=False)
    src = os.path.join(CSRC, "fg_torch.cpp")
    deps = [src, LIB, os.path.join(os.path.dirname(HERE), "include", "fastgate_b200.h")]
    if not force and _newer(EXT, deps):
        return EXT
    import torch
    from torch.utils import cpp_extension as ce

    inc = []
    for p in ce.include_paths(device_type="cuda") if "device_type" in ce.include_paths.__code__.co_varnames else ce.include_paths(cuda=True):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cxx11 = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    cmd = [
        "g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={cxx11}",
        "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
        *inc, src, "-o", EXT,
        f"-L{HERE}", "-lfastgate_b200", "-Wl,-rpath,$ORIGIN",
        f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
        f"-Wl,-rpath,{torch_lib}",
    ]
    subprocess.run(cmd, check=True, cwd=CSRC)
    return EXT


def build_all(force: bool = False) -> None:
    build_lib(force)
    build_ext(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print(LIB)
    print(EXT)
