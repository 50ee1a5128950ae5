"""TEST INFRASTRUCTURE ONLY: builds the reference's own hot-path kernels for sm_100a.

The unmodified sources backend/cuda/hk/{edgemm,edgemm_tr,flatgemm,fastgemv}.cu and
backend/cuda/czn/fastgemm.cu are compiled from the reference checkout where it lies
(nothing is copied into this repository) and linked with ref_shim.cpp into
oracle/_ref/fastgate_ref.so, a torch extension.  ref_int4_launch.cu adds a launcher for
gemv_quantized_int4, a kernel the reference defines (hk/fastgemv.cuh:394-495) but never launches.  The reference's own setup.py is not used:
it lists source files that do not exist and defaults to another vendor's backend.

The result serves two purposes, both as a checker / comparator, never as the product:
  * GPU tests compare the new kernels with the reference's kernels on identical inputs;
  * bench.py can time the reference's kernels on the same B200.

Usage: python oracle/build_ref.py [/path/to/reference]
The checkout is looked for at the argument, else at $FASTGATE_REFERENCE; without either (or
when the path does not exist) nothing is built and an earlier build is reused.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SOURCES = ("hk/edgemm.cu", "hk/edgemm_tr.cu", "hk/flatgemm.cu", "hk/fastgemv.cu", "czn/fastgemm.cu")


def reference_root() -> str | None:
    """The reference checkout named by $FASTGATE_REFERENCE, if it is there."""
    root = os.environ.get("FASTGATE_REFERENCE", "")
    return root if root and os.path.isdir(os.path.join(root, "backend", "cuda")) else None


def build(reference: str | None = None, force: bool = False) -> str | None:
    reference = reference or reference_root() or ""
    cuda_dir = os.path.join(reference, "backend", "cuda")
    target = os.path.join(OUT, "fastgate_ref.so")
    if not reference or not os.path.isdir(cuda_dir):
        return target if os.path.exists(target) else None
    if os.path.exists(target) and not force:
        return target
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(OUT, exist_ok=True)
    inc = []
    for p in ce.include_paths(cuda=True) if "cuda" in ce.include_paths.__code__.co_varnames else ce.include_paths("cuda"):
        inc += ["-isystem", p]
    inc += ["-isystem", sysconfig.get_paths()["include"]]
    inc += ["-I", cuda_dir, "-I", os.path.join(cuda_dir, "hk"), "-I", os.path.join(cuda_dir, "czn"),
            "-I", os.path.join(cuda_dir, "common")]
    cxx11 = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    common = ["-std=c++17", "-O2", f"-D_GLIBCXX_USE_CXX11_ABI={cxx11}", "-DTORCH_EXTENSION_NAME=fastgate_ref",
              "-DTORCH_API_INCLUDE_EXTENSION_H", "-DNDEBUG"]
    nvcc = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "--expt-relaxed-constexpr",
            "-U__CUDA_NO_HALF_OPERATORS__", "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF2_OPERATORS__",
            "-Xcompiler", "-fPIC", "-w", *common, *inc, "-c"]

    def compile_one(rel: str) -> str:
        obj = os.path.join(OUT, rel.replace("/", "_").replace(".cu", ".o"))
        subprocess.run([*nvcc, os.path.join(cuda_dir, rel), "-o", obj], check=True)
        return obj

    def compile_launcher() -> str:  # our launcher around the reference's int4 kernel (no launcher upstream)
        obj = os.path.join(OUT, "ref_int4_launch.o")
        subprocess.run([*nvcc, os.path.join(HERE, "ref_int4_launch.cu"), "-o", obj], check=True)
        return obj

    with ThreadPoolExecutor(max_workers=6) as ex:
        launcher = ex.submit(compile_launcher)
        objs = list(ex.map(compile_one, SOURCES)) + [launcher.result()]
    shim_obj = os.path.join(OUT, "ref_shim.o")
    subprocess.run(["g++", "-fPIC", "-w", *common, *inc, "-c", os.path.join(HERE, "ref_shim.cpp"), "-o", shim_obj],
                   check=True)
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    subprocess.run(["nvcc", "-shared", "-o", target, shim_obj, *objs, f"-L{torch_lib}", "-ltorch", "-ltorch_cpu",
                    "-lc10", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda",
                    "-Xlinker", f"-rpath={torch_lib}"], check=True)
    return target


if __name__ == "__main__":
    args = [a for a in sys.argv[1:] if not a.startswith("--")]
    print(build(args[0] if args else None, force="--force" in sys.argv))
