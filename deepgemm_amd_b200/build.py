"""Builds lib/libdeepgemm_b200.so (the C-ABI library) in-tree with nvcc for sm_100a, and _C.so, the compiled
Python binding of the hot GEMM calls (a torch extension that links against the library).

    python deepgemm_amd_b200/build.py            # build what is older than its sources
    python deepgemm_amd_b200/build.py --force

(run it as a script: `python -m deepgemm_amd_b200.build` would import the package, which needs the library)

nvcc cross-compiles without a GPU.  The GEMM kernels themselves are compiled at run time by the
library's JIT runtime (or ahead of time by ``prebuild_kernels``) into ``_jit_cache/``.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libdeepgemm_b200.so")
SOURCES = ["dg_runtime.cpp", "dg_jit.cpp", "dg_gemm.cpp", "dg_layout.cu", "dg_splitk.cu", "dg_quant.cu"]
BINDING_SOURCE = os.path.join(CSRC, "python_binding.cpp")
BINDING_PATH = os.path.join(PKG_DIR, "_C.so")
HEADER = os.path.join(os.path.dirname(PKG_DIR), "include", "deepgemm_b200.h")


def _nvcc() -> str:
    for cand in (os.environ.get("DG_JIT_NVCC_COMPILER"), os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    return "nvcc"


def _newest_source_mtime() -> float:
    newest = 0.0
    for root, _, files in os.walk(CSRC):
        for f in files:
            newest = max(newest, os.path.getmtime(os.path.join(root, f)))
    newest = max(newest, os.path.getmtime(os.path.join(os.path.dirname(PKG_DIR), "include", "deepgemm_b200.h")))
    return newest


def build_library(force: bool = False, verbose: bool = False) -> str:
    if not force and os.path.isfile(LIB_PATH) and os.path.getmtime(LIB_PATH) >= _newest_source_mtime():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    cmd = [_nvcc(), "-std=c++17", "-O3", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
           "-shared", "-Xcompiler", "-fPIC,-Wall,-fvisibility=hidden", "-x", "cu", "-cudart", "static",
           "-DDG_BUILDING_LIBRARY",
           *[os.path.join(CSRC, s) for s in SOURCES], "-o", LIB_PATH + ".tmp", "-ldl"]
    if verbose:
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building {LIB_PATH} failed:\n{res.stdout}\n{res.stderr}")
    os.replace(LIB_PATH + ".tmp", LIB_PATH)
    return LIB_PATH


def build_binding(force: bool = False, verbose: bool = False) -> str:
    """_C.so: g++ on csrc/python_binding.cpp against torch's headers; the C-ABI library is found at run time next to it
    (rpath $ORIGIN/lib) and torch's own libraries are those `import torch` has already loaded."""
    build_library(force=False)
    newest = max(os.path.getmtime(BINDING_SOURCE), os.path.getmtime(HEADER))
    if not force and os.path.isfile(BINDING_PATH) and os.path.getmtime(BINDING_PATH) >= newest:
        return BINDING_PATH
    import sysconfig

    import torch
    from torch.utils import cpp_extension

    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    includes = [*cpp_extension.include_paths(), sysconfig.get_paths()["include"], os.path.join(cuda_home, "include")]
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    # the system g++ (the one nvcc uses as its host compiler), not $CXX: a toolchain wrapper that swaps the start
    # files and unwinder under the compiler produced a module that crashed on its first C++ exception
    cmd = [os.environ.get("DG_HOST_CXX") or shutil.which("g++") or "g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall",
           "-Wno-unused-function", "-DTORCH_EXTENSION_NAME=_C", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-I{i}" for i in includes], BINDING_SOURCE, "-o", BINDING_PATH + ".tmp",
           f"-L{torch_lib}", "-ltorch_python", "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda",
           f"-L{LIB_DIR}", "-ldeepgemm_b200", "-Wl,-rpath,$ORIGIN/lib"]
    if verbose:
        print(" ".join(cmd))
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"building {BINDING_PATH} failed:\n{res.stdout}\n{res.stderr}")
    os.replace(BINDING_PATH + ".tmp", BINDING_PATH)
    return BINDING_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True))
    print(build_binding(force="--force" in sys.argv, verbose=True))
