"""Builds lib/libdeepgemm_b200.so (the C-ABI library) in-tree with nvcc for sm_100a.

    python deepgemm_amd_b200/build.py            # build if sources are newer than the library
    python deepgemm_amd_b200/build.py --force

(run it as a script: `python -m deepgemm_amd_b200.build` would import the package, which needs the library)

nvcc cross-compiles without a GPU.  The GEMM kernels themselves are compiled at run time by the
library's JIT runtime (or ahead of time by ``prebuild_kernels``) into ``_jit_cache/``.
"""
from __future__ import annotations

import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libdeepgemm_b200.so")
SOURCES = ["dg_runtime.cpp", "dg_jit.cpp", "dg_gemm.cpp", "dg_layout.cu", "dg_splitk.cu", "dg_quant.cu"]


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


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose=True))
