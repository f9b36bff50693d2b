"""Installs the UNMODIFIED reference (DeepGEMM 2.8.1) into baseline/_ref so that its own sm_100 kernel can be timed
beside this repository's on the same GPU.

    python baseline/build_ref.py [--force]

The reference cannot be built as mounted: two of its git submodules are empty directories (third-party/deep_jit, its
whole JIT runtime, and third-party/cutlass).  This script copies the reference to a scratch directory, fills those two
directories -- deep_jit with the stand-in under baseline/deep_jit_standin (written from the reference's call sites),
cutlass with the CUTLASS/CuTe headers that ship inside the image's flashinfer wheel -- and then runs the reference's own
`setup.py` through pip, exactly as a user would:

    pip install --no-index --no-build-isolation --no-deps --target baseline/_ref <scratch copy>

Nothing of the reference's own sources is edited.  baseline/_ref is git-ignored (it holds the reference's package, its
headers and the built extension) and is left out of multi-GPU runs: it is used on one GPU only.
Needs the reference's source tree (DG_REFERENCE_TREE); without it the script reports that and leaves an existing
installation alone.
"""
from __future__ import annotations

import glob
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
REFERENCE = os.environ.get("DG_REFERENCE_TREE", "/root/reference")
TARGET = os.path.join(HERE, "_ref")
STANDIN = os.path.join(HERE, "deep_jit_standin", "include")
SCRATCH = os.environ.get("DG_REFERENCE_SCRATCH", "/tmp/dg_reference_build")


def cutlass_include_dir() -> str | None:
    """CUTLASS >= 4.0 headers (cute/ and cutlass/) bundled with a wheel of the image."""
    site = sysconfig.get_paths()["purelib"]
    for pattern in ("flashinfer/data/cutlass/include", "tilelang/3rdparty/cutlass/include"):
        for cand in glob.glob(os.path.join(site, pattern)):
            if os.path.isfile(os.path.join(cand, "cutlass", "version.h")) and os.path.isdir(os.path.join(cand, "cute")):
                return cand
    return None


def installed() -> bool:
    return bool(glob.glob(os.path.join(TARGET, "deep_gemm", "_C*.so")))


def build(force: bool = False, verbose: bool = True) -> str:
    """Returns "" on success, else one line saying why the reference is not available."""
    if installed() and not force:
        return ""
    if not os.path.isdir(os.path.join(REFERENCE, "csrc")):
        return f"the reference tree {REFERENCE} is not present on this machine"
    cutlass = cutlass_include_dir()
    if cutlass is None:
        return "no CUTLASS >= 4.0 header tree found in the image (flashinfer / tilelang wheels)"
    shutil.rmtree(SCRATCH, ignore_errors=True)
    shutil.copytree(REFERENCE, SCRATCH, ignore=shutil.ignore_patterns(".git", "__pycache__"))
    for sub, src in (("third-party/deep_jit/include", STANDIN), ("third-party/cutlass/include", cutlass)):
        dst = os.path.join(SCRATCH, sub)
        shutil.rmtree(dst, ignore_errors=True)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copytree(src, dst)
    env = dict(os.environ)
    env.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")          # no device code is compiled here; torch insists on a value without a GPU
    env.setdefault("MAX_JOBS", "4")
    env["DG_FORCE_BUILD"] = "1"
    shutil.rmtree(TARGET, ignore_errors=True)
    cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation", "--no-deps", "--find-links", "/opt/wheelhouse",
           "--target", TARGET, SCRATCH]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, env=env, capture_output=True, text=True)
    log = os.path.join(HERE, "_ref_build.log")
    if res.returncode != 0 or not installed():
        with open(log, "w") as f:
            f.write(res.stdout + "\n" + res.stderr)
        tail = (res.stderr or res.stdout).strip().splitlines()[-1:] or ["no output"]
        return f"pip install of the reference failed (log: {log}): {tail[0][:200]}"
    shutil.rmtree(SCRATCH, ignore_errors=True)
    return ""


if __name__ == "__main__":
    why = build(force="--force" in sys.argv)
    print("reference installed in " + TARGET if not why else "reference NOT installed: " + why)
    sys.exit(0 if not why else 1)
