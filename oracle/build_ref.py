"""Builds the ORIGINAL cuTT (unmodified sources, read where they lie) into oracle/_ref/libcutt_ref.so.

Test infrastructure only.  The original tree has no sm_100 path: its kernels use the
pre-Volta warp intrinsics (__shfl, __ballot without _sync), which nvcc refuses for any
target >= sm_70.  It does compile to PTX for compute_60, which the driver can translate
for the installed GPU at load time.  The sources are compiled directly with nvcc (the
original Makefile is not used); nothing is copied into this repository - only the built
library lands in oracle/_ref/, which git ignores.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SOURCES = ["cutt.cpp", "cuttplan.cpp", "cuttkernel.cu", "cuttGpuModel.cpp", "cuttGpuModelKernel.cu",
           "CudaUtils.cu", "cuttTimer.cpp"]


def build(reference_root: str | None = None, force: bool = False):
    """reference_root: checkout of the original library (argument, else $CUTT_REFERENCE_ROOT).
    Without one, a library built earlier is kept and returned."""
    reference_root = reference_root or os.environ.get("CUTT_REFERENCE_ROOT") or ""
    src = os.path.join(reference_root, "src") if reference_root else ""
    lib = os.path.join(OUT, "libcutt_ref.so")
    if not src or not os.path.isdir(src):
        return lib if os.path.exists(lib) else None
    if os.path.exists(lib) and not force:
        return lib
    os.makedirs(OUT, exist_ok=True)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, "-O3", "-std=c++14", "-shared", "-Xcompiler", "-fPIC", "-x", "cu",
           "-gencode", "arch=compute_60,code=compute_60", "-Wno-deprecated-gpu-targets",
           "-Wno-deprecated-declarations", "-I", src, "-o", lib]
    cmd += [os.path.join(src, s) for s in SOURCES] + [os.path.join(HERE, "ref_shim.cpp")]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    with open(os.path.join(OUT, "build.log"), "w") as f:
        f.write(" ".join(cmd) + "\n" + res.stdout)
    if res.returncode != 0:
        sys.stderr.write(res.stdout[-2000:])
        return None
    return lib


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else None, force=True))
