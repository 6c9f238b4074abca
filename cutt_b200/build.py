"""Builds the native library in-tree.

  cutt_b200/lib/libcutt.so          shared library (C++ API + C ABI), CUDA runtime linked statically
  cutt_b200/lib/libcutt.a           static archive, the drop-in for the original libcutt.a
                                    (consumers link it with g++ ... -lcutt -lcudart)
  cutt_b200/lib/libcutt_hostcheck.so  test-only: planner + host-side plan interpreter (no CUDA)

Device code is compiled for sm_100a only.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "build")

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
GENCODE = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v"] + GENCODE
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unknown-pragmas"]

CU_SOURCES = ["kernels.cu", "bulk_copy.cu", "small_elt.cu", "tma_transpose.cu", "tile2d.cu", "cutt.cu"]
CXX_SOURCES = ["planner.cpp"]
HEADERS = ["permute_desc.h", "permute_tile_impl.h", "planner.h", "kernels.h", "cost_model_data.h", "rowcopy_impl.h", "small_elt_impl.h",
           "tma_transpose.h", "tile2d.h",
           os.path.join("..", "..", "include", "cutt.h"), os.path.join("..", "..", "include", "cutt_c.h"),
           os.path.join("..", "..", "include", "cutt_mg.h")]


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.exists(d) and os.path.getmtime(d) > t for d in deps)


def _run(cmd, log=None):
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.write("$ " + " ".join(cmd) + "\n" + res.stdout + "\n")
    if res.returncode != 0:
        sys.stderr.write(res.stdout)
        raise RuntimeError("build step failed: " + " ".join(cmd))
    return res.stdout


def build(force: bool = False, verbose: bool = False) -> dict:
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    hdrs = [os.path.join(CSRC, h) for h in HEADERS] + [os.path.abspath(__file__)]
    objs = []
    with open(os.path.join(OBJDIR, "build.log"), "a") as log:
        for src in CU_SOURCES:
            s = os.path.join(CSRC, src)
            o = os.path.join(OBJDIR, src + ".o")
            if force or _newer(o, [s] + hdrs):
                out = _run([NVCC] + NVCC_FLAGS + ["-c", s, "-o", o], log)
                if verbose:
                    print(out)
            objs.append(o)
        for src in CXX_SOURCES:
            s = os.path.join(CSRC, src)
            o = os.path.join(OBJDIR, src + ".o")
            if force or _newer(o, [s] + hdrs):
                _run(["g++"] + CXX_FLAGS + ["-c", s, "-o", o], log)
            objs.append(o)
        so = os.path.join(LIBDIR, "libcutt.so")
        if force or _newer(so, objs):
            _run([NVCC, "-shared", "-o", so] + objs + GENCODE, log)
        ar = os.path.join(LIBDIR, "libcutt.a")
        if force or _newer(ar, objs):
            if os.path.exists(ar):
                os.remove(ar)
            _run(["ar", "rcs", ar] + objs, log)
        hc = os.path.join(LIBDIR, "libcutt_hostcheck.so")
        hsrc = [os.path.join(CSRC, "host_interp.cpp"), os.path.join(CSRC, "planner.cpp")]
        if force or _newer(hc, hsrc + hdrs):
            _run(["g++"] + CXX_FLAGS + ["-shared", "-o", hc] + hsrc, log)
    return {"so": so, "a": ar, "hostcheck": hc}


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
