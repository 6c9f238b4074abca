"""Python side of the CPU oracle (test infrastructure only).

Three independent restatements of the permutation the reference's checker
defines (src/TensorTester.cu:151-170 for the constants, :56-70 for the sum):

* ``source_index_formula_py`` - the checker's formula in pure Python (small cases);
* ``transpose_numpy``         - numpy: Fortran-order reshape, ``transpose(perm)``;
* ``transpose_formula`` / ``transpose_blocked`` - the C library built from
  host_transpose.c (literal formula, and the blocked OpenMP loop nest that the
  benchmark times as the CPU baseline).

Convention (README.md:94-97 of the reference): ``dim[0]`` is the fastest-varying
dimension and ``out_dim[i] = dim[perm[i]]``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SRC = os.path.join(_HERE, "host_transpose.c")
_LIB = os.path.join(_HERE, "liboracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile host_transpose.c into liboracle.so (gcc, OpenMP). Returns the path."""
    if (not force and os.path.exists(_LIB)
            and os.path.getmtime(_LIB) >= os.path.getmtime(_SRC)):
        return _LIB
    # No -march=native: the library is built in one container and run in another.
    cmd = ["gcc", "-O3", "-fopenmp", "-shared", "-fPIC", "-o", _LIB, _SRC]
    subprocess.run(cmd, check=True)
    return _LIB


def load():
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(build())
        ip = ctypes.POINTER(ctypes.c_int)
        for name in ("cutt_oracle_formula", "cutt_oracle_blocked"):
            fn = getattr(lib, name)
            fn.argtypes = [ctypes.c_int, ip, ip, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p]
            fn.restype = ctypes.c_int
        lib.cutt_oracle_source_index.argtypes = [ctypes.c_int, ip, ip, ctypes.c_int64]
        lib.cutt_oracle_source_index.restype = ctypes.c_int64
        lib.cutt_oracle_check_input.argtypes = [ctypes.c_int, ip, ip, ctypes.c_size_t]
        lib.cutt_oracle_check_input.restype = ctypes.c_int
        lib.cutt_oracle_num_threads.restype = ctypes.c_int
        lib.cutt_oracle_set_num_threads.argtypes = [ctypes.c_int]
        lib.cutt_oracle_set_num_threads.restype = ctypes.c_int
        _lib = lib
    return _lib


def _iarr(v: Sequence[int]):
    return (ctypes.c_int * len(v))(*[int(x) for x in v])


def _as_words(a: np.ndarray, elt: int) -> np.ndarray:
    a = np.ascontiguousarray(a).reshape(-1)
    if a.dtype.itemsize != elt:
        raise ValueError("array itemsize %d != element size %d" % (a.dtype.itemsize, elt))
    return a.view(np.uint32 if elt == 4 else np.uint64)


def _call_c(name, dim, perm, a: np.ndarray, out: np.ndarray | None = None) -> np.ndarray:
    elt = a.dtype.itemsize
    src = _as_words(a, elt)
    vol = int(np.prod([int(d) for d in dim], dtype=np.int64))
    if src.size != vol:
        raise ValueError("input has %d elements, dims need %d" % (src.size, vol))
    if out is None:
        dst = np.empty_like(src)
    else:  # caller-owned output (timing loops: no allocation or page faults inside the loop)
        if out.dtype.itemsize != elt or out.size != vol or not out.flags.c_contiguous:
            raise ValueError("out must be a contiguous array of the input's shape and element size")
        dst = out.reshape(-1).view(src.dtype)
    rc = getattr(load(), name)(len(dim), _iarr(dim), _iarr(perm), elt,
                               src.ctypes.data, dst.ctypes.data)
    if rc != 0:
        raise ValueError("oracle rejected the input (code %d)" % rc)
    return dst.view(a.dtype)


def transpose_formula(dim, perm, a: np.ndarray) -> np.ndarray:
    """out[o] = in[sum_j ((o/c_j) mod d_j) ct_j], one element at a time (C)."""
    return _call_c("cutt_oracle_formula", dim, perm, a)


def transpose_blocked(dim, perm, a: np.ndarray, out: np.ndarray | None = None) -> np.ndarray:
    """Blocked OpenMP loop nest (C); the CPU baseline of the benchmark."""
    return _call_c("cutt_oracle_blocked", dim, perm, a, out)


def transpose_numpy(dim, perm, a: np.ndarray) -> np.ndarray:
    """numpy restatement: Fortran-order view, axes permuted, Fortran-order flatten."""
    a = np.ascontiguousarray(a).reshape(-1)
    t = a.reshape(tuple(int(d) for d in dim), order="F").transpose(tuple(int(p) for p in perm))
    return np.ascontiguousarray(t.reshape(-1, order="F"))


def source_index_formula_py(dim, perm, o: int) -> int:
    """The checker's sum for one output index, in plain Python integers."""
    rank = len(dim)
    c = [0] * rank
    ct = [0] * rank
    c[perm[0]] = 1
    ct[0] = 1
    for i in range(1, rank):
        c[perm[i]] = c[perm[i - 1]] * dim[perm[i - 1]]
        ct[i] = ct[i - 1] * dim[i - 1]
    return sum(((o // c[j]) % dim[j]) * ct[j] for j in range(rank))


def index_pattern(vol: int, elt: int) -> np.ndarray:
    """The reference test fixture: consecutive 32-bit words 0,1,2,... over the whole
    buffer (src/TensorTester.cu:33-37); for 8-byte elements element j therefore holds
    the words (2j, 2j+1)."""
    words = np.arange(vol * (elt // 4), dtype=np.uint32)
    return words.view(np.uint32 if elt == 4 else np.uint64)


def num_threads() -> int:
    return int(load().cutt_oracle_num_threads())


def use_all_cores() -> int:
    """Lets the OpenMP loops use every core this process may run on, whatever OMP_NUM_THREADS
    the launcher exported.  Returns the thread count now in effect."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    return int(load().cutt_oracle_set_num_threads(n))
