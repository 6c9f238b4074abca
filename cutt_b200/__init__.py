"""cutt_b200 - Blackwell (sm_100a) tensor-transpose library behind the cuTT API.

This package is a thin host-side mirror of the C++ interface declared in ``include/cutt.h``
(``cuttPlan``, ``cuttPlanMeasure``, ``cuttExecute``, ``cuttDestroy``; the original:
src/cutt.h:57-101 of ap-hynninen/cutt).  It binds the library's C ABI (``include/cutt_c.h``)
with ctypes; data pointers are raw device addresses (e.g. ``tensor.data_ptr()``), streams are
raw ``cudaStream_t`` values (e.g. ``torch.cuda.current_stream().cuda_stream``).

There is no CPU fallback: if the native library has not been built the import of the
bindings raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import Sequence

__all__ = [
    "CUTT_SUCCESS", "CUTT_INVALID_PLAN", "CUTT_INVALID_PARAMETER", "CUTT_INVALID_DEVICE",
    "CUTT_INTERNAL_ERROR", "CUTT_UNDEFINED_ERROR", "CuttError", "lib", "lib_path",
    "cuttPlan", "cuttPlanMeasure", "cuttExecute", "cuttDestroy", "plan_describe",
    "num_candidates", "plan_candidate", "plan_params", "transpose_host", "launch_count", "copy_timeouts", "copy_noalloc", "copy_noalloc_timeouts",
    "clear_plan_cache", "debug_force_wide", "plan_cache_save", "plan_cache_load", "plan_cache_size", "Plan",
]

# cuttResult (src/cutt.h:34-41): fixed values
CUTT_SUCCESS = 0
CUTT_INVALID_PLAN = 1
CUTT_INVALID_PARAMETER = 2
CUTT_INVALID_DEVICE = 3
CUTT_INTERNAL_ERROR = 4
CUTT_UNDEFINED_ERROR = 5

_RESULT_NAMES = {
    0: "CUTT_SUCCESS", 1: "CUTT_INVALID_PLAN", 2: "CUTT_INVALID_PARAMETER",
    3: "CUTT_INVALID_DEVICE", 4: "CUTT_INTERNAL_ERROR", 5: "CUTT_UNDEFINED_ERROR",
}

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None


class CuttError(RuntimeError):
    def __init__(self, code: int, what: str = ""):
        self.code = code
        super().__init__("%s%s" % (_RESULT_NAMES.get(code, "code %d" % code), (": " + what) if what else ""))


def lib_path() -> str:
    return os.path.join(_HERE, "lib", "libcutt.so")


def lib() -> ctypes.CDLL:
    """The native library.  Raises if it has not been built (python -m cutt_b200.build)."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise ImportError(
            "cutt_b200: %s is missing - build it with `python -m cutt_b200.build`; "
            "there is no non-CUDA fallback" % path)
    L = ctypes.CDLL(path)
    ip = ctypes.POINTER(ctypes.c_int)
    up = ctypes.POINTER(ctypes.c_uint)
    vp = ctypes.c_void_p
    L.cutt_c_plan.argtypes = [up, ctypes.c_int, ip, ip, ctypes.c_size_t, vp]
    L.cutt_c_plan_measure.argtypes = [up, ctypes.c_int, ip, ip, ctypes.c_size_t, vp, vp, vp]
    L.cutt_c_plan_ext.argtypes = [up, ctypes.c_int, ip, ip, ctypes.c_size_t, vp]
    L.cutt_c_plan_measure_ext.argtypes = [up, ctypes.c_int, ip, ip, ctypes.c_size_t, vp, vp, vp]
    L.cutt_c_execute.argtypes = [ctypes.c_uint, vp, vp]
    L.cutt_c_destroy.argtypes = [ctypes.c_uint]
    L.cutt_c_plan_describe.argtypes = [ctypes.c_uint, ctypes.c_char_p, ctypes.c_size_t]
    L.cutt_c_num_candidates.argtypes = [ctypes.c_int, ip, ip, ctypes.c_size_t]
    L.cutt_c_plan_candidate.argtypes = [up, ctypes.c_int, ip, ip, ctypes.c_size_t, vp, ctypes.c_int]
    L.cutt_c_plan_params.argtypes = [up, ctypes.c_int, ip, ip, ctypes.c_size_t, vp, ctypes.c_int,
                                     ctypes.c_uint, ctypes.c_uint, ctypes.c_uint, ctypes.c_int,
                                     ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    L.cutt_c_transpose_host.argtypes = [ctypes.c_int, ip, ip, ctypes.c_size_t, vp, vp]
    L.cutt_c_launch_count.restype = ctypes.c_ulonglong
    L.cutt_c_clear_plan_cache.restype = None
    L.cutt_c_debug_force_wide.argtypes = [ctypes.c_int]
    L.cutt_c_debug_force_wide.restype = None
    L.cutt_c_version.restype = ctypes.c_char_p
    L.cutt_c_plan_cache_save.argtypes = [ctypes.c_char_p]
    L.cutt_c_plan_cache_load.argtypes = [ctypes.c_char_p]
    L.cutt_c_plan_cache_save.restype = ctypes.c_int
    L.cutt_c_plan_cache_load.restype = ctypes.c_int
    L.cutt_c_plan_cache_size.restype = ctypes.c_int
    L.cutt_c_copy_timeouts.restype = ctypes.c_int
    L.cutt_c_copy_noalloc.argtypes = [vp, vp, ctypes.c_size_t, vp]
    L.cutt_c_copy_noalloc.restype = ctypes.c_int
    L.cutt_c_copy_noalloc_timeouts.restype = ctypes.c_int
    vpp = ctypes.POINTER(ctypes.c_void_p)
    L.cutt_mg_plan.argtypes = [up, ctypes.c_int, ip, ip, ctypes.c_size_t, vp, ctypes.c_int, ctypes.c_int]
    L.cutt_mg_plan_measure.argtypes = [up, ctypes.c_int, ip, ip, ctypes.c_size_t, vp, ctypes.c_int, ctypes.c_int, vp, vpp]
    L.cutt_mg_execute.argtypes = [ctypes.c_uint, vp, vpp]
    L.cutt_mg_num_candidates.argtypes = [ctypes.c_int, ip, ip, ctypes.c_size_t, ctypes.c_int, ctypes.c_int]
    L.cutt_mg_plan_candidate.argtypes = [up, ctypes.c_int, ip, ip, ctypes.c_size_t, vp, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    L.cutt_mg_mode.argtypes = [ctypes.c_uint]
    L.cutt_mg_local_volume.argtypes = [ctypes.c_uint]
    L.cutt_mg_local_volume.restype = ctypes.c_longlong
    L.cutt_mg_ipc_export.argtypes = [vp, ctypes.c_char_p]
    L.cutt_mg_ipc_open.argtypes = [ctypes.c_char_p, vpp]
    L.cutt_mg_ipc_close.argtypes = [vp]
    L.cutt_mg_enable_peer_access.argtypes = [ctypes.c_int]
    for name in ("cutt_mg_plan", "cutt_mg_plan_measure", "cutt_mg_num_candidates", "cutt_mg_plan_candidate", "cutt_mg_execute", "cutt_mg_mode", "cutt_mg_ipc_export",
                 "cutt_mg_ipc_open", "cutt_mg_ipc_close", "cutt_mg_enable_peer_access"):
        getattr(L, name).restype = ctypes.c_int
    for name in ("cutt_c_plan", "cutt_c_plan_measure", "cutt_c_execute", "cutt_c_destroy",
                 "cutt_c_plan_ext", "cutt_c_plan_measure_ext",
                 "cutt_c_plan_describe", "cutt_c_num_candidates", "cutt_c_plan_candidate",
                 "cutt_c_plan_params", "cutt_c_transpose_host"):
        getattr(L, name).restype = ctypes.c_int
    _lib = L
    return L


def _iarr(v: Sequence[int]):
    return (ctypes.c_int * max(1, len(v)))(*[int(x) for x in v])


# --- the four functions of cutt.h; each returns (result_code[, handle]) like the C API ---

def cuttPlan(rank: int, dim: Sequence[int], permutation: Sequence[int], sizeofType: int, stream: int = 0):
    """cuttPlan (src/cutt.h:57-58). Returns (result, handle)."""
    h = ctypes.c_uint(0)
    rc = lib().cutt_c_plan(ctypes.byref(h), rank, _iarr(dim), _iarr(permutation), sizeofType, stream)
    return rc, h.value


def cuttPlanMeasure(rank: int, dim: Sequence[int], permutation: Sequence[int], sizeofType: int,
                    stream: int, idata: int, odata: int):
    """cuttPlanMeasure (src/cutt.h:75-76). Overwrites odata. Returns (result, handle)."""
    h = ctypes.c_uint(0)
    rc = lib().cutt_c_plan_measure(ctypes.byref(h), rank, _iarr(dim), _iarr(permutation), sizeofType,
                                   stream, idata, odata)
    return rc, h.value


def cuttExecute(handle: int, idata: int, odata: int) -> int:
    """cuttExecute (src/cutt.h:101)."""
    return lib().cutt_c_execute(handle, idata, odata)


def cuttDestroy(handle: int) -> int:
    """cuttDestroy (src/cutt.h:87)."""
    return lib().cutt_c_destroy(handle)


# --- additions without a counterpart in the original library ---

def plan_ext(dim: Sequence[int], permutation: Sequence[int], sizeofType: int, stream: int = 0):
    """cuttPlan for element sizes 1, 2, 4, 8 or 16 bytes. Returns (result, handle)."""
    h = ctypes.c_uint(0)
    rc = lib().cutt_c_plan_ext(ctypes.byref(h), len(dim), _iarr(dim), _iarr(permutation), sizeofType, stream)
    return rc, h.value


def plan_measure_ext(dim: Sequence[int], permutation: Sequence[int], sizeofType: int, stream: int,
                     idata: int, odata: int):
    """cuttPlanMeasure for element sizes 1, 2, 4, 8 or 16 bytes. Overwrites odata."""
    h = ctypes.c_uint(0)
    rc = lib().cutt_c_plan_measure_ext(ctypes.byref(h), len(dim), _iarr(dim), _iarr(permutation), sizeofType,
                                       stream, idata, odata)
    return rc, h.value


def plan_describe(handle: int) -> str:
    buf = ctypes.create_string_buffer(4096)
    rc = lib().cutt_c_plan_describe(handle, buf, 4096)
    if rc != CUTT_SUCCESS:
        raise CuttError(rc, "plan_describe")
    return buf.value.decode()


def num_candidates(dim, permutation, sizeofType) -> int:
    return lib().cutt_c_num_candidates(len(dim), _iarr(dim), _iarr(permutation), sizeofType)


def plan_candidate(dim, permutation, sizeofType, index, stream=0):
    h = ctypes.c_uint(0)
    rc = lib().cutt_c_plan_candidate(ctypes.byref(h), len(dim), _iarr(dim), _iarr(permutation),
                                     sizeofType, stream, index)
    return rc, h.value


def plan_params(dim, permutation, sizeofType, stream=0, method=2, tin=256, tout=256, vtarget=16384,
                extend=0, loop_order=0, max_vec=16, max_v=16, nthreads=256, stages=2):
    h = ctypes.c_uint(0)
    rc = lib().cutt_c_plan_params(ctypes.byref(h), len(dim), _iarr(dim), _iarr(permutation), sizeofType,
                                  stream, method, tin, tout, vtarget, extend, loop_order, max_vec,
                                  max_v, nthreads, stages)
    return rc, h.value


def transpose_host(dim, permutation, sizeofType, hin: int, hout: int) -> int:
    """Host buffers in, host buffers out (addresses); copies, executes, synchronises."""
    return lib().cutt_c_transpose_host(len(dim), _iarr(dim), _iarr(permutation), sizeofType, hin, hout)


def launch_count() -> int:
    return int(lib().cutt_c_launch_count())


def copy_timeouts() -> int:
    return int(lib().cutt_c_copy_timeouts())


def copy_noalloc(src: int, dst: int, nbytes: int, stream: int = 0) -> int:
    """Device-to-device copy that allocates nothing (see cutt_c_copy_noalloc in include/cutt_c.h)."""
    return lib().cutt_c_copy_noalloc(src, dst, nbytes, stream)


def copy_noalloc_timeouts() -> int:
    return int(lib().cutt_c_copy_noalloc_timeouts())


def debug_force_wide(on: bool) -> None:
    """Test aid: build every tiled plan with 64-bit row offsets from now on (see cutt_c.h)."""
    lib().cutt_c_debug_force_wide(1 if on else 0)


def clear_plan_cache() -> None:
    lib().cutt_c_clear_plan_cache()


def plan_cache_save(path: str) -> int:
    return lib().cutt_c_plan_cache_save(path.encode())


def plan_cache_load(path: str) -> int:
    return lib().cutt_c_plan_cache_load(path.encode())


def plan_cache_size() -> int:
    return lib().cutt_c_plan_cache_size()


class Plan:
    """RAII convenience around a handle: ``Plan(dim, perm, elt).execute(in_ptr, out_ptr)``."""

    def __init__(self, dim, permutation, sizeofType, stream: int = 0, measure=None):
        if measure is None:
            rc, h = cuttPlan(len(dim), dim, permutation, sizeofType, stream)
        else:
            rc, h = cuttPlanMeasure(len(dim), dim, permutation, sizeofType, stream, measure[0], measure[1])
        if rc != CUTT_SUCCESS:
            raise CuttError(rc, "plan")
        self.handle = h

    def execute(self, idata: int, odata: int) -> None:
        rc = cuttExecute(self.handle, idata, odata)
        if rc != CUTT_SUCCESS:
            raise CuttError(rc, "execute")

    def describe(self) -> str:
        return plan_describe(self.handle)

    def destroy(self) -> None:
        if self.handle is not None:
            cuttDestroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass
