"""Host side of the multi-GPU extension (include/cutt_mg.h): one rank per GPU.

The original cuTT is single-GPU; everything here is an addition.  A tensor is sharded along its
slowest dimension on the input side and along the output's slowest dimension on the output side.
``mode 0`` (slab) needs no communication; in ``mode 1`` every rank stores its tiles directly into
the peers' output slabs from inside the transpose kernel (CUDA IPC mappings between processes).

``ShardedTranspose`` is written for ``torch.distributed`` process groups (any backend: only small
host objects travel through it; the tensor data moves over NVLink by the kernel's stores).
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence

from . import CUTT_SUCCESS, CuttError, _iarr, lib

IPC_BYTES = 80


def shard_shapes(dims: Sequence[int], perm: Sequence[int], world: int):
    """(local input dims, local output dims, mode) of one rank; raises if not shardable."""
    rank = len(dims)
    s = perm[rank - 1]
    if dims[rank - 1] % world or dims[s] % world:
        raise ValueError("dims[%d]=%d and dims[%d]=%d must both be divisible by world=%d"
                         % (rank - 1, dims[rank - 1], s, dims[s], world))
    local_in = list(dims)
    local_in[rank - 1] //= world
    out_dims = [dims[p] for p in perm]
    out_dims[rank - 1] //= world
    return local_in, out_dims, (0 if s == rank - 1 else 1)


def mg_plan(dims, perm, elt, world, me, stream=0):
    h = ctypes.c_uint(0)
    rc = lib().cutt_mg_plan(ctypes.byref(h), len(dims), _iarr(dims), _iarr(perm), elt, stream, world, me)
    return rc, h.value


def mg_plan_measure(dims, perm, elt, world, me, stream, idata: int, odata: Sequence[int]):
    h = ctypes.c_uint(0)
    arr = (ctypes.c_void_p * len(odata))(*odata)
    rc = lib().cutt_mg_plan_measure(ctypes.byref(h), len(dims), _iarr(dims), _iarr(perm), elt, stream,
                                    world, me, idata, arr)
    return rc, h.value


def mg_num_candidates(dims, perm, elt, world, me) -> int:
    return lib().cutt_mg_num_candidates(len(dims), _iarr(dims), _iarr(perm), elt, world, me)


def mg_plan_candidate(dims, perm, elt, world, me, index, stream=0):
    h = ctypes.c_uint(0)
    rc = lib().cutt_mg_plan_candidate(ctypes.byref(h), len(dims), _iarr(dims), _iarr(perm), elt, stream,
                                      world, me, index)
    return rc, h.value


def mg_execute(handle: int, idata: int, odata: Sequence[int]) -> int:
    arr = (ctypes.c_void_p * len(odata))(*odata)
    return lib().cutt_mg_execute(handle, idata, arr)


def mg_mode(handle: int) -> int:
    return lib().cutt_mg_mode(handle)


def ipc_export(devptr: int) -> bytes:
    buf = ctypes.create_string_buffer(IPC_BYTES)
    rc = lib().cutt_mg_ipc_export(devptr, buf)
    if rc != CUTT_SUCCESS:
        raise CuttError(rc, "ipc_export")
    return buf.raw


def ipc_open(token: bytes) -> int:
    p = ctypes.c_void_p(0)
    rc = lib().cutt_mg_ipc_open(token, ctypes.byref(p))
    if rc != CUTT_SUCCESS:
        raise CuttError(rc, "ipc_open")
    return int(p.value)


def ipc_close(devptr: int) -> None:
    lib().cutt_mg_ipc_close(devptr)


class ShardedTranspose:
    """One rank's view of a sharded transpose inside a torch.distributed job.

    ``out`` is this rank's output slab (a torch tensor owned by the object); ``execute(inp)``
    enqueues the kernel; ``finish()`` synchronises the stream and meets the other ranks at a
    barrier, after which ``out`` is complete everywhere.
    """

    def __init__(self, dims, perm, elt, group=None, measure_input=None, measure_topk=32):
        import torch
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.me = dist.get_rank(group) if dist.is_initialized() else 0
        self.dims, self.perm, self.elt = list(dims), list(perm), elt
        self.local_in, self.local_out, self.mode = shard_shapes(dims, perm, self.world)
        vol = 1
        for d in self.local_in:
            vol *= d
        self.local_volume = vol
        dt = torch.int32 if elt == 4 else torch.int64
        self.out = torch.empty(vol, dtype=dt, device="cuda")
        self.peer_ptrs: List[int] = [0] * self.world
        self._opened: List[int] = []
        self.peer_ptrs[self.me] = self.out.data_ptr()
        if self.mode == 1 and self.world > 1:
            tokens: List[bytes] = [b""] * self.world
            dist.all_gather_object(tokens, ipc_export(self.out.data_ptr()), group=group)
            for h, tok in enumerate(tokens):
                if h != self.me:
                    p = ipc_open(tok)
                    self._opened.append(p)
                    self.peer_ptrs[h] = p
        else:
            self.peer_ptrs = [self.out.data_ptr()] * self.world
        stream = torch.cuda.current_stream().cuda_stream
        self.measured = None
        if measure_input is not None and self.mode == 1 and self.world > 1:
            rc, self.handle = self._measure_together(measure_input, stream, measure_topk)
        elif measure_input is not None:
            self._barrier()
            rc, self.handle = mg_plan_measure(self.dims, self.perm, elt, self.world, self.me, stream,
                                              measure_input.data_ptr(), self.peer_ptrs)
            torch.cuda.synchronize()
            self._barrier()
        else:
            rc, self.handle = mg_plan(self.dims, self.perm, elt, self.world, self.me, stream)
        if rc != CUTT_SUCCESS:
            raise CuttError(rc, "cutt_mg_plan")

    def _barrier(self):
        if self.world > 1:
            self.dist.barrier(group=self.group)

    def _reduce(self, value: float, op: str) -> float:
        """max / min of a host number over the ranks (through a device tensor, so that it works
        with the nccl backend as well as with gloo)."""
        import torch
        dev = "cuda" if self.dist.get_backend(self.group) == "nccl" else "cpu"
        t = torch.tensor([value], dtype=torch.float64, device=dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX if op == "max" else self.dist.ReduceOp.MIN,
                             group=self.group)
        return float(t.item())

    def _measure_together(self, inp, stream, topk):
        """All-to-all plans are chosen by the whole job: every rank builds candidate i of the
        planner's list, all ranks run it at the same time, and the slowest rank's time counts -
        what a rank's stores cost depends on what the other GPUs send meanwhile.  The score of a
        candidate is the slower of two warm runs (as in the single-GPU measurement)."""
        import torch
        n = mg_num_candidates(self.dims, self.perm, self.elt, self.world, self.me)
        n = int(self._reduce(float(n), "min"))
        if n <= 0:
            return CUTT_SUCCESS + 4, None
        best_t, best_i, timings = None, None, []
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        for i in range(min(n, max(1, topk))):
            rc, h = mg_plan_candidate(self.dims, self.perm, self.elt, self.world, self.me, i, stream)
            ok = self._reduce(1.0 if rc == CUTT_SUCCESS else 0.0, "min") > 0.5
            if not ok:
                if rc == CUTT_SUCCESS:
                    from . import cuttDestroy
                    cuttDestroy(h)
                continue
            ts = []
            for rep in range(3):
                torch.cuda.synchronize()
                self._barrier()
                e0.record()
                rc = mg_execute(h, inp.data_ptr(), self.peer_ptrs)
                e1.record()
                torch.cuda.synchronize()
                t = self._reduce(e0.elapsed_time(e1) if rc == CUTT_SUCCESS else 1e30, "max")
                ts.append(t)
                # the first run doubles as warm-up; clearly slower candidates stop after it
                if rep == 0 and best_t is not None and t > 1.3 * best_t:
                    break
            from . import cuttDestroy
            cuttDestroy(h)
            score = max(ts[1:]) if len(ts) == 3 else ts[0]
            timings.append((i, score))
            if len(ts) == 3 and (best_t is None or score < best_t):
                best_t, best_i = score, i
        self._barrier()
        if best_i is None:
            return mg_plan(self.dims, self.perm, self.elt, self.world, self.me, stream)
        self.measured = {"candidate": best_i, "ms": best_t, "timed": len(timings)}
        return mg_plan_candidate(self.dims, self.perm, self.elt, self.world, self.me, best_i, stream)

    def execute(self, inp) -> None:
        rc = mg_execute(self.handle, inp.data_ptr(), self.peer_ptrs)
        if rc != CUTT_SUCCESS:
            raise CuttError(rc, "cutt_mg_execute")

    def finish(self) -> None:
        import torch
        torch.cuda.synchronize()
        self._barrier()

    def close(self) -> None:
        from . import cuttDestroy
        if getattr(self, "handle", None) is not None:
            cuttDestroy(self.handle)
            self.handle = None
        self._barrier()  # nobody may still be writing into a slab that is about to be unmapped
        for p in self._opened:
            ipc_close(p)
        self._opened = []
