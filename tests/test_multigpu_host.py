"""Host-side logic of the multi-GPU extension, on CPU: the sharding arithmetic and the
per-rank tile descriptors are executed by the host interpreter; a two-process gloo job plays
the ranks, the "peer stores" become per-destination staging arrays exchanged with all_to_all."""
import ctypes
import os
import sys

import numpy as np
import pytest

from helpers import raw_bits, volume

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _hostcheck():
    lib = ctypes.CDLL(os.path.join(ROOT, "cutt_b200", "lib", "libcutt_hostcheck.so"))
    ip = ctypes.POINTER(ctypes.c_int)
    lib.cutt_hostcheck_run_sharded.argtypes = [ctypes.c_int, ip, ip, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                               ctypes.c_char_p, ctypes.c_int]
    return lib


def _iarr(v):
    return (ctypes.c_int * len(v))(*v)


CASES = [
    ([64, 48, 8, 16], [1, 0, 2, 3]),      # slab mode (config C5a in miniature)
    ([64, 48, 8, 16], [3, 2, 0, 1]),      # all-to-all (C5b in miniature)
    ([32, 16, 8], [2, 0, 1]),
    ([32, 16, 8], [1, 2, 0]),
    ([6, 10, 4, 8, 12], [4, 0, 3, 1, 2]),
    ([128, 130, 8], [2, 1, 0]),
]


@pytest.mark.parametrize("dims,perm", CASES)
@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_sharded_plan_in_one_process(native, oracle_mod, dims, perm, world):
    from cutt_b200.multigpu import shard_shapes
    if dims[-1] % world or dims[perm[-1]] % world:
        with pytest.raises(ValueError):
            shard_shapes(dims, perm, world)
        return
    lib = _hostcheck()
    local_in, local_out, mode = shard_shapes(dims, perm, world)
    assert volume(local_in) == volume(local_out) == volume(dims) // world
    for elt in (4, 8):
        a = raw_bits(volume(dims), elt, 3)
        want = oracle_mod.transpose_blocked(dims, perm, a)
        loc = volume(dims) // world
        outs = [np.zeros(loc, dtype=a.dtype) for _ in range(world)]
        ptrs = (ctypes.c_void_p * world)(*[o.ctypes.data for o in outs])
        for index in (0, 3):
            for o in outs:
                o[:] = 0
            for g in range(world):
                src = np.ascontiguousarray(a[g * loc:(g + 1) * loc])
                m = lib.cutt_hostcheck_run_sharded(len(dims), _iarr(dims), _iarr(perm), elt, world, g, index,
                                                   src.ctypes.data, ptrs, None, 0)
                assert m == mode, (m, mode)
            assert np.array_equal(np.concatenate(outs), want), (dims, perm, world, elt, index)


@pytest.mark.parametrize("world", [2, 4, 8])
def test_both_destination_orders(native, oracle_mod, world):
    """All-to-all plans exist in two tile orders: destination GPU as an ordinary digit of the tile
    index, and destination fastest, rotated by the rank ("peers-first").  Both must give the
    same output."""
    lib = _hostcheck()
    dims, perm, elt = [64, 48, 8, 16], [3, 2, 0, 1], 4
    a = raw_bits(volume(dims), elt, 4)
    want = oracle_mod.transpose_blocked(dims, perm, a)
    loc = volume(dims) // world
    outs = [np.zeros(loc, dtype=a.dtype) for _ in range(world)]
    ptrs = (ctypes.c_void_p * world)(*[o.ctypes.data for o in outs])
    seen = {True: 0, False: 0}
    for index in range(24):
        for o in outs:
            o[:] = 0
        first = None
        for g in range(world):
            src = np.ascontiguousarray(a[g * loc:(g + 1) * loc])
            lab = ctypes.create_string_buffer(4096)
            m = lib.cutt_hostcheck_run_sharded(len(dims), _iarr(dims), _iarr(perm), elt, world, g, index,
                                               src.ctypes.data, ptrs, lab, 4096)
            assert m == 1
            if g == 0:
                first = "peers-first" in lab.value.decode()
        seen[first] += 1
        assert np.array_equal(np.concatenate(outs), want), (world, index)
    assert seen[True] > 0 and seen[False] > 0, seen


def _gloo_worker(rank, world, port, dims, perm, elt, result_queue):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lib = _hostcheck()
        vol = volume(dims)
        loc = vol // world
        a = raw_bits(vol, elt, 3)                       # every rank can rebuild the global tensor
        mine = np.ascontiguousarray(a[rank * loc:(rank + 1) * loc])
        # this rank's stores, one staging array per destination (zero where it writes nothing)
        staged = [np.zeros(loc, dtype=a.dtype) for _ in range(world)]
        ptrs = (ctypes.c_void_p * world)(*[s.ctypes.data for s in staged])
        mode = lib.cutt_hostcheck_run_sharded(len(dims), _iarr(dims), _iarr(perm), elt, world, rank, 0,
                                              mine.ctypes.data, ptrs, None, 0)
        assert mode in (0, 1)
        send = [torch.from_numpy(s.view(np.int64 if elt == 8 else np.int32)) for s in staged]
        recv = [torch.empty_like(t) for t in send]
        # gloo has no all_to_all: exchange with point-to-point sends in a fixed order
        reqs = []
        for h in range(world):
            if h == rank:
                recv[h].copy_(send[h])
            else:
                reqs.append(dist.isend(send[h], h))
                reqs.append(dist.irecv(recv[h], h))
        for r in reqs:
            r.wait()
        # every output element has exactly one writer, so the sum over sources is the value
        total = torch.zeros_like(recv[0])
        for t in recv:
            total += t
        want = oracle.transpose_blocked(dims, perm, a)[rank * loc:(rank + 1) * loc]
        ok = np.array_equal(total.numpy().view(a.dtype), want)
        flags = [None] * world
        dist.all_gather_object(flags, bool(ok))
        if rank == 0:
            result_queue.put((mode, all(flags)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("dims,perm", [([64, 48, 8, 16], [3, 2, 0, 1]), ([64, 48, 8, 16], [1, 0, 2, 3]),
                                       ([32, 16, 8], [1, 2, 0])])
def test_two_gloo_ranks(native, dims, perm):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, dims, perm, 8, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    mode, ok = q.get(timeout=10)
    assert ok
    assert mode == (0 if perm[-1] == len(dims) - 1 else 1)
