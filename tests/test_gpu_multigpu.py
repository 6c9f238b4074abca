"""Multi-GPU extension on real devices.

* On ONE GPU the ranks of a sharded transpose are emulated one after the other: every "peer"
  output slab is simply another buffer of the same device.  The kernels do not wait for each
  other, so running them back to back is legitimate and exercises the peer-store path.
* With two or more GPUs a child process per rank maps the peers' slabs through CUDA IPC and
  the tiles cross NVLink (skipped when the box has one GPU).
"""
import os
import sys

import numpy as np
import pytest

from helpers import assert_bit_exact, raw_bits, volume

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CASES = [
    ([256, 192, 8, 32], [1, 0, 2, 3]),     # slab
    ([256, 192, 8, 32], [3, 2, 0, 1]),     # all-to-all, shape family of the 34 GB benchmark tensor
    ([96, 64, 40], [2, 0, 1]),
    ([96, 64, 40], [1, 2, 0]),
    ([6, 10, 4, 8, 16], [4, 0, 3, 1, 2]),
    ([130, 128, 24], [2, 1, 0]),
]


@pytest.mark.parametrize("dims,perm", CASES)
@pytest.mark.parametrize("world", [2, 4, 8])
def test_emulated_ranks_on_one_gpu(native, oracle_mod, dims, perm, world):
    import torch
    from cutt_b200 import multigpu as mg
    if dims[-1] % world or dims[perm[-1]] % world:
        pytest.skip("not divisible")
    for elt in (4, 8):
        a = raw_bits(volume(dims), elt, 5)
        want = oracle_mod.transpose_blocked(dims, perm, a)
        loc = volume(dims) // world
        dt = np.int32 if elt == 4 else np.int64
        ins = [torch.from_numpy(a[g * loc:(g + 1) * loc].view(dt).copy()).cuda() for g in range(world)]
        outs = [torch.full((loc,), -1, dtype=ins[0].dtype, device="cuda") for _ in range(world)]
        ptrs = [o.data_ptr() for o in outs]
        for planner in ("plan", "measure"):
            for o in outs:
                o.fill_(-1)
            handles = []
            for g in range(world):
                if planner == "plan":
                    rc, h = mg.mg_plan(dims, perm, elt, world, g, 0)
                else:
                    rc, h = mg.mg_plan_measure(dims, perm, elt, world, g, 0, ins[g].data_ptr(), ptrs)
                assert rc == 0, rc
                handles.append(h)
            if planner == "measure":
                for o in outs:
                    o.fill_(-1)
            expect_mode = 0 if perm[-1] == len(dims) - 1 else 1
            for g, h in enumerate(handles):
                assert mg.mg_mode(h) == expect_mode
                assert mg.mg_execute(h, ins[g].data_ptr(), ptrs) == 0
            torch.cuda.synchronize()
            for h in handles:
                assert native.cuttDestroy(h) == 0
            got = torch.cat(outs).cpu().numpy()
            assert_bit_exact(got, want, "%s %s world=%d %s" % (dims, perm, world, planner))


@pytest.mark.parametrize("world", [2, 4, 8])
def test_candidates_in_both_destination_orders(native, oracle_mod, world):
    """cutt_mg_plan_candidate over the first candidates of an all-to-all problem (emulated ranks):
    both tile orders - destination as an ordinary digit, and destination fastest and rotated by
    the rank - produce the same slabs."""
    import json
    import torch
    from cutt_b200 import multigpu as mg
    dims, perm, elt = [256, 192, 8, 32], [3, 2, 0, 1], 4
    a = raw_bits(volume(dims), elt, 6)
    want = oracle_mod.transpose_blocked(dims, perm, a)
    loc = volume(dims) // world
    ins = [torch.from_numpy(a[g * loc:(g + 1) * loc].view(np.int32).copy()).cuda() for g in range(world)]
    outs = [torch.full((loc,), -1, dtype=torch.int32, device="cuda") for _ in range(world)]
    ptrs = [o.data_ptr() for o in outs]
    n = min(mg.mg_num_candidates(dims, perm, elt, world, g) for g in range(world))
    assert n > 4
    seen = {True: 0, False: 0}
    for index in list(range(min(n, 12))) + [n - 1]:
        for o in outs:
            o.fill_(-1)
        for g in range(world):
            rc, h = mg.mg_plan_candidate(dims, perm, elt, world, g, index)
            assert rc == 0
            if g == 0:
                seen["peers-first" in json.loads(native.plan_describe(h))["label"]] += 1
            assert mg.mg_execute(h, ins[g].data_ptr(), ptrs) == 0
            native.cuttDestroy(h)
        torch.cuda.synchronize()
        assert_bit_exact(torch.cat(outs).cpu().numpy(), want, "world=%d candidate %d" % (world, index))
    assert seen[True] > 0 and seen[False] > 0, seen
    assert mg.mg_plan_candidate(dims, perm, elt, world, 0, n)[0] == native.CUTT_INVALID_PARAMETER
    assert mg.mg_num_candidates(dims, perm, elt, 3, 0) == 0


def test_mg_error_codes(native):
    import torch
    from cutt_b200 import multigpu as mg
    dims, perm = [64, 48, 8, 16], [3, 2, 0, 1]
    assert mg.mg_plan(dims, perm, 4, 3, 0)[0] == native.CUTT_INVALID_PARAMETER     # 16 % 3 != 0
    assert mg.mg_plan(dims, perm, 4, 2, 2)[0] == native.CUTT_INVALID_PARAMETER     # rank out of range
    assert mg.mg_plan(dims, perm, 4, 9, 0)[0] == native.CUTT_INVALID_PARAMETER     # world too large
    rc, h = mg.mg_plan(dims, perm, 4, 2, 0)
    assert rc == 0 and mg.mg_mode(h) == 1
    x = torch.zeros(volume(dims) // 2, dtype=torch.int32, device="cuda")
    y = torch.zeros_like(x)
    # a plain execute cannot serve an all-to-all plan
    assert native.cuttExecute(h, x.data_ptr(), y.data_ptr()) == native.CUTT_INVALID_PARAMETER
    assert mg.mg_execute(h, x.data_ptr(), [y.data_ptr(), x.data_ptr()]) == native.CUTT_INVALID_PARAMETER
    assert native.cuttDestroy(h) == 0
    rc, h = native.cuttPlan(2, [16, 16], [1, 0], 4, 0)
    assert mg.mg_mode(h) == -1
    native.cuttDestroy(h)


def _ipc_worker(rank, world, port, dims, perm, elt, q):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import oracle
    from cutt_b200.multigpu import ShardedTranspose
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        vol = volume(dims)
        loc = vol // world
        a = raw_bits(vol, elt, 7)
        dt = np.int32 if elt == 4 else np.int64
        inp = torch.from_numpy(a[rank * loc:(rank + 1) * loc].view(dt).copy()).cuda()
        ok = True
        for measure in (False, True):
            st = ShardedTranspose(dims, perm, elt, measure_input=inp if measure else None)
            st.out.fill_(-1)
            st.finish()
            st.execute(inp)
            st.finish()
            want = oracle.transpose_blocked(dims, perm, a)[rank * loc:(rank + 1) * loc]
            ok = ok and np.array_equal(st.out.cpu().numpy().view(a.dtype), want)
            st.close()
        flags = [None] * world
        dist.all_gather_object(flags, bool(ok))
        if rank == 0:
            q.put(all(flags))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("dims,perm", [([256, 192, 8, 32], [3, 2, 0, 1]), ([256, 192, 8, 32], [1, 0, 2, 3]),
                                       ([96, 64, 40], [1, 2, 0])])
def test_ipc_ranks_on_several_gpus(native, dims, perm):
    import torch
    import torch.multiprocessing as mp
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 2000)
    procs = [ctx.Process(target=_ipc_worker, args=(r, world, port, dims, perm, 8, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert q.get(timeout=10)
