"""The tensor-map (TMA) transpose on the GPU: forced through the parameter entry point (method 6)
for every tile shape, picked by the planners, edge tiles, loop dimensions, buffers that are not
16-byte aligned (fallback to the tiled kernel), against the host oracle."""
import json
import random

import numpy as np
import pytest

from helpers import assert_bit_exact, gpu_transpose, raw_bits, volume

pytestmark = pytest.mark.gpu

SHAPES = [
    ([64, 64], [1, 0]), ([132, 200], [1, 0]), ([1024, 1028], [1, 0]), ([36, 8, 44], [2, 1, 0]),
    ([40, 6, 52], [1, 2, 0]), ([72, 3, 5, 56], [3, 0, 2, 1]), ([24, 4, 3, 2, 40], [4, 2, 0, 3, 1]),
    ([256, 96, 3], [1, 0, 2]), ([16, 10, 36], [2, 0, 1]), ([2048, 6, 1500], [2, 1, 0]),
]


@pytest.mark.parametrize("dims,perm", SHAPES)
def test_forced_tile_shapes(native, oracle_mod, dims, perm):
    ran = 0
    for elt in (4, 8):
        a = raw_bits(volume(dims), elt, 51)
        want = oracle_mod.transpose_blocked(dims, perm, a)
        for ta in (128, 256, 512):
            for tb in (128, 256, 512):
                for kw in (dict(nthreads=128, stages=4, loop_order=0), dict(nthreads=256, stages=2, loop_order=1)):
                    rc, h = native.plan_params(dims, perm, elt, 0, method=6, tin=ta, tout=tb, **kw)
                    if rc == native.CUTT_INVALID_PARAMETER:
                        continue
                    assert rc == 0
                    native.cuttDestroy(h)
                    out, desc = gpu_transpose(native, dims, perm, elt, a, planner="params", method=6, tin=ta, tout=tb, **kw)
                    assert json.loads(desc)["label"].startswith("tma "), desc
                    assert_bit_exact(out, want, desc)
                    ran += 1
    assert ran >= 4
    assert native.copy_timeouts() == 0


def test_rejected_problems(native):
    bad = native.CUTT_INVALID_PARAMETER
    assert native.plan_params([66, 64], [1, 0], 4, 0, method=6, tin=128, tout=128)[0] == bad   # 264-byte rows
    assert native.plan_params([64, 8, 64], [0, 2, 1], 4, 0, method=6, tin=128, tout=128)[0] == bad
    assert native.plan_params([64, 64], [1, 0], 4, 0, method=6, tin=128, tout=128, stages=0)[0] == bad
    assert native.plan_params([64, 64], [1, 0], 4, 0, method=6, tin=128, tout=128, stages=9)[0] == bad


def test_planners_consider_it_and_stay_exact(native, oracle_mod):
    """cuttPlan / cuttPlanMeasure on problems inside the class (whatever they pick must be exact)
    and every tensor-map candidate of the enumeration."""
    rng = random.Random(8)
    seen = 0
    for dims, perm in [([2048, 2052], [1, 0]), ([512, 12, 516], [2, 1, 0]), ([128, 6, 10, 132], [3, 1, 0, 2])]:
        for elt in (4, 8):
            a = raw_bits(volume(dims), elt, 5)
            want = oracle_mod.transpose_blocked(dims, perm, a)
            for planner in ("plan", "measure"):
                out, desc = gpu_transpose(native, dims, perm, elt, a, planner=planner)
                assert_bit_exact(out, want, desc)
            n = native.num_candidates(dims, perm, elt)
            for i in range(n):
                rc, h = native.plan_candidate(dims, perm, elt, i)
                assert rc == 0
                label = json.loads(native.plan_describe(h))["label"]
                native.cuttDestroy(h)
                if label.startswith("tma "):
                    out, desc = gpu_transpose(native, dims, perm, elt, a, planner="candidate", index=i)
                    assert_bit_exact(out, want, desc)
                    seen += 1
    assert seen >= 12
    assert native.copy_timeouts() == 0


def test_unaligned_buffers_take_the_fallback(native, oracle_mod):
    import torch
    dims, perm = [256, 260], [1, 0]
    for elt in (4, 8):
        vol = volume(dims)
        a = raw_bits(vol, elt, 3)
        dt = torch.int32 if elt == 4 else torch.int64
        big_in = torch.zeros(vol + 1, dtype=dt, device="cuda")
        big_out = torch.full((vol + 1,), -1, dtype=dt, device="cuda")
        big_in[1:] = torch.from_numpy(a.view(np.int32 if elt == 4 else np.int64)).cuda()
        rc, h = native.plan_params(dims, perm, elt, 0, method=6, tin=128, tout=128, stages=3, nthreads=128)
        assert rc == 0
        assert native.cuttExecute(h, big_in.data_ptr() + elt, big_out.data_ptr() + elt) == 0
        torch.cuda.synchronize()
        native.cuttDestroy(h)
        out = big_out[1:].cpu().numpy().view(np.uint32 if elt == 4 else np.uint64)
        assert_bit_exact(out, oracle_mod.transpose_blocked(dims, perm, a))
        assert int(big_out[0].item()) == -1
