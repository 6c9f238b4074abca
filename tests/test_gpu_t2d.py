"""The swizzled two-dimensional tile method (method 7) on the GPU: forced through the parameter
entry point for every tile shape and access width, odd extents (rows on 4- and 8-byte boundaries,
edge tiles), loop dimensions, buffers that are only element-aligned, against the host oracle."""
import json

import numpy as np
import pytest

from helpers import assert_bit_exact, gpu_transpose, raw_bits, volume

pytestmark = pytest.mark.gpu

SHAPES = [
    ([64, 64], [1, 0]), ([129, 130], [1, 0]), ([131, 67], [1, 0]), ([1026, 1031], [1, 0]), ([132, 200], [1, 0]),
    ([36, 8, 44], [2, 1, 0]), ([41, 6, 53], [1, 2, 0]), ([72, 3, 5, 57], [3, 0, 2, 1]), ([25, 4, 3, 2, 40], [4, 2, 0, 3, 1]),
    ([30, 2, 3, 2, 2, 3, 2, 34], [7, 6, 5, 4, 3, 2, 1, 0]), ([585, 585, 7], [1, 0, 2]), ([2047, 5, 1500], [2, 1, 0]),
]


@pytest.mark.parametrize("dims,perm", SHAPES)
def test_forced_tile_shapes_and_widths(native, oracle_mod, dims, perm):
    labels = set()
    for elt in (4, 8):
        a = raw_bits(volume(dims), elt, 53)
        want = oracle_mod.transpose_blocked(dims, perm, a)
        for ta in (128, 256):
            for tb in (32, 64):
                for kw in (dict(nthreads=128, loop_order=0), dict(nthreads=256, loop_order=1), dict(nthreads=128, loop_order=2),
                           dict(nthreads=256, loop_order=3)):
                    rc, h = native.plan_params(dims, perm, elt, 0, method=7, tin=ta, tout=tb * elt, stages=1, **kw)
                    if rc == native.CUTT_INVALID_PARAMETER and kw["loop_order"] >= 2:
                        continue      # banded orders need at least 8 tiles across the band dimension
                    assert rc == 0
                    native.cuttDestroy(h)
                    for maxvec, force in ((16, 0), (16, 1), (8, 0), (4, 0)):
                        if maxvec < elt:
                            continue
                        out, desc = gpu_transpose(native, dims, perm, elt, a, planner="params", method=7, tin=ta,
                                                  tout=tb * elt, stages=1, max_vec=maxvec, extend=force, **kw)
                        label = json.loads(desc)["label"]
                        assert label.startswith("t2d "), desc
                        assert_bit_exact(out, want, desc)
                        labels.add(label.split(" lo=")[0])
    assert len(labels) >= 4
    assert any("in/shift out/shear" in l for l in labels)


def test_rejected_problems(native):
    bad = native.CUTT_INVALID_PARAMETER
    assert native.plan_params([64, 8, 64], [0, 2, 1], 4, 0, method=7, tin=128, tout=128, stages=1)[0] == bad
    assert native.plan_params([64, 64], [1, 0], 4, 0, method=7, tin=192, tout=128, stages=1)[0] == bad
    assert native.plan_params([64, 64], [1, 0], 4, 0, method=7, tin=128, tout=96, stages=1)[0] == bad
    assert native.plan_params([8, 64], [1, 0], 4, 0, method=7, tin=128, tout=128, stages=1)[0] == bad


@pytest.mark.parametrize("off_in,off_out", [(1, 0), (0, 1), (1, 1), (3, 2), (2, 3)])
def test_element_aligned_buffers(native, oracle_mod, off_in, off_out):
    """A plan whose strides allow aligned 16-byte accesses, executed on buffers that start 1-3
    elements past a 16-byte boundary, takes the shift / shear form of the same tile; a plan already
    in that form takes them directly.  The words around the output stay untouched."""
    import torch
    for dims, perm in (([256, 260], [1, 0]), ([131, 67, 5], [1, 0, 2]), ([130, 3, 34], [2, 1, 0])):
        for elt in (4, 8):
            ve = 16 // elt
            vol = volume(dims)
            a = raw_bits(vol, elt, 3)
            dt = torch.int32 if elt == 4 else torch.int64
            oi, oo = off_in % ve, off_out % ve
            big_in = torch.zeros(vol + 8, dtype=dt, device="cuda")
            big_out = torch.full((vol + 8,), -1, dtype=dt, device="cuda")
            big_in[oi:oi + vol] = torch.from_numpy(a.view(np.int32 if elt == 4 else np.int64)).cuda()
            rc, h = native.plan_params(dims, perm, elt, 0, method=7, tin=256, tout=64 * elt, stages=1, nthreads=128)
            assert rc == 0
            assert native.cuttExecute(h, big_in.data_ptr() + oi * elt, big_out.data_ptr() + oo * elt) == 0
            torch.cuda.synchronize()
            native.cuttDestroy(h)
            got = big_out.cpu().numpy().view(np.uint32 if elt == 4 else np.uint64)
            assert_bit_exact(got[oo:oo + vol], oracle_mod.transpose_blocked(dims, perm, a), (dims, perm, elt))
            ones = np.iinfo(got.dtype).max
            assert (got[:oo] == ones).all() and (got[oo + vol:] == ones).all()
