"""Shared helpers of the test-suite (case generators, GPU round trip through the C ABI)."""
from __future__ import annotations

import itertools
import random

import numpy as np


def dims_of_test1(rank: int):
    """Dimensions of the reference's all-permutations test (src/cutt_test.cpp:138-158)."""
    return [2 + r * (16 - 2) // rank for r in range(rank)]


# Hand-picked shapes of the reference's test3 (src/cutt_test.cpp:245-366), (dims, permutation).
TEST3_CASES = [
    ([43, 67], [1, 0]),
    ([65536 * 32, 2], [1, 0]),
    ([1305, 599, 88], [0, 2, 1]),
    ([24, 330, 64, 147], [1, 0, 2, 3]),
    ([2, 5, 9, 12], [0, 1, 2, 3]),
    ([2, 4, 6, 9, 11, 13], [0, 1, 2, 3, 4, 5]),
    ([5, 42, 75, 86, 57], [1, 3, 4, 2, 0]),
    ([5, 3, 2, 9, 14], [0, 1, 3, 2, 4]),
]

# Streaming test of the reference (src/cutt_test.cpp:371-404).
TEST4_CASE = ([24, 32, 16, 36, 43, 9], [5, 1, 4, 2, 3, 0])

# README example of the original library (README.md:94-97).
README_CASE = ([31, 549, 2, 3], [3, 0, 2, 1])


def random_case(rng: random.Random, rank: int, max_vol: int):
    """Seeded stand-in for the reference's time-seeded random test (src/cutt_test.cpp:164-240)."""
    while True:
        dims = [rng.randint(2, 40) for _ in range(rank)]
        vol = 1
        for d in dims:
            vol *= d
        while vol > max_vol:
            i = max(range(rank), key=lambda k: dims[k])
            if dims[i] <= 2:
                break
            vol //= dims[i]
            dims[i] = max(2, dims[i] // 2)
            vol *= dims[i]
        if vol <= max_vol:
            break
    perm = list(range(rank))
    rng.shuffle(perm)
    return dims, perm


def volume(dims):
    v = 1
    for d in dims:
        v *= int(d)
    return v


def raw_bits(vol: int, elt: int, seed: int) -> np.ndarray:
    """Arbitrary bit patterns (NaNs, denormals, negative zero included)."""
    rng = np.random.default_rng(seed)
    if elt == 4:
        return rng.integers(0, 2**32, size=vol, dtype=np.uint64).astype(np.uint32)
    return rng.integers(0, 2**63, size=vol, dtype=np.uint64) * np.uint64(2) + rng.integers(0, 2, size=vol, dtype=np.uint64)


def gpu_transpose(native, dims, perm, elt, host_in: np.ndarray, planner="plan", **kw):
    """Runs the library on the GPU through the C ABI and returns the output as numpy."""
    import torch
    tin = torch.from_numpy(host_in.view(np.int32 if elt == 4 else np.int64)).cuda()
    tout = torch.full_like(tin, -1)
    torch.cuda.synchronize()
    stream = kw.pop("stream", 0)
    if planner == "plan":
        rc, h = native.cuttPlan(len(dims), dims, perm, elt, stream)
    elif planner == "measure":
        rc, h = native.cuttPlanMeasure(len(dims), dims, perm, elt, stream, tin.data_ptr(), tout.data_ptr())
        tout.fill_(-1)
        torch.cuda.synchronize()
    elif planner == "candidate":
        rc, h = native.plan_candidate(dims, perm, elt, kw.pop("index"), stream)
    elif planner == "params":
        rc, h = native.plan_params(dims, perm, elt, stream, **kw)
    else:
        raise ValueError(planner)
    assert rc == native.CUTT_SUCCESS, (rc, dims, perm, elt, planner, kw)
    try:
        rc = native.cuttExecute(h, tin.data_ptr(), tout.data_ptr())
        assert rc == native.CUTT_SUCCESS, rc
        torch.cuda.synchronize()
        desc = native.plan_describe(h)
    finally:
        native.cuttDestroy(h)
    out = tout.cpu().numpy().view(np.uint32 if elt == 4 else np.uint64)
    return out, desc


def assert_bit_exact(got: np.ndarray, want: np.ndarray, what=""):
    got = got.view(np.uint32 if got.dtype.itemsize == 4 else np.uint64)
    want = want.view(got.dtype)
    if got.shape != want.shape or not np.array_equal(got, want):
        bad = np.nonzero(got != want)[0]
        raise AssertionError("mismatch %s: %d of %d differ, first at %d" % (
            what, bad.size, got.size, int(bad[0]) if bad.size else -1))
