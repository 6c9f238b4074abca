"""GPU parity of the extension entry points for 1-, 2- and 16-byte elements
(cutt_c_plan_ext / cutt_c_plan_measure_ext), against the CPU oracle.  The oracle states a
16-byte element as two 8-byte words under an unpermuted innermost dimension of extent 2, and
1/2-byte elements through its dtype-independent numpy restatement."""
import itertools
import random

import numpy as np
import pytest

from helpers import random_case, volume

pytestmark = pytest.mark.gpu


def expected(oracle_mod, dims, perm, elt, raw: np.ndarray) -> np.ndarray:
    """raw: uint8 array of volume*elt bytes.  Returns the permuted bytes."""
    if elt == 16:
        words = raw.view(np.uint64)
        out = oracle_mod.transpose_blocked([2] + list(dims), [0] + [p + 1 for p in perm], words)
        return out.view(np.uint8)
    typed = raw.view(np.uint8 if elt == 1 else np.uint16)
    return oracle_mod.transpose_numpy(dims, perm, typed).view(np.uint8)


def run_ext(native, dims, perm, elt, raw: np.ndarray, planner="plan", offset=0):
    """Runs through the C ABI; `offset` (bytes) shifts both device buffers off their natural
    256-byte alignment."""
    import torch
    n = raw.size
    tin = torch.zeros(n + 64, dtype=torch.uint8, device="cuda")
    tout = torch.full((n + 64,), 0xEE, dtype=torch.uint8, device="cuda")
    tin[offset:offset + n] = torch.from_numpy(raw).cuda()
    pin, pout = tin.data_ptr() + offset, tout.data_ptr() + offset
    torch.cuda.synchronize()
    if planner == "plan":
        rc, h = native.plan_ext(dims, perm, elt, 0)
    else:
        rc, h = native.plan_measure_ext(dims, perm, elt, 0, pin, pout)
        tout.fill_(0xEE)
        torch.cuda.synchronize()
    assert rc == native.CUTT_SUCCESS, (rc, dims, perm, elt, planner)
    try:
        rc = native.cuttExecute(h, pin, pout)
        assert rc == native.CUTT_SUCCESS, (rc, dims, perm, elt)
        torch.cuda.synchronize()
        desc = native.plan_describe(h)
    finally:
        native.cuttDestroy(h)
    host = tout.cpu().numpy()
    assert np.all(host[:offset] == 0xEE) and np.all(host[offset + n:] == 0xEE), "wrote outside the tensor: " + desc
    return host[offset:offset + n], desc


def raw_bytes(n, seed):
    return np.random.default_rng(seed).integers(0, 256, n, dtype=np.uint8)


@pytest.mark.parametrize("elt", [1, 2, 16])
def test_small_shapes_all_permutations(native, oracle_mod, elt):
    for dims in ([3, 5], [4, 6], [8, 3, 5], [2, 3, 4, 5], [7, 66, 5], [130, 70], [258, 3, 9], [132, 76], [8, 12, 20], [2, 5000], [4, 3000]):
        raw = raw_bytes(volume(dims) * elt, 11 + elt)
        for perm in itertools.permutations(range(len(dims))):
            out, desc = run_ext(native, dims, list(perm), elt, raw)
            assert np.array_equal(out, expected(oracle_mod, dims, list(perm), elt, raw)), (dims, perm, elt, desc)


@pytest.mark.parametrize("elt", [1, 2, 16])
def test_random_ranks(native, oracle_mod, elt):
    rng = random.Random(977 + elt)
    for rank in range(2, 11):
        for rep in range(4):
            dims, perm = random_case(rng, rank, 300_000)
            raw = raw_bytes(volume(dims) * elt, rank * 10 + rep)
            out, desc = run_ext(native, dims, perm, elt, raw)
            assert np.array_equal(out, expected(oracle_mod, dims, perm, elt, raw)), (dims, perm, elt, desc)


@pytest.mark.parametrize("elt,dims,perm", [
    (2, [4100, 3001], [1, 0]),            # element-wise kernel, partial tiles on both sides
    (2, [4100, 3002], [1, 0]),            # the same with 4-byte packing on both sides
    (1, [5004, 4100], [1, 0]),
    (1, [5004, 4099], [1, 0]),            # packed loads, element stores
    (1, [5003, 4099], [1, 0]),
    (2, [6, 2000, 700], [2, 0, 1]),       # short fastest dimension
    (2, [64, 300, 500], [0, 2, 1]),       # kept run of 128 bytes: re-stated in 8-byte units
    (1, [36, 300, 700], [0, 2, 1]),       # kept run of 36 bytes: 4-byte units
    (2, [7, 300, 1100], [0, 2, 1]),       # kept run of 14 bytes: element-wise, rows along A
    (16, [300, 257, 40], [2, 0, 1]),
    (16, [1000, 999], [1, 0]),
])
@pytest.mark.parametrize("planner", ["plan", "measure"])
def test_larger_cases(native, oracle_mod, elt, dims, perm, planner):
    raw = raw_bytes(volume(dims) * elt, 5)
    out, desc = run_ext(native, dims, perm, elt, raw, planner=planner)
    assert np.array_equal(out, expected(oracle_mod, dims, perm, elt, raw)), desc


def test_method_choice(native):
    def label(dims, perm, elt):
        rc, h = native.plan_ext(dims, perm, elt, 0)
        assert rc == native.CUTT_SUCCESS
        d = native.plan_describe(h)
        native.cuttDestroy(h)
        return d
    assert '"label": "small' in label([4100, 3001], [1, 0], 2)
    assert '"label": "memcpy"' in label([12, 34, 5], [0, 1, 2], 1)
    assert '"elt": 8' in label([64, 300, 500], [0, 2, 1], 2)
    assert '"elt": 4' in label([36, 300, 700], [0, 2, 1], 1)
    assert '"elt": 8' in label([100, 99], [1, 0], 16)


@pytest.mark.parametrize("elt,dims,perm", [
    (2, [64, 300, 50], [0, 2, 1]),    # re-stated in 8-byte units; the buffers below are not 8-byte aligned
    (1, [36, 30, 70], [0, 2, 1]),
    (16, [30, 25, 40], [2, 0, 1]),
    (2, [301, 200], [1, 0]),
    (2, [300, 200], [1, 0]),          # 4-byte packing planned, dropped for these buffers
    (1, [64, 300], [1, 0]),
])
def test_buffers_aligned_for_the_element_type_only(native, oracle_mod, elt, dims, perm):
    raw = raw_bytes(volume(dims) * elt, 9)
    off = 8 if elt == 16 else elt
    out, desc = run_ext(native, dims, perm, elt, raw, offset=off)
    assert np.array_equal(out, expected(oracle_mod, dims, perm, elt, raw)), desc


def test_rejects_what_it_cannot_do(native):
    import torch
    bad = native.CUTT_INVALID_PARAMETER
    assert native.plan_ext([4, 4], [1, 0], 3, 0)[0] == bad
    assert native.plan_ext([4, 4], [1, 0], 32, 0)[0] == bad
    assert native.plan_ext([4, 1], [1, 0], 2, 0)[0] == bad
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    rc, h = native.plan_ext([10, 12], [1, 0], 2, 0)
    assert rc == native.CUTT_SUCCESS
    try:
        # a 2-byte tensor at an odd address
        assert native.cuttExecute(h, buf.data_ptr() + 1, buf.data_ptr() + 1025) == bad
        assert native.cuttExecute(h, buf.data_ptr(), buf.data_ptr()) == bad   # in place
    finally:
        native.cuttDestroy(h)


def test_two_byte_elements_on_swizzled_tiles(native, oracle_mod):
    """2-byte elements with output rows on 16-byte boundaries run on the two-dimensional tile kernel
    (8 x 8 register transpose); the same plans on buffers shifted by 2 bytes fall back to the
    element-wise kernel; shapes outside the class never leave it."""
    cases = [([64, 72], [1, 0]), ([136, 200], [1, 0]), ([36, 264], [1, 0]), ([34, 8, 40], [2, 1, 0]),
             ([130, 3, 5, 48], [3, 0, 2, 1]), ([72, 6, 136], [1, 2, 0]), ([2000, 2008], [1, 0]), ([1032, 7, 520], [2, 1, 0]),
             ([64, 70], [1, 0]), ([33, 72], [1, 0]),
             ([72, 68], [1, 0]), ([134, 204], [1, 0]), ([40, 5, 132], [2, 1, 0]), ([2004, 2012], [1, 0])]   # 8-byte output rows
    kinds = {}
    for dims, perm in cases:
        raw = raw_bytes(volume(dims) * 2, 77)
        want = expected(oracle_mod, dims, perm, 2, raw)
        for planner in ("plan", "measure"):
            for offset in (0, 2, 16):
                got, desc = run_ext(native, dims, perm, 2, raw, planner=planner, offset=offset)
                assert np.array_equal(got, want), (dims, perm, planner, offset, desc)
        kinds[tuple(dims)] = desc
    assert "t2d " in kinds[(64, 72)] and "t2d " in kinds[(2000, 2008)] and "t2d " in kinds[(34, 8, 40)]
    assert "small" in kinds[(64, 70)] and "small" in kinds[(33, 72)]
    assert "t2d " in kinds[(72, 68)] and "out/w4" in kinds[(2004, 2012)]


def test_one_byte_elements_on_swizzled_tiles(native, oracle_mod):
    """1-byte elements with output rows on 16-byte boundaries run on the two-dimensional tile kernel
    (16 x 16 byte transpose in registers); the same plans on buffers shifted by 1 or 2 bytes fall
    back to the element-wise kernel; shapes outside the class never leave it."""
    cases = [([128, 64], [1, 0]), ([272, 208], [1, 0]), ([72, 272], [1, 0]), ([68, 8, 80], [2, 1, 0]),
             ([260, 3, 5, 48], [3, 0, 2, 1]), ([144, 6, 144], [1, 2, 0]), ([4000, 4016], [1, 0]), ([2064, 7, 528], [2, 1, 0]),
             ([128, 72], [1, 0]), ([66, 80], [1, 0]), ([128, 76], [1, 0]), ([264, 200], [1, 0]), ([72, 5, 136], [2, 1, 0]),
             ([4000, 4008], [1, 0])]
    kinds = {}
    for dims, perm in cases:
        raw = raw_bytes(volume(dims), 78)
        want = expected(oracle_mod, dims, perm, 1, raw)
        for planner in ("plan", "measure"):
            for offset in (0, 1, 2, 16):
                got, desc = run_ext(native, dims, perm, 1, raw, planner=planner, offset=offset)
                assert np.array_equal(got, want), (dims, perm, planner, offset, desc)
        kinds[tuple(dims)] = desc
    assert "t2d " in kinds[(128, 64)] and "t2d " in kinds[(4000, 4016)] and "t2d " in kinds[(68, 8, 80)]
    assert "t2d " in kinds[(128, 72)] and "out/w8" in kinds[(4000, 4008)]          # 8-byte output rows
    assert "small" in kinds[(128, 76)] and "small" in kinds[(66, 80)]
