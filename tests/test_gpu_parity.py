"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.
Bit-exact equality is required everywhere (the path only moves bytes)."""
import itertools
import random

import numpy as np
import pytest

from helpers import (README_CASE, TEST3_CASES, TEST4_CASE, assert_bit_exact, gpu_transpose,
                     random_case, raw_bits, dims_of_test1, volume)

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("elt", [4, 8])
@pytest.mark.parametrize("planner", ["plan", "measure"])
def test_readme_example(native, oracle_mod, elt, planner):
    dims, perm = README_CASE
    a = raw_bits(volume(dims), elt, 1)
    out, desc = gpu_transpose(native, dims, perm, elt, a, planner=planner)
    assert_bit_exact(out, oracle_mod.transpose_formula(dims, perm, a), desc)


@pytest.mark.parametrize("rank", [2, 3, 4, 5, 6, 7])
def test_all_permutations(native, oracle_mod, rank):
    """Every permutation (identity included) of the reference's test1 tensor, both sizes."""
    dims = dims_of_test1(rank)
    vol = volume(dims)
    for elt in (8, 4):
        a = raw_bits(vol, elt, 100 + rank)
        for perm in itertools.permutations(range(rank)):
            out, desc = gpu_transpose(native, dims, list(perm), elt, a)
            assert_bit_exact(out, oracle_mod.transpose_blocked(dims, list(perm), a), "%s %s" % (perm, desc))


@pytest.mark.parametrize("case", range(len(TEST3_CASES)))
@pytest.mark.parametrize("elt", [4, 8])
def test_hand_picked(native, oracle_mod, case, elt):
    dims, perm = TEST3_CASES[case]
    a = oracle_mod.index_pattern(volume(dims), elt)
    for planner in ("plan", "measure"):
        out, desc = gpu_transpose(native, dims, perm, elt, a, planner=planner)
        assert_bit_exact(out, oracle_mod.transpose_blocked(dims, perm, a), desc)


def test_random_ranks(native, oracle_mod):
    rng = random.Random(20240607)
    for rank in range(2, 16):
        for rep in range(12):
            dims, perm = random_case(rng, rank, 400_000)
            for elt in (4, 8):
                a = raw_bits(volume(dims), elt, rank * 100 + rep)
                out, desc = gpu_transpose(native, dims, perm, elt, a)
                assert_bit_exact(out, oracle_mod.transpose_blocked(dims, perm, a), "%s %s %s" % (dims, perm, desc))


@pytest.mark.parametrize("dims,perm", [
    ([31, 549, 2, 3], [3, 0, 2, 1]),
    ([129, 130], [1, 0]),
    ([4, 3, 5, 40, 7, 24], [4, 1, 5, 0, 3, 2]),
    ([1305, 59, 8], [0, 2, 1]),
    ([6, 500, 7], [2, 1, 0]),
    ([1000, 3, 70], [1, 2, 0]),
])
def test_every_candidate(native, oracle_mod, dims, perm):
    for elt in (4, 8):
        n = native.num_candidates(dims, perm, elt)
        assert n > 0
        a = raw_bits(volume(dims), elt, 7)
        want = oracle_mod.transpose_blocked(dims, perm, a)
        for i in range(n):
            out, desc = gpu_transpose(native, dims, perm, elt, a, planner="candidate", index=i)
            assert_bit_exact(out, want, desc)


@pytest.mark.parametrize("kw", [
    dict(max_vec=4, max_v=4), dict(max_vec=8, max_v=8), dict(max_v=4), dict(max_vec=4), dict(stages=1), dict(nthreads=128), dict(nthreads=512),
    dict(nthreads=64, stages=1), dict(tin=128, tout=1024), dict(tin=1024, tout=128, vtarget=32768),
    dict(loop_order=1, extend=1), dict(method=3),
])
def test_forced_parameters(native, oracle_mod, kw):
    rng = random.Random(5)
    cases = [([64, 48, 20], [2, 1, 0]), ([130, 257], [1, 0]), ([8, 6, 30, 50], [3, 0, 2, 1]),
             ([256, 64, 12], [1, 0, 2]), ([96, 40, 33], [0, 2, 1])]
    cases += [random_case(rng, r, 300_000) for r in (3, 4, 5, 6)]
    for dims, perm in cases:
        if perm == sorted(perm):
            continue
        for elt in (4, 8):
            a = raw_bits(volume(dims), elt, 11)
            out, desc = gpu_transpose(native, dims, perm, elt, a, planner="params", **kw)
            assert_bit_exact(out, oracle_mod.transpose_blocked(dims, perm, a), "%s %s %s" % (dims, perm, desc))


@pytest.mark.parametrize("dims,perm", [
    ([317, 107, 6], [0, 2, 1]), ([1305, 59, 8], [0, 2, 1]), ([131, 7, 5, 3], [0, 3, 1, 2]), ([128, 10, 6], [0, 2, 1]),
    ([4099, 5, 3], [0, 2, 1]), ([1031, 5, 4], [0, 2, 1]), ([31713, 75, 6], [0, 2, 1]), ([2, 150, 9, 12], [0, 1, 3, 2]),
])
def test_row_copy_method(native, oracle_mod, dims, perm):
    """Forced strided row copy (method 4): misaligned rows, heads and tails, both element sizes."""
    for elt in (4, 8):
        a = raw_bits(volume(dims), elt, 21)
        out, desc = gpu_transpose(native, dims, perm, elt, a, planner="params", method=4)
        assert "rowcopy" in desc
        assert_bit_exact(out, oracle_mod.transpose_blocked(dims, perm, a), desc)
    # not applicable when the fastest dimension moves, nor for rows shorter than 512 bytes
    rc, _ = native.plan_params([64, 48], [1, 0], 4, method=4)
    assert rc == native.CUTT_INVALID_PARAMETER
    rc, _ = native.plan_params([31, 7, 5], [0, 2, 1], 4, method=4)
    assert rc == native.CUTT_INVALID_PARAMETER


def test_row_copy_unaligned_buffers(native, oracle_mod):
    import torch
    dims, perm = [317, 107, 6], [0, 2, 1]
    vol = volume(dims)
    a = raw_bits(vol, 4, 5)
    big_in = torch.zeros(vol + 3, dtype=torch.int32, device="cuda")
    big_out = torch.full((vol + 3,), -1, dtype=torch.int32, device="cuda")
    big_in[1:vol + 1] = torch.from_numpy(a.view(np.int32)).cuda()
    rc, h = native.plan_params(dims, perm, 4, method=4)
    assert rc == 0
    assert native.cuttExecute(h, big_in.data_ptr() + 4, big_out.data_ptr() + 8) == 0
    torch.cuda.synchronize()
    native.cuttDestroy(h)
    assert_bit_exact(big_out[2:vol + 2].cpu().numpy().view(np.uint32), oracle_mod.transpose_blocked(dims, perm, a))
    assert int(big_out[0].item()) == -1 and int(big_out[1].item()) == -1 and int(big_out[vol + 2].item()) == -1


@pytest.mark.parametrize("dims", [[2, 5, 9, 12], [1000, 1000, 6], [4099, 33, 77], [65536, 64], [8191, 3, 5]])
def test_identity_copy_methods(native, oracle_mod, dims):
    """Identity permutations: the library's copy kernels (bulk-copy-engine path for large aligned
    buffers, vector/word kernels otherwise) and the driver copy, all bit-exact."""
    perm = list(range(len(dims)))
    for elt in (4, 8):
        a = raw_bits(volume(dims), elt, 13)
        for method in (0, 1):
            out, desc = gpu_transpose(native, dims, perm, elt, a, planner="params", method=method)
            assert_bit_exact(out, a, desc)
        out, desc = gpu_transpose(native, dims, perm, elt, a)
        assert_bit_exact(out, a, desc)
    assert native.copy_timeouts() == 0


def test_identity_copy_unaligned(native):
    import torch
    n = 3_000_001
    src = torch.arange(n + 4, dtype=torch.int32, device="cuda")
    dst = torch.full((n + 4,), -1, dtype=torch.int32, device="cuda")
    rc, h = native.plan_params([n // 7, 7], [0, 1], 4, method=0)
    assert rc == 0
    m = (n // 7) * 7
    assert native.cuttExecute(h, src.data_ptr() + 4, dst.data_ptr() + 12) == 0
    torch.cuda.synchronize()
    native.cuttDestroy(h)
    assert torch.equal(dst[3:3 + m], src[1:1 + m])
    assert int(dst[2].item()) == -1 and int(dst[3 + m].item()) == -1
    assert native.copy_timeouts() == 0


def test_identity_copy_equally_misaligned(native):
    """Both buffers miss a 16-byte boundary by the same number of words: a head of one to three
    words, then the aligned body (large enough for the bulk copy engine) and a tail."""
    import torch
    for off in (1, 2, 3):
        n = 9_000_003
        src = torch.arange(n + 8, dtype=torch.int32, device="cuda")
        dst = torch.full((n + 8,), -1, dtype=torch.int32, device="cuda")
        rc, h = native.plan_params([n // 3, 3], [0, 1], 4, method=0)
        assert rc == 0
        assert native.cuttExecute(h, src.data_ptr() + 4 * off, dst.data_ptr() + 4 * off) == 0
        torch.cuda.synchronize()
        native.cuttDestroy(h)
        assert torch.equal(dst[off:off + n], src[off:off + n])
        assert bool((dst[:off] == -1).all()) and bool((dst[off + n:] == -1).all())
        assert native.copy_timeouts() == 0


def test_small_tensor_element_kernel(native, oracle_mod, monkeypatch):
    """Tensors of up to 1 MB: cuttPlan picks the element-per-thread kernel; with that candidate
    switched off the tiled plans still serve the same problem.  Both are bit-exact."""
    import json
    import numpy as np
    import torch
    for dims, perm, elt in [([31, 549, 2, 3], [3, 0, 2, 1], 8), ([300, 340], [1, 0], 4),
                            ([7, 11, 13, 17, 3], [4, 3, 2, 1, 0], 4)]:
        n = int(np.prod(dims))
        a = np.random.default_rng(3).integers(1, 2**31 - 1, n).astype(np.int64 if elt == 8 else np.int32)
        want = oracle_mod.transpose_formula(dims, perm, a)
        src = torch.from_numpy(a).cuda()
        labels = []
        for off in (False, True):
            if off:
                monkeypatch.setenv("CUTT_NO_NAIVE_CANDIDATE", "1")
            else:
                monkeypatch.delenv("CUTT_NO_NAIVE_CANDIDATE", raising=False)
            native.clear_plan_cache()
            dst = torch.zeros_like(src)
            rc, h = native.cuttPlan(len(dims), dims, perm, elt)
            assert rc == 0
            labels.append(json.loads(native.plan_describe(h))["label"])
            assert native.cuttExecute(h, src.data_ptr(), dst.data_ptr()) == 0
            torch.cuda.synchronize()
            native.cuttDestroy(h)
            assert np.array_equal(dst.cpu().numpy(), want), (dims, perm, elt, labels)
        assert labels[0] == "naive" and labels[1] != "naive", labels
    native.clear_plan_cache()


def test_small_tensor_element_kernel_all_permutations(native, oracle_mod, monkeypatch):
    """The element-per-thread kernel with 32-bit indices over every permutation of ranks 2-6 (the
    reference's test1 shapes), chosen by cuttPlan and by cuttPlanMeasure."""
    import itertools
    import json
    monkeypatch.delenv("CUTT_NO_NAIVE_CANDIDATE", raising=False)
    native.clear_plan_cache()
    picked = 0
    for rank in (2, 3, 4, 5, 6):
        dims = dims_of_test1(rank)
        for elt in (4, 8):
            a = raw_bits(volume(dims), elt, 40 + rank)
            for k, perm in enumerate(itertools.permutations(range(rank))):
                if list(perm) == sorted(perm) or (rank == 6 and k % 7):
                    continue
                out, desc = gpu_transpose(native, dims, list(perm), elt, a, planner="measure" if k % 5 == 0 else "plan")
                assert_bit_exact(out, oracle_mod.transpose_blocked(dims, list(perm), a), desc)
                picked += 1 if json.loads(desc)["label"] == "naive" else 0
    native.clear_plan_cache()
    assert picked > 150


def test_streams(native, oracle_mod):
    """Ten plans on ten streams, all writing the same output (src/cutt_test.cpp:371-404)."""
    import torch
    dims, perm = TEST4_CASE
    a = oracle_mod.index_pattern(volume(dims), 8)
    tin = torch.from_numpy(a.view(np.int64)).cuda()
    tout = torch.full_like(tin, -1)
    streams = [torch.cuda.Stream() for _ in range(10)]
    torch.cuda.synchronize()
    handles = []
    for s in streams:
        rc, h = native.cuttPlan(len(dims), dims, perm, 8, s.cuda_stream)
        assert rc == 0
        assert native.cuttExecute(h, tin.data_ptr(), tout.data_ptr()) == 0
        handles.append(h)
    torch.cuda.synchronize()
    for h in handles:
        assert native.cuttDestroy(h) == 0
    assert_bit_exact(tout.cpu().numpy().view(np.uint64), oracle_mod.transpose_blocked(dims, perm, a))


def test_unaligned_pointers(native, oracle_mod):
    """Buffers that are only element-aligned must take the scalar-access variant."""
    import torch
    dims, perm = [64, 48, 20], [2, 1, 0]
    for elt in (4, 8):
        vol = volume(dims)
        a = raw_bits(vol, elt, 3)
        dt = torch.int32 if elt == 4 else torch.int64
        big_in = torch.zeros(vol + 1, dtype=dt, device="cuda")
        big_out = torch.full((vol + 1,), -1, dtype=dt, device="cuda")
        big_in[1:] = torch.from_numpy(a.view(np.int32 if elt == 4 else np.int64)).cuda()
        rc, h = native.cuttPlan(len(dims), dims, perm, elt, 0)
        assert rc == 0
        assert native.cuttExecute(h, big_in.data_ptr() + elt, big_out.data_ptr() + elt) == 0
        torch.cuda.synchronize()
        native.cuttDestroy(h)
        out = big_out[1:].cpu().numpy().view(np.uint32 if elt == 4 else np.uint64)
        assert_bit_exact(out, oracle_mod.transpose_blocked(dims, perm, a))
        assert int(big_out[0].item()) == -1


def test_error_codes_on_device(native):
    import torch
    dims, perm = [16, 16], [1, 0]
    x = torch.zeros(256, dtype=torch.int32, device="cuda")
    y = torch.zeros(256, dtype=torch.int32, device="cuda")
    rc, h0 = native.cuttPlan(2, dims, perm, 4, 0)
    assert rc == native.CUTT_SUCCESS
    # handles count up by one per accepted plan call (src/cutt.cpp:96-97)
    rc, h1 = native.cuttPlan(2, dims, perm, 4, 0)
    assert rc == native.CUTT_SUCCESS and h1 == h0 + 1
    # rejected input does not consume a handle
    rc, _ = native.cuttPlan(2, [16, 1], perm, 4, 0)
    assert rc == native.CUTT_INVALID_PARAMETER
    rc, h2 = native.cuttPlan(2, dims, perm, 8, 0)
    assert rc == native.CUTT_SUCCESS and h2 == h1 + 1
    assert native.cuttExecute(h0, x.data_ptr(), x.data_ptr()) == native.CUTT_INVALID_PARAMETER
    rc, _ = native.cuttPlanMeasure(2, dims, perm, 4, 0, x.data_ptr(), x.data_ptr())
    assert rc == native.CUTT_INVALID_PARAMETER
    assert native.cuttExecute(h0, x.data_ptr(), y.data_ptr()) == native.CUTT_SUCCESS
    for h in (h0, h1, h2):
        assert native.cuttDestroy(h) == native.CUTT_SUCCESS
    assert native.cuttDestroy(h0) == native.CUTT_INVALID_PLAN
    assert native.cuttExecute(h0, x.data_ptr(), y.data_ptr()) == native.CUTT_INVALID_PLAN
    torch.cuda.synchronize()


def test_transpose_host_entry(native, oracle_mod):
    dims, perm = [300, 70, 9], [2, 0, 1]
    for elt in (4, 8):
        a = raw_bits(volume(dims), elt, 9)
        out = np.empty_like(a)
        assert native.transpose_host(dims, perm, elt, a.ctypes.data, out.ctypes.data) == 0
        assert_bit_exact(out, oracle_mod.transpose_blocked(dims, perm, a))
