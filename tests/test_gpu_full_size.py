"""Parity at the sizes the benchmark numbers are quoted on: the plans cuttPlanMeasure picks for the
~200 M-element benchmark tensors, the 403 M-element small-leading-dimension tensor, a tensor of more
than 2^32 elements (64-bit tile offsets), checked bit for bit against the host oracle and against
the 64-bit index checker (the role of src/TensorTester.cu:39-96 in the reference's own tests)."""
import json

import numpy as np
import pytest

from helpers import volume

pytestmark = pytest.mark.gpu


def _device_input(vol, elt, seed):
    import torch
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    words = torch.randint(-2**31, 2**31 - 1, (vol * (elt // 4),), dtype=torch.int32, device="cuda", generator=g)
    return words.view(torch.int32 if elt == 4 else torch.int64)


def _run(native, dims, perm, elt, tin, measure=True):
    import torch
    tout = torch.full_like(tin, -1)
    s = torch.cuda.current_stream().cuda_stream
    if measure:
        rc, h = native.cuttPlanMeasure(len(dims), dims, perm, elt, s, tin.data_ptr(), tout.data_ptr())
        tout.fill_(-1)
    else:
        rc, h = native.cuttPlan(len(dims), dims, perm, elt, s)
    assert rc == 0
    assert native.cuttExecute(h, tin.data_ptr(), tout.data_ptr()) == 0
    torch.cuda.synchronize()
    label = json.loads(native.plan_describe(h))["label"]
    native.cuttDestroy(h)
    return tout, label


def _against_host_oracle(oracle_mod, dims, perm, tin, tout, what):
    """Downloads the input, permutes it on the host cores, uploads the result and compares on the
    device (bit patterns)."""
    import torch
    a = tin.cpu().numpy()
    want = torch.from_numpy(oracle_mod.transpose_blocked(dims, perm, a)).cuda()
    assert torch.equal(tout, want), what


@pytest.mark.parametrize("elt", [4, 8])
def test_matrix_transpose_full_size(native, oracle_mod, elt):
    from cutt_b200 import workloads as W
    from oracle import device_check as DC
    oracle_mod.use_all_cores()
    dims, perm = W.C2
    tin = _device_input(volume(dims), elt, 11)
    tout, label = _run(native, dims, perm, elt, tin)
    _against_host_oracle(oracle_mod, dims, perm, tin, tout, label)
    assert DC.count_mismatches(dims, perm, tout, tin) == 0, label


def test_small_leading_dimensions_full_size(native, oracle_mod):
    from cutt_b200 import workloads as W
    from oracle import device_check as DC
    oracle_mod.use_all_cores()
    dims, perm = W.C4
    tin = _device_input(volume(dims), 4, 12)
    for measure in (False, True):
        tout, label = _run(native, dims, perm, 4, tin, measure=measure)
        _against_host_oracle(oracle_mod, dims, perm, tin, tout, label)
        assert DC.count_mismatches(dims, perm, tout, tin) == 0, label


def test_random_suite_full_size(native, oracle_mod):
    """All 100 suite tensors, both element sizes.  The first 25 are planned by measurement and
    compared with the host oracle; all are compared with the index checker."""
    import torch
    from cutt_b200 import workloads as W
    from oracle import device_check as DC
    oracle_mod.use_all_cores()
    cases = W.c3_cases(100)
    maxvol = max(volume(d) for d, _ in cases)
    words = _device_input(maxvol, 8, 13)
    labels = set()
    for ci, (dims, perm) in enumerate(cases):
        vol = volume(dims)
        for elt in (8, 4):
            tin = words.view(torch.int32 if elt == 4 else torch.int64)[:vol]
            tout, label = _run(native, dims, perm, elt, tin, measure=ci < 25)
            labels.add(label.split(" t=")[0])
            assert DC.count_mismatches(dims, perm, tout, tin) == 0, (ci, dims, perm, elt, label)
            if ci < 25:
                _against_host_oracle(oracle_mod, dims, perm, tin, tout, (ci, dims, perm, elt, label))
            del tout
    assert labels  # (plan families seen: tiles, rowcopy, ...)


def test_more_than_2_32_elements(native):
    """4.36 G elements (17.4 GB per side): element offsets beyond 32 bits in the tile decoder, and
    for the permutation that moves the slowest dimension to the front a tile that spans more
    than 2^32 elements, which selects the kernel variant with 64-bit row offsets."""
    import torch
    from oracle import device_check as DC
    dims = [1024, 1024, 32, 130]
    vol = volume(dims)
    assert vol > 2**32
    free, _ = torch.cuda.mem_get_info()
    if free < 3 * vol * 4:
        pytest.skip("needs %.0f GB of free device memory" % (3 * vol * 4 / 1e9))
    tin = torch.empty(vol, dtype=torch.int32, device="cuda")
    DC.fill_pattern(tin)
    tout = torch.empty_like(tin)
    s = torch.cuda.current_stream().cuda_stream
    wide_seen = False
    for perm, planner in (([1, 0, 2, 3], "plan"), ([1, 0, 2, 3], "measure"), ([3, 2, 0, 1], "plan"),
                          ([3, 2, 0, 1], "measure"), ([3, 2, 0, 1], "params")):
        if planner == "plan":
            rc, h = native.cuttPlan(4, dims, perm, 4, s)
        elif planner == "measure":
            rc, h = native.cuttPlanMeasure(4, dims, perm, 4, s, tin.data_ptr(), tout.data_ptr())
        else:   # a tile over the whole slowest dimension: 129 * 2^25 elements between its rows
            rc, h = native.plan_params(dims, perm, 4, s, tin=256, tout=1024, vtarget=32768)
        assert rc == 0, (perm, planner)
        label = json.loads(native.plan_describe(h))["label"]
        wide_seen = wide_seen or " wide" in label
        tout.fill_(-1)
        assert native.cuttExecute(h, tin.data_ptr(), tout.data_ptr()) == 0
        torch.cuda.synchronize()
        native.cuttDestroy(h)
        assert DC.count_mismatches(dims, perm, tout, None) == 0, (perm, planner, label)
        if planner == "params":
            assert " wide" in label, label
    assert wide_seen
