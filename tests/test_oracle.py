"""The CPU oracle against the reference's closed-form known answers (tests/golden/) and its
three restatements against each other."""
import hashlib
import itertools
import json
import os
import random

import numpy as np
import pytest

from helpers import README_CASE, dims_of_test1, random_case, raw_bits, volume

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_shapes.json")


def _golden():
    with open(GOLDEN) as f:
        return json.load(f)


@pytest.mark.parametrize("rec", _golden(), ids=lambda r: "x".join(map(str, r["dims"])) + "_" + "".join(map(str, r["perm"])))
def test_golden_reference_shapes(oracle_mod, rec):
    dims, perm, vol = rec["dims"], rec["perm"], rec["volume"]
    if "sample_pos" in rec:
        for pos, src in list(zip(rec["sample_pos"], rec["sample_src"]))[::4]:
            assert oracle_mod.load().cutt_oracle_source_index(
                len(dims), oracle_mod.oracle._iarr(dims), oracle_mod.oracle._iarr(perm), pos) == src
        # the full transposes must agree with the sampled closed form as well
        a = oracle_mod.index_pattern(vol, 4)
        out = oracle_mod.transpose_blocked(dims, perm, a)
        assert np.array_equal(out[np.array(rec["sample_pos"])], np.array(rec["sample_src"], dtype=np.uint32))
        return
    for elt in (4, 8):
        a = oracle_mod.index_pattern(vol, elt)
        for fn in (oracle_mod.transpose_formula, oracle_mod.transpose_blocked, oracle_mod.transpose_numpy):
            got = fn(dims, perm, a)
            assert hashlib.sha256(np.ascontiguousarray(got).tobytes()).hexdigest() == rec["sha256_elt%d" % elt], \
                (fn.__name__, dims, perm, elt)


def test_readme_example_by_hand(oracle_mod):
    """README.md:94-97 of the reference: (31,549,2,3) with (3,0,2,1) gives (3,31,2,549)."""
    dims, perm = README_CASE
    a = np.arange(volume(dims), dtype=np.int64)
    out = oracle_mod.transpose_formula(dims, perm, a)
    # output index o = i3 + 3*(i0 + 31*(i2 + 2*i1)) holds input index i0 + 31*(i1 + 549*(i2 + 2*i3))
    for (i0, i1, i2, i3) in [(0, 0, 0, 0), (1, 0, 0, 2), (30, 548, 1, 2), (7, 100, 1, 0), (12, 345, 0, 1)]:
        o = i3 + 3 * (i0 + 31 * (i2 + 2 * i1))
        assert out[o] == i0 + 31 * (i1 + 549 * (i2 + 2 * i3))
    assert oracle_mod.source_index_formula_py(dims, perm, 5) == 68077


def test_restatements_agree_on_all_small_permutations(oracle_mod):
    for rank in (2, 3, 4, 5):
        dims = dims_of_test1(rank)
        for perm in itertools.permutations(range(rank)):
            for elt in (4, 8):
                a = raw_bits(volume(dims), elt, rank)
                f = oracle_mod.transpose_formula(dims, list(perm), a)
                assert np.array_equal(f, oracle_mod.transpose_blocked(dims, list(perm), a))
                assert np.array_equal(f, oracle_mod.transpose_numpy(dims, list(perm), a))


def test_restatements_agree_on_random_ranks(oracle_mod):
    rng = random.Random(9)
    for rank in range(2, 16):
        for _ in range(3):
            dims, perm = random_case(rng, rank, 200_000)
            a = raw_bits(volume(dims), 8, rank)
            f = oracle_mod.transpose_formula(dims, perm, a)
            assert np.array_equal(f, oracle_mod.transpose_blocked(dims, perm, a))
            assert np.array_equal(f, oracle_mod.transpose_numpy(dims, perm, a))


def test_pure_python_formula_matches_c(oracle_mod):
    rng = random.Random(3)
    for rank in (2, 4, 7):
        dims, perm = random_case(rng, rank, 50_000)
        lib = oracle_mod.load()
        for o in rng.sample(range(volume(dims)), 200):
            assert lib.cutt_oracle_source_index(rank, oracle_mod.oracle._iarr(dims), oracle_mod.oracle._iarr(perm), o) \
                == oracle_mod.source_index_formula_py(dims, perm, o)


def test_bit_patterns_survive(oracle_mod):
    """NaN payloads, negative zero, denormals: elements are moved as integers."""
    dims, perm = [5, 7, 3], [2, 0, 1]
    a = raw_bits(volume(dims), 8, 1)
    a[:4] = np.array([0x7FF8000000000001, 0xFFF0000000000000, 0x8000000000000000, 0x0000000000000001], dtype=np.uint64)
    out = oracle_mod.transpose_blocked(dims, perm, a.view(np.float64)).view(np.uint64)
    assert sorted(out.tolist()) == sorted(a.tolist())
    assert np.array_equal(out, oracle_mod.transpose_numpy(dims, perm, a))


def test_validation_rules(oracle_mod):
    """src/cutt.cpp:59-82."""
    chk = lambda r, d, p, e: oracle_mod.load().cutt_oracle_check_input(r, oracle_mod.oracle._iarr(d), oracle_mod.oracle._iarr(p), e)
    assert chk(2, [4, 4], [1, 0], 4) == 0
    assert chk(2, [4, 4], [1, 0], 2) != 0
    assert chk(1, [4], [0], 4) != 0
    assert chk(2, [4, 1], [1, 0], 4) != 0
    assert chk(2, [4, 4], [1, 1], 4) != 0
    assert chk(2, [4, 4], [0, 2], 4) != 0
