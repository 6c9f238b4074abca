"""The kernel variant with 64-bit row offsets on the GPU.  Tensors need more than 2^32 elements to
select it by themselves (tests/test_gpu_full_size.py has one); here the planner is told to build
every tile that way, so the variant runs over the reference's test shapes and random ranks."""
import itertools
import json
import random

import pytest

from helpers import README_CASE, TEST3_CASES, assert_bit_exact, dims_of_test1, gpu_transpose, random_case, raw_bits, volume

pytestmark = pytest.mark.gpu


@pytest.fixture()
def wide(native):
    native.clear_plan_cache()
    native.debug_force_wide(True)
    yield native
    native.debug_force_wide(False)
    native.clear_plan_cache()


def test_wide_variant_all_permutations(wide, oracle_mod):
    seen = 0
    for rank in (2, 3, 4, 5):
        dims = dims_of_test1(rank)
        for elt in (4, 8):
            a = raw_bits(volume(dims), elt, rank)
            for perm in itertools.permutations(range(rank)):
                if list(perm) == sorted(perm):
                    continue
                out, desc = gpu_transpose(wide, dims, list(perm), elt, a)
                assert_bit_exact(out, oracle_mod.transpose_blocked(dims, list(perm), a), desc)
                seen += 1 if " wide" in json.loads(desc)["label"] else 0
    assert seen > 100


def test_wide_variant_shapes_and_candidates(wide, oracle_mod):
    rng = random.Random(4)
    cases = [README_CASE, TEST3_CASES[0], TEST3_CASES[2], TEST3_CASES[3], TEST3_CASES[6],
             ([129, 130], [1, 0]), ([4, 3, 5, 40, 7, 24], [4, 1, 5, 0, 3, 2])]
    cases += [random_case(rng, r, 300_000) for r in (3, 4, 5, 6, 7, 9)]
    for dims, perm in cases:
        if perm == sorted(perm):
            continue
        for elt in (4, 8):
            a = raw_bits(volume(dims), elt, 2)
            want = oracle_mod.transpose_blocked(dims, perm, a)
            for planner in ("plan", "measure"):
                out, desc = gpu_transpose(wide, dims, perm, elt, a, planner=planner)
                assert_bit_exact(out, want, desc)
            n = wide.num_candidates(dims, perm, elt)
            for i in sorted(random.Random(elt).sample(range(n), min(n, 8))):
                out, desc = gpu_transpose(wide, dims, perm, elt, a, planner="candidate", index=i)
                assert_bit_exact(out, want, desc)
