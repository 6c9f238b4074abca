"""Generates tests/golden/reference_shapes.json.

The original cuTT stores no output vectors: its tests fill the input with consecutive 32-bit
words 0,1,2,... (src/TensorTester.cu:33-37) and a checker recomputes, for every output index o,
the expected source index  sum_j ((o / c_j) mod d_j) * ct_j  (src/TensorTester.cu:56-70, constants
from calcTensorConv, :151-170).  That closed form IS the known answer.  This script evaluates it
with numpy int64 arithmetic, independently of the C oracle, on the shapes of the original tests
(src/cutt_test.cpp:138-158, 245-366, 371-404; README.md:94-97) and records

  * for tensors up to 5 M elements: the SHA-256 of the expected output (both element sizes),
  * for larger ones: 512 seeded sample positions with their expected source indices.

Run:  python tests/golden/make_golden.py      (rewrites the JSON next to this file)
"""
import hashlib
import itertools
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
from helpers import README_CASE, TEST3_CASES, TEST4_CASE, dims_of_test1  # noqa: E402


def conv_constants(dims, perm):
    rank = len(dims)
    c = [0] * rank
    ct = [0] * rank
    c[perm[0]] = 1
    ct[0] = 1
    for i in range(1, rank):
        c[perm[i]] = c[perm[i - 1]] * dims[perm[i - 1]]
        ct[i] = ct[i - 1] * dims[i - 1]
    return c, ct


def source_indices(dims, perm, o):
    c, ct = conv_constants(dims, perm)
    o = np.asarray(o, dtype=np.int64)
    src = np.zeros_like(o)
    for j in range(len(dims)):
        src += ((o // c[j]) % dims[j]) * ct[j]
    return src


def expected_output(dims, perm, elt):
    vol = int(np.prod(dims, dtype=np.int64))
    src = source_indices(dims, perm, np.arange(vol, dtype=np.int64))
    if elt == 4:
        return src.astype(np.uint32)
    s = src.astype(np.uint64)
    return ((2 * s + 1) << np.uint64(32)) | (2 * s)


def main():
    cases = [README_CASE, TEST4_CASE] + list(TEST3_CASES)
    for rank in range(2, 8):
        dims = dims_of_test1(rank)
        perms = list(itertools.permutations(range(rank)))
        pick = perms[:3] + perms[-3:] + perms[len(perms) // 2: len(perms) // 2 + 2]
        cases += [(dims, list(p)) for p in pick]
    out = []
    for dims, perm in cases:
        vol = int(np.prod(dims, dtype=np.int64))
        rec = {"dims": list(dims), "perm": list(perm), "volume": vol}
        if vol <= 5_000_000:
            for elt in (4, 8):
                rec["sha256_elt%d" % elt] = hashlib.sha256(expected_output(dims, perm, elt).tobytes()).hexdigest()
        else:
            rng = np.random.default_rng(vol)
            pos = np.sort(rng.integers(0, vol, size=512))
            rec["sample_pos"] = [int(x) for x in pos]
            rec["sample_src"] = [int(x) for x in source_indices(dims, perm, pos)]
        out.append(rec)
    with open(os.path.join(HERE, "reference_shapes.json"), "w") as f:
        json.dump(out, f, indent=0)
    print("wrote %d cases" % len(out))


if __name__ == "__main__":
    main()
