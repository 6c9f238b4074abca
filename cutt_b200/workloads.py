"""Benchmark workloads: the shapes named by the benchmark configurations, as (dims, perm).

Synthetic, seeded stand-ins for the reference's random benchmark suites
(src/cutt_bench.cpp:440-546 draws ranks, dimensions and permutations from rand()/time seeds,
so nothing reproducible exists upstream): same shape family - about 200 M elements,
ranks 2-7, random dimensions and permutations.
"""
from __future__ import annotations

import json
import math
import os
import random

_HERE = os.path.dirname(os.path.abspath(__file__))
C3_FILE = os.path.join(_HERE, "c3_cases.json")

C1 = ([31, 549, 2, 3], [3, 0, 2, 1])                      # README example, fp64
C2 = ([14142, 14142], [1, 0])                             # matrix transpose, fp32 and fp64
C4 = ([4, 3, 5, 400, 7, 2400], [4, 1, 5, 0, 3, 2])        # tiny leading dimensions, fp32
C5_DIMS = [1024, 1024, 32, 256]                           # multi-GPU tensor, fp32, sharded on the last dim
C5A_PERM = [1, 0, 2, 3]
C5B_PERM = [3, 2, 0, 1]


def _volume(dims):
    v = 1
    for d in dims:
        v *= d
    return v


def generate_c3_case(i: int, target: float = 2.0e8, tol: float = 0.05):
    """Case i of the random rank 2-7 suite (deterministic in i)."""
    seed = 1000 + i
    while True:
        rng = random.Random(seed)
        rank = 2 + rng.randrange(6)
        dims = [int(round(2.0 ** (1.0 + 15.0 * rng.random()))) for _ in range(rank)]
        scale = (target / _volume(dims)) ** (1.0 / rank)
        dims = [max(2, int(round(d * scale))) for d in dims]
        # nudge the largest dimension until the volume is within tolerance
        ok = False
        for _ in range(64):
            vol = _volume(dims)
            if abs(vol - target) <= tol * target:
                ok = True
                break
            k = max(range(rank), key=lambda j: dims[j])
            rest = vol // dims[k]
            dims[k] = max(2, int(round(target / rest)))
            if abs(_volume(dims) - target) > tol * target and dims[k] == 2:
                break
        ok = ok or abs(_volume(dims) - target) <= tol * target
        if ok and all(2 <= d <= 2**31 - 1 for d in dims):
            perm = list(range(rank))
            while perm == list(range(rank)):
                rng.shuffle(perm)
            return dims, perm
        seed += 100000


def c3_cases(n: int = 100):
    """The committed case list (regenerated and compared by the tests)."""
    if os.path.exists(C3_FILE):
        with open(C3_FILE) as f:
            cases = json.load(f)
        return [(c["dims"], c["perm"]) for c in cases[:n]]
    return [generate_c3_case(i) for i in range(n)]


def c3_holdout_cases(n: int = 100):
    """Further cases of the same generator (seeds 2000 and up) that the planner's cost model was
    never fitted to: its training sweep covered cases 0-199 (seeds 1000-1199)."""
    return [generate_c3_case(1000 + i) for i in range(n)]


# Bounded sample of the multi-GPU tensor for legs that run on the host cores or through host
# buffers: the same permutation on a slab of 32 positions of the sharded dimension (4.29 GB per side).
C5_SAMPLE_DIMS = [1024, 1024, 32, 32]


def write_c3_file(n: int = 100):
    cases = [generate_c3_case(i) for i in range(n)]
    with open(C3_FILE, "w") as f:
        f.write("[\n" + ",\n".join(json.dumps({"dims": d, "perm": p}) for d, p in cases) + "\n]\n")
    return cases


if __name__ == "__main__":
    for d, p in write_c3_file():
        print(d, p, _volume(d))
