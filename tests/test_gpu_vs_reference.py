"""Parity with the ORIGINAL cuTT itself, where it can run: oracle/_ref/libcutt_ref.so is the
unmodified reference compiled to compute_60 PTX (the only form it compiles to with a current
toolkit), which the driver translates for the installed GPU.  For every case the reference's
output, this library's output and the CPU oracle's output must be identical bit for bit.
Skipped when the reference library has not been built (its sources are not on this machine)."""
import hashlib
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest

from helpers import README_CASE, TEST3_CASES, TEST4_CASE, dims_of_test1, gpu_transpose, random_case, volume

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cases():
    rng = random.Random(4242)
    cases = [README_CASE, TEST4_CASE] + [c for c in TEST3_CASES if volume(c[0]) <= 70_000_000]
    for rank in range(2, 8):
        dims = dims_of_test1(rank)
        perm = list(range(rank))
        rng.shuffle(perm)
        cases.append((dims, perm))
        cases.append(random_case(rng, rank, 3_000_000))
    return cases


def test_reference_library_agrees(native, oracle_mod, tmp_path):
    from oracle import ref_runner
    if not ref_runner.available():
        pytest.skip("oracle/_ref/libcutt_ref.so not built")
    spec = []
    for dims, perm in _cases():
        for elt in (4, 8):
            spec.append({"dims": list(dims), "perm": list(perm), "elt": elt})
    path = str(tmp_path / "cases.json")
    with open(path, "w") as f:
        json.dump(spec, f)
    res = subprocess.run([sys.executable, "-m", "oracle.ref_runner", path, "--reps", "1", "--check"], cwd=ROOT,
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [json.loads(ln) for ln in res.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == len(spec)
    for rec in lines:
        assert "error" not in rec and "skipped" not in rec, rec
        # the reference agrees with the CPU oracle (this pins the oracle to the real library) ...
        assert rec["oracle_equal"], rec
        # ... and with this library's output on the same seeded input
        dims, perm, elt = rec["dims"], rec["perm"], rec["elt"]
        a = ref_runner.input_bits(volume(dims), elt, 1234).view(np.uint32 if elt == 4 else np.uint64)
        out, desc = gpu_transpose(native, dims, perm, elt, a)
        assert hashlib.sha256(np.ascontiguousarray(out).tobytes()).hexdigest() == rec["sha256"], (rec, desc)
