"""The cutt_bench-style command line (cutt_b200/bench_cli.py; options and benchmark families of
src/cutt_bench.cpp:85-152,376-456,479-546,693-728) on cut-down volumes, every output checked
with the 64-bit index formula instead of the program's default check."""
import random

import pytest

pytestmark = pytest.mark.gpu


def _formula_checker():
    import torch
    from oracle import device_check as DC

    def check(dims, perm, tin, tout):
        it = torch.int32 if tin.element_size() == 4 else torch.int64
        if tin.element_size() in (4, 8):
            return DC.count_mismatches(dims, perm, tout.view(it), tin.view(it)) == 0
        # 1- and 2-byte elements: the source index formula gathers the expected values directly
        o = torch.arange(tout.numel(), dtype=torch.int64, device=tout.device)
        return bool(torch.equal(tout, tin[DC.source_index(dims, perm, o)]))
    return check


@pytest.mark.parametrize("argv", [
    ["-dim", "31", "549", "2", "3", "-permutation", "3", "0", "2", "1"],
    ["-dim", "300", "70", "90", "-permutation", "2", "0", "1", "-elemsize", "4", "-measure", "-plantimer"],
    ["-dim", "130", "70", "9", "-permutation", "1", "2", "0", "-elemsize", "2"],
    ["-bench", "1", "-volume", "3000000", "-elemsize", "4"],
    ["-bench", "2", "-volume", "3000000"],
    ["-bench", "3", "-volume", "2000000", "-samples", "2", "-seed", "7"],
    ["-bench", "515", "-volume", "2000000", "-samples", "3", "-elemsize", "4"],
    ["-bench", "7", "-volume", "2000000", "-samples", "4", "-measure"],
])
def test_command_line_runs_and_checks(native, capsys, argv):
    from cutt_b200 import bench_cli
    rc = bench_cli.main(argv, checker=_formula_checker())
    out = capsys.readouterr().out
    assert rc == 0, out[-2000:]
    assert "bench OK" in out and "FAIL" not in out
    assert "rank  best  worst  average  median" in out


def test_default_checker_and_failure_reporting(native, capsys):
    from cutt_b200 import bench_cli
    assert bench_cli.main(["-dim", "64", "48", "-permutation", "1", "0", "-elemsize", "4"]) == 0
    assert "bench OK" in capsys.readouterr().out
    # a checker that rejects everything must turn into exit code 1 and "bench FAIL"
    assert bench_cli.main(["-dim", "64", "48", "-permutation", "1", "0"], checker=lambda *a: False) == 1
    assert "bench FAIL" in capsys.readouterr().out


def test_generators_follow_the_original_families():
    from cutt_b200 import bench_cli as B
    v = 200_000_000
    c1 = B.bench_cases(1, random.Random(1), v)
    assert [len(d) for d, _ in c1] == [2, 3, 4, 5, 6, 7, 8, 15]
    assert c1[0][0] == [14142, 14142] and c1[3][0][0] == 32 and c1[3][0][-1] == 32
    assert all(p == list(range(len(p) - 1, -1, -1)) for _, p in c1)
    c2 = B.bench_cases(2, random.Random(1), v)
    assert all(0.85 * v <= B._vol(d) <= v for d, _ in c2)
    c3 = B.bench_cases(3, random.Random(1), v, samples=3)
    assert len(c3) == 24 and all(abs(B._vol(d) - v) <= 0.3 * v for d, _ in c3)
    c5 = B.bench_cases(515, random.Random(1), v, samples=2)
    assert len(c5) == 12 and all(p != sorted(p) for _, p in c5)
    assert all(max(d) / min(d) >= 7 for d, _ in c5)
    c7 = B.bench_cases(7, random.Random(1), v, samples=5)
    assert sorted(c7[0][0]) == sorted([5, 3, 2, 4, 35, 33, 37, 40]) and len(c7[-1][0]) == 12
