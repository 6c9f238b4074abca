"""Command-line benchmark with the options of the original ``cutt_bench``
(src/cutt_bench.cpp:92-152): ``-device``, ``-measure``, ``-seed``, ``-elemsize``,
``-dim ... -permutation ...`` and ``-bench N``.

Every tensor is planned (``cuttPlan``, or ``cuttPlanMeasure`` with ``-measure``), executed four
times between CUDA events after the output was filled with 0xFF (as src/cutt_bench.cpp:818-827
does), checked against ``torch.permute`` on the device, and reported as GB/s =
``2 * volume * elemsize / time`` (src/cuttTimer.cpp:92).  At the end the per-rank best / worst /
average / median table of the original's timer (src/cuttTimer.cpp:152-246) is printed.

Benchmarks:
  -bench 1   ranks 2-7, 32 random permutations each of a ~200 M-element tensor with equal dims
  -bench 3   ranks 2-8 and 12, random dims (ratio up to 1:15) and permutations, 20 each
  -bench 5   the 100-case random suite of this repository (cutt_b200/c3_cases.json)
The original's bench 6 (a fixed list taken from another project's benchmark) is not reproduced.
"""
from __future__ import annotations

import argparse
import json
import random
import statistics
import sys


def _vol(dims):
    v = 1
    for d in dims:
        v *= int(d)
    return v


def _reference_permute(tin, dims, perm):
    r = len(dims)
    axes = [r - 1 - perm[r - 1 - k] for k in range(r)]
    return tin.view(*reversed(dims)).permute(*axes).contiguous().view(-1)


def run_case(C, torch, dims, perm, elt, measure, buf_in, buf_out, check=True):
    vol = _vol(dims)
    words = 1
    if elt == 16:   # checked as two 64-bit words per element under an unpermuted innermost dimension
        words = 2
    dt = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64, 16: torch.int64}[elt]
    tin = buf_in[:vol * elt // 8 + 1].view(dt)[:vol * words]
    tout = buf_out[:vol * elt // 8 + 1].view(dt)[:vol * words]
    stream = torch.cuda.current_stream().cuda_stream
    if elt not in (4, 8):   # sizes the original rejects: extension entry points
        if measure:
            rc, h = C.plan_measure_ext(dims, perm, elt, stream, tin.data_ptr(), tout.data_ptr())
        else:
            rc, h = C.plan_ext(dims, perm, elt, stream)
    elif measure:
        rc, h = C.cuttPlanMeasure(len(dims), dims, perm, elt, stream, tin.data_ptr(), tout.data_ptr())
    else:
        rc, h = C.cuttPlan(len(dims), dims, perm, elt, stream)
    if rc != 0:
        raise RuntimeError("plan failed with code %d for %s %s" % (rc, dims, perm))
    times = []
    for _ in range(4):
        tout.fill_(255 if elt == 1 else -1)
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        if C.cuttExecute(h, tin.data_ptr(), tout.data_ptr()) != 0:
            raise RuntimeError("execute failed")
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    plan = json.loads(C.plan_describe(h))["label"]
    C.cuttDestroy(h)
    ok = True
    if check:
        if elt == 16:
            ok = bool(torch.equal(tout, _reference_permute(tin, [2] + list(dims), [0] + [p + 1 for p in perm])))
        else:
            ok = bool(torch.equal(tout, _reference_permute(tin, dims, perm)))
    gbs = [2 * vol * elt / (t * 1e-3) / 1e9 for t in times]
    return gbs, ok, plan


def random_dims(rng, rank, target, max_ratio):
    lo = 1.0
    dims = [lo * (max_ratio ** rng.random()) for _ in range(rank)]
    scale = (target / _vol([max(1.0, d) for d in dims])) ** (1.0 / rank)
    return [max(2, int(round(d * scale))) for d in dims]


def bench_cases(which, rng):
    from . import workloads as W
    cases = []
    if which == 1:
        for rank in range(2, 8):
            d = max(2, int(round(2.0e8 ** (1.0 / rank))))
            for _ in range(32):
                perm = list(range(rank))
                while perm == list(range(rank)):
                    rng.shuffle(perm)
                cases.append(([d] * rank, perm))
    elif which == 3:
        for rank in (2, 3, 4, 5, 6, 7, 8, 12):
            for _ in range(20):
                dims = random_dims(rng, rank, 2.0e8, 15.0)
                perm = list(range(rank))
                while perm == list(range(rank)):
                    rng.shuffle(perm)
                cases.append((dims, perm))
    elif which == 5:
        cases = W.c3_cases(100)
    else:
        raise SystemExit("unknown -bench %d (1, 3 and 5 are available)" % which)
    return cases


def main(argv=None):
    ap = argparse.ArgumentParser(prog="cutt_b200.bench_cli", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("-device", type=int, default=0)
    ap.add_argument("-measure", action="store_true")
    ap.add_argument("-seed", type=int, default=12345)
    ap.add_argument("-elemsize", type=int, default=8, choices=[1, 2, 4, 8, 16],
                    help="4 and 8 as in the original; 1, 2 and 16 go through the extension entry points")
    ap.add_argument("-dim", type=int, nargs="+")
    ap.add_argument("-permutation", type=int, nargs="+")
    ap.add_argument("-bench", type=int, default=0)
    ap.add_argument("-nocheck", action="store_true")
    args = ap.parse_args(argv)
    import torch
    import cutt_b200 as C
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device")
    torch.cuda.set_device(args.device)
    C.lib()
    rng = random.Random(args.seed)
    if args.dim:
        if not args.permutation or len(args.permutation) != len(args.dim):
            raise SystemExit("-dim and -permutation must have the same length")
        cases = [(args.dim, args.permutation)]
    elif args.bench:
        cases = bench_cases(args.bench, rng)
    else:
        raise SystemExit("give -dim/-permutation or -bench N")
    maxbytes = max(_vol(d) for d, _ in cases) * args.elemsize
    buf_in = torch.randint(-2**62, 2**62, (maxbytes // 8 + 2,), dtype=torch.int64, device="cuda")
    buf_out = torch.empty_like(buf_in)
    per_rank = {}
    failed = 0
    for dims, perm in cases:
        gbs, ok, plan = run_case(C, torch, list(dims), list(perm), args.elemsize, args.measure, buf_in, buf_out,
                                 check=not args.nocheck)
        failed += 0 if ok else 1
        print("dims %s perm %s : %s GB/s %s  [%s]" % (list(dims), list(perm), " ".join("%.1f" % g for g in gbs),
                                                      "OK" if ok else "FAIL", plan))
        per_rank.setdefault(len(dims), []).extend([(g, dims, perm) for g in gbs])
    print("\nrank  best  worst  average  median   (GB/s)")
    for rank in sorted(per_rank):
        v = sorted(g for g, _, _ in per_rank[rank])
        print("%4d %6.1f %6.1f %8.1f %7.1f" % (rank, v[-1], v[0], statistics.mean(v), statistics.median(v)))
        worst = min(per_rank[rank], key=lambda x: x[0])
        print("      worst case: dims %s perm %s" % (list(worst[1]), list(worst[2])))
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
