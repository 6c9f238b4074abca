"""Command-line benchmark with the options of the original ``cutt_bench``
(src/cutt_bench.cpp:85-152): ``-device``, ``-measure``, ``-plantimer``, ``-seed``, ``-elemsize``,
``-dim ... -permutation ...`` and ``-bench N``.

Every tensor is planned (``cuttPlan``, or ``cuttPlanMeasure`` with ``-measure``), executed four
times between CUDA events after the output was filled with 0xFF (as src/cutt_bench.cpp:818-827
does), checked on the device, and reported as GB/s = ``2 * volume * elemsize / time``
(src/cuttTimer.cpp:92).  At the end the per-rank best / worst / average / median table of the
original's timer (src/cuttTimer.cpp:152-246) is printed, then ``bench OK`` or ``bench FAIL``.

Benchmarks (numbering and shape families of the original; the random draws come from a seeded
Python generator, so a seed reproduces a run here but not the original's rand() sequence):
  -bench 1    ranks 2-8 and 15, inverse permutation, first and last dimension 32 (or the average
              extent when that is >= 100), the rest spread evenly  (src/cutt_bench.cpp:376-407)
  -bench 2    ranks 2-8 and 15, inverse permutation, dimensions spread evenly       (:412-435)
  -bench 3    ranks 2-8 and 15, random dimensions and permutations, -samples each   (:440-456, 743-771)
  -bench 5RR  ranks 2-7, -samples each; extents grow linearly from the smallest to RR times the
              smallest, volume drawn around 200 M elements, dimensions shuffled, random
              non-trivial permutations (the original's ``-bench 5RR``)              (:479-546)
  -bench 7    ranks 8 and 12 with four large and otherwise small dimensions: the inverse
              permutation, then -samples shuffles of dimensions and permutation     (:693-728)
  -suite      the 100-case random suite of this repository (cutt_b200/c3_cases.json)
The original's bench 6 (a fixed table taken from another project's benchmark, :551-690) is not
reproduced; other bench numbers (a plain memory-copy benchmark there) are not offered.

``-method M`` forces an implementation for every tensor (this library's method numbers: 0 copy
kernel and 1 driver copy for identity permutations, 2 tiled kernel with default tile parameters,
3 one thread per element, 4 strided row copy, 6 tensor-map transpose, 7 two-dimensional tiles with
swizzled shared memory) and ``-offset B`` shifts both device buffers by B
bytes (a multiple of the element size): profiling aids without a counterpart in the original.

``-volume`` scales every generated tensor (default 200 M elements, as the original); ``-samples``
defaults to the original's counts (50 for bench 3, 500 for benches 5 and 7).
"""
from __future__ import annotations

import argparse
import json
import math
import random
import statistics
import sys
import time


def _vol(dims):
    v = 1
    for d in dims:
        v *= int(d)
    return v


def _reference_permute(tin, dims, perm):
    r = len(dims)
    axes = [r - 1 - perm[r - 1 - k] for k in range(r)]
    return tin.view(*reversed(dims)).permute(*axes).contiguous().view(-1)


def permute_checker(torch):
    """Default check: the same permutation done by torch on the device, compared bit for bit."""
    def check(dims, perm, tin, tout):
        return bool(torch.equal(tout, _reference_permute(tin, dims, perm)))
    return check


def run_case(C, torch, dims, perm, elt, measure, buf_in, buf_out, checker=None, plantimer=False,
             method=None, offset=0, stages=None, threads=None):
    vol = _vol(dims)
    words = 1
    if elt == 16:   # checked as two 64-bit words per element under an unpermuted innermost dimension
        words = 2
    dt = {1: torch.uint8, 2: torch.int16, 4: torch.int32, 8: torch.int64, 16: torch.int64}[elt]
    e0 = offset // (elt // words)      # buffer offset in units of the checked word type
    tin = buf_in[:(vol * elt + offset) // 8 + 1].view(dt)[e0:e0 + vol * words]
    tout = buf_out[:(vol * elt + offset) // 8 + 1].view(dt)[e0:e0 + vol * words]
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    if method is not None:
        kw = {}
        if method in (6, 7):    # swizzled-tile kernels: 256-byte x 64-row (4-byte) / 32-row (8-byte) tiles, one per block
            kw = dict(tin=256, tout=256, stages=1, nthreads=128)
        if stages is not None:
            kw["stages"] = stages
        if threads is not None:
            kw["nthreads"] = threads
        rc, h = C.plan_params(dims, perm, elt, stream, method=method, **kw)
    elif elt not in (4, 8):   # sizes the original rejects: extension entry points
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
    if plantimer:
        print("plan took %f ms" % ((time.perf_counter() - t0) * 1e3))
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
    if checker is not None:
        if elt == 16:
            ok = checker([2] + list(dims), [0] + [p + 1 for p in perm], tin, tout)
        else:
            ok = checker(dims, perm, tin, tout)
    gbs = [2 * vol * elt / (t * 1e-3) / 1e9 for t in times]
    return gbs, ok, plan


_RANKS = (2, 3, 4, 5, 6, 7, 8, 15)


def _is_trivial(perm):
    return all(p == i for i, p in enumerate(perm))


def _inverse(rank):
    return [rank - 1 - r for r in range(rank)]


def _even_spread(volume, rank, dims, first):
    """Fills dims[first:rank-?] the way src/cutt_bench.cpp:392-398 / :420-424 do: each extent is
    the integer part of the k-th root of what is left."""
    left = float(volume)
    for r in range(first, rank):
        dims[r] = max(2, int(left ** (1.0 / (rank - r))))
        left /= dims[r]
    return dims


def random_dims(rng, volume, rank):
    """Random extents around the average one, rescaled to the volume; redrawn until the volume is
    within 30 % (src/cutt_bench.cpp:743-771).  Where the original gives up after 5000 draws (tiny
    -volume with a high rank cannot get that close), the closest draw is used."""
    ave = math.floor(volume ** (1.0 / rank))
    best = None
    for _ in range(5000 if ave > 2 else 50):
        dims = [round(ave + (rng.random() - 0.5) * 2.0 * (ave - 2.0)) for _ in range(rank)]
        cur = 1.0
        for d in dims:
            cur *= max(d, 1)
        scale = (volume / cur) ** (1.0 / rank)
        dims = [max(2, int(d * scale)) for d in dims]
        err = abs(_vol(dims) - volume) / volume
        if err <= 0.3:
            return dims
        if best is None or err < best[0]:
            best = (err, dims)
    return best[1]


def bench_cases(which, rng, volume=200_000_000, samples=None):
    cases = []
    if which == 1:
        for rank in _RANKS:
            ave = int(volume ** (1.0 / rank))
            edge = 32 if ave < 100 else ave
            dims = [0] * rank
            dims[0] = dims[rank - 1] = edge
            if rank > 2:
                left = volume / float(edge * edge)
                n = rank - 2
                for r in range(1, rank - 1):
                    dims[r] = max(2, int(left ** (1.0 / n)))
                    left /= dims[r]
                    n -= 1
            cases.append((dims, _inverse(rank)))
    elif which == 2:
        for rank in _RANKS:
            cases.append((_even_spread(volume, rank, [0] * rank, 0), _inverse(rank)))
    elif which == 3:
        for rank in _RANKS:
            perm = list(range(rank))
            for _ in range(samples or 50):
                rng.shuffle(perm)
                cases.append((random_dims(rng, volume, rank), list(perm)))
    elif which // 100 == 5:
        ratio = which % 100
        if ratio < 1:
            raise SystemExit("-bench 5RR needs a ratio RR >= 1 (e.g. 515)")
        for rank in range(2, 8):
            for _ in range(samples or 500):
                target = max(1000.0, rng.gauss(volume, 0.2 * volume))
                dimf = [1.0 + r * (ratio - 1.0) / (rank - 1) for r in range(rank)]
                volf = 1.0
                for d in dimf:
                    volf *= d
                scale = (target / volf) ** (1.0 / rank)
                dims = [max(2, int(round(d * scale))) for d in dimf]
                dims[rank - 1] = max(2, ratio * dims[0])
                # nudge the middle dimensions while the volume is more than 5 % off
                step = 1 if _vol(dims) < target else -1
                r = 1
                while abs(_vol(dims) - target) / target > 0.05 and r < rank:
                    dims[r] = max(2, dims[r] + step)
                    r += 1
                rng.shuffle(dims)
                perm = list(range(rank))
                while _is_trivial(perm):
                    rng.shuffle(perm)
                cases.append((dims, perm))
    elif which == 7:
        for base in ([5, 3, 2, 4, 35, 33, 37, 40], [2, 3, 4, 3, 2, 2, 3, 2, 20, 18, 22, 24]):
            dims = list(base)
            if volume != 200_000_000:   # scaled runs: shrink the four large dimensions
                f = (volume / 200_000_000.0) ** 0.25
                dims = [d if d < 16 else max(2, int(round(d * f))) for d in dims]
            rank = len(dims)
            cases.append((list(dims), _inverse(rank)))
            perm = list(range(rank))
            for _ in range(samples or 500):
                rng.shuffle(dims)
                rng.shuffle(perm)
                if not _is_trivial(perm):
                    cases.append((list(dims), list(perm)))
    else:
        raise SystemExit("unknown -bench %d (1, 2, 3, 5RR and 7 are available; 6 is not reproduced)" % which)
    return cases


def main(argv=None, checker="permute"):
    """``checker``: "permute" (default: compare with torch's permutation on the device), None, or a
    callable ``(dims, perm, tin, tout) -> bool`` (the tests pass the index-formula checker)."""
    ap = argparse.ArgumentParser(prog="cutt_b200.bench_cli", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("-device", type=int, default=0)
    ap.add_argument("-measure", action="store_true")
    ap.add_argument("-plantimer", action="store_true")
    ap.add_argument("-seed", type=int, default=12345)
    ap.add_argument("-elemsize", type=int, default=8, choices=[1, 2, 4, 8, 16],
                    help="4 and 8 as in the original; 1, 2 and 16 go through the extension entry points")
    ap.add_argument("-dim", type=int, nargs="+")
    ap.add_argument("-permutation", type=int, nargs="+")
    ap.add_argument("-bench", type=int, default=0)
    ap.add_argument("-suite", action="store_true", help="the 100-case random suite of this repository")
    ap.add_argument("-volume", type=int, default=200_000_000, help="elements per generated tensor")
    ap.add_argument("-samples", type=int, default=None, help="random draws per rank (benches 3, 5RR, 7)")
    ap.add_argument("-nocheck", action="store_true")
    ap.add_argument("-method", type=int, default=None, choices=[0, 1, 2, 3, 4, 6, 7])
    ap.add_argument("-offset", type=int, default=0, help="byte offset of both device buffers")
    ap.add_argument("-stages", type=int, default=None, help="with -method: shared-memory stages")
    ap.add_argument("-threads", type=int, default=None, help="with -method: threads per block")
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
    elif args.suite:
        from . import workloads as W
        cases = W.c3_cases(100)
    elif args.bench:
        cases = bench_cases(args.bench, rng, args.volume, args.samples)
    else:
        raise SystemExit("give -dim/-permutation, -bench N or -suite")
    if args.nocheck:
        checker = None
    elif checker == "permute":
        checker = permute_checker(torch)
    if args.offset % args.elemsize or args.offset < 0:
        raise SystemExit("-offset must be a non-negative multiple of the element size")
    if args.method is not None and args.elemsize not in (4, 8):
        raise SystemExit("-method needs -elemsize 4 or 8")
    maxbytes = max(_vol(d) for d, _ in cases) * args.elemsize + args.offset
    buf_in = torch.randint(-2**62, 2**62, (maxbytes // 8 + 2,), dtype=torch.int64, device="cuda")
    buf_out = torch.empty_like(buf_in)
    per_rank = {}
    failed = 0
    for dims, perm in cases:
        gbs, ok, plan = run_case(C, torch, list(dims), list(perm), args.elemsize, args.measure, buf_in, buf_out,
                                 checker=checker, plantimer=args.plantimer, method=args.method, offset=args.offset,
                                 stages=args.stages, threads=args.threads)
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
    print("bench FAIL" if failed else "bench OK")
    print("seed %d" % args.seed)
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
