"""Runs the ORIGINAL cuTT (oracle/_ref/libcutt_ref.so, built by oracle/build_ref.py from the
unmodified sources as compute_60 PTX, translated for the installed GPU by the driver) on a list
of cases, in a process of its own: the original library calls exit(1) on any CUDA error, which
must not take a test run or the benchmark down with it.

Test infrastructure only (the tests use it as a second checker, the benchmark as the
"reference cuTT on this GPU" baseline).

usage: python -m oracle.ref_runner CASES.json [--measure] [--reps N] [--check] [--seed S]
  CASES.json: [{"dims": [...], "perm": [...], "elt": 4|8}, ...]
prints one JSON line per case: {"dims", "perm", "elt", "ms", "gbs", "sha256"[, "oracle_equal"]}
"""
from __future__ import annotations

import argparse
import ctypes
import hashlib
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "_ref", "libcutt_ref.so")


def available() -> bool:
    return os.path.exists(LIB)


def _load():
    lib = ctypes.CDLL(LIB)
    ip, up, vp = ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_uint), ctypes.c_void_p
    lib.ref_cutt_plan.argtypes = [up, ctypes.c_int, ip, ip, ctypes.c_size_t, vp]
    lib.ref_cutt_plan_measure.argtypes = [up, ctypes.c_int, ip, ip, ctypes.c_size_t, vp, vp, vp]
    lib.ref_cutt_execute.argtypes = [ctypes.c_uint, vp, vp]
    lib.ref_cutt_destroy.argtypes = [ctypes.c_uint]
    return lib


def input_bits(vol: int, elt: int, seed: int):
    """Seeded raw bit patterns; the callers regenerate the same input to compare outputs."""
    import numpy as np
    rng = np.random.default_rng(seed)
    return rng.integers(0, 2**32, size=vol * (elt // 4), dtype=np.uint64).astype(np.uint32)


def main():
    import numpy as np
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("cases")
    ap.add_argument("--measure", action="store_true")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--check", action="store_true", help="also compare with the CPU oracle")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--no-hash", action="store_true")
    ap.add_argument("--device-input", action="store_true",
                    help="timing only: random input generated on the device, output not read back")
    args = ap.parse_args()
    with open(args.cases) as f:
        cases = json.load(f)
    lib = _load()
    ia = lambda v: (ctypes.c_int * len(v))(*v)
    for c in cases:
        dims, perm, elt = c["dims"], c["perm"], c["elt"]
        vol = 1
        for d in dims:
            vol *= d
        if vol >= 2**31:
            print(json.dumps({"dims": dims, "perm": perm, "elt": elt, "skipped": "volume >= 2^31: outside the original's int range"}))
            continue
        if args.device_input:
            a = None
            tin = torch.randint(-2**31, 2**31 - 1, (vol * (elt // 4),), dtype=torch.int32, device="cuda")
        else:
            a = input_bits(vol, elt, args.seed)
            tin = torch.from_numpy(a.view(np.int32)).cuda()
        tout = torch.zeros_like(tin)
        torch.cuda.synchronize()
        h = ctypes.c_uint(0)
        if args.measure:
            rc = lib.ref_cutt_plan_measure(ctypes.byref(h), len(dims), ia(dims), ia(perm), elt, None,
                                           tin.data_ptr(), tout.data_ptr())
        else:
            rc = lib.ref_cutt_plan(ctypes.byref(h), len(dims), ia(dims), ia(perm), elt, None)
        if rc != 0:
            print(json.dumps({"dims": dims, "perm": perm, "elt": elt, "error": "plan rc %d" % rc}))
            continue
        tout.zero_()
        torch.cuda.synchronize()
        lib.ref_cutt_execute(h.value, tin.data_ptr(), tout.data_ptr())
        torch.cuda.synchronize()
        ts = []
        for _ in range(args.reps):
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            lib.ref_cutt_execute(h.value, tin.data_ptr(), tout.data_ptr())
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        lib.ref_cutt_destroy(h.value)
        ms = min(ts) if ts else None
        rec = {"dims": dims, "perm": perm, "elt": elt, "ms": ms,
               "gbs": (2 * vol * elt / (ms * 1e-3) / 1e9) if ms else None}
        if args.device_input:
            print(json.dumps(rec))
            sys.stdout.flush()
            del tin, tout
            continue
        out = tout.cpu().numpy()
        if not args.no_hash:
            rec["sha256"] = hashlib.sha256(out.tobytes()).hexdigest()
        if args.check:
            sys.path.insert(0, os.path.dirname(HERE))
            import oracle
            dt = np.uint32 if elt == 4 else np.uint64
            rec["oracle_equal"] = bool(np.array_equal(out.view(dt), oracle.transpose_blocked(dims, perm, a.view(dt))))
        print(json.dumps(rec))
        sys.stdout.flush()
        del tin, tout


if __name__ == "__main__":
    main()
