"""Training-data sweep for the planner's cost model (run on a B200).

Times every candidate of the benchmark shapes (C2, C4, C5 slabs, the random C3 suite) through the
C ABI, three repetitions each, and writes one JSON line per candidate with the feature vector
the library reports.  usage: python -m cutt_b200.cost_model.sweep OUT.jsonl FIRST_CASE LAST_CASE   (cases 0-99: the committed suite;
100 and up: further seeds of the same generator)
"""
import json, sys, os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import numpy as np, torch
import cutt_b200 as c
from cutt_b200 import workloads as W
def main():
    out = open(sys.argv[1], "w")
    lo, hi = int(sys.argv[2]), int(sys.argv[3])
    cases = []
    if lo == 0:
        cases += [("C2", *W.C2, 4), ("C2", *W.C2, 8), ("C4", *W.C4, 4), ("C4", *W.C4, 8),
                  ("C5a8", [1024, 1024, 1024], [1, 0, 2], 4), ("C5b1", [1048576, 32, 32], [2, 1, 0], 4)]
    for i, (d, p) in enumerate(W.c3_cases(100)):
        if lo <= i < hi:
            cases += [("C3_%d" % i, d, p, 8), ("C3_%d" % i, d, p, 4)]
    # indices from 100 on: further shapes from the same generator (other seeds), training data only
    for i in range(max(lo, 100), hi):
        d, p = W.generate_c3_case(i)
        cases += [("X3_%d" % i, d, p, 8), ("X3_%d" % i, d, p, 4)]
    buf_in = torch.randint(-2**31, 2**31 - 1, (550_000_000,), dtype=torch.int64, device="cuda")
    buf_out = torch.empty_like(buf_in)
    for name, dims, perm, elt in cases:
        vol = int(np.prod(np.array(dims, dtype=np.int64)))
        assert vol * elt <= buf_in.numel() * 8
        n = c.num_candidates(dims, perm, elt)
        best = 0
        for i in range(n):
            rc, h = c.plan_candidate(dims, perm, elt, i)
            if rc != 0: continue
            desc = json.loads(c.plan_describe(h))
            c.cuttExecute(h, buf_in.data_ptr(), buf_out.data_ptr())
            ts = []
            for _ in range(3):
                e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                e0.record(); c.cuttExecute(h, buf_in.data_ptr(), buf_out.data_ptr()); e1.record()
                torch.cuda.synchronize(); ts.append(e0.elapsed_time(e1))
            c.cuttDestroy(h)
            gbs = 2 * vol * elt / (min(ts) * 1e-3) / 1e9
            best = max(best, gbs)
            out.write(json.dumps({"case": name, "elt": elt, "idx": i, "gbs": gbs, "ms": min(ts), "label": desc["label"], "feat": desc["feat"], "model_us": desc["model_us"]}) + "\n")
        out.flush()
        print(name, elt, n, "best %.0f" % best); sys.stdout.flush()
main()
