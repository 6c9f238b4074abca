"""Fits the planner's cost model to measured candidate timings and writes it as a C++ header.

Input:  one or more JSON-lines files produced by cutt_b200/cost_model/sweep.py on a B200
        (one record per timed candidate: its feature vector and the achieved GB/s).
Output: cutt_b200/csrc/cost_model_data.h - a gradient-boosted ensemble of small regression trees
        predicting the fraction of the copy bandwidth a candidate reaches, as flat arrays.

usage: python -m cutt_b200.cost_model.train data1.jsonl [data2.jsonl ...] [--trees 250] [--depth 4]
"""
from __future__ import annotations

import argparse
import collections
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(os.path.dirname(HERE), "csrc", "cost_model_data.h")
REF_GBS = 6500.0  # efficiencies are fractions of this copy bandwidth


def load(paths):
    rows = []
    for p in paths:
        with open(p) as f:
            for line in f:
                if '"feat"' in line:
                    r = json.loads(line)
                    # only tile candidates carry features; other methods have closed-form costs
                    if len(r["feat"]) and r["gbs"] > 0 and r["label"].startswith("tiles"):
                        rows.append(r)
    return rows


def evaluate(model, rows, X, y, groups):
    """Quality of the ranking per (case, element size): achieved / best for top-1 and top-8."""
    pred = model.predict(X)
    by = collections.defaultdict(list)
    for i, g in enumerate(groups):
        by[g].append(i)
    t1, t8, t24 = [], [], []
    for g, idx in by.items():
        idx = np.array(idx)
        order = idx[np.argsort(-pred[idx])]
        best = y[idx].max()
        t1.append(y[order[0]] / best)
        t8.append(y[order[:8]].max() / best)
        t24.append(y[order[:24]].max() / best)
    q = lambda v: (float(np.median(v)), float(np.min(v)), float(np.mean(v)))
    return {"top1": q(t1), "top8": q(t8), "top24": q(t24)}


def main():
    from sklearn.ensemble import GradientBoostingRegressor
    ap = argparse.ArgumentParser()
    ap.add_argument("data", nargs="+")
    ap.add_argument("--trees", type=int, default=300)
    ap.add_argument("--depth", type=int, default=5)
    ap.add_argument("--lr", type=float, default=0.05)
    ap.add_argument("--wpow", type=float, default=6.0,
                    help="sample weight = (achieved / best of its case)^wpow: accuracy matters near the top")
    ap.add_argument("--no-write", action="store_true")
    ap.add_argument("--mask", default="", help="comma-separated feature indices to zero (features whose meaning changed)")
    args = ap.parse_args()
    rows = load(args.data)
    X = np.array([r["feat"] for r in rows], dtype=np.float32)
    for m in [int(x) for x in args.mask.split(",") if x]:
        X[:, m] = 0.0
    y = np.array([min(r["gbs"] / REF_GBS, 1.2) for r in rows], dtype=np.float64)
    groups = ["%s/%d" % (r["case"], r["elt"]) for r in rows]
    cases = sorted(set(r["case"] for r in rows))
    print("records %d, cases %d, features %d" % (len(rows), len(cases), X.shape[1]))

    best = collections.defaultdict(float)
    for g, v in zip(groups, y):
        best[g] = max(best[g], v)
    weight = np.array([(v / best[g]) ** args.wpow for g, v in zip(groups, y)])

    def fit(mask):
        return GradientBoostingRegressor(n_estimators=args.trees, max_depth=args.depth, learning_rate=args.lr,
                                         subsample=0.8, random_state=0).fit(X[mask], y[mask], sample_weight=weight[mask])

    # leave-cases-out cross validation (both element sizes of a case are held out together)
    rng = np.random.default_rng(0)
    perm = rng.permutation(len(cases))
    case_of = np.array([r["case"] for r in rows])
    for k in range(4):
        held = set(cases[i] for i in perm[k::4])
        te = np.array([c in held for c in case_of])
        m = fit(~te)
        res = evaluate(m, [r for r, t in zip(rows, te) if t], X[te], y[te], [g for g, t in zip(groups, te) if t])
        print("fold %d  top1 med/min/mean %.3f/%.3f/%.3f  top8 %.3f/%.3f/%.3f  top24 %.3f/%.3f/%.3f"
              % ((k,) + res["top1"] + res["top8"] + res["top24"]))
    model = fit(np.ones(len(rows), dtype=bool))
    res = evaluate(model, rows, X, y, groups)
    print("all data (in-sample) top1 %.3f/%.3f/%.3f top8 %.3f/%.3f/%.3f" % (res["top1"] + res["top8"]))
    imp = sorted(enumerate(model.feature_importances_), key=lambda kv: -kv[1])[:12]
    print("importances:", ", ".join("f%d %.3f" % kv for kv in imp))
    if args.no_write:
        return
    # flatten
    feat, thr, left, right, val, roots = [], [], [], [], [], []
    for est in model.estimators_[:, 0]:
        t = est.tree_
        base = len(feat)
        roots.append(base)
        for i in range(t.node_count):
            leaf = t.children_left[i] < 0
            feat.append(-1 if leaf else int(t.feature[i]))
            thr.append(0.0 if leaf else float(t.threshold[i]))
            left.append(0 if leaf else base + int(t.children_left[i]))
            right.append(0 if leaf else base + int(t.children_right[i]))
            val.append(float(t.value[i][0][0]) * args.lr)
    init = float(model.init_.constant_[0][0]) if hasattr(model.init_, "constant_") else float(np.mean(y))
    with open(OUT, "w") as f:
        f.write("// GENERATED by cutt_b200/cost_model/train.py from B200 candidate timings - do not edit.\n")
        f.write("// Gradient-boosted regression trees: predicted fraction of %.0f GB/s a tile candidate reaches.\n" % REF_GBS)
        f.write("// records %d, cases %d, trees %d, depth %d\n" % (len(rows), len(cases), args.trees, args.depth))
        f.write("#pragma once\nnamespace cuttb {\nnamespace cost_model {\n")
        f.write("constexpr int kFeatures = %d;\nconstexpr int kTrees = %d;\nconstexpr int kNodes = %d;\n" % (X.shape[1], len(roots), len(feat)))
        f.write("constexpr float kRefGBs = %.1ff;\nconstexpr float kInit = %.8ff;\n" % (REF_GBS, init))

        def arr(name, ctype, data, fmt):
            f.write("static const %s %s[] = {\n" % (ctype, name))
            for i in range(0, len(data), 16):
                f.write("  " + ", ".join(fmt % x for x in data[i:i + 16]) + ",\n")
            f.write("};\n")
        arr("kRoot", "int", roots, "%d")
        arr("kFeat", "signed char", feat, "%d")
        arr("kThr", "float", thr, "%.8ef")
        arr("kLeft", "unsigned short", left, "%d")
        arr("kRight", "unsigned short", right, "%d")
        arr("kVal", "float", val, "%.8ef")
        f.write("}  // namespace cost_model\n}  // namespace cuttb\n")
    print("wrote", OUT, "nodes", len(feat))


if __name__ == "__main__":
    main()
