"""Applies a fitted cost model (the generated C++ header) to candidate timings it may never have seen.

For every (shape, element size) of a JSON-lines file written by cutt_b200/cost_model/sweep.py the
candidates are ranked by the model and the achieved bandwidth of the first pick, of the best of
the first 8 and of the best of the first 48 (what cuttPlanMeasure times) is compared with the best
candidate of the sweep.

usage: python -m cutt_b200.cost_model.evaluate DATA.jsonl [--header cutt_b200/csrc/cost_model_data.h]
"""
from __future__ import annotations

import argparse
import collections
import json
import os
import re

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_HEADER = os.path.join(os.path.dirname(HERE), "csrc", "cost_model_data.h")


def load_model(path):
    text = open(path).read()

    def arr(name, conv):
        m = re.search(name + r"\[\] = \{(.*?)\};", text, re.S)
        return np.array([conv(x.rstrip("f")) for x in m.group(1).replace("\n", " ").split(",") if x.strip()])

    return {"root": arr("kRoot", int), "feat": arr("kFeat", int), "thr": arr("kThr", float),
            "left": arr("kLeft", int), "right": arr("kRight", int), "val": arr("kVal", float),
            "init": float(re.search(r"kInit = ([^;]+)f;", text).group(1))}


def predict(model, X):
    """Tree ensemble evaluated for all rows at once (one vector step per tree level)."""
    n_rows = len(X)
    rows = np.arange(n_rows)
    pred = np.full(n_rows, model["init"])
    for root in model["root"]:
        node = np.full(n_rows, root)
        for _ in range(16):
            f = model["feat"][node]
            leaf = f < 0
            if leaf.all():
                break
            left = X[rows, np.maximum(f, 0)] <= model["thr"][node]
            node = np.where(leaf, node, np.where(left, model["left"][node], model["right"][node]))
        pred += model["val"][node]
    return pred


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("data", nargs="+")
    ap.add_argument("--header", default=DEFAULT_HEADER)
    ap.add_argument("--worst", type=int, default=5, help="list this many worst first picks")
    args = ap.parse_args()
    rows = []
    for p in args.data:
        with open(p) as f:
            rows += [json.loads(line) for line in f if '"feat"' in line]
    rows = [r for r in rows if r["label"].startswith("tiles") and r["gbs"] > 0]
    X = np.array([r["feat"] for r in rows], dtype=np.float32)
    y = np.array([r["gbs"] for r in rows])
    pred = predict(load_model(args.header), X)
    groups = collections.defaultdict(list)
    for i, r in enumerate(rows):
        groups[(r["case"], r["elt"])].append(i)
    top = {1: [], 8: [], 48: []}
    picks = []
    for g, idx in groups.items():
        idx = np.array(idx)
        order = idx[np.argsort(-pred[idx])]
        best = y[idx].max()
        for k in top:
            top[k].append(y[order[:k]].max() / best)
        picks.append((y[order[0]] / best, g, rows[order[0]]["label"]))
    print("records %d, groups %d" % (len(rows), len(groups)))
    for k, v in top.items():
        print("best of first %-2d: median %.3f  mean %.3f  min %.3f" % (k, np.median(v), np.mean(v), np.min(v)))
    for frac, g, label in sorted(picks)[:args.worst]:
        print("  %.3f  %s/%d  %s" % (frac, g[0], g[1], label))


if __name__ == "__main__":
    main()
