"""The plan cache that cuttPlan consults: winners of cuttPlanMeasure are served to later plans of
the same problem (the role of src/LRUCache.h:35-98 in the reference is a per-plan launch
configuration cache; here the cached object is the measured plan choice), the least recently
used entry is evicted at capacity, a saved cache is reused by another process, and damaged
entries are ignored rather than trusted."""
import json
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from helpers import assert_bit_exact, gpu_transpose, raw_bits, volume

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _plan(native, dims, perm, elt, measure, bufs=None):
    import torch
    if measure:
        rc, h = native.cuttPlanMeasure(len(dims), dims, perm, elt, 0, bufs[0].data_ptr(), bufs[1].data_ptr())
    else:
        rc, h = native.cuttPlan(len(dims), dims, perm, elt, 0)
    assert rc == 0
    d = json.loads(native.plan_describe(h))
    return h, d


def test_measured_winner_is_served_to_cuttPlan(native, oracle_mod, monkeypatch, capfd):
    import torch
    dims, perm, elt = [300, 70, 90], [2, 0, 1], 4
    a = raw_bits(volume(dims), elt, 3)
    tin = torch.from_numpy(a.view(np.int32)).cuda()
    tout = torch.zeros_like(tin)
    native.clear_plan_cache()
    monkeypatch.setenv("CUTT_VERBOSE", "1")
    h0, d0 = _plan(native, dims, perm, elt, False)            # nothing cached: the cost model decides
    assert "(model)" in capfd.readouterr().err
    h1, d1 = _plan(native, dims, perm, elt, True, (tin, tout))
    assert "(measured)" in capfd.readouterr().err
    assert native.plan_cache_size() == 1
    h2, d2 = _plan(native, dims, perm, elt, False)            # now the measured winner
    assert "(cache)" in capfd.readouterr().err
    assert d2["label"] == d1["label"]
    # cuttPlanMeasure served from the cache still overwrites odata and synchronises
    tout.zero_()
    h3, d3 = _plan(native, dims, perm, elt, True, (tin, tout))
    assert "(cache)" in capfd.readouterr().err
    assert d3["label"] == d1["label"]
    assert int(tout[0].item()) == -1 and int(tout[-1].item()) == -1
    want = oracle_mod.transpose_blocked(dims, perm, a)
    for h in (h0, h1, h2, h3):
        tout.zero_()
        assert native.cuttExecute(h, tin.data_ptr(), tout.data_ptr()) == 0
        torch.cuda.synchronize()
        assert_bit_exact(tout.cpu().numpy().view(np.uint32), want)
        native.cuttDestroy(h)
    # another element size or permutation is another key
    h4, d4 = _plan(native, dims, perm, 8, False)
    assert "(model)" in capfd.readouterr().err
    native.cuttDestroy(h4)
    native.clear_plan_cache()


def test_damaged_cache_entries_are_ignored(native, oracle_mod, tmp_path):
    """A copy method stored for a transposing problem, or tile parameters no tile can be built
    from, must not be used: the plan falls back to the cost model and stays correct."""
    import torch
    dims, perm, elt = [64, 48, 20], [2, 1, 0], 4
    key = "%d/%d/%s/%s" % (torch.cuda.current_device(), elt, "".join("%d," % d for d in dims),
                           "".join("%d," % p for p in perm))
    a = raw_bits(volume(dims), elt, 9)
    want = oracle_mod.transpose_blocked(dims, perm, a)
    for entry in ("1 256 256 16384 0 256 2 16 16 0 1 1 0 1 0 0",    # memcpy for a non-identity problem
                  "0 256 256 16384 0 256 2 16 16 0 1 1 0 1 0 0",    # copy kernel, same
                  "2 4 4 4 0 512 2 16 16 0 1 1 0 1 0 0"):           # legal fields, absurdly small tile
        path = str(tmp_path / "c.txt")
        with open(path, "w") as f:
            f.write("# cutt-b200 plan cache v4\n%s %s\n" % (key, entry))
        native.clear_plan_cache()
        assert native.plan_cache_load(path) == 0
        out, desc = gpu_transpose(native, dims, perm, elt, a)
        assert_bit_exact(out, want, desc)
    native.clear_plan_cache()


_CHILD = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, %(root)r)
    sys.path.insert(0, os.path.join(%(root)r, "tests"))
    import numpy as np, torch
    import cutt_b200 as C, oracle
    from helpers import raw_bits, volume
    mode, path = sys.argv[1], sys.argv[2]
    C.lib()
    cases = [([300, 70, 90], [2, 0, 1], 4), ([257, 130, 6], [1, 0, 2], 8), ([40, 50, 60], [1, 2, 0], 4)]
    out = {"labels": [], "notes": [], "sizes": []}
    if mode == "load":
        assert C.plan_cache_load(path) == 0
    for dims, perm, elt in cases:
        a = raw_bits(volume(dims), elt, 1)
        tin = torch.from_numpy(a.view(np.int32 if elt == 4 else np.int64)).cuda()
        tout = torch.zeros_like(tin)
        if mode == "load":
            rc, h = C.cuttPlan(len(dims), dims, perm, elt, 0)
        else:
            rc, h = C.cuttPlanMeasure(len(dims), dims, perm, elt, 0, tin.data_ptr(), tout.data_ptr())
        assert rc == 0
        tout.zero_()
        assert C.cuttExecute(h, tin.data_ptr(), tout.data_ptr()) == 0
        torch.cuda.synchronize()
        want = oracle.transpose_blocked(dims, perm, a)
        assert np.array_equal(tout.cpu().numpy().view(want.dtype), want)
        out["labels"].append(json.loads(C.plan_describe(h))["label"])
        out["sizes"].append(C.plan_cache_size())
        C.cuttDestroy(h)
    if mode == "measure":
        assert C.plan_cache_save(path) == 0
    print("RESULT " + json.dumps(out))
""")


def _child(mode, path, env=None):
    e = dict(os.environ)
    e["CUTT_VERBOSE"] = "1"
    e.update(env or {})
    res = subprocess.run([sys.executable, "-c", _CHILD % {"root": ROOT}, mode, path], env=e,
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("RESULT ")][-1]
    return json.loads(line[7:]), res.stderr


def test_cache_file_is_reused_by_another_process(native, tmp_path):
    """Winners measured and saved by one process are what cuttPlan picks in the next, and the
    plans built from the file are bit-exact (checked inside the child against the oracle)."""
    path = str(tmp_path / "plans.txt")
    first, _ = _child("measure", path)
    assert first["sizes"] == [1, 2, 3]
    second, err = _child("load", path)
    assert second["labels"] == first["labels"]
    assert err.count("(cache)") == 3 and "(model)" not in err


def test_least_recently_used_entry_is_evicted(native, tmp_path):
    """Capacity 2 (CUTT_PLAN_CACHE_SIZE): measuring a third problem evicts the first."""
    path = str(tmp_path / "plans.txt")
    first, _ = _child("measure", path, {"CUTT_PLAN_CACHE_SIZE": "2"})
    assert first["sizes"] == [1, 2, 2]
    text = open(path).read()
    assert "/300,70,90,/" not in text and "/257,130,6,/" in text and "/40,50,60,/" in text
