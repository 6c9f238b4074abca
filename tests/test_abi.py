"""The drop-in boundary without a GPU: the library loads, exports every symbol its headers
declare (C ABI and the C++-mangled names of the original interface), and rejects bad input
with the original result codes before touching the device."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Itanium-mangled names of the four functions of the original cutt.h (no extern "C" there).
MANGLED = [
    "_Z8cuttPlanPjiPiS0_mP11CUstream_st",
    "_Z15cuttPlanMeasurePjiPiS0_mP11CUstream_stPvS3_",
    "_Z11cuttExecutejPvS_",
    "_Z11cuttDestroyj",
]


def _declared_c_symbols():
    text = open(os.path.join(ROOT, "include", "cutt_c.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(cutt_c_\w+)\s*\(", text)))


def _nm(path, dynamic):
    out = subprocess.run(["nm", "-D" if dynamic else "-g", "--defined-only", path],
                         stdout=subprocess.PIPE, text=True, check=True).stdout
    return set(line.split()[-1] for line in out.splitlines() if line.strip())


def test_shared_library_exports_everything_declared(native):
    syms = _nm(native.lib_path(), dynamic=True)
    declared = _declared_c_symbols()
    assert len(declared) >= 14
    for s in declared + MANGLED:
        assert s in syms, s
    for s in declared:
        assert hasattr(native.lib(), s)


def test_static_archive_exports_the_original_symbols(native):
    ar = os.path.join(os.path.dirname(native.lib_path()), "libcutt.a")
    syms = _nm(ar, dynamic=False)
    for s in MANGLED + _declared_c_symbols():
        assert s in syms, s


def test_header_matches_original_interface():
    text = open(os.path.join(ROOT, "include", "cutt.h")).read()
    code = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    enum = re.search(r"typedef enum cuttResult_t \{(.*?)\} cuttResult;", code, flags=re.S).group(1)
    names = [x.strip() for x in enum.split(",") if x.strip()]
    assert names == ["CUTT_SUCCESS", "CUTT_INVALID_PLAN", "CUTT_INVALID_PARAMETER", "CUTT_INVALID_DEVICE",
                     "CUTT_INTERNAL_ERROR", "CUTT_UNDEFINED_ERROR"]
    assert "typedef unsigned int cuttHandle;" in code
    flat = " ".join(code.split())
    assert "cuttResult cuttPlan(cuttHandle* handle, int rank, int* dim, int* permutation, size_t sizeofType, cudaStream_t stream);" in flat
    assert ("cuttResult cuttPlanMeasure(cuttHandle* handle, int rank, int* dim, int* permutation, size_t sizeofType, "
            "cudaStream_t stream, void* idata, void* odata);") in flat
    assert "cuttResult cuttDestroy(cuttHandle handle);" in flat
    assert "cuttResult cuttExecute(cuttHandle handle, void* idata, void* odata);" in flat


def test_validation_codes_without_device(native):
    """Rules and order of src/cutt.cpp:59-82: they are applied before any CUDA call."""
    P = native.cuttPlan
    bad = native.CUTT_INVALID_PARAMETER
    assert P(2, [4, 4], [1, 0], 3, 0)[0] == bad          # element size
    assert P(2, [4, 4], [1, 0], 16, 0)[0] == bad
    assert P(1, [4], [0], 4, 0)[0] == bad                # rank
    assert P(0, [], [], 4, 0)[0] == bad
    assert P(2, [4, 1], [1, 0], 4, 0)[0] == bad          # dims must be >= 2
    assert P(2, [0, 4], [1, 0], 4, 0)[0] == bad
    assert P(3, [4, 4, 4], [0, 1, 1], 4, 0)[0] == bad    # permutation must be a bijection
    assert P(3, [4, 4, 4], [0, 1, 3], 4, 0)[0] == bad
    assert P(3, [4, 4, 4], [0, -1, 2], 4, 0)[0] == bad
    rc, _ = native.cuttPlanMeasure(2, [4, 4], [1, 0], 3, 0, 0, 0)
    assert rc == bad
    assert native.cuttExecute(123456, 0, 0) == native.CUTT_INVALID_PLAN
    assert native.cuttDestroy(123456) == native.CUTT_INVALID_PLAN
    assert native.lib().cutt_c_version().startswith(b"cutt-b200")


def test_extension_entry_validation_without_device(native):
    """cutt_c_plan_ext accepts 1, 2, 4, 8, 16 bytes and applies the original's other rules."""
    bad = native.CUTT_INVALID_PARAMETER
    for elt in (0, 3, 5, 12, 32):
        assert native.plan_ext([4, 4], [1, 0], elt, 0)[0] == bad
    for elt in (1, 2, 4, 8, 16):
        assert native.plan_ext([4], [0], elt, 0)[0] == bad
        assert native.plan_ext([4, 1], [1, 0], elt, 0)[0] == bad
        assert native.plan_ext([4, 4, 4], [0, 1, 1], elt, 0)[0] == bad


def test_missing_library_fails_loudly(monkeypatch, native):
    import cutt_b200
    monkeypatch.setattr(cutt_b200, "_lib", None)
    monkeypatch.setattr(cutt_b200, "lib_path", lambda: "/nonexistent/libcutt.so")
    with pytest.raises(ImportError):
        cutt_b200.lib()


def test_plan_cache_file_roundtrip(native, tmp_path):
    path = str(tmp_path / "plans.txt")
    with open(path, "w") as f:
        f.write("# cutt-b200 plan cache v4\n0/4/64,48,/1,0, 2 128 512 65536 1 512 2 16 16 1 2 4 0 1 0 0\n")
    native.clear_plan_cache()
    assert native.plan_cache_load(path) == 0
    assert native.plan_cache_size() == 1
    out = str(tmp_path / "out.txt")
    assert native.plan_cache_save(out) == 0
    assert "0/4/64,48,/1,0, 2 128 512 65536 1 512 2 16 16 1 2 4 0 1 0 0" in open(out).read()
    native.clear_plan_cache()
    assert native.plan_cache_size() == 0


def test_plan_cache_load_rejects_foreign_and_damaged_files(native, tmp_path):
    """Only this format version is read; entries with fields out of range are skipped, so a stale
    or edited file can never install a method or tile parameters the planner would not produce."""
    good = "0/4/64,48,/1,0, 2 128 512 65536 1 512 2 16 16 1 2 4 0 1 0 0"
    bad_param = native.CUTT_INVALID_PARAMETER

    def load(text):
        path = str(tmp_path / "p.txt")
        with open(path, "w") as f:
            f.write(text)
        native.clear_plan_cache()
        return native.plan_cache_load(path), native.plan_cache_size()

    assert load("# cutt-b200 plan cache v4\n" + good + "\n") == (0, 1)
    # an older layout, no header, or a header that only starts the same way: nothing is read
    assert load("# cutt-b200 plan cache v3\n" + good + "\n") == (bad_param, 0)
    assert load(good + "\n") == (bad_param, 0)
    assert load("# cutt-b200 plan cache v41\n" + good + "\n") == (bad_param, 0)
    assert load("") == (bad_param, 0)
    # damaged entries: thread count 0 or not a power of two, 3 stages, odd vector bytes, the
    # small-element method (5), unknown methods, short lines
    body = "\n".join([
        "0/4/64,48,/1,0, 2 128 512 65536 1 0 2 16 16 1 2 4 0 1 0 0",
        "0/4/64,48,/1,0, 2 128 512 65536 1 384 2 16 16 1 2 4 0 1 0 0",
        "0/4/64,48,/1,0, 2 128 512 65536 1 256 3 16 16 1 2 4 0 1 0 0",
        "0/4/64,48,/1,0, 2 128 512 65536 1 256 2 12 16 1 2 4 0 1 0 0",
        "0/4/64,48,/1,0, 2 128 512 65536 1 256 2 16 16 1 3 4 0 1 0 0",
        "0/4/64,48,/1,0, 5 128 512 65536 1 256 2 16 16 1 2 4 0 1 0 0",
        "0/4/64,48,/1,0, 9 128 512 65536 1 256 2 16 16 1 2 4 0 1 0 0",
        "0/4/64,48,/1,0, 2 128 512",
    ])
    assert load("# cutt-b200 plan cache v4\n" + body + "\n") == (bad_param, 0)
    assert load("# cutt-b200 plan cache v4\n" + body + "\n" + good + "\n") == (0, 1)
    # the element-per-thread kernel (3) can be a measured winner for small tensors
    assert load("# cutt-b200 plan cache v4\n"
                "0/4/64,48,/1,0, 3 128 512 65536 1 256 2 16 16 1 2 4 0 1 0 0\n") == (0, 1)
    native.clear_plan_cache()


def test_c3_case_list_is_reproducible():
    from cutt_b200 import workloads as W
    cases = W.c3_cases(100)
    assert len(cases) == 100
    for i in (0, 17, 63, 99):
        assert W.generate_c3_case(i) == (cases[i][0], cases[i][1])
    for dims, perm in cases:
        vol = 1
        for d in dims:
            vol *= d
        assert abs(vol - 2.0e8) <= 0.05 * 2.0e8 and 2 <= len(dims) <= 7 and all(d >= 2 for d in dims)
        assert sorted(perm) == list(range(len(dims))) and perm != sorted(perm)


def test_cost_model_evaluate_tool(tmp_path):
    """The fitted model header parses and ranks sweep records (cutt_b200/cost_model/evaluate.py)."""
    import json
    import subprocess
    import sys
    import numpy as np
    rng = np.random.default_rng(0)
    path = tmp_path / "sweep.jsonl"
    with open(path, "w") as f:
        for case in ("A", "B"):
            for i in range(12):
                feat = [float(x) for x in rng.uniform(0, 64, 32)]
                f.write(json.dumps({"case": case, "elt": 4, "idx": i, "gbs": float(1000 + 100 * i), "ms": 1.0,
                                    "label": "tiles synthetic %d" % i, "feat": feat, "model_us": 1.0}) + "\n")
    res = subprocess.run([sys.executable, "-m", "cutt_b200.cost_model.evaluate", str(path)], cwd=ROOT,
                         stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    assert "records 24, groups 2" in res.stdout and "best of first 48: median 1.000" in res.stdout
