"""CPU tests of the plan builder and the kernels' index arithmetic.

libcutt_hostcheck.so (test-only) runs a plan's tile descriptor on host memory by calling
the same per-thread load/store phase functions the CUDA kernel calls.  Every result is
compared bit for bit with the CPU oracle."""
import ctypes
import itertools
import json
import os
import random

import numpy as np
import pytest

from helpers import README_CASE, TEST3_CASES, TEST4_CASE, dims_of_test1, random_case, raw_bits, volume


@pytest.fixture(scope="module")
def hc(native):
    path = os.path.join(os.path.dirname(native.lib_path()), "libcutt_hostcheck.so")
    lib = ctypes.CDLL(path)
    ip = ctypes.POINTER(ctypes.c_int)
    lib.cutt_hostcheck_num_candidates.argtypes = [ctypes.c_int, ip, ip, ctypes.c_int]
    lib.cutt_hostcheck_run.argtypes = [ctypes.c_int, ip, ip, ctypes.c_int, ctypes.c_int,
                                       ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    lib.cutt_hostcheck_run_params.argtypes = [ctypes.c_int, ip, ip, ctypes.c_int, ctypes.c_uint, ctypes.c_uint,
                                              ctypes.c_uint, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                              ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    lib.cutt_hostcheck_fastdiv.restype = ctypes.c_longlong
    lib.cutt_hostcheck_fastdiv.argtypes = [ctypes.c_uint, ctypes.c_ulonglong, ctypes.c_ulonglong]
    return lib


def _iarr(v):
    return (ctypes.c_int * len(v))(*v)


def _ext_expected(oracle_mod, dims, perm, elt, raw):
    """Permuted bytes of a tensor of 1-, 2- or 16-byte elements (the oracle handles 16 bytes as two
    8-byte words under an unpermuted innermost dimension of extent 2)."""
    if elt == 16:
        return oracle_mod.transpose_blocked([2] + list(dims), [0] + [p + 1 for p in perm],
                                            raw.view(np.uint64)).view(np.uint8)
    return oracle_mod.transpose_numpy(dims, perm, raw.view(np.uint8 if elt == 1 else np.uint16)).view(np.uint8)


@pytest.mark.parametrize("elt", [1, 2, 16])
def test_extension_element_sizes(hc, oracle_mod, elt):
    """The problems as the extension entry points re-state them, and the element-wise kernel's
    index arithmetic, on host memory with every access range-checked."""
    hc.cutt_hostcheck_run_ext.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                          ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_char_p, ctypes.c_int]
    rng = random.Random(31 + elt)
    cases = []
    for dims in ([3, 5], [4, 6], [8, 3, 5], [2, 3, 4, 5], [7, 66, 5], [130, 70], [258, 3, 9], [5, 300, 2, 3],
                 [132, 76], [8, 12, 20], [6, 4, 10, 8], [2, 5000], [4, 3000]):
        cases += [(dims, list(p)) for p in itertools.permutations(range(len(dims)))]
    for rank in range(2, 10):
        cases += [random_case(rng, rank, 60_000) for _ in range(3)]
    labels, seen = set(), set()
    for dims, perm in cases:
        raw = np.random.default_rng(volume(dims)).integers(0, 256, volume(dims) * elt, dtype=np.uint8)
        want = _ext_expected(oracle_mod, dims, perm, elt, raw)
        for idx in range(2):
            out = np.full_like(raw, 0xEE)
            lab = ctypes.create_string_buffer(4096)
            rc = hc.cutt_hostcheck_run_ext(len(dims), _iarr(dims), _iarr(perm), elt, idx, raw.ctypes.data,
                                           out.ctypes.data, lab, 4096)
            if rc == 3:
                break
            assert rc == 0, (rc, dims, perm, elt, idx)
            assert np.array_equal(out, want), (dims, perm, elt, idx, lab.value.decode())
            labels.add(lab.value.decode()[:5])
            seen.add(lab.value.decode()[:40])
    if elt < 4:
        assert "small" in labels and "memcp" in labels and '{"met' in labels
        assert any("ld32" in l for l in seen) and any("st32" in l for l in seen) and any("rows" in l for l in seen)


def _check_candidates(hc, oracle_mod, dims, perm, elts=(4, 8), max_cands=None, seed=0):
    for elt in elts:
        n = hc.cutt_hostcheck_num_candidates(len(dims), _iarr(dims), _iarr(perm), elt)
        assert n > 0, (dims, perm, elt)
        a = raw_bits(volume(dims), elt, seed + elt)
        want = oracle_mod.transpose_blocked(dims, perm, a)
        idx = range(n) if max_cands is None or n <= max_cands else sorted(random.Random(seed).sample(range(n), max_cands))
        for i in idx:
            out = np.full_like(a, 0xAB)
            lab = ctypes.create_string_buffer(2048)
            rc = hc.cutt_hostcheck_run(len(dims), _iarr(dims), _iarr(perm), elt, i, a.ctypes.data,
                                       out.ctypes.data, lab, 2048)
            assert rc == 0, (rc, dims, perm, elt, i)
            assert np.array_equal(out, want), (dims, perm, elt, i, lab.value.decode())


def test_small_tensors_get_enough_tiles(hc):
    """Latency-bound tensors: the model's first pick must spread the work over the SMs (the README
    example is 0.8 MB; a 64 KB tile would leave 135 of 148 SMs idle)."""
    for dims, perm in (README_CASE, ([256, 256], [1, 0]), ([64, 64, 64], [2, 1, 0])):
        for elt in (4, 8):
            a = raw_bits(volume(dims), elt, 1)
            out = np.empty_like(a)
            lab = ctypes.create_string_buffer(4096)
            rc = hc.cutt_hostcheck_run(len(dims), _iarr(dims), _iarr(perm), elt, 0, a.ctypes.data,
                                       out.ctypes.data, lab, 4096)
            assert rc == 0
            d = json.loads(lab.value.decode())
            assert d["num_tiles"] >= 64, (dims, elt, d["label"])


def test_fastdiv(hc):
    for d in [1, 2, 3, 5, 7, 31, 32, 33, 549, 1000, 14142, 65535, 65536, 65537,
              2**31 - 1, 2**31, 2**31 + 1, 2**32 - 1]:
        assert hc.cutt_hostcheck_fastdiv(d, 2**32 - 1, 99991) == 0, d


@pytest.mark.parametrize("rank", [2, 3, 4, 5])
def test_all_permutations_small(hc, oracle_mod, rank):
    dims = dims_of_test1(rank)
    for perm in itertools.permutations(range(rank)):
        _check_candidates(hc, oracle_mod, dims, list(perm), max_cands=3, seed=rank)


def test_all_permutations_rank6_sampled(hc, oracle_mod):
    dims = dims_of_test1(6)
    perms = list(itertools.permutations(range(6)))
    for perm in random.Random(6).sample(perms, 40):
        _check_candidates(hc, oracle_mod, dims, list(perm), elts=(4,), max_cands=2, seed=6)


@pytest.mark.parametrize("dims,perm", [README_CASE, TEST4_CASE] + [c for c in TEST3_CASES if volume(c[0]) < 3_000_000])
def test_reference_shapes(hc, oracle_mod, dims, perm):
    _check_candidates(hc, oracle_mod, dims, perm, max_cands=4, seed=1)


@pytest.mark.parametrize("dims,perm", [
    ([129, 130], [1, 0]), ([1000, 3], [1, 0]), ([3, 1000], [1, 0]), ([300, 301], [1, 0]),
    ([64, 48, 20], [2, 1, 0]), ([19, 16, 39], [2, 1, 0]), ([8, 6, 30, 50], [3, 0, 2, 1]),
    ([4, 3, 5, 40, 7, 24], [4, 1, 5, 0, 3, 2]), ([130, 4, 70], [0, 2, 1]), ([260, 70, 3], [1, 2, 0]),
    ([2, 2, 2, 2, 2, 2, 2, 2, 2, 2, 2], [10, 9, 8, 7, 6, 5, 4, 3, 2, 1, 0]),
    ([512, 66, 5], [1, 0, 2]), ([70, 66, 6, 4], [1, 0, 3, 2]),
])
def test_every_candidate(hc, oracle_mod, dims, perm):
    _check_candidates(hc, oracle_mod, dims, perm, seed=3)


def test_random_shapes(hc, oracle_mod):
    rng = random.Random(77)
    for rank in range(2, 13):
        for rep in range(5):
            dims, perm = random_case(rng, rank, 120_000)
            _check_candidates(hc, oracle_mod, dims, perm, max_cands=4, seed=rank * 10 + rep)


@pytest.mark.parametrize("kw", [
    dict(mv=4, mV=4), dict(mv=8, mV=8), dict(mv=16, mV=4), dict(mv=4, mV=16), dict(nt=128), dict(nt=512),
    dict(tin=128, tout=1024), dict(tin=1024, tout=128, vt=32768), dict(lo=1, ext=1), dict(tin=64, tout=64, vt=2048),
    dict(gi=2, tin=64, tout=64, vt=1024), dict(gi=4, go=4, tin=32, tout=32, vt=512), dict(go=2, lo=1, tin=64, tout=128, vt=2048),
])
def test_forced_parameters(hc, oracle_mod, kw):
    rng = random.Random(5)
    cases = [([64, 48, 20], [2, 1, 0]), ([130, 257], [1, 0]), ([8, 6, 30, 50], [3, 0, 2, 1]),
             ([256, 64, 12], [1, 0, 2]), ([96, 40, 33], [0, 2, 1]), ([132, 260, 3], [1, 0, 2])]
    cases += [random_case(rng, r, 100_000) for r in (3, 4, 5, 6)]
    for dims, perm in cases:
        if perm == sorted(perm):
            continue
        for elt in (4, 8):
            a = raw_bits(volume(dims), elt, 11)
            out = np.full_like(a, 0xCD)
            lab = ctypes.create_string_buffer(2048)
            rc = hc.cutt_hostcheck_run_params(
                len(dims), _iarr(dims), _iarr(perm), elt, kw.get("tin", 256), kw.get("tout", 256),
                kw.get("vt", 16384), kw.get("ext", 0), kw.get("lo", 0), kw.get("mv", 16), kw.get("mV", 16),
                kw.get("nt", 256), kw.get("gi", 1), kw.get("go", 1), a.ctypes.data, out.ctypes.data, lab, 2048)
            assert rc == 0, (rc, dims, perm, kw)
            assert np.array_equal(out, oracle_mod.transpose_blocked(dims, perm, a)), (dims, perm, elt, lab.value.decode())


@pytest.mark.parametrize("dims,perm", [
    ([130, 257], [1, 0]), ([64, 48, 20], [2, 1, 0]), ([64, 48, 20], [1, 0, 2]), ([31, 54, 2, 9], [3, 0, 2, 1]),
    ([317, 17, 6], [0, 2, 1]), ([8, 6, 30, 50], [3, 0, 2, 1]), ([12, 10, 7], [0, 1, 2]),
])
def test_host_pipeline_slabs(hc, oracle_mod, dims, perm):
    """Slabs of the input permuted into the strided full output (the host-buffer pipeline)."""
    hc.cutt_hostcheck_run_chunked.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                              ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    for elt in (4, 8):
        a = raw_bits(volume(dims), elt, 2)
        want = oracle_mod.transpose_blocked(dims, perm, a)
        for nslab in (1, 2, 3, 8):
            for index in (0, 2):
                out = np.full_like(a, 0x5A)
                rc = hc.cutt_hostcheck_run_chunked(len(dims), _iarr(dims), _iarr(perm), elt, nslab, index,
                                                   a.ctypes.data, out.ctypes.data)
                assert rc == 0, (rc, dims, perm, elt, nslab, index)
                assert np.array_equal(out, want), (dims, perm, elt, nslab, index)


def test_candidate_descriptions_are_json(hc):
    dims, perm = [64, 48, 20], [2, 1, 0]
    a = raw_bits(volume(dims), 4, 1)
    out = np.empty_like(a)
    lab = ctypes.create_string_buffer(2048)
    assert hc.cutt_hostcheck_run(3, _iarr(dims), _iarr(perm), 4, 0, a.ctypes.data, out.ctypes.data, lab, 2048) == 0
    d = json.loads(lab.value.decode())
    assert d["fused_dims"] == [64, 48, 20] and d["elt"] == 4 and d["num_tiles"] >= 1


def test_wide_row_offsets(hc, oracle_mod):
    """The kernel variant with 64-bit row offsets (selected by tiles that span 2^32 elements or
    more) on small problems: the planner is told to build every tile that way."""
    hc.cutt_hostcheck_force_wide.argtypes = [ctypes.c_int]
    hc.cutt_hostcheck_force_wide(1)
    try:
        rng = random.Random(77)
        cases = [README_CASE, ([129, 130], [1, 0]), ([4, 3, 5, 40, 7, 24], [4, 1, 5, 0, 3, 2]),
                 ([1305, 59, 8], [0, 2, 1]), ([64, 48, 20], [2, 1, 0])]
        cases += [random_case(rng, r, 40_000) for r in (2, 3, 4, 5, 6, 7)]
        wide = 0
        for dims, perm in cases:
            if perm == sorted(perm):
                continue
            for elt in (4, 8):
                n = hc.cutt_hostcheck_num_candidates(len(dims), _iarr(dims), _iarr(perm), elt)
                a = raw_bits(volume(dims), elt, 5 + elt)
                want = oracle_mod.transpose_blocked(dims, perm, a)
                for i in sorted(random.Random(elt).sample(range(n), min(n, 6))):
                    out = np.full_like(a, 0xAB)
                    lab = ctypes.create_string_buffer(2048)
                    rc = hc.cutt_hostcheck_run(len(dims), _iarr(dims), _iarr(perm), elt, i, a.ctypes.data,
                                               out.ctypes.data, lab, 2048)
                    assert rc == 0, (rc, dims, perm, elt, i)
                    assert np.array_equal(out, want), (dims, perm, elt, i, lab.value.decode())
                    wide += 1 if " wide" in lab.value.decode() else 0
        assert wide > 20
    finally:
        hc.cutt_hostcheck_force_wide(0)


def _tma(hc):
    hc.cutt_hostcheck_run_tma.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                          ctypes.c_int, ctypes.c_uint, ctypes.c_uint, ctypes.c_int, ctypes.c_int,
                                          ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    return hc.cutt_hostcheck_run_tma


@pytest.mark.parametrize("dims,perm", [
    ([64, 64], [1, 0]), ([132, 200], [1, 0]), ([36, 8, 44], [2, 1, 0]), ([40, 6, 52], [1, 2, 0]),
    ([72, 3, 5, 56], [3, 0, 2, 1]), ([24, 4, 3, 2, 40], [4, 2, 0, 3, 1]), ([256, 96, 3], [1, 0, 2]),
    ([16, 10, 36], [2, 0, 1]),
])
def test_tensor_map_transpose(hc, oracle_mod, dims, perm):
    """The tensor-map method on the host: box loads emulated (128-byte swizzle, zero fill outside
    the tensor), store phase = the device code, every access range- and alignment-checked.  All
    tile shapes, both tile orders, both element sizes; edge tiles in both dimensions."""
    run = _tma(hc)
    ran = 0
    for elt in (4, 8):
        a = raw_bits(volume(dims), elt, 41)
        want = oracle_mod.transpose_blocked(dims, perm, a)
        for ta in (128, 256, 512):
            for tb in (128, 256, 512):
                for order in (0, 1):
                    out = np.full_like(a, 0xAB)
                    lab = ctypes.create_string_buffer(2048)
                    rc = run(len(dims), _iarr(dims), _iarr(perm), elt, ta, tb, 1 + 2 * order, 128, order, a.ctypes.data,
                             out.ctypes.data, lab, 2048)
                    if rc == 2:
                        continue          # this tile shape does not apply to this problem
                    assert rc == 0, (rc, dims, perm, elt, ta, tb)
                    assert np.array_equal(out, want), (dims, perm, elt, ta, tb, order, lab.value.decode())
                    ran += 1
    assert ran >= 8, ran


def test_tensor_map_transpose_rejects_what_it_cannot_do(hc):
    run = _tma(hc)
    a = np.zeros(1 << 16, dtype=np.uint64)
    out = np.zeros_like(a)

    def rc(dims, perm, elt, ta=128, tb=128):
        return run(len(dims), _iarr(dims), _iarr(perm), elt, ta, tb, 3, 128, 0, a.ctypes.data, out.ctypes.data, None, 0)

    assert rc([64, 64], [1, 0], 4) == 0
    assert rc([66, 64], [1, 0], 4) == 2            # input rows of 264 bytes: not a multiple of 16
    assert rc([64, 66], [1, 0], 4) == 2            # output rows of 264 bytes
    assert rc([66, 64], [1, 0], 8) == 0            # the same extents are legal for 8-byte elements
    assert rc([64, 8, 64], [0, 2, 1], 4) == 2      # fastest dimension kept: not a transpose
    assert rc([64, 64], [0, 1], 4) == 2            # identity
    assert rc([16, 2, 2, 2, 2, 2, 16], [6, 5, 4, 3, 2, 1, 0], 4) == 2   # fused rank 7 > 5
    assert rc([64, 64], [1, 0], 4, ta=192) == 2    # tile bytes along dimension 0 must be 128, 256 or 512
    assert rc([64, 64], [1, 0], 4, tb=96) == 2     # 24 rows: not a multiple of 32


def test_tensor_map_candidates_are_enumerated_for_legal_strides_only(hc):
    def labels(dims, perm, elt):
        n = hc.cutt_hostcheck_num_candidates(len(dims), _iarr(dims), _iarr(perm), elt)
        a = np.zeros(volume(dims), dtype=np.uint32 if elt == 4 else np.uint64)
        out = np.zeros_like(a)
        res = []
        for i in range(n):
            lab = ctypes.create_string_buffer(2048)
            assert hc.cutt_hostcheck_run(len(dims), _iarr(dims), _iarr(perm), elt, i, a.ctypes.data, out.ctypes.data,
                                         lab, 2048) == 0
            res.append(json.loads(lab.value.decode())["label"])
        return res
    assert any(l.startswith("tma ") for l in labels([128, 96], [1, 0], 4))
    assert any(l.startswith("tma ") for l in labels([130, 98], [1, 0], 8))
    assert not any(l.startswith("tma ") for l in labels([130, 98], [1, 0], 4))


def _t2d(hc):
    hc.cutt_hostcheck_run_t2d.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                          ctypes.c_int, ctypes.c_uint, ctypes.c_uint, ctypes.c_int, ctypes.c_int,
                                          ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_char_p,
                                          ctypes.c_int]
    return hc.cutt_hostcheck_run_t2d


T2D_SHAPES = [
    ([300, 530], [1, 0]), ([1030, 9, 260], [2, 1, 0]), ([64, 64], [1, 0]), ([129, 130], [1, 0]), ([131, 67], [1, 0]), ([66, 202], [1, 0]), ([132, 200], [1, 0]),
    ([36, 8, 44], [2, 1, 0]), ([41, 6, 53], [1, 2, 0]), ([72, 3, 5, 57], [3, 0, 2, 1]), ([25, 4, 3, 2, 40], [4, 2, 0, 3, 1]),
    ([30, 2, 3, 2, 2, 3, 2, 34], [7, 6, 5, 4, 3, 2, 1, 0]), ([16, 10, 36], [2, 0, 1]), ([250, 3, 18], [2, 1, 0]),
    ([63, 65], [1, 0]), ([97, 16], [1, 0]),
]


@pytest.mark.parametrize("dims,perm", T2D_SHAPES)
def test_two_dimensional_tiles(hc, oracle_mod, dims, perm):
    """The swizzled two-dimensional tile method on the host, every access range- and
    alignment-checked: the wide modes the strides select (aligned cp.async / 16-byte stores, or the
    shift loads and sheared stores for rows that are not 16-byte aligned), the same forced to
    shift + shear, and the plain narrow modes; every tile shape, both tile orders, both element
    sizes; odd extents give edge tiles in both dimensions."""
    run = _t2d(hc)
    modes = set()
    for elt in (4, 8):
        a = raw_bits(volume(dims), elt, 43)
        want = oracle_mod.transpose_blocked(dims, perm, a)
        for ta in (128, 256):
            for tb in (32, 64):
                for order, nt in ((0, 128), (1, 256), (2, 128), (3, 256)):
                    for maxvec, force in ((16, 0), (16, 1), (8, 0), (4, 0)):
                        if maxvec < elt:
                            continue
                        out = np.full_like(a, 0xAB)
                        lab = ctypes.create_string_buffer(2048)
                        rc = run(len(dims), _iarr(dims), _iarr(perm), elt, ta, tb, nt, order, maxvec, force,
                                 a.ctypes.data, out.ctypes.data, lab, 2048)
                        if rc == 2 and order >= 2:
                            continue          # banded orders need at least 8 tiles across the band dimension
                        assert rc == 0, (rc, dims, perm, elt, ta, tb, maxvec, force)
                        label = json.loads(lab.value.decode())["label"]
                        assert np.array_equal(out, want), (dims, perm, elt, label)
                        modes.add(label.split(" lo=")[0].split(" ", 2)[2])
    assert "in/shift out/shear" in modes


@pytest.mark.parametrize("off_in,off_out", [(0, 0), (1, 0), (0, 1), (1, 1), (3, 2), (2, 3)])
def test_two_dimensional_tiles_on_unaligned_buffers(hc, oracle_mod, off_in, off_out):
    """Shift loads and sheared stores take any element-aligned buffer address: the buffers start
    1-3 elements past a 16-byte boundary; the words around the output must stay untouched."""
    run = _t2d(hc)
    for dims, perm in (([131, 67], [1, 0]), ([64, 64], [1, 0]), ([41, 6, 53], [1, 2, 0]), ([130, 3, 34], [2, 1, 0])):
        for elt in (4, 8):
            vol = volume(dims)
            a = raw_bits(vol, elt, 47)
            want = oracle_mod.transpose_blocked(dims, perm, a)
            dt = a.dtype
            backing_in = np.zeros(vol + 8, dtype=dt)
            backing_out = np.full(vol + 8, 0x5A, dtype=dt)
            base_in = (-backing_in.ctypes.data // elt) % (16 // elt)      # elements up to the next 16-byte boundary
            base_out = (-backing_out.ctypes.data // elt) % (16 // elt)
            oi, oo = base_in + off_in % (16 // elt), base_out + off_out % (16 // elt)
            backing_in[oi:oi + vol] = a
            for ta, tb in ((128, 32), (256, 64)):
                backing_out[:] = 0x5A
                rc = run(len(dims), _iarr(dims), _iarr(perm), elt, ta, tb, 128, 0, 16, 1,
                         backing_in.ctypes.data + oi * elt, backing_out.ctypes.data + oo * elt, None, 0)
                assert rc == 0, (rc, dims, perm, elt, off_in, off_out)
                assert np.array_equal(backing_out[oo:oo + vol], want), (dims, perm, elt, off_in, off_out)
                assert (backing_out[:oo] == 0x5A).all() and (backing_out[oo + vol:] == 0x5A).all()


def test_two_dimensional_tiles_modes_and_rejections(hc):
    run = _t2d(hc)
    a = np.zeros(1 << 16, dtype=np.uint64)
    out = np.zeros_like(a)

    def label(dims, perm, elt, maxvec=16, force=0):
        lab = ctypes.create_string_buffer(2048)
        rc = run(len(dims), _iarr(dims), _iarr(perm), elt, 128, 32, 128, 0, maxvec, force, a.ctypes.data, out.ctypes.data,
                 lab, 2048)
        return rc, (json.loads(lab.value.decode())["label"] if rc == 0 else "")

    assert "in/w4 out/w4" in label([64, 64], [1, 0], 4)[1]
    assert "in/w2 out/w4" in label([66, 64], [1, 0], 4)[1]       # input rows on 8-byte boundaries
    assert "in/w4 out/w1" in label([64, 67], [1, 0], 4)[1]       # output rows on 4-byte boundaries
    assert "in/w1 out/w2" in label([67, 66], [1, 0], 4)[1]
    assert "in/w1 out/w1" in label([67, 67], [1, 0], 8)[1]
    assert "in/w2 out/w2" in label([66, 66], [1, 0], 8)[1]
    assert "in/shift out/shear" in label([67, 66], [1, 0], 4, force=1)[1]
    assert "in/shift out/shear" in label([64, 64], [1, 0], 4, force=1)[1]
    assert "in/w2 out/w1" in label([66, 67], [1, 0], 4, maxvec=8)[1]
    assert "in/w1 out/w1" in label([64, 64], [1, 0], 4, maxvec=4)[1]
    assert label([64, 8, 64], [0, 2, 1], 4)[0] == 2              # fastest dimension kept
    assert label([64, 64], [0, 1], 4)[0] == 2                    # identity
    assert label([8, 64], [1, 0], 4)[0] == 2                     # 32-byte rows: mostly padding
    assert label([64, 8], [1, 0], 4)[0] == 2


def test_two_byte_elements_on_swizzled_tiles(hc, oracle_mod):
    """2-byte elements whose output rows start on 16-byte boundaries take the two-dimensional tile
    method with its 8 x 8 register transpose (input rows on 16-, 8- or 4-byte boundaries); other
    shapes stay on the element-wise kernel."""
    hc.cutt_hostcheck_run_ext.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                          ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_char_p, ctypes.c_int]
    seen = set()
    cases = [([64, 72], [1, 0]), ([136, 200], [1, 0]), ([36, 264], [1, 0]), ([34, 8, 40], [2, 1, 0]), ([130, 3, 5, 48], [3, 0, 2, 1]),
             ([72, 6, 136], [1, 2, 0]), ([200, 3, 24], [2, 0, 1]), ([64, 70], [1, 0]), ([33, 72], [1, 0]),
             ([72, 68], [1, 0]), ([134, 204], [1, 0]), ([40, 5, 132], [2, 1, 0]), ([260, 3, 76], [2, 0, 1])]   # 8-byte output rows
    for dims, perm in cases:
        raw = np.random.default_rng(volume(dims)).integers(0, 65536, volume(dims), dtype=np.uint16)
        want = oracle_mod.transpose_numpy(dims, perm, raw)
        out = np.full_like(raw, 0xEEEE)
        lab = ctypes.create_string_buffer(4096)
        rc = hc.cutt_hostcheck_run_ext(len(dims), _iarr(dims), _iarr(perm), 2, 0, raw.ctypes.data, out.ctypes.data, lab, 4096)
        assert rc == 0, (rc, dims, perm)
        assert np.array_equal(out, want), (dims, perm, lab.value.decode())
        seen.add((tuple(dims), lab.value.decode().split(" ")[0]))
    assert ((64, 72), "t2d") in seen and ((136, 200), "t2d") in seen and ((36, 264), "t2d") in seen
    assert ((34, 8, 40), "t2d") in seen                     # input rows on 4-byte boundaries
    assert ((64, 70), "small") in seen                      # output rows of 140 bytes: on 4-byte boundaries only
    assert ((33, 72), "small") in seen                      # input rows on 2-byte boundaries
    for d in ((72, 68), (134, 204), (40, 5, 132), (260, 3, 76)):
        assert (d, "t2d") in seen                           # 8-byte stores


def test_swizzled_tile_candidates_lead_with_the_frequent_winners(hc):
    """cuttPlanMeasure times only the first few candidates of the two-dimensional tile family; for a
    large tensor those are the forms that win most often (256-byte x 64-row tiles, banded tile order
    2, 256 threads), and the whole family sits inside the range the measurement covers."""
    import json
    hc.cutt_hostcheck_describe.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                           ctypes.c_int, ctypes.c_int, ctypes.c_char_p, ctypes.c_int]
    buf = ctypes.create_string_buffer(8192)
    for dims, perm, elt, tile in (([14142, 14142], [1, 0], 8, "t=32x64"), ([1024, 1024, 512], [1, 0, 2], 4, "t=64x64")):
        n = hc.cutt_hostcheck_num_candidates(len(dims), _iarr(dims), _iarr(perm), elt)
        first = []
        for i in range(n):
            assert hc.cutt_hostcheck_describe(len(dims), _iarr(dims), _iarr(perm), elt, i, buf, 8192) == 0
            d = json.loads(buf.value.decode())
            if d["label"].startswith("t2d"):
                first.append((i, d["label"]))
        assert first and first[0][0] < 48, first[:2]
        assert tile in first[0][1] and "lo=2" in first[0][1] and "nt=256" in first[0][1], first[0]
        assert all(tile in lab for _, lab in first[:8]), first[:8]
    assert hc.cutt_hostcheck_describe(2, _iarr([64, 64]), _iarr([1, 0]), 4, 100000, buf, 8192) == 3


@pytest.mark.parametrize("elt", [1, 2])
def test_small_elements_random_shapes(hc, oracle_mod, elt):
    """Random rank 2-4 shapes whose extents are multiples of 4, 8 or 16 elements: whatever path the
    extension picks (swizzled tiles with 16- or 8-byte stores, re-stated units, element-wise kernel),
    every access stays in range and aligned and the result is the permutation."""
    import random
    hc.cutt_hostcheck_run_ext.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                          ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_char_p, ctypes.c_int]
    rng = random.Random(100 + elt)
    kinds = {}
    for _ in range(60):
        rank = rng.choice([2, 2, 3, 3, 4])
        unit = rng.choice([4, 8, 16])
        dims = [unit * rng.randint(2, 24 if rank == 2 else 9) if rng.random() < 0.8 else rng.randint(2, 9) for _ in range(rank)]
        if volume(dims) > 150_000:
            continue
        perm = list(range(rank))
        while perm == sorted(perm):
            rng.shuffle(perm)
        raw = np.random.default_rng(volume(dims)).integers(0, 256 ** elt, volume(dims), dtype=np.uint8 if elt == 1 else np.uint16)
        want = oracle_mod.transpose_numpy(dims, perm, raw)
        out = np.full_like(raw, 0xEE)
        lab = ctypes.create_string_buffer(4096)
        rc = hc.cutt_hostcheck_run_ext(len(dims), _iarr(dims), _iarr(perm), elt, 0, raw.ctypes.data, out.ctypes.data, lab, 4096)
        assert rc == 0, (rc, dims, perm, lab.value.decode())
        assert np.array_equal(out, want), (dims, perm, lab.value.decode())
        text = lab.value.decode()
        kind = text.split(" ")[0] + (" " + [w for w in text.split(" ") if w.startswith("out/")][0] if text.startswith("t2d") else "")
        kinds[kind] = kinds.get(kind, 0) + 1
    assert any(k.startswith("t2d") for k in kinds), kinds
    assert sum(kinds.values()) >= 40, kinds


def test_one_byte_elements_on_swizzled_tiles(hc, oracle_mod):
    """1-byte elements whose output rows start on 16-byte boundaries take the two-dimensional tile
    method with its 16 x 16 byte transpose (input rows on 16-, 8- or 4-byte boundaries, ragged
    edges along both tile dimensions); other shapes stay on the element-wise kernel."""
    hc.cutt_hostcheck_run_ext.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                          ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_char_p, ctypes.c_int]
    seen = set()
    cases = [([128, 64], [1, 0]), ([272, 208], [1, 0]), ([72, 272], [1, 0]), ([68, 8, 80], [2, 1, 0]), ([260, 3, 5, 48], [3, 0, 2, 1]),
             ([144, 6, 144], [1, 2, 0]), ([400, 3, 32], [2, 0, 1]), ([300, 16], [1, 0]), ([128, 72], [1, 0]), ([66, 80], [1, 0]),
             ([128, 76], [1, 0]), ([264, 200], [1, 0]), ([72, 5, 136], [2, 1, 0])]
    for dims, perm in cases:
        raw = np.random.default_rng(volume(dims)).integers(0, 256, volume(dims), dtype=np.uint8)
        want = oracle_mod.transpose_numpy(dims, perm, raw)
        out = np.full_like(raw, 0xEE)
        lab = ctypes.create_string_buffer(4096)
        rc = hc.cutt_hostcheck_run_ext(len(dims), _iarr(dims), _iarr(perm), 1, 0, raw.ctypes.data, out.ctypes.data, lab, 4096)
        assert rc == 0, (rc, dims, perm)
        assert np.array_equal(out, want), (dims, perm, lab.value.decode())
        seen.add((tuple(dims), lab.value.decode().split(" ")[0]))
    assert ((128, 64), "t2d") in seen and ((272, 208), "t2d") in seen and ((72, 272), "t2d") in seen
    assert ((68, 8, 80), "t2d") in seen                     # input rows on 4-byte boundaries
    assert ((300, 16), "t2d") in seen                       # a single vector along the output rows
    assert ((128, 72), "t2d") in seen and ((264, 200), "t2d") in seen and ((72, 5, 136), "t2d") in seen   # 8-byte stores
    assert ((128, 76), "small") in seen                     # output rows of 76 bytes: on 4-byte boundaries only
    assert ((66, 80), "small") in seen                      # input rows on 2-byte boundaries
