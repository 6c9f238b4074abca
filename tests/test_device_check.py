"""The 64-bit device-side index checker (oracle/device_check.py) against the host oracle, on CPU
tensors: the GPU tests and the benchmark rely on it for tensors the host oracle cannot hold."""
import random

import numpy as np
import torch

from helpers import TEST3_CASES, README_CASE, random_case, raw_bits, volume
from oracle import device_check as DC


def _t(a):
    return torch.from_numpy(a.view(np.int32 if a.dtype.itemsize == 4 else np.int64))


def test_source_index_matches_the_c_oracle(oracle_mod):
    lib = oracle_mod.load()
    import ctypes
    rng = random.Random(3)
    for rank in range(2, 8):
        dims, perm = random_case(rng, rank, 50_000)
        vol = volume(dims)
        o = torch.arange(vol, dtype=torch.int64)
        src = DC.source_index(dims, perm, o).numpy()
        ia = (ctypes.c_int * rank)(*dims)
        pa = (ctypes.c_int * rank)(*perm)
        for k in [0, 1, vol // 3, vol - 1]:
            assert src[k] == lib.cutt_oracle_source_index(rank, ia, pa, k)
            assert src[k] == oracle_mod.source_index_formula_py(dims, perm, k)
        assert sorted(src.tolist()) == list(range(vol))


def test_accepts_oracle_output_and_counts_corruptions(oracle_mod):
    cases = [README_CASE, TEST3_CASES[0], TEST3_CASES[6], ([7, 5, 3, 4, 2], [4, 2, 0, 3, 1])]
    for dims, perm in cases:
        for elt in (4, 8):
            a = raw_bits(volume(dims), elt, 17)
            out = oracle_mod.transpose_blocked(dims, perm, a)
            assert DC.count_mismatches(dims, perm, _t(out), _t(a), chunk=1000) == 0
            bad = out.copy()
            bad[[1, bad.size // 2]] ^= 1
            assert DC.count_mismatches(dims, perm, _t(bad), _t(a), chunk=1000) == 2
            # the input itself is not the permutation of itself (no identity among the cases)
            assert DC.count_mismatches(dims, perm, _t(a), _t(a)) > 0


def test_pattern_mode_and_slabs(oracle_mod):
    dims, perm = [12, 10, 6, 8], [3, 2, 0, 1]
    vol = volume(dims)
    for elt in (4, 8):
        tin = torch.empty(vol, dtype=torch.int32 if elt == 4 else torch.int64)
        DC.fill_pattern(tin, 0, chunk=777)
        a = tin.numpy().view(np.uint32 if elt == 4 else np.uint64)
        assert len(np.unique(a)) == vol
        out = _t(oracle_mod.transpose_blocked(dims, perm, a))
        assert DC.count_mismatches(dims, perm, out, None, chunk=500) == 0
        # a slab of the output checked on its own, as one rank of a sharded job does
        lo, hi = vol // 4, vol // 2
        assert DC.count_mismatches(dims, perm, out[lo:hi].clone(), None, out_first=lo) == 0
        assert DC.count_mismatches(dims, perm, out[lo:hi].clone(), None, out_first=lo + 1) > 0
        # a slab of the input: perm keeps the last dimension, so output slab k reads input slab k
        dims2, perm2 = [12, 10, 6, 8], [1, 0, 2, 3]
        out2 = _t(oracle_mod.transpose_blocked(dims2, perm2, a))
        s = vol // 8
        assert DC.count_mismatches(dims2, perm2, out2[3 * s:4 * s].clone(), tin[3 * s:4 * s].clone(),
                                   out_first=3 * s, in_first=3 * s) == 0


def test_indices_beyond_32_bits():
    """Index arithmetic must not wrap at 2^31 or 2^32 elements."""
    dims, perm = [1024, 1024, 32, 256], [3, 2, 0, 1]
    o = torch.tensor([0, 2**31 + 5, 2**32 + 7, 2**33 - 1], dtype=torch.int64)
    src = DC.source_index(dims, perm, o).tolist()
    for oo, ss in zip(o.tolist(), src):
        # output order: dim3, dim2, dim0, dim1
        c3 = oo % 256; c2 = (oo // 256) % 32; c0 = (oo // 8192) % 1024; c1 = oo // (8192 * 1024)
        assert ss == c0 + 1024 * c1 + 1024 * 1024 * c2 + 1024 * 1024 * 32 * c3
    w = DC.pattern_words(torch.tensor([2**33 - 1], dtype=torch.int64), 4)
    assert w.dtype == torch.int32
    assert (int(w[0]) & 0xFFFFFFFF) == (((2**33 - 1) * 0x9E3779B1 + 0x7F4A7C15) & 0xFFFFFFFF)
