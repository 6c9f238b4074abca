"""64-bit index checker for permuted tensors that are too large for the host oracle.

TEST INFRASTRUCTURE ONLY (like the rest of this package): tests, the smoke check and the
benchmark's verification step use it; nothing in the shipped library does.

It plays the role of the reference's GPU checker (src/TensorTester.cu:39-96 evaluates, per
output element, the source index ``sum_j ((o / c_j) mod d_j) * ct_j`` built by
src/TensorTester.cu:151-170) with two differences: all index arithmetic is 64-bit, so tensors
of 2^31 elements and more can be checked (the reference's checker uses ``int``), and the
expected value is either gathered from the input tensor or recomputed from a closed-form
pattern of the source index, which lets one GPU check its slab of a tensor that is sharded over
several GPUs without reading the other GPUs' memory.

Everything is written with torch int64 tensor arithmetic over chunks of the output, so the same
code runs on a CUDA device and (for the unit tests against the host oracle) on the CPU.
"""
from __future__ import annotations

from typing import Optional, Sequence

import torch

_MUL = 0x9E3779B1          # odd 32-bit multiplier: consecutive indices give unrelated words
_ADD = 0x7F4A7C15


def conv_constants(dim: Sequence[int], perm: Sequence[int]):
    """c, d, ct of src/TensorTester.cu:151-170 as Python integers."""
    rank = len(dim)
    c = [0] * rank
    ct = [0] * rank
    c[perm[0]] = 1
    ct[0] = 1
    for i in range(1, rank):
        c[perm[i]] = c[perm[i - 1]] * int(dim[perm[i - 1]])
        ct[i] = ct[i - 1] * int(dim[i - 1])
    return c, [int(x) for x in dim], ct


def source_index(dim, perm, o: torch.Tensor) -> torch.Tensor:
    """Source element index for every output index in ``o`` (int64 tensor)."""
    c, d, ct = conv_constants(dim, perm)
    src = torch.zeros_like(o)
    for j in range(len(dim)):
        src += torch.remainder(torch.div(o, c[j], rounding_mode="floor"), d[j]) * ct[j]
    return src


def pattern_words(idx: torch.Tensor, elt: int) -> torch.Tensor:
    """Closed-form content of element ``idx`` (int64 tensor): a 32-bit hash of the index for
    4-byte elements; for 8-byte elements the index itself in the high word and the hash in the
    low word.  Returned as int32 / int64 bit patterns."""
    h = (idx * _MUL + _ADD) & 0xFFFFFFFF
    if elt == 4:
        return torch.where(h >= 2**31, h - 2**32, h).to(torch.int32)
    return (idx << 32) | h


def fill_pattern(t: torch.Tensor, first_index: int = 0, chunk: int = 1 << 26) -> None:
    """Writes the pattern of elements ``first_index ..`` into ``t`` (int32 or int64, 1-D)."""
    elt = t.element_size()
    n = t.numel()
    for a in range(0, n, chunk):
        b = min(n, a + chunk)
        idx = torch.arange(first_index + a, first_index + b, dtype=torch.int64, device=t.device)
        t[a:b] = pattern_words(idx, elt)


def count_mismatches(dim, perm, out: torch.Tensor, inp: Optional[torch.Tensor] = None, *,
                     out_first: int = 0, in_first: int = 0, chunk: int = 1 << 26,
                     sample_stride: int = 1) -> int:
    """Number of output elements that differ from the permutation of the input.

    ``out`` holds the output elements ``out_first .. out_first + out.numel()`` of the whole
    tensor (int32/int64 bit patterns, 1-D).  The expected value of output element o is
    ``inp[src(o) - in_first]`` when ``inp`` is given, else ``pattern_words(src(o))``.
    With ``sample_stride`` k > 1 only every k-th chunk-sized block of the output is checked
    (blocks keep whole tiles of any kernel inside the sample).
    """
    elt = out.element_size()
    if elt not in (4, 8):
        raise ValueError("out must hold 4- or 8-byte words")
    if inp is not None and inp.element_size() != elt:
        raise ValueError("input and output element sizes differ")
    n = out.numel()
    bad = 0
    for k, a in enumerate(range(0, n, chunk)):
        if sample_stride > 1 and k % sample_stride:
            continue
        b = min(n, a + chunk)
        o = torch.arange(out_first + a, out_first + b, dtype=torch.int64, device=out.device)
        src = source_index(dim, perm, o)
        del o
        if inp is not None:
            want = inp[src - in_first]
        else:
            want = pattern_words(src, elt)
        del src
        bad += int((out[a:b] != want).sum().item())
        del want
    return bad
