"""The copy entry point that allocates nothing (cutt_c_copy_noalloc).

Some hosts cannot allocate device memory when they need a copy (the device's memory is managed
by their own allocator, or an allocation's device-wide synchronisation is not allowed where they
are), so this entry point keeps its status words in a fixed array inside the library.  The test
calls it through the C ABI twice in a row and compares both results, bit for bit, with what the
library's regular identity plan (cuttPlan + cuttExecute) produces for the same input; the second
call also checks that the shared array was cleared and reused correctly.

The file name makes pytest collect it last."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_no_alloc_copy_matches_regular_copy(native):
    import torch
    dims = [4099, 32, 77]                      # 10.1 M elements; the byte count is not a multiple of the 32 KB stage
    perm = [0, 1, 2]
    vol = 4099 * 32 * 77
    assert (vol * 4) % 16 == 0 and (vol * 4) % 32768 != 0
    for elt, dt in ((8, torch.int64), (4, torch.int32)):
        nbytes = vol * elt
        if nbytes % 16:
            continue
        g = torch.Generator(device="cuda")
        g.manual_seed(77 + elt)
        src = torch.randint(-2**31, 2**31 - 1, (vol,), dtype=dt, device="cuda", generator=g)
        # the existing entry points: an identity plan executed by the library's copy kernel
        want = torch.full_like(src, -1)
        rc, h = native.plan_params(dims, perm, elt, 0, method=0)
        assert rc == native.CUTT_SUCCESS
        assert native.cuttExecute(h, src.data_ptr(), want.data_ptr()) == native.CUTT_SUCCESS
        torch.cuda.synchronize()
        assert native.cuttDestroy(h) == native.CUTT_SUCCESS
        assert torch.equal(want, src)
        # the no-allocation entry point, two calls in a row into fresh outputs
        stream = torch.cuda.current_stream().cuda_stream
        for call in range(2):
            got = torch.full_like(src, -1)
            assert native.copy_noalloc(src.data_ptr(), got.data_ptr(), nbytes, stream) == 0
            torch.cuda.synchronize()
            assert native.copy_noalloc_timeouts() == 0
            assert torch.equal(got, want), (elt, call)
    # a small copy (one stage, one block) and the documented rejections
    a = torch.arange(4096, dtype=torch.int32, device="cuda")
    b = torch.zeros_like(a)
    assert native.copy_noalloc(a.data_ptr(), b.data_ptr(), 4096 * 4, 0) == 0
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    bad = native.CUTT_INVALID_PARAMETER
    assert native.copy_noalloc(a.data_ptr() + 4, b.data_ptr(), 1024, 0) == bad        # misaligned source
    assert native.copy_noalloc(a.data_ptr(), b.data_ptr(), 1000, 0) == bad            # not a multiple of 16
    assert native.copy_noalloc(a.data_ptr(), a.data_ptr(), 1024, 0) == bad            # in place
    assert native.copy_noalloc(a.data_ptr(), b.data_ptr(), (1 << 40) + 16, 0) == bad  # over the size limit
    assert native.copy_noalloc(0, b.data_ptr(), 1024, 0) == bad
    assert native.copy_noalloc_timeouts() == 0


def test_no_alloc_status_after_a_large_then_a_small_copy_on_a_side_stream(native):
    """The status reader must wait for the copy itself (the stream here is one of torch's side
    streams, which a plain blocking copy does not wait for) and must report only the latest call:
    a large launch (one block per SM) is followed by a one-block launch, with no synchronisation
    by the caller in between or before the status is read."""
    import torch
    side = torch.cuda.Stream()
    big = torch.arange(64 << 20, dtype=torch.int32, device="cuda")      # 256 MB: every SM gets chunks
    big_out = torch.zeros_like(big)
    small = torch.arange(2048, dtype=torch.int32, device="cuda") * 3    # 8 KB: a single block
    small_out = torch.zeros_like(small)
    torch.cuda.synchronize()
    s = side.cuda_stream
    assert native.copy_noalloc(big.data_ptr(), big_out.data_ptr(), big.numel() * 4, s) == 0
    assert native.copy_noalloc(small.data_ptr(), small_out.data_ptr(), small.numel() * 4, s) == 0
    assert native.copy_noalloc_timeouts() == 0      # waits for both copies before reading
    assert torch.equal(small_out, small)
    assert torch.equal(big_out, big)
    # the regular copy's counter has the same waiting rule
    assert native.copy_timeouts() == 0
