"""The cumulative sum that brings its own scratch, for callers that cannot allocate device memory.

Called through the C ABI only, and compared bit for bit with the entry point that takes the caller's
scratch.  Two calls in a row share the library's built-in array: the second (a shorter input of the
other integer width) must not be disturbed by what the first left there.  This file sorts after the
other test files on purpose, so a run that stops at the first failure has already run them all; it also
passes on its own in a fresh process.
"""
import numpy as np
import pytest


def _both(cabi, torch, x):
    """(result of the entry point with caller scratch, result of the one without) for the host array x."""
    lib = cabi.lib()
    bits = x.dtype.itemsize * 8
    t = torch.from_numpy(x).cuda()
    want = torch.empty(x.size + 1, dtype=t.dtype, device="cuda")
    got = torch.full((x.size + 1,), -7, dtype=t.dtype, device="cuda")
    need = lib.tbe_b200_complete_cumsum_scratch_bytes(x.size)
    scratch = torch.empty(max(need, 8), dtype=torch.uint8, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    cabi.check(lib.tbe_b200_complete_cumsum(t.data_ptr(), x.size, bits, want.data_ptr(), scratch.data_ptr(), need, stream), "cumsum")
    cabi.check(lib.tbe_b200_complete_cumsum_static(t.data_ptr(), x.size, bits, got.data_ptr(), stream), "cumsum without allocation")
    torch.cuda.synchronize()
    return want.cpu().numpy(), got.cpu().numpy()


@pytest.mark.gpu
def test_cumsum_without_allocation_matches_on_two_calls_in_a_row():
    import torch
    import fbgemm_ascend_b200  # noqa: F401
    from fbgemm_ascend_b200 import cabi

    rng = np.random.default_rng(11)
    first = rng.integers(0, 1000, 3_000_001).astype(np.int64)        # 1465 tiles of the built-in array get written
    second = rng.integers(0, 100, 70_000).astype(np.int32)           # 35 tiles; the rest still holds the first call's sums
    for x in (first, second):
        want, got = _both(cabi, torch, x)
        assert np.array_equal(got, want)
        assert np.array_equal(got[1:], np.cumsum(x, dtype=x.dtype)) and got[0] == 0
    # short inputs (one tile, no scratch at all) and the empty input
    for n in (0, 1, 2048):
        want, got = _both(cabi, torch, np.arange(n, dtype=np.int64))
        assert np.array_equal(got, want)


@pytest.mark.gpu
def test_cumsum_without_allocation_refuses_inputs_beyond_its_array():
    import torch
    import fbgemm_ascend_b200  # noqa: F401
    from fbgemm_ascend_b200 import cabi

    lib = cabi.lib()
    limit = lib.tbe_b200_complete_cumsum_static_max_elements()
    assert limit == 8192 * 2048
    t = torch.zeros(8, dtype=torch.int64, device="cuda")
    rc = lib.tbe_b200_complete_cumsum_static(t.data_ptr(), limit + 1, 64, t.data_ptr(), None)   # refused before any launch
    assert rc != 0 and str(limit) in cabi.last_error()
    assert lib.tbe_b200_complete_cumsum_static(t.data_ptr(), 4, 16, t.data_ptr(), None) != 0      # only 32- and 64-bit integers
