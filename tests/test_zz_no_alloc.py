"""volta_b200_colsum_noalloc: the column-sum entry point for callers that may not allocate
(latency-critical host threads, processes whose device memory is all in their own pool,
plug-ins barred from the allocator after start-up).  Its scratch is a buffer inside the library
image, shared by every call, so the checks are: same bits as the entry point with caller scratch,
twice in a row with different inputs (the second call finds the first call's leftovers in the
buffer), and a clean refusal beyond the built-in size.  Collected last on purpose."""
import numpy as np
import pytest
import torch

from volta_b200 import load_library

pytestmark = pytest.mark.gpu


def _both(lib, a):
    rows, cols = a.shape
    da = torch.from_numpy(a).cuda()
    ref = torch.zeros(cols, device="cuda")
    scratch = torch.zeros(max(1, lib.volta_b200_colsum_scratch_floats(rows, cols)), device="cuda")
    assert lib.volta_b200_colsum(ref.data_ptr(), da.data_ptr(), rows, cols, scratch.data_ptr(), None) == 0
    out = torch.full((cols,), float("nan"), device="cuda")
    assert lib.volta_b200_colsum_noalloc(out.data_ptr(), da.data_ptr(), rows, cols, None) == 0
    torch.cuda.synchronize()
    return ref.cpu().numpy(), out.cpu().numpy()


def test_noalloc_colsum_matches_the_allocating_entry_point_twice_in_a_row():
    lib = load_library()
    rs = np.random.RandomState(123)
    # first call: a tall input that fills many scratch chunks; second: a different shape, so it
    # reads a buffer still holding the first call's partials
    for rows, cols in ((70000, 130), (4096, 1024), (64, 1)):
        a = rs.randn(rows, cols).astype(np.float32)
        ref, out = _both(lib, a)
        assert np.array_equal(ref.view(np.uint32), out.view(np.uint32))
        exact = a.astype(np.float64).sum(axis=0)
        assert np.all(np.abs(out - exact) <= 1e-6 * np.abs(a).astype(np.float64).sum(axis=0) + 1e-30)


def test_noalloc_colsum_refuses_what_does_not_fit():
    lib = load_library()
    rows, cols = 4096, 1200000         # one chunk of 1.2 M columns > 1 Mi scratch floats
    assert lib.volta_b200_colsum_scratch_floats(rows, cols) > (1 << 20)
    a = torch.zeros(8, device="cuda")  # never touched: the size check comes first
    assert lib.volta_b200_colsum_noalloc(a.data_ptr(), a.data_ptr(), rows, cols, None) == 7
    assert lib.volta_b200_colsum_noalloc(None, a.data_ptr(), 4, 4, None) == 1
