"""The tcgen05 3xTF32 GEMM through the C ABI (volta_b200_gemm, tensor path) against fp64
and against the FFMA kernel: exact on tf32-representable integers (any layout or
descriptor mistake shows as a wrong integer), fp32-grade on real data."""
import numpy as np
import pytest
import torch

from volta_b200 import load_library

pytestmark = pytest.mark.gpu

NN, NT, TN = 0, 1, 2
FFMA, TENSOR, PAIR = 1, 2, 3


def _run(layout, path, A, B):
    lib = load_library()
    m, k = A.shape
    n = B.shape[1]
    a_store = A if layout in (NN, NT) else np.ascontiguousarray(A.T)
    b_store = B if layout in (NN, TN) else np.ascontiguousarray(B.T)
    da = torch.from_numpy(np.ascontiguousarray(a_store)).cuda()
    db = torch.from_numpy(np.ascontiguousarray(b_store)).cuda()
    out = torch.full((m, n), float("nan"), device="cuda")
    rc = lib.volta_b200_gemm(layout, path, out.data_ptr(), da.data_ptr(), db.data_ptr(), m, n, k, None)
    torch.cuda.synchronize()
    return rc, out.cpu().numpy()


# m, n, k: single tile / single k-block first, then multi-tile, ragged edges, long K, small M
SHAPES = [(128, 128, 32), (128, 128, 256), (256, 384, 64), (64, 1024, 1024), (1024, 1024, 64), (200, 72, 300),
          (132, 260, 36), (4, 8, 4), (512, 128, 4096), (1000, 520, 260)]


def _supported(layout, m, n, k):
    a_inner = m if layout == TN else k
    b_inner = k if layout == NT else n
    return a_inner % 4 == 0 and b_inner % 4 == 0


@pytest.mark.parametrize("layout", [NT, NN, TN])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_tensor_gemm_exact_on_small_integers(layout, m, n, k):
    if not _supported(layout, m, n, k):
        pytest.skip("contiguous extent not a multiple of 4: takes the FFMA path")
    rs = np.random.RandomState(m + 3 * n + 7 * k + layout)
    A = rs.randint(-4, 5, size=(m, k)).astype(np.float32)
    B = rs.randint(-4, 5, size=(k, n)).astype(np.float32)
    rc, got = _run(layout, TENSOR, A, B)
    assert rc == 0
    ref = (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32)
    bad = np.argwhere(got != ref)
    assert bad.size == 0, "first mismatches (row, col): %s of %d" % (bad[:8].tolist(), len(bad))


@pytest.mark.parametrize("layout", [NT, NN, TN])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_tensor_gemm_fp32_grade_accuracy(layout, m, n, k):
    if not _supported(layout, m, n, k):
        pytest.skip("contiguous extent not a multiple of 4: takes the FFMA path")
    rs = np.random.RandomState(11 * m + n + k + layout)
    A = (rs.randn(m, k) * np.exp(rs.randn(m, 1))).astype(np.float32)
    B = rs.randn(k, n).astype(np.float32)
    rc, got = _run(layout, TENSOR, A, B)
    assert rc == 0
    ref = A.astype(np.float64) @ B.astype(np.float64)
    bound = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64)
    err = np.abs(got - ref) / (bound + 1e-30)
    # 3xTF32: each product carries < 3 * 2^-22; fp32 accumulation adds ~2^-24 per partial sum
    assert float(err.max()) <= 1.0e-6, float(err.max())
    rc2, ffma = _run(layout, FFMA, A, B)
    assert rc2 == 0
    err_ffma = np.abs(ffma - ref) / (bound + 1e-30)
    # no worse than an order of magnitude from plain fp32 FFMA accumulation
    assert float(err.max()) <= max(10 * float(err_ffma.max()), 4e-7)


def test_unsupported_shape_is_refused_not_faulted():
    A = np.ones((6, 6), np.float32)
    B = np.ones((6, 6), np.float32)
    rc, _ = _run(NN, TENSOR, A, B)
    assert rc == 6  # VB200_ERR_UNSUPPORTED


PAIR_SHAPES = [(256, 256, 32), (256, 512, 256), (512, 256, 4096), (1000, 520, 260), (384, 640, 96), (2048, 2048, 512)]


@pytest.mark.parametrize("layout", [NT, NN, TN])
@pytest.mark.parametrize("m,n,k", PAIR_SHAPES)
def test_cta_pair_gemm_exact_on_integers_and_close_on_reals(layout, m, n, k):
    """The cta_group::2 kernel (two CTAs per 256 x 256 tile) against fp64 and the single-CTA kernel."""
    rs = np.random.RandomState(5 * m + n + k + layout)
    A = rs.randint(-4, 5, size=(m, k)).astype(np.float32)
    B = rs.randint(-4, 5, size=(k, n)).astype(np.float32)
    rc, got = _run(layout, PAIR, A, B)
    assert rc == 0
    ref = (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32)
    bad = np.argwhere(got != ref)
    assert bad.size == 0, "first mismatches (row, col): %s of %d" % (bad[:8].tolist(), len(bad))
    A = rs.randn(m, k).astype(np.float32)
    B = rs.randn(k, n).astype(np.float32)
    rc, got = _run(layout, PAIR, A, B)
    assert rc == 0
    ref = A.astype(np.float64) @ B.astype(np.float64)
    bound = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64)
    assert float((np.abs(got - ref) / (bound + 1e-30)).max()) <= 2.0e-6


# The CTA-pair kernel with its own (unsplit) epilogue on ragged edges in every dimension: K short enough that no
# split is taken, so that the masked, staged stores of the kernel itself run in all three layouts.
PAIR_RAGGED = [(2300, 2308, 480), (516, 772, 260), (260, 1028, 36)]


@pytest.mark.parametrize("layout", [NT, NN, TN])
@pytest.mark.parametrize("m,n,k", PAIR_RAGGED)
def test_pair_kernel_unsplit_on_ragged_shapes(layout, m, n, k):
    import ctypes as C
    lib = load_library()
    splits = C.c_int32()
    assert lib.volta_b200_gemm_route(layout, 3, m, n, k, C.byref(splits)) == 2 and splits.value == 1
    rs = np.random.RandomState(m + n + k + layout)
    A = rs.randint(-4, 5, size=(m, k)).astype(np.float32)
    B = rs.randint(-4, 5, size=(k, n)).astype(np.float32)
    rc, got = _run(layout, 3, A, B)
    assert rc == 0
    assert np.array_equal(got, (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32))
    A = rs.randn(m, k).astype(np.float32)
    B = rs.randn(k, n).astype(np.float32)
    rc, got = _run(layout, 3, A, B)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    bound = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64)
    assert float(np.max(np.abs(got - ref) / (bound + 1e-30))) <= 1.0e-6

