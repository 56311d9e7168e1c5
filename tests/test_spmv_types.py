"""The complex and int8 instances of the reference's SpMV type table
(cuda/kernel/level2/alphasparse_spmv.cu:246-262, 276-287).

CPU part: the complex restatement of the oracle against the reference's own compiled
alphasparse_c_mv / alphasparse_z_mv (within rounding: the reference's assembly unrolls its partial
sums).  GPU part: the CUDA instances through the C ABI against the oracle - complex within the
tolerances of the real types (relative L2 1e-5 / 1e-12), int8 with int32 arithmetic exactly, int8
with float arithmetic within 1e-5.  The int8 instances have no CPU counterpart in the reference:
their parity is against the restated arithmetic only.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import rel_l2
from library_b200 import generators as G


def _complex_case(A, dtype, seed):
    rng = np.random.default_rng(seed)
    rp, ci, _ = A.numpy()
    rt = np.float32 if dtype == np.complex64 else np.float64
    v = (rng.normal(size=A.nnz) + 1j * rng.normal(size=A.nnz)).astype(dtype)
    x = (rng.uniform(-1, 1, A.cols) + 1j * rng.uniform(-1, 1, A.cols)).astype(dtype)
    y0 = (rng.uniform(-1, 1, A.rows) + 1j * rng.uniform(-1, 1, A.rows)).astype(dtype)
    return rp, ci, v, x, y0, rt


@pytest.mark.parametrize("dtype,tol", [(np.complex64, 1e-6), (np.complex128, 1e-14)])
def test_complex_restatement_against_the_compiled_reference(dtype, tol):
    if not oracle.have_ref():
        pytest.skip("the reference's CPU code was not built here")
    for A in (G.rmat(10, 8, seed=41), G.laplacian_2d_5pt(24), G.poisson_random(500, 700, 5.0, seed=42)):
        rp, ci, v, x, y0, _ = _complex_case(A, dtype, 43)
        for alpha, beta in ((1.0, 0.0), (1.5 - 0.5j, 0.25 + 2.0j)):
            want = oracle.ref_spmv_complex(rp, ci, v, x, alpha, beta, y0, cols=A.cols)
            got = oracle.spmv_complex(rp, ci, v, x, alpha, beta, y0)
            assert np.linalg.norm(got - want) <= tol * np.linalg.norm(want)


def test_int8_restatement_small_case_by_hand():
    rp = np.array([0, 2, 2, 5], dtype=np.int32)
    ci = np.array([0, 2, 0, 1, 2], dtype=np.int32)
    v = np.array([3, -4, 127, -128, 5], dtype=np.int8)
    x = np.array([2, -7, 100], dtype=np.int8)
    y0 = np.array([10, 20, 30], dtype=np.int32)
    want = np.array([2 * (3 * 2 - 4 * 100) - 3 * 10, -3 * 20, 2 * (127 * 2 + 128 * 7 + 5 * 100) - 3 * 30])
    assert np.array_equal(oracle.spmv_int8(rp, ci, v, x, 2, -3, y0), want)
    got = oracle.spmv_int8(rp, ci, v, x, 2.0, -3.0, y0.astype(np.float32))
    assert np.array_equal(got, want.astype(np.float32))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(np.complex64, 1e-5), (np.complex128, 1e-12)])
@pytest.mark.parametrize("off", [np.int32, np.int64])
def test_complex_spmv_on_the_gpu(handle, dtype, tol, off):
    from library_b200 import api
    handle.use_torch_stream()
    for A in (G.rmat(13, 16, seed=44), G.laplacian_2d_5pt(40), G.poisson_random(3000, 2000, 9.0, seed=45)):
        rp, ci, v, x, y0, _ = _complex_case(A, dtype, 46)
        Am = api.CsrMatrix(A.rows, A.cols, torch.from_numpy(rp.astype(off)).cuda(), torch.from_numpy(ci).cuda(),
                           torch.from_numpy(v).cuda())
        for alpha, beta in ((1.0, 0.0), (1.5 - 0.5j, 0.25 + 2.0j)):
            want = oracle.spmv_complex(rp, ci, v, x, alpha, beta, y0)
            y = torch.from_numpy(y0.copy()).cuda()
            api.spmv(handle, Am, api.DnVec(torch.from_numpy(x).cuda()), api.DnVec(y), alpha, beta)
            torch.cuda.synchronize()
            got = y.cpu().numpy()
            assert np.linalg.norm(got - want) <= tol * np.linalg.norm(want)
        with pytest.raises(api.AlphaSparseError):      # no conjugate transpose (the transposed copy keeps the values)
            api.spmv(handle, Am, api.DnVec(torch.zeros(A.rows, dtype=y.dtype, device="cuda")),
                     api.DnVec(torch.zeros(A.cols, dtype=y.dtype, device="cuda")), 1.0, 0.0, op=api.OP_C)


@pytest.mark.gpu
@pytest.mark.parametrize("ydtype", [np.int32, np.float32])
def test_int8_spmv_on_the_gpu(handle, ydtype):
    from library_b200 import api
    handle.use_torch_stream()
    rng = np.random.default_rng(47)
    for A in (G.rmat(13, 16, seed=48), G.poisson_random(3000, 2000, 9.0, seed=49)):
        rp, ci, _ = A.numpy()
        v = rng.integers(-128, 128, size=A.nnz).astype(np.int8)
        x = rng.integers(-128, 128, size=A.cols).astype(np.int8)
        y0 = rng.integers(-1000, 1000, size=A.rows).astype(ydtype)
        want = oracle.spmv_int8(rp, ci, v, x, 3, -2, y0)
        Am = api.CsrMatrix(A.rows, A.cols, torch.from_numpy(rp).cuda(), torch.from_numpy(ci).cuda(), torch.from_numpy(v).cuda())
        y = torch.from_numpy(y0.copy()).cuda()
        api.spmv(handle, Am, api.DnVec(torch.from_numpy(x).cuda()), api.DnVec(y), 3, -2)
        torch.cuda.synchronize()
        got = y.cpu().numpy()
        if ydtype == np.int32:
            assert np.array_equal(got, want)
        else:
            assert rel_l2(got, want) <= 1e-5
