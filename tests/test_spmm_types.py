"""The complex, int8 and fp16 instances of the reference's SpMM type table
(cuda/kernel/level3/alphasparse_spmm.cu:556-596).

CPU part: the complex restatement of the oracle (the generic row kernel of the reference's CPU backend,
hygon/kernel/level3/mm/gemm/gemm_csr_row.hpp:76-122) against the reference's own compiled alphasparse_c_mm /
alphasparse_z_mm, within rounding; the oracle's fp16 conversions against numpy's.  GPU part: the CUDA instances
through the C ABI against the oracle - complex within the tolerances of the real types (relative L2 1e-5 / 1e-12:
the oracle scales by beta first and adds alpha*a*x entry by entry, the kernel sums and scales at the end), int8 with
int32 arithmetic exactly, the float-arithmetic instances bit for bit (same operations in the same order).  The
int8 and fp16 instances have no CPU counterpart in the reference: their parity is against the restated arithmetic
only.
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import rel_l2
from library_b200 import generators as G


def _cplx(rng, shape, dtype):
    return (rng.uniform(-1, 1, shape) + 1j * rng.uniform(-1, 1, shape)).astype(dtype)


@pytest.mark.parametrize("dtype,tol", [(np.complex64, 1e-6), (np.complex128, 1e-14)])
def test_complex_spmm_restatement_against_the_compiled_reference(dtype, tol):
    if not oracle.have_ref():
        pytest.skip("the reference's CPU code was not built here")
    rng = np.random.default_rng(51)
    for A in (G.rmat(9, 8, seed=52), G.laplacian_2d_5pt(20), G.poisson_random(400, 300, 5.0, seed=53)):
        rp, ci, _ = A.numpy()
        v = _cplx(rng, A.nnz, dtype)
        for n in (1, 7, 33):
            X, Y0 = _cplx(rng, (A.cols, n), dtype), _cplx(rng, (A.rows, n), dtype)
            for alpha, beta in ((1.0, 0.0), (1.5 - 0.5j, 0.25 + 2.0j)):
                want = oracle.ref_spmm_complex(rp, ci, v, X, alpha, beta, Y0)
                got = oracle.spmm_complex(rp, ci, v, X, alpha, beta, Y0)
                assert np.linalg.norm(got - want) <= tol * np.linalg.norm(want)


def test_complex_restatements_against_the_golden_vectors():
    """The committed outputs of the reference's complex mv / mm (tests/golden/csr_golden_complex.npz) pin the oracle's
    complex restatements where the reference itself is not at hand."""
    from conftest import load_golden_complex
    for name, c in load_golden_complex().items():
        tol = 1e-6 if c["v"].dtype == np.complex64 else 1e-14
        if c["kind"] == "mv":
            got = oracle.spmv_complex(c["rp"], c["ci"], c["v"], c["x"], c["alpha"], c["beta"], c["y0"])
        else:
            got = oracle.spmm_complex(c["rp"], c["ci"], c["v"], c["x"], c["alpha"], c["beta"], c["y0"])
        assert rel_l2(got, c["y"]) <= tol, name


@pytest.mark.gpu
def test_complex_kernels_against_the_golden_vectors(handle):
    """The CUDA complex SpMV and SpMM against the reference's committed outputs."""
    from conftest import load_golden_complex
    from library_b200 import api
    handle.use_torch_stream()
    for name, c in load_golden_complex().items():
        tol = 1e-5 if c["v"].dtype == np.complex64 else 1e-12
        dev = "cuda"
        Am = api.CsrMatrix(len(c["rp"]) - 1, c["cols"], torch.from_numpy(c["rp"]).to(dev), torch.from_numpy(c["ci"]).to(dev),
                           torch.from_numpy(c["v"]).to(dev))
        y = torch.from_numpy(np.array(c["y0"], copy=True)).to(dev)
        x = torch.from_numpy(c["x"]).to(dev)
        if c["kind"] == "mv":
            api.spmv(handle, Am, api.DnVec(x), api.DnVec(y), c["alpha"], c["beta"])
        else:
            api.spmm(handle, Am, api.DnMat(x), api.DnMat(y), c["alpha"], c["beta"])
        torch.cuda.synchronize()
        assert rel_l2(y.cpu().numpy(), c["y"]) <= tol, name


def test_fp16_conversions_of_the_oracle_match_numpy():
    """Every half bit pattern widens to numpy's float32, and rounding back (through the fp16 -> fp16 instance with an
    identity matrix) is numpy's round-to-nearest-even, ties and subnormals included."""
    h = np.arange(65536, dtype=np.uint32).astype(np.uint16).view(np.float16)
    h = h[np.isfinite(h) & (h.view(np.uint16) != 0x8000)]      # -0 + (+0) = +0 in the sum: not a conversion matter
    n = h.size
    rp = np.arange(n + 1, dtype=np.int32)
    ci = np.arange(n, dtype=np.int32)
    one = np.ones(n, dtype=np.float16)
    X = h.reshape(n, 1)
    wide = oracle.spmm_wide(rp, ci, one, X, 1.0, 0.0, np.zeros((n, 1), np.float32))
    assert np.array_equal(wide[:, 0], h.astype(np.float32))
    rng = np.random.default_rng(5)
    scale = np.float32(rng.uniform(0.3, 3.0))
    back = oracle.spmm_wide(rp, ci, one, X, float(scale), 0.0, np.zeros((n, 1), np.float16))
    with np.errstate(over="ignore"):
        want = (scale * h.astype(np.float32)).astype(np.float16)
    assert np.array_equal(back[:, 0].view(np.uint16), want.view(np.uint16))


def _run(handle, A, v, X, Y0, alpha, beta, ld_pad=0, col_major=False, off=np.int32):
    from library_b200 import api
    dev = "cuda"
    rp, ci, _ = A.numpy()
    Am = api.CsrMatrix(A.rows, A.cols, torch.from_numpy(rp.astype(off)).to(dev), torch.from_numpy(ci).to(dev),
                       torch.from_numpy(v).to(dev))
    n = X.shape[1]
    Xt, Yt = torch.from_numpy(X).to(dev), torch.from_numpy(np.array(Y0, copy=True)).to(dev)
    if ld_pad:
        bx = torch.zeros(X.shape[0], n + ld_pad, dtype=Xt.dtype, device=dev)
        bx[:, :n] = Xt
        Xt = bx[:, :n]
        by = torch.zeros(Y0.shape[0], n + ld_pad, dtype=Yt.dtype, device=dev)
        by[:, :n] = Yt
        Yt = by[:, :n]
    if col_major:
        Xt, Yt = Xt.t().contiguous().t(), Yt.t().contiguous().t()
    handle.use_torch_stream()
    Bd, Cd = api.DnMat(Xt), api.DnMat(Yt)
    buf = None
    if col_major:
        buf = torch.empty(api.spmm_buffer_size(handle, Am, Bd, Cd), dtype=torch.uint8, device=dev)
    api.spmm(handle, Am, Bd, Cd, alpha, beta, buffer=buf)
    torch.cuda.synchronize()
    assert api.spmm_last_variant(Am) == "types"
    assert Am.plan(handle)[0]["device_error"] == 0
    return Yt.cpu().numpy()


MATS = [lambda: G.rmat(11, 12, seed=61), lambda: G.laplacian_2d_5pt(30), lambda: G.poisson_random(2000, 1500, 7.0, seed=62)]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [(np.complex64, 1e-5), (np.complex128, 1e-12)])
def test_complex_spmm_on_the_gpu(handle, dtype, tol):
    rng = np.random.default_rng(63)
    for make in MATS:
        A = make()
        rp, ci, _ = A.numpy()
        v = _cplx(rng, A.nnz, dtype)
        for n, pad in ((1, 0), (20, 4), (64, 0)):
            X, Y0 = _cplx(rng, (A.cols, n), dtype), _cplx(rng, (A.rows, n), dtype)
            for alpha, beta in ((1.0, 0.0), (0.5 + 1.5j, -1.25 + 0.5j)):
                want = oracle.spmm_complex(rp, ci, v, X, alpha, beta, Y0)
                got = _run(handle, A, v, X, Y0, alpha, beta, ld_pad=pad)
                assert rel_l2(got, want) <= tol
    got = _run(handle, A, v, X, Y0, alpha, beta, col_major=True)      # column-major B and C through the copies
    assert rel_l2(got, want) <= tol


@pytest.mark.gpu
def test_int8_spmm_on_the_gpu(handle):
    rng = np.random.default_rng(64)
    for make in MATS:
        A = make()
        rp, ci, _ = A.numpy()
        v = rng.integers(-128, 128, A.nnz).astype(np.int8)
        for n in (1, 20, 64):
            X = rng.integers(-128, 128, (A.cols, n)).astype(np.int8)
            Yi = rng.integers(-10**6, 10**6, (A.rows, n)).astype(np.int32)
            for alpha, beta in ((1, 0), (3, -2)):
                assert np.array_equal(_run(handle, A, v, X, Yi, alpha, beta), oracle.spmm_wide(rp, ci, v, X, alpha, beta, Yi))
                assert np.array_equal(_run(handle, A, v, X, Yi, alpha, beta, off=np.int64),      # 64-bit row offsets
                                      oracle.spmm_wide(rp.astype(np.int64), ci, v, X, alpha, beta, Yi))
                Yf = Yi.astype(np.float32) / 1000
                got = _run(handle, A, v, X, Yf, float(alpha), float(beta))
                assert np.array_equal(got, oracle.spmm_wide(rp, ci, v, X, float(alpha), float(beta), Yf))


@pytest.mark.gpu
def test_fp16_spmm_on_the_gpu(handle):
    rng = np.random.default_rng(65)
    for make in MATS:
        A = make()
        rp, ci, _ = A.numpy()
        v = rng.standard_normal(A.nnz).astype(np.float16)
        for n, pad in ((1, 0), (20, 2), (64, 0)):
            X = rng.uniform(-1, 1, (A.cols, n)).astype(np.float16)
            Y32 = rng.uniform(-1, 1, (A.rows, n)).astype(np.float32)
            for alpha, beta in ((1.0, 0.0), (1.5, 0.5)):
                got = _run(handle, A, v, X, Y32, alpha, beta, ld_pad=pad)
                assert np.array_equal(got, oracle.spmm_wide(rp, ci, v, X, alpha, beta, Y32))
                Y16 = Y32.astype(np.float16)
                got = _run(handle, A, v, X, Y16, alpha, beta, ld_pad=pad)
                want = oracle.spmm_wide(rp, ci, v, X, alpha, beta, Y16)
                assert np.array_equal(got.view(np.uint16), want.view(np.uint16))


def _transposed(A, v):
    """CSR of the transpose (numpy), entries of a row in ascending column order like the device copy."""
    rp, ci, _ = A.numpy()
    rows_of = np.repeat(np.arange(A.rows, dtype=np.int64), np.diff(rp))
    order = np.lexsort((rows_of, ci))
    trp = np.zeros(A.cols + 1, dtype=np.int32)
    np.add.at(trp, ci + 1, 1)
    trp = np.cumsum(trp).astype(np.int32)
    return trp, rows_of[order].astype(np.int32), v[order]


@pytest.mark.gpu
def test_transposed_a_for_complex_and_int8(handle):
    """opA = TRANSPOSE runs on a transposed copy the plan builds on the device (values moved as they are, 1- to
    16-byte elements): SpMV and SpMM against the oracle on the explicitly transposed matrix.  The conjugate
    transpose of a complex matrix is refused."""
    from library_b200 import api
    handle.use_torch_stream()
    dev = "cuda"
    rng = np.random.default_rng(66)
    A = G.poisson_random(900, 1300, 6.0, seed=67)
    rp, ci, _ = A.numpy()
    for dtype, tol in ((np.complex64, 1e-5), (np.complex128, 1e-12)):
        v = _cplx(rng, A.nnz, dtype)
        trp, tci, tv = _transposed(A, v)
        Am = api.CsrMatrix(A.rows, A.cols, torch.from_numpy(rp).to(dev), torch.from_numpy(ci).to(dev), torch.from_numpy(v).to(dev))
        x, y0 = _cplx(rng, A.rows, dtype), _cplx(rng, A.cols, dtype)
        y = torch.from_numpy(y0.copy()).to(dev)
        api.spmv(handle, Am, api.DnVec(torch.from_numpy(x).to(dev)), api.DnVec(y), 0.5 - 1j, 2.0 + 0.5j, op=api.OP_T)
        torch.cuda.synchronize()
        assert rel_l2(y.cpu().numpy(), oracle.spmv_complex(trp, tci, tv, x, 0.5 - 1j, 2.0 + 0.5j, y0)) <= tol
        X, Y0 = _cplx(rng, (A.rows, 12), dtype), _cplx(rng, (A.cols, 12), dtype)
        Y = torch.from_numpy(Y0.copy()).to(dev)
        api.spmm(handle, Am, api.DnMat(torch.from_numpy(X).to(dev)), api.DnMat(Y), 1.5, -0.5j, op=api.OP_T)
        torch.cuda.synchronize()
        assert rel_l2(Y.cpu().numpy(), oracle.spmm_complex(trp, tci, tv, X, 1.5, -0.5j, Y0)) <= tol
        with pytest.raises(api.AlphaSparseError) as e:
            api.spmv(handle, Am, api.DnVec(torch.from_numpy(x).to(dev)), api.DnVec(y), 1.0, 0.0, op=api.OP_C)
        assert e.value.status == 6
    v8 = rng.integers(-128, 128, A.nnz).astype(np.int8)
    trp, tci, tv = _transposed(A, v8)
    Am = api.CsrMatrix(A.rows, A.cols, torch.from_numpy(rp).to(dev), torch.from_numpy(ci).to(dev), torch.from_numpy(v8).to(dev))
    x8 = rng.integers(-128, 128, A.rows).astype(np.int8)
    y0 = rng.integers(-1000, 1000, A.cols).astype(np.int32)
    y = torch.from_numpy(y0.copy()).to(dev)
    api.spmv(handle, Am, api.DnVec(torch.from_numpy(x8).to(dev)), api.DnVec(y), 3, -2, op=api.OP_T)
    torch.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy(), oracle.spmv_int8(trp, tci, tv, x8, 3, -2, y0))
    X8 = rng.integers(-128, 128, (A.rows, 9)).astype(np.int8)
    Y0 = rng.integers(-1000, 1000, (A.cols, 9)).astype(np.int32)
    Y = torch.from_numpy(Y0.copy()).to(dev)
    api.spmm(handle, Am, api.DnMat(torch.from_numpy(X8).to(dev)), api.DnMat(Y), 3, -2, op=api.OP_T)
    torch.cuda.synchronize()
    assert np.array_equal(Y.cpu().numpy(), oracle.spmm_wide(trp, tci, tv, X8, 3, -2, Y0))
