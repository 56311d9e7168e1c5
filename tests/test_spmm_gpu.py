"""CUDA SpMM through the C ABI against the CPU oracle and the reference-made golden vectors.

The SIMT kernel accumulates every C element in the same order and with the same fma as the
reference's CPU kernel, so fp32 / fp64 results are compared bit for bit as well as within the
stated tolerance (relative L2 1e-5 fp32, 1e-12 fp64)."""
import functools

import numpy as np
import pytest
import torch

import oracle
from conftest import load_golden, rel_l2
from library_b200 import api
from library_b200 import generators as G

pytestmark = pytest.mark.gpu
TOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float64): 1e-12}
MM_CASES = sorted(k for k, c in load_golden().items() if c["kind"] == "mm")


def run_spmm(handle, rp, ci, v, X, alpha, beta, Y0, cols, ldx=None, ldy=None, alg=api.SPMM_ALG_DEFAULT,
             use_buffer=False, want_variant=None):
    dev = "cuda"
    A = api.CsrMatrix(len(rp) - 1, cols, torch.from_numpy(rp).to(dev), torch.from_numpy(ci).to(dev),
                      torch.from_numpy(v).to(dev))
    n = X.shape[1]
    Xt = torch.from_numpy(X).to(dev)
    Yt = torch.from_numpy(np.array(Y0, copy=True)).to(dev)
    if ldx:
        buf = torch.zeros(X.shape[0], ldx, dtype=Xt.dtype, device=dev)
        buf[:, :n] = Xt
        Xt = buf[:, :n]
    if ldy:
        buf = torch.full((Y0.shape[0], ldy), 7.0, dtype=Yt.dtype, device=dev)
        buf[:, :n] = Yt
        Yt = buf[:, :n]
    handle.use_torch_stream()
    Bd, Cd = api.DnMat(Xt), api.DnMat(Yt)
    ext = None
    if use_buffer:
        ext = torch.empty(api.spmm_buffer_size(handle, A, Bd, Cd, alg), dtype=torch.uint8, device=dev)
    api.spmm(handle, A, Bd, Cd, alpha, beta, alg=alg, buffer=ext)
    torch.cuda.synchronize()
    if want_variant:
        assert api.spmm_last_variant(A) == want_variant
    assert A.plan(handle)[0]["device_error"] == 0
    if ldy:
        assert bool((buf[:, n:] == 7.0).all())  # padding untouched
    return Yt.cpu().numpy()


@pytest.mark.parametrize("name", MM_CASES)
def test_golden(handle, golden, name):
    c = golden[name]
    Y = run_spmm(handle, c["rp"], c["ci"], c["v"], c["x"], c["alpha"], c["beta"], c["y0"], c["cols"])
    assert rel_l2(Y, c["y"]) <= TOL[c["v"].dtype]
    assert np.array_equal(Y, c["y"])


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("n", [1, 3, 4, 8, 20, 32, 64, 128, 130, 256])
def test_stencil_against_oracle(handle, dtype, n):
    t = torch.float32 if dtype == np.float32 else torch.float64
    A = G.stencil_3d_27pt(12, seed=4, dtype=t)
    rp, ci, v = A.numpy()
    X = G.uniform((A.cols, n), -1, 1, dtype=t, seed=60 + n).numpy()
    Y0 = G.uniform((A.rows, n), -1, 1, dtype=t, seed=61 + n).numpy()
    for alpha, beta in ((1.0, 0.0), (0.5, -1.5)):
        want = oracle.spmm(rp, ci, v, X, alpha, beta, Y0)
        got = run_spmm(handle, rp, ci, v, X, alpha, beta, Y0, A.cols)
        assert rel_l2(got, want) <= TOL[np.dtype(dtype)]
        assert np.array_equal(got, want)


@pytest.mark.parametrize("n", [8, 32])
def test_skewed_and_long_rows(handle, n):
    """Empty rows and rows longer than the shared-memory staging chunk."""
    A = G.rmat(13, 16, seed=71)
    rp, ci, v = A.numpy()
    assert np.diff(rp).max() > 1024 and (np.diff(rp) == 0).any()
    X = G.uniform((A.cols, n), -1, 1, seed=72).numpy()
    Y0 = G.uniform((A.rows, n), -1, 1, seed=73).numpy()
    want = oracle.spmm(rp, ci, v, X, 1.0, 1.0, Y0)
    # ALG1 = the reference's row-balanced algorithm: rows stay whole, so the result is the oracle's bit for bit
    got = run_spmm(handle, rp, ci, v, X, 1.0, 1.0, Y0, A.cols, alg=api.SPMM_CSR_ALG1, want_variant="row-block")
    assert np.array_equal(got, want)


@functools.lru_cache(maxsize=None)
def _skewed_cases():
    rng = np.random.default_rng(5)
    out = {"rmat": G.rmat(14, 16, seed=71)}
    # one 30,000-entry row (15 merge-path tiles) between runs of empty rows, short rows after it
    lens = np.concatenate([np.zeros(200, np.int64), [30000], np.zeros(3000, np.int64), rng.integers(0, 9, size=5000),
                           [5000], np.zeros(10, np.int64)])
    cols = 40000
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ci = np.concatenate([np.sort(rng.choice(cols, size=int(l), replace=False)) for l in lens if l]).astype(np.int32)
    out["one_long_row"] = G.Csr(len(lens), cols, torch.from_numpy(rp), torch.from_numpy(ci),
                                torch.from_numpy(rng.normal(size=ci.size).astype(np.float32)))
    out["no_entries"] = G.Csr(300, 50, torch.zeros(301, dtype=torch.int32), torch.zeros(0, dtype=torch.int32),
                              torch.zeros(0, dtype=torch.float32))
    return out


@pytest.mark.parametrize("case", ["rmat", "one_long_row", "no_entries"])
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("n", [4, 8, 32, 64, 128, 160])
def test_merge_path_spmm_on_skewed_rows(handle, case, dtype, n):
    """The load-balanced kernel (the reference's ALG2 / ALG3 / ALG5, and the default for matrices whose row
    blocks do not fit the row kernels' staging): rows are split over lane groups and tiles, so the result
    matches the oracle within the tolerance, not bit for bit."""
    A = _skewed_cases()[case]
    rp, ci, v = A.numpy()
    v = v.astype(dtype)
    t = torch.float32 if dtype == np.float32 else torch.float64
    X = G.uniform((A.cols, n), -1, 1, dtype=t, seed=74).numpy()
    Y0 = G.uniform((A.rows, n), -1, 1, dtype=t, seed=75).numpy()
    for (alpha, beta), alg, use_buffer in (((1.0, 0.0), api.SPMM_CSR_ALG2, True), ((1.5, -0.5), api.SPMM_ALG_DEFAULT, False),
                                           ((2.0, 1.0), api.SPMM_CSR_ALG3, False)):
        want = oracle.spmm(rp, ci, v, X, alpha, beta, Y0)
        variant = None if (alg == api.SPMM_ALG_DEFAULT and case == "no_entries") else "merge-path"
        got = run_spmm(handle, rp, ci, v, X, alpha, beta, Y0, A.cols, alg=alg, use_buffer=use_buffer, want_variant=variant)
        assert rel_l2(got, want) <= TOL[np.dtype(dtype)], (case, n, alg)
    if n == 32:     # 64-bit row offsets and padded leading dimensions
        want = oracle.spmm(rp, ci, v, X, 1.0, 0.0, Y0)
        got = run_spmm(handle, rp.astype(np.int64), ci, v, X, 1.0, 0.0, Y0, A.cols, ldx=n + 4, ldy=n + 8,
                       alg=api.SPMM_CSR_ALG5, want_variant="merge-path")
        assert rel_l2(got, want) <= TOL[np.dtype(dtype)]


def test_merge_path_spmm_is_reproducible(handle):
    A = G.rmat(14, 16, seed=71)
    rp, ci, v = A.numpy()
    X = G.uniform((A.cols, 32), -1, 1, seed=76).numpy()
    Y0 = np.zeros((A.rows, 32), np.float32)
    a = run_spmm(handle, rp, ci, v, X, 1.0, 0.0, Y0, A.cols, alg=api.SPMM_CSR_ALG2)
    b = run_spmm(handle, rp, ci, v, X, 1.0, 0.0, Y0, A.cols, alg=api.SPMM_CSR_ALG2)
    assert np.array_equal(a, b)      # no atomics: the same bits every run


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("n", [16, 32, 48, 64, 128, 192])
def test_staged_kernel_on_a_stencil(handle, dtype, n, monkeypatch):
    """B through shared memory by TMA (opt-in with ASP_SPMM_STAGE=1, for blocks that touch B in runs): the same
    bits as the oracle and as the kernel that reads B from global memory, with padded leading dimensions and
    beta != 0."""
    monkeypatch.setenv("ASP_SPMM_STAGE", "1")
    t = torch.float32 if dtype == np.float32 else torch.float64
    A = G.stencil_3d_27pt(20, seed=9, dtype=t)        # 8,000 rows: 63 row blocks, the last one partial
    rp, ci, v = A.numpy()
    X = G.uniform((A.cols, n), -1, 1, dtype=t, seed=91).numpy()
    Y0 = G.uniform((A.rows, n), -1, 1, dtype=t, seed=92).numpy()
    want = oracle.spmm(rp, ci, v, X, 1.25, 0.5, Y0)
    # (16-byte fp64 entries: a 256-row block of this stencil does not fit the staging buffer, the tile kernel runs)
    got = run_spmm(handle, rp, ci, v, X, 1.25, 0.5, Y0, A.cols, ldx=n + 8, ldy=n + 4,
                   want_variant="staged" if dtype == np.float32 else None)
    assert np.array_equal(got, want)
    monkeypatch.setenv("ASP_SPMM_STAGE", "0")
    plain = run_spmm(handle, rp, ci, v, X, 1.25, 0.5, Y0, A.cols, ldx=n + 8, ldy=n + 4, want_variant="tile")
    assert np.array_equal(plain, want)


def test_staged_kernel_is_not_chosen_for_scattered_columns(handle, monkeypatch):
    monkeypatch.setenv("ASP_SPMM_STAGE", "1")
    A = G.poisson_random(5000, 5000, mean_len=12, seed=93)      # a chunk of 64 rows of B per entry would be waste
    rp, ci, v = A.numpy()
    X = G.uniform((A.cols, 32), -1, 1, seed=94).numpy()
    Y0 = np.zeros((A.rows, 32), np.float32)
    got = run_spmm(handle, rp, ci, v, X, 1.0, 0.0, Y0, A.cols, want_variant="tile")
    assert np.array_equal(got, oracle.spmm(rp, ci, v, X, 1.0, 0.0, Y0))


def test_leading_dimensions_and_i64_offsets(handle):
    A = G.poisson_random(700, 900, mean_len=6, seed=81)
    rp, ci, v = A.numpy()
    X = G.uniform((A.cols, 12), -1, 1, seed=82).numpy()
    Y0 = G.uniform((A.rows, 12), -1, 1, seed=83).numpy()
    want = oracle.spmm(rp, ci, v, X, 2.0, 0.5, Y0)
    assert np.array_equal(run_spmm(handle, rp, ci, v, X, 2.0, 0.5, Y0, A.cols, ldx=16, ldy=20), want)
    assert np.array_equal(run_spmm(handle, rp, ci, v, X, 2.0, 0.5, Y0, A.cols, ldx=13, ldy=12), want)
    assert np.array_equal(run_spmm(handle, rp.astype(np.int64), ci, v, X, 2.0, 0.5, Y0, A.cols), want)


def test_status_codes(handle):
    import ctypes as C
    lib = api.load()
    A = G.poisson_random(10, 12, mean_len=3, seed=91)
    Am = api.CsrMatrix.from_csr(A)
    B = api.DnMat(torch.zeros(12, 8, device="cuda"))
    Cm = api.DnMat(torch.zeros(10, 8, device="cuda"))
    one = C.c_float(1.0)

    def call(opa=0, opb=0, b=B.d, c=Cm.d, ct=api.R_32F, alg=0):
        return lib.alphasparseSpMM(handle.h, opa, opb, C.byref(one), Am.d, b, C.byref(one), c, ct, alg, None)
    assert call() == 0
    assert call(opa=1) == 10 and call(opb=1) == 6   # transposed A: B must have A's row count
    assert call(b=api.DnMat(torch.zeros(11, 8, device="cuda")).d) == 10
    assert call(c=api.DnMat(torch.zeros(10, 4, device="cuda")).d) == 10
    assert call(ct=api.R_64F) == 6
    d = C.c_void_p()
    t = torch.zeros(12, 8, device="cuda")
    assert lib.alphasparseCreateDnMat(C.byref(d), C.c_int64(12), C.c_int64(8), C.c_int64(12),
                                      C.c_void_p(t.data_ptr()), api.R_32F, api.ORDER_COL) == 0
    assert call(b=d) == 6  # B column-major with C row-major: orders must agree
    dc = C.c_void_p()
    tc = torch.zeros(10, 8, device="cuda")
    assert lib.alphasparseCreateDnMat(C.byref(dc), C.c_int64(10), C.c_int64(8), C.c_int64(10),
                                      C.c_void_p(tc.data_ptr()), api.R_32F, api.ORDER_COL) == 0
    assert call(b=d, c=dc) == 7  # both column-major: needs the external buffer (invalid pointer without)
    lib.alphasparseDestroyDnMat(d)
    lib.alphasparseDestroyDnMat(dc)
    size = C.c_size_t()
    assert lib.alphasparseSpMM_bufferSize(handle.h, 0, 0, C.byref(one), Am.d, B.d, C.byref(one), Cm.d,
                                          api.R_32F, 0, C.byref(size)) == 0 and size.value > 0


@pytest.mark.parametrize("dtype,n", [(np.float32, 8), (np.float32, 20), (np.float64, 32), (np.float32, 128)])
def test_column_major_operands(handle, dtype, n):
    """Column-major B and C (leading dimensions larger than the row counts): same result, bit for bit,
    as the row-major call, padding untouched, B unchanged."""
    A = G.stencil_3d_27pt(12, seed=5)
    rp, ci, v = A.row_ptr.numpy(), A.col_idx.numpy(), A.val.numpy().astype(dtype)
    X = G.uniform((A.cols, n), -1, 1, dtype=torch.from_numpy(np.zeros(1, dtype)).dtype, seed=30).numpy()
    Y0 = G.uniform((A.rows, n), -1, 1, dtype=torch.from_numpy(np.zeros(1, dtype)).dtype, seed=31).numpy()
    Am = api.CsrMatrix(A.rows, A.cols, torch.from_numpy(rp).cuda(), torch.from_numpy(ci).cuda(),
                       torch.from_numpy(v).cuda())
    for alpha, beta in ((1.0, 0.0), (0.5, 2.0)):
        want = oracle.spmm(rp, ci, v, X, alpha, beta, Y0)
        ldb, ldc = A.cols + 3, A.rows + 5
        bbuf = torch.full((n, ldb), 9.0, dtype=torch.from_numpy(X).dtype, device="cuda")
        cbuf = torch.full((n, ldc), 7.0, dtype=torch.from_numpy(X).dtype, device="cuda")
        bbuf[:, :A.cols] = torch.from_numpy(X).cuda().t()
        cbuf[:, :A.rows] = torch.from_numpy(Y0).cuda().t()
        Bd, Cd = api.DnMat(bbuf[:, :A.cols].t()), api.DnMat(cbuf[:, :A.rows].t())
        assert Bd.order == api.ORDER_COL and Cd.order == api.ORDER_COL
        b_before = bbuf.clone()
        buf = torch.empty(api.spmm_buffer_size(handle, Am, Bd, Cd), dtype=torch.uint8, device="cuda")
        api.spmm(handle, Am, Bd, Cd, alpha, beta, buffer=buf)
        torch.cuda.synchronize()
        got = cbuf[:, :A.rows].t().cpu().numpy()
        assert np.array_equal(got, want)
        assert bool((cbuf[:, A.rows:] == 7.0).all()) and torch.equal(bbuf, b_before)


def test_transposed_a(handle):
    """C = alpha * A^T * B + beta * C equals the oracle on the host-transposed matrix."""
    A = G.poisson_random(700, 900, 7.0, seed=41)
    rp, ci, v = A.row_ptr.numpy(), A.col_idx.numpy(), A.val.numpy()
    rows_of = np.repeat(np.arange(A.rows, dtype=np.int32), np.diff(rp).astype(np.int64))
    order = np.argsort(ci, kind="stable")
    t_rp = np.zeros(A.cols + 1, dtype=rp.dtype)
    np.cumsum(np.bincount(ci, minlength=A.cols), out=t_rp[1:])
    X = G.uniform((A.rows, 16), -1, 1, seed=42).numpy()
    Y0 = G.uniform((A.cols, 16), -1, 1, seed=43).numpy()
    want = oracle.spmm(t_rp, rows_of[order], v[order], X, 2.0, -1.0, Y0)
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr.cuda(), A.col_idx.cuda(), A.val.cuda())
    Y = torch.from_numpy(Y0.copy()).cuda()
    import ctypes as C
    al, be = C.c_float(2.0), C.c_float(-1.0)
    B, Cm = api.DnMat(torch.from_numpy(X).cuda()), api.DnMat(Y)
    st = api.load().alphasparseSpMM(handle.h, api.OP_T, api.OP_N, C.byref(al), Am.d, B.d, C.byref(be), Cm.d,
                                    api.R_32F, 0, None)
    torch.cuda.synchronize()
    assert st == 0
    assert np.array_equal(Y.cpu().numpy(), want)


def test_empty_inputs(handle):
    """A matrix without entries scales C by beta; zero columns of B and C and zero rows are no-ops."""
    dev = "cuda"
    rows, cols, n = 300, 200, 16
    Am = api.CsrMatrix(rows, cols, torch.zeros(rows + 1, dtype=torch.int32, device=dev),
                       torch.zeros(0, dtype=torch.int32, device=dev), torch.zeros(0, device=dev))
    X = torch.ones(cols, n, device=dev)
    Y0 = G.uniform((rows, n), -1, 1, seed=6).to(dev)
    Y = Y0.clone()
    api.spmm(handle, Am, api.DnMat(X), api.DnMat(Y), 1.0, -2.0)
    torch.cuda.synchronize()
    assert torch.equal(Y, -2.0 * Y0)
    Y = torch.full((rows, n), float("nan"), device=dev)
    api.spmm(handle, Am, api.DnMat(X), api.DnMat(Y), 1.0, 0.0)
    torch.cuda.synchronize()
    assert torch.equal(Y, torch.zeros(rows, n, device=dev))
    Az = api.CsrMatrix(0, cols, torch.zeros(1, dtype=torch.int32, device=dev),
                       torch.zeros(0, dtype=torch.int32, device=dev), torch.zeros(0, device=dev))
    api.spmm(handle, Az, api.DnMat(X), api.DnMat(torch.zeros(0, n, device=dev)), 1.0, 0.0)
