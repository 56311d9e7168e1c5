"""CUDA SpMV through the C ABI against the CPU oracle (the restated arithmetic of the
reference's hygon CSR mv) and against the golden vectors made by the reference's own code.

Tolerances (relative L2): fp32 1e-5, fp64 1e-12.  Preprocessing output is compared bit for bit
with the numpy twin in tests/preprocess_twin.py.
"""
import os

import numpy as np
import pytest
import torch

import oracle
import preprocess_twin as twin
from conftest import load_golden, rel_l2
from library_b200 import api
from library_b200 import generators as G

pytestmark = pytest.mark.gpu
TOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float64): 1e-12}
MV_CASES = sorted(k for k, c in load_golden().items() if c["kind"] == "mv")
VARIANTS = ["binned", "merge"]


def run_spmv(handle, rp, ci, v, x, alpha, beta, y0, cols, variant=None, alg=api.SPMV_ALG_DEFAULT,
             use_buffer=False):
    dev = "cuda"
    A = api.CsrMatrix(len(rp) - 1, cols, torch.from_numpy(rp).to(dev), torch.from_numpy(ci).to(dev),
                      torch.from_numpy(v).to(dev))
    xd = api.DnVec(torch.from_numpy(x).to(dev))
    yt = torch.from_numpy(np.array(y0, copy=True)).to(dev)
    yd = api.DnVec(yt)
    buf = None
    if use_buffer:
        buf = torch.empty(api.spmv_buffer_size(handle, A, xd, yd, alpha, beta, alg), dtype=torch.uint8, device=dev)
    old = os.environ.pop("ASP_SPMV_VARIANT", None)
    if variant:
        os.environ["ASP_SPMV_VARIANT"] = variant
    try:
        handle.use_torch_stream()
        api.spmv(handle, A, xd, yd, alpha, beta, alg=alg, buffer=buf)
        torch.cuda.synchronize()
    finally:
        os.environ.pop("ASP_SPMV_VARIANT", None)
        if old is not None:
            os.environ["ASP_SPMV_VARIANT"] = old
    return yt.cpu().numpy(), A


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("name", MV_CASES)
def test_golden(handle, golden, name, variant):
    c = golden[name]
    y, A = run_spmv(handle, c["rp"], c["ci"], c["v"], c["x"], c["alpha"], c["beta"], c["y0"], c["cols"], variant)
    assert A.last_variant() == variant
    assert rel_l2(y, c["y"]) <= TOL[c["v"].dtype]


def _mk(kind, dtype):
    t = torch.float32 if dtype == np.float32 else torch.float64
    if kind == "lap2d":
        return G.laplacian_2d_5pt(96, dtype=t)
    if kind == "poisson":
        return G.poisson_random(50000, mean_len=16, seed=21, dtype=t)
    if kind == "poisson_wide":
        return G.poisson_random(3000, 100000, mean_len=300, seed=22, dtype=t)
    if kind == "rmat":
        return G.rmat(15, 16, seed=23, dtype=t)
    if kind == "s27":
        return G.stencil_3d_27pt(24, seed=24, dtype=t)
    if kind == "lap3d_i64":
        return G.laplacian_3d_7pt(40, dtype=t, index64=True)
    if kind == "tiny":
        return G.poisson_random(3, 5, mean_len=2, seed=25, dtype=t)
    raise KeyError(kind)


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("kind", ["lap2d", "poisson", "poisson_wide", "rmat", "s27", "lap3d_i64", "tiny"])
def test_against_oracle(handle, kind, dtype, variant):
    A = _mk(kind, dtype)
    rp, ci, v = A.numpy()
    t = torch.float32 if dtype == np.float32 else torch.float64
    x = G.uniform((A.cols,), -1, 1, dtype=t, seed=31).numpy()
    y0 = G.uniform((A.rows,), -1, 1, dtype=t, seed=32).numpy()
    for alpha, beta in ((1.0, 0.0), (1.5, 0.5)):
        want = oracle.spmv(rp, ci, v, x, alpha, beta, y0)
        got, _ = run_spmv(handle, rp, ci, v, x, alpha, beta, y0, A.cols, variant, use_buffer=(beta != 0))
        assert rel_l2(got, want) <= TOL[np.dtype(dtype)], (kind, alpha, beta)


def _skewed(dtype):
    """Empty rows, a few rows far beyond the CTA-per-row threshold, unaligned row starts."""
    rng = np.random.default_rng(5)
    rows, cols = 5000, 40000
    lens = rng.integers(0, 12, size=rows)
    lens[rng.random(rows) < 0.4] = 0
    lens[7] = 30000
    lens[8] = 1
    lens[4000] = 5000
    lens[4999] = 4097
    lens[123] = 65
    lens[124] = 64
    rp = np.zeros(rows + 1, dtype=np.int32)
    rp[1:] = np.cumsum(lens)
    ci = np.concatenate([np.sort(rng.choice(cols, size=l, replace=False)) for l in lens]).astype(np.int32)
    v = rng.standard_normal(rp[-1]).astype(dtype)
    return rp, ci, v, cols


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_skewed_rows(handle, dtype, variant):
    rp, ci, v, cols = _skewed(dtype)
    rng = np.random.default_rng(6)
    x = rng.uniform(-1, 1, cols).astype(dtype)
    y0 = rng.uniform(-1, 1, len(rp) - 1).astype(dtype)
    for alpha, beta in ((1.0, 0.0), (-2.0, 0.25)):
        want = oracle.spmv(rp, ci, v, x, alpha, beta, y0)
        got, _ = run_spmv(handle, rp, ci, v, x, alpha, beta, y0, cols, variant)
        assert rel_l2(got, want) <= TOL[np.dtype(dtype)]
        # rows with no entries: exactly beta*y0
        empty = np.diff(rp) == 0
        assert np.array_equal(got[empty], (np.array(beta, dtype) * y0[empty]) if beta else np.zeros(empty.sum(), dtype))


@pytest.mark.parametrize("variant", VARIANTS)
def test_one_row_spanning_many_tiles(handle, variant):
    """A single row of 50,000 entries between empty rows: the merge-path carry chain."""
    rows, cols, L = 9, 60000, 50000
    rp = np.array([0, 0, 0, L, L, L, L + 3, L + 3, L + 3, L + 3], dtype=np.int32)
    rng = np.random.default_rng(9)
    ci = np.concatenate([np.sort(rng.choice(cols, L, replace=False)), [1, 5, 9]]).astype(np.int32)
    v = rng.standard_normal(L + 3)
    x = rng.uniform(-1, 1, cols)
    y0 = rng.uniform(-1, 1, rows)
    want = oracle.spmv(rp, ci, v, x, 0.5, 2.0, y0)
    got, _ = run_spmv(handle, rp, ci, v, x, 0.5, 2.0, y0, cols, variant)
    assert rel_l2(got, want) <= 1e-12


def test_unaligned_arrays_use_scalar_loads(handle):
    """Value / column arrays that do not start on a 16-byte boundary."""
    A = G.poisson_random(4000, mean_len=9, seed=41)
    rp, ci, v = A.numpy()
    x = G.uniform((A.cols,), -1, 1, seed=42).numpy()
    want = oracle.spmv(rp, ci, v, x, 1.0, 0.0)
    dev = "cuda"
    cbuf = torch.zeros(len(ci) + 1, dtype=torch.int32, device=dev)
    vbuf = torch.zeros(len(v) + 1, dtype=torch.float32, device=dev)
    cbuf[1:] = torch.from_numpy(ci).to(dev)
    vbuf[1:] = torch.from_numpy(v).to(dev)
    for variant in VARIANTS:
        Am = api.CsrMatrix(A.rows, A.cols, torch.from_numpy(rp).to(dev), cbuf[1:], vbuf[1:])
        xd = api.DnVec(torch.from_numpy(x).to(dev))
        yt = torch.zeros(A.rows, dtype=torch.float32, device=dev)
        os.environ["ASP_SPMV_VARIANT"] = variant
        try:
            api.spmv(handle, Am, xd, api.DnVec(yt))
        finally:
            os.environ.pop("ASP_SPMV_VARIANT")
        torch.cuda.synchronize()
        assert rel_l2(yt.cpu().numpy(), want) <= 1e-5


def test_beta_zero_does_not_read_y(handle):
    A = G.laplacian_2d_5pt(20, dtype=torch.float32)
    rp, ci, v = A.numpy()
    x = np.ones(A.cols, np.float32)
    y0 = np.full(A.rows, np.nan, np.float32)
    for variant in VARIANTS:
        got, _ = run_spmv(handle, rp, ci, v, x, 1.0, 0.0, y0, A.cols, variant)
        assert np.isfinite(got).all()


@pytest.mark.parametrize("kind", ["lap2d", "poisson", "rmat", "lap3d_i64"])
def test_preprocessing_bit_exact(handle, kind):
    A = _mk(kind, np.float32)
    Am = api.CsrMatrix.from_csr(A)
    Am.analyse(handle)
    stats, bins, tiles = Am.plan(handle)
    rp, ci, _ = A.numpy()
    want_stats, want_bins, want_tiles = twin.plan(rp, 4, ci)
    assert stats == want_stats
    assert np.array_equal(bins, want_bins)
    assert np.array_equal(tiles, want_tiles)


def test_preprocessing_skewed_bit_exact(handle):
    rp, ci, v, cols = _skewed(np.float64)
    dev = "cuda"
    Am = api.CsrMatrix(len(rp) - 1, cols, torch.from_numpy(rp).to(dev), torch.from_numpy(ci).to(dev),
                       torch.from_numpy(v).to(dev))
    Am.analyse(handle)
    stats, bins, tiles = Am.plan(handle)
    want_stats, want_bins, want_tiles = twin.plan(rp, 8, ci)
    assert stats == want_stats and np.array_equal(bins, want_bins) and np.array_equal(tiles, want_tiles)
    assert stats["num_long"] == 3 and stats["num_medium"] == 1 and stats["variant"] == 0


def test_results_reproducible_run_to_run(handle):
    A = _mk("rmat", np.float32)
    rp, ci, v = A.numpy()
    x = G.uniform((A.cols,), 0, 1, seed=51).numpy()
    for variant in VARIANTS:
        a, _ = run_spmv(handle, rp, ci, v, x, 1.0, 0.0, np.zeros(A.rows, np.float32), A.cols, variant)
        b, _ = run_spmv(handle, rp, ci, v, x, 1.0, 0.0, np.zeros(A.rows, np.float32), A.cols, variant)
        assert np.array_equal(a, b)


def test_alg_enum_selects_variant(handle):
    A = _mk("poisson", np.float32)
    rp, ci, v = A.numpy()
    x = G.uniform((A.cols,), -1, 1, seed=52).numpy()
    y0 = np.zeros(A.rows, np.float32)
    _, Am = run_spmv(handle, rp, ci, v, x, 1.0, 0.0, y0, A.cols, alg=api.SPMV_ALG_MERGE)
    assert Am.last_variant() == "merge"
    _, Am = run_spmv(handle, rp, ci, v, x, 1.0, 0.0, y0, A.cols, alg=api.SPMV_ALG_VECTOR)
    assert Am.last_variant() == "binned"
    # the reference's own CSR tests pass ALG_COO (cuda/test/level2/spmv_csr_r_f32_test.cu:238): still computed
    got, _ = run_spmv(handle, rp, ci, v, x, 1.0, 0.0, y0, A.cols, alg=api.SPMV_ALG_COO)
    assert rel_l2(got, oracle.spmv(rp, ci, v, x, 1.0, 0.0)) <= 1e-5


def test_status_codes(handle):
    import ctypes as C
    lib = api.load()
    A = _mk("tiny", np.float32)
    Am = api.CsrMatrix.from_csr(A)
    x = api.DnVec(torch.zeros(A.cols, device="cuda"))
    y = api.DnVec(torch.zeros(A.rows, device="cuda"))
    one = C.c_float(1.0)

    def call(op=0, a=C.byref(one), mat=Am.d, vx=x.d, b=C.byref(one), vy=y.d, ct=api.R_32F):
        return lib.alphasparseSpMV(handle.h, op, a, mat, vx, b, vy, ct, 0, None)
    assert call() == 0
    assert call(op=api.OP_T) == (0 if A.rows == A.cols else 10)   # transposed: x and y swap sizes
    assert call(a=None) == 7
    assert call(mat=None) == 7
    assert call(ct=api.R_64F) == 6
    bad = api.DnVec(torch.zeros(A.cols + 1, device="cuda"))
    assert call(vx=bad.d) == 10
    xd = api.DnVec(torch.zeros(A.cols, device="cuda", dtype=torch.float64))
    assert call(vx=xd.d) == 6


def test_invalid_structure_is_rejected_not_run(handle):
    """Column index out of range and decreasing offsets come back as INVALID_VALUE from analysis."""
    rp = torch.tensor([0, 2, 4], dtype=torch.int32, device="cuda")
    ci = torch.tensor([0, 1, 0, 7], dtype=torch.int32, device="cuda")
    v = torch.ones(4, device="cuda")
    Am = api.CsrMatrix(2, 3, rp, ci, v)
    with pytest.raises(api.AlphaSparseError) as e:
        Am.analyse(handle)
    assert e.value.status == 3
    rp2 = torch.tensor([0, 3, 2, 4], dtype=torch.int32, device="cuda")
    Am2 = api.CsrMatrix(3, 8, rp2, ci, v)
    with pytest.raises(api.AlphaSparseError) as e:
        Am2.analyse(handle)
    assert e.value.status == 3


def test_partition_and_rebase_match_oracle(handle):
    A = _mk("rmat", np.float32)
    rp, _, _ = A.numpy()
    for dt in (torch.int32, torch.int64):
        rpd = torch.from_numpy(rp).to("cuda").to(dt)
        for parts in (1, 2, 4, 8):
            got = api.partition_rows_by_nnz(handle, rpd, parts)
            assert np.array_equal(got, oracle.partition_rows_by_nnz(rp, parts))
        b = api.partition_rows_by_nnz(handle, rpd, 4)
        loc = api.rebase_row_offsets(handle, rpd, int(b[1]), int(b[2]), torch.int32)
        torch.cuda.synchronize()
        assert np.array_equal(loc.cpu().numpy(), rp[b[1]:b[2] + 1] - rp[b[1]])


def test_coo2csr_matches_row_offsets(handle):
    """alphasparseXcoo2csr: offsets rebuilt from the expanded (ascending) row indices of a CSR matrix,
    empty rows at both ends included."""
    A = _mk("rmat", np.float32)
    rp, _, _ = A.numpy()
    rp = np.concatenate([[0, 0], rp, [rp[-1], rp[-1]]]).astype(np.int32)    # leading / trailing empty rows
    rows = len(rp) - 1
    coo = np.repeat(np.arange(rows, dtype=np.int32), np.diff(rp))
    d = torch.from_numpy(coo).to("cuda")
    for dt in (torch.int32, torch.int64):
        got = api.coo2csr(d, rows, dt)
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy(), rp)
    assert np.array_equal(api.coo2csr(d[:0], 5).cpu().numpy(), np.zeros(6, np.int32))


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("kind", ["rect_poisson", "rmat", "i64"])
def test_transposed(handle, dtype, kind):
    """y = alpha * A^T * x + beta * y through the transposed copy the plan builds on the device: the same
    numbers as the library's own product with an explicitly transposed matrix (scipy-free CSR transpose on
    the host), and as the oracle on that matrix."""
    tdt = torch.float32 if dtype == np.float32 else torch.float64
    if kind == "rect_poisson":
        A = G.poisson_random(3000, 5000, 9.0, dtype=tdt, seed=21)
    elif kind == "rmat":
        A = G.rmat(12, 8, dtype=tdt, seed=22)
    else:
        A = G.laplacian_3d_7pt(20, dtype=tdt, index64=True)
    rp, ci, v = A.row_ptr.numpy(), A.col_idx.numpy(), A.val.numpy()
    # host transpose: stable sort of the entries by column keeps rows ascending inside a column
    rows_of = np.repeat(np.arange(A.rows, dtype=np.int32), np.diff(rp).astype(np.int64))
    order = np.argsort(ci, kind="stable")
    t_ci, t_v = rows_of[order], v[order]
    t_rp = np.zeros(A.cols + 1, dtype=rp.dtype)
    np.cumsum(np.bincount(ci, minlength=A.cols), out=t_rp[1:])
    x = G.uniform((A.rows,), -1, 1, dtype=tdt, seed=23).numpy()
    y0 = G.uniform((A.cols,), -1, 1, dtype=tdt, seed=24).numpy()
    want = oracle.spmv(t_rp, t_ci, t_v, x, 1.5, 0.5, y0)
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr.cuda(), A.col_idx.cuda(), A.val.cuda())
    y = torch.from_numpy(y0.copy()).cuda()
    api.spmv(handle, Am, api.DnVec(torch.from_numpy(x).cuda()), api.DnVec(y), 1.5, 0.5, op=api.OP_T)
    torch.cuda.synchronize()
    assert rel_l2(y.cpu().numpy(), want) <= TOL[np.dtype(dtype)]
    # the plain product still works on the same descriptor, and A's arrays are untouched
    x2 = G.uniform((A.cols,), -1, 1, dtype=tdt, seed=25).numpy()
    y2 = torch.zeros(A.rows, dtype=tdt, device="cuda")
    api.spmv(handle, Am, api.DnVec(torch.from_numpy(x2).cuda()), api.DnVec(y2), 1.0, 0.0)
    torch.cuda.synchronize()
    assert rel_l2(y2.cpu().numpy(), oracle.spmv(rp, ci, v, x2, 1.0, 0.0)) <= TOL[np.dtype(dtype)]
    assert np.array_equal(Am.col_idx.cpu().numpy(), ci) and np.array_equal(Am.val.cpu().numpy(), v)


@pytest.mark.parametrize("variant", VARIANTS)
def test_empty_inputs(handle, variant, monkeypatch):
    """No entries at all (y = beta * y), no rows, one row: nothing to launch or a single tiny launch, never
    an error."""
    monkeypatch.setenv("ASP_SPMV_VARIANT", variant)
    dev = "cuda"
    # rows but no entries
    rows, cols = 1000, 700
    Am = api.CsrMatrix(rows, cols, torch.zeros(rows + 1, dtype=torch.int32, device=dev),
                       torch.zeros(0, dtype=torch.int32, device=dev), torch.zeros(0, device=dev))
    x = torch.ones(cols, device=dev)
    y0 = G.uniform((rows,), -1, 1, seed=5).to(dev)
    y = y0.clone()
    api.spmv(handle, Am, api.DnVec(x), api.DnVec(y), 2.0, 0.5)
    torch.cuda.synchronize()
    assert torch.equal(y, 0.5 * y0)
    y = torch.full((rows,), float("nan"), device=dev)
    api.spmv(handle, Am, api.DnVec(x), api.DnVec(y), 2.0, 0.0)
    torch.cuda.synchronize()
    assert torch.equal(y, torch.zeros(rows, device=dev))
    # no rows
    Az = api.CsrMatrix(0, cols, torch.zeros(1, dtype=torch.int32, device=dev),
                       torch.zeros(0, dtype=torch.int32, device=dev), torch.zeros(0, device=dev))
    api.spmv(handle, Az, api.DnVec(x), api.DnVec(torch.zeros(0, device=dev)), 1.0, 0.0)
    # one row, one entry
    A1 = api.CsrMatrix(1, cols, torch.tensor([0, 1], dtype=torch.int32, device=dev),
                       torch.tensor([699], dtype=torch.int32, device=dev), torch.tensor([3.0], device=dev))
    y1 = torch.tensor([10.0], device=dev)
    api.spmv(handle, A1, api.DnVec(x), api.DnVec(y1), 2.0, 1.0)
    torch.cuda.synchronize()
    assert float(y1[0]) == 16.0


def test_transposed_without_entries(handle):
    rows, cols = 40, 70
    Am = api.CsrMatrix(rows, cols, torch.zeros(rows + 1, dtype=torch.int32, device="cuda"),
                       torch.zeros(0, dtype=torch.int32, device="cuda"), torch.zeros(0, device="cuda"))
    y0 = G.uniform((cols,), -1, 1, seed=4).cuda()
    y = y0.clone()
    api.spmv(handle, Am, api.DnVec(torch.ones(rows, device="cuda")), api.DnVec(y), 1.0, 3.0, op=api.OP_T)
    torch.cuda.synchronize()
    assert torch.equal(y, 3.0 * y0)


def test_a_wait_that_runs_out_is_reported(handle, monkeypatch):
    """Failure detection without a fault: with ASP_TEST_DROP_COPY the tile kernel announces its bulk copies to
    the mbarrier but never issues them, so every CTA's bounded wait runs out after ASP_WAIT_POLLS polls; the
    CTAs raise the plan's flag and return, nothing faults, the context stays usable and the flag shows in the
    plan statistics.  A fresh analysis gives a clean plan again."""
    A = G.poisson_random(20000, 20000, mean_len=16, seed=301).to("cuda")
    x = G.uniform((A.cols,), -1, 1, device="cuda", seed=302)
    y = torch.zeros(A.rows, device="cuda")
    handle.use_torch_stream()
    monkeypatch.setenv("ASP_SPMV_VARIANT", "merge")
    monkeypatch.setenv("ASP_TEST_DROP_COPY", "1")
    monkeypatch.setenv("ASP_WAIT_POLLS", "2")
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    Am.analyse(handle)                                 # the plan takes the wait settings from the environment
    monkeypatch.delenv("ASP_TEST_DROP_COPY")
    monkeypatch.delenv("ASP_WAIT_POLLS")
    api.spmv(handle, Am, api.DnVec(x), api.DnVec(y), 1.0, 0.0)      # launches; every CTA gives up and leaves
    torch.cuda.synchronize()                                         # no error from the runtime: nothing faulted
    assert Am.plan(handle)[0]["device_error"] == 1
    Am.analyse(handle)                                               # new plan, normal waits
    api.spmv(handle, Am, api.DnVec(x), api.DnVec(y), 1.0, 0.0)
    torch.cuda.synchronize()
    assert Am.plan(handle)[0]["device_error"] == 0
    import oracle
    want = oracle.spmv(*A.numpy(), x.cpu().numpy(), 1.0, 0.0)
    assert rel_l2(y.cpu().numpy(), want) <= 1e-5
