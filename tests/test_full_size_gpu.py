"""The configurations at their full sizes.  First through properties that need no CPU oracle run:

* checksum: sum(y) = (column sums of A) . x, with the column sums formed by torch in float64
  (an independent scatter-add, not a kernel of the library);
* linearity: A (a x1 + x2) = a A x1 + A x2;
* the two SpMV kernel families agree;
* analytic: the 7-point Laplacian (diagonal 6, off-diagonals -1) times the vector of ones is 0 on
  interior grid points and the number of missing neighbours on the boundary.

Then (second half of the file) against the CPU oracle itself at the same sizes, with the tolerances
of the benchmark specification.

Sizes: Poisson(16) 4,194,304 rows; R-MAT scale 22; 27-point stencil 128^3 with N = 32 (fp32) and
N = 128 (bf16, tcgen05); Laplacian 512^3 with 64-bit row offsets (937,951,232 entries, ~15 GB).
"""
import os

import pytest
import torch

from library_b200 import api
from library_b200 import generators as G

pytestmark = pytest.mark.gpu


def col_sums(A, dtype=torch.float64):
    cs = torch.zeros(A.cols, dtype=dtype, device=A.val.device)
    cs.index_add_(0, A.col_idx.long(), A.val.to(dtype))
    return cs


def rel(a, b):
    return float(abs(a - b) / max(abs(b), 1e-300))


@pytest.mark.parametrize("kind", ["poisson16", "rmat22"])
def test_spmv_full_size_properties(handle, kind, monkeypatch):
    A = (G.poisson_random(4194304, 4194304, 16.0, device="cuda", seed=2) if kind == "poisson16"
         else G.rmat(22, 16, device="cuda", seed=3))
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    x1 = G.uniform((A.cols,), -1, 1, device="cuda", seed=11)
    x2 = G.uniform((A.cols,), -1, 1, device="cuda", seed=12)
    cs = col_sums(A)
    ys = {}
    for variant in ("merge", "binned"):
        monkeypatch.setenv("ASP_SPMV_VARIANT", variant)
        y = torch.zeros(A.rows, device="cuda")
        api.spmv(handle, Am, api.DnVec(x1), api.DnVec(y), 1.0, 0.0)
        torch.cuda.synchronize()
        ys[variant] = y
        # checksum against the independent column sums; the terms have mixed signs, so the error is
        # measured against the sum of magnitudes
        scale = float((cs.abs() * x1.double().abs()).sum())
        assert abs(float(y.double().sum()) - float((cs * x1.double()).sum())) <= 1e-6 * scale
    d = (ys["merge"].double() - ys["binned"].double()).norm() / ys["binned"].double().norm()
    assert float(d) <= 1e-6
    monkeypatch.setenv("ASP_SPMV_VARIANT", "merge")
    y2 = torch.zeros(A.rows, device="cuda")
    y12 = torch.zeros(A.rows, device="cuda")
    api.spmv(handle, Am, api.DnVec(x2), api.DnVec(y2), 1.0, 0.0)
    api.spmv(handle, Am, api.DnVec(0.5 * x1 + x2), api.DnVec(y12), 1.0, 0.0)
    torch.cuda.synchronize()
    lin = (y12.double() - (0.5 * ys["merge"].double() + y2.double())).norm() / y12.double().norm()
    assert float(lin) <= 1e-5
    assert Am.plan(handle)[0]["device_error"] == 0


def test_laplacian_512_cubed_times_ones(handle):
    if torch.cuda.mem_get_info()[0] < 60e9:
        pytest.skip("needs about 40 GB of free device memory")
    n = 512
    A = G.laplacian_3d_7pt(n, dtype=torch.float64, device="cuda", index64=True)
    assert A.nnz == 7 * n ** 3 - 6 * n ** 2 and A.row_ptr.dtype == torch.int64
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    x = torch.ones(A.cols, dtype=torch.float64, device="cuda")
    y = torch.full((A.rows,), 7.0, dtype=torch.float64, device="cuda")
    api.spmv(handle, Am, api.DnVec(x), api.DnVec(y), 1.0, 0.0)
    torch.cuda.synchronize()
    # 6 minus the number of neighbours = faces of the cube the grid point lies on; exact in floating point
    y3 = y.view(n, n, n)
    assert float(y3[1:-1, 1:-1, 1:-1].abs().max()) == 0.0
    idx = torch.arange(n, device="cuda")
    on = ((idx == 0) | (idx == n - 1)).double()
    want = on.view(n, 1, 1) + on.view(1, n, 1) + on.view(1, 1, n)
    assert torch.equal(y3, want)
    assert Am.plan(handle)[0]["device_error"] == 0


def test_more_than_2_to_31_entries(handle):
    """A matrix whose entry count does not fit 32 bits (7-point Laplacian on 680^3: 2,198,249,600 entries,
    fp32 values, 64-bit row offsets): the analytic result again, so every 64-bit offset path is exercised."""
    if torch.cuda.mem_get_info()[0] < 90e9:
        pytest.skip("needs about 60 GB of free device memory")
    n = 680
    A = G.laplacian_3d_7pt(n, dtype=torch.float32, device="cuda", index64=True)
    assert A.nnz == 7 * n ** 3 - 6 * n ** 2 and A.nnz > 2 ** 31
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    x = torch.ones(A.cols, device="cuda")
    y = torch.full((A.rows,), 7.0, device="cuda")
    api.spmv(handle, Am, api.DnVec(x), api.DnVec(y), 1.0, 0.0)
    torch.cuda.synchronize()
    idx = torch.arange(n, device="cuda")
    on = ((idx == 0) | (idx == n - 1)).float()
    want = on.view(n, 1, 1) + on.view(1, n, 1) + on.view(1, 1, n)
    assert torch.equal(y.view(n, n, n), want)
    assert Am.plan(handle)[0]["device_error"] == 0


def test_spmm_stencil_128_cubed_checksum(handle):
    A = G.stencil_3d_27pt(128, device="cuda", seed=4)
    assert A.nnz == 382 ** 3
    cs = col_sums(A)
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    X = G.uniform((A.cols, 32), -1, 1, device="cuda", seed=21)
    Y = torch.zeros(A.rows, 32, device="cuda")
    api.spmm(handle, Am, api.DnMat(X), api.DnMat(Y), 1.0, 0.0)
    torch.cuda.synchronize()
    got = Y.double().sum(dim=0)                       # per column of Y: sum over rows
    want = cs @ X.double()
    scale = cs.abs() @ X.double().abs()
    assert bool(((got - want).abs() <= 1e-6 * scale).all())
    # bf16 operands on the tensor-core kernel, N = 128
    Ab = G.Csr(A.rows, A.cols, A.row_ptr, A.col_idx, A.val.to(torch.bfloat16))
    csb = col_sums(Ab)
    Xb = G.uniform((A.cols, 128), -1, 1, device="cuda", seed=22).to(torch.bfloat16)
    Yb = torch.zeros(A.rows, 128, device="cuda")
    Amb = api.CsrMatrix(A.rows, A.cols, Ab.row_ptr, Ab.col_idx, Ab.val)
    api.spmm(handle, Amb, api.DnMat(Xb), api.DnMat(Yb), 1.0, 0.0)
    torch.cuda.synchronize()
    got = Yb.double().sum(dim=0)
    want = csb @ Xb.double()
    scale = csb.abs() @ Xb.double().abs()
    assert bool(((got - want).abs() <= 1e-6 * scale).all())
    assert Amb.plan(handle)[0]["device_error"] == 0


# ---- the benchmark configurations at their own sizes against the CPU oracle ---------------------
# Tolerances: relative L2 error <= 1e-5 (fp32), <= 1e-12 (fp64), <= 1e-2 (bf16 operands on the tensor
# cores); fp32 / fp64 SpMM is bit-equal to the oracle (same order of fma per element).  The reference's
# own pass criterion, max|a-b| / max|b| (cuda/test/check.cu:145-158,199-212), is printed beside it.

def _np(t):
    return t.cpu().numpy()


def _report(name, got, want, tol):
    from conftest import max_rel, rel_l2
    e, m = rel_l2(got, want), max_rel(got, want)
    print(f"{name}: rel L2 {e:.3e} (tolerance {tol:g}), max|a-b|/max|b| {m:.3e}")
    assert e <= tol, (name, e)


def test_config1_laplacian_256_squared_fp64(handle, monkeypatch):
    import oracle
    A = G.laplacian_2d_5pt(256, dtype=torch.float64, device="cuda")
    assert A.rows == 65536 and A.nnz == 326656
    x = G.uniform((A.cols,), -1, 1, dtype=torch.float64, device="cuda", seed=1)
    want = oracle.spmv(*A.numpy(), _np(x), 1.0, 0.0)
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    for variant in ("auto", "binned", "merge"):
        if variant == "auto":
            monkeypatch.delenv("ASP_SPMV_VARIANT", raising=False)
        else:
            monkeypatch.setenv("ASP_SPMV_VARIANT", variant)
        y = torch.full((A.rows,), 3.0, dtype=torch.float64, device="cuda")
        for _ in range(2):      # the configuration is "one call plus repeats": the repeat must give the same y
            api.spmv(handle, Am, api.DnVec(x), api.DnVec(y), 1.0, 0.0)
        torch.cuda.synchronize()
        _report(f"config 1 ({variant})", _np(y), want, 1e-12)


@pytest.mark.parametrize("kind", ["poisson16", "rmat22"])
def test_config2_and_3_fp32_against_the_oracle(handle, kind, monkeypatch):
    import oracle
    if kind == "poisson16":
        A, alpha, beta, lo = G.poisson_random(4194304, 4194304, 16.0, device="cuda", seed=2), 1.5, 0.5, -1.0
    else:
        A, alpha, beta, lo = G.rmat(22, 16, device="cuda", seed=3), 1.0, 0.0, 0.0
    x = G.uniform((A.cols,), lo, 1, device="cuda", seed=11)
    y0 = G.uniform((A.rows,), -1, 1, device="cuda", seed=12)
    want = oracle.spmv(*A.numpy(), _np(x), alpha, beta, _np(y0))
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    for variant in ("merge", "binned"):
        monkeypatch.setenv("ASP_SPMV_VARIANT", variant)
        y = y0.clone()
        api.spmv(handle, Am, api.DnVec(x), api.DnVec(y), alpha, beta)
        torch.cuda.synchronize()
        _report(f"config {2 if kind == 'poisson16' else 3} ({variant})", _np(y), want, 1e-5)
    assert Am.plan(handle)[0]["device_error"] == 0


@pytest.mark.parametrize("n", [8, 32, 128])
def test_config4_spmm_fp32_bit_equal_to_the_oracle(handle, n):
    import numpy as np
    import oracle
    A = G.stencil_3d_27pt(128, device="cuda", seed=4)
    X = G.uniform((A.cols, n), -1, 1, device="cuda", seed=21)
    want = oracle.spmm(*A.numpy(), _np(X), 1.0, 0.0)
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    Y = torch.full((A.rows, n), 2.0, device="cuda")
    api.spmm(handle, Am, api.DnMat(X), api.DnMat(Y), 1.0, 0.0)
    torch.cuda.synchronize()
    got = _np(Y)
    _report(f"config 4, N={n} ({api.spmm_last_variant(Am)})", got, want, 1e-5)
    assert np.array_equal(got, want)
    assert Am.plan(handle)[0]["device_error"] == 0


def test_config4_tensor_core_n128_against_the_bf16_oracle(handle):
    import numpy as np
    import oracle
    A = G.stencil_3d_27pt(128, device="cuda", seed=4)
    A.val = A.val.to(torch.bfloat16)
    X = G.uniform((A.cols, 128), -1, 1, device="cuda", seed=22).to(torch.bfloat16)

    def bits(t):
        return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)
    want = oracle.spmm(_np(A.row_ptr), _np(A.col_idx), bits(A.val), bits(X), 1.0, 0.0)
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    Y = torch.zeros(A.rows, 128, device="cuda")
    api.spmm(handle, Am, api.DnMat(X), api.DnMat(Y), 1.0, 0.0)
    torch.cuda.synchronize()
    assert api.spmm_last_variant(Am) == "tcgen05"
    _report("config 4, N=128, bf16 operands on tcgen05", _np(Y), want, 1e-2)
    assert Am.plan(handle)[0]["device_error"] == 0


def _check_slabs(handle, A, x, tol, name, slab=1 << 22):
    """y of the whole product against the 64-bit CPU restatement on three row slabs (first, middle,
    last), each with its offsets rebased; the oracle reads the whole x."""
    import oracle
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    y = torch.full((A.rows,), 7.0, dtype=A.val.dtype, device="cuda")
    api.spmv(handle, Am, api.DnVec(x), api.DnVec(y), 1.0, 0.0)
    torch.cuda.synchronize()
    assert Am.plan(handle)[0]["device_error"] == 0
    xh = _np(x)
    mid = (A.rows // 2 // slab) * slab
    for r0 in (0, mid, A.rows - slab):
        r1 = r0 + slab
        k0, k1 = int(A.row_ptr[r0]), int(A.row_ptr[r1])
        rp = _np(A.row_ptr[r0:r1 + 1] - k0)
        want = oracle.spmv(rp, _np(A.col_idx[k0:k1]), _np(A.val[k0:k1]), xh, 1.0, 0.0)
        _report(f"{name}, rows [{r0}, {r1})", _np(y[r0:r1]), want, tol)


def test_config5a_laplacian_512_cubed_slabs_against_the_oracle(handle):
    torch.cuda.empty_cache()
    if torch.cuda.mem_get_info()[0] < 60e9:
        pytest.skip("needs about 40 GB of free device memory")
    A = G.laplacian_3d_7pt(512, dtype=torch.float64, device="cuda", index64=True)
    x = G.uniform((A.cols,), -1, 1, dtype=torch.float64, device="cuda", seed=11)
    _check_slabs(handle, A, x, 1e-12, "config 5a")


def test_config5b_rmat26_slabs_against_the_oracle(handle):
    import gc
    gc.collect()
    torch.cuda.empty_cache()          # blocks the earlier tests freed are still in torch's cache
    if torch.cuda.mem_get_info()[0] < 120e9:
        pytest.skip("building R-MAT scale 26 needs most of a 180 GB device")
    A = G.rmat(26, 32, device="cuda", seed=5, index64=True)
    assert A.row_ptr.dtype == torch.int64 and A.rows == 1 << 26
    x = G.uniform((A.cols,), 0, 1, device="cuda", seed=11)
    _check_slabs(handle, A, x, 1e-5, "config 5b")
