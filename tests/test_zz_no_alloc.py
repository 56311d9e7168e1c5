"""alphasparseSpMVCsrNoAlloc: the SpMV entry point for callers that may not allocate device memory
(no handle, no descriptor, no analysis; scratch lives in a fixed device array inside the library).

Checked through the C ABI against the CPU oracle and against alphasparseSpMV on the same inputs, on
two calls in a row that use different matrices - a larger one first, so the second call finds the
shared scratch array full of the first call's tile rows and carries.  This file sorts last on
purpose: a run that stops at the first failure has then already run every other test.
"""
import os

import numpy as np
import pytest
import torch

from conftest import rel_l2
from library_b200 import api
from library_b200 import generators as G

pytestmark = pytest.mark.gpu
TOL = {torch.float32: 1e-5, torch.float64: 1e-12}


def _reference_call(handle, A, x, y0, alpha, beta):
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    y = y0.clone()
    os.environ["ASP_SPMV_VARIANT"] = "merge"
    try:
        handle.use_torch_stream()
        api.spmv(handle, Am, api.DnVec(x), api.DnVec(y), alpha, beta)
    finally:
        os.environ.pop("ASP_SPMV_VARIANT", None)
    torch.cuda.synchronize()
    return y


def _oracle_call(A, x, y0, alpha, beta):
    import oracle
    return oracle.spmv(A.row_ptr.cpu().numpy(), A.col_idx.cpu().numpy(), A.val.cpu().numpy(), x.cpu().numpy(),
                       alpha, beta, y0.cpu().numpy())


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("off", [torch.int32, torch.int64])
def test_two_calls_in_a_row_match_the_oracle_and_the_descriptor_api(handle, dtype, off):
    big = G.rmat(15, 16, seed=101, dtype=dtype).to("cuda")        # skewed rows, many tiles, long carries
    small = G.poisson_random(3000, 5000, mean_len=9, seed=102, dtype=dtype).to("cuda")
    for A, (alpha, beta) in ((big, (1.0, 0.0)), (small, (1.5, 0.5))):
        A.row_ptr = A.row_ptr.to(off)
        x = G.uniform((A.cols,), -1, 1, dtype=dtype, device="cuda", seed=103)
        y0 = G.uniform((A.rows,), -1, 1, dtype=dtype, device="cuda", seed=104)
        got = y0.clone()
        st = api.spmv_csr_noalloc(A.row_ptr, A.col_idx, A.val, x, got, alpha, beta)
        assert st == 0
        torch.cuda.synchronize()
        assert rel_l2(got.cpu().numpy(), _oracle_call(A, x, y0, alpha, beta)) <= TOL[dtype]
        want = _reference_call(handle, A, x, y0, alpha, beta)
        assert rel_l2(got.cpu().numpy(), want.cpu().numpy()) <= TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_one_row_across_many_tiles_between_empty_rows_and_unaligned_arrays(handle, dtype):
    """A 50,000-entry row (25 tiles of the merge list) between runs of empty rows, then short rows; once
    with 16-byte aligned arrays and once with the column and value arrays starting one element in,
    which takes the kernel's element-wise load path."""
    rng = np.random.default_rng(7)
    lens = np.concatenate([np.zeros(300, np.int64), [50000], np.zeros(2500, np.int64),
                           rng.integers(0, 12, size=4000)])
    cols_n = 60000
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ci = np.concatenate([np.sort(rng.choice(cols_n, size=int(l), replace=False)) for l in lens if l]).astype(np.int32)
    v = rng.normal(size=ci.size)
    npdt = np.float32 if dtype == torch.float32 else np.float64
    x = torch.from_numpy(rng.uniform(-1, 1, cols_n).astype(npdt)).cuda()
    y0 = torch.from_numpy(rng.uniform(-1, 1, lens.size).astype(npdt)).cuda()
    import oracle
    want = oracle.spmv(rp, ci, v.astype(npdt), x.cpu().numpy(), 1.5, 0.5, y0.cpu().numpy())
    for shift in (0, 1):
        cbuf = torch.zeros(ci.size + 4, dtype=torch.int32, device="cuda")
        vbuf = torch.zeros(ci.size + 4, dtype=dtype, device="cuda")
        col, val = cbuf[shift:shift + ci.size], vbuf[shift:shift + ci.size]
        col.copy_(torch.from_numpy(ci))
        val.copy_(torch.from_numpy(v.astype(npdt)))
        assert (col.data_ptr() % 16 == 0) == (shift == 0)
        got = y0.clone()
        assert api.spmv_csr_noalloc(torch.from_numpy(rp).cuda(), col, val, x, got, 1.5, 0.5) == 0
        torch.cuda.synchronize()
        assert rel_l2(got.cpu().numpy(), want) <= TOL[dtype], shift


def test_rejects_sizes_beyond_the_fixed_scratch_and_bad_arguments(handle):
    import ctypes as C
    lib = api.load()
    one = C.c_float(1.0)
    p = C.c_void_p(0x1000)  # never dereferenced: every case below is refused before any launch

    def call(rows=10, cols=10, nnz=10, rp=p, rt=api.INDEX_I32, ci=p, v=p, dt=api.R_32F, a=C.byref(one),
             x=p, b=C.byref(one), y=p):
        return lib.alphasparseSpMVCsrNoAlloc(None, C.c_int64(rows), C.c_int64(cols), C.c_int64(nnz), rp, rt,
                                             ci, v, dt, a, x, b, y)
    assert call(rows=1 << 20, nnz=api.NOALLOC_MAX_ITEMS) == 10     # INVALID_SIZE: over the limit
    assert call(rows=-1) == 10
    assert call(rp=None) == 7 and call(a=None) == 7 and call(y=None) == 7
    assert call(dt=api.R_16BF) == 6 and call(rt=api.INDEX_I32 - 1) == 6
    assert call(rows=0, nnz=0) == 0                                # nothing to do


def test_no_device_allocation_happens(handle):
    """Device memory in use does not move across calls (the library's own array is static)."""
    A = G.poisson_random(20000, mean_len=12, seed=105).to("cuda")
    x = G.uniform((A.cols,), -1, 1, device="cuda", seed=106)
    y = torch.zeros(A.rows, device="cuda")
    assert api.spmv_csr_noalloc(A.row_ptr, A.col_idx, A.val, x, y) == 0   # includes the one-time symbol look-up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        assert api.spmv_csr_noalloc(A.row_ptr, A.col_idx, A.val, x, y) == 0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0
