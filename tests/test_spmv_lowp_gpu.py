"""SpMV with 16-bit operands and fp32 arithmetic (the reference's half -> float and
bf16 -> bf16 instances, cuda/kernel/level2/alphasparse_spmv.cu:288-300), through the C ABI.

The check is plain arithmetic on the same rounded inputs in float64: products of two 16-bit
numbers are exact in fp32, so an fp32-accumulated result with fp32 y must agree to 1e-5
(relative L2); a bf16 y is rounded once more (2^-9 per element), bound 1e-2.
"""
import numpy as np
import pytest
import torch

from conftest import rel_l2
from library_b200 import api
from library_b200 import generators as G

pytestmark = pytest.mark.gpu


def reference(A, val, x, y0, alpha, beta):
    """alpha * A * x + beta * y0 in float64, row by row."""
    rp = A.row_ptr.numpy().astype(np.int64)
    ci = A.col_idx.numpy()
    prod = val.double().numpy() * x.double().numpy()[ci]
    out = np.add.reduceat(np.concatenate([prod, [0.0]]), np.minimum(rp[:-1], len(prod)))
    out[rp[1:] == rp[:-1]] = 0.0
    return alpha * out + beta * y0.double().numpy()


CASES = {
    "stencil27": lambda: G.stencil_3d_27pt(24, seed=3),
    "poisson": lambda: G.poisson_random(20000, 30000, 12.0, seed=5),
    "rmat": lambda: G.rmat(14, 16, seed=6),
    "lap3d_i64": lambda: G.laplacian_3d_7pt(30, dtype=torch.float32, index64=True),
}


@pytest.mark.parametrize("name", sorted(CASES))
@pytest.mark.parametrize("kind", ["f16_f32", "bf16_bf16"])
@pytest.mark.parametrize("variant", ["binned", "merge"])
def test_lowp_spmv(handle, name, kind, variant, monkeypatch):
    monkeypatch.setenv("ASP_SPMV_VARIANT", variant)
    A = CASES[name]()
    ta, ty, tol = (torch.float16, torch.float32, 1e-5) if kind == "f16_f32" else (torch.bfloat16, torch.bfloat16, 1e-2)
    val = A.val.to(torch.float32).clamp(-8, 8).to(ta)
    x = G.uniform((A.cols,), -1, 1, seed=11).to(ta)
    y0 = G.uniform((A.rows,), -1, 1, seed=12).to(ty)
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr.cuda(), A.col_idx.cuda(), val.cuda())
    for alpha, beta in ((1.0, 0.0), (1.5, -0.5)):
        y = y0.clone().cuda()
        api.spmv(handle, Am, api.DnVec(x.cuda()), api.DnVec(y), alpha, beta)
        torch.cuda.synchronize()
        want = reference(A, val, x, y0, alpha, beta)
        assert rel_l2(y.float().cpu().numpy(), want) <= tol
        assert Am.last_variant() == variant
        assert Am.plan(handle)[0]["device_error"] == 0


def test_lowp_unaligned_and_empty_rows(handle):
    """Arrays that start 2 / 4 bytes past a 16-byte boundary take the entry-by-entry loads; empty
    rows give beta * y."""
    A = G.poisson_random(5000, 7000, 3.0, seed=9)          # Poisson(3): about 5 % empty rows
    val = A.val.to(torch.float16)
    x = G.uniform((A.cols,), -1, 1, seed=1).to(torch.float16)
    y0 = G.uniform((A.rows,), -1, 1, seed=2)
    vbuf = torch.zeros(A.nnz + 8, dtype=torch.float16, device="cuda")
    cbuf = torch.zeros(A.nnz + 8, dtype=torch.int32, device="cuda")
    vbuf[1:1 + A.nnz] = val.cuda()
    cbuf[1:1 + A.nnz] = A.col_idx.cuda()
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr.cuda(), cbuf[1:1 + A.nnz], vbuf[1:1 + A.nnz])
    y = y0.clone().cuda()
    api.spmv(handle, Am, api.DnVec(x.cuda()), api.DnVec(y), 2.0, 1.0)
    torch.cuda.synchronize()
    want = reference(A, val, x, y0, 2.0, 1.0)
    assert rel_l2(y.cpu().numpy(), want) <= 1e-5
    empty = (A.row_ptr[1:] == A.row_ptr[:-1]).numpy()
    assert empty.any() and np.array_equal(y.cpu().numpy()[empty], y0.numpy()[empty])


def test_lowp_type_combinations(handle):
    """Only the reference's two instances exist: half/half/float and bf16/bf16/bf16."""
    A = G.laplacian_2d_5pt(16, dtype=torch.float32)
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr.cuda(), A.col_idx.cuda(), A.val.to(torch.float16).cuda())
    x = torch.ones(A.cols, dtype=torch.float16, device="cuda")
    with pytest.raises(api.AlphaSparseError):
        api.spmv(handle, Am, api.DnVec(x), api.DnVec(torch.zeros(A.rows, dtype=torch.float16, device="cuda")))
    with pytest.raises(api.AlphaSparseError):
        api.spmv(handle, Am, api.DnVec(x.float()), api.DnVec(torch.zeros(A.rows, device="cuda")))


def test_lowp_without_entries(handle):
    rows, cols = 500, 300
    Am = api.CsrMatrix(rows, cols, torch.zeros(rows + 1, dtype=torch.int32, device="cuda"),
                       torch.zeros(0, dtype=torch.int32, device="cuda"),
                       torch.zeros(0, dtype=torch.float16, device="cuda"))
    y0 = G.uniform((rows,), -1, 1, seed=4).cuda()
    y = y0.clone()
    api.spmv(handle, Am, api.DnVec(torch.ones(cols, dtype=torch.float16, device="cuda")), api.DnVec(y), 1.0, -1.0)
    torch.cuda.synchronize()
    assert torch.equal(y, -y0)
