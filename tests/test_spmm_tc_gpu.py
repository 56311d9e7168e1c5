"""tcgen05 SpMM (bf16 A and B, fp32 accumulation and C) through the C ABI against the CPU oracle
of the same arithmetic.  Tolerance: relative L2 1e-2 (the stated bound for bf16 operands); the
products are exact in fp32 and only the summation order differs, so the observed error is
orders of magnitude smaller and is also checked against 1e-5."""
import os

import numpy as np
import pytest
import torch

import oracle
from conftest import rel_l2
from library_b200 import api
from library_b200 import generators as G

pytestmark = pytest.mark.gpu


def bits(t):
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


# The three kernels of the path: A in tensor memory (the default; N = 256 as two passes of 128 columns), A tiles
# in shared memory (on request), one CTA per row block (on request, or for blocks with many chunks).
KERNELS = {"tcgen05": {}, "tcgen05-smem": {"ASP_TC_A_TMEM": "0"}, "tcgen05-simple": {"ASP_TC_PERSISTENT": "0"}}


def run_tc(handle, A, X, Y0, alpha, beta, ldx=None, ldy=None, kernel=None):
    env = KERNELS.get(kernel, {})
    old = {k: os.environ.get(k) for k in env}
    os.environ.update(env)
    try:
        return _run_tc(handle, A, X, Y0, alpha, beta, ldx, ldy, kernel)
    finally:
        for k, v in old.items():
            if v is None:
                del os.environ[k]
            else:
                os.environ[k] = v


def _run_tc(handle, A, X, Y0, alpha, beta, ldx, ldy, kernel):
    dev = "cuda"
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr.to(dev), A.col_idx.to(dev), A.val.to(dev))
    n = X.shape[1]
    Xd = X.to(dev)
    Yd = Y0.clone().to(dev)
    if ldx:
        buf = torch.zeros(X.shape[0], ldx, dtype=X.dtype, device=dev)
        buf[:, :n] = Xd
        Xd = buf[:, :n]
    if ldy:
        buf2 = torch.full((Y0.shape[0], ldy), 3.0, dtype=Y0.dtype, device=dev)
        buf2[:, :n] = Yd
        Yd = buf2[:, :n]
    handle.use_torch_stream()
    B, C = api.DnMat(Xd), api.DnMat(Yd)
    api.spmm_preprocess(handle, Am, B, C)
    api.spmm(handle, Am, B, C, alpha, beta)
    torch.cuda.synchronize()
    stats, _, _ = Am.plan(handle)
    assert stats["device_error"] == 0
    if kernel:
        assert api.spmm_last_variant(Am) == kernel
    if ldy:
        assert bool((buf2[:, n:] == 3.0).all())
    return Yd.cpu().numpy()


@pytest.mark.parametrize("kernel", list(KERNELS))
@pytest.mark.parametrize("n", [64, 128, 192, 256])
@pytest.mark.parametrize("grid", [16, 10])
def test_stencil_bf16(handle, n, grid, kernel):
    A = G.stencil_3d_27pt(grid, seed=4)          # grid 10: 1000 rows, last row block partial
    A.val = A.val.to(torch.bfloat16)
    X = G.uniform((A.cols, n), -1, 1, dtype=torch.bfloat16, seed=70 + n)
    Y0 = G.uniform((A.rows, n), -1, 1, seed=71 + n)
    rp, ci = A.row_ptr.numpy(), A.col_idx.numpy()
    for alpha, beta in ((1.0, 0.0), (0.5, -1.5)):
        want = oracle.spmm(rp, ci, bits(A.val), bits(X), alpha, beta, Y0.numpy())
        got = run_tc(handle, A, X, Y0, alpha, beta, kernel=kernel)
        err = rel_l2(got, want)
        assert err <= 1e-2 and err <= 1e-5, err


@pytest.mark.parametrize("kernel", list(KERNELS))
def test_dense_blocks_and_empty_rows_bf16(handle, kernel):
    """Block-dense matrix (every touched 64-column chunk well filled) with empty rows and an empty
    row block in the middle."""
    rng = np.random.default_rng(3)
    rows, cols = 640, 512
    dense = np.zeros((rows, cols), dtype=np.float32)
    for rb in range(0, rows, 128):
        if rb == 256:
            continue                              # an entirely empty row block
        for cb in rng.choice(cols // 64, size=3, replace=False):
            blk = rng.standard_normal((128, 64)).astype(np.float32)
            blk[rng.random((128, 64)) < 0.5] = 0
            dense[rb:rb + 128, cb * 64:(cb + 1) * 64] = blk
    dense[5] = 0
    dense[130:140] = 0
    rp = np.zeros(rows + 1, dtype=np.int32)
    ci, v = [], []
    for r in range(rows):
        nz = np.nonzero(dense[r])[0]
        ci.append(nz)
        v.append(dense[r, nz])
        rp[r + 1] = rp[r] + len(nz)
    A = G.Csr(rows, cols, torch.from_numpy(rp), torch.from_numpy(np.concatenate(ci).astype(np.int32)),
              torch.from_numpy(np.concatenate(v)).to(torch.bfloat16))
    X = G.uniform((cols, 128), -1, 1, dtype=torch.bfloat16, seed=80)
    Y0 = G.uniform((rows, 128), -1, 1, seed=81)
    want = oracle.spmm(rp, A.col_idx.numpy(), bits(A.val), bits(X), 2.0, 1.0, Y0.numpy())
    got = run_tc(handle, A, X, Y0, 2.0, 1.0, ldx=136, ldy=132, kernel=kernel)
    assert rel_l2(got, want) <= 1e-5


@pytest.mark.parametrize("half", [12, 20])
def test_many_row_blocks_per_cta_bf16(handle, half):
    """More row blocks than SMs (every CTA of the persistent kernels walks several, the staging buffers and
    both accumulators wrap around) and rows whose run inside a chunk is long (a banded matrix): 25 entries
    per row are staged in shared memory, 41 per row (5,248 per row block) are read from global memory."""
    rows = 128 * 700 + 37
    r = np.arange(rows, dtype=np.int64)
    lo = np.maximum(r - half, 0)
    hi = np.minimum(r + half, rows - 1)
    rp = np.zeros(rows + 1, dtype=np.int32)
    rp[1:] = np.cumsum(hi - lo + 1)
    ci = np.concatenate([np.arange(a, b + 1, dtype=np.int32) for a, b in zip(lo[:4096], hi[:4096])]
                        + [(np.arange(-half, half + 1, dtype=np.int64)[None, :] + r[4096:rows - 4096, None]).reshape(-1).astype(np.int32)]
                        + [np.arange(a, b + 1, dtype=np.int32) for a, b in zip(lo[rows - 4096:], hi[rows - 4096:])])
    rng = np.random.default_rng(12)
    v = torch.from_numpy(rng.standard_normal(len(ci)).astype(np.float32)).to(torch.bfloat16)
    A = G.Csr(rows, rows, torch.from_numpy(rp), torch.from_numpy(ci), v)
    n = 128
    X = G.uniform((rows, n), -1, 1, dtype=torch.bfloat16, seed=85)
    Y0 = G.uniform((rows, n), -1, 1, seed=86)
    want = oracle.spmm(rp, ci, bits(A.val), bits(X), 1.0, 0.5, Y0.numpy())
    for kernel in ("tcgen05", "tcgen05-smem"):
        got = run_tc(handle, A, X, Y0, 1.0, 0.5, kernel=kernel)
        assert rel_l2(got, want) <= 1e-5, kernel


def test_sparse_random_matrix_is_refused(handle):
    """Uniform random columns: almost every entry sits alone in its chunk, far from dense enough."""
    A = G.poisson_random(1 << 16, 1 << 16, mean_len=16, seed=90).to("cuda")
    A.val = A.val.to(torch.bfloat16)
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr, A.col_idx, A.val)
    B = api.DnMat(torch.zeros(A.cols, 128, dtype=torch.bfloat16, device="cuda"))
    C = api.DnMat(torch.zeros(A.rows, 128, device="cuda"))
    with pytest.raises(api.AlphaSparseError) as e:
        api.spmm(handle, Am, B, C)
    assert e.value.status == 6


def test_column_major_bf16(handle):
    """Column-major B (bf16) and C (fp32) through the row-major copies in the caller's buffer."""
    A = G.stencil_3d_27pt(12, seed=4)
    A.val = A.val.to(torch.bfloat16)
    n = 64
    X = G.uniform((A.cols, n), -1, 1, dtype=torch.bfloat16, seed=75)
    Y0 = G.uniform((A.rows, n), -1, 1, seed=76)
    want = oracle.spmm(A.row_ptr.numpy(), A.col_idx.numpy(), bits(A.val), bits(X), 1.5, 0.5, Y0.numpy())
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr.cuda(), A.col_idx.cuda(), A.val.cuda())
    Bc = X.cuda().t().contiguous().t()        # column-major storage of the same matrix
    Cc = Y0.cuda().t().contiguous().t()
    Bd, Cd = api.DnMat(Bc), api.DnMat(Cc)
    assert Bd.order == api.ORDER_COL
    api.spmm_preprocess(handle, Am, Bd, Cd)
    buf = torch.empty(api.spmm_buffer_size(handle, Am, Bd, Cd), dtype=torch.uint8, device="cuda")
    api.spmm(handle, Am, Bd, Cd, 1.5, 0.5, buffer=buf)
    torch.cuda.synchronize()
    assert rel_l2(Cc.cpu().numpy(), want) <= 1e-5


def test_matrix_without_entries_bf16(handle):
    """No entries: C = beta * C, also on the bf16 path (no chunk, no MMA)."""
    rows, cols, n = 300, 256, 64
    Am = api.CsrMatrix(rows, cols, torch.zeros(rows + 1, dtype=torch.int32, device="cuda"),
                       torch.zeros(0, dtype=torch.int32, device="cuda"),
                       torch.zeros(0, dtype=torch.bfloat16, device="cuda"))
    X = torch.ones(cols, n, dtype=torch.bfloat16, device="cuda")
    Y0 = G.uniform((rows, n), -1, 1, seed=9).cuda()
    Y = Y0.clone()
    api.spmm(handle, Am, api.DnMat(X), api.DnMat(Y), 1.0, 0.25)
    torch.cuda.synchronize()
    assert torch.equal(Y, 0.25 * Y0)


def test_repeated_and_unsorted_columns(handle):
    """CSR allows a column to appear twice in a row and rows in any column order.  The SIMT kernels add
    entries in storage order whatever it is (checked against the oracle, SpMM bit for bit); the tensor-core
    plan places one entry per tile element and walks ascending columns, so it refuses such a matrix."""
    rng = np.random.default_rng(5)
    rows, cols, per = 512, 256, 24
    ci = rng.integers(0, cols, size=(rows, per)).astype(np.int32)     # repeats and no order
    ci[:, 1] = ci[:, 0]                                                # a certain repeat in every row
    rp = (np.arange(rows + 1) * per).astype(np.int32)
    v = rng.standard_normal(rows * per).astype(np.float32)
    ci = ci.reshape(-1)
    x = rng.standard_normal(cols).astype(np.float32)
    want = oracle.spmv(rp, ci, v, x, 1.0, 0.0)
    Am = api.CsrMatrix(rows, cols, torch.from_numpy(rp).cuda(), torch.from_numpy(ci).cuda(), torch.from_numpy(v).cuda())
    for variant in ("binned", "merge"):
        os.environ["ASP_SPMV_VARIANT"] = variant
        try:
            y = torch.zeros(rows, device="cuda")
            api.spmv(handle, Am, api.DnVec(torch.from_numpy(x).cuda()), api.DnVec(y), 1.0, 0.0)
            torch.cuda.synchronize()
        finally:
            del os.environ["ASP_SPMV_VARIANT"]
        assert rel_l2(y.cpu().numpy(), want) <= 1e-5
    X = rng.standard_normal((cols, 64)).astype(np.float32)
    Y = torch.zeros(rows, 64, device="cuda")
    api.spmm(handle, Am, api.DnMat(torch.from_numpy(X).cuda()), api.DnMat(Y), 1.0, 0.0)
    torch.cuda.synchronize()
    assert np.array_equal(Y.cpu().numpy(), oracle.spmm(rp, ci, v, X, 1.0, 0.0))
    Ab = api.CsrMatrix(rows, cols, torch.from_numpy(rp).cuda(), torch.from_numpy(ci).cuda(),
                       torch.from_numpy(v).cuda().to(torch.bfloat16))
    with pytest.raises(api.AlphaSparseError) as e:
        api.spmm(handle, Ab, api.DnMat(torch.from_numpy(X).cuda().to(torch.bfloat16)), api.DnMat(Y), 1.0, 0.0)
    assert e.value.status == 6
    # sorted rows with one repeated column: refused as well
    cs = np.sort(ci.reshape(rows, per), axis=1).reshape(-1)
    Ab2 = api.CsrMatrix(rows, cols, torch.from_numpy(rp).cuda(), torch.from_numpy(cs).cuda(),
                        torch.from_numpy(v).cuda().to(torch.bfloat16))
    with pytest.raises(api.AlphaSparseError) as e:
        api.spmm(handle, Ab2, api.DnMat(torch.from_numpy(X).cuda().to(torch.bfloat16)), api.DnMat(Y), 1.0, 0.0)
    assert e.value.status == 6


def test_waits_that_run_out_are_reported_bf16(handle, monkeypatch):
    """Failure detection without a fault, on the tensor-memory kernel: with ASP_TEST_DROP_COPY the loader warps
    announce the B slices' bytes to the stage barriers but never ask for the copies, so no stage ever fills.
    Every role's bounded wait runs out (ASP_WAIT_POLLS polls), the CTA raises the plan's flag, frees its tensor
    memory and leaves: nothing faults, the context stays usable, the flag shows in the plan statistics, and a
    fresh plan computes the right product."""
    A = G.stencil_3d_27pt(16, seed=4)
    A.val = A.val.to(torch.bfloat16)
    n = 128
    X = G.uniform((A.cols, n), -1, 1, dtype=torch.bfloat16, seed=95)
    Y0 = G.uniform((A.rows, n), -1, 1, seed=96)
    handle.use_torch_stream()
    Am = api.CsrMatrix(A.rows, A.cols, A.row_ptr.cuda(), A.col_idx.cuda(), A.val.cuda())
    B, C = api.DnMat(X.cuda()), api.DnMat(Y0.clone().cuda())
    monkeypatch.setenv("ASP_TEST_DROP_COPY", "1")
    monkeypatch.setenv("ASP_WAIT_POLLS", "64")
    api.spmm_preprocess(handle, Am, B, C)             # the plan takes the wait settings from the environment
    monkeypatch.delenv("ASP_TEST_DROP_COPY")
    monkeypatch.delenv("ASP_WAIT_POLLS")
    api.spmm(handle, Am, B, C, 1.0, 0.0)              # launches; every role gives up and the CTAs leave
    torch.cuda.synchronize()                          # no error from the runtime: nothing faulted
    assert api.spmm_last_variant(Am) == "tcgen05"
    assert Am.plan(handle)[0]["device_error"] == 1
    want = oracle.spmm(A.row_ptr.numpy(), A.col_idx.numpy(), bits(A.val), bits(X), 1.0, 0.0, Y0.numpy())
    got = run_tc(handle, A, X, Y0, 1.0, 0.0, kernel="tcgen05")     # a new descriptor: new plan, normal waits
    assert rel_l2(got, want) <= 1e-5


@pytest.mark.parametrize("kernel", ["tcgen05", "tcgen05-smem"])
def test_row_blocks_with_many_chunks_bf16(handle, kernel):
    """Row blocks that touch 40 column chunks each: more than the tensor-memory kernel stages run words for
    (the rest come from global memory), few entries per chunk, a partial last block; B is tall, so the
    density test still accepts the matrix."""
    rng = np.random.default_rng(21)
    rows, cols = 1024 + 17, 65536
    cis, lens = [], []
    for r in range(rows):
        b = r // 128
        js = np.sort(rng.choice(40, size=30, replace=False))
        c = 64 * ((b * 37 + js * 53) % 1024) + (r * 7 + js) % 64
        c = np.sort(c)
        cis.append(c.astype(np.int32))
        lens.append(len(c))
    rp = np.zeros(rows + 1, dtype=np.int32)
    rp[1:] = np.cumsum(lens)
    ci = np.concatenate(cis)
    v = torch.from_numpy(rng.standard_normal(len(ci)).astype(np.float32)).to(torch.bfloat16)
    A = G.Csr(rows, cols, torch.from_numpy(rp), torch.from_numpy(ci), v)
    n = 128
    X = G.uniform((cols, n), -1, 1, dtype=torch.bfloat16, seed=87)
    Y0 = G.uniform((rows, n), -1, 1, seed=88)
    want = oracle.spmm(rp, ci, bits(A.val), bits(X), 0.75, -0.5, Y0.numpy())
    got = run_tc(handle, A, X, Y0, 0.75, -0.5, kernel=kernel)
    assert rel_l2(got, want) <= 1e-5
