"""The CPU oracle (oracle/csr_oracle.c) against the golden vectors produced by the reference's
own hygon code, and against that code live when oracle/_ref/libasp_ref.so is present."""
import numpy as np
import pytest

import oracle
from conftest import load_golden, rel_l2

CASES = sorted(load_golden().keys())


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_reference_golden(golden, name):
    c = golden[name]
    if c["kind"] == "mv":
        y = oracle.spmv(c["rp"], c["ci"], c["v"], c["x"], c["alpha"], c["beta"], c["y0"])
    else:
        y = oracle.spmm(c["rp"], c["ci"], c["v"], c["x"], c["alpha"], c["beta"], c["y0"])
    # same summation order as the reference's kernels: bit-exact
    assert np.array_equal(y, c["y"]), rel_l2(y, c["y"])


@pytest.mark.parametrize("name", CASES)
def test_oracle_i64_offsets_same_as_i32(golden, name):
    c = golden[name]
    rp64 = c["rp"].astype(np.int64)
    if c["kind"] == "mv":
        y = oracle.spmv(rp64, c["ci"], c["v"], c["x"], c["alpha"], c["beta"], c["y0"])
    else:
        y = oracle.spmm(rp64, c["ci"], c["v"], c["x"], c["alpha"], c["beta"], c["y0"])
    assert np.array_equal(y, c["y"])


@pytest.mark.skipif(not oracle.have_ref(), reason="reference library not built")
@pytest.mark.parametrize("name", CASES)
def test_live_reference_matches_golden(golden, name):
    c = golden[name]
    oracle.ref_set_threads(3)
    if c["kind"] == "mv":
        y, _ = oracle.ref_spmv(c["rp"], c["ci"], c["v"], c["x"], c["alpha"], c["beta"], c["y0"], cols=c["cols"])
    else:
        y, _ = oracle.ref_spmm(c["rp"], c["ci"], c["v"], c["x"], c["alpha"], c["beta"], c["y0"])
    assert np.array_equal(y, c["y"])


def test_analytic_laplacian_row_sums():
    """A*1 for the 5-point Laplacian: 0 in the interior, positive on the border."""
    from library_b200 import generators as G
    A = G.laplacian_2d_5pt(16)
    rp, ci, v = A.numpy()
    y = oracle.spmv(rp, ci, v, np.ones(A.cols), 1.0, 0.0)
    y = y.reshape(16, 16)
    assert np.all(y[1:-1, 1:-1] == 0.0)
    assert np.all(y[0, :] > 0) and np.all(y[:, 0] > 0) and y[0, 0] == 2.0


def test_bf16_oracle_matches_widened_f32():
    import torch
    from library_b200 import generators as G
    A = G.stencil_3d_27pt(5, seed=1)
    rp, ci, v = A.numpy()
    vb = torch.from_numpy(v).to(torch.bfloat16)
    X = G.uniform((A.cols, 16), -1, 1, dtype=torch.bfloat16, seed=3)
    Yb = oracle.spmm(rp, ci, vb.view(torch.int16).numpy().view(np.uint16),
                     X.view(torch.int16).numpy().view(np.uint16), 1.0, 0.0)
    Yf = oracle.spmm(rp, ci, vb.float().numpy(), X.float().numpy(), 1.0, 0.0)
    assert np.array_equal(Yb, Yf)


def test_partition_matches_reference_rule():
    from library_b200 import generators as G
    A = G.rmat(10, 8, seed=1)
    rp, _, _ = A.numpy()
    for parts in (1, 2, 3, 8):
        b = oracle.partition_rows_by_nnz(rp, parts)
        b64 = oracle.partition_rows_by_nnz(rp.astype(np.int64), parts)
        assert np.array_equal(b, b64)
        assert b[0] == 0 and b[-1] == A.rows and np.all(np.diff(b) >= 0)
        # restated rule: first j in [0, rows-1] with row_end[j] >= (nnz/parts)*i
        row_end = rp[1:]
        nnz = int(row_end[-1])
        for i in range(1, parts):
            target = (nnz // parts) * i
            j = int(np.searchsorted(row_end[:-1], target, side="left"))
            assert b[i] == j


def test_empty_and_degenerate_inputs():
    rp = np.zeros(5, dtype=np.int32)
    y = oracle.spmv(rp, np.zeros(0, np.int32), np.zeros(0, np.float32), np.ones(3, np.float32), 2.0, 0.5,
                    np.full(4, 4.0, np.float32))
    assert np.array_equal(y, np.full(4, 2.0, np.float32))
    # one row holding every entry
    rp = np.array([0, 0, 7, 7], dtype=np.int32)
    ci = np.arange(7, dtype=np.int32)
    v = np.arange(1, 8, dtype=np.float64)
    y = oracle.spmv(rp, ci, v, np.ones(7), 1.0, 0.0)
    assert np.array_equal(y, np.array([0.0, 28.0, 0.0]))
