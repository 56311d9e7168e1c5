"""MatrixMarket reader and COO ordering (host functions of the C ABI): what the reference's test
drivers do before alphasparseXcoo2csr (cuda/test/io.cu:1227-1238, cuda/format/coo_order.h:25-43).
The file contents below are written by this test."""
import ctypes as C

import numpy as np
import pytest
import torch

from library_b200 import api


def write(tmp_path, name, text):
    p = tmp_path / name
    p.write_text(text)
    return str(p)


def test_general_real(tmp_path):
    f = write(tmp_path, "g.mtx", "%%MatrixMarket matrix coordinate real general\n% a comment\n\n"
              "3 4 4\n3 1 2.5\n1 4 -1e-2\n1 2 7\n2 2 0.125\n")
    m, n, r, c, v = api.read_mtx(f, torch.float64, ordered=False)
    assert (m, n) == (3, 4)
    assert r.tolist() == [2, 0, 0, 1] and c.tolist() == [0, 3, 1, 1]        # file order, zero-based
    assert v.tolist() == [2.5, -1e-2, 7.0, 0.125]
    m, n, r, c, v = api.read_mtx(f, torch.float32)                           # sorted by (row, column)
    assert r.tolist() == [0, 0, 1, 2] and c.tolist() == [1, 3, 1, 0]
    assert np.allclose(v.numpy(), np.array([7, -1e-2, 0.125, 2.5], np.float32))


def test_symmetric_pattern_and_integer(tmp_path):
    f = write(tmp_path, "s.mtx", "%%MatrixMarket matrix coordinate pattern symmetric\n3 3 3\n1 1\n3 1\n3 2\n")
    m, n, r, c, v = api.read_mtx(f, torch.float32, ordered=False)
    # an off-diagonal entry is followed by its mirror image; pattern entries are 1
    assert r.tolist() == [0, 2, 0, 2, 1] and c.tolist() == [0, 0, 2, 1, 2] and v.tolist() == [1.0] * 5
    f = write(tmp_path, "k.mtx", "%%MatrixMarket matrix coordinate integer skew-symmetric\n2 2 1\n2 1 3\n")
    _, _, r, c, v = api.read_mtx(f, torch.float64, ordered=False)
    assert r.tolist() == [1, 0] and c.tolist() == [0, 1] and v.tolist() == [3.0, 3.0]   # same value, as the reference


def test_errors(tmp_path):
    with pytest.raises(api.AlphaSparseError) as e:
        api.read_mtx(str(tmp_path / "missing.mtx"))
    assert e.value.status == 3
    f = write(tmp_path, "a.mtx", "%%MatrixMarket matrix array real general\n2 2\n1\n2\n3\n4\n")
    with pytest.raises(api.AlphaSparseError) as e:
        api.read_mtx(f)
    assert e.value.status == 6
    f = write(tmp_path, "b.mtx", "%%MatrixMarket matrix coordinate real general\n2 2 2\n1 1 1.0\n3 1 2.0\n")
    with pytest.raises(api.AlphaSparseError) as e:       # row 3 of a 2 x 2 matrix
        api.read_mtx(f)
    assert e.value.status == 3
    f = write(tmp_path, "t.mtx", "%%MatrixMarket matrix coordinate real general\n2 2 3\n1 1 1.0\n")
    with pytest.raises(api.AlphaSparseError):             # fewer entries than announced
        api.read_mtx(f)


def test_order_is_stable():
    lib = api.load()
    r = np.array([1, 0, 1, 0, 1], np.int32)
    c = np.array([2, 5, 2, 1, 0], np.int32)
    v = np.array([10, 20, 30, 40, 50], np.float64)
    assert lib.alphasparseCooOrder(C.c_int64(5), r.ctypes.data_as(C.c_void_p), c.ctypes.data_as(C.c_void_p),
                                   v.ctypes.data_as(C.c_void_p), api.R_64F) == 0
    assert r.tolist() == [0, 0, 1, 1, 1] and c.tolist() == [1, 5, 0, 2, 2]
    assert v.tolist() == [40, 20, 50, 10, 30]             # the two (1, 2) entries keep their file order


def _write_random_matrix(tmp_path):
    from library_b200 import generators as G
    A = G.poisson_random(300, 400, 6.0, dtype=torch.float64, seed=17)
    rp, ci, v = A.numpy()
    rows_of = np.repeat(np.arange(A.rows), np.diff(rp))
    perm = np.random.default_rng(0).permutation(A.nnz)     # entries in arbitrary order in the file
    lines = [f"{rows_of[k] + 1} {ci[k] + 1} {float(v[k])!r}" for k in perm]
    f = write(tmp_path, "p.mtx", "%%MatrixMarket matrix coordinate real general\n"
              f"{A.rows} {A.cols} {A.nnz}\n" + "\n".join(lines) + "\n")
    return A, f


def test_file_round_trip(tmp_path):
    """A matrix written entry by entry in random order comes back, after ordering, as its CSR arrays
    (repr of a double is exact, so values match bit for bit)."""
    A, f = _write_random_matrix(tmp_path)
    rp, ci, v = A.numpy()
    m, n, r, c, vals = api.read_mtx(f, torch.float64)
    assert (m, n, len(r)) == (A.rows, A.cols, A.nnz)
    assert np.array_equal(c.numpy(), ci) and np.array_equal(vals.numpy(), v)
    assert np.array_equal(np.searchsorted(r.numpy(), np.arange(m + 1)), rp)


@pytest.mark.gpu
def test_file_to_spmv(handle, tmp_path):
    """File -> COO -> ordered -> device CSR (alphasparseXcoo2csr) -> SpMV, against the oracle."""
    import oracle
    from conftest import rel_l2
    from library_b200 import generators as G
    A, f = _write_random_matrix(tmp_path)
    rp, ci, v = A.numpy()
    m, n, r, c, vals = api.read_mtx(f, torch.float64)
    row_ptr = api.coo2csr(r.cuda(), m)
    assert np.array_equal(row_ptr.cpu().numpy(), rp)
    Am = api.CsrMatrix(m, n, row_ptr, c.cuda(), vals.cuda())
    x = G.uniform((n,), -1, 1, dtype=torch.float64, seed=3)
    y = torch.zeros(m, dtype=torch.float64, device="cuda")
    api.spmv(handle, Am, api.DnVec(x.cuda()), api.DnVec(y), 1.0, 0.0)
    torch.cuda.synchronize()
    assert rel_l2(y.cpu().numpy(), oracle.spmv(rp, ci, v, x.numpy(), 1.0, 0.0)) <= 1e-12


def _write_bin(path, rows, cols, recs, fields, sym):
    """The reference drivers' dump format: eight int64, then int32 row, int32 column (one-based), `fields` doubles."""
    mirrored = sum(2 if (sym and r != c) else 1 for r, c, *_ in recs)
    with open(path, "wb") as f:
        np.array([rows, cols, len(recs), mirrored, fields, 0, sym, 0], dtype=np.int64).tofile(f)
        for r, c, *vals in recs:
            np.array([r, c], dtype=np.int32).tofile(f)
            np.array(vals[:fields], dtype=np.float64).tofile(f)


def test_binary_dump_general_symmetric_pattern_and_complex(tmp_path):
    p = str(tmp_path / "g.bin")
    _write_bin(p, 3, 4, [(3, 1, 2.5), (1, 4, -1e-2), (1, 2, 7.0)], 1, 0)
    m, n, r, c, v = api.read_mtx(p, torch.float64, ordered=False)
    assert (m, n) == (3, 4) and r.tolist() == [2, 0, 0] and c.tolist() == [0, 3, 1] and v.tolist() == [2.5, -1e-2, 7.0]
    m, n, r, c, v = api.read_mtx(p, torch.float32)                           # ordered by (row, column)
    assert r.tolist() == [0, 0, 2] and c.tolist() == [1, 3, 0]
    p = str(tmp_path / "s.bin")
    _write_bin(p, 3, 3, [(1, 1, 4.0), (3, 1, -1.0)], 1, 1)                   # symmetric: the mirror follows the entry
    _, _, r, c, v = api.read_mtx(p, torch.float64, ordered=False)
    assert r.tolist() == [0, 2, 0] and c.tolist() == [0, 0, 2] and v.tolist() == [4.0, -1.0, -1.0]
    p = str(tmp_path / "p.bin")
    _write_bin(p, 2, 2, [(1, 2), (2, 2)], 0, 0)                              # pattern: value 1
    _, _, r, c, v = api.read_mtx(p, torch.float32, ordered=False)
    assert r.tolist() == [0, 1] and c.tolist() == [1, 1] and v.tolist() == [1.0, 1.0]
    p = str(tmp_path / "z.bin")
    _write_bin(p, 2, 2, [(1, 1, 3.0, 9.0)], 2, 0)                            # complex: the real part, as the reference
    _, _, r, c, v = api.read_mtx(p, torch.float64, ordered=False)
    assert v.tolist() == [3.0]


def test_binary_dump_errors(tmp_path):
    lib = api.load()
    out = [C.c_int64() for _ in range(3)]
    ptrs = [C.c_void_p() for _ in range(3)]

    def read(path):
        return lib.alphasparseReadBinCoo(path.encode(), *[C.byref(o) for o in out], *[C.byref(p) for p in ptrs], api.R_32F)
    assert read(str(tmp_path / "missing.bin")) == 3
    p = str(tmp_path / "short.bin")
    _write_bin(p, 3, 3, [(1, 1, 1.0)], 1, 0)
    with open(p, "r+b") as f:
        f.truncate(64 + 8 + 4)                                               # the record is cut off
    assert read(p) == 3
    p = str(tmp_path / "range.bin")
    _write_bin(p, 3, 3, [(4, 1, 1.0)], 1, 0)                                 # row outside the announced size
    assert read(p) == 3
