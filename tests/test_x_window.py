"""Column-window exchange of x for a row-sharded matrix (x sharded like y).

CPU part: the exchange plan (who sends which range to whom) against a brute-force statement, and
the exchange itself on gloo ranks (world 2 and 3): every rank's window equals the same slice of
the whole x, and a banded matrix moves only its halo.  GPU part: a windowed x descriptor through
the C ABI gives the same y as the whole x on one device (the exchange over NCCL on two devices is
covered by tests/test_mg.py).
"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_exchange_plan_brute_force():
    from library_b200.sharding import exchange_plan
    rng = np.random.default_rng(3)
    for world in (1, 2, 3, 5):
        n = 1000
        cuts = np.sort(rng.integers(0, n + 1, size=world - 1))
        own = np.concatenate([[0], cuts, [n]])
        windows = []
        for _ in range(world):
            a, b = sorted(rng.integers(0, n + 1, size=2))
            windows.append((int(a), int(b)) if rng.random() > 0.2 else (0, 0))
        owner = np.searchsorted(own[1:], np.arange(n), side="right")
        for r in range(world):
            sends, recvs = exchange_plan(own, windows, r)
            got = np.full(n, -1)
            for p, a, b in recvs:
                assert np.all(owner[a:b] == p) and np.all(got[a:b] == -1)
                got[a:b] = p
            lo, hi = windows[r]
            want = np.full(n, -1)
            want[lo:hi] = owner[lo:hi]
            assert np.array_equal(got, want)
            # what r sends to p is what p expects from r
            for p, a, b in sends:
                assert (r, a, b) in exchange_plan(own, windows, p)[1]


def _cpu_worker(rank, world, port, out_dir, kind):
    sys.path.insert(0, ROOT)
    import oracle
    from library_b200 import generators as G
    from library_b200.sharding import partition_bounds_host, XWindowExchange
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    A = G.laplacian_2d_5pt(48) if kind == "banded" else G.rmat(11, 8, seed=5, dtype=torch.float64)
    rp, ci, v = A.numpy()
    x = G.uniform((A.cols,), -1, 1, dtype=torch.float64, seed=6).numpy()
    b = partition_bounds_host(rp, world)
    r0, r1 = int(b[rank]), int(b[rank + 1])
    k0, k1 = int(rp[r0]), int(rp[r1])
    cols = ci[k0:k1]
    cmin, cmax = (int(cols.min()), int(cols.max())) if len(cols) else (0, -1)
    ex = XWindowExchange(b, cmin, cmax, rank, world, torch.float64, "cpu")
    win = ex.run(torch.from_numpy(x[r0:r1].copy()))          # this rank holds only its own part of x
    assert np.array_equal(win.numpy(), x[ex.lo:ex.hi])
    # the same with x kept inside the window (no local copy): only the halo is filled in
    ex.window.fill_(float("nan"))
    xv = ex.own_view()
    a = max(ex.lo, r0)
    xv.copy_(torch.from_numpy(x[a:a + xv.numel()].copy()))
    assert np.array_equal(ex.run(xv).numpy(), x[ex.lo:ex.hi])
    # the oracle indexes x from 0: place the window in a vector of NaN so that any read outside it shows
    xw = np.full(A.cols, np.nan)
    xw[ex.lo:ex.hi] = win.numpy()
    local_rp = (rp[r0:r1 + 1] - rp[r0]).astype(np.int32)
    y = oracle.spmv(local_rp, cols, v[k0:k1], xw, 1.5, 0.0)
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y)
    np.save(os.path.join(out_dir, f"recv{rank}.npy"), np.array([ex.bytes_received]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,kind", [(2, "banded"), (3, "banded"), (3, "rmat")])
def test_window_exchange_on_cpu_ranks(tmp_path, world, kind):
    import oracle
    from library_b200 import generators as G
    mp.spawn(_cpu_worker, args=(world, _free_port(), str(tmp_path), kind), nprocs=world, join=True)
    A = G.laplacian_2d_5pt(48) if kind == "banded" else G.rmat(11, 8, seed=5, dtype=torch.float64)
    rp, ci, v = A.numpy()
    x = G.uniform((A.cols,), -1, 1, dtype=torch.float64, seed=6).numpy()
    want = oracle.spmv(rp, ci, v, x, 1.5, 0.0)
    got = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(world)])
    assert np.array_equal(got, want)
    recv = [int(np.load(tmp_path / f"recv{r}.npy")[0]) for r in range(world)]
    if kind == "banded":
        # a rank of the 48-wide grid needs at most one grid line (plus alignment slack) per neighbour
        assert max(recv) <= 2 * (48 + 32) * 8


def test_interior_row_range():
    """Rows whose columns all lie in the rank's own part of x need no halo."""
    from library_b200 import generators as G
    from library_b200.sharding import interior_row_range
    A = G.laplacian_2d_5pt(16)                         # 256 rows, grid lines of 16
    rp, ci = A.row_ptr, A.col_idx
    r0, r1 = 64, 128
    k0, k1 = int(rp[r0]), int(rp[r1])
    local = rp[r0:r1 + 1] - rp[r0]
    assert interior_row_range(local, ci[k0:k1], 64, 128) == (16, 48)     # first and last grid line reach out
    assert interior_row_range(local, ci[k0:k1], 0, 256) == (0, 64)
    assert interior_row_range(local, ci[k0:k1], 0, 10) == (0, 0)
    # brute force on a random matrix: every row of the range is inside, the row before and after are not
    B = G.poisson_random(200, 300, 4.0, seed=8)
    i0, i1 = interior_row_range(B.row_ptr, B.col_idx, 20, 280)
    rp, ci = B.row_ptr.numpy(), B.col_idx.numpy()
    inside = [all(20 <= c < 280 for c in ci[rp[r]:rp[r + 1]]) for r in range(200)]
    assert all(inside[i0:i1]) and (i0 == 0 or not inside[i0 - 1] or i0 == inside.index(True)) and (i1 == 200 or not inside[i1])


@pytest.mark.gpu
def test_windowed_x_equals_whole_x(handle):
    from library_b200 import api
    from library_b200 import generators as G
    A = G.laplacian_3d_7pt(40, dtype=torch.float32, index64=False).to("cuda")
    x = G.uniform((A.cols,), -1, 1, device="cuda", seed=3)
    r0, r1 = 20000, 41000
    k0, k1 = int(A.row_ptr[r0]), int(A.row_ptr[r1])
    rp = api.rebase_row_offsets(handle, A.row_ptr, r0, r1)
    col = A.col_idx[k0:k1].clone()
    val = A.val[k0:k1].clone()
    lo, hi = api.column_range(handle, col)
    assert (lo, hi) == (int(col.min()), int(col.max()))
    assert api.column_range(handle, col[:0]) == (0, -1)
    Am = api.CsrMatrix(r1 - r0, A.cols, rp, col, val)
    y_full = torch.zeros(r1 - r0, device="cuda")
    api.spmv(handle, Am, api.DnVec(x), api.DnVec(y_full), 1.0, 0.0)
    lo_al = lo // 32 * 32
    win = x[lo_al:hi + 1].clone()
    for variant in ("binned", "merge"):
        os.environ["ASP_SPMV_VARIANT"] = variant
        try:
            y_win = torch.full((r1 - r0,), 7.0, device="cuda")
            api.spmv(handle, Am, api.DnVecWindow(win, A.cols, lo_al), api.DnVec(y_win), 1.0, 0.0)
            torch.cuda.synchronize()
        finally:
            del os.environ["ASP_SPMV_VARIANT"]
        assert torch.allclose(y_win, y_full, rtol=1e-6, atol=1e-6)
    with pytest.raises(api.AlphaSparseError):
        api.DnVecWindow(win, A.cols, A.cols - 1)          # window runs past the logical end
