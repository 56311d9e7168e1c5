"""Multi-GPU SpMV behind the C ABI (alphasparseMg*).

CPU part: the host-side exchange planner against a brute-force statement and against its Python
twin; argument checks that need no device.  GPU part, one device: a world of one rank gives the
oracle's y in every exchange mode.  GPU part, two devices (skipped otherwise; NVLS off): every
exchange mode and both SpMV kernel families against the CPU oracle on the whole matrix, the
interior row range against its Python twin, the halo size of a banded matrix, x kept inside the
window, and the statuses for arguments that do not fit the communicator.
"""
import ctypes as C
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


def test_exchange_plan_through_the_c_abi():
    from library_b200 import api
    from library_b200.sharding import exchange_plan
    rng = np.random.default_rng(3)
    for world in (1, 2, 3, 5, 8):
        n = 1000
        cuts = np.sort(rng.integers(0, n + 1, size=world - 1))
        own = np.concatenate([[0], cuts, [n]]).astype(np.int64)
        windows = []
        for _ in range(world):
            a, b = sorted(rng.integers(0, n + 1, size=2))
            windows.append((int(a), int(b)) if rng.random() > 0.2 else (0, 0))
        owner = np.searchsorted(own[1:], np.arange(n), side="right")
        plans = [api.mg_exchange_plan(own, windows, r) for r in range(world)]
        for r in range(world):
            sends, recvs = plans[r]
            assert (sends, recvs) == exchange_plan(own, windows, r)        # the Python twin
            got = np.full(n, -1)
            for p, a, b in recvs:
                assert np.all(owner[a:b] == p) and np.all(got[a:b] == -1)
                got[a:b] = p
            lo, hi = windows[r]
            want = np.full(n, -1)
            want[lo:hi] = owner[lo:hi]
            assert np.array_equal(got, want)
            for p, a, b in sends:                                          # what r sends, p expects
                assert (r, a, b) in plans[p][1]


def test_argument_checks_without_a_device():
    from library_b200 import api
    lib = api.load()
    mg = C.c_void_p()
    assert lib.alphasparseMgCreate(C.byref(mg), None, None, 0, 1) == 8          # INVALID_HANDLE
    assert lib.alphasparseMgCreate(None, None, None, 0, 1) == 7                 # INVALID_POINTER
    assert lib.alphasparseMgSpMV(None, None, None, None, None, 0) == 8
    assert lib.alphasparseMgSetShard(None, None, None, 0, 0) == 8
    one = np.zeros(3, dtype=np.int64)
    n = C.c_int(0)
    p = one.ctypes.data_as(C.c_void_p)
    assert lib.alphasparseMgExchangePlan(2, 2, p, p, p, C.byref(n), p, C.byref(n)) == 10   # rank outside the world
    down = np.array([0, 5, 3], dtype=np.int64)
    w = np.zeros(4, dtype=np.int64)
    buf = np.zeros(6, dtype=np.int64)
    assert lib.alphasparseMgExchangePlan(2, 0, down.ctypes.data_as(C.c_void_p), w.ctypes.data_as(C.c_void_p),
                                         buf.ctypes.data_as(C.c_void_p), C.byref(n),
                                         buf.ctypes.data_as(C.c_void_p), C.byref(n)) == 3   # bounds not ascending


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [0, 1, 2, 3])
def test_world_of_one_rank(handle, mode):
    import oracle
    from conftest import rel_l2
    from library_b200 import api
    from library_b200 import generators as G
    A = G.rmat(13, 12, seed=21)
    rp, ci, v = A.numpy()
    x = G.uniform((A.cols,), 0, 1, seed=22)
    y0 = G.uniform((A.rows,), -1, 1, seed=23)
    want = oracle.spmv(rp, ci, v, x.numpy(), 1.5, 0.5, y0.numpy())
    handle.use_torch_stream()
    Am = api.CsrMatrix.from_csr(A)
    mg = api.Mg(handle, 0, 1)
    mg.set_shard(Am, [0, A.cols], mode)
    y = y0.cuda()
    mg.spmv(x.cuda(), y, 1.5, 0.5)
    torch.cuda.synchronize()
    assert rel_l2(y.cpu().numpy(), want) <= 1e-5
    mg.close()


def _cases():
    from library_b200 import generators as G
    return {
        "lap3d_f64": (lambda: G.laplacian_3d_7pt(48, dtype=torch.float64), torch.float64, 1e-12, (-1.0, 1.0)),
        "rmat_f32": (lambda: G.rmat(16, 16, seed=7), torch.float32, 1e-5, (0.0, 1.0)),
    }


def _gpu_worker(rank, world, port, out_dir):
    """A rank whose check fails leaves at once, without running finalisers: tearing down its communicator would
    wait for the other ranks, which wait for it in their next collective, and nobody would ever report."""
    try:
        _gpu_worker_body(rank, world, port, out_dir)
    except BaseException:
        import traceback
        traceback.print_exc()
        sys.stderr.flush()
        os._exit(1)


def _gpu_worker_body(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    from library_b200 import api
    from library_b200 import generators as G
    from library_b200.sharding import interior_row_range, shard_csr
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    h = api.Handle()
    stream = torch.cuda.Stream()
    h.set_stream(stream.cuda_stream)
    mg = api.Mg(h, rank, world)
    # a communicator of another shape is refused on the host, before anything is enqueued
    bad = C.c_void_p()
    assert api.load().alphasparseMgCreate(C.byref(bad), h.h, mg.comm, rank, world + 1) == 3
    for name, (make, dt, tol, (xlo, xhi)) in _cases().items():
        A = make().to(dev)
        x = G.uniform((A.cols,), xlo, xhi, dtype=dt, seed=8).to(dev)      # the host generator's stream: same on every rank
        y0 = G.uniform((A.rows,), -1, 1, dtype=dt, seed=9).to(dev)
        with torch.cuda.stream(stream):
            bounds = api.partition_rows_by_nnz(h, A.row_ptr, world)
            Aloc, (r0, r1) = shard_csr(h, A.rows, A.cols, A.row_ptr, A.col_idx, A.val, rank, world)
        torch.cuda.synchronize()
        x_own = x[r0:r1].clone()
        torch.cuda.synchronize()
        # x bounds that do not cover the vector are refused
        wrong = np.array(bounds, dtype=np.int64)
        wrong[-1] -= 1
        with pytest.raises(api.AlphaSparseError):
            mg.set_shard(Aloc, wrong, api.MG_X_WINDOW)
        for mode in (api.MG_X_BROADCAST, api.MG_X_ALLGATHER, api.MG_X_WINDOW, api.MG_X_WINDOW_OVERLAP):
            mg.set_shard(Aloc, bounds, mode, root=0)
            info = mg.info()
            for variant in ("binned", "merge"):
                os.environ["ASP_SPMV_VARIANT"] = variant
                y = y0[r0:r1].clone()
                torch.cuda.synchronize()
                xin = (x.clone() if rank == 0 else None) if mode == api.MG_X_BROADCAST else x_own
                torch.cuda.synchronize()
                for _ in range(2):                     # twice: the second call meets the first one's window
                    y.copy_(y0[r0:r1])
                    torch.cuda.synchronize()
                    mg.spmv(xin, y, 1.5, 0.5)
                    torch.cuda.synchronize()
                np.save(os.path.join(out_dir, f"{name}_m{mode}_{variant}_y{rank}.npy"), y.cpu().numpy())
            os.environ.pop("ASP_SPMV_VARIANT", None)
            np.save(os.path.join(out_dir, f"{name}_m{mode}_recv{rank}.npy"), np.array([info["bytes_received"]]))
            if mode == api.MG_X_WINDOW_OVERLAP:
                i0, i1 = interior_row_range(Aloc.row_ptr, Aloc.col_idx, int(bounds[rank]), int(bounds[rank + 1]), align=4)
                assert (info["interior_begin"], info["interior_end"]) == (i0, i1)
                if name == "lap3d_f64":
                    assert i1 > i0 and (i0 > 0 or i1 < Aloc.rows)       # a slab's first or last grid plane reaches out
                    if 0 < rank < world - 1:
                        assert i0 > 0 and i1 < Aloc.rows                # a middle rank: halo rows on both sides
                    # x kept inside the window: only the halo moves, same y
                    xv = mg.own_view()
                    assert xv.numel() == r1 - r0
                    xv.copy_(x_own)
                    y = y0[r0:r1].clone()
                    torch.cuda.synchronize()
                    mg.spmv(xv, y, 1.5, 0.5)
                    torch.cuda.synchronize()
                    np.save(os.path.join(out_dir, f"{name}_inplace_y{rank}.npy"), y.cpu().numpy())
        assert Aloc.plan(h)[0]["device_error"] == 0
    torch.cuda.synchronize()
    dist.barrier()
    mg.close()
    dist.destroy_process_group()


def _spawn_bounded(fn, args, nprocs, seconds):
    """mp.spawn with a limit: ranks that wait for one another in a collective never return by themselves, so a
    stalled run is ended here (the processes are terminated) and reported as a failure instead of lasting as long
    as whoever runs the tests lets it."""
    import time
    ctx = mp.spawn(fn, args=args, nprocs=nprocs, join=False)
    deadline = time.monotonic() + seconds
    while not ctx.join(timeout=5):
        if time.monotonic() > deadline:
            for proc in ctx.processes:
                if proc.is_alive():
                    proc.terminate()
            pytest.fail(f"the {nprocs} ranks did not finish within {seconds} s")


def _sleep_worker(rank, seconds):
    import time
    time.sleep(seconds if rank == 1 else 0.1)


def test_a_stalled_multi_rank_run_is_ended():
    """The limit of _spawn_bounded: ranks that finish pass, a rank that does not come back fails the test after
    the limit instead of holding it."""
    _spawn_bounded(_sleep_worker, (0.2,), 2, seconds=60)
    with pytest.raises(pytest.fail.Exception):
        _spawn_bounded(_sleep_worker, (600,), 2, seconds=6)


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4])
def test_every_mode_on_several_gpus_against_the_oracle(tmp_path, world):
    """Two ranks: each has one neighbour.  Four ranks: the middle ranks have two, so their shard is cut into
    top boundary rows, interior rows and bottom boundary rows."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} CUDA devices")
    import oracle
    from conftest import rel_l2
    from library_b200 import generators as G
    _spawn_bounded(_gpu_worker, (world, _free_port(), str(tmp_path)), world, seconds=240)
    for name, (make, dt, tol, (xlo, xhi)) in _cases().items():
        A = make()
        rp, ci, v = A.numpy()
        x = G.uniform((A.cols,), xlo, xhi, dtype=dt, seed=8).numpy()
        y0 = G.uniform((A.rows,), -1, 1, dtype=dt, seed=9).numpy()
        want = oracle.spmv(rp, ci, v, x, 1.5, 0.5, y0)
        for mode in (0, 1, 2, 3):
            for variant in ("binned", "merge"):
                got = np.concatenate([np.load(tmp_path / f"{name}_m{mode}_{variant}_y{r}.npy") for r in range(world)])
                assert got.shape == want.shape and rel_l2(got, want) <= tol, (name, mode, variant)
        if name == "lap3d_f64":
            got = np.concatenate([np.load(tmp_path / f"{name}_inplace_y{r}.npy") for r in range(world)])
            assert rel_l2(got, want) <= tol
            for mode in (2, 3):
                recv = [int(np.load(tmp_path / f"{name}_m{mode}_recv{r}.npy")[0]) for r in range(world)]
                planes = 1 if world == 2 else 2                     # a middle rank has a neighbour on either side
                assert 0 < max(recv) <= planes * (48 * 48 + 32) * 8 # one grid plane per neighbour (plus alignment slack)
            recv = [int(np.load(tmp_path / f"{name}_m1_recv{r}.npy")[0]) for r in range(world)]
            assert max(recv) >= (A.cols * (world - 1) // world - 48 * 48) * 8     # all-gather: everybody else's part
