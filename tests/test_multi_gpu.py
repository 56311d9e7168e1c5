"""Row-sharded SpMV across ranks.

CPU part (gloo, world_size 2, runs anywhere): the host-side planning - bounds, rebased offsets,
replication of x with a broadcast, sharded y - assembled from per-rank oracle results equals the
single-process oracle bit for bit.  The GPU side of the same split (NCCL, through the C ABI) is
covered by tests/test_mg.py.
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


def _cpu_worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import oracle
    from library_b200 import generators as G
    from library_b200.sharding import partition_bounds_host
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    A = G.rmat(12, 8, seed=5, dtype=torch.float64)          # every rank builds the same matrix
    rp, ci, v = A.numpy()
    x = torch.zeros(A.cols, dtype=torch.float64)
    if rank == 0:
        x = G.uniform((A.cols,), -1, 1, dtype=torch.float64, seed=6)
    dist.broadcast(x, src=0)                                   # the exchange step of the path
    b = partition_bounds_host(rp, world)
    assert np.array_equal(b, oracle.partition_rows_by_nnz(rp, world))
    r0, r1 = int(b[rank]), int(b[rank + 1])
    k0, k1 = int(rp[r0]), int(rp[r1])
    local_rp = (rp[r0:r1 + 1] - rp[r0]).astype(np.int32)
    y_local = oracle.spmv(local_rp, ci[k0:k1], v[k0:k1], x.numpy(), 1.5, 0.0)
    np.save(os.path.join(out_dir, f"y{rank}.npy"), y_local)
    np.save(os.path.join(out_dir, f"b{rank}.npy"), b)
    dist.barrier()
    dist.destroy_process_group()


def test_row_sharding_on_cpu_ranks(tmp_path):
    import oracle
    from library_b200 import generators as G
    world = 2
    mp.spawn(_cpu_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    A = G.rmat(12, 8, seed=5, dtype=torch.float64)
    rp, ci, v = A.numpy()
    x = G.uniform((A.cols,), -1, 1, dtype=torch.float64, seed=6).numpy()
    want = oracle.spmv(rp, ci, v, x, 1.5, 0.0)
    got = np.concatenate([np.load(tmp_path / f"y{r}.npy") for r in range(world)])
    assert np.array_equal(got, want)
    b = np.load(tmp_path / "b0.npy")
    nnz_per = np.diff(rp[b])
    assert abs(int(nnz_per[0]) - int(nnz_per[1])) <= int(np.diff(rp).max()) + 1  # balanced up to one row


def test_partition_edge_cases_host():
    from library_b200.sharding import partition_bounds_host
    import oracle
    for rp in (np.array([0], np.int64), np.array([0, 0, 0, 0], np.int64), np.array([0, 5], np.int64),
               np.array([0, 1, 2, 3, 4, 5, 6, 7, 8], np.int64)):
        for parts in (1, 2, 3, 8):
            if len(rp) > 1:
                assert np.array_equal(partition_bounds_host(rp, parts), oracle.partition_rows_by_nnz(rp, parts))
