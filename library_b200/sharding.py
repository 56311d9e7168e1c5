"""Row sharding of one CSR matrix across ranks (one process per GPU).

Rows are split into contiguous ranges of near-equal nnz by the C ABI call
alphasparseCsrPartitionRowsByNnz (the rule of the reference's CPU partitioner,
hygon/util/partition.cpp:83-96, in 64-bit).  A shard keeps global column indices, its own
rebased row offsets (32-bit when the shard's nnz allows) and the matching slices of the column
and value arrays; x is replicated to every rank, y stays sharded by rows.
"""
from __future__ import annotations

import numpy as np
import torch

from . import api


def partition_bounds_host(row_ptr: np.ndarray, parts: int) -> np.ndarray:
    """The same rule on the host (numpy), for planning without a GPU:
    bounds[i] = first j in [0, rows-1] with row_end[j] >= (nnz // parts) * i."""
    row_ptr = np.asarray(row_ptr, dtype=np.int64)
    rows = len(row_ptr) - 1
    out = np.zeros(parts + 1, dtype=np.int64)
    out[parts] = max(rows, 0)
    if rows <= 0:
        return out
    row_end = row_ptr[1:]
    ave = int(row_end[rows - 1]) // parts
    for i in range(1, parts):
        out[i] = int(np.searchsorted(row_end[: rows - 1], ave * i, side="left"))
    return out


def shard_csr(handle: api.Handle, rows: int, cols: int, row_ptr: torch.Tensor, col_idx: torch.Tensor,
              val: torch.Tensor, rank: int, world: int):
    """Returns (CsrMatrix of this rank's rows, (row_begin, row_end)).  Device tensors in, device
    views out (col/val are slices, offsets are a new small tensor)."""
    bounds = api.partition_rows_by_nnz(handle, row_ptr, world)
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    k0 = int(row_ptr[r0].item())
    k1 = int(row_ptr[r1].item())
    out_dtype = torch.int32 if (k1 - k0) < 2 ** 31 else torch.int64
    local_rp = api.rebase_row_offsets(handle, row_ptr, r0, r1, out_dtype)
    A = api.CsrMatrix(r1 - r0, cols, local_rp, col_idx[k0:k1], val[k0:k1])
    return A, (r0, r1)
