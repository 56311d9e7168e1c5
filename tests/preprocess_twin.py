"""CPU twin (numpy) of the CSR preprocessing pass, used to check the device result bit for bit.

Restates, in 64-bit integer arithmetic:
  * the row classes (short / medium / long by row length) and per-class row lists in row order,
  * the merge-path start coordinate of every tile: the search of the reference's
    merge_path_search (cuda/kernel/level2/alphasparse_spmv_csr_merge_ginkgo.h:11-35) applied
    to diagonals t * items,
  * the lane-group width and variant rules of library_b200/csrc/analysis.cu.
"""
import numpy as np

SHORT_MAX = 64
MEDIUM_MAX = 4096
MERGE_ITEMS = 2048
SMALL_PROBLEM_TILES = 1200


def merge_path_row(row_end, nnz, diag):
    rows = len(row_end)
    lo = max(diag - nnz, 0)
    hi = min(diag, rows)
    while lo < hi:
        mid = (lo + hi) >> 1
        if row_end[mid] <= diag - mid - 1:
            lo = mid + 1
        else:
            hi = mid
    return lo


def col_step(row_ptr, col_idx):
    """Mean |first column of row r+1 - first column of row r| over neighbouring non-empty rows, rounded
    half up (the statistic that decides the L2 policy of the bulk copies of A)."""
    row_ptr = np.asarray(row_ptr, dtype=np.int64)
    col_idx = np.asarray(col_idx, dtype=np.int64)
    a, b, c = row_ptr[:-2], row_ptr[1:-1], row_ptr[2:]
    ok = (b > a) & (c > b)
    if not ok.any():
        return 0
    d = np.abs(col_idx[b[ok]] - col_idx[a[ok]])
    return int(int(d.sum()) / int(ok.sum()) + 0.5)


def plan(row_ptr, val_bytes, col_idx=None):
    row_ptr = np.asarray(row_ptr, dtype=np.int64)
    rows = len(row_ptr) - 1
    nnz = int(row_ptr[-1]) if rows >= 0 and len(row_ptr) else 0
    lens = np.diff(row_ptr)
    cls = np.where(lens <= SHORT_MAX, 0, np.where(lens <= MEDIUM_MAX, 1, 2))
    bins = np.concatenate([np.nonzero(cls == c)[0] for c in range(3)]).astype(np.int32)
    n_short, n_medium, n_long = (int((cls == c).sum()) for c in range(3))
    empty = int((lens == 0).sum())
    nnz_short = int(lens[cls == 0].sum())
    vec = 16 // val_bytes
    nonempty = max(n_short - empty, 1)
    mean = nnz_short / nonempty
    g = 2
    while g < 32 and g * vec < mean:
        g <<= 1
    tiles = (rows + nnz + MERGE_ITEMS - 1) // MERGE_ITEMS
    row_end = row_ptr[1:]
    tile_row = np.array([merge_path_row(row_end, nnz, min(t * MERGE_ITEMS, rows + nnz))
                         for t in range(tiles + 1)], dtype=np.int32)
    max_len = int(lens.max()) if rows > 0 else 0
    mean_all = nnz / rows if rows > 0 else 0.0
    variant = 0 if tiles < SMALL_PROBLEM_TILES else 1
    stats = dict(max_len=max_len, empty_rows=empty, num_short=n_short, num_medium=n_medium,
                 num_long=n_long, group_lanes=g, merge_items=MERGE_ITEMS, merge_tiles=tiles,
                 variant=variant, identity_short=int(n_short == rows), nnz_short=nnz_short, device_error=0)
    if col_idx is not None:
        stats["col_step"] = col_step(row_ptr, col_idx)
    return stats, bins, tile_row
