"""Row sharding of one CSR matrix across ranks (one process per GPU): the harness side.

Rows are split into contiguous ranges of near-equal nnz by the C ABI call
alphasparseCsrPartitionRowsByNnz (the rule of the reference's CPU partitioner,
hygon/util/partition.cpp:83-96, in 64-bit).  A shard keeps global column indices, its own
rebased row offsets (32-bit when the shard's nnz allows) and the matching slices of the column
and value arrays; y stays sharded by rows.

On GPUs the exchange of x and the product run behind the C ABI (alphasparseMg*, api.Mg).  What
is left here: ``shard_csr`` (cutting one device-resident matrix into this rank's shard), and
Python twins of the library's host-side planning - ``partition_bounds_host``, ``exchange_plan``,
``interior_row_range`` and ``XWindowExchange`` over torch.distributed - which the CPU tests run
on gloo ranks and compare with the library's own answers.
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


WINDOW_ALIGN = 32  # the window starts on a multiple of this many elements (keeps 128-byte alignment)


def exchange_plan(own_bounds, windows, rank: int):
    """Who sends what for the column-window exchange.  ``own_bounds`` (world + 1 ascending integers):
    rank p owns x[own_bounds[p], own_bounds[p+1]).  ``windows`` (world pairs): rank p needs
    x[lo_p, hi_p) (hi_p <= lo_p: nothing).  Returns (sends, recvs) for ``rank``:
    sends = [(peer, a, b)]: x[a, b) of this rank's own part goes to peer;
    recvs = [(peer, a, b)]: x[a, b) arrives from peer.  Global element indices, peers ascending,
    the rank's own overlap listed as a copy to itself (peer == rank)."""
    world = len(windows)
    my_lo, my_hi = int(own_bounds[rank]), int(own_bounds[rank + 1])
    w_lo, w_hi = int(windows[rank][0]), int(windows[rank][1])
    sends, recvs = [], []
    for p in range(world):
        a, b = max(my_lo, int(windows[p][0])), min(my_hi, int(windows[p][1]))
        if b > a:
            sends.append((p, a, b))
        a, b = max(w_lo, int(own_bounds[p])), min(w_hi, int(own_bounds[p + 1]))
        if b > a:
            recvs.append((p, a, b))
    return sends, recvs


class XWindowExchange:
    """x sharded like y (rank p owns x[own_bounds[p], own_bounds[p+1])); before each SpMV a rank
    fills a buffer holding x[lo, hi), the column window of its shard, from the owners.  Peers
    exchange with point-to-point sends (NCCL over NVLink on GPUs, gloo on CPU), the own part is a
    local copy.  For a banded matrix the traffic is the halo, not the vector."""

    def __init__(self, own_bounds, col_min: int, col_max: int, rank: int, world: int, dtype, device,
                 group=None):
        import torch.distributed as dist
        self.rank, self.world, self.group = rank, world, group
        self.own_bounds = [int(b) for b in own_bounds]
        lo = (col_min // WINDOW_ALIGN) * WINDOW_ALIGN if col_max >= col_min else 0
        hi = col_max + 1 if col_max >= col_min else 0
        self.lo, self.hi = lo, hi
        mine = torch.tensor([lo, hi], dtype=torch.int64)
        if world > 1:
            # windows of all ranks (two integers each); NCCL needs device tensors
            t = mine.to(device) if dist.get_backend(group) == "nccl" else mine
            allw = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(allw, t, group=group)
            self.windows = [(int(w[0]), int(w[1])) for w in allw]
        else:
            self.windows = [(lo, hi)]
        self.sends, self.recvs = exchange_plan(self.own_bounds, self.windows, rank)
        self.window = torch.empty(max(hi - lo, 0), dtype=dtype, device=device)
        self.bytes_received = sum(b - a for p, a, b in self.recvs if p != rank) * self.window.element_size()

    def own_view(self) -> torch.Tensor:
        """The part of the window that holds this rank's own elements of x (those inside the window):
        a caller that keeps its x there (``run(own_view())``) spares the local copy of every step.
        Element i of the view is x[max(lo, own_lo) + i]."""
        o0, o1 = self.own_bounds[self.rank], self.own_bounds[self.rank + 1]
        a, b = max(o0, self.lo), min(o1, self.hi)
        return self.window[a - self.lo:max(b, a) - self.lo]

    def _own_in_place(self, x_own: torch.Tensor) -> bool:
        v = self.own_view()
        return v.numel() > 0 and x_own.data_ptr() == v.data_ptr() and x_own.numel() == v.numel()

    def run(self, x_own: torch.Tensor) -> torch.Tensor:
        """x_own = this rank's part of x, or own_view() when x is kept inside the window.  Returns the
        window buffer (element i is x[lo + i]).  Ordered on the current stream."""
        import torch.distributed as dist
        o0 = self.own_bounds[self.rank]
        in_place = self._own_in_place(x_own)
        if in_place:
            o0 = max(o0, self.lo)      # the view starts at the first own element inside the window
        ops = []
        for p, a, b in self.recvs:
            if p == self.rank:
                if not in_place:
                    self.window[a - self.lo:b - self.lo].copy_(x_own[a - o0:b - o0])
            else:
                ops.append(dist.P2POp(dist.irecv, self.window[a - self.lo:b - self.lo], p, group=self.group))
        for p, a, b in self.sends:
            if p != self.rank:
                ops.append(dist.P2POp(dist.isend, x_own[a - o0:b - o0], p, group=self.group))
        if ops:
            for r in dist.batch_isend_irecv(ops):
                r.wait()
        return self.window


def interior_row_range(row_ptr: torch.Tensor, col_idx: torch.Tensor, own_lo: int, own_hi: int, align: int = 1):
    """Rows [i0, i1) of a shard (local CSR, ascending global columns inside a row) all of whose
    columns lie in [own_lo, own_hi): they need nothing from other ranks.  The largest such range that
    is one contiguous run starting at the first interior row; (0, 0) when there is none.  With
    ``align`` > 1 (the library uses 4) a cut that is not the shard's first or last row moves inwards,
    by at most 4095 rows, to a row whose first entry's index is a multiple of ``align`` - the slices of
    the entry arrays then start on a 16-byte boundary; (0, 0) if there is no such row.  Works on host
    or device tensors."""
    n = row_ptr.numel() - 1
    if n <= 0 or col_idx.numel() == 0:
        return 0, 0
    rp = row_ptr.to(torch.int64)
    empty = rp[1:] == rp[:-1]
    first = col_idx[torch.clamp(rp[:-1], max=col_idx.numel() - 1)].to(torch.int64)
    last = col_idx[torch.clamp(rp[1:] - 1, min=0)].to(torch.int64)
    inside = empty | ((first >= own_lo) & (last < own_hi))
    idx = torch.nonzero(inside).flatten()
    if idx.numel() == 0:
        return 0, 0
    i0 = int(idx[0])
    rest = torch.nonzero(~inside[i0:]).flatten()
    i1 = i0 + (int(rest[0]) if rest.numel() else n - i0)
    if align > 1 and i1 > i0:
        look = 4096
        c0, c1 = i0, i1
        if i0 > 0:
            w = rp[i0:min(i0 + look, n + 1)] % align == 0
            hit = torch.nonzero(w).flatten()
            c0 = i0 + int(hit[0]) if hit.numel() else -1
        if i1 < n:
            a = max(i1 - look + 1, 0)
            w = rp[a:i1 + 1] % align == 0
            hit = torch.nonzero(w).flatten()
            c1 = a + int(hit[-1]) if hit.numel() else -1
        if c0 < 0 or c1 < 0 or c1 <= c0:
            return 0, 0
        i0, i1 = c0, c1
    return i0, i1
