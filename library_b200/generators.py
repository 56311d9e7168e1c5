"""Seeded synthetic CSR matrices with the shapes and value distributions of the benchmark
configurations (they stand in for the SuiteSparse sweep the reference's scripts use,
tool/run_florida.sh:1-17; nothing from that collection is reproduced).

Everything is built with torch tensor ops on the requested device, so the same code makes
the small CPU test cases and the full-size inputs directly in HBM.  A given (seed, device
type) always yields the same matrix; CPU and CUDA streams differ, which is why parity tests
copy the generated arrays to the host for the oracle instead of regenerating them.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass
class Csr:
    rows: int
    cols: int
    row_ptr: torch.Tensor  # int32 or int64, rows+1
    col_idx: torch.Tensor  # int32, nnz, ascending inside each row
    val: torch.Tensor      # nnz

    @property
    def nnz(self) -> int:
        return int(self.col_idx.numel())

    def to(self, device) -> "Csr":
        return Csr(self.rows, self.cols, self.row_ptr.to(device), self.col_idx.to(device),
                   self.val.to(device))

    def numpy(self):
        return (self.row_ptr.cpu().numpy(), self.col_idx.cpu().numpy(), self.val.cpu().numpy())


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def _row_ptr_from_counts(counts: torch.Tensor, index64: bool) -> torch.Tensor:
    rp = torch.zeros(counts.numel() + 1, dtype=torch.int64, device=counts.device)
    torch.cumsum(counts, 0, out=rp[1:])
    if not index64:
        assert int(rp[-1]) < 2 ** 31, "nnz needs 64-bit row offsets"
        rp = rp.to(torch.int32)
    return rp


def stencil(dims, offsets, weights=None, *, dtype=torch.float64, device="cpu", seed=None,
            index64=False, chunk_rows=1 << 24) -> Csr:
    """Finite-difference style stencil on a regular grid with truncated (Dirichlet) borders.

    ``dims`` = (nx,) / (nx, ny) / (nx, ny, nz); grid point (x, y, z) is row x + nx*(y + ny*z).
    ``offsets`` = list of (dx, dy, dz).  Values: ``weights[k]`` per offset, or N(0,1) from
    ``seed`` when ``weights`` is None.  Columns come out ascending in every row.
    """
    dims = tuple(dims) + (1,) * (3 - len(dims))
    nx, ny, nz = dims
    rows = nx * ny * nz
    offs = [tuple(o) + (0,) * (3 - len(o)) for o in offsets]
    flat = [dx + nx * (dy + ny * dz) for dx, dy, dz in offs]
    order = sorted(range(len(offs)), key=lambda k: flat[k])
    offs = [offs[k] for k in order]
    flat_t = torch.tensor([flat[k] for k in order], dtype=torch.int64, device=device)
    w_t = None
    if weights is not None:
        w_t = torch.tensor([weights[k] for k in order], dtype=dtype, device=device)
    dxs = torch.tensor([o[0] for o in offs], dtype=torch.int64, device=device)
    dys = torch.tensor([o[1] for o in offs], dtype=torch.int64, device=device)
    dzs = torch.tensor([o[2] for o in offs], dtype=torch.int64, device=device)

    counts, cols, vals = [], [], []
    for r0 in range(0, rows, chunk_rows):
        r = torch.arange(r0, min(rows, r0 + chunk_rows), dtype=torch.int64, device=device)
        x = (r % nx)[:, None]
        y = ((r // nx) % ny)[:, None]
        z = (r // (nx * ny))[:, None]
        ok = ((x + dxs >= 0) & (x + dxs < nx) & (y + dys >= 0) & (y + dys < ny)
              & (z + dzs >= 0) & (z + dzs < nz))
        counts.append(ok.sum(1))
        cols.append((r[:, None] + flat_t)[ok].to(torch.int32))
        if w_t is not None:
            vals.append(w_t.expand(ok.shape)[ok])
        del x, y, z, ok
    col_idx = torch.cat(cols)
    del cols
    row_ptr = _row_ptr_from_counts(torch.cat(counts), index64)
    if w_t is not None:
        val = torch.cat(vals)
    else:
        val = torch.randn(col_idx.numel(), dtype=dtype, device=device,
                          generator=_gen(seed if seed is not None else 0, device))
    return Csr(rows, rows, row_ptr, col_idx, val)


def laplacian_2d_5pt(n=256, *, dtype=torch.float64, device="cpu") -> Csr:
    """5-point Laplacian on an n x n grid: diagonal 4, off-diagonals -1."""
    offs = [(0, 0), (-1, 0), (1, 0), (0, -1), (0, 1)]
    return stencil((n, n), offs, [4.0, -1.0, -1.0, -1.0, -1.0], dtype=dtype, device=device)


def laplacian_3d_7pt(n=512, *, dtype=torch.float64, device="cpu", index64=True) -> Csr:
    """7-point Laplacian on an n^3 grid: diagonal 6, off-diagonals -1."""
    offs = [(0, 0, 0), (-1, 0, 0), (1, 0, 0), (0, -1, 0), (0, 1, 0), (0, 0, -1), (0, 0, 1)]
    return stencil((n, n, n), offs, [6.0] + [-1.0] * 6, dtype=dtype, device=device,
                   index64=index64, chunk_rows=1 << 23)


def stencil_3d_27pt(n=128, *, dtype=torch.float32, device="cpu", seed=4) -> Csr:
    """27-point stencil pattern on an n^3 grid with N(0,1) values."""
    offs = [(dx, dy, dz) for dz in (-1, 0, 1) for dy in (-1, 0, 1) for dx in (-1, 0, 1)]
    return stencil((n, n, n), offs, None, dtype=dtype, device=device, seed=seed,
                   chunk_rows=1 << 21)


def _csr_from_keys(keys: torch.Tensor, rows: int, cols: int, index64: bool):
    """Sorted unique (row*cols+col) keys -> row_ptr, col_idx."""
    keys = torch.unique(keys, sorted=True)
    r = torch.div(keys, cols, rounding_mode="floor")
    col_idx = (keys - r * cols).to(torch.int32)
    counts = torch.bincount(r, minlength=rows)
    return _row_ptr_from_counts(counts, index64), col_idx


def poisson_random(rows, cols=None, mean_len=16.0, *, dtype=torch.float32, device="cpu",
                   seed=2, index64=False) -> Csr:
    """Row lengths ~ Poisson(mean_len); columns uniform over [0, cols), distinct and ascending
    inside a row (a duplicate draw inside a row is dropped, which shortens about
    mean_len^2 / (2*cols) of the rows by one); values ~ N(0,1)."""
    cols = rows if cols is None else cols
    g = _gen(seed, device)
    lens = torch.poisson(torch.full((rows,), float(mean_len), device=device), generator=g)
    lens = lens.to(torch.int64).clamp_(max=cols)
    r = torch.repeat_interleave(torch.arange(rows, dtype=torch.int64, device=device), lens)
    c = torch.randint(0, cols, (r.numel(),), dtype=torch.int64, device=device, generator=g)
    keys = r * cols + c
    del r, c
    row_ptr, col_idx = _csr_from_keys(keys, rows, cols, index64)
    val = torch.randn(col_idx.numel(), dtype=dtype, device=device, generator=g)
    return Csr(rows, cols, row_ptr, col_idx, val)


def rmat(scale, edge_factor=16, probs=(0.57, 0.19, 0.19, 0.05), *, dtype=torch.float32,
         device="cpu", seed=3, index64=False, chunk_edges=1 << 26) -> Csr:
    """R-MAT graph: edge_factor * 2^scale recursive-quadrant draws with probabilities
    (a, b, c, d), no vertex permutation, duplicate edges merged, self-loops kept,
    values ~ U(0,1)."""
    n = 1 << scale
    a, b, c, _ = probs
    g = _gen(seed, device)
    total = edge_factor * n
    parts = []
    for e0 in range(0, total, chunk_edges):
        m = min(chunk_edges, total - e0)
        r = torch.zeros(m, dtype=torch.int64, device=device)
        cidx = torch.zeros(m, dtype=torch.int64, device=device)
        for _level in range(scale):
            u = torch.rand(m, device=device, generator=g)
            down = u >= (a + b)                      # quadrants c, d: lower half (row bit 1)
            right = ((u >= a) & (u < a + b)) | (u >= a + b + c)   # quadrants b, d
            r = r * 2 + down
            cidx = cidx * 2 + right
        parts.append(torch.unique(r * n + cidx))
        del r, cidx, u, down, right
    keys = torch.cat(parts) if len(parts) > 1 else parts[0]
    del parts
    row_ptr, col_idx = _csr_from_keys(keys, n, n, index64)
    del keys
    val = torch.rand(col_idx.numel(), dtype=dtype, device=device, generator=g)
    return Csr(n, n, row_ptr, col_idx, val)


def uniform(shape, lo, hi, *, dtype=torch.float32, device="cpu", seed=0) -> torch.Tensor:
    """Dense operand ~ U(lo, hi)."""
    t = torch.rand(shape, dtype=torch.float32 if dtype == torch.bfloat16 else dtype,
                   device=device, generator=_gen(seed, device))
    t = t * (hi - lo) + lo
    return t.to(dtype)


def spmv_bytes(rows, cols, nnz, val_bytes, off_bytes, beta_nonzero) -> int:
    """Algorithmic bytes of one y = alpha*A*x + beta*y: every array touched once."""
    return (nnz * (val_bytes + 4) + (rows + 1) * off_bytes + cols * val_bytes
            + rows * val_bytes * (2 if beta_nonzero else 1))


def spmm_bytes(rows, cols, nnz, n, val_bytes, off_bytes, x_bytes, y_bytes, beta_nonzero) -> int:
    """Algorithmic bytes of one Y = alpha*A*X + beta*Y with an n-column dense operand."""
    return (nnz * (val_bytes + 4) + (rows + 1) * off_bytes + cols * n * x_bytes
            + rows * n * y_bytes * (2 if beta_nonzero else 1))
