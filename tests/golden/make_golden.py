"""Generates tests/golden/csr_golden.npz and tests/golden/csr_golden_complex.npz by running the REFERENCE's own
hygon CSR mv / mm code (oracle/_ref/libasp_ref.so, built by `make -C oracle ref` from the mounted reference
tree) on small seeded inputs.  Inputs and the reference's outputs are both stored, so the
fixture pins the oracle restatement and the CUDA path on machines without the reference.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from library_b200 import generators as G  # noqa: E402


def cases():
    f32, f64 = torch.float32, torch.float64
    out = {}

    def add_mv(name, A, dtype, alpha, beta, xlo, xhi, seed):
        rp, ci, v = A.numpy()
        v = v.astype(np.float32 if dtype == f32 else np.float64)
        x = G.uniform((A.cols,), xlo, xhi, dtype=dtype, seed=seed).numpy()
        y0 = G.uniform((A.rows,), -1, 1, dtype=dtype, seed=seed + 100).numpy()
        y, _ = oracle.ref_spmv(rp, ci, v, x, alpha, beta, y0)
        out[name] = dict(kind="mv", rp=rp, ci=ci, v=v, x=x, y0=y0, alpha=alpha, beta=beta, y=y,
                         cols=A.cols)

    def add_mm(name, A, dtype, n, alpha, beta, seed):
        rp, ci, v = A.numpy()
        v = v.astype(np.float32 if dtype == f32 else np.float64)
        X = G.uniform((A.cols, n), -1, 1, dtype=dtype, seed=seed).numpy()
        Y0 = G.uniform((A.rows, n), -1, 1, dtype=dtype, seed=seed + 100).numpy()
        Y, _ = oracle.ref_spmm(rp, ci, v, X, alpha, beta, Y0)
        out[name] = dict(kind="mm", rp=rp, ci=ci, v=v, x=X, y0=Y0, alpha=alpha, beta=beta, y=Y,
                         cols=A.cols)

    add_mv("lap2d_32_f64", G.laplacian_2d_5pt(32), f64, 1.0, 0.0, -1, 1, 1)
    add_mv("lap2d_32_f64_ab", G.laplacian_2d_5pt(32), f64, 2.1, 3.2, -1, 1, 2)
    add_mv("poisson_3000_f32", G.poisson_random(3000, mean_len=16, seed=2), f32, 1.5, 0.5, -1, 1, 3)
    add_mv("poisson_3000_f64", G.poisson_random(3000, mean_len=16, seed=2, dtype=f64), f64, 1.5, 0.5, -1, 1, 3)
    add_mv("rmat_11_f32", G.rmat(11, 16, seed=3), f32, 1.0, 0.0, 0, 1, 4)
    add_mv("rmat_10_f64", G.rmat(10, 8, seed=5, dtype=f64), f64, -0.75, 1.25, 0, 1, 5)
    add_mv("lap3d_12_f64", G.laplacian_3d_7pt(12, index64=False), f64, 1.0, 0.0, -1, 1, 6)
    add_mv("rect_2000x700_f32", G.poisson_random(2000, 700, mean_len=5, seed=8), f32, 2.0, 3.0, -1, 1, 7)
    add_mm("s27_8_f32_n8", G.stencil_3d_27pt(8, seed=4), f32, 8, 1.0, 0.0, 9)
    add_mm("s27_8_f32_n32", G.stencil_3d_27pt(8, seed=4), f32, 32, 1.0, 0.0, 10)
    add_mm("s27_6_f32_n128", G.stencil_3d_27pt(6, seed=4), f32, 128, 1.0, 0.0, 11)
    add_mm("poisson_500_f32_n5", G.poisson_random(500, 300, mean_len=7, seed=12), f32, 5, 0.5, 2.0, 12)
    add_mm("rmat_9_f64_n12", G.rmat(9, 8, seed=13, dtype=f64), f64, 12, 1.5, -0.5, 13)
    return out


def complex_cases():
    """Complex mv / mm through the reference's alphasparse_{c,z}_mv and alphasparse_{c,z}_mm.  These pin the
    oracle's complex restatements within rounding (the reference's kernels unroll their sums), not bit for bit."""
    out = {}
    rng = np.random.default_rng(77)

    def cplx(shape, dtype):
        return (rng.uniform(-1, 1, shape) + 1j * rng.uniform(-1, 1, shape)).astype(dtype)

    mats = {"rmat_9": G.rmat(9, 8, seed=21), "lap2d_20": G.laplacian_2d_5pt(20),
            "poisson_400x300": G.poisson_random(400, 300, mean_len=6, seed=22)}
    for mname, A in mats.items():
        rp, ci, _ = A.numpy()
        for dtype, tag in ((np.complex64, "c32"), (np.complex128, "c64")):
            v = cplx(A.nnz, dtype)
            alpha, beta = 1.5 - 0.5j, 0.25 + 2.0j
            x, y0 = cplx(A.cols, dtype), cplx(A.rows, dtype)
            y = oracle.ref_spmv_complex(rp, ci, v, x, alpha, beta, y0, cols=A.cols)
            out[f"{mname}_{tag}_mv"] = dict(kind="mv", rp=rp, ci=ci, v=v, x=x, y0=y0, alpha=alpha, beta=beta, y=y,
                                            cols=A.cols)
            X, Y0 = cplx((A.cols, 7), dtype), cplx((A.rows, 7), dtype)
            Y = oracle.ref_spmm_complex(rp, ci, v, X, alpha, beta, Y0)
            out[f"{mname}_{tag}_mm"] = dict(kind="mm", rp=rp, ci=ci, v=v, x=X, y0=Y0, alpha=alpha, beta=beta, y=Y,
                                            cols=A.cols)
    return out


def save(name, cs):
    flat = {}
    for cname, c in cs.items():
        for k, val in c.items():
            flat[f"{cname}/{k}"] = np.asarray(val)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), name)
    np.savez_compressed(path, **flat)
    print(path, os.path.getsize(path), "bytes,", len(cs), "cases")


def main():
    if not oracle.have_ref():
        raise SystemExit("oracle/_ref/libasp_ref.so is missing: run `make -C oracle ref` first")
    oracle.ref_set_threads(4)
    save("csr_golden.npz", cases())
    save("csr_golden_complex.npz", complex_cases())


if __name__ == "__main__":
    main()
