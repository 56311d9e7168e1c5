"""The drop-in boundary proved with compiled callers: two C++ programs (tests/abi_caller/) that make
the reference test drivers' call sequence against include/alphasparse_b200.h - template creators,
handle->stream, buffer-size query, the timers - are compiled and linked against the library (CPU
test), then run on a GPU with their result compared with the CPU oracle (GPU test).
"""
import os
import shutil
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "abi_caller")
OUT = os.path.join(ROOT, "tests", "abi_caller", "build")
LIBDIR = os.path.join(ROOT, "library_b200")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def build_caller(name):
    """g++ only: a caller needs the header, the CUDA runtime API and the shared library."""
    os.makedirs(OUT, exist_ok=True)
    exe = os.path.join(OUT, name)
    src = os.path.join(SRC, name + ".cpp")
    deps = [src, os.path.join(SRC, "caller_io.h"), os.path.join(ROOT, "include", "alphasparse_b200.h"),
            os.path.join(LIBDIR, "libalphasparse_b200.so")]
    if os.path.exists(exe) and all(os.path.getmtime(d) <= os.path.getmtime(exe) for d in deps):
        return exe
    cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"),
           src, "-o", exe, "-L", LIBDIR, "-lalphasparse_b200", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath," + LIBDIR, "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return exe


def have_toolchain():
    return shutil.which("g++") and os.path.exists(os.path.join(CUDA, "include", "cuda_runtime.h"))


@pytest.mark.parametrize("name", ["spmv_caller", "spmm_caller"])
def test_callers_compile_and_link_against_the_header(name):
    if not have_toolchain():
        pytest.skip("needs g++ and the CUDA runtime headers")
    exe = build_caller(name)
    assert os.path.exists(exe)
    # without arguments the program leaves before touching CUDA: it loads, so every symbol it uses resolved
    assert subprocess.run([exe], capture_output=True).returncode == 1


def _write_input(path, kind, A, dense_in, dense_out, alpha, beta, n):
    rp, ci, v = A.numpy()
    rows = np.repeat(np.arange(A.rows, dtype=np.int32), np.diff(rp))
    with open(path, "wb") as f:
        np.array([kind, A.rows, A.cols, A.nnz, n, 0], dtype=np.int64).tofile(f)
        np.array([alpha, beta], dtype=np.float32).tofile(f)
        rows.tofile(f)
        ci.astype(np.int32).tofile(f)
        v.astype(np.float32).tofile(f)
        dense_in.astype(np.float32).tofile(f)
        dense_out.astype(np.float32).tofile(f)


@pytest.mark.gpu
def test_spmv_caller_result_equals_the_oracle(tmp_path):
    if not have_toolchain():
        pytest.skip("needs g++ and the CUDA runtime headers")
    import oracle
    from conftest import rel_l2
    from library_b200 import generators as G
    exe = build_caller("spmv_caller")
    for A in (G.rmat(14, 16, seed=31), G.poisson_random(3000, 2500, 7.0, seed=32)):     # the second one: rows != cols
        rp, ci, v = A.numpy()
        x = G.uniform((A.cols,), -1, 1, seed=33).numpy()
        y0 = G.uniform((A.rows,), -1, 1, seed=34).numpy()
        _write_input(tmp_path / "in.bin", 0, A, x, y0, 1.5, 0.5, 1)
        r = subprocess.run([exe, str(tmp_path / "in.bin"), str(tmp_path / "out.bin")], capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        assert "alphasparse:" in r.stdout
        got = np.fromfile(tmp_path / "out.bin", dtype=np.float32)
        want = oracle.spmv(rp, ci, v, x, 1.5, 0.5, y0)
        assert got.shape == want.shape and rel_l2(got, want) <= 1e-5


@pytest.mark.gpu
def test_spmm_caller_result_equals_the_oracle(tmp_path):
    if not have_toolchain():
        pytest.skip("needs g++ and the CUDA runtime headers")
    import oracle
    from library_b200 import generators as G
    exe = build_caller("spmm_caller")
    A = G.stencil_3d_27pt(12, seed=35)
    rp, ci, v = A.numpy()
    n = 32
    B = G.uniform((A.cols, n), -1, 1, seed=36).numpy()
    C0 = G.uniform((A.rows, n), -1, 1, seed=37).numpy()
    _write_input(tmp_path / "in.bin", 1, A, B, C0, 2.0, 0.5, n)
    r = subprocess.run([exe, str(tmp_path / "in.bin"), str(tmp_path / "out.bin")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    got = np.fromfile(tmp_path / "out.bin", dtype=np.float32).reshape(A.rows, n)
    want = oracle.spmm(rp, ci, v, B, 2.0, 0.5, C0)
    # the caller passes CSR_ALG2 as the reference's driver does: the merge-path kernel, equal within rounding
    from conftest import rel_l2
    assert got.shape == want.shape and rel_l2(got, want) <= 1e-5
