"""TEST INFRASTRUCTURE ONLY: ctypes access to the two CPU checkers.

* ``libasp_oracle.so``  - the plain-C restatement in ``csr_oracle.c`` (always buildable).
* ``_ref/libasp_ref.so`` - the reference's own hygon CSR mv/mm code behind ``ref_shim.cpp``
  (built by ``make -C oracle ref`` where the reference tree is mounted; the prebuilt file
  travels with the repository snapshot to machines that do not have the tree).

Only tests, the smoke check and the CPU-baseline / reference arm of the benchmark import
this package.  The CUDA library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_ORACLE_SO = os.path.join(_HERE, "libasp_oracle.so")
_REF_SO = os.path.join(_HERE, "_ref", "libasp_ref.so")

_oracle = None
_ref = None


def reference_root() -> str:
    """Where a checkout of the reference project lies: $ALPHASPARSE_REFERENCE, else a directory
    named ``reference`` beside this repository (it need not exist)."""
    return os.environ.get("ALPHASPARSE_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build(ref: bool = True) -> None:
    """Compile the restatement and, when the reference tree is present, the reference."""
    subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True)
    if ref:
        subprocess.run(["make", "-s", "-j8", "-C", _HERE, "ref", "REF=" + reference_root()], check=True)


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def lib():
    global _oracle
    if _oracle is None:
        if not os.path.exists(_ORACLE_SO):
            build(ref=False)
        _oracle = C.CDLL(_ORACLE_SO)
    return _oracle


def have_ref() -> bool:
    return os.path.exists(_REF_SO)


def ref_lib():
    global _ref
    if _ref is None:
        _ref = C.CDLL(_REF_SO)
        _ref.ref_get_threads.restype = C.c_int
    return _ref


def _off_suffix(row_ptr: np.ndarray) -> str:
    if row_ptr.dtype == np.int32:
        return "i32"
    if row_ptr.dtype == np.int64:
        return "i64"
    raise TypeError("row_ptr must be int32 or int64")


def spmv(row_ptr, col_idx, val, x, alpha, beta, y0=None):
    """y = alpha*A*x + beta*y0 with the restated hygon row arithmetic."""
    rows = row_ptr.shape[0] - 1
    row_ptr = np.ascontiguousarray(row_ptr)
    col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
    val = np.ascontiguousarray(val)
    x = np.ascontiguousarray(x, dtype=val.dtype)
    y = np.zeros(rows, dtype=val.dtype) if y0 is None else np.array(y0, dtype=val.dtype, copy=True)
    if val.dtype == np.float32:
        fn = getattr(lib(), "oracle_spmv_f32_" + _off_suffix(row_ptr))
        ft = C.c_float
    elif val.dtype == np.float64:
        fn = getattr(lib(), "oracle_spmv_f64_" + _off_suffix(row_ptr))
        ft = C.c_double
    else:
        raise TypeError(val.dtype)
    fn.restype = None
    fn(C.c_int64(rows), _p(row_ptr), _p(col_idx), _p(val), _p(x), ft(alpha), ft(beta), _p(y))
    return y


def spmv_complex(row_ptr, col_idx, val, x, alpha, beta, y0=None):
    """Complex y = alpha*A*x + beta*y0 (numpy complex64 / complex128 arrays, Python complex scalars)."""
    rows = row_ptr.shape[0] - 1
    row_ptr = np.ascontiguousarray(row_ptr)
    col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
    val = np.ascontiguousarray(val)
    x = np.ascontiguousarray(x, dtype=val.dtype)
    y = np.zeros(rows, dtype=val.dtype) if y0 is None else np.array(y0, dtype=val.dtype, copy=True)
    tn, rt = {np.dtype(np.complex64): ("c32", np.float32), np.dtype(np.complex128): ("c64", np.float64)}[val.dtype]
    a = np.array([complex(alpha).real, complex(alpha).imag], dtype=rt)
    b = np.array([complex(beta).real, complex(beta).imag], dtype=rt)
    fn = getattr(lib(), f"oracle_spmv_{tn}_" + _off_suffix(row_ptr))
    fn.restype = None
    fn(C.c_int64(rows), _p(row_ptr), _p(col_idx), _p(val), _p(x), _p(a), _p(b), _p(y))
    return y


def spmv_int8(row_ptr, col_idx, val, x, alpha, beta, y0):
    """int8 A and x; y0's dtype (int32 or float32) selects the instance (int32 or float arithmetic)."""
    rows = row_ptr.shape[0] - 1
    row_ptr = np.ascontiguousarray(row_ptr)
    col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
    val = np.ascontiguousarray(val, dtype=np.int8)
    x = np.ascontiguousarray(x, dtype=np.int8)
    y = np.array(y0, copy=True)
    if y.dtype == np.int32:
        fn, ct = getattr(lib(), "oracle_spmv_i8_i32_" + _off_suffix(row_ptr)), C.c_int32
    elif y.dtype == np.float32:
        fn, ct = getattr(lib(), "oracle_spmv_i8_f32_" + _off_suffix(row_ptr)), C.c_float
    else:
        raise TypeError(y.dtype)
    fn.restype = None
    fn(C.c_int64(rows), _p(row_ptr), _p(col_idx), _p(val), _p(x), ct(alpha), ct(beta), _p(y))
    return y


def spmm(row_ptr, col_idx, val, X, alpha, beta, Y0=None):
    """Row-major Y = alpha*A*X + beta*Y0.  ``val``/``X`` of dtype uint16 are bf16 bit patterns
    (fp32 accumulation and fp32 Y)."""
    rows = row_ptr.shape[0] - 1
    row_ptr = np.ascontiguousarray(row_ptr)
    col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
    val = np.ascontiguousarray(val)
    X = np.ascontiguousarray(X)
    n = X.shape[1]
    if val.dtype == np.uint16:
        Y = np.zeros((rows, n), np.float32) if Y0 is None else np.array(Y0, dtype=np.float32, copy=True)
        assert row_ptr.dtype == np.int32 and X.dtype == np.uint16
        fn = lib().oracle_spmm_bf16_i32
        ft = C.c_float
    else:
        X = X.astype(val.dtype, copy=False)
        Y = np.zeros((rows, n), val.dtype) if Y0 is None else np.array(Y0, dtype=val.dtype, copy=True)
        tn = {np.dtype(np.float32): "f32", np.dtype(np.float64): "f64"}[val.dtype]
        fn = getattr(lib(), f"oracle_spmm_{tn}_" + _off_suffix(row_ptr))
        ft = C.c_float if tn == "f32" else C.c_double
    fn.restype = None
    fn(C.c_int64(rows), _p(row_ptr), _p(col_idx), _p(val), _p(X), C.c_int64(n), C.c_int64(n),
       ft(alpha), ft(beta), _p(Y), C.c_int64(n))
    return Y


def spmm_complex(row_ptr, col_idx, val, X, alpha, beta, Y0=None):
    """Complex row-major Y = alpha*A*X + beta*Y0 (numpy complex64 / complex128, Python complex scalars)."""
    rows = row_ptr.shape[0] - 1
    row_ptr = np.ascontiguousarray(row_ptr)
    col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
    val = np.ascontiguousarray(val)
    X = np.ascontiguousarray(X, dtype=val.dtype)
    n = X.shape[1]
    Y = np.zeros((rows, n), val.dtype) if Y0 is None else np.array(Y0, dtype=val.dtype, copy=True)
    tn, rt = {np.dtype(np.complex64): ("c32", np.float32), np.dtype(np.complex128): ("c64", np.float64)}[val.dtype]
    a = np.array([complex(alpha).real, complex(alpha).imag], dtype=rt)
    b = np.array([complex(beta).real, complex(beta).imag], dtype=rt)
    fn = getattr(lib(), f"oracle_spmm_{tn}_" + _off_suffix(row_ptr))
    fn.restype = None
    fn(C.c_int64(rows), _p(row_ptr), _p(col_idx), _p(val), _p(X), C.c_int64(n), C.c_int64(n), _p(a), _p(b), _p(Y),
       C.c_int64(n))
    return Y


def spmm_wide(row_ptr, col_idx, val, X, alpha, beta, Y0):
    """int8 or fp16 A and X with a wider (or, for fp16, equal) Y: (int8, int32), (int8, float32), (float16, float32),
    (float16, float16).  Y0's dtype selects the instance; float16 arrays travel as their bit patterns."""
    rows = row_ptr.shape[0] - 1
    row_ptr = np.ascontiguousarray(row_ptr)
    col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
    val = np.ascontiguousarray(val)
    X = np.ascontiguousarray(X, dtype=val.dtype)
    n = X.shape[1]
    Y = np.array(Y0, copy=True, order="C")
    key = (val.dtype, Y.dtype)
    name, ct = {(np.dtype(np.int8), np.dtype(np.int32)): ("i8_i32", C.c_int32),
                (np.dtype(np.int8), np.dtype(np.float32)): ("i8_f32", C.c_float),
                (np.dtype(np.float16), np.dtype(np.float32)): ("f16_f32", C.c_float),
                (np.dtype(np.float16), np.dtype(np.float16)): ("f16_f16", C.c_float)}[key]
    fn = getattr(lib(), f"oracle_spmm_{name}_" + _off_suffix(row_ptr))
    fn.restype = None
    fn(C.c_int64(rows), _p(row_ptr), _p(col_idx), _p(val), _p(X), C.c_int64(n), C.c_int64(n), ct(alpha), ct(beta),
       _p(Y), C.c_int64(n))
    return Y


def partition_rows_by_nnz(row_ptr, parts: int) -> np.ndarray:
    row_ptr = np.ascontiguousarray(row_ptr)
    rows = row_ptr.shape[0] - 1
    out = np.zeros(parts + 1, dtype=np.int64)
    fn = getattr(lib(), "oracle_partition_rows_by_nnz_" + _off_suffix(row_ptr))
    fn.restype = None
    fn(_p(row_ptr), C.c_int64(rows), C.c_int64(parts), _p(out))
    return out


# ---- the reference's own code (int32 only) ---------------------------------------------

def ref_set_threads(n: int) -> None:
    """Threads of the reference's OpenMP regions: its own setting, the environment variable it re-reads
    on every call (hygon/util/thread.cpp:32-42) and the OpenMP runtime's default (a torchrun launch
    starts the process with OMP_NUM_THREADS=1)."""
    os.environ["OMP_NUM_THREADS"] = str(n)
    lib = ref_lib()
    lib.ref_set_threads(C.c_int(n))
    try:
        lib.omp_set_num_threads(C.c_int(n))   # resolved through the library's dependency on libgomp
    except AttributeError:
        pass


def ref_threads() -> int:
    return int(ref_lib().ref_get_threads())


def ref_spmv(row_ptr, col_idx, val, x, alpha, beta, y0=None, cols=None, repeats=1):
    """The reference's alphasparse_{s,d}_mv.  Returns (y, per-call seconds)."""
    rows = row_ptr.shape[0] - 1
    cols = int(x.shape[0]) if cols is None else cols
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
    col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
    val = np.ascontiguousarray(val)
    x = np.ascontiguousarray(x, dtype=val.dtype)
    y = np.zeros(rows, dtype=val.dtype) if y0 is None else np.array(y0, dtype=val.dtype, copy=True)
    times = np.zeros(max(1, repeats), dtype=np.float64)
    if val.dtype == np.float32:
        fn, ft = ref_lib().ref_s_mv, C.c_float
    else:
        fn, ft = ref_lib().ref_d_mv, C.c_double
    fn.restype = C.c_int
    st = fn(C.c_int(rows), C.c_int(cols), _p(row_ptr), _p(col_idx), _p(val), _p(x), ft(alpha),
            ft(beta), _p(y), C.c_int(repeats), _p(times))
    if st != 0:
        raise RuntimeError(f"reference mv returned status {st}")
    return y, times


def ref_spmv_complex(row_ptr, col_idx, val, x, alpha, beta, y0=None, cols=None):
    """The reference's alphasparse_{c,z}_mv."""
    rows = row_ptr.shape[0] - 1
    cols = int(x.shape[0]) if cols is None else cols
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
    col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
    val = np.ascontiguousarray(val)
    x = np.ascontiguousarray(x, dtype=val.dtype)
    y = np.zeros(rows, dtype=val.dtype) if y0 is None else np.array(y0, dtype=val.dtype, copy=True)
    fn, rt = (ref_lib().ref_c_mv, np.float32) if val.dtype == np.complex64 else (ref_lib().ref_z_mv, np.float64)
    a = np.array([complex(alpha).real, complex(alpha).imag], dtype=rt)
    b = np.array([complex(beta).real, complex(beta).imag], dtype=rt)
    fn.restype = C.c_int
    st = fn(C.c_int(rows), C.c_int(cols), _p(row_ptr), _p(col_idx), _p(val), _p(x), _p(a), _p(b), _p(y))
    if st != 0:
        raise RuntimeError(f"reference complex mv returned status {st}")
    return y


def ref_spmm(row_ptr, col_idx, val, X, alpha, beta, Y0=None, repeats=1):
    """The reference's alphasparse_{s,d}_mm, row-major.  Returns (Y, per-call seconds)."""
    rows = row_ptr.shape[0] - 1
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
    col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
    val = np.ascontiguousarray(val)
    X = np.ascontiguousarray(X, dtype=val.dtype)
    cols, n = X.shape
    Y = np.zeros((rows, n), val.dtype) if Y0 is None else np.array(Y0, dtype=val.dtype, copy=True)
    times = np.zeros(max(1, repeats), dtype=np.float64)
    if val.dtype == np.float32:
        fn, ft = ref_lib().ref_s_mm, C.c_float
    else:
        fn, ft = ref_lib().ref_d_mm, C.c_double
    fn.restype = C.c_int
    st = fn(C.c_int(rows), C.c_int(cols), _p(row_ptr), _p(col_idx), _p(val), _p(X), C.c_int(n),
            C.c_int(n), ft(alpha), ft(beta), _p(Y), C.c_int(n), C.c_int(repeats), _p(times))
    if st != 0:
        raise RuntimeError(f"reference mm returned status {st}")
    return Y, times


def ref_spmm_complex(row_ptr, col_idx, val, X, alpha, beta, Y0=None):
    """The reference's alphasparse_{c,z}_mm, row-major."""
    rows = row_ptr.shape[0] - 1
    row_ptr = np.ascontiguousarray(row_ptr, dtype=np.int32)
    col_idx = np.ascontiguousarray(col_idx, dtype=np.int32)
    val = np.ascontiguousarray(val)
    X = np.ascontiguousarray(X, dtype=val.dtype)
    cols, n = X.shape
    Y = np.zeros((rows, n), val.dtype) if Y0 is None else np.array(Y0, dtype=val.dtype, copy=True)
    fn, rt = (ref_lib().ref_c_mm, np.float32) if val.dtype == np.complex64 else (ref_lib().ref_z_mm, np.float64)
    a = np.array([complex(alpha).real, complex(alpha).imag], dtype=rt)
    b = np.array([complex(beta).real, complex(beta).imag], dtype=rt)
    fn.restype = C.c_int
    st = fn(C.c_int(rows), C.c_int(cols), _p(row_ptr), _p(col_idx), _p(val), _p(X), C.c_int(n), C.c_int(n), _p(a),
            _p(b), _p(Y), C.c_int(n))
    if st != 0:
        raise RuntimeError(f"reference complex mm returned status {st}")
    return Y
