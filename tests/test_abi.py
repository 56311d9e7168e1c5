"""The C-ABI library loads without a GPU and exports every function include/*.h declares;
descriptor creators (which make no CUDA call) validate their arguments like the reference's
(cuda/util/handle.cu:657-738)."""
import ctypes as C
import os
import re

import pytest

from library_b200 import api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    inc = os.path.join(ROOT, "include")
    for fn in sorted(os.listdir(inc)):
        if not fn.endswith(".h"):
            continue
        text = open(os.path.join(inc, fn)).read()
        text = text.split("#ifdef __cplusplus\n} /* extern \"C\" */")[0]  # C part only
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"^(?:alphasparseStatus_t|double|int64_t|void|const char\*)\s+(\w+)\s*\(", text, re.M):
            names.append(m.group(1))
    return names


def test_header_declares_the_hot_path_api():
    names = set(declared_functions())
    for must in ("alphasparseSpMV", "alphasparseSpMV_bufferSize", "alphasparseSpMM",
                 "alphasparseSpMM_bufferSize", "alphasparseCreateCsr", "alphasparseCreateDnVec",
                 "alphasparseCreateDnMat", "alphasparseGetHandle", "initHandle",
                 "alphasparse_destory_handle", "alphasparseSpMV_analysis", "alphasparseSpMM_preprocess"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = api.load()
    for name in declared_functions():
        assert hasattr(lib, name), name
    assert set(declared_functions()) == set(api.EXPORTS)


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(api, "_lib", None)
    monkeypatch.setattr(api, "LIB_PATH", "/nonexistent/libalphasparse_b200.so")
    with pytest.raises(ImportError):
        api.load()


def test_descriptor_argument_checks():
    lib = api.load()
    d = C.c_void_p()
    dummy = C.c_void_p(0x1000)  # never dereferenced by the creators
    assert lib.alphasparseCreateDnVec(None, C.c_int64(4), dummy, api.R_32F) == 7   # INVALID_POINTER
    assert lib.alphasparseCreateDnVec(C.byref(d), C.c_int64(-1), dummy, api.R_32F) == 10  # INVALID_SIZE
    assert lib.alphasparseCreateDnVec(C.byref(d), C.c_int64(4), None, api.R_32F) == 7
    assert lib.alphasparseCreateDnVec(C.byref(d), C.c_int64(0), None, api.R_32F) == 0
    lib.alphasparseDestroyDnVec(d)
    assert lib.alphasparseCreateDnMat(C.byref(d), C.c_int64(-2), C.c_int64(3), C.c_int64(3), dummy, api.R_32F, 0) == 10
    assert lib.alphasparseCreateDnMat(C.byref(d), C.c_int64(2), C.c_int64(3), C.c_int64(3), None, api.R_32F, 0) == 7
    assert lib.alphasparseCreateDnMat(C.byref(d), C.c_int64(2), C.c_int64(3), C.c_int64(2), dummy, api.R_32F, 0) == 10
    assert lib.alphasparseCreateDnMat(C.byref(d), C.c_int64(2), C.c_int64(3), C.c_int64(3), dummy, api.R_32F, 0) == 0
    lib.alphasparseDestroyDnMat(d)

    def csr(rows, cols, nnz, rp, ci, v, rt=api.INDEX_I32, ct=api.INDEX_I32, base=0, dt=api.R_32F):
        return lib.alphasparseCreateCsr(C.byref(d), C.c_int64(rows), C.c_int64(cols), C.c_int64(nnz),
                                        rp, ci, v, rt, ct, base, dt)
    assert csr(-1, 3, 0, dummy, dummy, dummy) == 10
    assert csr(3, 3, 2, None, dummy, dummy) == 7
    assert csr(3, 3, 2, dummy, None, dummy) == 7
    assert csr(3, 3, 2, dummy, dummy, dummy, base=1) == 6          # NOT_SUPPORTED
    assert csr(3, 3, 2, dummy, dummy, dummy, ct=api.INDEX_I64) == 6
    assert csr(3, 3, 2 ** 31, dummy, dummy, dummy) == 10           # does not fit 32-bit offsets
    assert csr(3, 3, 2 ** 31, dummy, dummy, dummy, rt=api.INDEX_I64) == 0
    lib.alphasparseDestroySpMat(d)
    assert csr(3, 3, 2, dummy, dummy, dummy, dt=6) == 6            # half-precision complex: no instance
    assert csr(3, 3, 2, dummy, dummy, dummy, dt=api.C_32F) == 0    # complex float has an SpMV instance
    lib.alphasparseDestroySpMat(d)
    assert csr(3, 3, 0, dummy, None, None) == 0                    # empty matrix needs no arrays
    lib.alphasparseDestroySpMat(d)


def test_null_handle_is_rejected_without_cuda():
    lib = api.load()
    one = C.c_float(1.0)
    size = C.c_size_t()
    assert lib.alphasparseSpMV(None, 0, C.byref(one), None, None, C.byref(one), None, 0, 0, None) == 8
    assert lib.alphasparseSpMM(None, 0, 0, C.byref(one), None, None, C.byref(one), None, 0, 0, None) == 8
    assert lib.alphasparseSpMV_bufferSize(None, 0, C.byref(one), None, None, C.byref(one), None, 0, 0,
                                          C.byref(size)) == 8
    assert lib.alphasparseSetStream(None, None) == 8


def test_outlier_filtered_mean():
    lib = api.load()
    arr = (C.c_double * 5)(1.0, 1.0, 1.0, 1.0, 100.0)
    assert abs(lib.get_avg_time_n(arr, 5) - 1.0) < 1e-12
