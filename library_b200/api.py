"""ctypes bindings of libalphasparse_b200.so plus thin torch-tensor conveniences.

The functions in ``lib`` are the C ABI declared in include/alphasparse_b200.h, bound one to
one.  The classes below only hold descriptors and device pointers of torch tensors (torch is
the allocator and stream provider here, nothing more).  There is no fallback: if the shared
library is missing or a call returns a non-zero status, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libalphasparse_b200.so")

# enums (include/alphasparse_b200.h)
STATUS_SUCCESS = 0
STATUS_NAMES = {
    0: "SUCCESS", 1: "NOT_INITIALIZED", 2: "ALLOC_FAILED", 3: "INVALID_VALUE",
    4: "EXECUTION_FAILED", 5: "INTERNAL_ERROR", 6: "NOT_SUPPORTED", 7: "INVALID_POINTER",
    8: "INVALID_HANDLE", 9: "INVALID_KERNEL_PARAM", 10: "INVALID_SIZE",
}
OP_N, OP_T, OP_C = 0, 1, 2
ORDER_ROW, ORDER_COL = 0, 1
R_32F, R_64F, C_32F, C_64F, R_16F, R_16BF, R_8I, R_32I = 0, 1, 2, 3, 4, 5, 8, 9
INDEX_I32, INDEX_I64 = 2, 3
BASE_ZERO, BASE_ONE = 0, 1
SPMV_ALG_DEFAULT, SPMV_ALG_COO, SPMV_ALG_VECTOR, SPMV_ALG_MERGE = 0, 1, 6, 9
SPMM_ALG_DEFAULT, SPMM_CSR_ALG1, SPMM_CSR_ALG2, SPMM_CSR_ALG3, SPMM_CSR_ALG4, SPMM_CSR_ALG5, SPMM_CSR_ALG6 = 0, 5, 6, 7, 8, 9, 10
MG_X_BROADCAST, MG_X_ALLGATHER, MG_X_WINDOW, MG_X_WINDOW_OVERLAP = 0, 1, 2, 3
MG_INFO_NAMES = ["window_lo", "window_hi", "bytes_received", "interior_begin", "interior_end", "num_sends",
                 "num_recvs", "mode"]
STAT_NAMES = ["max_len", "empty_rows", "num_short", "num_medium", "num_long", "group_lanes",
              "merge_items", "merge_tiles", "variant", "identity_short", "nnz_short", "device_error", "col_step"]

EXPORTS = [
    "initHandle", "alphasparseGetHandle", "alphasparse_destory_handle", "alphasparseSetStream",
    "alphasparseGetStream", "alphasparseCreateCsr", "alphasparseCreateDnVec",
    "alphasparseCreateDnMat", "alphasparseDestroySpMat", "alphasparseDestroyDnVec",
    "alphasparseDestroyDnMat", "alphasparseDnVecSetValues", "alphasparseDnMatSetValues",
    "alphasparseSpMV", "alphasparseSpMV_bufferSize", "alphasparseSpMV_analysis",
    "alphasparseSpMV_clear", "alphasparseSpMV_clearMat", "alphasparseSpMM",
    "alphasparseSpMM_bufferSize", "alphasparseSpMM_preprocess",
    "alphasparseCsrPartitionRowsByNnz", "alphasparseCsrRebaseRowOffsets", "alphasparseCsrPlanGet",
    "alphasparseCsrLastVariant", "alphasparseCsrLastSpmmVariant", "alphasparseGetLaunchCount", "get_time_us", "get_avg_time_n",
    "alphasparseSpMVCsrNoAlloc", "alphasparseXcoo2csr", "alphasparseCsrColumnRange",
    "alphasparseCreateDnVecWindow", "alphasparseReadMtxCoo", "alphasparseReadBinCoo", "alphasparseFreeHost", "alphasparseCooOrder",
    "alphasparseMgCreate", "alphasparseMgDestroy", "alphasparseMgSetShard", "alphasparseMgSpMV",
    "alphasparseMgExchange", "alphasparseMgOwnView", "alphasparseMgGetInfo", "alphasparseMgExchangePlan",
    "alphasparseMgGetUniqueId", "alphasparseMgCommInitRank", "alphasparseMgCommDestroy",
]


class AlphaSparseError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: ALPHA_SPARSE_STATUS_{STATUS_NAMES.get(status, status)}")


_lib = None


def load():
    """Load the CUDA library.  Raises if it has not been built (python -m library_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python library_b200/build.py` "
                              "(there is no CPU or PyTorch fallback)")
        lib = C.CDLL(LIB_PATH)
        for name in EXPORTS:
            getattr(lib, name)  # AttributeError if a declared symbol is not exported
        lib.alphasparseCsrLastVariant.restype = C.c_char_p
        lib.alphasparseCsrLastSpmmVariant.restype = C.c_char_p
        lib.alphasparseGetLaunchCount.restype = C.c_int64
        lib.get_time_us.restype = C.c_double
        lib.get_avg_time_n.restype = C.c_double
        _lib = lib
    return _lib


def _check(st: int, where: str):
    if st != STATUS_SUCCESS:
        raise AlphaSparseError(st, where)


def _dtype_code(dt: torch.dtype) -> int:
    return {torch.float32: R_32F, torch.float64: R_64F, torch.bfloat16: R_16BF, torch.float16: R_16F,
            torch.complex64: C_32F, torch.complex128: C_64F, torch.int8: R_8I, torch.int32: R_32I}[dt]


def _spmv_compute_code(dt: torch.dtype) -> int:
    """16-bit matrices are multiplied in fp32 (alpha and beta are floats then)."""
    return R_32F if dt in (torch.float16, torch.bfloat16) else _dtype_code(dt)


def _scalar(value, code):
    if code == C_32F:
        return (C.c_float * 2)(complex(value).real, complex(value).imag)
    if code == C_64F:
        return (C.c_double * 2)(complex(value).real, complex(value).imag)
    if code == R_32I:
        return C.c_int32(int(value))
    return C.c_double(value) if code == R_64F else C.c_float(value)


class Handle:
    """alphasparseHandle_t bound to the current CUDA device; work runs on torch's current stream
    unless ``set_stream`` is called."""

    def __init__(self):
        self.lib = load()
        self.h = C.c_void_p()
        _check(self.lib.alphasparseGetHandle(C.byref(self.h)), "alphasparseGetHandle")
        self.use_torch_stream()

    def use_torch_stream(self):
        self.set_stream(torch.cuda.current_stream().cuda_stream)

    def set_stream(self, cuda_stream: int):
        _check(self.lib.alphasparseSetStream(self.h, C.c_void_p(cuda_stream)), "alphasparseSetStream")

    @property
    def launches(self) -> int:
        return int(self.lib.alphasparseGetLaunchCount(self.h))

    def close(self):
        if self.h:
            self.lib.alphasparse_destory_handle(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DnVec:
    def __init__(self, t: torch.Tensor):
        assert t.is_cuda and t.is_contiguous()
        self.t = t
        self.d = C.c_void_p()
        _check(load().alphasparseCreateDnVec(C.byref(self.d), C.c_int64(t.numel()),
                                             C.c_void_p(t.data_ptr()), _dtype_code(t.dtype)),
               "alphasparseCreateDnVec")

    def __del__(self):
        # at interpreter shutdown module globals may already be gone: then the process's exit frees the descriptor
        if getattr(self, "d", None) and load is not None:
            try:
                load().alphasparseDestroyDnVec(self.d)
            except Exception:
                pass


class DnVecWindow(DnVec):
    """A vector of logical length ``size`` of which only [first, first + t.numel()) exists, in t."""

    def __init__(self, t: torch.Tensor, size: int, first: int):
        assert t.is_cuda and t.is_contiguous()
        self.t = t
        self.size, self.first = size, first
        self.d = C.c_void_p()
        _check(load().alphasparseCreateDnVecWindow(C.byref(self.d), C.c_int64(size), C.c_int64(first),
                                                   C.c_int64(t.numel()), C.c_void_p(t.data_ptr()),
                                                   _dtype_code(t.dtype)), "alphasparseCreateDnVecWindow")


class DnMat:
    """Dense matrix descriptor over a 2-D device tensor: row-major when its columns are contiguous
    (stride(1) == 1), column-major when its rows are (stride(0) == 1, e.g. ``x.t()`` of a
    contiguous tensor); the other stride is the leading dimension."""

    def __init__(self, t: torch.Tensor):
        assert t.is_cuda and t.dim() == 2 and (t.stride(1) == 1 or t.stride(0) == 1)
        self.t = t
        self.d = C.c_void_p()
        row = t.stride(1) == 1
        self.order = ORDER_ROW if row else ORDER_COL
        _check(load().alphasparseCreateDnMat(C.byref(self.d), C.c_int64(t.shape[0]),
                                             C.c_int64(t.shape[1]), C.c_int64(t.stride(0) if row else t.stride(1)),
                                             C.c_void_p(t.data_ptr()), _dtype_code(t.dtype),
                                             self.order), "alphasparseCreateDnMat")

    def __del__(self):
        # at interpreter shutdown module globals may already be gone: then the process's exit frees the descriptor
        if getattr(self, "d", None) and load is not None:
            try:
                load().alphasparseDestroyDnMat(self.d)
            except Exception:
                pass


class CsrMatrix:
    """alphasparseSpMatDescr_t over three device tensors (kept alive by this object)."""

    def __init__(self, rows, cols, row_ptr: torch.Tensor, col_idx: torch.Tensor, val: torch.Tensor):
        assert row_ptr.is_cuda and col_idx.is_cuda and val.is_cuda
        self.rows, self.cols, self.nnz = int(rows), int(cols), int(col_idx.numel())
        self.row_ptr, self.col_idx, self.val = row_ptr, col_idx, val
        rt = {torch.int32: INDEX_I32, torch.int64: INDEX_I64}[row_ptr.dtype]
        assert col_idx.dtype == torch.int32
        self.d = C.c_void_p()
        _check(load().alphasparseCreateCsr(
            C.byref(self.d), C.c_int64(rows), C.c_int64(cols), C.c_int64(self.nnz),
            C.c_void_p(row_ptr.data_ptr()), C.c_void_p(col_idx.data_ptr()),
            C.c_void_p(val.data_ptr()), rt, INDEX_I32, BASE_ZERO, _dtype_code(val.dtype)),
            "alphasparseCreateCsr")

    @classmethod
    def from_csr(cls, m, device="cuda"):
        m = m.to(device)
        return cls(m.rows, m.cols, m.row_ptr, m.col_idx, m.val)

    def analyse(self, handle: Handle):
        _check(load().alphasparseSpMV_analysis(handle.h, OP_N, self.d, SPMV_ALG_DEFAULT),
               "alphasparseSpMV_analysis")

    def plan(self, handle: Handle):
        """Host copy of the analysed plan: (stats dict, bin_rows, merge_tile_row) as numpy."""
        import numpy as np
        lib = load()
        stats = (C.c_int64 * 16)()
        _check(lib.alphasparseCsrPlanGet(handle.h, self.d, stats, None, None), "alphasparseCsrPlanGet")
        s = {n: int(stats[i]) for i, n in enumerate(STAT_NAMES)}
        bins = np.zeros(max(self.rows, 1), dtype=np.int32)
        tiles = np.zeros(s["merge_tiles"] + 1, dtype=np.int32)
        _check(lib.alphasparseCsrPlanGet(handle.h, self.d, None, bins.ctypes.data_as(C.c_void_p),
                                         tiles.ctypes.data_as(C.c_void_p)), "alphasparseCsrPlanGet")
        return s, bins[: self.rows], tiles

    def last_variant(self) -> str:
        return load().alphasparseCsrLastVariant(self.d).decode()

    def __del__(self):
        # at interpreter shutdown module globals may already be gone: then the process's exit frees the descriptor
        if getattr(self, "d", None) and load is not None:
            try:
                load().alphasparseDestroySpMat(self.d)
            except Exception:
                pass


def spmv_buffer_size(handle: Handle, A: CsrMatrix, x: DnVec, y: DnVec, alpha=1.0, beta=0.0,
                     alg=SPMV_ALG_DEFAULT) -> int:
    code = _spmv_compute_code(A.val.dtype)
    a, b = _scalar(alpha, code), _scalar(beta, code)
    size = C.c_size_t(0)
    _check(load().alphasparseSpMV_bufferSize(handle.h, OP_N, C.byref(a), A.d, x.d, C.byref(b), y.d,
                                             code, alg, C.byref(size)), "alphasparseSpMV_bufferSize")
    return int(size.value)


def spmv(handle: Handle, A: CsrMatrix, x: DnVec, y: DnVec, alpha=1.0, beta=0.0,
         alg=SPMV_ALG_DEFAULT, buffer: torch.Tensor | None = None, op=OP_N):
    """y = alpha*A*x + beta*y on handle's stream (asynchronous).  The compute type is the matrix type,
    fp32 for 16-bit matrices, and y's type (int32 or fp32) for int8 matrices."""
    code = _dtype_code(y.t.dtype) if A.val.dtype == torch.int8 else _spmv_compute_code(A.val.dtype)
    a, b = _scalar(alpha, code), _scalar(beta, code)
    buf = C.c_void_p(buffer.data_ptr()) if buffer is not None else C.c_void_p()
    _check(load().alphasparseSpMV(handle.h, op, C.byref(a), A.d, x.d, C.byref(b), y.d, code, alg, buf),
           "alphasparseSpMV")


def _spmm_compute_code(dt: torch.dtype) -> int:
    """The compute type of an SpMM is C's type; a 16-bit C is computed in fp32."""
    return R_32F if dt in (torch.float16, torch.bfloat16) else _dtype_code(dt)


def spmm_buffer_size(handle: Handle, A: CsrMatrix, B: DnMat, Cm: DnMat, alg=SPMM_ALG_DEFAULT) -> int:
    code = _spmm_compute_code(Cm.t.dtype)
    a, b = _scalar(1.0, code), _scalar(0.0, code)
    size = C.c_size_t(0)
    _check(load().alphasparseSpMM_bufferSize(handle.h, OP_N, OP_N, C.byref(a), A.d, B.d, C.byref(b), Cm.d,
                                             code, alg, C.byref(size)), "alphasparseSpMM_bufferSize")
    return int(size.value)


def spmm(handle: Handle, A: CsrMatrix, B: DnMat, Cm: DnMat, alpha=1.0, beta=0.0,
         alg=SPMM_ALG_DEFAULT, compute=None, buffer: torch.Tensor | None = None, op=OP_N):
    """C = alpha*A*B + beta*C on handle's stream (asynchronous).  B and C both row-major, or both
    column-major with a ``buffer`` of spmm_buffer_size bytes."""
    code = _spmm_compute_code(Cm.t.dtype) if compute is None else compute
    a, b = _scalar(alpha, code), _scalar(beta, code)
    buf = C.c_void_p(buffer.data_ptr()) if buffer is not None else C.c_void_p()
    _check(load().alphasparseSpMM(handle.h, op, OP_N, C.byref(a), A.d, B.d, C.byref(b), Cm.d, code,
                                  alg, buf), "alphasparseSpMM")


def spmm_last_variant(A: CsrMatrix) -> str:
    return load().alphasparseCsrLastSpmmVariant(A.d).decode()


def spmm_preprocess(handle: Handle, A: CsrMatrix, B: DnMat, Cm: DnMat, alg=SPMM_ALG_DEFAULT):
    code = _spmm_compute_code(Cm.t.dtype)
    a, b = _scalar(1.0, code), _scalar(0.0, code)
    size = C.c_size_t(0)
    _check(load().alphasparseSpMM_preprocess(handle.h, OP_N, OP_N, C.byref(a), A.d, B.d, C.byref(b),
                                             Cm.d, code, alg, C.byref(size)),
           "alphasparseSpMM_preprocess")
    return int(size.value)


def partition_rows_by_nnz(handle: Handle, row_ptr: torch.Tensor, parts: int):
    import numpy as np
    rt = {torch.int32: INDEX_I32, torch.int64: INDEX_I64}[row_ptr.dtype]
    out = np.zeros(parts + 1, dtype=np.int64)
    _check(load().alphasparseCsrPartitionRowsByNnz(handle.h, C.c_int64(row_ptr.numel() - 1),
                                                   C.c_void_p(row_ptr.data_ptr()), rt, parts,
                                                   out.ctypes.data_as(C.c_void_p)),
           "alphasparseCsrPartitionRowsByNnz")
    return out


def column_range(handle: Handle, col_idx: torch.Tensor):
    """(min, max) column index of a device col_idx slice; (0, -1) when it is empty."""
    lo, hi = C.c_int64(0), C.c_int64(-1)
    _check(load().alphasparseCsrColumnRange(handle.h, C.c_int64(col_idx.numel()),
                                            C.c_void_p(col_idx.data_ptr()), INDEX_I32, C.byref(lo),
                                            C.byref(hi)), "alphasparseCsrColumnRange")
    return int(lo.value), int(hi.value)


def rebase_row_offsets(handle: Handle, row_ptr: torch.Tensor, row_begin: int, row_end: int,
                       out_dtype=torch.int32) -> torch.Tensor:
    it = {torch.int32: INDEX_I32, torch.int64: INDEX_I64}
    out = torch.empty(row_end - row_begin + 1, dtype=out_dtype, device=row_ptr.device)
    _check(load().alphasparseCsrRebaseRowOffsets(handle.h, C.c_void_p(row_ptr.data_ptr()),
                                                 it[row_ptr.dtype], C.c_int64(row_begin),
                                                 C.c_int64(row_end), C.c_void_p(out.data_ptr()),
                                                 it[out_dtype]), "alphasparseCsrRebaseRowOffsets")
    return out


NOALLOC_MAX_ITEMS = 134217728


def spmv_csr_noalloc(row_ptr: torch.Tensor, col_idx: torch.Tensor, val: torch.Tensor, x: torch.Tensor,
                     y: torch.Tensor, alpha=1.0, beta=0.0, cols=None, stream=None) -> int:
    """alphasparseSpMVCsrNoAlloc on torch tensors; returns the status instead of raising so that
    callers can test the size limit."""
    code = _dtype_code(val.dtype)
    a, b = _scalar(alpha, code), _scalar(beta, code)
    rt = {torch.int32: INDEX_I32, torch.int64: INDEX_I64}[row_ptr.dtype]
    st = torch.cuda.current_stream().cuda_stream if stream is None else stream
    return int(load().alphasparseSpMVCsrNoAlloc(
        C.c_void_p(st), C.c_int64(row_ptr.numel() - 1), C.c_int64(x.numel() if cols is None else cols),
        C.c_int64(col_idx.numel()), C.c_void_p(row_ptr.data_ptr()), rt, C.c_void_p(col_idx.data_ptr()),
        C.c_void_p(val.data_ptr()), code, C.byref(a), C.c_void_p(x.data_ptr()), C.byref(b),
        C.c_void_p(y.data_ptr())))


def coo2csr(coo_row: torch.Tensor, rows: int, out_dtype=torch.int32, stream=None) -> torch.Tensor:
    """Row offsets (rows+1) from ascending int32 COO row indices on the device."""
    assert coo_row.is_cuda and coo_row.dtype == torch.int32
    out = torch.empty(rows + 1, dtype=out_dtype, device=coo_row.device)
    st = torch.cuda.current_stream().cuda_stream if stream is None else stream
    _check(load().alphasparseXcoo2csr(C.c_void_p(st), C.c_void_p(coo_row.data_ptr()), C.c_int64(coo_row.numel()),
                                      C.c_int64(rows), C.c_void_p(out.data_ptr()),
                                      INDEX_I64 if out_dtype == torch.int64 else INDEX_I32), "alphasparseXcoo2csr")
    return out


def read_mtx(path: str, dtype=torch.float32, ordered: bool = True):
    """MatrixMarket coordinate file (or, for a name ending in .bin, the reference drivers' binary dump) ->
    (rows, cols, row_index, col_index, values) as host tensors,
    sorted by (row, column) when ``ordered`` (what coo2csr needs)."""
    import numpy as np
    lib = load()
    lib.alphasparseFreeHost.restype = None
    code = _dtype_code(dtype)
    m, n, nnz = C.c_int64(), C.c_int64(), C.c_int64()
    ri, ci, v = C.c_void_p(), C.c_void_p(), C.c_void_p()
    reader = lib.alphasparseReadBinCoo if path.endswith(".bin") else lib.alphasparseReadMtxCoo
    _check(reader(path.encode(), C.byref(m), C.byref(n), C.byref(nnz), C.byref(ri), C.byref(ci),
                  C.byref(v), code), "alphasparseReadBinCoo" if path.endswith(".bin") else "alphasparseReadMtxCoo")
    try:
        k = nnz.value
        if ordered:
            _check(lib.alphasparseCooOrder(C.c_int64(k), ri, ci, v, code), "alphasparseCooOrder")
        npdt = np.float32 if dtype == torch.float32 else np.float64
        def arr(p, t):
            return np.ctypeslib.as_array(C.cast(p, C.POINTER(t)), shape=(k,)).copy() if k else np.zeros(0, dtype=t)
        rows_i = arr(ri, C.c_int32)
        cols_i = arr(ci, C.c_int32)
        vals = arr(v, C.c_float if npdt == np.float32 else C.c_double)
    finally:
        for p in (ri, ci, v):
            lib.alphasparseFreeHost(p)
    return m.value, n.value, torch.from_numpy(rows_i), torch.from_numpy(cols_i), torch.from_numpy(vals)


# ---- multi-GPU SpMV (alphasparseMg*) ------------------------------------------------------

def mg_exchange_plan(own_bounds, windows, rank: int):
    """alphasparseMgExchangePlan (host only).  ``windows``: one (lo, hi) pair per rank.  Returns
    (sends, recvs), lists of (peer, begin, end)."""
    import numpy as np
    world = len(windows)
    ob = np.ascontiguousarray(own_bounds, dtype=np.int64)
    w = np.ascontiguousarray(np.asarray(windows, dtype=np.int64).reshape(-1))
    sends = np.zeros(3 * world, dtype=np.int64)
    recvs = np.zeros(3 * world, dtype=np.int64)
    ns, nr = C.c_int(0), C.c_int(0)
    _check(load().alphasparseMgExchangePlan(world, rank, ob.ctypes.data_as(C.c_void_p), w.ctypes.data_as(C.c_void_p),
                                            sends.ctypes.data_as(C.c_void_p), C.byref(ns),
                                            recvs.ctypes.data_as(C.c_void_p), C.byref(nr)),
           "alphasparseMgExchangePlan")
    tri = lambda a, n: [tuple(int(v) for v in a[3 * i:3 * i + 3]) for i in range(n)]
    return tri(sends, ns.value), tri(recvs, nr.value)


class _DevicePointer:
    """Lets torch view device memory it did not allocate (the window buffer inside the library)."""

    def __init__(self, ptr: int, count: int, dtype: torch.dtype):
        typestr = {torch.float32: "<f4", torch.float64: "<f8"}[dtype]
        self.__cuda_array_interface__ = {"shape": (count,), "typestr": typestr, "data": (ptr, False),
                                         "version": 2, "strides": None}


class Mg:
    """alphasparseMgHandle_t: row-sharded SpMV over an NCCL communicator of its own, created from a
    unique id that rank 0 makes and torch.distributed hands round (any transport would do)."""

    def __init__(self, handle: Handle, rank: int, world: int, group=None):
        self.lib, self.handle, self.rank, self.world = load(), handle, rank, world
        self.comm = C.c_void_p()
        self.mg = C.c_void_p()
        if world > 1:
            import torch.distributed as dist
            ident = (C.c_char * 128)()
            if rank == 0:
                _check(self.lib.alphasparseMgGetUniqueId(ident), "alphasparseMgGetUniqueId")
            box = [bytes(ident.raw)]
            dist.broadcast_object_list(box, src=0, group=group)
            ident = (C.c_char * 128).from_buffer_copy(box[0])
            _check(self.lib.alphasparseMgCommInitRank(C.byref(self.comm), world, ident, rank),
                   "alphasparseMgCommInitRank")
        _check(self.lib.alphasparseMgCreate(C.byref(self.mg), handle.h, self.comm, rank, world),
               "alphasparseMgCreate")
        self.A = None

    def set_shard(self, A: CsrMatrix, x_bounds=None, mode=MG_X_WINDOW_OVERLAP, root=0):
        import numpy as np
        xb = None if x_bounds is None else np.ascontiguousarray(x_bounds, dtype=np.int64)
        _check(self.lib.alphasparseMgSetShard(self.mg, A.d, None if xb is None else xb.ctypes.data_as(C.c_void_p),
                                              mode, root), "alphasparseMgSetShard")
        self.A = A            # keeps the arrays alive

    def _scalars(self, alpha, beta):
        code = _dtype_code(self.A.val.dtype)
        return _scalar(alpha, code), _scalar(beta, code)

    def spmv(self, x: torch.Tensor | None, y: torch.Tensor, alpha=1.0, beta=0.0, alg=SPMV_ALG_DEFAULT):
        a, b = self._scalars(alpha, beta)
        _check(self.lib.alphasparseMgSpMV(self.mg, C.byref(a), C.c_void_p(x.data_ptr() if x is not None else 0),
                                          C.byref(b), C.c_void_p(y.data_ptr()), alg), "alphasparseMgSpMV")

    def exchange(self, x: torch.Tensor | None):
        _check(self.lib.alphasparseMgExchange(self.mg, C.c_void_p(x.data_ptr() if x is not None else 0)),
               "alphasparseMgExchange")

    def own_view(self) -> torch.Tensor:
        """This rank's own part of x inside the library's window buffer, as a tensor."""
        p, first, count = C.c_void_p(), C.c_int64(), C.c_int64()
        _check(self.lib.alphasparseMgOwnView(self.mg, C.byref(p), C.byref(first), C.byref(count)),
               "alphasparseMgOwnView")
        return torch.as_tensor(_DevicePointer(p.value, count.value, self.A.val.dtype), device=self.A.val.device)

    def info(self) -> dict:
        out = (C.c_int64 * 8)()
        _check(self.lib.alphasparseMgGetInfo(self.mg, out), "alphasparseMgGetInfo")
        return {n: int(out[i]) for i, n in enumerate(MG_INFO_NAMES)}

    def close(self):
        if self.mg:
            self.lib.alphasparseMgDestroy(self.mg)
            self.mg = C.c_void_p()
        if self.comm:
            self.lib.alphasparseMgCommDestroy(self.comm)
            self.comm = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
