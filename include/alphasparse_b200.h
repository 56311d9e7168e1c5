/* alphasparse_b200.h - C ABI of the Blackwell (sm_100a) CSR SpMV / SpMM library.
 *
 * Every entry point is extern "C" with plain pointers and sizes.  Names, argument order,
 * argument meaning and enum values are those of the AlphaSparse generic API for this path,
 * so a caller of the reference recompiles against this header.  Each declaration cites the
 * reference interface it replaces (path within the reference project : line).
 *
 * Conventions shared by all entry points
 *   - descriptors capture caller-owned DEVICE pointers (no copy, never freed here);
 *   - alpha / beta are HOST pointers to a value of the compute type, read synchronously;
 *   - work is stream-ordered on handle->stream; SpMV / SpMM do not synchronise and do not
 *     allocate once the matrix has been analysed (alphasparseSpMV_analysis /
 *     alphasparseSpMM_preprocess; otherwise the first call analyses, which allocates the
 *     plan with cudaMalloc and synchronises once);
 *   - errors come back as alphasparseStatus_t, nothing is printed, nothing exits;
 *   - beta == 0 means y / Y is written without being read.
 * Supported beyond the plain case: opA = TRANSPOSE for SpMV and SpMM (on a transposed copy the
 * plan builds on the device, A itself untouched), column-major B and C in SpMM (through
 * row-major copies in the caller's buffer), fp16 / bf16 A and x with fp32 arithmetic in SpMV,
 * complex (C_32F, C_64F) and int8 (to int32 or fp32) SpMV and SpMM, fp16 A and B with fp32 or
 * fp16 C in SpMM, bf16 A and B with fp32 C in SpMM (the tcgen05 kernels), 32- or 64-bit row
 * offsets.
 * Not supported (ALPHA_SPARSE_STATUS_NOT_SUPPORTED): transposed B, index base one, formats
 * other than CSR, half-precision complex, device pointer mode.  There is no CPU fallback.
 */
#ifndef ALPHASPARSE_B200_H
#define ALPHASPARSE_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>
#include <cuda_runtime_api.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- enums: values identical to include/alphasparse/spdef.h ------------------------- */
typedef enum { /* spdef.h:10-22 */
  ALPHA_SPARSE_STATUS_SUCCESS = 0,
  ALPHA_SPARSE_STATUS_NOT_INITIALIZED = 1,
  ALPHA_SPARSE_STATUS_ALLOC_FAILED = 2,
  ALPHA_SPARSE_STATUS_INVALID_VALUE = 3,
  ALPHA_SPARSE_STATUS_EXECUTION_FAILED = 4,
  ALPHA_SPARSE_STATUS_INTERNAL_ERROR = 5,
  ALPHA_SPARSE_STATUS_NOT_SUPPORTED = 6,
  ALPHA_SPARSE_STATUS_INVALID_POINTER = 7,
  ALPHA_SPARSE_STATUS_INVALID_HANDLE = 8,
  ALPHA_SPARSE_STATUS_INVALID_KERNEL_PARAM = 9,
  ALPHA_SPARSE_STATUS_INVALID_SIZE = 10
} alphasparseStatus_t;

typedef enum { /* spdef.h:25-29 */
  ALPHA_SPARSE_OPERATION_NON_TRANSPOSE = 0,
  ALPHA_SPARSE_OPERATION_TRANSPOSE = 1,
  ALPHA_SPARSE_OPERATION_CONJUGATE_TRANSPOSE = 2
} alphasparseOperation_t;

typedef enum { /* spdef.h:48-51 */
  ALPHA_SPARSE_INDEX_BASE_ZERO = 0,
  ALPHA_SPARSE_INDEX_BASE_ONE = 1
} alphasparseIndexBase_t;

typedef enum { /* spdef.h:83-86 */
  ALPHASPARSE_ORDER_ROW = 0,
  ALPHASPARSE_ORDER_COL = 1
} alphasparseOrder_t;

typedef enum { /* spdef.h:125-140 (only CSR is accepted on this path) */
  ALPHA_SPARSE_FORMAT_COO = 0,
  ALPHA_SPARSE_FORMAT_CSR = 1,
  ALPHA_SPARSE_FORMAT_CSC = 2
} alphasparseFormat_t;

typedef enum { /* spdef.h:144-155 */
  ALPHA_R_32F = 0,
  ALPHA_R_64F = 1,
  ALPHA_C_32F = 2,
  ALPHA_C_64F = 3,
  ALPHA_R_16F = 4,
  ALPHA_R_16BF = 5,
  ALPHA_C_16F = 6,
  ALPHA_C_16BF = 7,
  ALPHA_R_8I = 8,
  ALPHA_R_32I = 9
} alphasparseDataType;

typedef enum { /* spdef.h:299-302 */
  ALPHA_SPARSE_POINTER_MODE_HOST = 0,
  ALPHA_SPARSE_POINTER_MODE_DVICE = 1
} alphasparse_pointer_mode_t;

typedef enum { /* spdef.h:304-308 */
  ALPHA_SPARSE_LAYER_MODE_NONE = 0,
  ALPHA_SPARSE_LAYER_MODE_LOG_TRACE = 1,
  ALPHA_SPARSE_LAYER_MODE_LOG_BENCH = 2
} alphasparse_layer_mode_t;

typedef enum { /* spdef.h:310-314 */
  ALPHA_SPARSE_INDEXTYPE_U16 = 1,
  ALPHA_SPARSE_INDEXTYPE_I32 = 2,
  ALPHA_SPARSE_INDEXTYPE_I64 = 3
} alphasparseIndexType_t;

/* spdef.h:345-365.  How this library maps them: DEFAULT picks from the analysed row-length
 * statistics; SCALAR / VECTOR / ADAPTIVE / CSR_ADAPTIVE / LINE* select the row-length-binned
 * kernel; MERGE / ROW_PARTITION / LOAD_BALANCE / FLAT* / CSR_STREAM select the merge-path
 * kernel.  COO and ELL name other formats' algorithms; for a CSR matrix they are taken as DEFAULT
 * (the reference's own CSR test drivers pass ALG_COO, and its dispatcher then does nothing). */
typedef enum {
  ALPHA_SPARSE_SPMV_ALG_DEFAULT = 0,
  ALPHA_SPARSE_SPMV_ALG_COO = 1,
  ALPHA_SPARSE_SPMV_ALG_CSR_ADAPTIVE = 2,
  ALPHA_SPARSE_SPMV_ALG_CSR_STREAM = 3,
  ALPHA_SPARSE_SPMV_ALG_ELL = 4,
  ALPHA_SPARSE_SPMV_ALG_SCALAR = 5,
  ALPHA_SPARSE_SPMV_ALG_VECTOR = 6,
  ALPHA_SPARSE_SPMV_ROW_PARTITION = 7,
  ALPHA_SPARSE_SPMV_ADAPTIVE = 8,
  ALPHA_SPARSE_SPMV_ALG_MERGE = 9,
  ALPHA_SPARSE_SPMV_ALG_LINE = 10,
  ALPHA_SPARSE_SPMV_ALG_FLAT1 = 11,
  ALPHA_SPARSE_SPMV_ALG_FLAT4 = 12,
  ALPHA_SPARSE_SPMV_ALG_FLAT8 = 13,
  ALPHA_SPARSE_SPMV_ALG_ACC = 14,
  ALPHA_SPARSE_SPMV_ALG_FLAT = 15,
  ALPHA_SPARSE_SPMV_ALG_LINE_ENHANCE = 16,
  ALPHA_SPARSE_SPMV_ALG_LOAD_BALANCE = 17,
  ALPHA_SPARSE_SPMV_ALG_PFLAT = 18
} alphasparseSpMVAlg_t;

/* spdef.h:390-402.  DEFAULT picks per (N, row statistics); CSR_ALG1..5 select the SIMT
 * row-block kernel; CSR_ALG6 (the matrix-unit algorithm of the HIP backend,
 * hip/kernel/level3/alphasparse_spmm_tc4csr.h:228-255) selects the tcgen05 kernel and needs
 * bf16 A and X with fp32 Y.  COO algorithms are taken as DEFAULT for a CSR matrix. */
typedef enum {
  ALPHASPARSE_SPMM_ALG_DEFAULT = 0,
  ALPHASPARSE_SPMM_COO_ALG1 = 1,
  ALPHASPARSE_SPMM_COO_ALG2 = 2,
  ALPHASPARSE_SPMM_COO_ALG3 = 3,
  ALPHASPARSE_SPMM_COO_ALG4 = 4,
  ALPHASPARSE_SPMM_CSR_ALG1 = 5,
  ALPHASPARSE_SPMM_CSR_ALG2 = 6,
  ALPHASPARSE_SPMM_CSR_ALG3 = 7,
  ALPHASPARSE_SPMM_CSR_ALG4 = 8,
  ALPHASPARSE_SPMM_CSR_ALG5 = 9,
  ALPHASPARSE_SPMM_CSR_ALG6 = 10
} alphasparseSpMMAlg_t;

/* ---- handle: include/alphasparse/handle.h:26-85 ------------------------------------- *
 * Public like the reference's (its callers assign handle->stream directly, there is no
 * setter); `stream` is honoured by every launch.  `impl` is private to the library.      */
typedef struct alphasparse_handle_s {
  int device;          /* the device that was current at creation (the reference hard-codes 0) */
  int wavefront_size;  /* 32 */
  int asic_rev;
  cudaStream_t stream;
  cudaStream_t streams[6];
  alphasparse_pointer_mode_t pointer_mode; /* HOST only */
  alphasparse_layer_mode_t layer_mode;
  size_t buffer_size;
  void* buffer;
  float* sone;
  double* done;
  bool check_flag;
  int* process;
  void* pflat_analysis_data;
  void* impl;
} alphasparse_handle;
typedef alphasparse_handle* alphasparseHandle_t;

/* ---- descriptors: include/alphasparse/handle.h:395-435, 478-499 --------------------- */
struct _alphasparseSpMatDescr {
  bool init;
  bool analysed;       /* true once a plan (row bins + merge-path partition) is attached */
  int64_t rows, cols, nnz;
  int64_t nwarps;
  int* row_data;       /* set when row_type is I32 (reference field) */
  int* col_data;
  int* ind_data;
  void* val_data;
  const int* const_row_data;
  const int* const_col_data;
  const int* const_ind_data;
  const void* const_val_data;
  alphasparseIndexType_t row_type, col_type;
  alphasparseDataType data_type;
  alphasparseIndexBase_t idx_base;
  alphasparseFormat_t format;
  void* descr;
  void* info;          /* the analysis plan, owned by the descriptor */
  const void* row_offsets; /* row offsets of either width (I32 or I64); extension */
  int64_t batch_count, batch_stride, offsets_batch_stride, columns_values_batch_stride;
};
struct _alphasparse_dnvec_descr {
  bool init;
  int64_t size;
  void* values;
  alphasparseDataType data_type;
};
struct _alphasparse_dnmat_descr {
  bool init;
  int64_t rows, cols, ld;
  void* values;
  alphasparseDataType data_type;
  alphasparseOrder_t order;
};
typedef struct _alphasparseSpMatDescr* alphasparseSpMatDescr_t;
typedef struct _alphasparse_dnvec_descr* alphasparseDnVecDescr_t;
typedef struct _alphasparse_dnmat_descr* alphasparseDnMatDescr_t;

/* ---- handle and stream -------------------------------------------------------------- */
/* handle.h:520-524; cuda/util/handle.cu:52-73 (initHandle), :75-156 (alphasparseGetHandle),
 * :161-175 (alphasparse_destory_handle, spelling kept). */
alphasparseStatus_t initHandle(alphasparseHandle_t* handle);
alphasparseStatus_t alphasparseGetHandle(alphasparseHandle_t* handle);
alphasparseStatus_t alphasparse_destory_handle(alphasparseHandle_t handle);
/* Extension: the reference has no accessor, callers write handle->stream (handle.h:37). */
alphasparseStatus_t alphasparseSetStream(alphasparseHandle_t handle, cudaStream_t stream);
alphasparseStatus_t alphasparseGetStream(alphasparseHandle_t handle, cudaStream_t* stream);

/* ---- descriptors -------------------------------------------------------------------- */
/* cuda/format/alphasparse_create_csr.h:6-63 is a header template with int sizes and int
 * pointers; this is the C form with 64-bit sizes and void pointers.  Row offsets may be
 * I32 or I64, column indices I32.  Pointer capture only. */
alphasparseStatus_t alphasparseCreateCsr(alphasparseSpMatDescr_t* spMatDescr, int64_t rows,
                                         int64_t cols, int64_t nnz, void* csrRowOffsets,
                                         void* csrColInd, void* csrValues,
                                         alphasparseIndexType_t csrRowOffsetsType,
                                         alphasparseIndexType_t csrColIndType,
                                         alphasparseIndexBase_t idxBase,
                                         alphasparseDataType valueType);
/* handle.h:593-597; cuda/util/handle.cu:657-693 */
alphasparseStatus_t alphasparseCreateDnVec(alphasparseDnVecDescr_t* descr, int64_t size,
                                           void* values, alphasparseDataType data_type);
/* handle.h:599-606; cuda/util/handle.cu:696-738 */
alphasparseStatus_t alphasparseCreateDnMat(alphasparseDnMatDescr_t* dnMatDescr, int64_t rows,
                                           int64_t cols, int64_t ld, void* values,
                                           alphasparseDataType valueType,
                                           alphasparseOrder_t order);
/* Extensions: the reference never frees its descriptors. */
alphasparseStatus_t alphasparseDestroySpMat(alphasparseSpMatDescr_t spMatDescr);
alphasparseStatus_t alphasparseDestroyDnVec(alphasparseDnVecDescr_t descr);
alphasparseStatus_t alphasparseDestroyDnMat(alphasparseDnMatDescr_t descr);
/* Re-point a dense descriptor without re-creating it (cuSPARSE-style; extension). */
alphasparseStatus_t alphasparseDnVecSetValues(alphasparseDnVecDescr_t descr, void* values);
alphasparseStatus_t alphasparseDnMatSetValues(alphasparseDnMatDescr_t descr, void* values);

/* ---- SpMV: y = alpha*op(A)*x + beta*y ----------------------------------------------- */
/* spapi.h:6895-6905; cuda/kernel/level2/alphasparse_spmv.cu:221-339.  Type combinations
 * (A and x / y / computeType, alpha and beta host pointers of the compute type):
 *   R_32F / R_32F / R_32F  (:234)      R_64F / R_64F / R_64F  (:240)
 *   R_16F / R_32F / R_32F  (:288-292)  R_16BF / R_16BF / R_32F (:294-300)
 *   C_32F / C_32F / C_32F  (:246-253)  C_64F / C_64F / C_64F  (:255-262)
 *   R_8I  / R_32I / R_32I  (:276-281)  R_8I  / R_32F / R_32F  (:282-287)
 * with 32- or 64-bit row offsets (complex and int8: one plain kernel over the plan's row
 * classes; opA = TRANSPOSE on the transposed copy, CONJUGATE_TRANSPOSE of a complex matrix
 * NOT_SUPPORTED - the copy keeps the values as they are).  The reference's half-precision complex instances are
 * not provided.
 * opA = TRANSPOSE (or CONJUGATE_TRANSPOSE, the same for real types): x has A's row count, y its
 * column count; the first such call (or alphasparseSpMV_analysis with that opA) builds a
 * transposed copy of A on the device, which allocates and synchronises; A itself is not
 * modified (the reference's transpose_csr overwrites A, cuda/format/transpose_csr.h:9-78).  The
 * copy holds A's values as of then: after changing them call alphasparseSpMV_clearMat.
 * Matrices with 2^31 or more entries are not transposed (NOT_SUPPORTED). */
alphasparseStatus_t alphasparseSpMV(alphasparseHandle_t handle, alphasparseOperation_t opA,
                                    const void* alpha, alphasparseSpMatDescr_t matA,
                                    alphasparseDnVecDescr_t vecX, const void* beta,
                                    alphasparseDnVecDescr_t vecY,
                                    alphasparseDataType computeType, alphasparseSpMVAlg_t alg,
                                    void* externalBuffer);
/* spapi.h:6907-6917; cuda/kernel/level2/alphasparse_spmv.cu:341-421.  The size covers the
 * per-tile carry array of the merge-path kernel for this matrix, for any alg. */
alphasparseStatus_t alphasparseSpMV_bufferSize(alphasparseHandle_t handle,
                                               alphasparseOperation_t opA, const void* alpha,
                                               alphasparseSpMatDescr_t matA,
                                               alphasparseDnVecDescr_t vecX, const void* beta,
                                               alphasparseDnVecDescr_t vecY,
                                               alphasparseDataType computeType,
                                               alphasparseSpMVAlg_t alg, size_t* bufferSize);
/* spapi.h:6919-6923 (declared; the CUDA backend never defines it, the HIP backend returns
 * NOT_SUPPORTED, hip/kernel/level2/alphasparse_spmv.hip:229-256).  Here it runs the
 * preprocessing pass: row-length bins, merge-path tile partition, statistics. */
alphasparseStatus_t alphasparseSpMV_analysis(alphasparseHandle_t handle,
                                             alphasparseOperation_t opA,
                                             alphasparseSpMatDescr_t matA,
                                             alphasparseSpMVAlg_t alg);
/* spapi.h:6925-6926 takes no matrix; it is kept and is a no-op.  The plan is released by
 * alphasparseSpMV_clearMat or alphasparseDestroySpMat. */
alphasparseStatus_t alphasparseSpMV_clear(alphasparseHandle_t handle, alphasparseSpMVAlg_t alg);
alphasparseStatus_t alphasparseSpMV_clearMat(alphasparseHandle_t handle,
                                             alphasparseSpMatDescr_t matA); /* extension */

/* No counterpart in the reference.  y = alpha*A*x + beta*y on raw CSR device arrays for callers
 * that must not allocate device memory around the call (a solver loop on a GPU whose memory a
 * framework's pool has claimed in full, or a latency-critical loop that cannot take the device
 * synchronisation and late failure of cudaMalloc / cudaFree).  Such callers cannot use
 * alphasparseSpMV either, because matrix analysis allocates the plan; so this call takes no
 * handle and no descriptor, runs the merge-path kernel, and keeps its scratch (per-tile start
 * rows and carry-outs, 786,688 bytes) in a fixed device array inside the library image, which
 * every GPU that loads the library holds until the process exits.  It calls no cudaMalloc,
 * cudaFree or any other allocating routine.
 *   - Limit: rows + nnz <= ALPHASPARSE_SPMV_NOALLOC_MAX_ITEMS, else ALPHA_SPARSE_STATUS_INVALID_SIZE.
 *   - fp32 / fp64 values, I32 / I64 row offsets, I32 zero-based columns; alpha, beta host pointers.
 *   - The CSR structure is NOT validated (validation needs scratch of its own): offsets must be
 *     non-decreasing from 0 to nnz and columns inside [0, cols).
 *   - The first call on each device looks the array's device address up once (with that device
 *     current), and with CUDA's lazy module loading it may also be the moment the library's device
 *     code - this array included - is loaded onto that GPU.  Make that first call at start-up,
 *     before a memory pool claims the device and outside any stream capture (rows = 1, nnz = 0 is
 *     enough); only the calls after it are free of any allocation.
 *   - All calls on a device share the one array.  Nothing in it has to be cleared between calls
 *     (every slot a call reads it has written first), but two calls whose kernels overlap on the
 *     GPU - different streams, or different host threads - race on it: keep calls on one device
 *     stream-ordered with respect to each other. */
#define ALPHASPARSE_SPMV_NOALLOC_MAX_ITEMS 134217728 /* 65,536 tiles of 2,048 merge items */
alphasparseStatus_t alphasparseSpMVCsrNoAlloc(cudaStream_t stream, int64_t rows, int64_t cols,
                                              int64_t nnz, const void* csrRowOffsets,
                                              alphasparseIndexType_t csrRowOffsetsType,
                                              const int32_t* csrColInd, const void* csrValues,
                                              alphasparseDataType valueType, const void* alpha,
                                              const void* x, const void* beta, void* y);

/* ---- SpMM: C = alpha*op(A)*op(B) + beta*C ------------------------------------------- */
/* spapi.h:6963-6974; cuda/kernel/level3/alphasparse_spmm.cu:531-612.  B and C both row-major
 * (no external buffer needed) or both column-major: then externalBuffer must hold
 * alphasparseSpMM_bufferSize bytes, into which row-major copies of B and C are made (the
 * reference transposes B and C in place with buffers it allocates per call, :131-285); B is
 * left untouched and C keeps its layout.  Type combinations (A and B / C / computeType, alpha and
 * beta host pointers of the compute type), the reference's table at :546-596:
 *   R_32F / R_32F / R_32F      R_64F / R_64F / R_64F      R_16BF / R_32F / R_32F (tcgen05)
 *   C_32F / C_32F / C_32F      C_64F / C_64F / C_64F
 *   R_8I  / R_32I / R_32I      R_8I  / R_32F / R_32F
 *   R_16F / R_32F / R_32F      R_16F / R_16F / R_32F
 * with 32- or 64-bit row offsets; the complex, int8 and fp16 rows run one plain kernel
 * (opA = TRANSPOSE on the transposed copy; CONJUGATE_TRANSPOSE of a complex matrix
 * NOT_SUPPORTED). */
alphasparseStatus_t alphasparseSpMM(alphasparseHandle_t handle, alphasparseOperation_t opA,
                                    alphasparseOperation_t opB, const void* alpha,
                                    alphasparseSpMatDescr_t matA, alphasparseDnMatDescr_t matB,
                                    const void* beta, alphasparseDnMatDescr_t matC,
                                    alphasparseDataType computeType, alphasparseSpMMAlg_t alg,
                                    void* externalBuffer);
/* spapi.h:7017-7028; cuda/kernel/level3/alphasparse_spmm.cu:614-759 */
alphasparseStatus_t alphasparseSpMM_bufferSize(alphasparseHandle_t handle,
                                               alphasparseOperation_t opA,
                                               alphasparseOperation_t opB, const void* alpha,
                                               alphasparseSpMatDescr_t matA,
                                               alphasparseDnMatDescr_t matB, const void* beta,
                                               alphasparseDnMatDescr_t matC,
                                               alphasparseDataType computeType,
                                               alphasparseSpMMAlg_t alg, size_t* bufferSize);
/* spapi.h:7004-7015; defined only by the HIP backend (alphasparse_spmm.hip:657-695). */
alphasparseStatus_t alphasparseSpMM_preprocess(alphasparseHandle_t handle,
                                               alphasparseOperation_t opA,
                                               alphasparseOperation_t opB, const void* alpha,
                                               alphasparseSpMatDescr_t matA,
                                               alphasparseDnMatDescr_t matB, const void* beta,
                                               alphasparseDnMatDescr_t matC,
                                               alphasparseDataType computeType,
                                               alphasparseSpMMAlg_t alg, size_t* bufferSize);

/* ---- multi-GPU row partition (extension; the reference is single-device) ------------ */
/* Contiguous row ranges of near-equal nnz, the rule of hygon/util/partition.cpp:83-96
 * (device twin: cuda/kernel/level2/alphasparse_spmv_csr_row_partition.h:26-45) lifted to
 * 64-bit: bounds[0]=0, bounds[parts]=rows, bounds[i]=first j in [0,rows-1] with
 * row_end[j] >= (nnz/parts)*i.  row_offsets is a DEVICE pointer; bounds is a HOST array of
 * parts+1 entries.  Synchronises handle->stream. */
alphasparseStatus_t alphasparseCsrPartitionRowsByNnz(alphasparseHandle_t handle, int64_t rows,
                                                     const void* row_offsets,
                                                     alphasparseIndexType_t rowOffsetsType,
                                                     int parts, int64_t* bounds);
/* local_offsets[i] = row_offsets[row_begin+i] - row_offsets[row_begin] for
 * i in [0, row_end-row_begin]; the output width may differ from the input width (a shard
 * with fewer than 2^31 nnz can use I32).  Device pointers, stream-ordered. */
alphasparseStatus_t alphasparseCsrRebaseRowOffsets(alphasparseHandle_t handle,
                                                   const void* row_offsets,
                                                   alphasparseIndexType_t inType,
                                                   int64_t row_begin, int64_t row_end,
                                                   void* local_offsets,
                                                   alphasparseIndexType_t outType);

/* Smallest and largest column index in col_idx[0, nnz) (DEVICE pointer, I32), written to HOST
 * integers; nnz = 0 gives {0, -1}.  A rank of a row-sharded matrix needs only
 * x[min_col, max_col]: for a banded matrix that is its own rows plus a halo.  Allocates 16 bytes
 * and synchronises handle->stream (a set-up call, not part of the SpMV path). */
alphasparseStatus_t alphasparseCsrColumnRange(alphasparseHandle_t handle, int64_t nnz,
                                              const void* col_idx, alphasparseIndexType_t colType,
                                              int64_t* min_col, int64_t* max_col);
/* A dense vector of logical length size of which only elements [first, first+count) exist, stored
 * at window_values[0, count).  alphasparseSpMV with such an x is valid when every column index of
 * A lies inside the window (alphasparseCsrColumnRange); nothing outside it is read.  As y it is
 * valid only for a matrix whose rows are the window.  No counterpart in the reference (its
 * vectors are always whole, handle.h:478-485). */
alphasparseStatus_t alphasparseCreateDnVecWindow(alphasparseDnVecDescr_t* descr, int64_t size,
                                                 int64_t first, int64_t count,
                                                 void* window_values, alphasparseDataType data_type);

/* ---- multi-GPU SpMV (extension; the reference is single-device) ----------------------- *
 * One process (or thread) per GPU.  Every rank holds a contiguous row range of one matrix
 * (alphasparseCsrPartitionRowsByNnz + alphasparseCsrRebaseRowOffsets; column indices stay
 * global) and the matching part of y; x is brought into the rank's own memory through NCCL
 * before its kernels read it.  The communicator is the caller's (an ncclComm_t passed as
 * void*); NCCL is looked up at run time, so this library loads without it and these calls
 * return NOT_SUPPORTED when no libnccl.so.2 can be found.  Work is ordered on handle->stream
 * (the overlapped mode adds one high-priority stream of its own, tied in with events).
 * Nothing here waits on the device; a failing peer shows as a status: arguments that do not
 * match the communicator are refused before anything is enqueued, and every call ends with one
 * non-blocking ncclCommGetAsyncError look (EXECUTION_FAILED when the communicator reports an
 * error). */
struct alphasparseMg;
typedef struct alphasparseMg* alphasparseMgHandle_t;
typedef enum {
  ALPHASPARSE_MG_X_BROADCAST = 0,      /* x whole on rank `root`, ncclBroadcast before the product */
  ALPHASPARSE_MG_X_ALLGATHER = 1,      /* x sharded; every rank collects the whole vector */
  ALPHASPARSE_MG_X_WINDOW = 2,         /* x sharded; a rank receives only x[min_col, max_col] of its rows */
  ALPHASPARSE_MG_X_WINDOW_OVERLAP = 3  /* WINDOW with the halo hidden behind the rows that need none */
} alphasparseMgExchange_t;
/* comm: ncclComm_t of `world` ranks in which this process is `rank` (checked); ignored when
 * world == 1.  The handle's device must be the communicator's. */
alphasparseStatus_t alphasparseMgCreate(alphasparseMgHandle_t* mg, alphasparseHandle_t handle,
                                        void* ncclComm, int rank, int world);
alphasparseStatus_t alphasparseMgDestroy(alphasparseMgHandle_t mg);
/* Set-up for one shard (allocates, synchronises, collective over the communicator: every rank
 * calls it).  matA_local: this rank's rows, column indices global, cols = length of x; fp32 or
 * fp64.  x_bounds (HOST, world+1 ascending, x_bounds[0] = 0, x_bounds[world] = cols): rank p owns
 * x[x_bounds[p], x_bounds[p+1]) - for a square matrix the row bounds; unused (may be NULL) for
 * BROADCAST, where `root` names the rank that holds x. */
alphasparseStatus_t alphasparseMgSetShard(alphasparseMgHandle_t mg, alphasparseSpMatDescr_t matA_local,
                                          const int64_t* x_bounds, alphasparseMgExchange_t mode,
                                          int root);
/* y_local = alpha * A_local * x + beta * y_local.  x (DEVICE): BROADCAST - the whole vector on
 * root (replicated in place), ignored elsewhere; other modes - this rank's own part of x, or the
 * pointer alphasparseMgOwnView returned (then no local copy is made).  alpha, beta: HOST
 * pointers of the matrix type.  Asynchronous. */
alphasparseStatus_t alphasparseMgSpMV(alphasparseMgHandle_t mg, const void* alpha, const void* x,
                                      const void* beta, void* y_local, alphasparseSpMVAlg_t alg);
/* The exchange step alone (what alphasparseMgSpMV runs before the product in the modes without
 * overlap), on handle->stream. */
alphasparseStatus_t alphasparseMgExchange(alphasparseMgHandle_t mg, const void* x);
/* Where this rank's own part of x lives inside its window buffer, for callers that keep x
 * there: element i of *ptr is x[*first + i].  NOT_SUPPORTED when the window does not hold the
 * whole own part (peers are sent from the caller's array then). */
alphasparseStatus_t alphasparseMgOwnView(alphasparseMgHandle_t mg, void** ptr, int64_t* first,
                                         int64_t* count);
enum {
  ASP_MG_INFO_WINDOW_LO = 0, ASP_MG_INFO_WINDOW_HI = 1, ASP_MG_INFO_BYTES_RECEIVED = 2,
  ASP_MG_INFO_INTERIOR_BEGIN = 3, ASP_MG_INFO_INTERIOR_END = 4, ASP_MG_INFO_NUM_SENDS = 5,
  ASP_MG_INFO_NUM_RECVS = 6, ASP_MG_INFO_MODE = 7, ASP_MG_INFO_COUNT = 8
};
alphasparseStatus_t alphasparseMgGetInfo(alphasparseMgHandle_t mg, int64_t* info /* ASP_MG_INFO_COUNT */);
/* Host-only planning of the window exchange (no GPU, no NCCL): rank p owns
 * x[own_bounds[p], own_bounds[p+1]) and needs x[windows[2p], windows[2p+1]) (nothing when the
 * second is not larger).  Outputs, triples (peer, begin, end) in global element indices, peers
 * ascending, the rank's own overlap listed with peer == rank: sends[3*world], recvs[3*world]. */
alphasparseStatus_t alphasparseMgExchangePlan(int world, int rank, const int64_t* own_bounds,
                                              const int64_t* windows, int64_t* sends, int* n_sends,
                                              int64_t* recvs, int* n_recvs);
/* Thin wrappers over ncclGetUniqueId / ncclCommInitRank / ncclCommDestroy of the NCCL this
 * library resolved, for callers that have no NCCL binding of their own (id128: 128 bytes, made
 * on one rank and handed to the others by any means). */
alphasparseStatus_t alphasparseMgGetUniqueId(void* id128);
alphasparseStatus_t alphasparseMgCommInitRank(void** ncclComm, int world, const void* id128, int rank);
alphasparseStatus_t alphasparseMgCommDestroy(void* ncclComm);

/* ---- the step before the path: MatrixMarket file -> COO (host) ------------------------- */
/* cuda/test/io.cu:1227-1238 (alpha_read_coo<T>(file, &m, &n, &nnz, &row_index, &col_index,
 * &values)), MatrixMarket part (:103-184, :490-575).  Reads a coordinate file into HOST arrays
 * allocated with malloc (release them with alphasparseFreeHost): zero-based indices, value 1
 * for pattern entries, and for symmetric / Hermitian / skew-symmetric files each off-diagonal
 * entry followed by its mirror image with the same value, as the reference's reader does.
 * valueType R_32F or R_64F.  Status instead of exit(): INVALID_VALUE for a missing or malformed
 * file or an index outside the announced size, NOT_SUPPORTED for array or complex files. */
alphasparseStatus_t alphasparseReadMtxCoo(const char* file, int64_t* rows, int64_t* cols, int64_t* nnz,
                                          int32_t** row_index, int32_t** col_index, void** values,
                                          alphasparseDataType valueType);
/* The binary dump format of the reference's drivers (header: cuda/test/include/io.h:41-50; records:
 * cuda/test/io.cu:596-725): eight int64 (rows, cols, records, entries after mirroring, value fields
 * per record, number type, symmetry, reserved), then per record int32 row, int32 column (one-based)
 * and 0, 1 or 2 doubles.  Same outputs and conventions as alphasparseReadMtxCoo (pattern -> 1, the
 * real part of a complex value, symmetric files mirrored). */
alphasparseStatus_t alphasparseReadBinCoo(const char* file, int64_t* rows, int64_t* cols, int64_t* nnz,
                                          int32_t** row_index, int32_t** col_index, void** values,
                                          alphasparseDataType valueType);
void alphasparseFreeHost(void* p);
/* cuda/format/coo_order.h:25-43: HOST arrays sorted by (row, column), stable. */
alphasparseStatus_t alphasparseCooOrder(int64_t nnz, int32_t* row_index, int32_t* col_index,
                                        void* values, alphasparseDataType valueType);

/* ---- the step before the path: COO -> CSR row offsets -------------------------------- */
/* cuda/format/coo2csr.h:82-92 (template alphasparseXcoo2csr<T>(row_data, nnz, m, csrRowPtr), default
 * stream).  cooRowInd: DEVICE array of nnz ascending, zero-based row indices; csrRowPtr: DEVICE array
 * of m+1 offsets (I32 or I64).  Stream-ordered on `stream`, no allocation. */
alphasparseStatus_t alphasparseXcoo2csr(cudaStream_t stream, const int32_t* cooRowInd, int64_t nnz,
                                        int64_t m, void* csrRowPtr,
                                        alphasparseIndexType_t rowOffsetsType);

/* ---- introspection (extension) ------------------------------------------------------ */
/* Copies the analysed plan to host arrays for bit-exact comparison with a CPU twin.
 * Any output pointer may be NULL.  stats[16]: see ASP_STAT_* below. */
enum {
  ASP_STAT_MAX_LEN = 0, ASP_STAT_EMPTY_ROWS = 1, ASP_STAT_NUM_SHORT = 2, ASP_STAT_NUM_MEDIUM = 3,
  ASP_STAT_NUM_LONG = 4, ASP_STAT_GROUP_LANES = 5, ASP_STAT_MERGE_ITEMS = 6,
  ASP_STAT_MERGE_TILES = 7, ASP_STAT_VARIANT = 8, ASP_STAT_IDENTITY_SHORT = 9,
  ASP_STAT_NNZ_SHORT = 10, ASP_STAT_DEVICE_ERROR = 11 /* 1 if a kernel's bounded wait ever expired */,
  ASP_STAT_COL_STEP = 12 /* mean |first column of row r+1 - first column of row r|, rounded */,
  ASP_STAT_COUNT = 16
};
alphasparseStatus_t alphasparseCsrPlanGet(alphasparseHandle_t handle,
                                          alphasparseSpMatDescr_t matA, int64_t* stats,
                                          int32_t* bin_rows /* rows */,
                                          int32_t* merge_tile_row /* tiles+1 */);
/* Name of the SpMV kernel variant the last alphasparseSpMV call on this matrix ran
 * ("binned" or "merge"), and how many kernels this library has launched on the handle. */
const char* alphasparseCsrLastVariant(alphasparseSpMatDescr_t matA);
/* The SpMM kernel family of the last alphasparseSpMM call on this matrix. */
const char* alphasparseCsrLastSpmmVariant(alphasparseSpMatDescr_t matA);
int64_t alphasparseGetLaunchCount(alphasparseHandle_t handle);

/* ---- timers the reference's test drivers call: handle.h:532-539, handle.cu:547-599 --- */
double get_time_us(void);
double get_avg_time_n(const double* times, int n);   /* outlier-filtered mean, handle.cu:556-573 */

#ifdef __cplusplus
} /* extern "C" */
#include <algorithm>
#include <vector>
/* handle.h:532-539, cuda/util/handle.cu:556-599: the overloads the reference's drivers call. */
inline double get_avg_time(std::vector<double> times) {
  return get_avg_time_n(times.data(), (int)times.size());
}
/* Mean of the samples within 10 % of the median; the median itself when none is. */
inline double get_avg_time_2(std::vector<double> times) {
  if (times.empty()) return 0.0;
  std::sort(times.begin(), times.end());
  const size_t n = times.size();
  const double med = n % 2 ? times[n / 2] : 0.5 * (times[n / 2 - 1] + times[n / 2]);
  double sum = 0;
  size_t kept = 0;
  for (double t : times)
    if (t >= 0.9 * med && t <= 1.1 * med) {
      sum += t;
      ++kept;
    }
  return kept ? sum / (double)kept : med;
}

/* Source compatibility with the reference's template creator
 * (cuda/format/alphasparse_create_csr.h:6-18). */
template <typename T>
inline alphasparseStatus_t alphasparseCreateCsr(alphasparseSpMatDescr_t* spMatDescr,
                                                const int rows, const int cols, const int nnz,
                                                int* csrRowOffsets, int* col_data, T* val_data,
                                                const alphasparseIndexType_t csrRowOffsetsType,
                                                const alphasparseIndexType_t csrColIndType,
                                                const alphasparseIndexBase_t idxBase,
                                                const alphasparseDataType valueType) {
  return alphasparseCreateCsr(spMatDescr, (int64_t)rows, (int64_t)cols, (int64_t)nnz,
                              (void*)csrRowOffsets, (void*)col_data, (void*)val_data,
                              csrRowOffsetsType, csrColIndType, idxBase, valueType);
}
/* Source compatibility with cuda/format/coo2csr.h:82-92 (default stream, as there). */
template <typename T>
inline alphasparseStatus_t alphasparseXcoo2csr(const int* row_data, int nnz, int m, T* csrRowPtr) {
  static_assert(sizeof(T) == 4 || sizeof(T) == 8, "row offsets are 32- or 64-bit integers");
  return alphasparseXcoo2csr((cudaStream_t)0, row_data, (int64_t)nnz, (int64_t)m, (void*)csrRowPtr,
                             sizeof(T) == 8 ? ALPHA_SPARSE_INDEXTYPE_I64 : ALPHA_SPARSE_INDEXTYPE_I32);
}
#endif
#endif /* ALPHASPARSE_B200_H */
