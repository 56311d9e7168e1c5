// Internal declarations shared by the translation units of libalphasparse_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <cstdint>
#include <cstdlib>

#include "alphasparse_b200.h"

namespace asp {

// ---- tuning constants of the preprocessing pass -----------------------------------------
// Row classes of the binned SpMV, by number of entries L in a row:
//   short  (L <= kShortMax)  : a group of G lanes per row (G = 2..32, one value per matrix)
//   medium (L <= kMediumMax) : one warp per row
//   long                     : one CTA per row
constexpr int kShortMax = 64;
constexpr int kMediumMax = 4096;
constexpr int kThreads = 256;        // every SpMV / SpMM CTA
constexpr int kShortUnroll = 2;      // rows in flight per lane group
// Merge-path SpMV: each CTA consumes kMergeItems (rows + entries) of the merge list.
constexpr int kMergeIpt = 8;
constexpr int kMergeItems = kThreads * kMergeIpt;

// Fewer merge tiles than this (about 2.5 M items): the matrix is L2-resident and launch-bound.
constexpr int64_t kSmallProblemTiles = 1200;
// SpMM: rows per CTA and entries of A a CTA can stage at once.
#ifndef ASP_SPMM_ROW_BLOCK
#define ASP_SPMM_ROW_BLOCK 128
#endif
constexpr int kSpmmRowBlock = ASP_SPMM_ROW_BLOCK;
constexpr int kSpmmStageCap32 = 4096;  // 4-byte values
constexpr int kSpmmStageCap64 = 3584;  // 8-byte values (48 KB of static shared memory)

enum Variant { kVariantBinned = 0, kVariantMerge = 1 };

struct HandleImpl {
  int sm_count = 148;
  int64_t launches = 0;
  size_t smem_optin = 0;
  // sustained rates estimated from the device's own attributes (clocks, SM count, bus width):
  // what the tensor-core SpMM's density test weighs MMA work against memory traffic with
  double bf16_flops = 1.4e15, hbm_bytes = 6.5e12;
};

// The analysis result attached to a CSR descriptor (matA->info).
struct Plan {
  int device = 0;
  int64_t rows = 0, cols = 0, nnz = 0;
  bool off64 = false;
  // statistics
  int64_t max_len = 0, empty_rows = 0;
  double col_step = 0;  // mean |first column of row r+1 - first column of row r| over neighbouring non-empty rows
  int64_t n_short = 0, n_medium = 0, n_long = 0, nnz_short = 0;
  int group_lanes = 4;
  bool identity_short = false;      // every row is short: no row list is needed
  int32_t* bin_rows = nullptr;      // device, rows entries: short | medium | long, each in row order
  // merge path
  int64_t merge_tiles = 0;
  int32_t* merge_tile_row = nullptr;  // device, merge_tiles + 1
  void* carry = nullptr;              // device, merge_tiles * 8 bytes (used when no external buffer)
  // Device flag a kernel raises when a bounded wait expires (read back, after a synchronisation, by
  // alphasparseCsrPlanGet).
  int* dev_err = nullptr;
  // Polls a bounded device-side wait may take (bit 31: testing only - the copy the wait is for is not
  // issued, so the wait does run out; bit 30: testing only - no L2 policy on the copies of A).  Read from
  // ASP_WAIT_POLLS / ASP_TEST_DROP_COPY / ASP_TILE_L2_HINT at analysis.
  uint32_t wait_cfg = 1u << 22;
  int variant_auto = kVariantBinned;
  int last_variant = -1;
  const char* last_spmm = "none";   // name of the SpMM kernel family the last call ran
  // SpMM
  int64_t max_block_nnz = 0;          // most entries in an aligned block of kSpmmRowBlock rows
  void* spmm_carry = nullptr;         // device, carry array of the balanced SpMM when the caller gave no buffer
  size_t spmm_carry_bytes = 0;
  void* spmm_tc = nullptr;            // plan of the tcgen05 variant (spmm_tc.cu)
  void* spmm_stage = nullptr;         // chunk lists of the kernel that stages B by TMA (spmm_stage.cu)
  void* transposed = nullptr;         // CSR of the transposed matrix with its own descriptor and plan (analysis.cu)
};

inline HandleImpl* impl(alphasparseHandle_t h) { return reinterpret_cast<HandleImpl*>(h->impl); }
inline Plan* plan_of(alphasparseSpMatDescr_t A) { return reinterpret_cast<Plan*>(A->info); }

// cudaError -> status, the table of cuda/util/handle.cu:18-50 in the reference.
inline alphasparseStatus_t status_of(cudaError_t e) {
  switch (e) {
    case cudaSuccess: return ALPHA_SPARSE_STATUS_SUCCESS;
    case cudaErrorMemoryAllocation: return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    case cudaErrorInvalidValue: return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    case cudaErrorInvalidDevicePointer: return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    case cudaErrorInvalidResourceHandle: return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    case cudaErrorLaunchFailure:
    case cudaErrorLaunchTimeout:
    case cudaErrorLaunchOutOfResources: return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    default: return ALPHA_SPARSE_STATUS_INTERNAL_ERROR;
  }
}

#define ASP_CUDA(call)                                   \
  do {                                                   \
    cudaError_t e_ = (call);                             \
    if (e_ != cudaSuccess) return ::asp::status_of(e_);  \
  } while (0)

inline size_t elem_size(alphasparseDataType t) {
  switch (t) {
    case ALPHA_R_32F: return 4;
    case ALPHA_R_64F: return 8;
    case ALPHA_R_16BF: case ALPHA_R_16F: return 2;
    case ALPHA_C_32F: return 8;
    case ALPHA_C_64F: return 16;
    case ALPHA_R_8I: return 1;
    case ALPHA_R_32I: return 4;
    default: return 0;
  }
}

constexpr uint32_t kWaitDropCopy = 1u << 31;
constexpr uint32_t kWaitNoL2Hint = 1u << 30;  // testing: bulk copies of A without the L2 evict-first policy
constexpr uint32_t kWaitPollMask = (1u << 30) - 1;

inline int env_int(const char* name, int dflt) {
  const char* s = getenv(name);
  return s && *s ? atoi(s) : dflt;
}

// analysis.cu
alphasparseStatus_t analyse(alphasparseHandle_t h, alphasparseSpMatDescr_t A);
void free_plan(Plan* p);
alphasparseStatus_t validate_csr(alphasparseSpMatDescr_t A);
// The CSR descriptor of A^T (built on the device at first use, owned by A's plan, analysed).
alphasparseStatus_t transposed_of(alphasparseHandle_t h, alphasparseSpMatDescr_t A, alphasparseSpMatDescr_t* At);

// spmm_tc.cu
void free_spmm_tc_plan(void* p);

// spmm_balanced.cu: the merge-path SpMM for skewed matrices; carry holds merge_tiles x carry_ld values
int64_t spmm_balanced_carry_ld(int64_t n, size_t elem);
template <typename T, typename OffT>
alphasparseStatus_t spmm_balanced_t(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const T* B, int64_t ldb, T* C,
                                    int64_t ldc, T alpha, T beta, int64_t n, void* carry);

// spmm_stage.cu: the kernel that stages B through shared memory by TMA.  *ran tells whether the product
// qualified (and, unless prepare_only, was launched); otherwise the caller runs another kernel.
void free_spmm_stage_plan(void* p);
template <typename T>
alphasparseStatus_t spmm_stage_try(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const T* B, int64_t ldb, T* C,
                                   int64_t ldc, T alpha, T beta, int64_t n, bool prepare_only, bool* ran);

// spmv_lowp.cu: 16-bit A and x with fp32 arithmetic (fp16 -> fp32 y, bf16 -> bf16 y)
bool spmv_lowp_types(alphasparseDataType a, alphasparseDataType x, alphasparseDataType y,
                     alphasparseDataType compute);
alphasparseStatus_t spmv_lowp_run(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const Plan* p,
                                  const void* x, void* y, float alpha, float beta);


// spmv_types.cu: complex and int8 instances of the reference's SpMV type table
// spmm_types.cu: complex, int8 and fp16 SpMM instances
bool spmm_other_types(alphasparseDataType a, alphasparseDataType b, alphasparseDataType c, alphasparseDataType compute);
bool spmm_other_reads_c(alphasparseDataType compute, const void* beta);
alphasparseStatus_t spmm_other_run(alphasparseHandle_t h, alphasparseSpMatDescr_t A, alphasparseDnMatDescr_t B,
                                   alphasparseDnMatDescr_t C, const void* alpha, const void* beta);
bool spmv_other_types(alphasparseDataType a, alphasparseDataType x, alphasparseDataType y, alphasparseDataType compute);
alphasparseStatus_t spmv_other_run(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const Plan* p, const void* x,
                                   void* y, alphasparseDataType y_type, const void* alpha, const void* beta);

}  // namespace asp
