// CSR SpMM for the remaining type combinations of the reference's dispatcher
// (cuda/kernel/level3/alphasparse_spmm.cu:556-596):  C = alpha * A * B + beta * C, row-major B and C, with
//   C_32F / C_64F   : complex A, B, C, alpha, beta; fused multiply-adds on the real and imaginary parts;
//   R_8I  -> R_32I  : products and sums in int32, alpha and beta host int32;
//   R_8I  -> R_32F  : values widened to fp32, fp32 arithmetic, alpha and beta host floats;
//   R_16F -> R_32F  : fp16 A and B widened to fp32, fp32 sums and C;
//   R_16F -> R_16F  : the same with C in fp16 (compute type fp32, one rounding at the end).
//
// One plain kernel: a warp owns a row, its lanes 32 neighbouring columns of B and C at a time; the
// row's entries are taken in storage order, so a sum does not depend on the launch.  These
// instances exist for coverage of the reference's type table; the tuned kernels are the fp32 /
// fp64 ones (spmm.cu, spmm_balanced.cu) and the bf16 tensor-core ones (spmm_tc.cu).
#include <cuComplex.h>
#include <cuda_fp16.h>

#include <climits>

#include "asp_internal.h"

namespace asp {
namespace {

// The arithmetic of one instance: TA (A and B), TY (C), TC (products, sums, alpha, beta).
template <typename TA, typename TY, typename TC> struct MmArith;

template <> struct MmArith<cuFloatComplex, cuFloatComplex, cuFloatComplex> {
  using C = cuFloatComplex;
  static __device__ __forceinline__ C zero() { return make_cuFloatComplex(0.f, 0.f); }
  static __device__ __forceinline__ C mad(C a, C x, C s) {
    return make_cuFloatComplex(fmaf(-a.y, x.y, fmaf(a.x, x.x, s.x)), fmaf(a.y, x.x, fmaf(a.x, x.y, s.y)));
  }
  static __device__ __forceinline__ bool is_zero(C b) { return b.x == 0.f && b.y == 0.f; }
  static __device__ __forceinline__ C finish(C alpha, C s, C beta, const C* y) {
    const C r = mad(alpha, s, zero());
    return is_zero(beta) ? r : mad(beta, *y, r);
  }
};
template <> struct MmArith<cuDoubleComplex, cuDoubleComplex, cuDoubleComplex> {
  using C = cuDoubleComplex;
  static __device__ __forceinline__ C zero() { return make_cuDoubleComplex(0.0, 0.0); }
  static __device__ __forceinline__ C mad(C a, C x, C s) {
    return make_cuDoubleComplex(fma(-a.y, x.y, fma(a.x, x.x, s.x)), fma(a.y, x.x, fma(a.x, x.y, s.y)));
  }
  static __device__ __forceinline__ bool is_zero(C b) { return b.x == 0.0 && b.y == 0.0; }
  static __device__ __forceinline__ C finish(C alpha, C s, C beta, const C* y) {
    const C r = mad(alpha, s, zero());
    return is_zero(beta) ? r : mad(beta, *y, r);
  }
};
template <> struct MmArith<int8_t, int32_t, int32_t> {
  using C = int32_t;
  static __device__ __forceinline__ C zero() { return 0; }
  static __device__ __forceinline__ C mad(int8_t a, int8_t x, C s) { return s + (int32_t)a * (int32_t)x; }
  static __device__ __forceinline__ bool is_zero(C b) { return b == 0; }
  static __device__ __forceinline__ int32_t finish(C alpha, C s, C beta, const int32_t* y) {
    return is_zero(beta) ? alpha * s : alpha * s + beta * (*y);
  }
};
template <> struct MmArith<int8_t, float, float> {
  using C = float;
  static __device__ __forceinline__ C zero() { return 0.f; }
  static __device__ __forceinline__ C mad(int8_t a, int8_t x, C s) { return fmaf((float)a, (float)x, s); }
  static __device__ __forceinline__ bool is_zero(C b) { return b == 0.f; }
  static __device__ __forceinline__ float finish(C alpha, C s, C beta, const float* y) {
    return is_zero(beta) ? alpha * s : fmaf(alpha, s, beta * (*y));
  }
};
template <> struct MmArith<__half, float, float> {
  using C = float;
  static __device__ __forceinline__ C zero() { return 0.f; }
  static __device__ __forceinline__ C mad(__half a, __half x, C s) { return fmaf(__half2float(a), __half2float(x), s); }
  static __device__ __forceinline__ bool is_zero(C b) { return b == 0.f; }
  static __device__ __forceinline__ float finish(C alpha, C s, C beta, const float* y) {
    return is_zero(beta) ? alpha * s : fmaf(alpha, s, beta * (*y));
  }
};
template <> struct MmArith<__half, __half, float> {
  using C = float;
  static __device__ __forceinline__ C zero() { return 0.f; }
  static __device__ __forceinline__ C mad(__half a, __half x, C s) { return fmaf(__half2float(a), __half2float(x), s); }
  static __device__ __forceinline__ bool is_zero(C b) { return b == 0.f; }
  static __device__ __forceinline__ __half finish(C alpha, C s, C beta, const __half* y) {
    return __float2half_rn(is_zero(beta) ? alpha * s : fmaf(alpha, s, beta * __half2float(*y)));
  }
};

template <typename TA, typename TY, typename TC, typename OffT>
__global__ void __launch_bounds__(kThreads)
spmm_types_kernel(const OffT* __restrict__ rp, const int* __restrict__ col, const TA* __restrict__ val,
                  const TA* __restrict__ B, int64_t ldb, TY* __restrict__ C, int64_t ldc, TC alpha, TC beta,
                  int64_t rows, int64_t n) {
  using Ar = MmArith<TA, TY, TC>;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
  if (row >= rows) return;  // the whole warp leaves together
  const int64_t s = (int64_t)rp[row], e = (int64_t)rp[row + 1];
  for (int64_t j0 = 0; j0 < n; j0 += 32) {
    const int64_t j = j0 + lane;
    TC sum = Ar::zero();
    if (j < n)
      for (int64_t k = s; k < e; ++k) sum = Ar::mad(val[k], B[(int64_t)col[k] * ldb + j], sum);
    if (j < n) C[row * ldc + j] = Ar::finish(alpha, sum, beta, C + row * ldc + j);
  }
}

template <typename TA, typename TY, typename TC, typename OffT>
alphasparseStatus_t run_t(alphasparseHandle_t h, alphasparseSpMatDescr_t A, alphasparseDnMatDescr_t B,
                          alphasparseDnMatDescr_t C, const void* alpha, const void* beta) {
  const int64_t per_cta = kThreads / 32;
  const int64_t grid = (A->rows + per_cta - 1) / per_cta;
  if (grid > INT_MAX) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (grid == 0 || C->cols == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  spmm_types_kernel<TA, TY, TC, OffT><<<(unsigned)grid, kThreads, 0, h->stream>>>(
      reinterpret_cast<const OffT*>(A->row_offsets), A->const_col_data, reinterpret_cast<const TA*>(A->const_val_data),
      reinterpret_cast<const TA*>(B->values), B->ld, reinterpret_cast<TY*>(C->values), C->ld,
      *reinterpret_cast<const TC*>(alpha), *reinterpret_cast<const TC*>(beta), A->rows, C->cols);
  impl(h)->launches++;
  return status_of(cudaGetLastError());
}

}  // namespace

bool spmm_other_types(alphasparseDataType a, alphasparseDataType b, alphasparseDataType c, alphasparseDataType compute) {
  if (b != a) return false;
  if (a == ALPHA_C_32F || a == ALPHA_C_64F) return c == a && compute == a;
  if (a == ALPHA_R_8I) return (c == ALPHA_R_32I && compute == ALPHA_R_32I) || (c == ALPHA_R_32F && compute == ALPHA_R_32F);
  if (a == ALPHA_R_16F) return (c == ALPHA_R_32F || c == ALPHA_R_16F) && compute == ALPHA_R_32F;
  return false;
}

// True when beta (a host value of the compute type) is not zero, i.e. C is read.
bool spmm_other_reads_c(alphasparseDataType compute, const void* beta) {
  switch (compute) {
    case ALPHA_C_32F: return reinterpret_cast<const float*>(beta)[0] != 0.f || reinterpret_cast<const float*>(beta)[1] != 0.f;
    case ALPHA_C_64F: return reinterpret_cast<const double*>(beta)[0] != 0.0 || reinterpret_cast<const double*>(beta)[1] != 0.0;
    case ALPHA_R_32I: return *reinterpret_cast<const int32_t*>(beta) != 0;
    default: return *reinterpret_cast<const float*>(beta) != 0.f;
  }
}

alphasparseStatus_t spmm_other_run(alphasparseHandle_t h, alphasparseSpMatDescr_t A, alphasparseDnMatDescr_t B,
                                   alphasparseDnMatDescr_t C, const void* alpha, const void* beta) {
  if (A->rows == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  const bool o64 = A->row_type == ALPHA_SPARSE_INDEXTYPE_I64;
#define ASP_RUN(TA, TY, TC) \
  (o64 ? run_t<TA, TY, TC, int64_t>(h, A, B, C, alpha, beta) : run_t<TA, TY, TC, int32_t>(h, A, B, C, alpha, beta))
  switch (A->data_type) {
    case ALPHA_C_32F: return ASP_RUN(cuFloatComplex, cuFloatComplex, cuFloatComplex);
    case ALPHA_C_64F: return ASP_RUN(cuDoubleComplex, cuDoubleComplex, cuDoubleComplex);
    case ALPHA_R_8I:
      return C->data_type == ALPHA_R_32I ? ASP_RUN(int8_t, int32_t, int32_t) : ASP_RUN(int8_t, float, float);
    case ALPHA_R_16F:
      return C->data_type == ALPHA_R_16F ? ASP_RUN(__half, __half, float) : ASP_RUN(__half, float, float);
    default: return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  }
#undef ASP_RUN
}

}  // namespace asp
