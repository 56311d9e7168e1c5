// CSR SpMV for the remaining value types of the reference's dispatcher
// (cuda/kernel/level2/alphasparse_spmv.cu:246-262 complex float / complex double,
// :276-287 int8 A and x with int32 or fp32 y):  y = alpha * A * x + beta * y  with
//   C_32F / C_64F : complex A, x, y, alpha, beta; fused multiply-adds on the real and imaginary parts;
//   R_8I  -> R_32I: products and sums in int32, alpha and beta host int32;
//   R_8I  -> R_32F: values widened to fp32, fp32 arithmetic, alpha and beta host floats.
//
// One kernel over the row-length classes of the analysis plan: short rows are shared by G lanes,
// medium rows get a warp, long rows a CTA; lanes step through a row entry by entry, neighbouring
// lanes on neighbouring entries, and combine with xor shuffles.  These instances exist for
// coverage of the reference's type table; the tuned kernels are the fp32 / fp64 / 16-bit ones.
#include <cuComplex.h>

#include <climits>

#include "asp_internal.h"

namespace asp {
namespace {

// The arithmetic of one instance: TA (A and x), TY (y), TC (products, sums, alpha, beta).
template <typename TA, typename TY, typename TC> struct Arith;

template <> struct Arith<cuFloatComplex, cuFloatComplex, cuFloatComplex> {
  using C = cuFloatComplex;
  static __device__ __forceinline__ C zero() { return make_cuFloatComplex(0.f, 0.f); }
  static __device__ __forceinline__ C mad(cuFloatComplex a, cuFloatComplex x, C s) {
    return make_cuFloatComplex(fmaf(-a.y, x.y, fmaf(a.x, x.x, s.x)), fmaf(a.y, x.x, fmaf(a.x, x.y, s.y)));
  }
  static __device__ __forceinline__ C add(C a, C b) { return cuCaddf(a, b); }
  static __device__ __forceinline__ C shfl(C v, int o) {
    return make_cuFloatComplex(__shfl_xor_sync(0xffffffffu, v.x, o), __shfl_xor_sync(0xffffffffu, v.y, o));
  }
  static __device__ __forceinline__ bool is_zero(C b) { return b.x == 0.f && b.y == 0.f; }
  static __device__ __forceinline__ cuFloatComplex finish(C alpha, C s, C beta, const cuFloatComplex* y) {
    C r = mad(alpha, s, zero());
    return is_zero(beta) ? r : add(r, mad(beta, *y, zero()));
  }
};
template <> struct Arith<cuDoubleComplex, cuDoubleComplex, cuDoubleComplex> {
  using C = cuDoubleComplex;
  static __device__ __forceinline__ C zero() { return make_cuDoubleComplex(0.0, 0.0); }
  static __device__ __forceinline__ C mad(cuDoubleComplex a, cuDoubleComplex x, C s) {
    return make_cuDoubleComplex(fma(-a.y, x.y, fma(a.x, x.x, s.x)), fma(a.y, x.x, fma(a.x, x.y, s.y)));
  }
  static __device__ __forceinline__ C add(C a, C b) { return cuCadd(a, b); }
  static __device__ __forceinline__ C shfl(C v, int o) {
    return make_cuDoubleComplex(__shfl_xor_sync(0xffffffffu, v.x, o), __shfl_xor_sync(0xffffffffu, v.y, o));
  }
  static __device__ __forceinline__ bool is_zero(C b) { return b.x == 0.0 && b.y == 0.0; }
  static __device__ __forceinline__ cuDoubleComplex finish(C alpha, C s, C beta, const cuDoubleComplex* y) {
    C r = mad(alpha, s, zero());
    return is_zero(beta) ? r : add(r, mad(beta, *y, zero()));
  }
};
template <> struct Arith<int8_t, int32_t, int32_t> {
  using C = int32_t;
  static __device__ __forceinline__ C zero() { return 0; }
  static __device__ __forceinline__ C mad(int8_t a, int8_t x, C s) { return s + (int32_t)a * (int32_t)x; }
  static __device__ __forceinline__ C add(C a, C b) { return a + b; }
  static __device__ __forceinline__ C shfl(C v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }
  static __device__ __forceinline__ bool is_zero(C b) { return b == 0; }
  static __device__ __forceinline__ int32_t finish(C alpha, C s, C beta, const int32_t* y) {
    return is_zero(beta) ? alpha * s : alpha * s + beta * (*y);
  }
};
template <> struct Arith<int8_t, float, float> {
  using C = float;
  static __device__ __forceinline__ C zero() { return 0.f; }
  static __device__ __forceinline__ C mad(int8_t a, int8_t x, C s) { return fmaf((float)a, (float)x, s); }
  static __device__ __forceinline__ C add(C a, C b) { return a + b; }
  static __device__ __forceinline__ C shfl(C v, int o) { return __shfl_xor_sync(0xffffffffu, v, o); }
  static __device__ __forceinline__ bool is_zero(C b) { return b == 0.f; }
  static __device__ __forceinline__ float finish(C alpha, C s, C beta, const float* y) {
    return is_zero(beta) ? alpha * s : fmaf(alpha, s, beta * (*y));
  }
};

template <typename TA, typename TY, typename TC, typename OffT>
struct TypeArgs {
  const OffT* rp;
  const int* col;
  const TA* val;
  const TA* x;
  TY* y;
  TC alpha, beta;
  const int32_t* rows_short;   // nullptr: row i of the class is row i of the matrix
  const int32_t* rows_medium;
  const int32_t* rows_long;
  int64_t n_short, n_medium, n_long;
  int cta_short, cta_medium;
};

template <typename TA, typename TY, typename TC, typename OffT, int G>
__global__ void __launch_bounds__(kThreads) spmv_types_kernel(const TypeArgs<TA, TY, TC, OffT> a) {
  using Ar = Arith<TA, TY, TC>;
  const int b = blockIdx.x;
  if (b < a.cta_short) {
    constexpr int NG = kThreads / G;
    const int lane = threadIdx.x & (G - 1);
    const int64_t i = (int64_t)b * NG + threadIdx.x / G;
    const int32_t row = i < a.n_short ? (a.rows_short ? a.rows_short[i] : (int32_t)i) : -1;
    TC sum = Ar::zero();
    if (row >= 0) {
      const int64_t s = (int64_t)a.rp[row], e = (int64_t)a.rp[row + 1];
      for (int64_t k = s + lane; k < e; k += G) sum = Ar::mad(a.val[k], a.x[a.col[k]], sum);
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) sum = Ar::add(sum, Ar::shfl(sum, o));
    if (lane == 0 && row >= 0) a.y[row] = Ar::finish(a.alpha, sum, a.beta, a.y + row);
  } else if (b < a.cta_short + a.cta_medium) {
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t)(b - a.cta_short) * (kThreads / 32) + (threadIdx.x >> 5);
    if (i >= a.n_medium) return;  // whole warp leaves together
    const int32_t row = a.rows_medium[i];
    const int64_t s = (int64_t)a.rp[row], e = (int64_t)a.rp[row + 1];
    TC sum = Ar::zero();
    for (int64_t k = s + lane; k < e; k += 32) sum = Ar::mad(a.val[k], a.x[a.col[k]], sum);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum = Ar::add(sum, Ar::shfl(sum, o));
    if (lane == 0) a.y[row] = Ar::finish(a.alpha, sum, a.beta, a.y + row);
  } else {
    __shared__ TC s_part[kThreads / 32];
    const int64_t i = (int64_t)(b - a.cta_short - a.cta_medium);
    const int32_t row = a.rows_long[i];
    const int64_t s = (int64_t)a.rp[row], e = (int64_t)a.rp[row + 1];
    TC sum = Ar::zero();
    for (int64_t k = s + threadIdx.x; k < e; k += kThreads) sum = Ar::mad(a.val[k], a.x[a.col[k]], sum);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum = Ar::add(sum, Ar::shfl(sum, o));
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
      TC tot = Ar::zero();
#pragma unroll
      for (int w = 0; w < kThreads / 32; ++w) tot = Ar::add(tot, s_part[w]);
      a.y[row] = Ar::finish(a.alpha, tot, a.beta, a.y + row);
    }
  }
}

template <typename TA, typename TY, typename TC, typename OffT>
alphasparseStatus_t run_t(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const Plan* p, const void* x, void* y,
                          const void* alpha, const void* beta) {
  TypeArgs<TA, TY, TC, OffT> a;
  a.rp = reinterpret_cast<const OffT*>(A->row_offsets);
  a.col = A->const_col_data;
  a.val = reinterpret_cast<const TA*>(A->const_val_data);
  a.x = reinterpret_cast<const TA*>(x);
  a.y = reinterpret_cast<TY*>(y);
  a.alpha = *reinterpret_cast<const TC*>(alpha);
  a.beta = *reinterpret_cast<const TC*>(beta);
  a.rows_short = p->identity_short ? nullptr : p->bin_rows;
  a.rows_medium = p->identity_short ? nullptr : p->bin_rows + p->n_short;
  a.rows_long = p->identity_short ? nullptr : p->bin_rows + p->n_short + p->n_medium;
  a.n_short = p->n_short;
  a.n_medium = p->n_medium;
  a.n_long = p->n_long;
  // one entry per lane and step: twice the plan's lanes per short row (chosen for 16-byte loads), at most a warp
  int g = p->group_lanes * 2;
  if (g > 32) g = 32;
  const int rows_per_cta = kThreads / g;
  const int64_t cs = (p->n_short + rows_per_cta - 1) / rows_per_cta;
  const int64_t cm = (p->n_medium + (kThreads / 32) - 1) / (kThreads / 32);
  const int64_t total = cs + cm + p->n_long;
  if (total > INT_MAX) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (total == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  a.cta_short = (int)cs;
  a.cta_medium = (int)cm;
  const dim3 grid((unsigned)total), block(kThreads);
  switch (g) {
    case 4: spmv_types_kernel<TA, TY, TC, OffT, 4><<<grid, block, 0, h->stream>>>(a); break;
    case 8: spmv_types_kernel<TA, TY, TC, OffT, 8><<<grid, block, 0, h->stream>>>(a); break;
    case 16: spmv_types_kernel<TA, TY, TC, OffT, 16><<<grid, block, 0, h->stream>>>(a); break;
    default: spmv_types_kernel<TA, TY, TC, OffT, 32><<<grid, block, 0, h->stream>>>(a); break;
  }
  impl(h)->launches++;
  return status_of(cudaGetLastError());
}

}  // namespace

bool spmv_other_types(alphasparseDataType a, alphasparseDataType x, alphasparseDataType y, alphasparseDataType compute) {
  if (x != a) return false;
  if (a == ALPHA_C_32F || a == ALPHA_C_64F) return y == a && compute == a;
  if (a == ALPHA_R_8I) return (y == ALPHA_R_32I && compute == ALPHA_R_32I) || (y == ALPHA_R_32F && compute == ALPHA_R_32F);
  return false;
}

alphasparseStatus_t spmv_other_run(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const Plan* p, const void* x,
                                   void* y, alphasparseDataType y_type, const void* alpha, const void* beta) {
  if (p->rows == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  const bool o64 = A->row_type == ALPHA_SPARSE_INDEXTYPE_I64;
#define ASP_RUN(TA, TY, TC) \
  (o64 ? run_t<TA, TY, TC, int64_t>(h, A, p, x, y, alpha, beta) : run_t<TA, TY, TC, int32_t>(h, A, p, x, y, alpha, beta))
  switch (A->data_type) {
    case ALPHA_C_32F: return ASP_RUN(cuFloatComplex, cuFloatComplex, cuFloatComplex);
    case ALPHA_C_64F: return ASP_RUN(cuDoubleComplex, cuDoubleComplex, cuDoubleComplex);
    case ALPHA_R_8I:
      return y_type == ALPHA_R_32I ? ASP_RUN(int8_t, int32_t, int32_t) : ASP_RUN(int8_t, float, float);
    default: return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  }
#undef ASP_RUN
}

}  // namespace asp
