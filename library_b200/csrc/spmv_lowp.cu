// CSR SpMV with 16-bit operands and fp32 accumulation: y = alpha * A * x + beta * y.
//
// Replaces the reference's mixed-precision instances of its SpMV dispatcher
// (cuda/kernel/level2/alphasparse_spmv.cu:288-292: half A and x, float y, float arithmetic;
// :294-300: nv_bfloat16 A, x and y, float arithmetic).  alpha and beta are host floats.
// Halving the bytes per entry of A (6 instead of 8) is the point: the kernel streams A.
//
// One kernel, the row-length classes of the analysis plan (asp_internal.h): short rows are shared
// by G lanes, medium rows get a warp, long rows a CTA.  A lane reads 16 bytes of values (eight
// entries) and the matching 32 bytes of column indices per step, starting on a multiple of eight
// entries (the row start is rounded down and the leading entries masked) so that neighbouring
// lanes read neighbouring lines; arrays that are not 16-byte aligned are read entry by entry.
// Products and sums are fp32; the result is rounded once when it is stored.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <climits>
#include <type_traits>

#include "asp_internal.h"

namespace asp {
namespace {

__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float to_f32(float v) { return v; }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

constexpr int kLowpChunk = 8;  // entries per 16-byte load of values

template <typename TA, typename TY, typename OffT>
struct LowpArgs {
  const OffT* rp;
  const int* col;
  const TA* val;
  const TA* x;
  TY* y;
  float alpha, beta;
  const int32_t* rows_short;   // nullptr: row i of the class is row i of the matrix
  const int32_t* rows_medium;
  const int32_t* rows_long;
  int64_t n_short, n_medium, n_long, nnz;
  int cta_short, cta_medium;
};

// Sum over the lane's eight entries starting at k (a multiple of eight) that lie inside [s, e).
template <typename TA, bool VL>
__device__ __forceinline__ float chunk_dot(const TA* __restrict__ val, const int* __restrict__ col,
                                           const TA* __restrict__ x, int64_t k, int64_t s, int64_t e,
                                           int64_t nnz) {
  float sum = 0.f;
  if (VL && k + kLowpChunk <= nnz) {
    const uint4 vv = __ldcs(reinterpret_cast<const uint4*>(val + k));
    const int4 c0 = __ldcs(reinterpret_cast<const int4*>(col + k));
    const int4 c1 = __ldcs(reinterpret_cast<const int4*>(col + k + 4));
    const uint32_t w[4] = {vv.x, vv.y, vv.z, vv.w};
    const int c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
    for (int j = 0; j < kLowpChunk; ++j) {
      const unsigned short bits = (unsigned short)(w[j >> 1] >> ((j & 1) * 16));
      TA v;
      *reinterpret_cast<unsigned short*>(&v) = bits;
      const int64_t kk = k + j;
      if (kk >= s && kk < e) sum = fmaf(to_f32(v), to_f32(x[c[j]]), sum);
    }
  } else {
#pragma unroll
    for (int j = 0; j < kLowpChunk; ++j) {
      const int64_t kk = k + j;
      if (kk >= s && kk < e) sum = fmaf(to_f32(val[kk]), to_f32(x[col[kk]]), sum);
    }
  }
  return sum;
}

template <typename TY>
__device__ __forceinline__ void store_y(TY* y, float alpha, float sum, float beta) {
  const float r = beta == 0.f ? alpha * sum : fmaf(alpha, sum, beta * to_f32(*y));
  *y = from_f32<TY>(r);
}

template <typename TA, typename TY, typename OffT, int G, bool VL>
__global__ void __launch_bounds__(kThreads) spmv_lowp_kernel(const LowpArgs<TA, TY, OffT> a) {
  const int b = blockIdx.x;
  if (b < a.cta_short) {
    constexpr int NG = kThreads / G;
    const int lane = threadIdx.x & (G - 1);
    const int64_t i = (int64_t)b * NG + threadIdx.x / G;
    const int32_t row = i < a.n_short ? (a.rows_short ? a.rows_short[i] : (int32_t)i) : -1;
    float sum = 0.f;
    if (row >= 0) {
      const int64_t s = (int64_t)a.rp[row], e = (int64_t)a.rp[row + 1];
      for (int64_t k = (s & ~(int64_t)(kLowpChunk - 1)) + lane * kLowpChunk; k < e; k += G * kLowpChunk)
        sum += chunk_dot<TA, VL>(a.val, a.col, a.x, k, s, e, a.nnz);
    }
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0 && row >= 0) store_y(a.y + row, a.alpha, sum, a.beta);
  } else if (b < a.cta_short + a.cta_medium) {
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t)(b - a.cta_short) * (kThreads / 32) + (threadIdx.x >> 5);
    if (i >= a.n_medium) return;  // whole warp leaves together
    const int32_t row = a.rows_medium[i];
    const int64_t s = (int64_t)a.rp[row], e = (int64_t)a.rp[row + 1];
    float sum = 0.f;
    for (int64_t k = (s & ~(int64_t)(kLowpChunk - 1)) + lane * kLowpChunk; k < e; k += 32 * kLowpChunk)
      sum += chunk_dot<TA, VL>(a.val, a.col, a.x, k, s, e, a.nnz);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) store_y(a.y + row, a.alpha, sum, a.beta);
  } else {
    __shared__ float s_part[kThreads / 32];
    const int64_t i = (int64_t)(b - a.cta_short - a.cta_medium);
    const int32_t row = a.rows_long[i];
    const int64_t s = (int64_t)a.rp[row], e = (int64_t)a.rp[row + 1];
    float sum = 0.f;
    for (int64_t k = (s & ~(int64_t)(kLowpChunk - 1)) + threadIdx.x * kLowpChunk; k < e; k += kThreads * kLowpChunk)
      sum += chunk_dot<TA, VL>(a.val, a.col, a.x, k, s, e, a.nnz);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
#pragma unroll
      for (int w = 0; w < kThreads / 32; ++w) tot += s_part[w];
      store_y(a.y + row, a.alpha, tot, a.beta);
    }
  }
}

template <typename TA, typename TY, typename OffT, bool VL>
alphasparseStatus_t launch(alphasparseHandle_t h, const Plan* p, LowpArgs<TA, TY, OffT> a) {
  // the plan's lane-group width was chosen for four entries per lane and step; here a lane takes eight
  int g = p->group_lanes / 2;
  if (g < 2) g = 2;
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
    case 2: spmv_lowp_kernel<TA, TY, OffT, 2, VL><<<grid, block, 0, h->stream>>>(a); break;
    case 4: spmv_lowp_kernel<TA, TY, OffT, 4, VL><<<grid, block, 0, h->stream>>>(a); break;
    case 8: spmv_lowp_kernel<TA, TY, OffT, 8, VL><<<grid, block, 0, h->stream>>>(a); break;
    default: spmv_lowp_kernel<TA, TY, OffT, 16, VL><<<grid, block, 0, h->stream>>>(a); break;
  }
  impl(h)->launches++;
  return status_of(cudaGetLastError());
}

template <typename TA, typename TY, typename OffT>
alphasparseStatus_t run_t(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const Plan* p, const void* x,
                          void* y, float alpha, float beta) {
  LowpArgs<TA, TY, OffT> a;
  a.rp = reinterpret_cast<const OffT*>(A->row_offsets);
  a.col = A->const_col_data;
  a.val = reinterpret_cast<const TA*>(A->const_val_data);
  a.x = reinterpret_cast<const TA*>(x);
  a.y = reinterpret_cast<TY*>(y);
  a.alpha = alpha;
  a.beta = beta;
  a.rows_short = p->identity_short ? nullptr : p->bin_rows;
  a.rows_medium = p->identity_short ? nullptr : p->bin_rows + p->n_short;
  a.rows_long = p->identity_short ? nullptr : p->bin_rows + p->n_short + p->n_medium;
  a.n_short = p->n_short;
  a.n_medium = p->n_medium;
  a.n_long = p->n_long;
  a.nnz = p->nnz;
  a.cta_short = a.cta_medium = 0;
  const bool vl = ((reinterpret_cast<uintptr_t>(a.val) | reinterpret_cast<uintptr_t>(a.col)) & 15) == 0;
  return vl ? launch<TA, TY, OffT, true>(h, p, a) : launch<TA, TY, OffT, false>(h, p, a);
}

}  // namespace

bool spmv_lowp_types(alphasparseDataType a, alphasparseDataType x, alphasparseDataType y,
                     alphasparseDataType compute) {
  if (compute != ALPHA_R_32F || x != a) return false;
  return (a == ALPHA_R_16F && y == ALPHA_R_32F) || (a == ALPHA_R_16BF && y == ALPHA_R_16BF);
}

alphasparseStatus_t spmv_lowp_run(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const Plan* p,
                                  const void* x, void* y, float alpha, float beta) {
  if (p->rows == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  const bool o64 = A->row_type == ALPHA_SPARSE_INDEXTYPE_I64;
  if (A->data_type == ALPHA_R_16F)
    return o64 ? run_t<__half, float, int64_t>(h, A, p, x, y, alpha, beta)
               : run_t<__half, float, int32_t>(h, A, p, x, y, alpha, beta);
  return o64 ? run_t<__nv_bfloat16, __nv_bfloat16, int64_t>(h, A, p, x, y, alpha, beta)
             : run_t<__nv_bfloat16, __nv_bfloat16, int32_t>(h, A, p, x, y, alpha, beta);
}

}  // namespace asp
