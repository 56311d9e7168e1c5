// CSR SpMV  y = alpha*A*x + beta*y  for sm_100a: the row-length-binned kernel and the
// merge-path kernel, the dispatcher and the buffer-size query.
//
// Replaces, for CSR with opA = N, the reference's dispatcher
// cuda/kernel/level2/alphasparse_spmv.cu:21-421 and its kernel headers
// alphasparse_spmv_csr_{scalar,vector,adaptive2,line_enhance,flat,merge_ginkgo,
// row_partition_ginkgo}.h.  Differences that matter to a caller:
//   - every launch goes to handle->stream (several reference variants use the default
//     stream or call cudaDeviceSynchronize, e.g. alphasparse_spmv_csr_merge_ginkgo.h:206,219
//     and alphasparse_spmv_csr_row_partition_ginkgo.h:411,482);
//   - partitioning is read from the analysed plan instead of being recomputed per call;
//   - no atomics on y: a row is summed by one lane group, warp or CTA, and the merge-path
//     kernel passes partial sums of rows that straddle CTAs through a carry array that a
//     second small kernel adds in tile order, so results are reproducible run to run.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <climits>
#include <cstring>
#include <mutex>
#include <type_traits>

#include "asp_internal.h"

namespace asp {
namespace {

template <typename T> struct VecTraits;
template <> struct VecTraits<float> {
  static constexpr int N = 4;
  using V = float4;
  using I = int4;
};
template <> struct VecTraits<double> {
  static constexpr int N = 2;
  using V = double2;
  using I = int2;
};

template <typename OffT>
using idx_t = typename std::conditional<std::is_same<OffT, int32_t>::value, uint32_t, int64_t>::type;

// One 16-byte load of values and the matching column indices at entry k (k a multiple of
// N), streamed past L1 and marked evict-first in L2 so that A does not displace x.  The last
// partial chunk of the arrays, or arrays that are not 16-byte aligned (VL = false), are read
// element by element.
template <typename T, bool VL, typename IdxT>
__device__ __forceinline__ void load_chunk(const T* __restrict__ val, const int* __restrict__ col,
                                           IdxT k, IdxT nnz, T (&v)[VecTraits<T>::N],
                                           int (&c)[VecTraits<T>::N]) {
  constexpr int N = VecTraits<T>::N;
  if (VL && k + N <= nnz) {
    typename VecTraits<T>::V vv = __ldcs(reinterpret_cast<const typename VecTraits<T>::V*>(val + k));
    typename VecTraits<T>::I cc = __ldcs(reinterpret_cast<const typename VecTraits<T>::I*>(col + k));
    if constexpr (N == 4) {
      v[0] = vv.x; v[1] = vv.y; v[2] = vv.z; v[3] = vv.w;
      c[0] = cc.x; c[1] = cc.y; c[2] = cc.z; c[3] = cc.w;
    } else {
      v[0] = vv.x; v[1] = vv.y;
      c[0] = cc.x; c[1] = cc.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < N; ++j) {
      const bool in = k + j < nnz;
      v[j] = in ? __ldcs(val + k + j) : T(0);
      c[j] = in ? __ldcs(col + k + j) : 0;
    }
  }
}

template <typename T>
__device__ __forceinline__ T finish(T alpha, T sum, T beta, const T* y) {
  return beta == T(0) ? alpha * sum : fma(alpha, sum, beta * (*y));
}

// ------------------------------------------------------------------------------------------
// Row-length-binned kernel.  One launch; CTA index ranges select the class:
//   [0, cta_short)                     short rows : G lanes per row, kShortUnroll rows in flight
//   [cta_short, cta_short+cta_medium)  medium rows: one warp per row
//   the rest                           long rows  : one CTA per row
// Every lane reads 16-byte chunks that start at a multiple of N entries (the row start is
// rounded down and the leading entries masked), so the loads of neighbouring lanes and of
// neighbouring rows coalesce into full lines.
// ------------------------------------------------------------------------------------------
template <typename T, typename OffT>
struct BinnedArgs {
  const OffT* rp;
  const int* col;
  const T* val;
  const T* x;
  T* y;
  T alpha, beta;
  const int32_t* rows_short;   // nullptr: row i of the class is row i of the matrix
  const int32_t* rows_medium;
  const int32_t* rows_long;
  int64_t n_short, n_medium, n_long, nnz;
  int cta_short, cta_medium;
};

template <typename T, typename OffT, int G, bool VL, int U>
__global__ void __launch_bounds__(kThreads) spmv_binned_kernel(const BinnedArgs<T, OffT> a) {
  constexpr int N = VecTraits<T>::N;
  using IdxT = idx_t<OffT>;
  const IdxT nnz = (IdxT)a.nnz;
  const int b = blockIdx.x;
  if (b < a.cta_short) {
    constexpr int NG = kThreads / G;
    const int lane = threadIdx.x & (G - 1);
    const int grp = threadIdx.x / G;
    const int64_t base = (int64_t)b * (NG * U);
    int32_t row[U];
    IdxT s[U], e[U], k[U];
    T sum[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = base + u * NG + grp;
      row[u] = i < a.n_short ? (a.rows_short ? a.rows_short[i] : (int32_t)i) : -1;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      s[u] = row[u] >= 0 ? (IdxT)a.rp[row[u]] : 0;
      e[u] = row[u] >= 0 ? (IdxT)a.rp[row[u] + 1] : 0;
      k[u] = (s[u] & ~(IdxT)(N - 1)) + (IdxT)(lane * N);
      sum[u] = T(0);
    }
    bool more = true;
    while (more) {
      more = false;
      T v[U][N];
      int c[U][N];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (k[u] < e[u]) load_chunk<T, VL, IdxT>(a.val, a.col, k[u], nnz, v[u], c[u]);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (k[u] < e[u]) {
#pragma unroll
          for (int j = 0; j < N; ++j) {
            const IdxT kk = k[u] + j;
            if (kk >= s[u] && kk < e[u]) sum[u] = fma(v[u][j], __ldg(a.x + c[u][j]), sum[u]);
          }
          k[u] += (IdxT)(G * N);
          more |= k[u] < e[u];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
#pragma unroll
      for (int o = G / 2; o > 0; o >>= 1) sum[u] += __shfl_xor_sync(0xffffffffu, sum[u], o);
      if (lane == 0 && row[u] >= 0) a.y[row[u]] = finish(a.alpha, sum[u], a.beta, a.y + row[u]);
    }
  } else if (b < a.cta_short + a.cta_medium) {
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t)(b - a.cta_short) * (kThreads / 32) + (threadIdx.x >> 5);
    if (i >= a.n_medium) return;  // whole warp leaves together
    const int32_t row = a.rows_medium[i];
    const IdxT s = (IdxT)a.rp[row], e = (IdxT)a.rp[row + 1];
    T sum = T(0);
    for (IdxT k = (s & ~(IdxT)(N - 1)) + (IdxT)(lane * N); k < e; k += 32 * N) {
      T v[N];
      int c[N];
      load_chunk<T, VL, IdxT>(a.val, a.col, k, nnz, v, c);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const IdxT kk = k + j;
        if (kk >= s && kk < e) sum = fma(v[j], __ldg(a.x + c[j]), sum);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) a.y[row] = finish(a.alpha, sum, a.beta, a.y + row);
  } else {
    __shared__ T s_part[kThreads / 32];
    const int64_t i = (int64_t)(b - a.cta_short - a.cta_medium);
    const int32_t row = a.rows_long[i];
    const IdxT s = (IdxT)a.rp[row], e = (IdxT)a.rp[row + 1];
    T sum = T(0);
    for (IdxT k = (s & ~(IdxT)(N - 1)) + (IdxT)(threadIdx.x * N); k < e; k += kThreads * N) {
      T v[N];
      int c[N];
      load_chunk<T, VL, IdxT>(a.val, a.col, k, nnz, v, c);
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const IdxT kk = k + j;
        if (kk >= s && kk < e) sum = fma(v[j], __ldg(a.x + c[j]), sum);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
      T tot = T(0);
#pragma unroll
      for (int w = 0; w < kThreads / 32; ++w) tot += s_part[w];
      a.y[row] = finish(a.alpha, tot, a.beta, a.y + row);
    }
  }
}

// ------------------------------------------------------------------------------------------
// Merge-path kernel (Merrill & Garland's decomposition; the reference's version is
// alphasparse_spmv_csr_merge_ginkgo.h:36-131).  CTA t owns items [t*kMergeItems, ...) of the
// merge of the row-end offsets with the entry indices; its start coordinate comes from the
// plan.  The CTA
//   (1) streams its entries with coalesced 16-byte loads, multiplies by the gathered x and
//       parks the products in shared memory (index skewed by one slot per 32 so that rows of
//       any stride read without bank conflicts);
//   (2) reduces rows.  If every row segment in the tile is short (<= kMergeShortSeg entries)
//       thread i sums segment i straight from shared memory and writes y[row_s+i] coalesced.
//       Otherwise every thread walks kMergeIpt items of the merge list serially and a
//       block-wide segmented scan hands partial sums of rows that span threads forward.
//   (3) the sum of the row still open at the tile's end goes to carry[t]; the fix-up kernel
//       adds carries to their rows in tile order.
// ------------------------------------------------------------------------------------------
constexpr int kMergeShortSeg = 64;
#ifndef ASP_TILE_MIN_CTAS
#define ASP_TILE_MIN_CTAS 6
#endif
constexpr int kTileMinCtas = ASP_TILE_MIN_CTAS;
#ifndef ASP_TILE_MIN_CTAS_LOWP
#define ASP_TILE_MIN_CTAS_LOWP 8   // 16-bit values: a tile is 12 KB, more tiles in flight per SM
#endif
#ifndef ASP_TILE_SHORT_SEG
#define ASP_TILE_SHORT_SEG 32
#endif
#ifndef ASP_MERGE_MIN_CTAS
#define ASP_MERGE_MIN_CTAS 6
#endif
constexpr int kMergeMinCtas = ASP_MERGE_MIN_CTAS;
#ifndef ASP_MERGE_THREADS
#define ASP_MERGE_THREADS 256
#endif
constexpr int kMergeThreads = ASP_MERGE_THREADS;
__device__ __forceinline__ int skew(int i) { return i + (i >> 5); }

template <typename T, typename OffT, bool VL>
__global__ void __launch_bounds__(kMergeThreads, kMergeMinCtas)
spmv_merge_kernel(const OffT* __restrict__ rp, const int* __restrict__ col,
                  const T* __restrict__ val, const T* __restrict__ x, T* __restrict__ y, T alpha,
                  T beta, int64_t rows, int64_t nnz64, const int32_t* __restrict__ tile_row,
                  T* __restrict__ carry) {
  constexpr int N = VecTraits<T>::N;
  constexpr int IPT = kMergeItems / kMergeThreads;
  constexpr int ITEMS = kMergeItems;
  constexpr int CH = ITEMS / (N * kMergeThreads) + 1;
  __shared__ T s_prod[ITEMS + ITEMS / 32 + 1];
  __shared__ int s_rowend[ITEMS + 1];
  __shared__ T s_wval[kMergeThreads / 32];
  __shared__ int s_wflag[kMergeThreads / 32];

  const int tid = threadIdx.x;
  const int64_t t = blockIdx.x;
  const int row_s = tile_row[t], row_e = tile_row[t + 1];
  const int64_t diag_s = t * (int64_t)ITEMS;
  int64_t diag_e = diag_s + ITEMS;
  if (diag_e > rows + nnz64) diag_e = rows + nnz64;
  const int64_t nz_s = diag_s - row_s, nz_e = diag_e - row_e;
  const int tile_rows = row_e - row_s;
  const int tile_nnz = (int)(nz_e - nz_s);

  // The row end this thread will publish, requested before the entry loads so that both
  // round trips to HBM overlap.
  OffT my_end = 0;
  if (tid < tile_rows) my_end = rp[row_s + tid + 1];

  // (1) products.  All indices below are 32-bit offsets from the tile's aligned first entry.
  {
    const int64_t a0 = nz_s & ~(int64_t)(N - 1);
    const T* __restrict__ tval = val + a0;
    const int* __restrict__ tcol = col + a0;
    const int lo = (int)(nz_s - a0);                 // first entry of the tile
    const int hi = lo + tile_nnz;                    // one past its last entry
    const int64_t rem = nnz64 - a0;                  // entries left in the arrays
    const int lim = rem > (int64_t)(ITEMS + 2 * N) ? ITEMS + 2 * N : (int)rem;
    T v[CH][N];
    int c[CH][N];
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int k = (i * kMergeThreads + tid) * N;
      if (k < hi) load_chunk<T, VL, int>(tval, tcol, k, lim, v[i], c[i]);
    }
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int k = (i * kMergeThreads + tid) * N;
      if (k < hi) {
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const int kk = k + j;
          if (kk >= lo && kk < hi) s_prod[skew(kk - lo)] = v[i][j] * __ldg(x + c[i][j]);
        }
      }
    }
  }
  // Row ends relative to the tile's first entry.  Rows row_s .. row_e-1 end inside the tile.
  if (tid < tile_rows) s_rowend[tid] = (int)((int64_t)my_end - nz_s);
  for (int i = tid + kMergeThreads; i < tile_rows; i += kMergeThreads)
    s_rowend[i] = (int)((int64_t)rp[row_s + i + 1] - nz_s);
  if (tid == 0) s_rowend[tile_rows] = INT_MAX;  // the row still open at the tile's end never "ends" here
  __syncthreads();
  bool long_seg = false;
  for (int i = tid; i <= tile_rows; i += kMergeThreads) {
    const int b = i == 0 ? 0 : s_rowend[i - 1];
    const int e = i < tile_rows ? s_rowend[i] : tile_nnz;
    long_seg |= (e - b) > kMergeShortSeg;
  }
  const int any_long = __syncthreads_or(long_seg ? 1 : 0);

  if (!any_long) {
    // (2a) one thread per row segment
    for (int i = tid; i <= tile_rows; i += kMergeThreads) {
      const int b = i == 0 ? 0 : s_rowend[i - 1];
      const int e = i < tile_rows ? s_rowend[i] : tile_nnz;
      T sum = T(0);
      for (int k = b; k < e; ++k) sum += s_prod[skew(k)];
      if (i < tile_rows) y[row_s + i] = finish(alpha, sum, beta, y + row_s + i);
      else carry[t] = sum;
    }
    return;
  }

  // (2b) per-thread walk
  const int tile_items = tile_rows + tile_nnz;
  int d = tid * IPT;
  if (d > tile_items) d = tile_items;
  int d_end = d + IPT;
  if (d_end > tile_items) d_end = tile_items;
  int lo = d > tile_nnz ? d - tile_nnz : 0;
  int hi = d < tile_rows ? d : tile_rows;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (s_rowend[mid] <= d - mid - 1) lo = mid + 1;
    else hi = mid;
  }
  int i = lo, j = d - lo;
  T running = T(0), first_val = T(0);
  int first_row = -1;
#pragma unroll
  for (int it = 0; it < IPT; ++it) {
    if (d + it < d_end) {
      if (j < s_rowend[i]) {
        running += s_prod[skew(j)];
        ++j;
      } else {
        if (first_row < 0) {
          first_row = i;
          first_val = running;
        } else {
          y[row_s + i] = finish(alpha, running, beta, y + row_s + i);
        }
        running = T(0);
        ++i;
      }
    }
  }

  // segmented scan of the carry-outs: a thread that finished a row starts a new segment
  const int lane = tid & 31, warp = tid >> 5;
  int flag = first_row >= 0 ? 1 : 0;
  T sv = running;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const T pv = __shfl_up_sync(0xffffffffu, sv, o);
    const int pf = __shfl_up_sync(0xffffffffu, flag, o);
    if (lane >= o) {
      if (!flag) sv += pv;
      flag |= pf;
    }
  }
  if (lane == 31) {
    s_wval[warp] = sv;
    s_wflag[warp] = flag;
  }
  T ev = __shfl_up_sync(0xffffffffu, sv, 1);
  int ef = __shfl_up_sync(0xffffffffu, flag, 1);
  if (lane == 0) {
    ev = T(0);
    ef = 0;
  }
  __syncthreads();
  T pv = T(0);  // sum flowing in from the warps before this one
  for (int w = 0; w < warp; ++w) pv = s_wflag[w] ? s_wval[w] : pv + s_wval[w];
  const T carry_in = ef ? ev : pv + ev;
  if (first_row >= 0) {
    const int r = row_s + first_row;
    y[r] = finish(alpha, carry_in + first_val, beta, y + r);
  }
  if (tid == kMergeThreads - 1) carry[t] = flag ? sv : pv + sv;
}

// ------------------------------------------------------------------------------------------
// TMA-staged merge-path kernel (the default for 16-byte aligned arrays).  Same tiles and the
// same carry protocol as spmv_merge_kernel, different data path:
//   (1) one elected thread asks the copy engine for the tile's value and column slices
//       (two 1-D bulk copies, cp.async.bulk, completion counted on an mbarrier); no register
//       or load/store-unit work is spent on streaming A.  Bulk copies need 16-byte aligned
//       source, destination and size, so a slice is widened to multiples of four entries,
//       clipped to the last full group of four of the array, and the elected thread fetches
//       the at most three entries beyond that with plain loads.
//   (2) while the copies fly, thread i reads the offsets of row segment i straight from
//       global memory (coalesced).
//   (3a) if every segment of the tile is short, thread i walks segment i: column and value
//       from shared memory, x gathered from global memory - for banded matrices the 32 lanes
//       of a warp then read 32 neighbouring x entries - and the sum stays in a register.
//       No product array, no second pass.
//   (3b) otherwise products are formed in place, entry-parallel, and the serial walk with the
//       block-wide segmented scan of spmv_merge_kernel takes over.
// The wait on the mbarrier is bounded; on expiry the CTA raises *err and leaves.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// The same copy with an L2 evict-first policy: A is read once, so its lines should be the first to
// leave L2 and x, which is gathered over and over, should stay.
// One lane of the converged warp, chosen by elect.sync: the compiler then knows that a single
// thread runs the guarded code (the bulk copies take their operands from uniform registers).
__device__ __forceinline__ bool elect_one_lane() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void bulk_g2s_stream(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
      : "memory");
}

constexpr int kTileSlot = kMergeItems + 16;    // entries per staged array (widening adds < 16)
constexpr int kTileShortSeg = ASP_TILE_SHORT_SEG;

// Storage <-> arithmetic conversions of the mixed-precision instances (TA = __half or __nv_bfloat16
// for A and x, arithmetic in T = float); identity for the fp32 / fp64 instances.
template <typename T> __device__ __forceinline__ T widen(T v) { return v; }
__device__ __forceinline__ float widen(__half v) { return __half2float(v); }
__device__ __forceinline__ float widen(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename TY, typename T> __device__ __forceinline__ TY narrow(T v) { return (TY)v; }
template <> __device__ __forceinline__ __half narrow<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16, float>(float v) { return __float2bfloat16_rn(v); }
template <typename T, typename TY>
__device__ __forceinline__ TY finish_as(T alpha, T sum, T beta, const TY* y) {
  return narrow<TY, T>(beta == T(0) ? alpha * sum : fma(alpha, sum, beta * widen(*y)));
}

// T: arithmetic type (and the carries'), TA: type of A's values and of x, TY: type of y.
template <typename T, typename OffT, typename TA = T, typename TY = T>
__global__ void __launch_bounds__(kThreads, (sizeof(TA) < 4 ? ASP_TILE_MIN_CTAS_LOWP : kTileMinCtas))
spmv_tile_kernel(const OffT* __restrict__ rp, const int* __restrict__ col, const TA* __restrict__ val,
                 const TA* __restrict__ x, TY* __restrict__ y, T alpha, T beta, int64_t rows,
                 int64_t nnz, const int32_t* __restrict__ tile_row, T* __restrict__ carry,
                 int* __restrict__ err, uint32_t wait_cfg) {
  constexpr int ITEMS = kMergeItems;
  constexpr int IPT = kMergeIpt;
  constexpr bool kSame = std::is_same<TA, T>::value;
  // a bulk copy moves whole 16-byte units of both arrays: groups of GA entries
  constexpr int GA = sizeof(TA) >= 4 ? 4 : 16 / (int)sizeof(TA);
  static_assert(kSame || sizeof(T) == sizeof(int), "mixed precision parks fp32 products in the column slots");
  __shared__ __align__(128) TA s_val[kTileSlot];
  __shared__ __align__(128) int s_col[kTileSlot];
  __shared__ __align__(8) unsigned char s_flags[ITEMS];  // 1 where an item of the merge list is a row end
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ T s_wval[kThreads / 32];
  __shared__ int s_wflag[kThreads / 32];
  __shared__ int s_wcnt[kThreads / 32];
  static_assert(IPT == 8, "a thread's row-end bytes are read as one 8-byte word");

  const int tid = threadIdx.x;
  const int64_t t = blockIdx.x;
  const int row_s = tile_row[t], row_e = tile_row[t + 1];
  const int64_t total = rows + nnz;
  const int64_t diag_s = t * (int64_t)ITEMS;
  const int64_t diag_e = diag_s + ITEMS < total ? diag_s + ITEMS : total;
  const int64_t nz_s = diag_s - row_s, nz_e = diag_e - row_e;
  const int tile_rows = row_e - row_s;
  const int tile_nnz = (int)(nz_e - nz_s);
  const int64_t a0 = nz_s & ~(int64_t)(GA - 1);
  const int lo = (int)(nz_s - a0);

  if (tid < 32 && elect_one_lane()) {
    mbar_init(&s_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const int64_t nnz4 = nnz & ~(int64_t)(GA - 1);
    int64_t a1 = (nz_e + (GA - 1)) & ~(int64_t)(GA - 1);
    if (a1 > nnz4) a1 = nnz4;
    if (a1 < a0) a1 = a0;
    const uint32_t cnt = (uint32_t)(a1 - a0);
    mbar_expect_tx(&s_bar, cnt * (uint32_t)(sizeof(TA) + sizeof(int)));
    if (cnt && !(wait_cfg & kWaitDropCopy)) {
      if (wait_cfg & kWaitNoL2Hint) {
        bulk_g2s(s_val, val + a0, cnt * (uint32_t)sizeof(TA), &s_bar);
        bulk_g2s(s_col, col + a0, cnt * (uint32_t)sizeof(int), &s_bar);
      } else {
        bulk_g2s_stream(s_val, val + a0, cnt * (uint32_t)sizeof(TA), &s_bar);
        bulk_g2s_stream(s_col, col + a0, cnt * (uint32_t)sizeof(int), &s_bar);
      }
    }
    for (int64_t e = a1 > nz_s ? a1 : nz_s; e < nz_e; ++e) {  // past the last full group of entries
      s_val[e - a0] = val[e];
      s_col[e - a0] = col[e];
    }
  }
  // (2) this thread's first row segment, from global memory while the copies are in flight
  int seg_b = 0, seg_e = 0;
  bool long_seg = false;
  if (tid <= tile_rows) {
    seg_b = tid == 0 ? 0 : (int)((int64_t)rp[row_s + tid] - nz_s);
    seg_e = tid < tile_rows ? (int)((int64_t)rp[row_s + tid + 1] - nz_s) : tile_nnz;
    long_seg = (seg_e - seg_b) > kTileShortSeg;
  }
  for (int i = tid + kThreads; i <= tile_rows; i += kThreads) {
    const int b = (int)((int64_t)rp[row_s + i] - nz_s);
    const int e = i < tile_rows ? (int)((int64_t)rp[row_s + i + 1] - nz_s) : tile_nnz;
    long_seg |= (e - b) > kTileShortSeg;
  }
  __syncthreads();  // the barrier is initialised (and thread 0's plain stores are visible)
  bool failed = false;
  {
    uint32_t tries = 0;
    while (!mbar_try_wait(&s_bar, 0)) {
      if (++tries > (wait_cfg & kWaitPollMask)) {
        failed = true;
        break;
      }
    }
  }
  // Two CTA-wide votes.  __syncthreads_or tells whether any thread's value was non-zero (not the values'
  // bitwise OR), so the common case - no long segment, no wait that ran out - takes one barrier, and only
  // a tile that has either takes a second one to tell them apart.
  const int any_long_or_failed = __syncthreads_or((long_seg || failed) ? 1 : 0);
  if (any_long_or_failed && __syncthreads_or(failed ? 1 : 0)) {
    if (tid == 0) atomicExch(err, 1);
    __nanosleep(1000000);  // let a copy still in flight land before the CTA's memory is released
    return;
  }
  const TA* sv = s_val + lo;
  const int* sc = s_col + lo;

  if (!any_long_or_failed) {
    // (3a) one thread per row segment, four entries in flight at a time
    for (int i = tid; i <= tile_rows; i += kThreads) {
      int b, e;
      if (i == tid) {
        b = seg_b;
        e = seg_e;
      } else {
        b = (int)((int64_t)rp[row_s + i] - nz_s);
        e = i < tile_rows ? (int)((int64_t)rp[row_s + i + 1] - nz_s) : tile_nnz;
      }
      T sum = T(0);
      int k = b;
      for (; k + 4 <= e; k += 4) {
        const int c0 = sc[k], c1 = sc[k + 1], c2 = sc[k + 2], c3 = sc[k + 3];
        const T x0 = widen(__ldg(x + c0)), x1 = widen(__ldg(x + c1)), x2 = widen(__ldg(x + c2)),
                x3 = widen(__ldg(x + c3));
        sum = fma(widen(sv[k]), x0, sum);
        sum = fma(widen(sv[k + 1]), x1, sum);
        sum = fma(widen(sv[k + 2]), x2, sum);
        sum = fma(widen(sv[k + 3]), x3, sum);
      }
      if (k < e) {
        const int c0 = sc[k];
        const int c1 = k + 1 < e ? sc[k + 1] : c0;
        const int c2 = k + 2 < e ? sc[k + 2] : c0;
        const T x0 = widen(__ldg(x + c0)), x1 = widen(__ldg(x + c1)), x2 = widen(__ldg(x + c2));
        sum = fma(widen(sv[k]), x0, sum);
        if (k + 1 < e) sum = fma(widen(sv[k + 1]), x1, sum);
        if (k + 2 < e) sum = fma(widen(sv[k + 2]), x2, sum);
      }
      if (i < tile_rows) y[row_s + i] = finish_as(alpha, sum, beta, y + row_s + i);
      else carry[t] = sum;
    }
    return;
  }

  // (3b) products in place, then the serial walk.  Row end i is item (row_end_i + i) of the tile's
  // merge list, so the rows mark their end items in a byte map and a thread learns from its eight
  // bytes which of its items are row ends; the number of row ends before its first item (a block
  // scan of the byte counts) is the row it starts in.  No search, no per-item offset reads.
  // (with 16-bit values the fp32 product goes into the entry's column slot, which is dead after the gather)
  T* sp;
  if constexpr (kSame) sp = s_val + lo;
  else sp = reinterpret_cast<T*>(s_col) + lo;
#pragma unroll
  for (int i = 0; i < IPT; ++i) {
    const int e = i * kThreads + tid;
    if (e < tile_nnz) sp[e] = widen(sv[e]) * widen(__ldg(x + sc[e]));
  }
  *reinterpret_cast<uint2*>(s_flags + IPT * tid) = make_uint2(0u, 0u);
  __syncthreads();
  for (int i = tid; i < tile_rows; i += kThreads) {
    const int e = i == tid ? seg_e : (int)((int64_t)rp[row_s + i + 1] - nz_s);
    s_flags[e + i] = 1;
  }
  __syncthreads();
  const int lane = tid & 31, warp = tid >> 5;
  const uint2 fl = *reinterpret_cast<const uint2*>(s_flags + IPT * tid);
  const unsigned long long ends = ((unsigned long long)fl.y << 32) | fl.x;
  const int cnt = __popc(fl.x) + __popc(fl.y);
  int inc = cnt;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += v;
  }
  if (lane == 31) s_wcnt[warp] = inc;
  __syncthreads();
  int i = inc - cnt;  // row ends before this thread's first item: the (tile-relative) row it starts in
  for (int w = 0; w < warp; ++w) i += s_wcnt[w];
  int j = IPT * tid - i;
  const int tile_items = tile_rows + tile_nnz;
  T running = T(0), first_val = T(0);
  int first_row = -1;
#pragma unroll
  for (int it = 0; it < IPT; ++it) {
    if (IPT * tid + it < tile_items) {
      if (!((ends >> (8 * it)) & 1ull)) {
        running += sp[j];
        ++j;
      } else {
        if (first_row < 0) {
          first_row = i;
          first_val = running;
        } else {
          y[row_s + i] = finish_as(alpha, running, beta, y + row_s + i);
        }
        running = T(0);
        ++i;
      }
    }
  }
  int flag = first_row >= 0 ? 1 : 0;
  T acc = running;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const T pv = __shfl_up_sync(0xffffffffu, acc, o);
    const int pf = __shfl_up_sync(0xffffffffu, flag, o);
    if (lane >= o) {
      if (!flag) acc += pv;
      flag |= pf;
    }
  }
  if (lane == 31) {
    s_wval[warp] = acc;
    s_wflag[warp] = flag;
  }
  T ev = __shfl_up_sync(0xffffffffu, acc, 1);
  int ef = __shfl_up_sync(0xffffffffu, flag, 1);
  if (lane == 0) {
    ev = T(0);
    ef = 0;
  }
  __syncthreads();
  T pv = T(0);
  for (int w = 0; w < warp; ++w) pv = s_wflag[w] ? s_wval[w] : pv + s_wval[w];
  const T carry_in = ef ? ev : pv + ev;
  if (first_row >= 0) {
    const int r = row_s + first_row;
    y[r] = finish_as(alpha, carry_in + first_val, beta, y + r);
  }
  if (tid == kThreads - 1) carry[t] = flag ? acc : pv + acc;
}

// Adds the sums that left tiles to the rows they belong to.  Tile t's carry belongs to row
// tile_row[t+1].  The thread of the first tile of a run of tiles that all end inside the same
// row adds the whole run, in tile order.
template <typename T, typename TY = T>
__global__ void __launch_bounds__(256) spmv_merge_fixup_kernel(const int32_t* __restrict__ tile_row,
                                                               const T* __restrict__ carry,
                                                               int64_t tiles, int64_t rows,
                                                               TY* __restrict__ y, T alpha) {
  const int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t >= tiles) return;
  const int32_t r = tile_row[t + 1];
  if (r >= rows) return;
  if (t > 0 && tile_row[t] == r) return;
  T sum = T(0);
  for (int64_t u = t; u < tiles && tile_row[u + 1] == r; ++u) sum += carry[u];
  y[r] = narrow<TY, T>(fma(alpha, sum, widen(y[r])));
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

template <typename T, typename OffT, bool VL, int U>
alphasparseStatus_t launch_binned(alphasparseHandle_t h, const Plan* p, const BinnedArgs<T, OffT>& a0) {
  BinnedArgs<T, OffT> a = a0;
  const int g = p->group_lanes;
  const int rows_per_cta = (kThreads / g) * U;
  const int64_t cs = (p->n_short + rows_per_cta - 1) / rows_per_cta;
  const int64_t cm = (p->n_medium + (kThreads / 32) - 1) / (kThreads / 32);
  const int64_t total = cs + cm + p->n_long;
  if (total > INT_MAX) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (total == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  a.cta_short = (int)cs;
  a.cta_medium = (int)cm;
  const dim3 grid((unsigned)total), block(kThreads);
  switch (g) {
    case 2: spmv_binned_kernel<T, OffT, 2, VL, U><<<grid, block, 0, h->stream>>>(a); break;
    case 4: spmv_binned_kernel<T, OffT, 4, VL, U><<<grid, block, 0, h->stream>>>(a); break;
    case 8: spmv_binned_kernel<T, OffT, 8, VL, U><<<grid, block, 0, h->stream>>>(a); break;
    case 16: spmv_binned_kernel<T, OffT, 16, VL, U><<<grid, block, 0, h->stream>>>(a); break;
    default: spmv_binned_kernel<T, OffT, 32, VL, U><<<grid, block, 0, h->stream>>>(a); break;
  }
  impl(h)->launches++;
  return status_of(cudaGetLastError());
}

template <typename T, typename OffT>
alphasparseStatus_t spmv_t(alphasparseHandle_t h, alphasparseSpMatDescr_t A, Plan* p, const T* x,
                           T* y, T alpha, T beta, int variant, void* ext) {
  const OffT* rp = reinterpret_cast<const OffT*>(A->row_offsets);
  const int* col = A->const_col_data;
  const T* val = reinterpret_cast<const T*>(A->const_val_data);
  const bool vl = aligned(val, 16) && aligned(col, 16);
  if (p->rows == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  if (variant == kVariantBinned) {
    BinnedArgs<T, OffT> a;
    a.rp = rp; a.col = col; a.val = val; a.x = x; a.y = y; a.alpha = alpha; a.beta = beta;
    a.rows_short = p->identity_short ? nullptr : p->bin_rows;
    a.rows_medium = p->identity_short ? nullptr : p->bin_rows + p->n_short;
    a.rows_long = p->identity_short ? nullptr : p->bin_rows + p->n_short + p->n_medium;
    a.n_short = p->n_short; a.n_medium = p->n_medium; a.n_long = p->n_long; a.nnz = p->nnz;
    a.cta_short = a.cta_medium = 0;
    if (!vl) return launch_binned<T, OffT, false, 2>(h, p, a);
    return env_int("ASP_SHORT_UNROLL", kShortUnroll) >= 4 ? launch_binned<T, OffT, true, 4>(h, p, a)
                                                          : launch_binned<T, OffT, true, 2>(h, p, a);
  }
  T* carry = reinterpret_cast<T*>(ext ? ext : p->carry);
  if (p->merge_tiles > INT_MAX) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  const dim3 grid((unsigned)p->merge_tiles), block(kMergeThreads);
  if (vl && env_int("ASP_MERGE_TMA", 1)) {
    spmv_tile_kernel<T, OffT><<<grid, kThreads, 0, h->stream>>>(rp, col, val, x, y, alpha, beta, p->rows, p->nnz,
                                                              p->merge_tile_row, carry, p->dev_err, p->wait_cfg);
    spmv_merge_fixup_kernel<T><<<(unsigned)((p->merge_tiles + 255) / 256), 256, 0, h->stream>>>(
        p->merge_tile_row, carry, p->merge_tiles, p->rows, y, alpha);
    impl(h)->launches += 2;
    return status_of(cudaGetLastError());
  }
  if (vl)
    spmv_merge_kernel<T, OffT, true><<<grid, block, 0, h->stream>>>(
        rp, col, val, x, y, alpha, beta, p->rows, p->nnz, p->merge_tile_row, carry);
  else
    spmv_merge_kernel<T, OffT, false><<<grid, block, 0, h->stream>>>(
        rp, col, val, x, y, alpha, beta, p->rows, p->nnz, p->merge_tile_row, carry);
  spmv_merge_fixup_kernel<T><<<(unsigned)((p->merge_tiles + 255) / 256), 256, 0, h->stream>>>(
      p->merge_tile_row, carry, p->merge_tiles, p->rows, y, alpha);
  impl(h)->launches += 2;
  return status_of(cudaGetLastError());
}

template <typename TA, typename TY, typename OffT>
alphasparseStatus_t spmv_lowp_tile(alphasparseHandle_t h, alphasparseSpMatDescr_t A, Plan* p, const void* x,
                                   void* y, float alpha, float beta, void* ext) {
  float* carry = reinterpret_cast<float*>(ext ? ext : p->carry);
  spmv_tile_kernel<float, OffT, TA, TY><<<(unsigned)p->merge_tiles, kThreads, 0, h->stream>>>(
      reinterpret_cast<const OffT*>(A->row_offsets), A->const_col_data, reinterpret_cast<const TA*>(A->const_val_data),
      reinterpret_cast<const TA*>(x), reinterpret_cast<TY*>(y), alpha, beta, p->rows, p->nnz, p->merge_tile_row,
      carry, p->dev_err, p->wait_cfg);
  spmv_merge_fixup_kernel<float, TY><<<(unsigned)((p->merge_tiles + 255) / 256), 256, 0, h->stream>>>(
      p->merge_tile_row, carry, p->merge_tiles, p->rows, reinterpret_cast<TY*>(y), alpha);
  impl(h)->launches += 2;
  return status_of(cudaGetLastError());
}

int variant_for(const Plan* p, alphasparseSpMVAlg_t alg) {
  const char* f = getenv("ASP_SPMV_VARIANT");
  if (f && !strcmp(f, "binned")) return kVariantBinned;
  if (f && !strcmp(f, "merge")) return kVariantMerge;
  switch (alg) {
    case ALPHA_SPARSE_SPMV_ALG_SCALAR:
    case ALPHA_SPARSE_SPMV_ALG_VECTOR:
    case ALPHA_SPARSE_SPMV_ADAPTIVE:
    case ALPHA_SPARSE_SPMV_ALG_CSR_ADAPTIVE:
    case ALPHA_SPARSE_SPMV_ALG_LINE:
    case ALPHA_SPARSE_SPMV_ALG_LINE_ENHANCE:
    case ALPHA_SPARSE_SPMV_ALG_ACC:
      return kVariantBinned;
    case ALPHA_SPARSE_SPMV_ALG_MERGE:
    case ALPHA_SPARSE_SPMV_ROW_PARTITION:
    case ALPHA_SPARSE_SPMV_ALG_LOAD_BALANCE:
    case ALPHA_SPARSE_SPMV_ALG_CSR_STREAM:
    case ALPHA_SPARSE_SPMV_ALG_FLAT:
    case ALPHA_SPARSE_SPMV_ALG_FLAT1:
    case ALPHA_SPARSE_SPMV_ALG_FLAT4:
    case ALPHA_SPARSE_SPMV_ALG_FLAT8:
    case ALPHA_SPARSE_SPMV_ALG_PFLAT:
      return kVariantMerge;
    default:
      return p->variant_auto;
  }
}

alphasparseStatus_t check_spmv_args(alphasparseHandle_t h, alphasparseOperation_t opA,
                                    const void* alpha, alphasparseSpMatDescr_t A,
                                    alphasparseDnVecDescr_t x, const void* beta,
                                    alphasparseDnVecDescr_t y, alphasparseDataType computeType) {
  if (!h || !h->impl) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!alpha || !beta || !A || !x || !y) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (h->pointer_mode != ALPHA_SPARSE_POINTER_MODE_HOST) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  // a transposed product runs on the transposed matrix the plan keeps; for these real types the
  // conjugate transpose is the transpose
  const bool tr = opA != ALPHA_SPARSE_OPERATION_NON_TRANSPOSE;
  alphasparseStatus_t s = validate_csr(A);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  if (!x->init || !y->init) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
  // complex: the transposed copy holds the values as they are, so the conjugate transpose is not offered
  if (opA == ALPHA_SPARSE_OPERATION_CONJUGATE_TRANSPOSE && (A->data_type == ALPHA_C_32F || A->data_type == ALPHA_C_64F))
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (!spmv_lowp_types(A->data_type, x->data_type, y->data_type, computeType) &&
      !spmv_other_types(A->data_type, x->data_type, y->data_type, computeType)) {
    if (A->data_type != ALPHA_R_32F && A->data_type != ALPHA_R_64F) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    if (x->data_type != A->data_type || y->data_type != A->data_type || computeType != A->data_type)
      return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  }
  if (x->size != (tr ? A->rows : A->cols) || y->size != (tr ? A->cols : A->rows)) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if ((x->size > 0 && !x->values) || (y->size > 0 && !y->values)) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

}  // namespace
}  // namespace asp

using namespace asp;

extern "C" {

alphasparseStatus_t alphasparseSpMV(alphasparseHandle_t h, alphasparseOperation_t opA,
                                    const void* alpha, alphasparseSpMatDescr_t A,
                                    alphasparseDnVecDescr_t x, const void* beta,
                                    alphasparseDnVecDescr_t y, alphasparseDataType computeType,
                                    alphasparseSpMVAlg_t alg, void* externalBuffer) {
  alphasparseStatus_t s = check_spmv_args(h, opA, alpha, A, x, beta, y, computeType);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  if (opA != ALPHA_SPARSE_OPERATION_NON_TRANSPOSE) {
    alphasparseSpMatDescr_t At = nullptr;  // built (allocating, synchronising) at the first transposed call
    s = transposed_of(h, A, &At);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    return alphasparseSpMV(h, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, alpha, At, x, beta, y, computeType, alg,
                           externalBuffer);
  }
  if (!A->info) {
    s = analyse(h, A);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  }
  Plan* p = plan_of(A);
  if (p->rows != A->rows || p->nnz != A->nnz || p->cols != A->cols) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
  if (p->device != h->device) return ALPHA_SPARSE_STATUS_INVALID_VALUE;  // the plan's arrays live on another GPU
  if (A->data_type == ALPHA_C_32F || A->data_type == ALPHA_C_64F || A->data_type == ALPHA_R_8I) {
    p->last_variant = kVariantBinned;  // complex and int8 instances: the row-length-binned kernel of spmv_types.cu
    return spmv_other_run(h, A, p, x->values, y->values, y->data_type, alpha, beta);
  }
  if (A->data_type == ALPHA_R_16F || A->data_type == ALPHA_R_16BF) {
    // 16-bit operands, fp32 arithmetic: the TMA-staged merge-path kernel when the plan chose merge-path
    // and the arrays can be bulk-copied, else the row-length-binned kernel of spmv_lowp.cu
    const float al = *(const float*)alpha, be = *(const float*)beta;
    const int variant = variant_for(p, alg);
    const bool tile_ok = variant == kVariantMerge && aligned(A->const_val_data, 16) && aligned(A->const_col_data, 16) &&
                         p->merge_tiles <= INT_MAX && p->rows > 0;
    p->last_variant = tile_ok ? kVariantMerge : kVariantBinned;
    if (!tile_ok) return spmv_lowp_run(h, A, p, x->values, y->values, al, be);
    const bool o64 = A->row_type == ALPHA_SPARSE_INDEXTYPE_I64;
    if (A->data_type == ALPHA_R_16F)
      return o64 ? spmv_lowp_tile<__half, float, int64_t>(h, A, p, x->values, y->values, al, be, externalBuffer)
                 : spmv_lowp_tile<__half, float, int32_t>(h, A, p, x->values, y->values, al, be, externalBuffer);
    return o64 ? spmv_lowp_tile<__nv_bfloat16, __nv_bfloat16, int64_t>(h, A, p, x->values, y->values, al, be, externalBuffer)
               : spmv_lowp_tile<__nv_bfloat16, __nv_bfloat16, int32_t>(h, A, p, x->values, y->values, al, be, externalBuffer);
  }
  const int variant = variant_for(p, alg);
  p->last_variant = variant;
  const bool o64 = A->row_type == ALPHA_SPARSE_INDEXTYPE_I64;
  if (A->data_type == ALPHA_R_32F) {
    const float al = *(const float*)alpha, be = *(const float*)beta;
    return o64 ? spmv_t<float, int64_t>(h, A, p, (const float*)x->values, (float*)y->values, al, be, variant, externalBuffer)
               : spmv_t<float, int32_t>(h, A, p, (const float*)x->values, (float*)y->values, al, be, variant, externalBuffer);
  }
  const double al = *(const double*)alpha, be = *(const double*)beta;
  return o64 ? spmv_t<double, int64_t>(h, A, p, (const double*)x->values, (double*)y->values, al, be, variant, externalBuffer)
             : spmv_t<double, int32_t>(h, A, p, (const double*)x->values, (double*)y->values, al, be, variant, externalBuffer);
}

alphasparseStatus_t alphasparseSpMV_bufferSize(alphasparseHandle_t h, alphasparseOperation_t opA,
                                               const void* alpha, alphasparseSpMatDescr_t A,
                                               alphasparseDnVecDescr_t x, const void* beta,
                                               alphasparseDnVecDescr_t y,
                                               alphasparseDataType computeType,
                                               alphasparseSpMVAlg_t, size_t* bufferSize) {
  if (!bufferSize) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  alphasparseStatus_t s = check_spmv_args(h, opA, alpha, A, x, beta, y, computeType);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  // One carry slot per merge-path tile, in 64-bit arithmetic (the reference adds rows+nnz in
  // int, cuda/kernel/level2/alphasparse_spmv.cu:357).
  const int64_t tiles = ((A->rows > A->cols ? A->rows : A->cols) + A->nnz + kMergeItems - 1) / kMergeItems;  // either op
  const size_t es_ = elem_size(A->data_type);
  const size_t slot = es_ < 4 ? 4 : (es_ > 8 ? 8 : es_);  // 16-bit matrices carry in fp32; complex / int8 use no carries
  size_t bytes = (size_t)(tiles > 0 ? tiles : 1) * slot;
  *bufferSize = (bytes + 255) & ~(size_t)255;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------
// Allocation-free SpMV entry point.
//
// alphasparseSpMV needs an analysed matrix, and analysis allocates the plan with cudaMalloc.
// Some callers may not allocate device memory at all around the call: an iterative solver
// running on a GPU whose memory a framework's pool has already claimed in full, or a
// latency-critical loop that cannot accept the implicit device synchronisation and the
// late failure mode of cudaMalloc / cudaFree.  For them this entry point runs the merge-path
// kernel on raw CSR arrays and keeps its two scratch arrays - the per-tile merge-path start
// rows and the per-tile carry-outs - in one fixed device array that is part of the library
// image.  Every GPU that loads the library holds these 786,688 bytes until the process exits.
// ------------------------------------------------------------------------------------------
namespace asp {
namespace {

constexpr int64_t kNoAllocMaxTiles = ALPHASPARSE_SPMV_NOALLOC_MAX_ITEMS / kMergeItems;
constexpr size_t kNoAllocTileBytes = (((size_t)(kNoAllocMaxTiles + 1) * sizeof(int32_t)) + 255) & ~(size_t)255;
constexpr size_t kNoAllocBytes = kNoAllocTileBytes + (size_t)kNoAllocMaxTiles * sizeof(double);
static_assert(ALPHASPARSE_SPMV_NOALLOC_MAX_ITEMS % kMergeItems == 0, "limit must be whole tiles");

static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

// In host code g_noalloc_scratch is only a handle for the symbol; the address kernels can use
// comes from cudaGetSymbolAddress, asked once per device with that device current.
constexpr int kNoAllocMaxDevices = 64;
void* g_noalloc_ptr[kNoAllocMaxDevices] = {nullptr};
std::mutex g_noalloc_mu;

template <typename OffT>
__global__ void __launch_bounds__(256) noalloc_tile_search_kernel(const OffT* __restrict__ rp,
                                                                  int64_t rows, int64_t nnz,
                                                                  int64_t tiles,
                                                                  int32_t* __restrict__ tile_row) {
  const int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t > tiles) return;
  const OffT* row_end = rp + 1;
  int64_t diag = t * (int64_t)kMergeItems;
  if (diag > rows + nnz) diag = rows + nnz;
  int64_t lo = diag > nnz ? diag - nnz : 0;
  int64_t hi = diag < rows ? diag : rows;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if ((int64_t)row_end[mid] <= diag - mid - 1) lo = mid + 1;
    else hi = mid;
  }
  tile_row[t] = (int32_t)lo;
}

template <typename T, typename OffT>
alphasparseStatus_t spmv_noalloc_t(cudaStream_t st, int64_t rows, int64_t nnz, const OffT* rp,
                                   const int* col, const T* val, const T* x, T* y, T alpha, T beta,
                                   void* scratch) {
  const int64_t tiles = (rows + nnz + kMergeItems - 1) / kMergeItems;
  int32_t* tile_row = reinterpret_cast<int32_t*>(scratch);
  T* carry = reinterpret_cast<T*>(reinterpret_cast<unsigned char*>(scratch) + kNoAllocTileBytes);
  noalloc_tile_search_kernel<OffT><<<(unsigned)((tiles + 1 + 255) / 256), 256, 0, st>>>(rp, rows, nnz, tiles, tile_row);
  const bool vl = aligned(val, 16) && aligned(col, 16);
  if (vl)
    spmv_merge_kernel<T, OffT, true><<<(unsigned)tiles, kMergeThreads, 0, st>>>(rp, col, val, x, y, alpha, beta, rows, nnz, tile_row, carry);
  else
    spmv_merge_kernel<T, OffT, false><<<(unsigned)tiles, kMergeThreads, 0, st>>>(rp, col, val, x, y, alpha, beta, rows, nnz, tile_row, carry);
  spmv_merge_fixup_kernel<T><<<(unsigned)((tiles + 255) / 256), 256, 0, st>>>(tile_row, carry, tiles, rows, y, alpha);
  return status_of(cudaGetLastError());
}

}  // namespace
}  // namespace asp

extern "C" alphasparseStatus_t alphasparseSpMVCsrNoAlloc(
    cudaStream_t stream, int64_t rows, int64_t cols, int64_t nnz, const void* csrRowOffsets,
    alphasparseIndexType_t csrRowOffsetsType, const int32_t* csrColInd, const void* csrValues,
    alphasparseDataType valueType, const void* alpha, const void* x, const void* beta, void* y) {
  if (rows < 0 || cols < 0 || nnz < 0 || rows >= (int64_t(1) << 31) || cols >= (int64_t(1) << 31))
    return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  // The scratch array is fixed: refuse anything that needs more tiles than it holds.
  if (rows + nnz > (int64_t)ALPHASPARSE_SPMV_NOALLOC_MAX_ITEMS) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (!alpha || !beta || !csrRowOffsets) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if ((nnz > 0 && (!csrColInd || !csrValues || !x)) || (rows > 0 && !y))  // x is read only through entries
    return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  const bool o64 = csrRowOffsetsType == ALPHA_SPARSE_INDEXTYPE_I64;
  if (!o64 && csrRowOffsetsType != ALPHA_SPARSE_INDEXTYPE_I32) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (valueType != ALPHA_R_32F && valueType != ALPHA_R_64F) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (rows == 0) return ALPHA_SPARSE_STATUS_SUCCESS;

  int dev = 0;
  ASP_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kNoAllocMaxDevices) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
      void* p = nullptr;
      ASP_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));  // first call on this device only
      g_noalloc_ptr[dev] = p;
    }
    scratch = g_noalloc_ptr[dev];
  }
  if (valueType == ALPHA_R_32F) {
    const float al = *(const float*)alpha, be = *(const float*)beta;
    return o64 ? spmv_noalloc_t<float, int64_t>(stream, rows, nnz, (const int64_t*)csrRowOffsets, csrColInd, (const float*)csrValues, (const float*)x, (float*)y, al, be, scratch)
               : spmv_noalloc_t<float, int32_t>(stream, rows, nnz, (const int32_t*)csrRowOffsets, csrColInd, (const float*)csrValues, (const float*)x, (float*)y, al, be, scratch);
  }
  const double al = *(const double*)alpha, be = *(const double*)beta;
  return o64 ? spmv_noalloc_t<double, int64_t>(stream, rows, nnz, (const int64_t*)csrRowOffsets, csrColInd, (const double*)csrValues, (const double*)x, (double*)y, al, be, scratch)
             : spmv_noalloc_t<double, int32_t>(stream, rows, nnz, (const int32_t*)csrRowOffsets, csrColInd, (const double*)csrValues, (const double*)x, (double*)y, al, be, scratch);
}
