// CSR SpMM  C = alpha*A*B + beta*C  with row-major B (cols x N) and C (rows x N) for sm_100a:
// the SIMT row-block kernel, the dispatcher and the buffer-size / preprocess queries.
//
// Replaces, for CSR with opA = opB = N and row-major dense operands, the reference's
// cuda/kernel/level3/alphasparse_spmm.cu:19-759 and the five algorithms of
// alphasparse_spmm_csr.h (:109-198 row-balanced, :241-393 element-balanced, :395-533 merge,
// :573-795 adaptive, :818-905 flat).  Differences that matter to a caller:
//   - no atomics and no separate C *= beta pass (the reference's default algorithm scales C
//     in a first kernel, alphasparse_spmm_csr.h:907-914,1067-1071, then accumulates with
//     atomicAdd): a row of C is owned by one lane group, initialised with beta*C and
//     accumulated in entry order with fma(alpha*a, b, c) - the order of the reference's CPU
//     kernel (hygon/kernel/level3/mm/gemm/gemm_csr_row.hpp:33-56), so fp32/fp64 results are
//     reproducible and equal to that kernel's;
//   - indices into B and C are 64-bit (the reference multiplies int32, e.g. :907-914);
//   - column-major B / C run through row-major copies in the caller's buffer; the caller's B and C
//     keep their layout (the reference transposes them in place, alphasparse_spmm.cu:134-162,274-283).
#include <climits>
#include <cstring>
#include <type_traits>

#include "asp_internal.h"

namespace asp {

alphasparseStatus_t spmm_tc_run(alphasparseHandle_t h, alphasparseSpMatDescr_t A,
                                alphasparseDnMatDescr_t B, alphasparseDnMatDescr_t C, float alpha,
                                float beta, bool preprocess_only);
bool spmm_tc_applicable(alphasparseSpMatDescr_t A, alphasparseDnMatDescr_t B,
                        alphasparseDnMatDescr_t C);

namespace {

constexpr int kChunk = 1024;  // entries of A staged in shared memory per round

template <typename T, int VN> struct Pack;
template <> struct Pack<float, 4> { using V = float4; };
template <> struct Pack<double, 2> { using V = double2; };
template <> struct Pack<float, 1> { using V = float; };
template <> struct Pack<double, 1> { using V = double; };

template <typename T, int VN>
__device__ __forceinline__ void load_pack(const T* p, T (&r)[VN]) {
  if constexpr (VN == 1) {
    r[0] = __ldg(p);
  } else {
    const typename Pack<T, VN>::V v = __ldg(reinterpret_cast<const typename Pack<T, VN>::V*>(p));
    if constexpr (VN == 4) { r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w; }
    else { r[0] = v.x; r[1] = v.y; }
  }
}

template <typename T, int VN>
__device__ __forceinline__ void store_pack(T* p, const T (&r)[VN]) {
  if constexpr (VN == 1) {
    *p = r[0];
  } else if constexpr (VN == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(r[0], r[1], r[2], r[3]);
  } else {
    *reinterpret_cast<double2*>(p) = make_double2(r[0], r[1]);
  }
}

// A CTA owns RB consecutive rows and one slab of LN*VN columns of C.  LN lanes share a row,
// each lane keeps VN adjacent columns in registers.  The CTA's entries of A go through
// shared memory kChunk at a time (coalesced loads, alpha folded into the value), and every
// lane group then walks the part of its rows that lies in the chunk, reading (col, alpha*a)
// as a shared-memory broadcast and the matching row segment of B with one vector load.
template <typename T, typename OffT, int LN, int VN>
__global__ void __launch_bounds__(kThreads)
spmm_rowblock_kernel(const OffT* __restrict__ rp, const int* __restrict__ col,
                     const T* __restrict__ val, const T* __restrict__ B, int64_t ldb,
                     T* __restrict__ C, int64_t ldc, T alpha, T beta, int64_t rows, int64_t n) {
  constexpr int NG = kThreads / LN;
  constexpr int RPG = NG >= 32 ? 1 : 32 / NG;
  constexpr int RB = NG * RPG;
  __shared__ int s_col[kChunk];
  __shared__ T s_val[kChunk];

  const int lane = threadIdx.x % LN;
  const int grp = threadIdx.x / LN;
  const int64_t r0 = (int64_t)blockIdx.x * RB;
  const int64_t r1 = r0 + RB < rows ? r0 + RB : rows;
  const int64_t c0 = ((int64_t)blockIdx.y * LN + lane) * VN;
  const bool col_ok = c0 < n;

  int64_t rs[RPG], re[RPG];
  T acc[RPG][VN];
#pragma unroll
  for (int i = 0; i < RPG; ++i) {
    const int64_t r = r0 + (int64_t)grp * RPG + i;
    rs[i] = r < rows ? (int64_t)rp[r] : 0;
    re[i] = r < rows ? (int64_t)rp[r + 1] : 0;
#pragma unroll
    for (int v = 0; v < VN; ++v) acc[i][v] = T(0);
    if (beta != T(0) && r < rows && col_ok) {
      T c[VN];
      load_pack<T, VN>(C + r * ldc + c0, c);
#pragma unroll
      for (int v = 0; v < VN; ++v) acc[i][v] = c[v] * beta;
    }
  }
  const int64_t e0 = (int64_t)rp[r0], e1 = (int64_t)rp[r1];
  for (int64_t base = e0; base < e1; base += kChunk) {
    const int cnt = (int)(e1 - base < kChunk ? e1 - base : kChunk);
    for (int i = threadIdx.x; i < cnt; i += kThreads) {
      s_col[i] = __ldcs(col + base + i);
      s_val[i] = alpha * __ldcs(val + base + i);
    }
    __syncthreads();
    if (col_ok) {
#pragma unroll
      for (int i = 0; i < RPG; ++i) {
        const int lo = (int)((rs[i] > base ? rs[i] : base) - base);
        const int hi = (int)((re[i] < base + cnt ? re[i] : base + cnt) - base);
#pragma unroll 4
        for (int k = lo; k < hi; ++k) {
          const T a = s_val[k];
          T b[VN];
          load_pack<T, VN>(B + (int64_t)s_col[k] * ldb + c0, b);
#pragma unroll
          for (int v = 0; v < VN; ++v) acc[i][v] = fma(a, b[v], acc[i][v]);
        }
      }
    }
    __syncthreads();
  }
  if (col_ok) {
#pragma unroll
    for (int i = 0; i < RPG; ++i) {
      const int64_t r = r0 + (int64_t)grp * RPG + i;
      if (r < rows) store_pack<T, VN>(C + r * ldc + c0, acc[i]);
    }
  }
}

// ------------------------------------------------------------------------------------------
// TMA-staged row-block kernel (default when every 128-row block of A has at most kSpmmStageCap32/64
// entries and the operands are 16-byte aligned).  A CTA owns kSpmmRowBlock consecutive rows and
// one slab of LN*VN columns of C:
//   (1) an elected thread asks the copy engine for the block's value and column slices (two 1-D
//       bulk copies counted on an mbarrier; slices widened to groups of four entries, the few
//       entries past the arrays' last full group fetched with plain loads) while all threads
//       stage the block's row offsets;
//   (2) LN lanes share a row and keep VN adjacent columns of C each.  A group reads four
//       (column, value) pairs from shared memory, issues the four matching row segments of B
//       as 16-byte global loads and then does the sixteen FMAs; the groups of a
//       warp work on neighbouring rows at the same time, so for banded matrices a warp's B loads
//       fall into a few cache lines.
// Arithmetic and order are those of spmm_rowblock_kernel: C row := beta*C row, then
// fma(alpha*a, b, c) entry by entry.  The wait on the mbarrier is bounded.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ bool mbar_try_wait0(uint64_t* bar) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar))
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

#ifndef ASP_SPMM_MIN_CTAS
#define ASP_SPMM_MIN_CTAS 6
#endif
template <typename T, typename OffT, int LN, int VN>
__global__ void __launch_bounds__(kThreads, ASP_SPMM_MIN_CTAS)
spmm_tile_kernel(const OffT* __restrict__ rp, const int* __restrict__ col, const T* __restrict__ val,
                 const T* __restrict__ B, int64_t ldb, T* __restrict__ C, int64_t ldc, T alpha, T beta,
                 int64_t rows, int64_t n, int64_t nnz, int* __restrict__ err, uint32_t wait_cfg) {
  constexpr int NG = kThreads / LN;
  constexpr int RB = kSpmmRowBlock;
  constexpr int RPG = RB >= NG ? RB / NG : 1;  // with one lane per row half the groups of a CTA idle
  constexpr int CAP = sizeof(T) == 4 ? kSpmmStageCap32 : kSpmmStageCap64;
  static_assert(RB % NG == 0 || NG > RB, "row block must be a multiple of the groups per CTA");
  __shared__ __align__(128) T s_val[CAP + 8];
  __shared__ __align__(128) int s_col[CAP + 8];
  __shared__ int s_rp[RB + 1];
  __shared__ __align__(8) uint64_t s_bar;

  const int tid = threadIdx.x;
  const int lane = tid % LN;
  const int grp = tid / LN;
  const int64_t r0 = (int64_t)blockIdx.x * RB;
  const int nr = (int)(r0 + RB < rows ? RB : rows - r0);
  // A lane holds VN columns as PK packs of VP (one 16-byte load each); pack p of the lanes of a row is
  // contiguous in memory: columns slab + p*LN*VP + lane*VP.
  constexpr int VP = (sizeof(T) == 4 && VN == 8) ? 4 : VN;
  constexpr int PK = VN / VP;
  const int64_t c0 = (int64_t)blockIdx.y * LN * VN + (int64_t)lane * VP;
  const bool col_ok = c0 < n;
  const int64_t e0 = (int64_t)rp[r0], e1 = (int64_t)rp[r0 + nr];
  const int64_t a0 = e0 & ~(int64_t)3;
  const int lo = (int)(e0 - a0);

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&s_bar)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const int64_t nnz4 = nnz & ~(int64_t)3;
    int64_t a1 = (e1 + 3) & ~(int64_t)3;
    if (a1 > nnz4) a1 = nnz4;
    if (a1 < a0) a1 = a0;
    const uint32_t cnt = (uint32_t)(a1 - a0);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&s_bar)),
                 "r"(cnt * (uint32_t)(sizeof(T) + sizeof(int)))
                 : "memory");
    if (cnt && !(wait_cfg & kWaitDropCopy)) {
      bulk_g2s(s_val, val + a0, cnt * (uint32_t)sizeof(T), &s_bar);
      bulk_g2s(s_col, col + a0, cnt * (uint32_t)sizeof(int), &s_bar);
    }
    for (int64_t e = a1 > e0 ? a1 : e0; e < e1; ++e) {
      s_val[e - a0] = val[e];
      s_col[e - a0] = col[e];
    }
  }
  for (int i = tid; i <= nr; i += kThreads) s_rp[i] = (int)((int64_t)rp[r0 + i] - a0);  // index into s_val/s_col
  __syncthreads();
  bool failed = false;
  {
    uint32_t tries = 0;
    while (!mbar_try_wait0(&s_bar)) {
      if (++tries > (wait_cfg & kWaitPollMask)) {
        failed = true;
        break;
      }
    }
  }
  if (__syncthreads_or(failed ? 1 : 0)) {
    if (tid == 0) atomicExch(err, 1);
    __nanosleep(1000000);
    return;
  }
  (void)lo;
  if (!col_ok) return;

#pragma unroll 1
  for (int i = 0; i < RPG; ++i) {
    const int lr = grp + i * NG;  // neighbouring groups take neighbouring rows
    if (lr >= nr) break;
    const int64_t r = r0 + lr;
    int k = s_rp[lr];
    const int e = s_rp[lr + 1];
    T acc[VN];
#pragma unroll
    for (int v = 0; v < VN; ++v) acc[v] = T(0);
    if (beta != T(0)) {
      T c[VN];
#pragma unroll
      for (int pk = 0; pk < PK; ++pk) load_pack<T, VP>(C + r * ldc + c0 + pk * LN * VP, *reinterpret_cast<T(*)[VP]>(c + pk * VP));
#pragma unroll
      for (int v = 0; v < VN; ++v) acc[v] = c[v] * beta;
    }
    const T* __restrict__ Bc = B + c0;
    auto load_row = [&](const T* src, T (&dst)[VN]) {
#pragma unroll
      for (int pk = 0; pk < PK; ++pk) load_pack<T, VP>(src + pk * LN * VP, *reinterpret_cast<T(*)[VP]>(dst + pk * VP));
    };
    // Four entries per step, counted from the row's first entry, so that the groups of a warp -
    // which hold neighbouring rows - ask for neighbouring rows of B in the same instruction.
    for (; k + 4 <= e; k += 4) {
      const int q0 = s_col[k], q1 = s_col[k + 1], q2 = s_col[k + 2], q3 = s_col[k + 3];
      T b0[VN], b1[VN], b2[VN], b3[VN];
      load_row(Bc + (int64_t)q0 * ldb, b0);
      load_row(Bc + (int64_t)q1 * ldb, b1);
      load_row(Bc + (int64_t)q2 * ldb, b2);
      load_row(Bc + (int64_t)q3 * ldb, b3);
      const T a0s = alpha * s_val[k], a1s = alpha * s_val[k + 1], a2s = alpha * s_val[k + 2],
              a3s = alpha * s_val[k + 3];
#pragma unroll
      for (int v = 0; v < VN; ++v) acc[v] = fma(a0s, b0[v], acc[v]);
#pragma unroll
      for (int v = 0; v < VN; ++v) acc[v] = fma(a1s, b1[v], acc[v]);
#pragma unroll
      for (int v = 0; v < VN; ++v) acc[v] = fma(a2s, b2[v], acc[v]);
#pragma unroll
      for (int v = 0; v < VN; ++v) acc[v] = fma(a3s, b3[v], acc[v]);
    }
    if (k < e) {  // up to three entries left
      const int q0 = s_col[k];
      const int q1 = k + 1 < e ? s_col[k + 1] : q0;
      const int q2 = k + 2 < e ? s_col[k + 2] : q0;
      T b0[VN], b1[VN], b2[VN];
      load_row(Bc + (int64_t)q0 * ldb, b0);
      load_row(Bc + (int64_t)q1 * ldb, b1);
      load_row(Bc + (int64_t)q2 * ldb, b2);
      const T a0s = alpha * s_val[k];
#pragma unroll
      for (int v = 0; v < VN; ++v) acc[v] = fma(a0s, b0[v], acc[v]);
      if (k + 1 < e) {
        const T a1s = alpha * s_val[k + 1];
#pragma unroll
        for (int v = 0; v < VN; ++v) acc[v] = fma(a1s, b1[v], acc[v]);
      }
      if (k + 2 < e) {
        const T a2s = alpha * s_val[k + 2];
#pragma unroll
        for (int v = 0; v < VN; ++v) acc[v] = fma(a2s, b2[v], acc[v]);
      }
    }
#pragma unroll
    for (int pk = 0; pk < PK; ++pk)
      store_pack<T, VP>(C + r * ldc + c0 + pk * LN * VP, *reinterpret_cast<const T(*)[VP]>(acc + pk * VP));
  }
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }
inline size_t round256(size_t b) { return (b + 255) & ~(size_t)255; }

template <typename T, typename OffT, int LN, int VN>
alphasparseStatus_t launch_rb(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const T* B,
                              int64_t ldb, T* C, int64_t ldc, T alpha, T beta, int64_t n) {
  constexpr int NG = kThreads / LN;
  constexpr int RB = NG * (NG >= 32 ? 1 : 32 / NG);
  const int64_t gx = (A->rows + RB - 1) / RB;
  const int64_t gy = (n + (int64_t)LN * VN - 1) / ((int64_t)LN * VN);
  if (gx > INT_MAX || gy > 65535) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  spmm_rowblock_kernel<T, OffT, LN, VN><<<dim3((unsigned)gx, (unsigned)gy), kThreads, 0, h->stream>>>(
      reinterpret_cast<const OffT*>(A->row_offsets), A->const_col_data,
      reinterpret_cast<const T*>(A->const_val_data), B, ldb, C, ldc, alpha, beta, A->rows, n);
  impl(h)->launches++;
  return status_of(cudaGetLastError());
}

template <typename T, typename OffT, int LN, int VN>
alphasparseStatus_t launch_tile(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const T* B,
                                int64_t ldb, T* C, int64_t ldc, T alpha, T beta, int64_t n) {
  const int64_t gx = (A->rows + kSpmmRowBlock - 1) / kSpmmRowBlock;
  const int64_t gy = (n + (int64_t)LN * VN - 1) / ((int64_t)LN * VN);
  if (gx > INT_MAX || gy > 65535) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  spmm_tile_kernel<T, OffT, LN, VN><<<dim3((unsigned)gx, (unsigned)gy), kThreads, 0, h->stream>>>(
      reinterpret_cast<const OffT*>(A->row_offsets), A->const_col_data,
      reinterpret_cast<const T*>(A->const_val_data), B, ldb, C, ldc, alpha, beta, A->rows, n, A->nnz,
      plan_of(A)->dev_err, plan_of(A)->wait_cfg);
  impl(h)->launches++;
  return status_of(cudaGetLastError());
}

// Bytes of the balanced kernel's carry array for this matrix and N.
inline size_t balanced_carry_bytes(alphasparseSpMatDescr_t A, int64_t n) {
  const size_t es = elem_size(A->data_type);
  if (A->data_type != ALPHA_R_32F && A->data_type != ALPHA_R_64F) return 0;  // only the fp32 / fp64 kernels carry
  const int64_t tiles = (A->rows + A->nnz + kMergeItems - 1) / kMergeItems;
  return round256((size_t)(tiles > 0 ? tiles : 1) * (size_t)spmm_balanced_carry_ld(n, es) * es);
}

// Which kernel family a call runs.  ALG1 names the reference's row-balanced algorithm: rows stay
// whole (tile / row-block kernels, bit-equal to the CPU path).  ALG2, ALG3 and ALG5 name its
// element-balanced, merge-path and flat algorithms: the merge-path kernel.  Everything else
// (DEFAULT, ALG4 "adaptive", the COO names) picks from the plan: whole rows while every 128-row
// block fits the staging buffer - then no row is long and the blocks are even - else merge-path.
enum SpmmFamily { kSpmmRows = 0, kSpmmBalanced = 1 };
inline SpmmFamily family_for(const Plan* p, alphasparseSpMMAlg_t alg, bool vec, size_t elem) {
  const char* f = getenv("ASP_SPMM_VARIANT");
  if (!vec) return kSpmmRows;  // the balanced kernel moves 16-byte packs
  if (f && !strcmp(f, "rows")) return kSpmmRows;
  if (f && !strcmp(f, "balanced")) return kSpmmBalanced;
  switch (alg) {
    case ALPHASPARSE_SPMM_CSR_ALG1: return kSpmmRows;
    case ALPHASPARSE_SPMM_CSR_ALG2:
    case ALPHASPARSE_SPMM_CSR_ALG3:
    case ALPHASPARSE_SPMM_CSR_ALG5: return kSpmmBalanced;
    default: return p->max_block_nnz <= (elem == 4 ? kSpmmStageCap32 : kSpmmStageCap64) ? kSpmmRows : kSpmmBalanced;
  }
}

template <typename T, typename OffT>
alphasparseStatus_t spmm_t(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const T* B, int64_t ldb,
                           T* C, int64_t ldc, T alpha, T beta, int64_t n, alphasparseSpMMAlg_t alg, void* ext) {
  constexpr int VN = 16 / (int)sizeof(T);
  if (A->rows == 0 || n == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  const bool vec = (n % VN == 0) && (ldb % VN == 0) && (ldc % VN == 0) && aligned(B, 16) && aligned(C, 16);
  Plan* p = plan_of(A);
  if (family_for(p, alg, vec, sizeof(T)) == kSpmmBalanced) {
    // carry array: the caller's buffer (alphasparseSpMM_bufferSize covers it), else one the plan keeps,
    // allocated when a product of this width is first prepared or run
    void* carry = ext;
    if (!carry) {
      const size_t need = balanced_carry_bytes(A, n);
      if (p->spmm_carry_bytes < need) {
        ASP_CUDA(cudaStreamSynchronize(h->stream));
        cudaFree(p->spmm_carry);
        p->spmm_carry = nullptr;
        p->spmm_carry_bytes = 0;
        ASP_CUDA(cudaMalloc(&p->spmm_carry, need));
        p->spmm_carry_bytes = need;
      }
      carry = p->spmm_carry;
    }
    p->last_spmm = "merge-path";
    return spmm_balanced_t<T, OffT>(h, A, B, ldb, C, ldc, alpha, beta, n, carry);
  }
  p->last_spmm = "row-block";
  if (!vec) return launch_rb<T, OffT, 32, 1>(h, A, B, ldb, C, ldc, alpha, beta, n);
  if (n >= env_int("ASP_SPMM_STAGE_MIN_N", 16) && env_int("ASP_SPMM_STAGE", 0)) {
    // opt-in (measured slower than the tile kernel, see the profile notes): blocks that touch B in runs take B
    // through shared memory by TMA, one fetch per 64-row chunk instead of one per entry
    bool ran = false;
    const alphasparseStatus_t s = spmm_stage_try<T>(h, A, B, ldb, C, ldc, alpha, beta, n, false, &ran);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    if (ran) {
      p->last_spmm = "staged";
      return s;
    }
  }
  const int64_t lanes = n / VN;
  const bool tile_ok = plan_of(A)->max_block_nnz <= (sizeof(T) == 4 ? kSpmmStageCap32 : kSpmmStageCap64) && aligned(A->const_val_data, 16) &&
                       aligned(A->const_col_data, 16) && env_int("ASP_SPMM_TMA", 1);
  if (tile_ok) {
    plan_of(A)->last_spmm = "tile";
    if constexpr (sizeof(T) == 4) {
      // from N = 128 on a lane keeps two 16-byte packs (half the instructions per entry and column; measured
      // 1.50 -> 1.44 ms at N = 128, but 0.37 -> 0.51 ms at N = 32, where it is not used)
      // (only when the lanes' packs tile N exactly: both packs of every lane are then inside the matrix)
      const int64_t l8 = n / 8;
      if (env_int("ASP_SPMM_WIDE", 1) && n % 8 == 0 && (l8 == 16 || (l8 >= 32 && l8 % 32 == 0))) {
        if (l8 <= 16) return launch_tile<T, OffT, 16, 8>(h, A, B, ldb, C, ldc, alpha, beta, n);
        return launch_tile<T, OffT, 32, 8>(h, A, B, ldb, C, ldc, alpha, beta, n);
      }
    }
    if (lanes <= 1) return launch_tile<T, OffT, 1, VN>(h, A, B, ldb, C, ldc, alpha, beta, n);
    if (lanes <= 2) return launch_tile<T, OffT, 2, VN>(h, A, B, ldb, C, ldc, alpha, beta, n);
    if (lanes <= 4) return launch_tile<T, OffT, 4, VN>(h, A, B, ldb, C, ldc, alpha, beta, n);
    if (lanes <= 8) return launch_tile<T, OffT, 8, VN>(h, A, B, ldb, C, ldc, alpha, beta, n);
    if (lanes <= 16) return launch_tile<T, OffT, 16, VN>(h, A, B, ldb, C, ldc, alpha, beta, n);
    return launch_tile<T, OffT, 32, VN>(h, A, B, ldb, C, ldc, alpha, beta, n);
  }
  if (lanes <= 1) return launch_rb<T, OffT, 1, VN>(h, A, B, ldb, C, ldc, alpha, beta, n);
  if (lanes <= 2) return launch_rb<T, OffT, 2, VN>(h, A, B, ldb, C, ldc, alpha, beta, n);
  if (lanes <= 4) return launch_rb<T, OffT, 4, VN>(h, A, B, ldb, C, ldc, alpha, beta, n);
  if (lanes <= 8) return launch_rb<T, OffT, 8, VN>(h, A, B, ldb, C, ldc, alpha, beta, n);
  if (lanes <= 16) return launch_rb<T, OffT, 16, VN>(h, A, B, ldb, C, ldc, alpha, beta, n);
  return launch_rb<T, OffT, 32, VN>(h, A, B, ldb, C, ldc, alpha, beta, n);
}

// dst[c * ld_dst + r] = src[r * ld_src + c] for an r_n x c_n row-major source: 32 x 32 tiles through
// shared memory, both sides coalesced.  Used to present column-major B and C to the row-major kernels
// (the reference transposes them in place with freshly allocated buffers on every call,
// cuda/kernel/level3/alphasparse_spmm.cu:131-285, cuda/format/transpose_dn_mat.h:17-34).
template <typename W>
__global__ void __launch_bounds__(256) transpose_kernel(const W* __restrict__ src, int64_t ld_src, int64_t r_n,
                                                        int64_t c_n, W* __restrict__ dst, int64_t ld_dst) {
  __shared__ W tile[32][33];
  const int64_t tiles_c = (c_n + 31) / 32;
  const int64_t tiles = ((r_n + 31) / 32) * tiles_c;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
    const int64_t r0 = (t / tiles_c) * 32, c0 = (t % tiles_c) * 32;
#pragma unroll
    for (int i = ty; i < 32; i += 8)
      if (r0 + i < r_n && c0 + tx < c_n) tile[i][tx] = src[(r0 + i) * ld_src + c0 + tx];
    __syncthreads();
#pragma unroll
    for (int i = ty; i < 32; i += 8)
      if (c0 + i < c_n && r0 + tx < r_n) dst[(c0 + i) * ld_dst + r0 + tx] = tile[tx][i];
    __syncthreads();
  }
}

alphasparseStatus_t transpose_any(alphasparseHandle_t h, const void* src, int64_t ld_src, int64_t r_n, int64_t c_n,
                                  void* dst, int64_t ld_dst, size_t elem) {
  if (r_n == 0 || c_n == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  int64_t tiles = ((r_n + 31) / 32) * ((c_n + 31) / 32);
  const int64_t cap = (int64_t)impl(h)->sm_count * 16;
  const unsigned grid = (unsigned)(tiles < cap ? tiles : cap);
  if (elem == 2)
    transpose_kernel<uint16_t><<<grid, 256, 0, h->stream>>>((const uint16_t*)src, ld_src, r_n, c_n, (uint16_t*)dst, ld_dst);
  else if (elem == 4)
    transpose_kernel<uint32_t><<<grid, 256, 0, h->stream>>>((const uint32_t*)src, ld_src, r_n, c_n, (uint32_t*)dst, ld_dst);
  else if (elem == 1)
    transpose_kernel<uint8_t><<<grid, 256, 0, h->stream>>>((const uint8_t*)src, ld_src, r_n, c_n, (uint8_t*)dst, ld_dst);
  else if (elem == 16)
    transpose_kernel<uint4><<<grid, 256, 0, h->stream>>>((const uint4*)src, ld_src, r_n, c_n, (uint4*)dst, ld_dst);
  else
    transpose_kernel<uint64_t><<<grid, 256, 0, h->stream>>>((const uint64_t*)src, ld_src, r_n, c_n, (uint64_t*)dst, ld_dst);
  impl(h)->launches++;
  return status_of(cudaGetLastError());
}

alphasparseStatus_t check_spmm_args(alphasparseHandle_t h, alphasparseOperation_t opA,
                                    alphasparseOperation_t opB, const void* alpha,
                                    alphasparseSpMatDescr_t A, alphasparseDnMatDescr_t B,
                                    const void* beta, alphasparseDnMatDescr_t C,
                                    alphasparseDataType computeType) {
  if (!h || !h->impl) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!alpha || !beta || !A || !B || !C) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (h->pointer_mode != ALPHA_SPARSE_POINTER_MODE_HOST) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (opB != ALPHA_SPARSE_OPERATION_NON_TRANSPOSE) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  const bool tr = opA != ALPHA_SPARSE_OPERATION_NON_TRANSPOSE;  // runs on the transposed matrix the plan keeps
  alphasparseStatus_t s = validate_csr(A);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  if (!B->init || !C->init) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
  if (B->order != C->order) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;  // both row-major or both column-major
  if (B->rows != (tr ? A->rows : A->cols) || C->rows != (tr ? A->cols : A->rows) || B->cols != C->cols)
    return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  const bool row = B->order == ALPHASPARSE_ORDER_ROW;
  if (B->ld < (row ? B->cols : B->rows) || C->ld < (row ? C->cols : C->rows)) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if ((!B->values && B->rows > 0 && B->cols > 0) || (!C->values && C->rows > 0 && C->cols > 0))
    return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  const bool plain = (A->data_type == ALPHA_R_32F || A->data_type == ALPHA_R_64F) &&
                     B->data_type == A->data_type && C->data_type == A->data_type &&
                     computeType == A->data_type;
  const bool mixed = A->data_type == ALPHA_R_16BF && B->data_type == ALPHA_R_16BF &&
                     C->data_type == ALPHA_R_32F && computeType == ALPHA_R_32F;
  // complex, int8 and fp16 instances: one plain kernel; complex: the transposed copy holds the values as
  // they are, so the conjugate transpose is not offered
  const bool conj_c = opA == ALPHA_SPARSE_OPERATION_CONJUGATE_TRANSPOSE &&
                      (A->data_type == ALPHA_C_32F || A->data_type == ALPHA_C_64F);
  const bool other = !conj_c && spmm_other_types(A->data_type, B->data_type, C->data_type, computeType);
  if (!plain && !mixed && !other) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

}  // namespace
}  // namespace asp

using namespace asp;

extern "C" {

alphasparseStatus_t alphasparseSpMM(alphasparseHandle_t h, alphasparseOperation_t opA,
                                    alphasparseOperation_t opB, const void* alpha,
                                    alphasparseSpMatDescr_t A, alphasparseDnMatDescr_t B,
                                    const void* beta, alphasparseDnMatDescr_t C,
                                    alphasparseDataType computeType, alphasparseSpMMAlg_t alg,
                                    void* externalBuffer) {
  alphasparseStatus_t s = check_spmm_args(h, opA, opB, alpha, A, B, beta, C, computeType);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  if (opA != ALPHA_SPARSE_OPERATION_NON_TRANSPOSE) {
    alphasparseSpMatDescr_t At = nullptr;
    s = transposed_of(h, A, &At);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    return alphasparseSpMM(h, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, opB, alpha, At, B, beta, C, computeType, alg,
                           externalBuffer);
  }
  if (!A->info) {
    s = analyse(h, A);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  }
  if (plan_of(A)->device != h->device) return ALPHA_SPARSE_STATUS_INVALID_VALUE;  // the plan's arrays live on another GPU
  if (B->order == ALPHASPARSE_ORDER_COL) {
    // Column-major B and C: row-major copies in the caller's buffer (sizes: alphasparseSpMM_bufferSize),
    // the row-major kernel, and C copied back.  B and C themselves keep their layout.
    if (!externalBuffer) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    const size_t eb = elem_size(B->data_type), ec = elem_size(C->data_type);
    const int64_t n = C->cols;
    _alphasparse_dnmat_descr Bt = *B, Ct = *C;
    Bt.order = Ct.order = ALPHASPARSE_ORDER_ROW;
    Bt.ld = Ct.ld = n;
    Bt.values = externalBuffer;
    Ct.values = reinterpret_cast<unsigned char*>(externalBuffer) + round256((size_t)B->rows * n * eb);
    void* rest = reinterpret_cast<unsigned char*>(Ct.values) + round256((size_t)C->rows * n * ec);  // the carry array's place
    s = transpose_any(h, B->values, B->ld, n, B->rows, Bt.values, n, eb);
    const bool reads_c = spmm_other_types(A->data_type, B->data_type, C->data_type, computeType)
                             ? spmm_other_reads_c(computeType, beta)
                             : (computeType == ALPHA_R_64F ? *(const double*)beta != 0.0 : *(const float*)beta != 0.f);
    if (s == ALPHA_SPARSE_STATUS_SUCCESS && reads_c) s = transpose_any(h, C->values, C->ld, n, C->rows, Ct.values, n, ec);
    if (s == ALPHA_SPARSE_STATUS_SUCCESS)
      s = alphasparseSpMM(h, opA, opB, alpha, A, &Bt, beta, &Ct, computeType, alg, rest);
    if (s == ALPHA_SPARSE_STATUS_SUCCESS) s = transpose_any(h, Ct.values, n, C->rows, n, C->values, C->ld, ec);
    return s;
  }
  const int64_t n = C->cols;
  if (spmm_other_types(A->data_type, B->data_type, C->data_type, computeType)) {
    plan_of(A)->last_spmm = "types";
    return spmm_other_run(h, A, B, C, alpha, beta);
  }
  if (A->data_type == ALPHA_R_16BF) {
    // bf16 operands exist only for the tensor-core variant.
    if (!spmm_tc_applicable(A, B, C)) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    plan_of(A)->last_spmm = "tcgen05";
    return spmm_tc_run(h, A, B, C, *(const float*)alpha, *(const float*)beta, false);
  }
  if (alg == ALPHASPARSE_SPMM_CSR_ALG6) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;  // needs bf16 operands
  const bool o64 = A->row_type == ALPHA_SPARSE_INDEXTYPE_I64;
  if (A->data_type == ALPHA_R_32F) {
    const float al = *(const float*)alpha, be = *(const float*)beta;
    return o64 ? spmm_t<float, int64_t>(h, A, (const float*)B->values, B->ld, (float*)C->values, C->ld, al, be, n, alg, externalBuffer)
               : spmm_t<float, int32_t>(h, A, (const float*)B->values, B->ld, (float*)C->values, C->ld, al, be, n, alg, externalBuffer);
  }
  const double al = *(const double*)alpha, be = *(const double*)beta;
  return o64 ? spmm_t<double, int64_t>(h, A, (const double*)B->values, B->ld, (double*)C->values, C->ld, al, be, n, alg, externalBuffer)
             : spmm_t<double, int32_t>(h, A, (const double*)B->values, B->ld, (double*)C->values, C->ld, al, be, n, alg, externalBuffer);
}

alphasparseStatus_t alphasparseSpMM_bufferSize(alphasparseHandle_t h, alphasparseOperation_t opA,
                                               alphasparseOperation_t opB, const void* alpha,
                                               alphasparseSpMatDescr_t A, alphasparseDnMatDescr_t B,
                                               const void* beta, alphasparseDnMatDescr_t C,
                                               alphasparseDataType computeType,
                                               alphasparseSpMMAlg_t, size_t* bufferSize) {
  if (!bufferSize) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  alphasparseStatus_t s = check_spmm_args(h, opA, opB, alpha, A, B, beta, C, computeType);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  // the carry array of the merge-path kernel (whichever kernel the call then runs), never zero so
  // that cudaMalloc returns a pointer; with column-major operands the row-major copies of B and C first
  const alphasparseSpMatDescr_t Aop = A;
  size_t carry = balanced_carry_bytes(Aop, C->cols);
  if (opA != ALPHA_SPARSE_OPERATION_NON_TRANSPOSE) {  // the product runs on the transposed matrix: cols + nnz items
    const size_t es = elem_size(A->data_type);
    const int64_t tiles = (A->cols + A->nnz + kMergeItems - 1) / kMergeItems;
    if (A->data_type == ALPHA_R_32F || A->data_type == ALPHA_R_64F) carry = round256((size_t)(tiles > 0 ? tiles : 1) * (size_t)spmm_balanced_carry_ld(C->cols, es) * es);
  }
  *bufferSize = carry > 256 ? carry : 256;
  if (B->order == ALPHASPARSE_ORDER_COL)
    *bufferSize += round256((size_t)B->rows * B->cols * elem_size(B->data_type)) +
                   round256((size_t)C->rows * C->cols * elem_size(C->data_type));
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseSpMM_preprocess(alphasparseHandle_t h, alphasparseOperation_t opA,
                                               alphasparseOperation_t opB, const void* alpha,
                                               alphasparseSpMatDescr_t A, alphasparseDnMatDescr_t B,
                                               const void* beta, alphasparseDnMatDescr_t C,
                                               alphasparseDataType computeType,
                                               alphasparseSpMMAlg_t alg, size_t* bufferSize) {
  alphasparseStatus_t s = check_spmm_args(h, opA, opB, alpha, A, B, beta, C, computeType);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  if (opA != ALPHA_SPARSE_OPERATION_NON_TRANSPOSE) {
    alphasparseSpMatDescr_t At = nullptr;
    s = transposed_of(h, A, &At);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    return alphasparseSpMM_preprocess(h, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, opB, alpha, At, B, beta, C, computeType,
                                      alg, bufferSize);
  }
  if (bufferSize) {
    const size_t carry = balanced_carry_bytes(A, C->cols);
    *bufferSize = carry > 256 ? carry : 256;
    if (B->order == ALPHASPARSE_ORDER_COL)
      *bufferSize += round256((size_t)B->rows * B->cols * elem_size(B->data_type)) +
                     round256((size_t)C->rows * C->cols * elem_size(C->data_type));
  }
  if (!A->info) {
    s = analyse(h, A);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  }
  if (spmm_other_types(A->data_type, B->data_type, C->data_type, computeType)) return ALPHA_SPARSE_STATUS_SUCCESS;
  if (A->data_type == ALPHA_R_16BF) {
    _alphasparse_dnmat_descr Bt = *B, Ct = *C;
    if (B->order == ALPHASPARSE_ORDER_COL) {  // the kernel will see the row-major copies (aligned, ld = N)
      Bt.order = Ct.order = ALPHASPARSE_ORDER_ROW;
      Bt.ld = Ct.ld = C->cols;
      Bt.values = Ct.values = reinterpret_cast<void*>(uintptr_t(256));
    }
    if (!spmm_tc_applicable(A, &Bt, &Ct)) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    return spmm_tc_run(h, A, &Bt, &Ct, 0.f, 0.f, true);
  }
  // The merge-path kernel's carry array, so that a later alphasparseSpMM without an external buffer
  // allocates nothing.  (Operand alignment is judged on the descriptors as they are now.)
  {
    Plan* p = plan_of(A);
    const size_t es = elem_size(A->data_type);
    const int64_t n = C->cols, vn = 16 / (int64_t)es;
    const bool row = B->order == ALPHASPARSE_ORDER_ROW;
    const bool vec = !row || ((n % vn == 0) && (B->ld % vn == 0) && (C->ld % vn == 0) && aligned(B->values, 16) &&
                              aligned(C->values, 16));
    if (row && vec && n > 0 && A->rows > 0 && family_for(p, alg, vec, es) == kSpmmRows &&
        n >= env_int("ASP_SPMM_STAGE_MIN_N", 16) && env_int("ASP_SPMM_STAGE", 0)) {
      bool would_run = false;  // builds the chunk lists of the staged kernel now
      s = es == 4 ? spmm_stage_try<float>(h, A, (const float*)B->values, B->ld, (float*)C->values, C->ld, 0.f, 0.f, n, true, &would_run)
                  : spmm_stage_try<double>(h, A, (const double*)B->values, B->ld, (double*)C->values, C->ld, 0.0, 0.0, n, true, &would_run);
      if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    }
    if (row && n > 0 && A->rows > 0 && family_for(p, alg, vec, es) == kSpmmBalanced) {
      const size_t need = balanced_carry_bytes(A, n);
      if (p->spmm_carry_bytes < need) {
        ASP_CUDA(cudaStreamSynchronize(h->stream));
        cudaFree(p->spmm_carry);
        p->spmm_carry = nullptr;
        p->spmm_carry_bytes = 0;
        ASP_CUDA(cudaMalloc(&p->spmm_carry, need));
        p->spmm_carry_bytes = need;
      }
    }
  }
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
