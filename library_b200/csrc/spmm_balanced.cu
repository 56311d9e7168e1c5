// Load-balanced CSR SpMM  C = alpha*A*B + beta*C  (row-major B and C) for matrices whose row
// lengths are skewed: the merge-path decomposition of the SpMV kernel carried over to N columns.
//
// The reference has four balanced algorithms (cuda/kernel/level3/alphasparse_spmm_csr.h:
// element-balanced :200-239,241-393, merge-path :64-106,395-533, adaptive :535-571,573-795, flat
// :797-905); all of them scale C by beta in a first pass and then accumulate with atomicAdd.  Here
// a CTA owns one tile of the analysed merge-path partition (kMergeItems rows + entries, the same
// tiles the SpMV kernel uses, so no row however long occupies more than one tile's worth of a CTA),
// splits the tile's ENTRIES evenly over its lane groups, and combines the pieces of rows that
// straddle groups in shared memory and the pieces of rows that straddle tiles through a carry
// array and a small second kernel - in a fixed order, without atomics, so results are reproducible
// run to run.  A row that is split is summed piecewise, so it equals the reference's CPU result
// within rounding, not bit for bit (rows inside one lane group's range still do).
#include <climits>

#include "asp_internal.h"

namespace asp {
namespace {

template <typename T> struct BPack;
template <> struct BPack<float> { using V = float4; static constexpr int N = 4; };
template <> struct BPack<double> { using V = double2; static constexpr int N = 2; };

template <typename T>
__device__ __forceinline__ void ldg_pack(const T* p, T (&r)[BPack<T>::N]) {
  const typename BPack<T>::V v = __ldg(reinterpret_cast<const typename BPack<T>::V*>(p));
  if constexpr (BPack<T>::N == 4) { r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w; }
  else { r[0] = v.x; r[1] = v.y; }
}
template <typename T>
__device__ __forceinline__ void st_pack(T* p, const T (&r)[BPack<T>::N]) {
  if constexpr (BPack<T>::N == 4) *reinterpret_cast<float4*>(p) = make_float4(r[0], r[1], r[2], r[3]);
  else *reinterpret_cast<double2*>(p) = make_double2(r[0], r[1]);
}

// C row := alpha*acc + beta*C row for the VN columns this lane owns.
template <typename T>
__device__ __forceinline__ void finish_row(T* c, const T (&acc)[BPack<T>::N], T alpha, T beta) {
  constexpr int VN = BPack<T>::N;
  T out[VN];
  if (beta == T(0)) {
#pragma unroll
    for (int v = 0; v < VN; ++v) out[v] = alpha * acc[v];
  } else {
    T old[VN];
    ldg_pack<T>(c, old);
#pragma unroll
    for (int v = 0; v < VN; ++v) out[v] = fma(alpha, acc[v], beta * old[v]);
  }
  st_pack<T>(c, out);
}

// One CTA per (merge-path tile, slab of LN*VN columns of C).  LN lanes share an entry range, each
// lane keeps VN adjacent columns.
template <typename T, typename OffT, int LN>
__global__ void __launch_bounds__(kThreads)
spmm_merge_kernel(const OffT* __restrict__ rp, const int* __restrict__ col, const T* __restrict__ val,
                  const T* __restrict__ B, int64_t ldb, T* __restrict__ C, int64_t ldc, T alpha, T beta,
                  int64_t rows, int64_t n, int64_t nnz, const int32_t* __restrict__ tile_row,
                  T* __restrict__ carry, int64_t carry_ld) {
  constexpr int VN = BPack<T>::N;
  constexpr int NG = kThreads / LN;
  constexpr int ITEMS = kMergeItems;
  constexpr int W = LN * VN;  // columns per slab
  __shared__ int s_col[ITEMS];
  __shared__ T s_val[ITEMS];
  __shared__ int s_end[ITEMS + 1];  // s_end[i]: where row row_s + i ends, counted from the tile's first entry
  __shared__ __align__(16) T s_head[NG][W];
  __shared__ __align__(16) T s_tail[NG][W];
  __shared__ int s_head_row[NG];    // tile-relative row of the group's head piece, -1: none
  __shared__ int s_tail_kind[NG];   // 0: no open piece, 1: the open row began in this group, 2: it began earlier

  const int tid = threadIdx.x;
  const int lane = tid % LN, grp = tid / LN;
  const int64_t t = blockIdx.x;
  const int row_s = tile_row[t], row_e = tile_row[t + 1];
  const int64_t total = rows + nnz;
  const int64_t diag_s = t * (int64_t)ITEMS;
  const int64_t diag_e = diag_s + ITEMS < total ? diag_s + ITEMS : total;
  const int64_t nz_s = diag_s - row_s, nz_e = diag_e - row_e;
  const int tile_rows = row_e - row_s;
  const int E = (int)(nz_e - nz_s);
  const int64_t c0 = (int64_t)blockIdx.y * W + (int64_t)lane * VN;
  const bool col_ok = c0 < n;

  for (int i = tid; i < E; i += kThreads) {
    s_col[i] = __ldcs(col + nz_s + i);
    s_val[i] = __ldcs(val + nz_s + i);
  }
  for (int i = tid; i < tile_rows; i += kThreads) s_end[i] = (int)((int64_t)rp[row_s + i + 1] - nz_s);
  if (tid == 0) s_end[tile_rows] = INT_MAX;  // the row still open at the tile's end never ends here
  if (tid < NG) {
    s_head_row[tid] = -1;
    s_tail_kind[tid] = 0;
  }
  __syncthreads();

  // rows without an entry in this tile: C row := beta * C row (a row that only ends here, with all
  // its entries in earlier tiles, is such a row too; the carry kernel adds what those tiles summed)
  if (col_ok) {
    for (int i = grp; i < tile_rows; i += NG) {
      const int b = i == 0 ? 0 : s_end[i - 1];
      if (s_end[i] == b) {
        T zero[VN];
#pragma unroll
        for (int v = 0; v < VN; ++v) zero[v] = T(0);
        finish_row<T>(C + (int64_t)(row_s + i) * ldc + c0, zero, alpha, beta);
      }
    }
  }

  // this group's share of the tile's entries
  const int per = (E + NG - 1) / NG;
  const int lo = grp * per < E ? grp * per : E;
  const int hi = lo + per < E ? lo + per : E;
  T acc[VN];
#pragma unroll
  for (int v = 0; v < VN; ++v) acc[v] = T(0);
  if (hi > lo) {
    // first row with an end beyond lo: the row entry lo belongs to
    int a = 0, b = tile_rows;
    while (a < b) {
      const int mid = (a + b) >> 1;
      if (s_end[mid] <= lo) a = mid + 1;
      else b = mid;
    }
    int i = a;
    bool fresh = (i == 0 ? 0 : s_end[i - 1]) == lo;  // the row starts exactly where the range starts
    int next_end = s_end[i];
    const T* __restrict__ Bc = B + c0;
    for (int k = lo; k < hi; k += 4) {
      int q[4];
      T av[4];
      T bv[4][VN];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool in = k + j < hi;
        q[j] = s_col[in ? k + j : lo];
        av[j] = in ? s_val[k + j] : T(0);
      }
      if (col_ok) {
#pragma unroll
        for (int j = 0; j < 4; ++j) ldg_pack<T>(Bc + (int64_t)q[j] * ldb, bv[j]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (k + j < hi) {
          if (col_ok) {
#pragma unroll
            for (int v = 0; v < VN; ++v) acc[v] = fma(av[j], bv[j][v], acc[v]);
          }
          if (k + j + 1 == next_end) {  // the row ends with this entry
            if (fresh) {
              if (col_ok) finish_row<T>(C + (int64_t)(row_s + i) * ldc + c0, acc, alpha, beta);
            } else {
              if (col_ok) st_pack<T>(&s_head[grp][lane * VN], acc);
              if (lane == 0) s_head_row[grp] = i;
            }
#pragma unroll
            for (int v = 0; v < VN; ++v) acc[v] = T(0);
            ++i;
            while (s_end[i] == k + j + 1) ++i;  // rows without entries (handled above)
            next_end = s_end[i];
            fresh = true;
          }
        }
      }
    }
    // an open piece: the last entry's row goes on beyond the range
    const int last_start = i == 0 ? 0 : s_end[i - 1];
    if (last_start < hi) {
      if (col_ok) st_pack<T>(&s_tail[grp][lane * VN], acc);
      if (lane == 0) s_tail_kind[grp] = fresh ? 1 : 2;
    }
  }
  __syncthreads();

  // pieces of a row that straddles groups, added in group order: the tail of the group it began
  // in, the pieces of the groups that lie wholly inside it, the head of the group it ends in
  const int G = per > 0 ? (E + per - 1) / per : 0;  // groups with entries
  if (col_ok) {
    if (s_head_row[grp] >= 0) {
      int gs = grp - 1;
      while (gs > 0 && s_tail_kind[gs] == 2) --gs;
      T sum[VN];
#pragma unroll
      for (int v = 0; v < VN; ++v) sum[v] = T(0);
      for (int g = gs; g < grp; ++g)
#pragma unroll
        for (int v = 0; v < VN; ++v) sum[v] += s_tail[g][lane * VN + v];
#pragma unroll
      for (int v = 0; v < VN; ++v) sum[v] += s_head[grp][lane * VN + v];
      finish_row<T>(C + (int64_t)(row_s + s_head_row[grp]) * ldc + c0, sum, alpha, beta);
    }
    // the row still open at the tile's end: its pieces go to the carry array
    if (grp == (G > 0 ? G - 1 : 0)) {
      T sum[VN];
#pragma unroll
      for (int v = 0; v < VN; ++v) sum[v] = T(0);
      if (G > 0 && s_tail_kind[grp] != 0) {
        int gs = grp;
        while (gs > 0 && s_tail_kind[gs] == 2) --gs;
        for (int g = gs; g <= grp; ++g)
#pragma unroll
          for (int v = 0; v < VN; ++v) sum[v] += s_tail[g][lane * VN + v];
      }
      st_pack<T>(carry + t * carry_ld + c0, sum);
    }
  }
}

// Adds what earlier tiles summed for a row to the row, in tile order: tile t's carry belongs to
// row tile_row[t+1]; the thread group of the first tile of a run of tiles that all end inside the
// same row adds the whole run.  One thread per (tile, column).
template <typename T>
__global__ void __launch_bounds__(256) spmm_merge_fixup_kernel(const int32_t* __restrict__ tile_row,
                                                               const T* __restrict__ carry, int64_t carry_ld,
                                                               int64_t tiles, int64_t rows, int64_t n,
                                                               T* __restrict__ C, int64_t ldc, T alpha) {
  const int64_t idx = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  const int64_t t = idx / n, c = idx % n;
  if (t >= tiles) return;
  const int32_t r = tile_row[t + 1];
  if (r >= rows) return;
  if (t > 0 && tile_row[t] == r) return;
  T sum = T(0);
  for (int64_t u = t; u < tiles && tile_row[u + 1] == r; ++u) sum += carry[u * carry_ld + c];
  C[(int64_t)r * ldc + c] = fma(alpha, sum, C[(int64_t)r * ldc + c]);
}

template <typename T, typename OffT, int LN>
alphasparseStatus_t launch_merge(alphasparseHandle_t h, alphasparseSpMatDescr_t A, Plan* p, const T* B, int64_t ldb,
                                 T* C, int64_t ldc, T alpha, T beta, int64_t n, T* carry, int64_t carry_ld) {
  constexpr int W = LN * BPack<T>::N;
  const int64_t gy = (n + W - 1) / W;
  if (p->merge_tiles > INT_MAX || gy > 65535) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  spmm_merge_kernel<T, OffT, LN><<<dim3((unsigned)p->merge_tiles, (unsigned)gy), kThreads, 0, h->stream>>>(
      reinterpret_cast<const OffT*>(A->row_offsets), A->const_col_data, reinterpret_cast<const T*>(A->const_val_data), B,
      ldb, C, ldc, alpha, beta, A->rows, n, A->nnz, p->merge_tile_row, carry, carry_ld);
  const int64_t threads = p->merge_tiles * n;
  spmm_merge_fixup_kernel<T><<<(unsigned)((threads + 255) / 256), 256, 0, h->stream>>>(
      p->merge_tile_row, carry, carry_ld, p->merge_tiles, A->rows, n, C, ldc, alpha);
  impl(h)->launches += 2;
  return status_of(cudaGetLastError());
}

}  // namespace

// Columns of the carry array per tile for an N-column product (N rounded up to whole 16-byte packs).
int64_t spmm_balanced_carry_ld(int64_t n, size_t elem) {
  const int64_t vn = 16 / (int64_t)elem;
  const int64_t w = 32 * vn;  // the widest slab
  return n <= w ? ((n + vn - 1) / vn) * vn : ((n + w - 1) / w) * w;
}

template <typename T, typename OffT>
alphasparseStatus_t spmm_balanced_t(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const T* B, int64_t ldb, T* C,
                                    int64_t ldc, T alpha, T beta, int64_t n, void* carry) {
  Plan* p = plan_of(A);
  constexpr int VN = BPack<T>::N;
  const int64_t ld = spmm_balanced_carry_ld(n, sizeof(T));
  T* cr = reinterpret_cast<T*>(carry);
  const int64_t lanes = (n + VN - 1) / VN;
  if (lanes <= 2) return launch_merge<T, OffT, 2>(h, A, p, B, ldb, C, ldc, alpha, beta, n, cr, ld);
  if (lanes <= 4) return launch_merge<T, OffT, 4>(h, A, p, B, ldb, C, ldc, alpha, beta, n, cr, ld);
  if (lanes <= 8) return launch_merge<T, OffT, 8>(h, A, p, B, ldb, C, ldc, alpha, beta, n, cr, ld);
  if (lanes <= 16) return launch_merge<T, OffT, 16>(h, A, p, B, ldb, C, ldc, alpha, beta, n, cr, ld);
  return launch_merge<T, OffT, 32>(h, A, p, B, ldb, C, ldc, alpha, beta, n, cr, ld);
}

template alphasparseStatus_t spmm_balanced_t<float, int32_t>(alphasparseHandle_t, alphasparseSpMatDescr_t, const float*, int64_t, float*, int64_t, float, float, int64_t, void*);
template alphasparseStatus_t spmm_balanced_t<float, int64_t>(alphasparseHandle_t, alphasparseSpMatDescr_t, const float*, int64_t, float*, int64_t, float, float, int64_t, void*);
template alphasparseStatus_t spmm_balanced_t<double, int32_t>(alphasparseHandle_t, alphasparseSpMatDescr_t, const double*, int64_t, double*, int64_t, double, double, int64_t, void*);
template alphasparseStatus_t spmm_balanced_t<double, int64_t>(alphasparseHandle_t, alphasparseSpMatDescr_t, const double*, int64_t, double*, int64_t, double, double, int64_t, void*);

}  // namespace asp
