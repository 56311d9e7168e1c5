// The preprocessing pass of the CSR descriptor: row-length classes with per-class row lists
// (stable, in row order), the merge-path tile partition, the statistics that pick the SpMV
// variant, a structural validator, and the nnz-balanced row partition used to shard a matrix
// across GPUs.
//
// The reference's CSR descriptor only records pointers
// (cuda/format/alphasparse_create_csr.h:6-63).  Its kernels redo their partitioning on every
// call: find_rows appends rows to bins with atomics, so the order depends on arrival
// (cuda/kernel/level2/alphasparse_spmv_csr_adaptive2.h:6-48), and the merge-path search runs
// per SpMV (alphasparse_spmv_csr_merge_ginkgo.h:133-158).  Here both are computed once,
// deterministically, and kept in the descriptor.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_select.cuh>
#include <thrust/iterator/counting_iterator.h>

#include <new>

#include "asp_internal.h"

namespace asp {

namespace {

enum { C_SHORT = 0, C_MEDIUM, C_LONG, C_EMPTY, C_NNZ_SHORT, C_MAXLEN, C_BAD, C_COUNT };

template <typename OffT>
__global__ void __launch_bounds__(256) row_stats_kernel(const OffT* __restrict__ rp, int64_t rows,
                                                        int64_t nnz,
                                                        unsigned long long* __restrict__ ctr) {
  unsigned long long loc[C_COUNT] = {0, 0, 0, 0, 0, 0, 0};
  for (int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; r < rows;
       r += (int64_t)gridDim.x * blockDim.x) {
    const int64_t s = (int64_t)rp[r], e = (int64_t)rp[r + 1];
    const int64_t len = e - s;
    if (len < 0 || s < 0 || e > nnz) {
      loc[C_BAD] = 1;
      continue;
    }
    if (len <= kShortMax) {
      loc[C_SHORT]++;
      loc[C_NNZ_SHORT] += (unsigned long long)len;
    } else if (len <= kMediumMax) {
      loc[C_MEDIUM]++;
    } else {
      loc[C_LONG]++;
    }
    if (len == 0) loc[C_EMPTY]++;
    if ((unsigned long long)len > loc[C_MAXLEN]) loc[C_MAXLEN] = (unsigned long long)len;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0 && rows > 0) {
    if ((int64_t)rp[0] != 0 || (int64_t)rp[rows] != nnz) loc[C_BAD] = 1;
  }
#pragma unroll
  for (int c = 0; c < C_COUNT; ++c) {
    unsigned long long v = loc[c];
    for (int o = 16; o > 0; o >>= 1) {
      unsigned long long w = __shfl_xor_sync(0xffffffffu, v, o);
      v = (c == C_MAXLEN || c == C_BAD) ? (v > w ? v : w) : v + w;
    }
    if ((threadIdx.x & 31) == 0 && v) {
      if (c == C_MAXLEN || c == C_BAD) atomicMax(&ctr[c], v);
      else atomicAdd(&ctr[c], v);
    }
  }
}

__global__ void __launch_bounds__(256) col_check_kernel(const int32_t* __restrict__ col, int64_t nnz,
                                                        int64_t cols,
                                                        unsigned long long* __restrict__ bad) {
  bool b = false;
  for (int64_t k = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; k < nnz;
       k += (int64_t)gridDim.x * blockDim.x) {
    const int32_t c = col[k];
    b |= (c < 0 || (int64_t)c >= cols);
  }
  if (__any_sync(0xffffffffu, b) && (threadIdx.x & 31) == 0) atomicMax(bad, 1ull);
}

// How far the first column moves from one row to the next, summed over neighbouring non-empty rows
// (out[0]) with the number of such pairs (out[1]).  Small for banded matrices and stencils, where
// the rows of a tile gather neighbouring parts of x; about cols / 3 for uniformly random columns.
template <typename OffT>
__global__ void __launch_bounds__(256) col_step_kernel(const OffT* __restrict__ rp, const int32_t* __restrict__ col,
                                                       int64_t rows, unsigned long long* __restrict__ out) {
  unsigned long long sum = 0, cnt = 0;
  for (int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; r + 1 < rows; r += (int64_t)gridDim.x * blockDim.x) {
    const int64_t a = (int64_t)rp[r], b = (int64_t)rp[r + 1], c = (int64_t)rp[r + 2];
    if (b > a && c > b) {
      const int64_t d = (int64_t)col[b] - (int64_t)col[a];
      sum += (unsigned long long)(d < 0 ? -d : d);
      ++cnt;
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    sum += __shfl_xor_sync(0xffffffffu, sum, o);
    cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  }
  if ((threadIdx.x & 31) == 0 && cnt) {
    atomicAdd(&out[0], sum);
    atomicAdd(&out[1], cnt);
  }
}

template <typename OffT>
struct RowClassIs {
  const OffT* rp;
  int cls;
  __device__ bool operator()(int32_t r) const {
    const int64_t len = (int64_t)rp[r + 1] - (int64_t)rp[r];
    const int c = len <= kShortMax ? C_SHORT : (len <= kMediumMax ? C_MEDIUM : C_LONG);
    return c == cls;
  }
};

// Merge-path coordinate of diagonal d in the merge of row_end[0..rows) with the entry indices
// 0..nnz): the number of row ends consumed before the diagonal.  Same search as the
// reference's merge_path_search (alphasparse_spmv_csr_merge_ginkgo.h:11-35).
template <typename OffT>
__global__ void __launch_bounds__(256) merge_tile_kernel(const OffT* __restrict__ rp, int64_t rows,
                                                         int64_t nnz, int64_t tiles, int items,
                                                         int32_t* __restrict__ tile_row) {
  const int64_t t = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
  if (t > tiles) return;
  const OffT* row_end = rp + 1;
  int64_t diag = t * (int64_t)items;
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

template <typename OffT>
__global__ void __launch_bounds__(256) block_nnz_max_kernel(const OffT* __restrict__ rp, int64_t rows,
                                                            int64_t blocks,
                                                            unsigned long long* __restrict__ out) {
  unsigned long long m = 0;
  for (int64_t b = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; b < blocks;
       b += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r0 = b * kSpmmRowBlock;
    const int64_t r1 = r0 + kSpmmRowBlock < rows ? r0 + kSpmmRowBlock : rows;
    const unsigned long long n = (unsigned long long)((int64_t)rp[r1] - (int64_t)rp[r0]);
    if (n > m) m = n;
  }
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long w = __shfl_xor_sync(0xffffffffu, m, o);
    if (w > m) m = w;
  }
  if ((threadIdx.x & 31) == 0 && m) atomicMax(out, m);
}

template <typename OffT>
__global__ void partition_kernel(const OffT* __restrict__ rp, int64_t rows, int parts,
                                 int64_t* __restrict__ bounds) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i > parts) return;
  if (i == 0) {
    bounds[0] = 0;
    return;
  }
  if (i == parts || rows <= 0) {
    bounds[i] = rows > 0 ? rows : 0;
    return;
  }
  const OffT* row_end = rp + 1;
  const int64_t nnz = (int64_t)row_end[rows - 1];
  const int64_t v = (nnz / parts) * i;
  int64_t l = 0, r = rows - 1;
  while (r > l) {
    const int64_t m = (l + r) / 2;
    if ((int64_t)row_end[m] < v) l = m + 1;
    else r = m;
  }
  bounds[i] = l;
}

template <typename InT, typename OutT>
__global__ void __launch_bounds__(256) rebase_kernel(const InT* __restrict__ rp, int64_t row_begin,
                                                     int64_t n, OutT* __restrict__ out) {
  const int64_t base = (int64_t)rp[row_begin];
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    out[i] = (OutT)((int64_t)rp[row_begin + i] - base);
}

// Smallest and largest column index of a slice of col_idx: out[0] = min, out[1] = max
// (out starts as {INT64_MAX, -1}).
__global__ void __launch_bounds__(256) col_range_kernel(const int32_t* __restrict__ col, int64_t nnz,
                                                        long long* __restrict__ out) {
  int32_t lo = INT32_MAX, hi = -1;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nnz;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int32_t c = __ldg(col + i);
    lo = min(lo, c);
    hi = max(hi, c);
  }
  for (int o = 16; o > 0; o >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  if ((threadIdx.x & 31) == 0 && hi >= 0) {
    atomicMin(out, (long long)lo);
    atomicMax(out + 1, (long long)hi);
  }
}

// Transposition, after the entries were sorted by column (stable, so rows ascend inside a column):
// entry i of the transposed matrix is entry perm[i] of A; its column index there is the row of A that
// holds perm[i] (last row whose offset is <= perm[i]), its value a copy.
template <typename OffT, typename W>
__global__ void __launch_bounds__(256) transpose_fill_kernel(const OffT* __restrict__ rp, int64_t rows,
                                                             const uint32_t* __restrict__ perm, int64_t nnz,
                                                             const W* __restrict__ val, int32_t* __restrict__ t_col,
                                                             W* __restrict__ t_val) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < nnz; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t e = perm[i];
    int64_t lo = 0, hi = rows;  // first row whose end offset is > e
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if ((int64_t)rp[mid + 1] <= e) lo = mid + 1;
      else hi = mid;
    }
    t_col[i] = (int32_t)lo;
    t_val[i] = val[e];
  }
}
__global__ void __launch_bounds__(256) iota_kernel(uint32_t* __restrict__ out, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = (uint32_t)i;
}

// csrRowPtr[r] = number of COO entries whose (ascending) row index is below r.
template <typename OutT>
__global__ void __launch_bounds__(256) coo2csr_kernel(const int32_t* __restrict__ coo_row, int64_t nnz,
                                                      int64_t m, OutT* __restrict__ row_ptr) {
  for (int64_t r = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; r <= m;
       r += (int64_t)gridDim.x * blockDim.x) {
    int64_t lo = 0, hi = nnz;
    while (lo < hi) {
      const int64_t mid = lo + ((hi - lo) >> 1);
      if ((int64_t)coo_row[mid] < r) lo = mid + 1;
      else hi = mid;
    }
    row_ptr[r] = (OutT)lo;
  }
}

inline int grid_for(int64_t n, int sm_count) {
  int64_t g = (n + 255) / 256;
  const int64_t cap = (int64_t)sm_count * 8;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

template <typename OffT>
alphasparseStatus_t analyse_t(alphasparseHandle_t h, alphasparseSpMatDescr_t A, Plan* p) {
  cudaStream_t st = h->stream;
  const OffT* rp = reinterpret_cast<const OffT*>(A->row_offsets);
  const int sms = impl(h)->sm_count;
  unsigned long long* d_ctr = nullptr;
  ASP_CUDA(cudaMalloc(&d_ctr, sizeof(unsigned long long) * (C_COUNT + 1)));
  auto fail = [&](alphasparseStatus_t s) {
    cudaFree(d_ctr);
    return s;
  };
  if (cudaMemsetAsync(d_ctr, 0, sizeof(unsigned long long) * (C_COUNT + 1), st) != cudaSuccess)
    return fail(ALPHA_SPARSE_STATUS_INTERNAL_ERROR);
  unsigned long long ctr[C_COUNT + 1] = {0};
  if (p->rows > 0) {
    row_stats_kernel<OffT><<<grid_for(p->rows, sms), 256, 0, st>>>(rp, p->rows, p->nnz, d_ctr);
    impl(h)->launches++;
  }
  if (cudaMemcpyAsync(ctr, d_ctr, sizeof(unsigned long long) * C_COUNT, cudaMemcpyDeviceToHost,
                      st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess)
    return fail(status_of(cudaGetLastError()));
  if (ctr[C_BAD]) return fail(ALPHA_SPARSE_STATUS_INVALID_VALUE);
  // Column range check only after the offsets are known to be sane.
  if (p->nnz > 0) {
    col_check_kernel<<<grid_for(p->nnz, sms), 256, 0, st>>>(A->const_col_data, p->nnz, p->cols,
                                                            d_ctr + C_COUNT);
    impl(h)->launches++;
    if (cudaMemcpyAsync(&ctr[C_COUNT], d_ctr + C_COUNT, sizeof(unsigned long long),
                        cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess)
      return fail(status_of(cudaGetLastError()));
    if (ctr[C_COUNT]) return fail(ALPHA_SPARSE_STATUS_INVALID_VALUE);
  }
  // column locality of neighbouring rows (the offsets and columns were just validated)
  if (p->rows > 1 && p->nnz > 0) {
    unsigned long long step[2] = {0, 0};
    if (cudaMemsetAsync(d_ctr, 0, sizeof(unsigned long long) * 2, st) != cudaSuccess) return fail(ALPHA_SPARSE_STATUS_INTERNAL_ERROR);
    col_step_kernel<OffT><<<grid_for(p->rows, sms), 256, 0, st>>>(rp, A->const_col_data, p->rows, d_ctr);
    impl(h)->launches++;
    if (cudaMemcpyAsync(step, d_ctr, sizeof step, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
        cudaStreamSynchronize(st) != cudaSuccess)
      return fail(status_of(cudaGetLastError()));
    p->col_step = step[1] ? (double)step[0] / (double)step[1] : 0.0;
  }
  cudaFree(d_ctr);
  d_ctr = nullptr;

  p->n_short = (int64_t)ctr[C_SHORT];
  p->n_medium = (int64_t)ctr[C_MEDIUM];
  p->n_long = (int64_t)ctr[C_LONG];
  p->empty_rows = (int64_t)ctr[C_EMPTY];
  p->nnz_short = (int64_t)ctr[C_NNZ_SHORT];
  p->max_len = (int64_t)ctr[C_MAXLEN];
  p->identity_short = (p->n_short == p->rows);

  // Lanes per short row: enough 16-byte loads to cover the mean short row in one pass.
  {
    const int vec = 16 / (int)elem_size(A->data_type == ALPHA_R_16BF ? ALPHA_R_32F : A->data_type);
    const int64_t nonempty = p->n_short - p->empty_rows > 0 ? p->n_short - p->empty_rows : 1;
    const double mean = (double)p->nnz_short / (double)nonempty;
    int g = 2;
    while (g < 32 && g * vec < mean) g <<= 1;
    const int forced = env_int("ASP_GROUP_LANES", 0);
    if (forced == 2 || forced == 4 || forced == 8 || forced == 16 || forced == 32) g = forced;
    p->group_lanes = g;
  }

  // Per-class row lists, each in ascending row order.
  if (p->rows > 0 && !p->identity_short) {
    ASP_CUDA(cudaMalloc(&p->bin_rows, sizeof(int32_t) * p->rows));  // owned by the plan: freed with it on any failure
    int* d_num = nullptr;
    ASP_CUDA(cudaMalloc(&d_num, sizeof(int)));
    size_t tmp_bytes = 0;
    thrust::counting_iterator<int32_t> it(0);
    RowClassIs<OffT> pred{rp, C_SHORT};
    cub::DeviceSelect::If(nullptr, tmp_bytes, it, p->bin_rows, d_num, (int)p->rows, pred, st);
    void* tmp = nullptr;
    if (cudaMalloc(&tmp, tmp_bytes ? tmp_bytes : 16) != cudaSuccess) {
      cudaFree(d_num);
      return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    const int64_t off[3] = {0, p->n_short, p->n_short + p->n_medium};
    for (int c = 0; c < 3; ++c) {
      pred.cls = c;
      cub::DeviceSelect::If(tmp, tmp_bytes, it, p->bin_rows + off[c], d_num, (int)p->rows, pred, st);
      impl(h)->launches++;
    }
    cudaError_t e = cudaStreamSynchronize(st);
    cudaFree(tmp);
    cudaFree(d_num);
    if (e != cudaSuccess) return status_of(e);
  }

  // Merge-path tiles.
  p->merge_tiles = (p->rows + p->nnz + kMergeItems - 1) / kMergeItems;
  ASP_CUDA(cudaMalloc(&p->merge_tile_row, sizeof(int32_t) * (p->merge_tiles + 1)));
  ASP_CUDA(cudaMalloc(&p->carry, sizeof(double) * (p->merge_tiles > 0 ? p->merge_tiles : 1)));
  ASP_CUDA(cudaMalloc(&p->dev_err, sizeof(int)));
  ASP_CUDA(cudaMemsetAsync(p->dev_err, 0, sizeof(int), st));
  {
    int polls = env_int("ASP_WAIT_POLLS", 1 << 22);
    if (polls < 1) polls = 1;
    p->wait_cfg = (uint32_t)polls & kWaitPollMask;
    if (env_int("ASP_TEST_DROP_COPY", 0)) p->wait_cfg |= kWaitDropCopy;
    // A's bulk copies carry an L2 evict-first policy where the rows of a tile gather from all over x
    // (measured +2 % to +5 % on random and power-law columns: x keeps its place in L2), not where
    // neighbouring rows read neighbouring columns (measured -1 % on stencils).  ASP_TILE_L2_HINT forces it.
    const int hint = env_int("ASP_TILE_L2_HINT", -1);
    if (hint == 0 || (hint < 0 && p->col_step < 64.0)) p->wait_cfg |= kWaitNoL2Hint;
  }
  merge_tile_kernel<OffT><<<(int)((p->merge_tiles + 1 + 255) / 256), 256, 0, st>>>(
      rp, p->rows, p->nnz, p->merge_tiles, kMergeItems, p->merge_tile_row);
  impl(h)->launches++;
  ASP_CUDA(cudaGetLastError());
  ASP_CUDA(cudaStreamSynchronize(st));

  // Variant choice.  The merge-path tile kernel streams A through the copy engine and gives every
  // CTA the same number of items whatever the row lengths are; it wins on everything measured
  // except problems so small that they are bound by launch latency, where the binned kernel's
  // single launch (no carry fix-up kernel) is shorter.
  p->variant_auto = (p->merge_tiles < kSmallProblemTiles) ? kVariantBinned : kVariantMerge;

  // SpMM: the largest number of entries in an aligned block of kSpmmRowBlock rows decides whether
  // a block's entries fit the staging buffer of the TMA-fed SpMM kernel.
  {
    unsigned long long* d_max = nullptr;
    ASP_CUDA(cudaMalloc(&d_max, sizeof(unsigned long long)));
    ASP_CUDA(cudaMemsetAsync(d_max, 0, sizeof(unsigned long long), st));
    const int64_t blocks = (p->rows + kSpmmRowBlock - 1) / kSpmmRowBlock;
    if (blocks > 0) {
      block_nnz_max_kernel<OffT><<<grid_for(blocks, sms), 256, 0, st>>>(rp, p->rows, blocks, d_max);
      impl(h)->launches++;
    }
    unsigned long long m = 0;
    cudaError_t e = cudaMemcpyAsync(&m, d_max, sizeof m, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d_max);
    if (e != cudaSuccess) return status_of(e);
    p->max_block_nnz = (int64_t)m;
  }
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

}  // namespace

alphasparseStatus_t validate_csr(alphasparseSpMatDescr_t A) {
  if (!A || !A->init) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
  if (A->format != ALPHA_SPARSE_FORMAT_CSR) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (A->idx_base != ALPHA_SPARSE_INDEX_BASE_ZERO) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (A->col_type != ALPHA_SPARSE_INDEXTYPE_I32) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (A->row_type != ALPHA_SPARSE_INDEXTYPE_I32 && A->row_type != ALPHA_SPARSE_INDEXTYPE_I64)
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (!A->row_offsets) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

// The transposed matrix a plan may own: three device arrays, a descriptor over them, that
// descriptor's own plan.
struct Transposed {
  void* rp = nullptr;
  int32_t* col = nullptr;
  void* val = nullptr;
  _alphasparseSpMatDescr d{};
};

void free_transposed(void* q) {
  Transposed* t = reinterpret_cast<Transposed*>(q);
  if (!t) return;
  if (t->d.info) free_plan(plan_of(&t->d));
  cudaFree(t->rp);
  cudaFree(t->col);
  cudaFree(t->val);
  delete t;
}

void free_plan(Plan* p) {
  if (!p) return;
  cudaFree(p->bin_rows);
  cudaFree(p->merge_tile_row);
  cudaFree(p->carry);
  cudaFree(p->dev_err);
  cudaFree(p->spmm_carry);
  if (p->spmm_tc) free_spmm_tc_plan(p->spmm_tc);
  if (p->spmm_stage) free_spmm_stage_plan(p->spmm_stage);
  if (p->transposed) free_transposed(p->transposed);
  delete p;
}

// A^T in CSR, on the device (the reference's transpose_csr copies the matrix to the host, transposes
// it there and overwrites A's arrays, cuda/format/transpose_csr.h:9-78).  Stable radix sort of the
// entry numbers by column, row offsets of the result by one search per column, then a gather of
// rows and values.  A itself is left as it is; the copy of the values is as of this call.
alphasparseStatus_t transposed_of(alphasparseHandle_t h, alphasparseSpMatDescr_t A, alphasparseSpMatDescr_t* At) {
  if (!A->info) {
    alphasparseStatus_t s = analyse(h, A);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  }
  Plan* p = plan_of(A);
  if (p->device != h->device) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
  if (p->transposed) {
    *At = &reinterpret_cast<Transposed*>(p->transposed)->d;
    return ALPHA_SPARSE_STATUS_SUCCESS;
  }
  if (A->nnz >= (int64_t(1) << 31) || A->rows >= (int64_t(1) << 31) || A->cols >= (int64_t(1) << 31))
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  const size_t es = elem_size(A->data_type);
  if (es == 0) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  Transposed* t = new (std::nothrow) Transposed();
  if (!t) return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  cudaStream_t st = h->stream;
  const int64_t nnz = A->nnz, n1 = nnz > 0 ? nnz : 1;
  const bool o64 = A->row_type == ALPHA_SPARSE_INDEXTYPE_I64;
  int32_t* keys = nullptr;
  uint32_t *ent = nullptr, *perm = nullptr;
  void* tmp = nullptr;
  size_t tmp_bytes = 0;
  int bits = 1;
  while ((int64_t(1) << bits) < A->cols && bits < 31) ++bits;
  cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, (const int32_t*)nullptr, (int32_t*)nullptr, (const uint32_t*)nullptr,
                                  (uint32_t*)nullptr, (int)nnz, 0, bits, st);
  cudaError_t e = cudaMalloc(&t->rp, (size_t)(A->cols + 1) * (o64 ? 8 : 4));
  if (e == cudaSuccess) e = cudaMalloc(&t->col, (size_t)n1 * 4);
  if (e == cudaSuccess) e = cudaMalloc(&t->val, (size_t)n1 * es);
  if (e == cudaSuccess) e = cudaMalloc(&keys, (size_t)n1 * 4);
  if (e == cudaSuccess) e = cudaMalloc(&ent, (size_t)n1 * 4);
  if (e == cudaSuccess) e = cudaMalloc(&perm, (size_t)n1 * 4);
  if (e == cudaSuccess) e = cudaMalloc(&tmp, tmp_bytes ? tmp_bytes : 16);
  alphasparseStatus_t s = status_of(e);
  if (s == ALPHA_SPARSE_STATUS_SUCCESS && nnz > 0) {
    const int g = grid_for(nnz, impl(h)->sm_count);
    iota_kernel<<<g, 256, 0, st>>>(ent, nnz);
    // keys: column of every entry, sorted into t->col for the moment (it is overwritten by the rows below
    // only after the offsets were derived from it)
    cub::DeviceRadixSort::SortPairs(tmp, tmp_bytes, A->const_col_data, keys, ent, perm, (int)nnz, 0, bits, st);
    if (o64) coo2csr_kernel<int64_t><<<grid_for(A->cols + 1, impl(h)->sm_count), 256, 0, st>>>(keys, nnz, A->cols, (int64_t*)t->rp);
    else coo2csr_kernel<int32_t><<<grid_for(A->cols + 1, impl(h)->sm_count), 256, 0, st>>>(keys, nnz, A->cols, (int32_t*)t->rp);
#define ASP_FILL(OFF, W)                                                                                         \
  transpose_fill_kernel<OFF, W><<<g, 256, 0, st>>>((const OFF*)A->row_offsets, A->rows, perm, nnz,                \
                                                  (const W*)A->const_val_data, t->col, (W*)t->val)
    if (o64) {
      if (es == 1) ASP_FILL(int64_t, uint8_t);
      else if (es == 2) ASP_FILL(int64_t, uint16_t);
      else if (es == 4) ASP_FILL(int64_t, uint32_t);
      else if (es == 16) ASP_FILL(int64_t, uint4);
      else ASP_FILL(int64_t, uint64_t);
    } else {
      if (es == 1) ASP_FILL(int32_t, uint8_t);
      else if (es == 2) ASP_FILL(int32_t, uint16_t);
      else if (es == 4) ASP_FILL(int32_t, uint32_t);
      else if (es == 16) ASP_FILL(int32_t, uint4);
      else ASP_FILL(int32_t, uint64_t);
    }
#undef ASP_FILL
    impl(h)->launches += 4;
    s = status_of(cudaGetLastError());
  } else if (s == ALPHA_SPARSE_STATUS_SUCCESS) {
    s = status_of(cudaMemsetAsync(t->rp, 0, (size_t)(A->cols + 1) * (o64 ? 8 : 4), st));
  }
  if (s == ALPHA_SPARSE_STATUS_SUCCESS) s = status_of(cudaStreamSynchronize(st));
  cudaFree(keys);
  cudaFree(ent);
  cudaFree(perm);
  cudaFree(tmp);
  if (s == ALPHA_SPARSE_STATUS_SUCCESS) {
    t->d = *A;
    t->d.rows = A->cols;
    t->d.cols = A->rows;
    t->d.info = nullptr;
    t->d.analysed = false;
    t->d.row_offsets = t->rp;
    t->d.row_data = o64 ? nullptr : reinterpret_cast<int*>(t->rp);
    t->d.const_row_data = t->d.row_data;
    t->d.col_data = t->col;
    t->d.const_col_data = t->col;
    t->d.val_data = t->val;
    t->d.const_val_data = t->val;
    s = analyse(h, &t->d);
  }
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) {
    free_transposed(t);
    return s;
  }
  p->transposed = t;
  *At = &t->d;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t analyse(alphasparseHandle_t h, alphasparseSpMatDescr_t A) {
  alphasparseStatus_t s = validate_csr(A);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  if (A->info) {
    free_plan(plan_of(A));
    A->info = nullptr;
    A->analysed = false;
  }
  Plan* p = new (std::nothrow) Plan();
  if (!p) return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  p->device = h->device;
  p->rows = A->rows;
  p->cols = A->cols;
  p->nnz = A->nnz;
  p->off64 = (A->row_type == ALPHA_SPARSE_INDEXTYPE_I64);
  s = p->off64 ? analyse_t<int64_t>(h, A, p) : analyse_t<int32_t>(h, A, p);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) {
    free_plan(p);
    return s;
  }
  A->info = p;
  A->analysed = true;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

}  // namespace asp

using namespace asp;

extern "C" {

alphasparseStatus_t alphasparseSpMV_analysis(alphasparseHandle_t h, alphasparseOperation_t opA,
                                             alphasparseSpMatDescr_t A, alphasparseSpMVAlg_t) {
  if (!h || !h->impl) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!A) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  alphasparseStatus_t s = analyse(h, A);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS || opA == ALPHA_SPARSE_OPERATION_NON_TRANSPOSE) return s;
  alphasparseSpMatDescr_t At = nullptr;  // a transposed product will follow: build and analyse A^T now
  return transposed_of(h, A, &At);
}

alphasparseStatus_t alphasparseSpMV_clear(alphasparseHandle_t h, alphasparseSpMVAlg_t) {
  return h ? ALPHA_SPARSE_STATUS_SUCCESS : ALPHA_SPARSE_STATUS_INVALID_HANDLE;
}

alphasparseStatus_t alphasparseSpMV_clearMat(alphasparseHandle_t h, alphasparseSpMatDescr_t A) {
  if (!h) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!A) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (A->info) {
    cudaStreamSynchronize(h->stream);
    free_plan(plan_of(A));
    A->info = nullptr;
  }
  A->analysed = false;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseCsrPlanGet(alphasparseHandle_t h, alphasparseSpMatDescr_t A,
                                          int64_t* stats, int32_t* bin_rows,
                                          int32_t* merge_tile_row) {
  if (!h) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!A) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  Plan* p = plan_of(A);
  if (!p) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
  ASP_CUDA(cudaStreamSynchronize(h->stream));
  if (stats) {
    for (int i = 0; i < ASP_STAT_COUNT; ++i) stats[i] = 0;
    stats[ASP_STAT_MAX_LEN] = p->max_len;
    stats[ASP_STAT_EMPTY_ROWS] = p->empty_rows;
    stats[ASP_STAT_NUM_SHORT] = p->n_short;
    stats[ASP_STAT_NUM_MEDIUM] = p->n_medium;
    stats[ASP_STAT_NUM_LONG] = p->n_long;
    stats[ASP_STAT_GROUP_LANES] = p->group_lanes;
    stats[ASP_STAT_MERGE_ITEMS] = kMergeItems;
    stats[ASP_STAT_MERGE_TILES] = p->merge_tiles;
    stats[ASP_STAT_VARIANT] = p->variant_auto;
    stats[ASP_STAT_IDENTITY_SHORT] = p->identity_short ? 1 : 0;
    stats[ASP_STAT_NNZ_SHORT] = p->nnz_short;
    stats[ASP_STAT_COL_STEP] = (int64_t)(p->col_step + 0.5);
    int e = 0;
    if (p->dev_err) ASP_CUDA(cudaMemcpy(&e, p->dev_err, sizeof(int), cudaMemcpyDeviceToHost));
    stats[ASP_STAT_DEVICE_ERROR] = e;
  }
  if (bin_rows && p->rows > 0) {
    if (p->identity_short) {
      for (int64_t i = 0; i < p->rows; ++i) bin_rows[i] = (int32_t)i;
    } else {
      ASP_CUDA(cudaMemcpy(bin_rows, p->bin_rows, sizeof(int32_t) * p->rows, cudaMemcpyDeviceToHost));
    }
  }
  if (merge_tile_row)
    ASP_CUDA(cudaMemcpy(merge_tile_row, p->merge_tile_row, sizeof(int32_t) * (p->merge_tiles + 1),
                        cudaMemcpyDeviceToHost));
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

const char* alphasparseCsrLastVariant(alphasparseSpMatDescr_t A) {
  if (!A || !A->info) return "none";
  switch (plan_of(A)->last_variant) {
    case kVariantBinned: return "binned";
    case kVariantMerge: return "merge";
    default: return "none";
  }
}

const char* alphasparseCsrLastSpmmVariant(alphasparseSpMatDescr_t A) {
  return (A && A->info) ? plan_of(A)->last_spmm : "none";
}

alphasparseStatus_t alphasparseCsrPartitionRowsByNnz(alphasparseHandle_t h, int64_t rows,
                                                     const void* row_offsets,
                                                     alphasparseIndexType_t rowT, int parts,
                                                     int64_t* bounds) {
  if (!h || !h->impl) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!row_offsets || !bounds) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (rows < 0 || parts < 1 || parts > 4096) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (rowT != ALPHA_SPARSE_INDEXTYPE_I32 && rowT != ALPHA_SPARSE_INDEXTYPE_I64)
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  // the handle's 1 MB scratch buffer holds the bounds of up to 4096 parts: no allocation per call
  int64_t* d = reinterpret_cast<int64_t*>(h->buffer);
  if (!d || h->buffer_size < sizeof(int64_t) * (size_t)(parts + 1)) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
  const int g = (parts + 1 + 127) / 128;
  if (rowT == ALPHA_SPARSE_INDEXTYPE_I32)
    partition_kernel<int32_t><<<g, 128, 0, h->stream>>>((const int32_t*)row_offsets, rows, parts, d);
  else
    partition_kernel<int64_t><<<g, 128, 0, h->stream>>>((const int64_t*)row_offsets, rows, parts, d);
  impl(h)->launches++;
  cudaError_t e = cudaMemcpyAsync(bounds, d, sizeof(int64_t) * (parts + 1), cudaMemcpyDeviceToHost,
                                  h->stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
  return status_of(e);
}

alphasparseStatus_t alphasparseCsrRebaseRowOffsets(alphasparseHandle_t h, const void* row_offsets,
                                                   alphasparseIndexType_t inT, int64_t row_begin,
                                                   int64_t row_end, void* local,
                                                   alphasparseIndexType_t outT) {
  if (!h || !h->impl) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!row_offsets || !local) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (row_begin < 0 || row_end < row_begin) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  const int64_t n = row_end - row_begin + 1;
  const int g = grid_for(n, impl(h)->sm_count);
  const bool i64 = inT == ALPHA_SPARSE_INDEXTYPE_I64, o64 = outT == ALPHA_SPARSE_INDEXTYPE_I64;
  if ((!i64 && inT != ALPHA_SPARSE_INDEXTYPE_I32) || (!o64 && outT != ALPHA_SPARSE_INDEXTYPE_I32))
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  cudaStream_t st = h->stream;
  if (i64 && o64) rebase_kernel<<<g, 256, 0, st>>>((const int64_t*)row_offsets, row_begin, n, (int64_t*)local);
  else if (i64) rebase_kernel<<<g, 256, 0, st>>>((const int64_t*)row_offsets, row_begin, n, (int32_t*)local);
  else if (o64) rebase_kernel<<<g, 256, 0, st>>>((const int32_t*)row_offsets, row_begin, n, (int64_t*)local);
  else rebase_kernel<<<g, 256, 0, st>>>((const int32_t*)row_offsets, row_begin, n, (int32_t*)local);
  impl(h)->launches++;
  return status_of(cudaGetLastError());
}

alphasparseStatus_t alphasparseCsrColumnRange(alphasparseHandle_t h, int64_t nnz, const void* col_idx,
                                              alphasparseIndexType_t colT, int64_t* min_col,
                                              int64_t* max_col) {
  if (!h || !h->impl) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!min_col || !max_col || (nnz > 0 && !col_idx)) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (nnz < 0) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (colT != ALPHA_SPARSE_INDEXTYPE_I32) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  *min_col = 0;
  *max_col = -1;
  if (nnz == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  long long* d = nullptr;
  ASP_CUDA(cudaMalloc(&d, 2 * sizeof(long long)));
  const long long init[2] = {INT64_MAX, -1};
  cudaError_t e = cudaMemcpyAsync(d, init, sizeof(init), cudaMemcpyHostToDevice, h->stream);
  long long out[2] = {0, -1};
  if (e == cudaSuccess) {
    col_range_kernel<<<grid_for(nnz, impl(h)->sm_count), 256, 0, h->stream>>>((const int32_t*)col_idx, nnz, d);
    impl(h)->launches++;
    e = cudaMemcpyAsync(out, d, sizeof(out), cudaMemcpyDeviceToHost, h->stream);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
  cudaFree(d);
  if (e == cudaSuccess) {
    *min_col = out[0];
    *max_col = out[1];
  }
  return status_of(e);
}

}  // extern "C"

// The step before the path: CSR row offsets from the ascending row indices of a COO matrix.
// Replaces cuda/format/coo2csr.h:82-92 of the reference (zero + atomicAdd histogram + thrust scan
// on the default stream, with a printf) by one stream-ordered kernel: row r's offset is the
// position of the first entry whose row index is >= r.
extern "C" alphasparseStatus_t alphasparseXcoo2csr(cudaStream_t stream, const int32_t* cooRowInd,
                                                   int64_t nnz, int64_t m, void* csrRowPtr,
                                                   alphasparseIndexType_t rowOffsetsType) {
  if (!csrRowPtr || (nnz > 0 && !cooRowInd)) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (nnz < 0 || m < 0) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  const bool o64 = rowOffsetsType == ALPHA_SPARSE_INDEXTYPE_I64;
  if (!o64 && rowOffsetsType != ALPHA_SPARSE_INDEXTYPE_I32) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (!o64 && nnz >= (int64_t(1) << 31)) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  int dev = 0, sms = 0;  // no handle on this entry point: ask the device the stream's work will run on
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1)
    return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
  int64_t g = (m + 1 + 255) / 256;
  if (g > (int64_t)sms * 16) g = (int64_t)sms * 16;
  if (o64) asp::coo2csr_kernel<int64_t><<<(unsigned)g, 256, 0, stream>>>(cooRowInd, nnz, m, (int64_t*)csrRowPtr);
  else asp::coo2csr_kernel<int32_t><<<(unsigned)g, 256, 0, stream>>>(cooRowInd, nnz, m, (int32_t*)csrRowPtr);
  return asp::status_of(cudaGetLastError());
}
