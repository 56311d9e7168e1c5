// CSR SpMM  C = alpha*A*B + beta*C  (fp32 / fp64, row-major B and C) with the dense operand staged
// through shared memory by the copy engine - for matrices whose row blocks touch B in runs
// (stencils, banded matrices): a block then needs far fewer distinct rows of B than it has entries.
//
// The reference's closest kernel is its row-balanced one (cuda/kernel/level3/
// alphasparse_spmm_csr.h:109-198): a warp per row, A's entries of the row through shared memory,
// every B row segment fetched from global memory once per entry.  Here:
//   * preprocessing (device, once per matrix): for every block of kStageRows rows, the ascending
//     list of kStageChunk-column chunks of A that hold at least one of its entries (a bitmap per
//     block, a scan, a fill);
//   * a CTA owns one row block and one slab of W = LN*VN columns of C.  A producer warp walks the
//     chunk list and asks the copy engine for the matching kStageChunk x W box of B per chunk
//     (cp.async.bulk.tensor.2d, completion counted on an mbarrier) into a ring of stages; no load
//     here uses cluster multicast;
//   * the consumer warps hold the block's accumulators in registers (LN lanes per row, VN adjacent
//     columns per lane, eight rows per lane group).  Per chunk a group advances a cursor through
//     each of its rows while the entry's column lies inside the chunk: (column, alpha*value) comes
//     from shared memory as one 8- or 16-byte word, the row of B from the staged box as one 16-byte
//     word.  Rows are sorted by column, so every C element is accumulated in entry order with
//     fma(alpha*a, b, c) starting from beta*c - the order and the arithmetic of the reference's CPU
//     kernel (hygon/kernel/level3/mm/gemm/gemm_csr_row.hpp:33-56): results equal it bit for bit;
//   * a warp releases a stage through a second mbarrier; the producer re-fills it when all have.
//     Every wait is bounded; on expiry the CTA raises *err and leaves.
#include <cuda.h>
#include <cub/device/device_reduce.cuh>
#include <cub/device/device_scan.cuh>

#include <climits>
#include <new>

#include "asp_internal.h"

namespace asp {
namespace {

#ifndef ASP_STAGE_ROWS
#define ASP_STAGE_ROWS 256
#endif
#ifndef ASP_STAGE_CHUNK
#define ASP_STAGE_CHUNK 64
#endif
constexpr int kStageRows = ASP_STAGE_ROWS;    // rows of A (and C) per CTA
constexpr int kStageChunk = ASP_STAGE_CHUNK;  // columns of A = rows of B per staged box
constexpr int kStageRpg = 8;                  // rows per lane group
constexpr int kStageGroups = kStageRows / kStageRpg;
// entries of a row block staged in shared memory: 64 KB of (column, value) words
template <typename T> constexpr int stage_cap() { return sizeof(T) == 4 ? kStageRows * 32 : kStageRows * 16; }
constexpr int kStageMaxChunks = 1024;         // chunk ids of a row block staged in shared memory
constexpr int kSpanWords = 2048;              // bitmap words of the plan builder: a block may span 65,536 chunks
constexpr uint32_t kMaxTries = 1u << 22;

struct StagePlan {
  int64_t blocks = 0, total_chunks = 0;
  int max_chunks = 0;
  bool usable = false;           // columns ascend inside every row, chunk span within the bitmap
  int32_t* off = nullptr;        // device, blocks + 1
  int32_t* cnt = nullptr;        // device, blocks
  int32_t* list = nullptr;       // device, off[blocks] chunk ids
};

// ---- preprocessing -------------------------------------------------------------------------
// One CTA per row block.  FILL = false: counts[b] = number of non-empty chunks; flags[0] |= 1 if the
// block spans more chunks than the bitmap, flags[1] |= 1 if a row's columns are not ascending.
// FILL = true: writes the chunk ids, ascending, at off[b].
template <bool FILL>
__global__ void __launch_bounds__(256) stage_chunks_kernel(const int32_t* __restrict__ rp, const int32_t* __restrict__ col,
                                                           int64_t rows, int32_t* __restrict__ counts,
                                                           const int32_t* __restrict__ off, int32_t* __restrict__ list,
                                                           int* __restrict__ flags) {
  __shared__ unsigned bm[kSpanWords];
  __shared__ int s_min;
  __shared__ int s_scan[256];
  const int tid = threadIdx.x;
  const int64_t r0 = (int64_t)blockIdx.x * kStageRows;
  const int64_t r1 = r0 + kStageRows < rows ? r0 + kStageRows : rows;
  const int e0 = rp[r0], e1 = rp[r1];
  for (int i = tid; i < kSpanWords; i += 256) bm[i] = 0u;
  if (tid == 0) s_min = INT_MAX;
  __syncthreads();
  int mn = INT_MAX;
  for (int k = e0 + tid; k < e1; k += 256) mn = min(mn, col[k]);
  for (int o = 16; o > 0; o >>= 1) mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  if ((tid & 31) == 0 && mn != INT_MAX) atomicMin(&s_min, mn);
  __syncthreads();
  const int base = s_min == INT_MAX ? 0 : s_min / kStageChunk;
  bool over = false;
  for (int k = e0 + tid; k < e1; k += 256) {
    const int c = col[k] / kStageChunk - base;
    if (c >= kSpanWords * 32) over = true;
    else atomicOr(&bm[c >> 5], 1u << (c & 31));
  }
  if (!FILL) {
    bool unsorted = false;
    for (int64_t r = r0 + tid; r < r1; r += 256)
      for (int k = rp[r] + 1; k < rp[r + 1]; ++k) unsorted |= col[k] < col[k - 1];
    if (over) atomicOr(&flags[0], 1);
    if (unsorted) atomicOr(&flags[1], 1);
  }
  __syncthreads();
  constexpr int WPT = kSpanWords / 256;
  int cnt = 0;
#pragma unroll
  for (int w = 0; w < WPT; ++w) cnt += __popc(bm[tid * WPT + w]);
  s_scan[tid] = cnt;
  __syncthreads();
  for (int o = 1; o < 256; o <<= 1) {
    const int v = tid >= o ? s_scan[tid - o] : 0;
    __syncthreads();
    s_scan[tid] += v;
    __syncthreads();
  }
  if (!FILL) {
    if (tid == 255) counts[blockIdx.x] = s_scan[255];
  } else {
    int pos = off[blockIdx.x] + s_scan[tid] - cnt;
    for (int w = 0; w < WPT; ++w) {
      unsigned bits = bm[tid * WPT + w];
      while (bits) {
        const int b = __ffs(bits) - 1;
        bits &= bits - 1;
        list[pos++] = base + (tid * WPT + w) * 32 + b;
      }
    }
  }
}

alphasparseStatus_t build_stage_plan(alphasparseHandle_t h, alphasparseSpMatDescr_t A, StagePlan* sp) {
  cudaStream_t st = h->stream;
  sp->blocks = (A->rows + kStageRows - 1) / kStageRows;
  if (sp->blocks == 0 || sp->blocks >= INT_MAX) return ALPHA_SPARSE_STATUS_SUCCESS;
  const int nb = (int)sp->blocks;
  int* flags = nullptr;
  void* tmp = nullptr;
  int32_t* d_max = nullptr;
  auto cleanup = [&]() {
    cudaFree(flags);
    cudaFree(tmp);
    cudaFree(d_max);
  };
  size_t scan_bytes = 0, max_bytes = 0;
  cub::DeviceScan::ExclusiveSum(nullptr, scan_bytes, sp->cnt, sp->off, nb + 1, st);
  cub::DeviceReduce::Max(nullptr, max_bytes, sp->cnt, d_max, nb, st);
  const size_t tmp_bytes = (scan_bytes > max_bytes ? scan_bytes : max_bytes) + 16;
  if (cudaMalloc(&sp->cnt, sizeof(int32_t) * (nb + 1)) != cudaSuccess ||
      cudaMalloc(&sp->off, sizeof(int32_t) * (nb + 1)) != cudaSuccess ||
      cudaMalloc(&flags, 2 * sizeof(int)) != cudaSuccess || cudaMalloc(&tmp, tmp_bytes) != cudaSuccess ||
      cudaMalloc(&d_max, sizeof(int32_t)) != cudaSuccess) {
    cleanup();
    return ALPHA_SPARSE_STATUS_ALLOC_FAILED;  // sp's arrays are freed with sp by the caller
  }
  cudaMemsetAsync(flags, 0, 2 * sizeof(int), st);
  cudaMemsetAsync(sp->cnt, 0, sizeof(int32_t) * (nb + 1), st);
  stage_chunks_kernel<false><<<(unsigned)nb, 256, 0, st>>>(A->const_row_data, A->const_col_data, A->rows, sp->cnt, nullptr,
                                                          nullptr, flags);
  size_t b = scan_bytes;
  cub::DeviceScan::ExclusiveSum(tmp, b, sp->cnt, sp->off, nb + 1, st);
  b = max_bytes;
  cub::DeviceReduce::Max(tmp, b, sp->cnt, d_max, nb, st);
  impl(h)->launches += 3;
  int hflags[2] = {0, 0};
  int32_t total = 0, mx = 0;
  cudaError_t e = cudaMemcpyAsync(hflags, flags, sizeof hflags, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaMemcpyAsync(&total, sp->off + nb, sizeof total, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaMemcpyAsync(&mx, d_max, sizeof mx, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    cleanup();
    return status_of(e);
  }
  sp->total_chunks = total;
  sp->max_chunks = mx;
  sp->usable = hflags[0] == 0 && hflags[1] == 0;
  if (sp->usable && total > 0) {
    if (cudaMalloc(&sp->list, sizeof(int32_t) * (size_t)total) != cudaSuccess) {
      cleanup();
      return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    stage_chunks_kernel<true><<<(unsigned)nb, 256, 0, st>>>(A->const_row_data, A->const_col_data, A->rows, nullptr, sp->off,
                                                           sp->list, nullptr);
    impl(h)->launches++;
    e = cudaStreamSynchronize(st);
  }
  cleanup();
  return status_of(e);
}

// ---- the kernel ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  uint32_t tries = 0;
  while (!mbar_try_wait(bar, parity))
    if (++tries > kMaxTries) return false;
  return true;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

template <typename T> struct Entry;  // (column, alpha * value) as one shared-memory word
template <> struct __align__(8) Entry<float> { int c; float v; };
template <> struct __align__(16) Entry<double> { int c; int pad; double v; };

template <typename T, int LN> struct StageGeom {
  static constexpr int VN = 16 / (int)sizeof(T);
  static constexpr int W = LN * VN;                          // columns of C per CTA
  static constexpr int CONSUMERS = kStageGroups * LN;        // consumer threads
  static constexpr int THREADS = CONSUMERS + 32;             // + the producer warp
  static constexpr int BOX_BYTES = kStageChunk * W * (int)sizeof(T);
  static constexpr int CAP = stage_cap<T>();
  static constexpr int FIXED = 128 /* alignment slack */ + CAP * (int)sizeof(Entry<T>) + (kStageRows + 1) * (int)sizeof(int) +
                               kStageMaxChunks * (int)sizeof(int);
  // two CTAs per SM when the ring can still be four boxes deep, else one CTA with all the memory
  static constexpr int BUDGET2 = 113 * 1024, BUDGET1 = 226 * 1024;
  static constexpr int S2 = (BUDGET2 - FIXED) / (BOX_BYTES + 16);
  static constexpr int S1 = (BUDGET1 - FIXED) / (BOX_BYTES + 16);
  static constexpr int STAGES = S2 >= 4 ? (S2 > 12 ? 12 : S2) : (S1 > 12 ? 12 : S1);
  static constexpr size_t SMEM = (size_t)FIXED + (size_t)STAGES * (BOX_BYTES + 16);
  static_assert(STAGES >= 2, "the ring needs at least two boxes");
  static_assert(CONSUMERS % 32 == 0 && THREADS <= 1024, "whole warps, one CTA");
};

template <typename T, int LN>
__global__ void __launch_bounds__(StageGeom<T, LN>::THREADS)
spmm_stage_kernel(const __grid_constant__ CUtensorMap tmB, const int32_t* __restrict__ rp, const int* __restrict__ col,
                  const T* __restrict__ val, const int32_t* __restrict__ chunk_off, const int32_t* __restrict__ chunk_cnt,
                  const int32_t* __restrict__ chunk_list, T* __restrict__ C, int64_t ldc, T alpha, T beta, int64_t rows,
                  int64_t n, int slabs, int* __restrict__ err) {
  using Gm = StageGeom<T, LN>;
  constexpr int VN = Gm::VN, W = Gm::W, NG = kStageGroups, RPG = kStageRpg, S = Gm::STAGES;
  constexpr int NT = Gm::THREADS, NC = Gm::CONSUMERS;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~(uintptr_t)127);
  // widest alignment first: boxes (128 bytes), mbarriers (8), entries (8 or 16), then the 4-byte arrays
  T* s_box = reinterpret_cast<T*>(base);
  uint64_t* s_full = reinterpret_cast<uint64_t*>(base + (size_t)S * Gm::BOX_BYTES);
  uint64_t* s_empty = s_full + S;
  Entry<T>* s_ent = reinterpret_cast<Entry<T>*>(s_empty + S);  // 16 * S bytes behind the boxes: 16-byte aligned
  int* s_rp = reinterpret_cast<int*>(s_ent + Gm::CAP);
  int* s_chunk = s_rp + kStageRows + 1;

  const int tid = threadIdx.x;
  const int64_t blk = blockIdx.x / slabs;  // the slabs of a row block are neighbours in launch order: they share A in L2
  const int slab_c0 = (int)(blockIdx.x % slabs) * W;
  const int64_t r0 = blk * kStageRows;
  const int nr = (int)(r0 + kStageRows < rows ? kStageRows : rows - r0);
  const int e0 = rp[r0], e1 = rp[r0 + nr];
  const int nch = chunk_cnt[blk];
  const int coff = chunk_off[blk];

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], NC / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < nch; i += NT) s_chunk[i] = chunk_list[coff + i];
  __syncthreads();

  if (tid >= NC) {
    // ---- producer warp: one lane feeds the ring (it starts before the entries are staged) ----
    if (tid == NC) {
      for (int ci = 0; ci < nch; ++ci) {
        const int s = ci % S, it = ci / S;
        if (it > 0 && !mbar_wait(&s_empty[s], (uint32_t)(it - 1) & 1u)) {
          atomicExch(err, 1);
          break;
        }
        mbar_expect_tx(&s_full[s], (uint32_t)Gm::BOX_BYTES);
        tma_load_2d(reinterpret_cast<unsigned char*>(s_box) + (size_t)s * Gm::BOX_BYTES, &tmB, slab_c0,
                    s_chunk[ci] * kStageChunk, &s_full[s]);
      }
    }
    return;
  }

  // ---- consumer warps ----
  for (int i = tid; i <= nr; i += NC) s_rp[i] = rp[r0 + i] - e0;
  for (int i = tid; i < e1 - e0; i += NC) {
    Entry<T> en;
    en.c = __ldcs(col + e0 + i);
    en.v = alpha * __ldcs(val + e0 + i);
    s_ent[i] = en;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(NC) : "memory");  // the consumers only: the producer is already at work

  const int lane = tid % LN, grp = tid / LN;
  const int64_t c0 = (int64_t)slab_c0 + lane * VN;
  const bool col_ok = c0 < n;
  int k[RPG], e[RPG];
  Entry<T> cur[RPG];
  T acc[RPG][VN];
#pragma unroll
  for (int i = 0; i < RPG; ++i) {
    const int lr = grp + i * NG;  // neighbouring groups take neighbouring rows
    k[i] = lr < nr ? s_rp[lr] : 0;
    e[i] = lr < nr ? s_rp[lr + 1] : 0;
    cur[i].c = INT_MAX;
    cur[i].v = T(0);
    if (k[i] < e[i]) cur[i] = s_ent[k[i]];
#pragma unroll
    for (int v = 0; v < VN; ++v) acc[i][v] = T(0);
    if (beta != T(0) && lr < nr && col_ok) {
      const T* cp = C + (r0 + lr) * ldc + c0;
      if constexpr (VN == 4) {
        const float4 o = *reinterpret_cast<const float4*>(cp);
        acc[i][0] = o.x * beta; acc[i][1] = o.y * beta; acc[i][2] = o.z * beta; acc[i][3] = o.w * beta;
      } else {
        const double2 o = *reinterpret_cast<const double2*>(cp);
        acc[i][0] = o.x * beta; acc[i][1] = o.y * beta;
      }
    }
  }
  bool failed = false;
  for (int ci = 0; ci < nch; ++ci) {
    const int s = ci % S;
    if (!mbar_wait(&s_full[s], (uint32_t)(ci / S) & 1u)) {
      failed = true;
      break;
    }
    const int cbase = s_chunk[ci] * kStageChunk;
    const int lim = cbase + kStageChunk;
    const T* box = s_box + (size_t)s * (kStageChunk * W) + lane * VN;
    bool more = true;
    while (more) {
      more = false;
#pragma unroll
      for (int i = 0; i < RPG; ++i) {
        if (cur[i].c < lim) {
          const T a = cur[i].v;
          const T* bp = box + (cur[i].c - cbase) * W;
          if constexpr (VN == 4) {
            const float4 b = *reinterpret_cast<const float4*>(bp);
            acc[i][0] = fma(a, b.x, acc[i][0]); acc[i][1] = fma(a, b.y, acc[i][1]);
            acc[i][2] = fma(a, b.z, acc[i][2]); acc[i][3] = fma(a, b.w, acc[i][3]);
          } else {
            const double2 b = *reinterpret_cast<const double2*>(bp);
            acc[i][0] = fma(a, b.x, acc[i][0]); acc[i][1] = fma(a, b.y, acc[i][1]);
          }
          ++k[i];
          cur[i].c = INT_MAX;
          if (k[i] < e[i]) cur[i] = s_ent[k[i]];
          more = true;
        }
      }
    }
    __syncwarp();
    if ((tid & 31) == 0) mbar_arrive(&s_empty[s]);
  }
  if (failed) {
    if ((tid & 31) == 0) atomicExch(err, 1);
    __nanosleep(1000000);  // let a copy still in flight land before the CTA's memory is released
    return;
  }
  if (!col_ok) return;
#pragma unroll
  for (int i = 0; i < RPG; ++i) {
    const int lr = grp + i * NG;
    if (lr >= nr) continue;
    T* cp = C + (r0 + lr) * ldc + c0;
    if constexpr (VN == 4) *reinterpret_cast<float4*>(cp) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
    else *reinterpret_cast<double2*>(cp) = make_double2(acc[i][0], acc[i][1]);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

template <typename T, int LN>
alphasparseStatus_t launch_stage(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const StagePlan* sp, const T* B, int64_t ldb,
                                 T* C, int64_t ldc, T alpha, T beta, int64_t n) {
  using Gm = StageGeom<T, LN>;
  EncodeTiledFn enc = encode_fn();
  if (!enc) return ALPHA_SPARSE_STATUS_INTERNAL_ERROR;
  alignas(64) CUtensorMap tm;
  const cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)A->cols};
  const cuuint64_t strides[1] = {(cuuint64_t)ldb * sizeof(T)};
  const cuuint32_t box[2] = {(cuuint32_t)Gm::W, (cuuint32_t)kStageChunk};
  const cuuint32_t estr[2] = {1, 1};
  if (enc(&tm, sizeof(T) == 8 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT64 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<T*>(B), dims,
          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return ALPHA_SPARSE_STATUS_INVALID_VALUE;
  const int64_t slabs = (n + Gm::W - 1) / Gm::W;
  if (sp->blocks * slabs > INT_MAX) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  static size_t attr_set[64] = {0};  // the attribute belongs to the device: remembered per device
  size_t& set = attr_set[h->device & 63];
  if (Gm::SMEM > set) {
    ASP_CUDA(cudaFuncSetAttribute(spmm_stage_kernel<T, LN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Gm::SMEM));
    set = Gm::SMEM;
  }
  spmm_stage_kernel<T, LN><<<(unsigned)(sp->blocks * slabs), Gm::THREADS, Gm::SMEM, h->stream>>>(
      tm, A->const_row_data, A->const_col_data, reinterpret_cast<const T*>(A->const_val_data), sp->off, sp->cnt, sp->list, C,
      ldc, alpha, beta, A->rows, n, (int)slabs, plan_of(A)->dev_err);
  impl(h)->launches++;
  return status_of(cudaGetLastError());
}

}  // namespace

void free_spmm_stage_plan(void* p) {
  StagePlan* sp = reinterpret_cast<StagePlan*>(p);
  if (!sp) return;
  cudaFree(sp->off);
  cudaFree(sp->cnt);
  cudaFree(sp->list);
  delete sp;
}

// Whether this product can run on the staged kernel - 32-bit offsets, sorted rows, every row block
// within the staging capacities, 16-byte aligned operands whose width is a multiple of a pack, and
// blocks that reuse their chunks - and, unless prepare_only, the launch.  Builds the chunk lists
// on first use (allocates and synchronises; part of preprocessing).
template <typename T>
alphasparseStatus_t spmm_stage_try(alphasparseHandle_t h, alphasparseSpMatDescr_t A, const T* B, int64_t ldb, T* C,
                                   int64_t ldc, T alpha, T beta, int64_t n, bool prepare_only, bool* ran) {
  *ran = false;
  constexpr int VN = 16 / (int)sizeof(T);
  Plan* p = plan_of(A);
  // a block of kStageRows rows is at most kStageRows / kSpmmRowBlock analysed blocks
  if (A->row_type != ALPHA_SPARSE_INDEXTYPE_I32 || p->max_block_nnz * (kStageRows / kSpmmRowBlock) > stage_cap<T>() ||
      n % VN != 0 || n < 2 * VN || ldb % VN != 0 || ldc % VN != 0 || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15) || A->cols >= (int64_t(1) << 31) - kStageChunk)
    return ALPHA_SPARSE_STATUS_SUCCESS;
  if (!p->spmm_stage) {
    StagePlan* sp = new (std::nothrow) StagePlan();
    if (!sp) return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    const alphasparseStatus_t s = build_stage_plan(h, A, sp);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) {
      free_spmm_stage_plan(sp);
      return s;
    }
    p->spmm_stage = sp;
  }
  const StagePlan* sp = reinterpret_cast<const StagePlan*>(p->spmm_stage);
  if (!sp->usable || !sp->list || sp->max_chunks > kStageMaxChunks) return ALPHA_SPARSE_STATUS_SUCCESS;
  // Worth it only when a block's chunks are reused: it must need far fewer staged rows of B than it has entries.
  if ((double)sp->total_chunks * kStageChunk > 0.5 * (double)A->nnz) return ALPHA_SPARSE_STATUS_SUCCESS;
  *ran = true;
  if (prepare_only) return ALPHA_SPARSE_STATUS_SUCCESS;
  const int64_t lanes = n / VN;
  if (lanes <= 2) return launch_stage<T, 2>(h, A, sp, B, ldb, C, ldc, alpha, beta, n);
  if (lanes <= 4) return launch_stage<T, 4>(h, A, sp, B, ldb, C, ldc, alpha, beta, n);
  if (lanes <= 8) return launch_stage<T, 8>(h, A, sp, B, ldb, C, ldc, alpha, beta, n);
  return launch_stage<T, 16>(h, A, sp, B, ldb, C, ldc, alpha, beta, n);
}

template alphasparseStatus_t spmm_stage_try<float>(alphasparseHandle_t, alphasparseSpMatDescr_t, const float*, int64_t, float*, int64_t, float, float, int64_t, bool, bool*);
template alphasparseStatus_t spmm_stage_try<double>(alphasparseHandle_t, alphasparseSpMatDescr_t, const double*, int64_t, double*, int64_t, double, double, int64_t, bool, bool*);

}  // namespace asp
