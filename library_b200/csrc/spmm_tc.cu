// Tensor-core SpMM for sm_100a:  C(fp32) = alpha * A(bf16, CSR) * B(bf16, row-major) + beta * C.
//
// The reference's CUDA backend has no tensor-core SpMM (its bf16 dispatch is commented out,
// cuda/kernel/level3/alphasparse_spmm.cu:597-610).  The precedent is the HIP backend's
// matrix-core algorithm ALG6 (hip/kernel/level3/alphasparse_spmm_tc4csr.h:43-255): a host pass
// turns CSR into dense 16x4 blocks, one wavefront then multiplies a 16x16 tile of C.  This file
// keeps the idea - treat the non-empty column blocks of a row block as small dense matrices -
// and rebuilds it for tcgen05:
//   * preprocessing (device): for every block of 128 rows, the ascending list of 64-column
//     chunks that hold at least one entry (a bitmap per row block, a scan, a fill); per chunk and
//     row where the row's run of entries inside the chunk starts and how long it is, and per entry
//     its column modulo 64 (or, for the kernels below the first, a per-chunk scatter list);
//   * spmm_tc_tmem_kernel (the default): one persistent, warp-specialised CTA per SM walks row
//     blocks.  The 128 x 64 chunk of A goes to the MMAs from TENSOR MEMORY: a builder thread owns a
//     row, gathers the row's few entries of the chunk and stores 32 registers with tcgen05.st;
//     loader warps fetch the chunk's 64 x N slice of B (cp.async.bulk.tensor, 128-byte swizzle,
//     completion on an mbarrier) into a ring of six stages; one warp issues four tcgen05.mma
//     (M=128, N, K=16) per chunk through an elected lane and tcgen05.commit hands the stage back;
//     an epilogue warp group reads the fp32 accumulators with tcgen05.ld and writes C (TMA stores
//     when beta = 0) while the next row block's chunks are already in the ring.  N = 192 and 256
//     run as two passes over 128 columns of B and C and the rest.
//   * spmm_tc_persistent_kernel (ASP_TC_A_TMEM=0, or when the run list cannot be built): the same
//     pipeline with builder warps clearing a 128 x 64 bf16 tile of A in shared memory and
//     scattering the chunk's entries into it.
//   * spmm_tc_kernel (ASP_TC_PERSISTENT=0): one CTA per row block, three B stages, two A tiles -
//     the simple form, also for matrices whose blocks hold more chunks than the persistent
//     shared-memory kernel stages.
// Every mbarrier wait is bounded; on expiry the CTA raises *err, frees its tensor memory and
// leaves.  No TMA load here uses cluster multicast.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cub/device/device_reduce.cuh>
#include <cub/device/device_scan.cuh>

#include <new>

#include "asp_internal.h"

namespace asp {

namespace {

constexpr int TC_M = 128;       // rows per CTA (the MMA's M)
static_assert(kSpmmRowBlock == TC_M, "Plan::max_block_nnz (per kSpmmRowBlock rows) bounds a row block's scatter offsets");
#ifndef ASP_TC_KC
#define ASP_TC_KC 64
#endif
constexpr int TC_KC = ASP_TC_KC; // columns of A per chunk (TC_KC / 16 MMAs of K = 16)
constexpr int TC_BBLK = TC_KC * 128;  // bytes of a chunk's B slice per 64 columns of B (TC_KC rows of 128 bytes)
constexpr int TC_THREADS = 128;
constexpr int TC_SPAN_WORDS = 2048;  // bitmap words: a row block may span 65,536 chunks
constexpr uint32_t TC_MAX_TRIES = 1u << 22;
constexpr int TC_A_BYTES = TC_M * TC_KC * 2;  // 16 KB, K-major core matrices, no swizzle
constexpr int TC_BSTAGES = 3;   // B slices in flight (two A tiles are enough: scatter is short)
constexpr int TC_CAP = 4096;    // entries of a row block staged in shared memory
constexpr int TC_MAXCH = 256;   // chunks of a row block whose ids and entry offsets are staged in shared memory
constexpr int TC_SRC_SHIFT = 13; // a scatter word = (entry's offset in the block's slice << 13) | element offset in the tile

struct TcPlan {
  int64_t blocks = 0, total_chunks = 0;
  int max_chunks = 0;
  bool usable = false;  // sorted columns, chunk span within the bitmap
  int32_t* chunk_off = nullptr;   // device, blocks + 1; every block's list starts on a multiple of four
  int32_t* chunk_cnt = nullptr;   // device, blocks: number of chunks of the block
  int32_t* chunk_list = nullptr;  // device, chunk_off[blocks] entries
  // The entries of A regrouped by chunk (within a row block; inside a chunk in row, then column
  // order), so that a tile is filled by independent threads instead of one serial walk per row:
  int32_t* chunk_ent = nullptr;   // device, parallel to chunk_list: first position in `scatter` of the chunk's entries
  uint32_t* scatter = nullptr;    // device, nnz words: where the entry comes from and where it goes
  // For the kernel that keeps A in tensor memory (a thread builds its own row of a chunk):
  uint32_t* runs = nullptr;       // device, 128 words per chunk slot: (first entry of the row's run in the chunk,
                                  // counted from the block's first entry rounded down to 16) << 7 | entries in the run
  uint8_t* kcol = nullptr;        // device, nnz bytes: the entry's column modulo 64 (its position in the chunk)
  bool runs_tried = false, scatter_tried = false;
};

// ---- preprocessing -------------------------------------------------------------------------
// One CTA per row block.  FILL = false: counts[b] = number of non-empty chunks, flags[0] |= 1 if
// the block spans more chunks than the bitmap, flags[1] |= 1 if a row's columns are not
// strictly ascending (out of order, or a column twice: two entries would land on one tile element).  FILL = true: writes the chunk ids, ascending, at chunk_off[b].
template <bool FILL>
__global__ void __launch_bounds__(256) tc_chunks_kernel(const int32_t* __restrict__ rp,
                                                        const int32_t* __restrict__ col, int64_t rows,
                                                        int32_t* __restrict__ counts,
                                                        int32_t* __restrict__ padded,
                                                        const int32_t* __restrict__ chunk_off,
                                                        int32_t* __restrict__ chunk_list,
                                                        int* __restrict__ flags) {
  __shared__ unsigned bm[TC_SPAN_WORDS];
  __shared__ int s_min;
  __shared__ int s_scan[256];
  const int tid = threadIdx.x;
  const int64_t r0 = (int64_t)blockIdx.x * TC_M;
  const int64_t r1 = r0 + TC_M < rows ? r0 + TC_M : rows;
  const int e0 = rp[r0], e1 = rp[r1];
  for (int i = tid; i < TC_SPAN_WORDS; i += 256) bm[i] = 0u;
  if (tid == 0) s_min = INT_MAX;
  __syncthreads();
  int mn = INT_MAX;
  for (int k = e0 + tid; k < e1; k += 256) mn = min(mn, col[k]);
  for (int o = 16; o > 0; o >>= 1) mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  if ((tid & 31) == 0 && mn != INT_MAX) atomicMin(&s_min, mn);
  __syncthreads();
  const int base = s_min == INT_MAX ? 0 : s_min / TC_KC;
  bool over = false;
  for (int k = e0 + tid; k < e1; k += 256) {
    const int c = col[k] / TC_KC - base;
    if (c >= TC_SPAN_WORDS * 32) over = true;
    else atomicOr(&bm[c >> 5], 1u << (c & 31));
  }
  if (!FILL) {
    bool unsorted = false;
    if (tid < (int)(r1 - r0)) {
      const int s = rp[r0 + tid], e = rp[r0 + tid + 1];
      for (int k = s + 1; k < e; ++k) unsorted |= col[k] <= col[k - 1];   // descending, or a column twice
    }
    if (over) atomicOr(&flags[0], 1);
    if (unsorted) atomicOr(&flags[1], 1);
  }
  __syncthreads();
  // 8 words per thread, block-wide exclusive scan of the popcounts
  int cnt = 0;
#pragma unroll
  for (int w = 0; w < TC_SPAN_WORDS / 256; ++w) cnt += __popc(bm[tid * (TC_SPAN_WORDS / 256) + w]);
  s_scan[tid] = cnt;
  __syncthreads();
  for (int o = 1; o < 256; o <<= 1) {
    const int v = tid >= o ? s_scan[tid - o] : 0;
    __syncthreads();
    s_scan[tid] += v;
    __syncthreads();
  }
  if (!FILL) {
    if (tid == 255) {
      counts[blockIdx.x] = s_scan[255];
      padded[blockIdx.x] = (s_scan[255] + 3) & ~3;
    }
  } else {
    int pos = chunk_off[blockIdx.x] + s_scan[tid] - cnt;
    for (int w = 0; w < TC_SPAN_WORDS / 256; ++w) {
      unsigned bits = bm[tid * (TC_SPAN_WORDS / 256) + w];
      while (bits) {
        const int b = __ffs(bits) - 1;
        bits &= bits - 1;
        chunk_list[pos++] = base + (tid * (TC_SPAN_WORDS / 256) + w) * 32 + b;
      }
    }
  }
}

// One CTA per row block, one thread per chunk of the block.  A chunk's entries are, row by row,
// the run of the row's (ascending) columns inside [64 c, 64 c + 64): two binary searches per row.
// FILL = false: counts[g] = entries of chunk g.  FILL = true: writes the chunk's scatter words at
// chunk_ent[g]; a word holds the entry's offset from the block's first entry rounded down to a
// multiple of eight (the staging kernel copies from there) and the bf16 element offset in the
// 128 x 64 tile.  An exclusive scan of the counts over all chunk slots (padding slots count zero)
// is the chunk's position: the chunks of earlier blocks hold exactly the entries before the block.
__device__ __forceinline__ int lower_bound_col(const int32_t* __restrict__ col, int lo, int hi, int key) {
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (col[mid] < key) lo = mid + 1;
    else hi = mid;
  }
  return lo;
}
template <bool FILL>
__global__ void __launch_bounds__(128) tc_scatter_kernel(const int32_t* __restrict__ rp,
                                                         const int32_t* __restrict__ col, int64_t rows,
                                                         const int32_t* __restrict__ chunk_off,
                                                         const int32_t* __restrict__ chunk_cnt,
                                                         const int32_t* __restrict__ chunk_list,
                                                         int32_t* __restrict__ counts,
                                                         const int32_t* __restrict__ chunk_ent,
                                                         uint32_t* __restrict__ scatter) {
  __shared__ int s_rp[TC_M + 1];
  const int64_t r0 = (int64_t)blockIdx.x * TC_M;
  const int nr = (int)(r0 + TC_M < rows ? TC_M : rows - r0);
  for (int i = threadIdx.x; i <= nr; i += 128) s_rp[i] = rp[r0 + i];
  __syncthreads();
  const int j0 = chunk_off[blockIdx.x], nch = chunk_cnt[blockIdx.x];
  const int a0 = s_rp[0] & ~7;
  for (int j = threadIdx.x; j < nch; j += 128) {
    const int cbeg = chunk_list[j0 + j] * TC_KC, cend = cbeg + TC_KC;
    int n = 0;
    int out = FILL ? chunk_ent[j0 + j] : 0;
    for (int r = 0; r < nr; ++r) {
      const int lo = lower_bound_col(col, s_rp[r], s_rp[r + 1], cbeg);
      const int hi = lower_bound_col(col, lo, s_rp[r + 1], cend);
      if (FILL) {
        for (int e = lo; e < hi; ++e) {
          const int x = col[e] - cbeg;
          scatter[out++] = ((uint32_t)(e - a0) << TC_SRC_SHIFT) |
                           (uint32_t)((x >> 3) * 1024 + (r >> 3) * 64 + (r & 7) * 8 + (x & 7));
        }
      } else {
        n += hi - lo;
      }
    }
    if (!FILL) counts[j0 + j] = n;
  }
}

// One CTA per row block, one thread per chunk of the block: for every row the run of its (ascending)
// columns inside the chunk, as (offset of the run's first entry from the block's first entry rounded
// down to a multiple of 16) << 7 | length.  Rows past the matrix keep the zero the array was cleared to.
__global__ void __launch_bounds__(128) tc_runs_kernel(const int32_t* __restrict__ rp, const int32_t* __restrict__ col,
                                                      int64_t rows, const int32_t* __restrict__ chunk_off,
                                                      const int32_t* __restrict__ chunk_cnt,
                                                      const int32_t* __restrict__ chunk_list,
                                                      uint32_t* __restrict__ runs) {
  __shared__ int s_rp[TC_M + 1];
  const int64_t r0 = (int64_t)blockIdx.x * TC_M;
  const int nr = (int)(r0 + TC_M < rows ? TC_M : rows - r0);
  for (int i = threadIdx.x; i <= nr; i += 128) s_rp[i] = rp[r0 + i];
  __syncthreads();
  const int j0 = chunk_off[blockIdx.x], nch = chunk_cnt[blockIdx.x];
  const int a0 = s_rp[0] & ~15;
  for (int j = threadIdx.x; j < nch; j += 128) {
    const int cbeg = chunk_list[j0 + j] * TC_KC, cend = cbeg + TC_KC;
    uint32_t* out = runs + (size_t)(j0 + j) * TC_M;
    for (int r = 0; r < nr; ++r) {
      const int lo = lower_bound_col(col, s_rp[r], s_rp[r + 1], cbeg);
      const int hi = lower_bound_col(col, lo, s_rp[r + 1], cend);
      out[r] = ((uint32_t)(lo - a0) << 7) | (uint32_t)(hi - lo);
    }
  }
}
__global__ void __launch_bounds__(256) tc_kcol_kernel(const int32_t* __restrict__ col, int64_t nnz,
                                                      uint8_t* __restrict__ kcol) {
  for (int64_t i = (int64_t)blockIdx.x * 256 + threadIdx.x; i < nnz; i += (int64_t)gridDim.x * 256)
    kcol[i] = (uint8_t)(col[i] % TC_KC);
}

// ---- PTX helpers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
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
// Bounded wait: false if the phase did not complete within `limit` polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = TC_MAX_TRIES) {
  for (uint32_t i = 0; i < limit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
  return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}
// Same with the descriptors given as (low, high) words: a stage's or K step's descriptor differs
// from a base descriptor only in the address field of the low word.
__device__ __forceinline__ void umma_bf16_lohi(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                               uint32_t b_hi, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(tmem_d),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(acc)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}

// Byte offset of element (row r, column k) in the 128 x 64 bf16 A tile: K-major core matrices
// of 8 rows x 8 columns (128 contiguous bytes), 16 of them down the rows (stride 128 B), 8
// across the columns (stride 2,048 B).  This is the no-swizzle canonical layout of the MMA's
// shared-memory descriptor with SBO = 128 and LBO = 2,048.
__device__ __forceinline__ int a_tile_off(int r, int k) {
  return (k >> 3) * 2048 + (r >> 3) * 128 + (r & 7) * 16 + (k & 7) * 2;
}

__global__ void __launch_bounds__(TC_THREADS)
spmm_tc_kernel(const __grid_constant__ CUtensorMap tmB, const int32_t* __restrict__ rp,
               const int32_t* __restrict__ col, const __nv_bfloat16* __restrict__ val,
               float* __restrict__ C, int64_t ldc, float alpha, float beta, int64_t rows, int64_t nnz, int n,
               const int32_t* __restrict__ chunk_off, const int32_t* __restrict__ chunk_cnt,
               const int32_t* __restrict__ chunk_list, int* __restrict__ err) {
  extern __shared__ unsigned char smem_raw[];
  // the swizzled B boxes (and the descriptors' address arithmetic) need a 1,024-byte aligned base
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int nblk = n / 64;                      // 64-column boxes of B per chunk
  const int b_stage_bytes = nblk * TC_BBLK;        // 64 rows x 128 B per box
  unsigned char* sA = smem;                     // 2 x 16 KB
  unsigned char* sB = smem + 2 * TC_A_BYTES;    // TC_BSTAGES x b_stage_bytes, 1,024-byte aligned
  int* s_col = reinterpret_cast<int*>(sB + TC_BSTAGES * b_stage_bytes);            // TC_CAP + 8
  __nv_bfloat16* s_val = reinterpret_cast<__nv_bfloat16*>(s_col + TC_CAP + 8);      // TC_CAP + 8
  int* s_chunks = reinterpret_cast<int*>(s_val + TC_CAP + 8);                       // TC_MAXCH
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_chunks + TC_MAXCH);
  uint64_t* full = bars;               // [TC_BSTAGES] B slice landed
  uint64_t* done = bars + TC_BSTAGES;  // [2] MMAs that read the A stage (and its B stage) retired
  uint64_t* csr_full = bars + TC_BSTAGES + 2;  // the row block's entries landed
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + TC_BSTAGES + 3);
  int* s_fail = reinterpret_cast<int*>(s_tmem + 1);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int64_t r0 = (int64_t)blockIdx.x * TC_M;
  const int nr = (int)(r0 + TC_M < rows ? TC_M : rows - r0);
  const int j0 = chunk_off[blockIdx.x];
  const int nchunks = chunk_cnt[blockIdx.x];
  const uint32_t tmem_cols = n <= 64 ? 64u : (n <= 128 ? 128u : 256u);

  // zero both A tiles, set up barriers and tensor memory
  for (int i = tid; i < 2 * TC_A_BYTES / 16; i += TC_THREADS) reinterpret_cast<uint4*>(sA)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    for (int i = 0; i < TC_BSTAGES; ++i) mbar_init(&full[i], 1);
    mbar_init(&done[0], 1);
    mbar_init(&done[1], 1);
    mbar_init(csr_full, 1);
    *s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                 "r"(tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *s_tmem;

  // instruction descriptor: D fp32, A and B bf16, A K-major, B MN-major, N = n, M = 128
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(n >> 3) << 17) |
                         ((uint32_t)(TC_M >> 4) << 24);

  // The row block's entries go to shared memory with two bulk copies (slices widened to groups of
  // eight entries, clipped to the arrays' last full group, the rest by plain loads); a block with
  // more than TC_CAP entries is read from global memory instead.  Chunk ids likewise.
  const int e0 = rp[r0], e1 = rp[r0 + nr];
  const int a0 = e0 & ~7;
  const bool staged = (e1 - a0) <= TC_CAP;
  const bool chunks_staged = nchunks <= TC_MAXCH;
  if (tid == 0 && staged) {
    int a1 = (e1 + 7) & ~7;
    const int nnz8 = (int)(nnz & ~(int64_t)7);
    if (a1 > nnz8) a1 = nnz8;
    if (a1 < a0) a1 = a0;
    const uint32_t cnt = (uint32_t)(a1 - a0);
    mbar_expect_tx(csr_full, cnt * 6u);
    if (cnt) {
      bulk_g2s(s_col, col + a0, cnt * 4u, csr_full);
      bulk_g2s(s_val, val + a0, cnt * 2u, csr_full);
    }
    for (int e = a1 > e0 ? a1 : e0; e < e1; ++e) {
      s_col[e - a0] = col[e];
      s_val[e - a0] = val[e];
    }
  }
  if (chunks_staged)
    for (int i = tid; i < nchunks; i += TC_THREADS) s_chunks[i] = chunk_list[j0 + i];
  const int* __restrict__ pc = staged ? s_col - a0 : col;               // indexed by the global entry number
  const __nv_bfloat16* __restrict__ pv = staged ? s_val - a0 : val;
  const int* __restrict__ pch = chunks_staged ? s_chunks : chunk_list + j0;

  // this thread's row of A: entries are consumed in column order as the chunks advance
  int k = 0, k_end = 0;
  if (tid < nr) {
    k = rp[r0 + tid];
    k_end = rp[r0 + tid + 1];
  }
  bool ok = true;
  __syncthreads();  // s_chunks and the plain-load tail are visible
  if (staged && !mbar_wait(csr_full, 0)) ok = false;

  // B slices run one chunk ahead of the MMAs: chunks 0 and 1 are requested here, chunk j + 1 as
  // soon as the MMAs of chunk j - 2 (which read the same B stage) have retired.
  auto request_b = [&](int jj) {
    const int bs = jj % TC_BSTAGES;
    mbar_expect_tx(&full[bs], (uint32_t)b_stage_bytes);
    for (int i = 0; i < nblk; ++i)
      tma_load_2d(sB + bs * b_stage_bytes + i * TC_BBLK, &tmB, i * 64, pch[jj] * TC_KC, &full[bs]);
  };
  if (tid == 0) {
    if (nchunks > 0) request_b(0);
    if (nchunks > 1) request_b(1);
  }

  for (int j = 0; j < nchunks; ++j) {
    const int s = j & 1;
    const int bs = j % TC_BSTAGES;
    const int chunk = pch[j];
    if (j >= 2) {
      // the MMAs of chunk j-2 must have finished reading this A stage and B stage (j-2) % 3
      if (ok && !mbar_wait(&done[s], (uint32_t)(((j >> 1) - 1) & 1))) ok = false;
    }
    if (tid == 0 && ok && j >= 1 && j + 1 < nchunks) request_b(j + 1);
    // re-zero this thread's row of the tile (eight 16-byte pieces, one per 8-column core matrix),
    // then scatter the row's entries that fall into this chunk
    unsigned char* tile = sA + s * TC_A_BYTES;
    if (j >= 2) {
#pragma unroll
      for (int q = 0; q < TC_KC / 8; ++q)
        *reinterpret_cast<uint4*>(tile + q * 2048 + (tid >> 3) * 128 + (tid & 7) * 16) = make_uint4(0, 0, 0, 0);
    }
    const int cbeg = chunk * TC_KC, cend = cbeg + TC_KC;
    while (k < k_end) {
      const int c = pc[k];
      if (c >= cend) break;
      *reinterpret_cast<__nv_bfloat16*>(tile + a_tile_off(tid, c - cbeg)) = pv[k];
      ++k;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // tile writes -> visible to the MMA
    const int any_fail = __syncthreads_or(ok ? 0 : 1);
    if (any_fail) {
      ok = false;
      break;
    }
    if (tid == 0) {
      if (!mbar_wait(&full[bs], (uint32_t)((j / TC_BSTAGES) & 1))) {
        *s_fail = 1;
      } else {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_base = smem_u32(tile);
        const uint32_t b_base = smem_u32(sB + bs * b_stage_bytes);
#pragma unroll
        for (int kk = 0; kk < TC_KC / 16; ++kk) {
          const uint64_t ad = umma_desc(a_base + kk * 4096, 2048, 128, 0);   // no swizzle, K-major
          const uint64_t bd = umma_desc(b_base + kk * 2048, TC_BBLK, 1024, 2);  // 128-byte swizzle, MN-major
          umma_bf16(tmem, ad, bd, idesc, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&done[s]);
      }
    }
  }

  // wait for the last chunk's MMAs, then the epilogue
  if (ok && nchunks > 0) {
    const int jl = nchunks - 1;
    if (!mbar_wait(&done[jl & 1], (uint32_t)((jl >> 1) & 1))) ok = false;
  }
  const int bad = __syncthreads_or((ok ? 0 : 1) | *s_fail);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (!bad) {
    const int row = tid;  // warp w reads tensor-memory lanes 32w .. 32w+31
    float* crow = C + (r0 + row) * ldc;
    for (int cb = 0; cb < n; cb += 32) {
      uint32_t acc[32];
      if (nchunks > 0) {
        tmem_ld32(tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)cb, acc);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = 0u;
      }
      if (row < nr) {
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float4 o;
          o.x = alpha * __uint_as_float(acc[i]);
          o.y = alpha * __uint_as_float(acc[i + 1]);
          o.z = alpha * __uint_as_float(acc[i + 2]);
          o.w = alpha * __uint_as_float(acc[i + 3]);
          if (beta != 0.f) {
            const float4 c0 = *reinterpret_cast<const float4*>(crow + cb + i);
            o.x = fmaf(beta, c0.x, o.x);
            o.y = fmaf(beta, c0.y, o.y);
            o.z = fmaf(beta, c0.z, o.z);
            o.w = fmaf(beta, c0.w, o.w);
          }
          *reinterpret_cast<float4*>(crow + cb + i) = o;
        }
      }
    }
  } else {
    if (tid == 0) atomicExch(err, 1);
    __nanosleep(1000000);  // give copies and MMAs still in flight time to retire
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(tmem_cols) : "memory");
}

// ------------------------------------------------------------------------------------------
// Persistent, warp-specialised form: one CTA per SM walks row blocks blockIdx.x, +gridDim.x, ...
// and splits the work of spmm_tc_kernel over roles that only meet through mbarriers, so that a
// row block's slices are staged a block ahead, several chunks are in flight at once and the
// epilogue of a row block overlaps the MMAs of the next one:
//   warps 0-15 builders : four groups of 128 threads take chunks in turn (running chunk number
//                         modulo four).  Per chunk a group waits for the ring stage, asks for the
//                         chunk's B slice by TMA, clears the A tile and fills it from the plan's
//                         scatter list: thread t copies the chunk's entries t, t+128, ... from
//                         the staged values to the tile elements the list names - no walk along
//                         rows, no column compare                     (st_empty -> st_full)
//   warps 16-19 epilogue: tcgen05.ld of the block's accumulators, alpha/beta, store C
//                                                                       (acc_full -> acc_empty)
//   warp 20    producer : bulk copies of the next block's slice of the scatter list, of the
//                         values, and of the block's chunk ids and chunk offsets
//                                                                       (csr_empty -> csr_full)
//   warps 21-22 MMA     : one thread each.  A thread's stream of wait / 4 x tcgen05.mma / commit
//                         takes about 560 cycles per chunk however small N is, the tensor core
//                         about 260 (N = 128), so two threads issue: even running chunk numbers
//                         to one, odd to the other, each into its own accumulator (tensor memory
//                         holds 2 blocks x 2 issuers x N columns when N <= 128; at N = 256 one
//                         thread issues).  Commits to st_empty per chunk and to acc_full per
//                         block; warp 21 owns the tensor-memory allocation
// A barrier of the "empty" kind is waited on with the inverted parity, so its first use passes.
// Every wait is bounded; a role whose wait expires raises the CTA's fail flag and stops working
// (builders keep walking their loop so that the groups' named barriers still match), the other
// roles then run into their own limits, and all meet at the final __syncthreads.
// ------------------------------------------------------------------------------------------
#ifndef ASP_TCP_GROUPS
#define ASP_TCP_GROUPS 4
#endif
constexpr int TCP_BWARPS = 16;                        // builder warps
constexpr int TCP_GROUPS = ASP_TCP_GROUPS;            // builder groups (4 of four warps, or 8 of two)
constexpr int TCP_GWARPS = TCP_BWARPS / TCP_GROUPS;   // warps of a group
constexpr int TCP_GTHREADS = TCP_GWARPS * 32;
constexpr int TCP_THREADS = (TCP_BWARPS + 7) * 32;    // builders, 4 epilogue warps, producer, 2 MMA warps
static_assert(TCP_GROUPS * TCP_GWARPS == TCP_BWARPS && TC_M % TCP_GTHREADS == 0, "builder groups");
constexpr int TCP_CSR = 3;  // row-block CSR buffers: staging block i+1 never waits for the builders of block i-1
#ifndef ASP_TCT_PARK_NS
#define ASP_TCT_PARK_NS 2000u
#endif
// Bounded wait that leaves the waiting to the hardware, for the roles whose waits are long
// (builders, loaders, epilogue): try_wait with a suspend-time hint parks the thread until the phase
// completes or the time is over, so a long wait costs a few polls instead of one every hundred
// cycles.  Every poll is a shared-memory access, and a warp that spins takes issue slots from the
// roles that share its scheduler.
__device__ __forceinline__ bool mbar_wait_parked(uint64_t* bar, uint32_t parity, uint32_t limit = TC_MAX_TRIES) {
  for (uint32_t i = 0; i < (limit >> 4) + 1u; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ASP_TCT_PARK_NS)
        : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ bool mbar_wait_backoff(uint64_t* bar, uint32_t parity) { return mbar_wait_parked(bar, parity); }

// Bounded spin on the non-blocking test: lowest wake-up latency, for the waits that sit on the
// per-chunk critical path (try_wait may park the thread for a scheduler time slice).
__device__ __forceinline__ bool mbar_spin(uint64_t* bar, uint32_t parity, uint32_t limit = TC_MAX_TRIES) {
  for (uint32_t i = 0; i < (limit << 4); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// One lane of the (converged) warp: unlike `lane == 0`, elect.sync tells the compiler that exactly
// one thread runs the guarded code, so that the operands of the instructions that take them from
// uniform registers (tcgen05.mma, tcgen05.commit, the TMA and bulk copies) need no per-lane
// serialisation.  Every lane named in the mask has to execute it.
__device__ __forceinline__ bool elect_one(uint32_t mask = 0xffffffffu) {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, %1;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred)
      : "r"(mask));
  return pred != 0;
}

// One non-blocking test of a barrier's phase.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(TCP_THREADS, 1)
spmm_tc_persistent_kernel(const __grid_constant__ CUtensorMap tmB, const int32_t* __restrict__ rp,
                          const int32_t* __restrict__ col, const __nv_bfloat16* __restrict__ val,
                          float* __restrict__ C, int64_t ldc, float alpha, float beta, int64_t rows,
                          int64_t nnz, int n, int nblocks, int sb,
                          const int32_t* __restrict__ chunk_off, const int32_t* __restrict__ chunk_cnt,
                          const int32_t* __restrict__ chunk_list, const int32_t* __restrict__ chunk_ent,
                          const uint32_t* __restrict__ scatter, int one_box, int issuers_max,
                          int* __restrict__ err) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int nblk = n / 64;
  const int b_stage_bytes = nblk * TC_BBLK;
  unsigned char* sA = smem;                               // sb x 16 KB (A tiles and B slices share one ring)
  unsigned char* sB = sA + (size_t)sb * TC_A_BYTES;       // sb x b_stage_bytes
  unsigned char* p = sB + (size_t)sb * b_stage_bytes;
  uint32_t* s_sc = reinterpret_cast<uint32_t*>(p);        // TCP_CSR x (TC_CAP + 8) scatter words
  __nv_bfloat16* s_val = reinterpret_cast<__nv_bfloat16*>(s_sc + TCP_CSR * (TC_CAP + 8));   // TCP_CSR x (TC_CAP + 8)
  int* s_chunks = reinterpret_cast<int*>(s_val + TCP_CSR * (TC_CAP + 8));                   // TCP_CSR x TC_MAXCH chunk ids
  int* s_ent = s_chunks + TCP_CSR * TC_MAXCH;                                               // TCP_CSR x TC_MAXCH entry offsets
  float* s_tr = reinterpret_cast<float*>(s_ent + TCP_CSR * TC_MAXCH);  // 4 epilogue warps x 32 x 33
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_tr + 4 * 32 * 33 + 2);
  uint64_t* csr_full = bars;            // [TCP_CSR]
  uint64_t* csr_empty = bars + 4;       // [TCP_CSR]
  uint64_t* acc_full = bars + 8;        // [2]
  uint64_t* acc_empty = bars + 10;      // [2]
  uint64_t* st_full = bars + 12;        // [sb] A tile built (4 builder warps) and B slice landed (producer + bytes)
  uint64_t* st_empty = st_full + sb;    // [sb] the chunk's MMAs retired: tile and slice are free
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(st_empty + sb);
  volatile int* s_fail = reinterpret_cast<volatile int*>(s_tmem + 1);

  // the warp number through a shuffle: provably the same in every lane, so that what derives from
  // it (roles, ring stages, descriptors) can live in uniform registers
  const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
  const uint32_t acc_cols = n <= 64 ? 64u : (n <= 128 ? 128u : 256u);
  // Two threads issue MMAs when tensor memory holds four accumulators (N <= 128): chunks with an
  // even running number go to one, odd ones to the other, each into an accumulator of its own
  // (the epilogue adds them).  One thread's stream of wait / 4 x tcgen05.mma / commit costs about
  // twice the 256 cycles the tensor core needs for a chunk, so a single issuer halves its rate.
  const int issuers = (acc_cols <= 128u && issuers_max >= 2) ? 2 : 1;

  for (int i = tid; i < sb * TC_A_BYTES / 16; i += TCP_THREADS)
    reinterpret_cast<uint4*>(sA)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    for (int i = 0; i < TCP_CSR; ++i) {
      mbar_init(&csr_full[i], 1);
      mbar_init(&csr_empty[i], TCP_BWARPS);   // one arrival per builder warp
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], (uint32_t)issuers);
      mbar_init(&acc_empty[i], 4);
    }
    for (int i = 0; i < sb; ++i) {
      mbar_init(&st_full[i], TCP_GWARPS + 1);   // the group's warps and the thread that announces the B slice's bytes
      mbar_init(&st_empty[i], 1);
    }
    *s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == TCP_BWARPS + 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                 "r"(2u * (uint32_t)issuers * acc_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *s_tmem;

  const int first = blockIdx.x, stride = gridDim.x;
  const int n_my = first < nblocks ? (nblocks - first + stride - 1) / stride : 0;

  if (warp == TCP_BWARPS + 4) {
    // ---------------- producer ----------------
    // The whole warp runs the loop (waits are warp-uniform): lane 0 stages the CSR slices and arms
    // the barriers, lanes 0..nblk-1 each issue one 64-column box of a chunk's B slice.  The scalars
    // a block's staging needs are loaded from global memory a block ahead of their use.
    {
      int p_e0 = 0, p_e1 = 0, p_j0 = 0, p_nch = 0;  // prefetched for the next block to stage
      auto prefetch = [&](int i) {
        const int b = first + i * stride;
        const int64_t r0 = (int64_t)b * TC_M;
        const int nr = (int)(r0 + TC_M < rows ? TC_M : rows - r0);
        p_e0 = rp[r0];
        p_e1 = rp[r0 + nr];
        p_j0 = chunk_off[b];
        p_nch = chunk_cnt[b];
      };
      auto stage_csr = [&](int i) -> bool {
        const int cs = i % TCP_CSR;
        if (!mbar_wait(&csr_empty[cs], (uint32_t)(((i / TCP_CSR) & 1) ^ 1))) return false;
        const int e0 = p_e0, e1 = p_e1, j0 = p_j0, nch = p_nch;
        if (i + 1 < n_my) prefetch(i + 1);
        if (lane == 0) {
          const int a0 = e0 & ~7;
          const bool staged = (e1 - a0) <= TC_CAP;
          uint32_t* dc = s_sc + cs * (TC_CAP + 8);
          __nv_bfloat16* dv = s_val + cs * (TC_CAP + 8);
          uint32_t cnt = 0;
          if (staged) {
            int a1 = (e1 + 7) & ~7;
            const int nnz8 = (int)(nnz & ~(int64_t)7);
            if (a1 > nnz8) a1 = nnz8;
            if (a1 < a0) a1 = a0;
            cnt = (uint32_t)(a1 - a0);
            for (int e = a1 > e0 ? a1 : e0; e < e1; ++e) {  // past the arrays' last full group of eight
              dc[e - a0] = scatter[e];
              dv[e - a0] = val[e];
            }
          }
          const uint32_t nch4 = (uint32_t)((nch + 3) & ~3);
          mbar_expect_tx(&csr_full[cs], cnt * 6u + nch4 * 8u);
          if (cnt) {
            bulk_g2s(dc, scatter + a0, cnt * 4u, &csr_full[cs]);
            bulk_g2s(dv, val + a0, cnt * 2u, &csr_full[cs]);
          }
          if (nch4) {
            bulk_g2s(s_chunks + cs * TC_MAXCH, chunk_list + j0, nch4 * 4u, &csr_full[cs]);
            bulk_g2s(s_ent + cs * TC_MAXCH, chunk_ent + j0, nch4 * 4u, &csr_full[cs]);
          }
        }
        return true;
      };
      bool ok = true;
      if (n_my > 0) {
        prefetch(0);
        ok = stage_csr(0);
      }
      // The chunks' B slices are requested by the builder groups: this warp only keeps the row
      // blocks' slices of the scatter list, the values and the chunk tables a block ahead.
      for (int i = 0; i < n_my && ok; ++i)
        if (i + 1 < n_my) ok = stage_csr(i + 1);
      if (!ok) *s_fail = 1;
    }
  } else if (warp >= TCP_BWARPS + 5) {
    // ---------------- MMA issuers ----------------
    // The whole warp walks the loop (every lane polls, votes keep the lanes together) and one
    // elected lane issues: with a lone thread behind `lane == 0` the stream of a chunk - wait,
    // four MMAs, commit - took about twice the tensor core's time for it.
    const int w = warp - (TCP_BWARPS + 5);
    if (w < issuers) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(n >> 3) << 17) |
                             ((uint32_t)(TC_M >> 4) << 24);
      bool ok = true;
      int st = w;               // ring stage and parity of this issuer's next chunk
      uint32_t ph = 0;
      while (st >= sb) {
        st -= sb;
        ph ^= 1u;
      }
      uint32_t cnum0 = 0, mine = (uint32_t)w;  // running numbers: the block's first chunk, this issuer's next chunk
      // A stage's descriptors differ from stage 0's only in the low word (the 14-bit address
      // field), so the loop adds small constants instead of rebuilding 64-bit descriptors.
      const uint64_t ad0 = umma_desc(smem_u32(sA), 2048, 128, 0);
      const uint64_t bd0 = umma_desc(smem_u32(sB), TC_BBLK, 1024, 2);
      const uint32_t a_hi = (uint32_t)(ad0 >> 32), b_hi = (uint32_t)(bd0 >> 32);
      const uint32_t a_lo0 = (uint32_t)ad0, b_lo0 = (uint32_t)bd0;
      const uint32_t a_step = TC_A_BYTES >> 4, b_step = (uint32_t)b_stage_bytes >> 4;
      int nch_next = n_my > 0 ? chunk_cnt[first] : 0;
      for (int i = 0; i < n_my && ok; ++i) {
        const int acc = (i & 1) * issuers + w;
        const int nch = nch_next;  // fetched one block ahead: no global latency between blocks
        if (i + 1 < n_my) nch_next = chunk_cnt[first + (i + 1) * stride];
        if (!__all_sync(0xffffffffu, mbar_wait(&acc_empty[i & 1], (uint32_t)(((i >> 1) & 1) ^ 1)))) {
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem + (uint32_t)acc * acc_cols;
        uint32_t first_acc = 0u;  // the issuer's first MMA of the block overwrites its accumulator
        for (int j = (int)(mine - cnum0); j < nch; j += issuers, mine += (uint32_t)issuers) {
          if (!__all_sync(0xffffffffu, mbar_spin(&st_full[st], ph))) {
            ok = false;
            break;
          }
          // no tcgen05.fence here: the mbarrier wait orders the MMAs after the TMA bytes and after
          // the builders' stores (made visible to the async proxy by their fence.proxy.async); a
          // fence in this loop would make the issuing thread wait for the previous chunk's MMAs
          const uint32_t a_lo = a_lo0 + (uint32_t)st * a_step, b_lo = b_lo0 + (uint32_t)st * b_step;
          if (elect_one()) {
            umma_bf16_lohi(d, a_lo, a_hi, b_lo, b_hi, idesc, first_acc);
#pragma unroll
            for (uint32_t kk = 1; kk < TC_KC / 16; ++kk)
              umma_bf16_lohi(d, a_lo + kk * 256u, a_hi, b_lo + kk * 128u, b_hi, idesc, 1u);
            umma_commit(&st_empty[st]);
          }
          __syncwarp();
          first_acc = 1u;
          st += issuers;
          while (st >= sb) {
            st -= sb;
            ph ^= 1u;
          }
        }
        cnum0 += (uint32_t)nch;
        // also with no chunk of its own: the barrier counts the issuers
        if (ok && elect_one()) umma_commit(&acc_full[i & 1]);
        __syncwarp();
      }
      if (!ok) *s_fail = 1;
    }
  } else if (warp < TCP_BWARPS) {
    // ---------------- builders: TCP_GROUPS groups of 128 threads ----------------
    // Group g takes the chunks whose running number (over all row blocks of this CTA) is g modulo
    // TCP_GROUPS.  Per chunk: wait for the ring stage, ask for the B slice (first warp), clear the
    // tile (16 bytes x 8 per thread), meet the group's other warps at a named barrier, then each
    // thread copies the chunk's entries t, t + 128, ... from the staged values to the tile element
    // its scatter word names, and the warp arrives on the stage's full barrier.  A warp whose wait
    // ran out keeps walking the loop without waiting or storing, so the barrier counts still match.
    // A wait by parity is only right for a waiter that sees every phase of its barrier, so a ring
    // stage must always come back to the same group: min(sb, TCP_GROUPS) groups work, group g on
    // the chunks g modulo that number (the host makes sb 2 or 4; with 2 two groups idle).
    bool ok = true;
    const int grp = warp / TCP_GWARPS;
    const int gt = tid % TCP_GTHREADS;
    const int ng = sb < TCP_GROUPS ? sb : TCP_GROUPS;
    const bool active = grp < ng;
    int sa = grp;                 // ring stage and parity of the group's next chunk
    uint32_t ph = 0;
    while (sa >= sb) {
      sa -= sb;
      ph ^= 1u;
    }
    uint32_t cnum0 = 0;           // running number of the block's first chunk
    uint32_t mine = (uint32_t)grp;  // running number of the group's next chunk
    int n_e0 = 0, n_e1 = 0, n_nch = 0;  // per-block scalars, fetched one block ahead
    auto fetch = [&](int i) {
      const int b = first + i * stride;
      const int64_t r0 = (int64_t)b * TC_M;
      const int nr = (int)(r0 + TC_M < rows ? TC_M : rows - r0);
      n_e0 = rp[r0];
      n_e1 = rp[r0 + nr];
      n_nch = chunk_cnt[b];
    };
    if (n_my > 0) fetch(0);
    for (int i = 0; i < n_my; ++i) {
      const int cs = i % TCP_CSR;
      const int e0 = n_e0, e1 = n_e1, nch = n_nch;
      const int a0 = e0 & ~7;
      const bool staged = (e1 - a0) <= TC_CAP;
      if (i + 1 < n_my) fetch(i + 1);
      if (ok && !mbar_wait_backoff(&csr_full[cs], (uint32_t)((i / TCP_CSR) & 1))) ok = false;
      const uint32_t* __restrict__ psc = staged ? s_sc + cs * (TC_CAP + 8) - a0 : scatter;  // by entry number
      const __nv_bfloat16* __restrict__ pv = staged ? s_val + cs * (TC_CAP + 8) : val + a0;  // by offset in the slice
      const int* pch = s_chunks + cs * TC_MAXCH;
      const int* pent = s_ent + cs * TC_MAXCH;
      for (int j = active ? (int)(mine - cnum0) : nch; j < nch; j += ng, mine += (uint32_t)ng) {
        // the chunk's scalars come out of shared memory while the stage is still awaited
        const int brow = pch[j] * TC_KC;
        const int beg = pent[j];
        const int end = j + 1 < nch ? pent[j + 1] : e1;
        if (ok && !mbar_wait_backoff(&st_empty[sa], ph ^ 1u)) ok = false;
        __nv_bfloat16* tile = reinterpret_cast<__nv_bfloat16*>(sA + sa * TC_A_BYTES);
        if (ok) {
          if (warp % TCP_GWARPS == 0) {
            // the slice's latency runs under the build, and four groups issue side by side
            // (one instruction for the whole slice when the map is the three-dimensional view
            // [column block][row][64 columns]: issuing a copy costs the warp some 300 cycles)
            if (elect_one(__activemask())) {
              mbar_expect_tx(&st_full[sa], (uint32_t)b_stage_bytes);
              if (one_box) tma_load_3d(sB + (size_t)sa * b_stage_bytes, &tmB, 0, brow, 0, &st_full[sa]);
            }
            __syncwarp();
            if (!one_box && lane < nblk)
              tma_load_2d(sB + (size_t)sa * b_stage_bytes + lane * TC_BBLK, &tmB, lane * 64, brow, &st_full[sa]);
          }
          if (mine >= (uint32_t)sb) {
#pragma unroll
            for (int q = 0; q < TC_KC / 8; ++q)
#pragma unroll
              for (int r = gt; r < TC_M; r += TCP_GTHREADS)
                *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(tile) + q * 2048 + r * 16) =
                    make_uint4(0, 0, 0, 0);
          }
        }
        asm volatile("bar.sync %0, %1;" ::"r"(grp + 1), "n"(TCP_GTHREADS) : "memory");
        if (ok) {
          // two entries per thread side by side (a chunk of a stencil matrix has under 256), the
          // rest in a loop: a lone thread's chain of dependent shared-memory accesses is what a
          // build's time is made of
          constexpr uint32_t kPos = (1u << TC_SRC_SHIFT) - 1u;
          const int t0 = beg + gt, t1 = t0 + TCP_GTHREADS;
          const uint32_t w0 = t0 < end ? psc[t0] : 0u;
          const uint32_t w1 = t1 < end ? psc[t1] : 0u;
          const __nv_bfloat16 v0 = pv[w0 >> TC_SRC_SHIFT], v1 = pv[w1 >> TC_SRC_SHIFT];
          if (t0 < end) tile[w0 & kPos] = v0;
          if (t1 < end) tile[w1 & kPos] = v1;
          for (int t = t1 + TCP_GTHREADS; t < end; t += TCP_GTHREADS) {
            const uint32_t w = psc[t];
            tile[w & kPos] = pv[w >> TC_SRC_SHIFT];
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&st_full[sa]);
        }
        sa += ng;
        while (sa >= sb) {
          sa -= sb;
          ph ^= 1u;
        }
      }
      cnum0 += (uint32_t)nch;
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(&csr_empty[cs]);
    }
    if (!ok) *s_fail = 1;
  } else {
    // ---------------- epilogue: four warps (ids = 0..3 mod 4) read tensor-memory lanes 32*(id mod 4) .. ----------------
    bool ok = true;
    const int row = tid - TCP_BWARPS * 32;
    int nch_next = n_my > 0 ? chunk_cnt[first] : 0;
    uint32_t cnum0 = 0;  // running number of the block's first chunk: tells which issuers had a chunk
    for (int i = 0; i < n_my && ok; ++i) {
      const int acc = i & 1;
      const int b = first + i * stride;
      const int64_t r0 = (int64_t)b * TC_M;
      const int nr = (int)(r0 + TC_M < rows ? TC_M : rows - r0);
      const int nch = nch_next;
      if (i + 1 < n_my) nch_next = chunk_cnt[first + (i + 1) * stride];
      if (!mbar_wait_backoff(&acc_full[acc], (uint32_t)((i >> 1) & 1))) {
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // tcgen05.ld hands lane l the 32 columns of row l; a per-warp 32 x 33 shared-memory tile turns
      // that around so that a store instruction writes 32 consecutive floats of one row (one line)
      // instead of 16 bytes of 32 different rows.
      float* tr = s_tr + (warp - TCP_BWARPS) * (32 * 33);
      const int wrow0 = (warp - TCP_BWARPS) * 32;
      (void)row;
      for (int cb = 0; cb < n; cb += 32) {
        uint32_t a[32];
        if (nch > 0) {
          // the issuer of the block's first chunk always has data; the other one from two chunks on
          const uint32_t w0 = issuers == 2 ? (cnum0 & 1u) : 0u;
          tmem_ld32(tmem + ((uint32_t)wrow0 << 16) + ((uint32_t)(acc * issuers) + w0) * acc_cols + (uint32_t)cb, a);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (issuers == 2 && nch > 1) {
            uint32_t a2[32];
            tmem_ld32(tmem + ((uint32_t)wrow0 << 16) + ((uint32_t)(acc * issuers) + (w0 ^ 1u)) * acc_cols + (uint32_t)cb, a2);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int q = 0; q < 32; ++q) a[q] = __float_as_uint(__uint_as_float(a[q]) + __uint_as_float(a2[q]));
          }
        } else {
#pragma unroll
          for (int q = 0; q < 32; ++q) a[q] = 0u;
        }
#pragma unroll
        for (int q = 0; q < 32; ++q) tr[lane * 33 + q] = alpha * __uint_as_float(a[q]);
        __syncwarp();
        const int rmax = nr - wrow0 < 32 ? nr - wrow0 : 32;
        for (int rr = 0; rr < rmax; ++rr) {
          float* cp = C + (r0 + wrow0 + rr) * ldc + cb + lane;
          float o = tr[rr * 33 + lane];
          if (beta != 0.f) o = fmaf(beta, *cp, o);
          *cp = o;
        }
        __syncwarp();
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      cnum0 += (uint32_t)nch;
    }
    if (!ok) *s_fail = 1;
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*s_fail) {
    if (tid == 0) atomicExch(err, 1);
    __nanosleep(1000000);  // let copies and MMAs still in flight retire before the memory goes away
  }
  if (warp == TCP_BWARPS + 5)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2u * (uint32_t)issuers * acc_cols) : "memory");
}

// ------------------------------------------------------------------------------------------
// The same pipeline with A in tensor memory (N <= 128).  tcgen05.mma takes its A operand from
// tensor memory as well as from shared memory: lane = row, a 32-bit column = two consecutive bf16
// of the row.  A builder thread then owns one row of the chunk: it drops the row's few entries
// into a private 128-byte line of shared memory (no other thread touches it: no barrier, no
// async-proxy fence, no clear of a 16 KB tile), reads back the 16-byte pieces it touched, zeroes
// what it wrote and hands 32 registers to tensor memory with one tcgen05.st.  What that frees:
//   * the A tiles' shared memory goes to B slices: six ring stages at N = 128 instead of four;
//   * the MMAs read half as much shared memory (B only) - the unit that bounds this kernel is the
//     SM's shared-memory / L1 data pipe, which the B slices alone (written by TMA, read by the
//     MMAs) keep busy for 256 of a chunk's cycles at N = 128;
//   * one warp issues (all lanes walk the loop, one elected lane issues: its stream keeps up with
//     the tensor core), so two accumulators are enough and tensor memory has room for the A stages:
//     columns [0, 2 acc) accumulators of two row blocks, then 32 columns per ring stage.
//   warps 0-11  builders : three groups of 128 threads (thread = row = tensor-memory lane) take
//                          chunks in turn; a group owns ring stages g and g + 3
//   warps 12-15 epilogue : tcgen05.ld, alpha; with beta = 0 the 32 x 32 blocks of C leave by TMA
//                          stores from a swizzled tile, else through a transposition tile and
//                          128-byte row stores
//   warp 16     producer : values, column bytes, per-row run words and the scalars of the next
//                          row block by bulk copies (the builders load nothing from global memory)
//   warp 17     MMA
//   warps 18-20 B loaders: warp g asks for the B slices of the chunks g modulo 3 as soon as their
//                          ring stage is free
// Waits that may be long park in hardware (try_wait with a suspend-time hint): every poll is a
// shared-memory access.  The plan holds, per chunk and row, where the row's run of entries inside
// the chunk starts and how long it is (tc_runs_kernel), and per entry its column modulo 64 as a byte.
// ------------------------------------------------------------------------------------------
constexpr int TCT_GROUPS = 3;
constexpr int TCT_BWARPS = TCT_GROUPS * 4;
constexpr int TCT_STAGES = 2 * TCT_GROUPS;
constexpr int TCT_THREADS = (TCT_BWARPS + 6 + TCT_GROUPS) * 32;
constexpr int TCT_CSR = 2;
constexpr int TCT_CAPB = TC_CAP + 16;      // staged entries of a row block (slice widened to multiples of 16)
constexpr int TCT_RUNCH = 32;              // chunks of a row block whose run words are staged (the rest: global loads)
constexpr int TCT_PRIV = TC_M * 128;       // a group's private lines: 128 rows x 64 bf16
constexpr uint32_t TCT_TMEM_COLS = 512;
constexpr int TCT_TRLD = 36;               // floats per row of an epilogue warp's transposition tile
constexpr int TCT_TRBYTES = 5120;          // an epilogue warp's tile: 32 x TCT_TRLD floats, or 32 x 128 bytes for a TMA store
static_assert(TC_KC == 64, "a row of a chunk is one 128-byte line / 32 tensor-memory columns");

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
// A from tensor memory, B through a shared-memory descriptor given as (low, high) words.
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi,
                                             uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}" ::"r"(tmem_d),
      "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(acc)
      : "memory");
}
// A load that stays where it is written: the compiler is free to sink a plain load of read-only
// data to its first use, which puts the whole global latency back into the chunk's chain.
__device__ __forceinline__ uint32_t ldg_here_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void sts_b16(uint32_t saddr, uint16_t v) {
  asm volatile("st.shared.b16 [%0], %1;" ::"r"(saddr), "h"(v) : "memory");
}
// The load happens only where `on` is set; elsewhere the registers keep what they hold.
__device__ __forceinline__ void lds_v4_if(uint32_t on, uint32_t saddr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "@p ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];\n\t}"
      : "+r"(a), "+r"(b), "+r"(c), "+r"(d)
      : "r"(saddr), "r"(on)
      : "memory");
}

__global__ void __launch_bounds__(TCT_THREADS, 1)
spmm_tc_tmem_kernel(const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC, int c_by_tma,
                    const int32_t* __restrict__ rp,
                    const __nv_bfloat16* __restrict__ val, float* __restrict__ C, int64_t ldc, float alpha,
                    float beta, int64_t rows, int64_t nnz, int n, int nblocks,
                    const int32_t* __restrict__ chunk_off, const int32_t* __restrict__ chunk_cnt,
                    const int32_t* __restrict__ chunk_list, const uint32_t* __restrict__ runs,
                    const uint8_t* __restrict__ kcol, int one_box, uint32_t wait_cfg, int* __restrict__ err) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int nblk = n / 64;
  const int b_stage_bytes = nblk * TC_BBLK;
  unsigned char* sB = smem;                                                   // TCT_STAGES x b_stage_bytes
  unsigned char* sP = sB + (size_t)TCT_STAGES * b_stage_bytes;                // TCT_GROUPS x 16 KB private lines
  float* s_tr = reinterpret_cast<float*>(sP + TCT_GROUPS * TCT_PRIV);                    // 4 x TCT_TRBYTES, 1,024-byte aligned
  __nv_bfloat16* s_val = reinterpret_cast<__nv_bfloat16*>(s_tr + 4 * (TCT_TRBYTES / 4)); // TCT_CSR x TCT_CAPB
  uint8_t* s_k = reinterpret_cast<uint8_t*>(s_val + TCT_CSR * TCT_CAPB);                 // TCT_CSR x TCT_CAPB
  uint32_t* s_runs = reinterpret_cast<uint32_t*>(s_k + TCT_CSR * TCT_CAPB);              // TCT_CSR x TCT_RUNCH x 128
  int* s_hdr = reinterpret_cast<int*>(s_runs + TCT_CSR * TCT_RUNCH * TC_M);              // TCT_CSR x 4: e0, e1, chunks, first slot
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_hdr + TCT_CSR * 4);
  uint64_t* csr_full = bars;            // [TCT_CSR]
  uint64_t* csr_empty = bars + 4;       // [TCT_CSR]
  uint64_t* acc_full = bars + 8;        // [2]
  uint64_t* acc_empty = bars + 10;      // [2]
  uint64_t* st_full = bars + 12;        // [TCT_STAGES] A stage stored (4 builder warps) and B slice landed
  uint64_t* st_empty = st_full + TCT_STAGES;  // [TCT_STAGES] the chunk's MMAs retired
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(st_empty + TCT_STAGES);
  volatile int* s_fail = reinterpret_cast<volatile int*>(s_tmem + 1);

  const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, tid >> 5, 0), lane = tid & 31;
  // the plan's wait settings: how many polls a wait may take, and the test hook that announces the
  // B slices' bytes to the barriers without asking for the copies (every wait then runs out)
  const uint32_t lim = wait_cfg & kWaitPollMask;
  const bool drop_copies = (wait_cfg & kWaitDropCopy) != 0u;
  const uint32_t acc_cols = n <= 64 ? 64u : 128u;
  const uint32_t a_col0 = 2u * acc_cols;

  for (int i = tid; i < TCT_GROUPS * TCT_PRIV / 16; i += TCT_THREADS)
    reinterpret_cast<uint4*>(sP)[i] = make_uint4(0, 0, 0, 0);
  if (tid == 0) {
    for (int i = 0; i < TCT_CSR; ++i) {
      mbar_init(&csr_full[i], 1);
      mbar_init(&csr_empty[i], TCT_BWARPS);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);
    }
    for (int i = 0; i < TCT_STAGES; ++i) {
      mbar_init(&st_full[i], 4 + 1);   // the group's warps and the thread that announces the B slice's bytes
      mbar_init(&st_empty[i], 1);
    }
    *s_fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == TCT_BWARPS + 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                 "r"(TCT_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *s_tmem;

  const int first = blockIdx.x, stride = gridDim.x;
  const int n_my = first < nblocks ? (nblocks - first + stride - 1) / stride : 0;

  if (warp == TCT_BWARPS + 4) {
    // ---------------- producer: the next row block's values, column bytes and chunk ids ----------------
    int p_e0 = 0, p_e1 = 0, p_j0 = 0, p_nch = 0;
    auto prefetch = [&](int i) {
      const int b = first + i * stride;
      const int64_t r0 = (int64_t)b * TC_M;
      const int nr = (int)(r0 + TC_M < rows ? TC_M : rows - r0);
      p_e0 = rp[r0];
      p_e1 = rp[r0 + nr];
      p_j0 = chunk_off[b];
      p_nch = chunk_cnt[b];
    };
    auto stage_csr = [&](int i) -> bool {
      const int cs = i % TCT_CSR;
      if (!__all_sync(0xffffffffu, mbar_wait(&csr_empty[cs], (uint32_t)(((i / TCT_CSR) & 1) ^ 1), lim))) return false;
      const int e0 = p_e0, e1 = p_e1, j0 = p_j0, nch = p_nch;
      if (i + 1 < n_my) prefetch(i + 1);
      if (elect_one()) {
        // the block's scalars travel with its data: the builders load nothing from global memory
        int* hdr = s_hdr + cs * 4;
        hdr[0] = e0;
        hdr[1] = e1;
        hdr[2] = nch;
        hdr[3] = j0;
        const int a0 = e0 & ~15;
        const bool staged = (e1 - a0) <= TC_CAP;
        __nv_bfloat16* dv = s_val + cs * TCT_CAPB;
        uint8_t* dk = s_k + cs * TCT_CAPB;
        uint32_t cnt = 0;
        if (staged) {
          int a1 = (e1 + 15) & ~15;
          const int nnz16 = (int)(nnz & ~(int64_t)15);
          if (a1 > nnz16) a1 = nnz16;
          if (a1 < a0) a1 = a0;
          cnt = (uint32_t)(a1 - a0);
          for (int e = a1 > e0 ? a1 : e0; e < e1; ++e) {  // past the arrays' last full group of 16
            dv[e - a0] = val[e];
            dk[e - a0] = kcol[e];
          }
        }
        const uint32_t nrun = (uint32_t)(nch < TCT_RUNCH ? nch : TCT_RUNCH);
        mbar_expect_tx(&csr_full[cs], cnt * 3u + nrun * (TC_M * 4u));
        if (cnt) {
          bulk_g2s(dv, val + a0, cnt * 2u, &csr_full[cs]);
          bulk_g2s(dk, kcol + a0, cnt, &csr_full[cs]);
        }
        if (nrun) bulk_g2s(s_runs + cs * (TCT_RUNCH * TC_M), runs + (size_t)j0 * TC_M, nrun * (TC_M * 4u), &csr_full[cs]);
      }
      __syncwarp();
      return true;
    };
    bool ok = true;
    if (n_my > 0) {
      prefetch(0);
      ok = stage_csr(0);
    }
    for (int i = 0; i < n_my && ok; ++i)
      if (i + 1 < n_my) ok = stage_csr(i + 1);
    if (!ok) *s_fail = 1;
  } else if (warp == TCT_BWARPS + 5) {
    // ---------------- MMA: the whole warp walks the loop, one elected lane issues ----------------
    const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(n >> 3) << 17) |
                           ((uint32_t)(TC_M >> 4) << 24);
    bool ok = true, ready = false;
    int st = 0;
    uint32_t ph = 0;
    const uint64_t bd0 = umma_desc(smem_u32(sB), TC_BBLK, 1024, 2);
    const uint32_t b_hi = (uint32_t)(bd0 >> 32), b_lo0 = (uint32_t)bd0;
    const uint32_t b_step = (uint32_t)b_stage_bytes >> 4;
    int nch_next = n_my > 0 ? chunk_cnt[first] : 0;
    for (int i = 0; i < n_my && ok; ++i) {
      const int nch = nch_next;  // fetched one block ahead: no global latency between blocks
      if (i + 1 < n_my) nch_next = chunk_cnt[first + (i + 1) * stride];
      if (!__all_sync(0xffffffffu, mbar_wait(&acc_empty[i & 1], (uint32_t)(((i >> 1) & 1) ^ 1), lim))) {
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t d = tmem + (uint32_t)(i & 1) * acc_cols;
      uint32_t first_acc = 0u;  // the block's first MMA overwrites the accumulator
      for (int j = 0; j < nch; ++j) {
        if (!ready && !__all_sync(0xffffffffu, mbar_spin(&st_full[st], ph, lim))) {
          ok = false;
          break;
        }
        // the builders' tcgen05.st have completed (their wait::st, then fence::before_thread_sync)
        // before they arrive on the barrier; this fence orders the MMAs after the wait on it
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_t = tmem + a_col0 + (uint32_t)st * 32u, b_lo = b_lo0 + (uint32_t)st * b_step;
        // The tensor core takes the next MMA while it works on one, but its queue is short: what the
        // warp does between a chunk's last MMA and the next chunk's first one is time the core
        // idles.  So the next stage's barrier is tested before this chunk's MMAs go out, the vote on
        // the answer sits before the last MMA, and only the commit and the loop's branch follow it.
        const int st_n = st + 1 == TCT_STAGES ? 0 : st + 1;
        const uint32_t ph_n = st + 1 == TCT_STAGES ? ph ^ 1u : ph;
        const bool early = mbar_test(&st_full[st_n], ph_n);
        if (elect_one()) {
          umma_bf16_ts(d, a_t, b_lo, b_hi, idesc, first_acc);
          umma_bf16_ts(d, a_t + 8u, b_lo + 128u, b_hi, idesc, 1u);
          umma_bf16_ts(d, a_t + 16u, b_lo + 256u, b_hi, idesc, 1u);
        }
        ready = __all_sync(0xffffffffu, early);
        if (elect_one()) {
          umma_bf16_ts(d, a_t + 24u, b_lo + 384u, b_hi, idesc, 1u);
          umma_commit(&st_empty[st]);
        }
        first_acc = 1u;
        st = st_n;
        ph = ph_n;
      }
      if (ok && elect_one()) umma_commit(&acc_full[i & 1]);
      __syncwarp();
    }
    if (!ok) *s_fail = 1;
  } else if (warp >= TCT_BWARPS + 6) {
    // ---------------- B loaders: warp g asks for the slices of the chunks g modulo TCT_GROUPS ----------------
    // (into ring stages g and g + TCT_GROUPS, as soon as the stage is free: issuing a copy keeps a
    // warp busy for some hundred cycles, which the builders' chain of a chunk should not carry).
    // Chunk ids come from global memory, one chunk of the warp ahead of their use.
    const int g = warp - (TCT_BWARPS + 6);
    bool ok = true;
    int sa = g;
    uint32_t ph = 0;
    uint32_t cnum0 = 0, mine = (uint32_t)g;
    int n_nch = 0, n_j0 = 0;
    auto fetch = [&](int i) {
      const int b = first + i * stride;
      n_nch = chunk_cnt[b];
      n_j0 = chunk_off[b];
    };
    if (n_my > 0) fetch(0);
    int id_next = 0;
    bool have_next = false;
    for (int i = 0; i < n_my && ok; ++i) {
      const int nch = n_nch, j0 = n_j0;
      if (i + 1 < n_my) fetch(i + 1);
      for (int j = (int)(mine - cnum0); j < nch; j += TCT_GROUPS, mine += (uint32_t)TCT_GROUPS) {
        const int id = have_next ? id_next : (int)ldg_here_u32(chunk_list + j0 + j);
        have_next = false;
        {
          const int j2 = j + TCT_GROUPS;
          if (j2 < nch) {
            id_next = (int)ldg_here_u32(chunk_list + j0 + j2);
            have_next = true;
          } else if (i + 1 < n_my && j2 - nch < n_nch) {
            id_next = (int)ldg_here_u32(chunk_list + n_j0 + j2 - nch);
            have_next = true;
          }
        }
        const int brow = id * TC_KC;
        // (a warp that polls flat out costs shared-memory bandwidth, which is what bounds this kernel)
        if (!__all_sync(0xffffffffu, mbar_wait_parked(&st_empty[sa], ph ^ 1u, lim))) {
          ok = false;
          break;
        }
        if (elect_one()) {
          mbar_expect_tx(&st_full[sa], (uint32_t)b_stage_bytes);
          if (drop_copies) {
          } else if (one_box) {
            tma_load_3d(sB + (size_t)sa * b_stage_bytes, &tmB, 0, brow, 0, &st_full[sa]);
          } else {
            for (int q = 0; q < nblk; ++q)
              tma_load_2d(sB + (size_t)sa * b_stage_bytes + q * TC_BBLK, &tmB, q * 64, brow, &st_full[sa]);
          }
        }
        __syncwarp();
        sa += TCT_GROUPS;
        if (sa >= TCT_STAGES) {
          sa -= TCT_STAGES;
          ph ^= 1u;
        }
      }
      cnum0 += (uint32_t)nch;
    }
    if (!ok) *s_fail = 1;
  } else if (warp < TCT_BWARPS) {
    // ---------------- builders ----------------
    // Group g takes the chunks whose running number (over all row blocks of this CTA) is g modulo
    // TCT_GROUPS, into ring stages g and g + TCT_GROUPS in turn.  Votes keep a warp's lanes
    // together (tcgen05.st is a warp-wide instruction); a warp whose wait ran out keeps walking the
    // loop without waiting or storing.
    bool ok = true;
    const int grp = warp >> 2;
    const int gt = tid - grp * 128;            // row of the block = tensor-memory lane
    const uint32_t priv = smem_u32(sP + grp * TCT_PRIV + gt * 128);
    const uint32_t swz = (uint32_t)(gt & 7);   // 16-byte pieces of a line are permuted by the row: lines of
                                               // eight neighbouring rows read as one conflict-free access
    const uint32_t t_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16) + a_col0;
    int sa = grp;
    uint32_t ph = 0;
    uint32_t cnum0 = 0;              // running number of the block's first chunk
    uint32_t mine = (uint32_t)grp;   // running number of the group's next chunk
    for (int i = 0; i < n_my; ++i) {
      const int cs = i % TCT_CSR;
      ok = __all_sync(0xffffffffu, mbar_wait_parked(&csr_full[cs], (uint32_t)((i / TCT_CSR) & 1), lim));
      if (!ok) break;   // the other roles then run into their own limits
      const int* hdr = s_hdr + cs * 4;
      const int e0 = hdr[0], e1 = hdr[1], nch = hdr[2], j0 = hdr[3];
      const int a0 = e0 & ~15;
      const bool staged = (e1 - a0) <= TC_CAP;
      const __nv_bfloat16* __restrict__ pv = staged ? s_val + cs * TCT_CAPB : val + a0;   // by offset in the slice
      const uint8_t* __restrict__ pk = staged ? s_k + cs * TCT_CAPB : kcol + a0;
      const uint32_t* prun = s_runs + cs * (TCT_RUNCH * TC_M) + gt;
      for (int j = (int)(mine - cnum0); j < nch; j += TCT_GROUPS, mine += (uint32_t)TCT_GROUPS) {
        const uint32_t word = j < TCT_RUNCH ? prun[j * TC_M] : ldg_here_u32(runs + (size_t)(j0 + j) * TC_M + gt);
        ok = __all_sync(0xffffffffu, mbar_wait_parked(&st_empty[sa], ph ^ 1u, lim));
        if (!ok) break;
        {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          // The first four entries of the run are read side by side (all loads issued before the first
          // store: a run of a stencil matrix has at most three), longer runs go on in a loop.
          const int start = (int)(word >> 7), cnt = (int)(word & 127u);
          uint32_t off[4];
          uint16_t vv[4];
          uint32_t touched = 0u;   // the 16-byte pieces of the line that hold an entry: only those are read back
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t k = e < cnt ? pk[start + e] : 0u;
            vv[e] = e < cnt ? __bfloat16_as_ushort(pv[start + e]) : (uint16_t)0;
            off[e] = priv + (((k >> 3) ^ swz) << 4) + ((k & 7u) << 1);
            if (e < cnt) touched |= 1u << (k >> 3);
          }
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (e < cnt) sts_b16(off[e], vv[e]);
          for (int e = 4; e < cnt; ++e) {
            const uint32_t k = pk[start + e];
            touched |= 1u << (k >> 3);
            sts_b16(priv + (((k >> 3) ^ swz) << 4) + ((k & 7u) << 1), __bfloat16_as_ushort(pv[start + e]));
          }
          uint32_t a[32];
#pragma unroll
          for (int q = 0; q < 32; ++q) a[q] = 0u;
#pragma unroll
          for (uint32_t q = 0; q < 8; ++q)
            lds_v4_if(touched & (1u << q), priv + ((q ^ swz) << 4), a[4 * q], a[4 * q + 1], a[4 * q + 2], a[4 * q + 3]);
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (e < cnt) sts_b16(off[e], (uint16_t)0);
          for (int e = 4; e < cnt; ++e) {
            const uint32_t k = pk[start + e];
            sts_b16(priv + (((k >> 3) ^ swz) << 4) + ((k & 7u) << 1), (uint16_t)0);
          }
          __syncwarp();
          tmem_st32(t_lane + (uint32_t)sa * 32u, a);
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&st_full[sa]);
          }
        sa += TCT_GROUPS;
        if (sa >= TCT_STAGES) {
          sa -= TCT_STAGES;
          ph ^= 1u;
        }
      }
      if (!ok) break;
      cnum0 += (uint32_t)nch;
      __syncwarp();
      if (lane == 0) mbar_arrive(&csr_empty[cs]);
    }
    if (!ok) *s_fail = 1;
  } else {
    // ---------------- epilogue: warps 12-15 read tensor-memory lanes 32 * (warp mod 4) .. ----------------
    bool ok = true;
    int nch_next = n_my > 0 ? chunk_cnt[first] : 0;
    for (int i = 0; i < n_my && ok; ++i) {
      const int acc = i & 1;
      const int b = first + i * stride;
      const int64_t r0 = (int64_t)b * TC_M;
      const int nr = (int)(r0 + TC_M < rows ? TC_M : rows - r0);
      const int nch = nch_next;
      if (i + 1 < n_my) nch_next = chunk_cnt[first + (i + 1) * stride];
      if (!__all_sync(0xffffffffu, mbar_wait_parked(&acc_full[acc], (uint32_t)((i >> 1) & 1), lim))) {
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // tcgen05.ld hands lane l the 32 columns of row l; a per-warp 32 x 36 shared-memory tile turns
      // that around (16-byte accesses both ways, free of bank conflicts) so that a store instruction
      // writes four whole 128-byte rows of C.
      float* tr = s_tr + (warp - TCT_BWARPS) * (TCT_TRBYTES / 4);
      const int wrow0 = (warp - TCT_BWARPS) * 32;
      if (c_by_tma) {
        // beta = 0: the tile goes out by one TMA store per 32 x 32 block of C (128-byte swizzle: lane
        // l writes the 16-byte piece q of its row at position q ^ (l mod 8), free of bank conflicts;
        // rows past the matrix are clipped by the copy)
        const uint32_t trow = smem_u32(tr) + (uint32_t)lane * 128u;
        for (int cb = 0; cb < n; cb += 32) {
          uint32_t a[32];
          if (nch > 0) {
            tmem_ld32(tmem + ((uint32_t)wrow0 << 16) + (uint32_t)acc * acc_cols + (uint32_t)cb, a);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          } else {
#pragma unroll
            for (int q = 0; q < 32; ++q) a[q] = 0u;
          }
          // the copy that read the tile last has to be through with it
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          __syncwarp();
#pragma unroll
          for (uint32_t q = 0; q < 8; ++q)
            asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(trow + ((q ^ (uint32_t)(lane & 7)) << 4)),
                         "f"(alpha * __uint_as_float(a[4 * q])), "f"(alpha * __uint_as_float(a[4 * q + 1])),
                         "f"(alpha * __uint_as_float(a[4 * q + 2])), "f"(alpha * __uint_as_float(a[4 * q + 3]))
                         : "memory");
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0 && wrow0 < nr) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(&tmC),
                         "r"(cb), "r"((int)(r0 + wrow0)), "r"(smem_u32(tr))
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        continue;
      }
      const int rmax = nr - wrow0 < 32 ? nr - wrow0 : 32;
      const int rsub = lane >> 3, c4 = (lane & 7) * 4;
      for (int cb = 0; cb < n; cb += 32) {
        uint32_t a[32];
        if (nch > 0) {
          tmem_ld32(tmem + ((uint32_t)wrow0 << 16) + (uint32_t)acc * acc_cols + (uint32_t)cb, a);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        } else {
#pragma unroll
          for (int q = 0; q < 32; ++q) a[q] = 0u;
        }
#pragma unroll
        for (int q = 0; q < 32; q += 4)
          *reinterpret_cast<float4*>(tr + lane * TCT_TRLD + q) =
              make_float4(alpha * __uint_as_float(a[q]), alpha * __uint_as_float(a[q + 1]),
                          alpha * __uint_as_float(a[q + 2]), alpha * __uint_as_float(a[q + 3]));
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rr = it * 4 + rsub;
          if (rr < rmax) {
            float4 o = *reinterpret_cast<const float4*>(tr + rr * TCT_TRLD + c4);
            float4* cp = reinterpret_cast<float4*>(C + (r0 + wrow0 + rr) * ldc + cb + c4);
            if (beta != 0.f) {
              const float4 c0 = *cp;
              o.x = fmaf(beta, c0.x, o.x);
              o.y = fmaf(beta, c0.y, o.y);
              o.z = fmaf(beta, c0.z, o.z);
              o.w = fmaf(beta, c0.w, o.w);
            }
            *cp = o;
          }
        }
        __syncwarp();
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
    }
    if (c_by_tma && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    if (!ok) *s_fail = 1;
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*s_fail) {
    if (tid == 0) atomicExch(err, 1);
    __nanosleep(1000000);  // let copies and MMAs still in flight retire before the memory goes away
  }
  if (warp == TCT_BWARPS + 5)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TCT_TMEM_COLS) : "memory");
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

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

alphasparseStatus_t build_plan(alphasparseHandle_t h, alphasparseSpMatDescr_t A, TcPlan* tp) {
  cudaStream_t st = h->stream;
  tp->blocks = (A->rows + TC_M - 1) / TC_M;
  if (tp->blocks == 0 || tp->blocks > INT_MAX) return ALPHA_SPARSE_STATUS_SUCCESS;
  const int nb = (int)tp->blocks;
  int32_t *padded = nullptr, *cnt_scan = nullptr;
  int* flags = nullptr;
  void* tmp = nullptr;
  auto cleanup = [&]() {
    cudaFree(padded);
    cudaFree(cnt_scan);
    cudaFree(flags);
    cudaFree(tmp);
  };
  ASP_CUDA(cudaMalloc(&tp->chunk_cnt, sizeof(int32_t) * (nb + 1)));
  ASP_CUDA(cudaMalloc(&tp->chunk_off, sizeof(int32_t) * (nb + 1)));
  if (cudaMalloc(&padded, sizeof(int32_t) * (nb + 1)) != cudaSuccess ||
      cudaMalloc(&cnt_scan, sizeof(int32_t) * (nb + 1)) != cudaSuccess ||
      cudaMalloc(&flags, 2 * sizeof(int)) != cudaSuccess) {
    cleanup();
    return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  }
  cudaMemsetAsync(flags, 0, 2 * sizeof(int), st);
  cudaMemsetAsync(tp->chunk_cnt, 0, sizeof(int32_t) * (nb + 1), st);
  cudaMemsetAsync(padded, 0, sizeof(int32_t) * (nb + 1), st);
  tc_chunks_kernel<false><<<(unsigned)nb, 256, 0, st>>>(A->const_row_data, A->const_col_data, A->rows,
                                                       tp->chunk_cnt, padded, nullptr, nullptr, flags);
  size_t tmp_bytes = 0;
  cub::DeviceScan::ExclusiveSum(nullptr, tmp_bytes, padded, tp->chunk_off, nb + 1, st);
  if (cudaMalloc(&tmp, tmp_bytes ? tmp_bytes : 16) != cudaSuccess) {
    cleanup();
    return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  }
  cub::DeviceScan::ExclusiveSum(tmp, tmp_bytes, padded, tp->chunk_off, nb + 1, st);
  cub::DeviceScan::ExclusiveSum(tmp, tmp_bytes, tp->chunk_cnt, cnt_scan, nb + 1, st);
  int hflags[2] = {0, 0};
  int32_t total_padded = 0, total = 0;
  cudaError_t e = cudaMemcpyAsync(hflags, flags, sizeof hflags, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaMemcpyAsync(&total_padded, tp->chunk_off + nb, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaMemcpyAsync(&total, cnt_scan + nb, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  impl(h)->launches += 3;
  if (e != cudaSuccess) {
    cleanup();
    return status_of(e);
  }
  tp->total_chunks = total;
  tp->usable = hflags[0] == 0 && hflags[1] == 0;
  if (tp->usable && total_padded > 0) {
    if (cudaMalloc(&tp->chunk_list, sizeof(int32_t) * (size_t)total_padded) != cudaSuccess) {
      cleanup();
      return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    cudaMemsetAsync(tp->chunk_list, 0, sizeof(int32_t) * (size_t)total_padded, st);
    tc_chunks_kernel<true><<<(unsigned)nb, 256, 0, st>>>(A->const_row_data, A->const_col_data, A->rows, nullptr,
                                                        nullptr, tp->chunk_off, tp->chunk_list, nullptr);
    impl(h)->launches++;
    e = cudaStreamSynchronize(st);
  }
  // the largest chunk count of a block decides whether chunk ids fit the persistent kernel's staging
  if (e == cudaSuccess && tp->usable) {
    size_t rb = 0;
    cub::DeviceReduce::Max(nullptr, rb, tp->chunk_cnt, cnt_scan, nb, st);
    if (rb <= tmp_bytes || (cudaFree(tmp), tmp = nullptr, cudaMalloc(&tmp, rb) == cudaSuccess)) {
      cub::DeviceReduce::Max(tmp, rb, tp->chunk_cnt, cnt_scan, nb, st);
      int32_t m = 0;
      e = cudaMemcpyAsync(&m, cnt_scan, sizeof m, cudaMemcpyDeviceToHost, st);
      if (e == cudaSuccess) e = cudaStreamSynchronize(st);
      tp->max_chunks = m;
    }
  }
  cleanup();
  return status_of(e);
}

// The scatter list of the kernels that build A tiles in shared memory: count per chunk, scan,
// fill.  Built when one of those kernels is first chosen (the default kernel keeps A in tensor
// memory and needs the run list instead).
alphasparseStatus_t build_scatter(alphasparseHandle_t h, alphasparseSpMatDescr_t A, TcPlan* tp) {
  tp->scatter_tried = true;
  if (!tp->usable || !tp->chunk_list || A->nnz == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  cudaStream_t st = h->stream;
  const int nb = (int)tp->blocks;
  int32_t total_padded = 0;
  cudaError_t e = cudaMemcpyAsync(&total_padded, tp->chunk_off + nb, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return status_of(e);
  if (total_padded <= 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  int32_t* ent_cnt = nullptr;
  void* tmp = nullptr;
  size_t sb_bytes = 0;
  cub::DeviceScan::ExclusiveSum(nullptr, sb_bytes, ent_cnt, tp->chunk_ent, total_padded, st);
  if (cudaMalloc(&ent_cnt, sizeof(int32_t) * (size_t)total_padded) != cudaSuccess ||
      cudaMalloc(&tp->chunk_ent, sizeof(int32_t) * (size_t)total_padded) != cudaSuccess ||
      cudaMalloc(&tp->scatter, sizeof(uint32_t) * (size_t)A->nnz) != cudaSuccess ||
      cudaMalloc(&tmp, sb_bytes ? sb_bytes : 16) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(ent_cnt);
    cudaFree(tmp);
    cudaFree(tp->chunk_ent);
    cudaFree(tp->scatter);
    tp->chunk_ent = nullptr;
    tp->scatter = nullptr;
    return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  }
  cudaMemsetAsync(ent_cnt, 0, sizeof(int32_t) * (size_t)total_padded, st);
  tc_scatter_kernel<false><<<(unsigned)nb, 128, 0, st>>>(A->const_row_data, A->const_col_data, A->rows, tp->chunk_off,
                                                        tp->chunk_cnt, tp->chunk_list, ent_cnt, nullptr, nullptr);
  cub::DeviceScan::ExclusiveSum(tmp, sb_bytes, ent_cnt, tp->chunk_ent, total_padded, st);
  tc_scatter_kernel<true><<<(unsigned)nb, 128, 0, st>>>(A->const_row_data, A->const_col_data, A->rows, tp->chunk_off,
                                                       tp->chunk_cnt, tp->chunk_list, nullptr, tp->chunk_ent, tp->scatter);
  impl(h)->launches += 3;
  e = cudaStreamSynchronize(st);
  cudaFree(ent_cnt);
  cudaFree(tmp);
  return status_of(e);
}

// The per-row run list and the column bytes of the kernel that keeps A in tensor memory.  Left
// out (runs stays null, the shared-memory kernel runs) when the device memory is not there.
alphasparseStatus_t build_runs(alphasparseHandle_t h, alphasparseSpMatDescr_t A, TcPlan* tp) {
  tp->runs_tried = true;
  if (!tp->usable || !tp->chunk_list || A->nnz == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
  cudaStream_t st = h->stream;
  const int nb = (int)tp->blocks;
  int32_t total_padded = 0;
  cudaError_t e = cudaMemcpyAsync(&total_padded, tp->chunk_off + nb, sizeof(int32_t), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return status_of(e);
  const size_t words = (size_t)total_padded * TC_M;
  if (cudaMalloc(&tp->runs, words * sizeof(uint32_t)) != cudaSuccess ||
      cudaMalloc(&tp->kcol, (size_t)A->nnz + 16) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(tp->runs);
    cudaFree(tp->kcol);
    tp->runs = nullptr;
    tp->kcol = nullptr;
    return ALPHA_SPARSE_STATUS_SUCCESS;
  }
  cudaMemsetAsync(tp->runs, 0, words * sizeof(uint32_t), st);
  tc_runs_kernel<<<(unsigned)nb, 128, 0, st>>>(A->const_row_data, A->const_col_data, A->rows, tp->chunk_off,
                                               tp->chunk_cnt, tp->chunk_list, tp->runs);
  int64_t g = (A->nnz + 255) / 256;
  const int64_t gmax = (int64_t)impl(h)->sm_count * 16;
  if (g > gmax) g = gmax;
  tc_kcol_kernel<<<(unsigned)g, 256, 0, st>>>(A->const_col_data, A->nnz, tp->kcol);
  impl(h)->launches += 2;
  return status_of(cudaStreamSynchronize(st));
}

}  // namespace

void free_spmm_tc_plan(void* p) {
  TcPlan* tp = reinterpret_cast<TcPlan*>(p);
  if (!tp) return;
  cudaFree(tp->chunk_off);
  cudaFree(tp->chunk_cnt);
  cudaFree(tp->chunk_list);
  cudaFree(tp->chunk_ent);
  cudaFree(tp->scatter);
  cudaFree(tp->runs);
  cudaFree(tp->kcol);
  delete tp;
}

// Shapes and types the kernel handles; the density test needs the plan and is done in spmm_tc_run.
bool spmm_tc_applicable(alphasparseSpMatDescr_t A, alphasparseDnMatDescr_t B, alphasparseDnMatDescr_t C) {
  const int64_t n = C->cols;
  return A->data_type == ALPHA_R_16BF && B->data_type == ALPHA_R_16BF && C->data_type == ALPHA_R_32F &&
         A->row_type == ALPHA_SPARSE_INDEXTYPE_I32 && n >= 64 && n <= 256 && n % 64 == 0 && B->ld % 8 == 0 &&
         C->ld % 4 == 0 && aligned(B->values, 16) && aligned(C->values, 16) && aligned(A->const_col_data, 16) &&
         aligned(A->const_val_data, 16) && A->cols < (int64_t(1) << 31);
}

alphasparseStatus_t spmm_tc_run(alphasparseHandle_t h, alphasparseSpMatDescr_t A, alphasparseDnMatDescr_t B,
                                alphasparseDnMatDescr_t C, float alpha, float beta, bool preprocess_only) {
  Plan* p = plan_of(A);
  if (!p) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
  if (!p->spmm_tc) {
    TcPlan* tp = new (std::nothrow) TcPlan();
    if (!tp) return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    alphasparseStatus_t s = build_plan(h, A, tp);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) {
      free_spmm_tc_plan(tp);
      return s;
    }
    p->spmm_tc = tp;
  }
  TcPlan* tp = reinterpret_cast<TcPlan*>(p->spmm_tc);
  const int n = (int)C->cols;
  // Dense enough: the MMA work over all non-empty chunks (at the sustained bf16 rate) must stay
  // within three times the time HBM needs for the algorithmic bytes.
  const double t_mma = (double)tp->total_chunks * TC_M * TC_KC * n * 2.0 / impl(h)->bf16_flops;
  const double t_hbm = ((double)A->nnz * 6.0 + (double)A->cols * n * 2.0 + (double)A->rows * n * 4.0) / impl(h)->hbm_bytes;
  if (!tp->usable || t_mma > 3.0 * t_hbm) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  // N = 256 runs the tensor-memory kernel as two passes over the matrix, 128 columns of B and C each
  // (A's lists are read twice, B and C once: measured faster than one pass with A in shared memory).
  const bool want_tmem = env_int("ASP_TC_A_TMEM", 1) && env_int("ASP_TC_PERSISTENT", 1) &&
                         p->max_block_nnz + 16 < (int64_t(1) << 25);
  if (want_tmem && !tp->runs_tried) {
    alphasparseStatus_t s = build_runs(h, A, tp);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  }
  if (!(want_tmem && tp->runs && tp->kcol) && env_int("ASP_TC_PERSISTENT", 1) && !tp->scatter_tried) {
    alphasparseStatus_t s = build_scatter(h, A, tp);   // the kernel with A tiles in shared memory will run
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  }
  if (preprocess_only || A->rows == 0) return ALPHA_SPARSE_STATUS_SUCCESS;

  EncodeTiledFn enc = encode_fn();
  if (!enc) return ALPHA_SPARSE_STATUS_INTERNAL_ERROR;
  CUtensorMap tm;
  const cuuint64_t dims[2] = {(cuuint64_t)n, (cuuint64_t)B->rows};
  const cuuint64_t strides[1] = {(cuuint64_t)B->ld * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)TC_KC};
  const cuuint32_t estr[2] = {1, 1};
  if (enc(&tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B->values, dims, strides, box, estr,
          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return ALPHA_SPARSE_STATUS_INVALID_VALUE;

  const size_t b_stage = (size_t)(n / 64) * TC_BBLK;
  if (want_tmem && tp->runs && tp->kcol) {
    const int np_max = n > 128 ? 128 : n;   // columns of a pass: 128, and what is left (N = 192: 128 + 64)
    const size_t b_stage_p = (size_t)(np_max / 64) * TC_BBLK;
    const size_t smem = 1024 + TCT_STAGES * b_stage_p + TCT_GROUPS * (size_t)TCT_PRIV + TCT_CSR * (size_t)TCT_CAPB * 3 +
                        TCT_CSR * (size_t)TCT_RUNCH * TC_M * 4 + TCT_CSR * 16 + 4 * TCT_TRBYTES +
                        (12 + 2 * TCT_STAGES) * 8 + 16;
    const size_t smem_max = impl(h)->smem_optin ? impl(h)->smem_optin : 232448;
    if (smem <= smem_max) {
      static size_t attr_t[64] = {0};
      size_t& set_t = attr_t[h->device & 63];
      if (smem > set_t) {
        ASP_CUDA(cudaFuncSetAttribute(spmm_tc_tmem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        set_t = smem;
      }
      int64_t g = impl(h)->sm_count;
      if (g > tp->blocks) g = tp->blocks;
      for (int c0 = 0; c0 < n; c0 += np_max) {
        const int np = n - c0 < np_max ? n - c0 : np_max;
        void* bp = reinterpret_cast<__nv_bfloat16*>(B->values) + c0;
        float* cp = reinterpret_cast<float*>(C->values) + c0;
        CUtensorMap tm3;
        const cuuint64_t dims3[3] = {64, (cuuint64_t)B->rows, (cuuint64_t)(np / 64)};
        const cuuint64_t strides3[2] = {(cuuint64_t)B->ld * 2, 128};
        const cuuint32_t box3[3] = {64, (cuuint32_t)TC_KC, (cuuint32_t)(np / 64)};
        const cuuint32_t estr3[3] = {1, 1, 1};
        const int one_box = np > 64 &&
                            enc(&tm3, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, bp, dims3, strides3, box3, estr3,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
        CUtensorMap tm2 = tm;   // a 64-column pass: one 2-D box per chunk
        if (!one_box) {
          const cuuint64_t dims2[2] = {(cuuint64_t)np, (cuuint64_t)B->rows};
          const cuuint64_t strides2[1] = {(cuuint64_t)B->ld * 2};
          const cuuint32_t box2[2] = {64, (cuuint32_t)TC_KC};
          if (np > 64 || enc(&tm2, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, bp, dims2, strides2, box2, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return ALPHA_SPARSE_STATUS_INVALID_VALUE;
        }
        // C leaves by TMA stores of 32 x 32 blocks when it is only written (beta = 0)
        CUtensorMap tmc = tm;
        const cuuint64_t dimsc[2] = {(cuuint64_t)np, (cuuint64_t)A->rows};
        const cuuint64_t stridesc[1] = {(cuuint64_t)C->ld * 4};
        const cuuint32_t boxc[2] = {32, 32};
        const int c_by_tma = beta == 0.f && env_int("ASP_TC_C_TMA", 1) &&
                             enc(&tmc, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, cp, dimsc, stridesc, boxc, estr,
                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
        spmm_tc_tmem_kernel<<<(unsigned)g, TCT_THREADS, smem, h->stream>>>(
            one_box ? tm3 : tm2, tmc, c_by_tma, A->const_row_data, reinterpret_cast<const __nv_bfloat16*>(A->const_val_data),
            cp, C->ld, alpha, beta, A->rows, A->nnz, np, (int)tp->blocks, tp->chunk_off, tp->chunk_cnt, tp->chunk_list,
            tp->runs, tp->kcol, one_box, p->wait_cfg, p->dev_err);
        impl(h)->launches++;
      }
      p->last_spmm = "tcgen05";
      return status_of(cudaGetLastError());
    }
  }
  if (env_int("ASP_TC_PERSISTENT", 1) && tp->max_chunks <= TC_MAXCH && tp->scatter &&
      p->max_block_nnz + 8 < (int64_t)(1u << (32 - TC_SRC_SHIFT))) {
    // one CTA per SM; whatever shared memory the fixed parts leave goes to B stages
    const size_t fixed = TCP_CSR * (size_t)(TC_CAP + 8) * 6 + TCP_CSR * TC_MAXCH * 8 + 4 * 32 * 33 * 4 + 16 + 1024 + 1024;
    const size_t smem_max = impl(h)->smem_optin ? impl(h)->smem_optin : 232448;
    int sb = (int)((smem_max - fixed) / (b_stage + TC_A_BYTES));
    // Ring depth 8, 4 (what fits at N = 128) or 2 (N = 256): the kernel's waits by parity need a
    // stage to come back to the same builder group (depth a multiple or a divisor of the number of
    // groups) and, for two MMA issuers, an even depth.
    int cap = env_int("ASP_TC_STAGES", 8);
    if (sb > cap) sb = cap;
    sb = sb >= 8 ? 8 : (sb >= 4 ? 4 : (sb >= 2 ? 2 : 0));
    if (sb >= 2) {
      const size_t smem = fixed + (size_t)sb * (b_stage + TC_A_BYTES);
      static size_t attr_p[64] = {0};  // the attribute belongs to the device: remembered per device
      size_t& set_p = attr_p[h->device & 63];
      if (smem > set_p) {
        ASP_CUDA(cudaFuncSetAttribute(spmm_tc_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        set_p = smem;
      }
      int64_t g = impl(h)->sm_count;
      if (g > tp->blocks) g = tp->blocks;
      // B as [column block of 64][row][64 columns]: one box {64, 64 rows, all column blocks} lands in
      // shared memory as the column blocks' 8 KB tiles one after the other, what the MMA descriptor expects.
      CUtensorMap tm3;
      const cuuint64_t dims3[3] = {64, (cuuint64_t)B->rows, (cuuint64_t)(n / 64)};
      const cuuint64_t strides3[2] = {(cuuint64_t)B->ld * 2, 128};
      const cuuint32_t box3[3] = {64, (cuuint32_t)TC_KC, (cuuint32_t)(n / 64)};
      const cuuint32_t estr3[3] = {1, 1, 1};
      const int one_box = env_int("ASP_TC_ONE_BOX", 1) && n > 64 &&
                          enc(&tm3, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, B->values, dims3, strides3, box3, estr3,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
      spmm_tc_persistent_kernel<<<(unsigned)g, TCP_THREADS, smem, h->stream>>>(
          one_box ? tm3 : tm, A->const_row_data, A->const_col_data, reinterpret_cast<const __nv_bfloat16*>(A->const_val_data),
          reinterpret_cast<float*>(C->values), C->ld, alpha, beta, A->rows, A->nnz, n, (int)tp->blocks, sb,
          tp->chunk_off, tp->chunk_cnt, tp->chunk_list, tp->chunk_ent, tp->scatter, one_box,
          env_int("ASP_TC_ISSUERS", 2), p->dev_err);
      p->last_spmm = "tcgen05-smem";
      impl(h)->launches++;
      return status_of(cudaGetLastError());
    }
  }
  const size_t smem = 2 * TC_A_BYTES + TC_BSTAGES * b_stage + (TC_CAP + 8) * 6 + TC_MAXCH * 4 + 128 + 1024;
  static size_t attr_bytes[64] = {0};
  size_t& set_b = attr_bytes[h->device & 63];
  if (smem > set_b) {
    ASP_CUDA(cudaFuncSetAttribute(spmm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    set_b = smem;
  }
  spmm_tc_kernel<<<(unsigned)tp->blocks, TC_THREADS, smem, h->stream>>>(
      tm, A->const_row_data, A->const_col_data, reinterpret_cast<const __nv_bfloat16*>(A->const_val_data),
      reinterpret_cast<float*>(C->values), C->ld, alpha, beta, A->rows, A->nnz, n, tp->chunk_off, tp->chunk_cnt,
      tp->chunk_list, p->dev_err);
  p->last_spmm = "tcgen05-simple";
  impl(h)->launches++;
  return status_of(cudaGetLastError());
}

}  // namespace asp
