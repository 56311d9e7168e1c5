// Multi-GPU SpMV behind the C ABI: one process (or thread) per GPU, each holding a contiguous,
// nnz-balanced row range of one CSR matrix with global column indices; y stays sharded by
// rows, x reaches a rank through NCCL before its kernels read it from local memory.
//
// The reference is single-device; what it offers for the split is the row partition rule of
// its CPU backend (hygon/util/partition.cpp:83-96, device twin
// cuda/kernel/level2/alphasparse_spmv_csr_row_partition.h:26-45), which
// alphasparseCsrPartitionRowsByNnz restates.  Everything in this file is an extension.
//
// Exchange modes
//   BROADCAST       x lives whole on one rank and is broadcast (ncclBroadcast) before the product.
//   ALLGATHER       x is sharded like y; every rank collects the whole vector.
//   WINDOW          x is sharded like y; a rank receives only x[min_col, max_col] of its rows by
//                   grouped ncclSend / ncclRecv: for a banded matrix its own part plus a halo.
//   WINDOW_OVERLAP  the same, with the rows that read only the rank's own part of x multiplied
//                   while the halo is in flight on a second, high-priority stream.
// ALLGATHER is WINDOW with the window forced to the whole vector, so one plan covers both.
//
// NCCL is looked up at run time (the copy the process has already loaded - e.g. the one a
// framework brought - else libnccl.so.2), so the library itself loads without NCCL and the
// single-GPU entry points never depend on it.  Kernels only read local memory; there are no
// device-side waits here.  A rank that fails is seen on the host: arguments that do not fit
// the communicator come back as a status before anything is enqueued, and after enqueuing
// ncclCommGetAsyncError is polled once (never a blocking wait).
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "asp_internal.h"

namespace asp {
namespace {

struct NcclApi {
  void* so = nullptr;
  decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
  decltype(&ncclCommInitRank) CommInitRank = nullptr;
  decltype(&ncclCommDestroy) CommDestroy = nullptr;
  decltype(&ncclCommCount) CommCount = nullptr;
  decltype(&ncclCommUserRank) CommUserRank = nullptr;
  decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
  decltype(&ncclGroupStart) GroupStart = nullptr;
  decltype(&ncclGroupEnd) GroupEnd = nullptr;
  decltype(&ncclSend) Send = nullptr;
  decltype(&ncclRecv) Recv = nullptr;
  decltype(&ncclBroadcast) Broadcast = nullptr;
  decltype(&ncclAllGather) AllGather = nullptr;
  bool ok = false;
};

NcclApi* nccl_api() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
      api.so = dlopen(n, RTLD_NOW | RTLD_NOLOAD);  // the copy already in the process, if any
      if (api.so) break;
    }
    for (int i = 0; !api.so && i < 2; ++i) api.so = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!api.so) return;
    bool all = true;
#define ASP_SYM(f)                                                   \
  api.f = reinterpret_cast<decltype(api.f)>(dlsym(api.so, "nccl" #f)); \
  all = all && api.f != nullptr
    ASP_SYM(GetUniqueId); ASP_SYM(CommInitRank); ASP_SYM(CommDestroy); ASP_SYM(CommCount);
    ASP_SYM(CommUserRank); ASP_SYM(CommGetAsyncError); ASP_SYM(GroupStart); ASP_SYM(GroupEnd);
    ASP_SYM(Send); ASP_SYM(Recv); ASP_SYM(Broadcast); ASP_SYM(AllGather);
#undef ASP_SYM
    api.ok = all;
  });
  return api.ok ? &api : nullptr;
}

inline alphasparseStatus_t nccl_status(ncclResult_t r) {
  switch (r) {
    case ncclSuccess:
    case ncclInProgress: return ALPHA_SPARSE_STATUS_SUCCESS;
    case ncclInvalidArgument:
    case ncclInvalidUsage: return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    case ncclUnhandledCudaError:
    case ncclSystemError:
    case ncclRemoteError: return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    default: return ALPHA_SPARSE_STATUS_INTERNAL_ERROR;
  }
}
#define ASP_NCCL(call)                                               \
  do {                                                               \
    ncclResult_t r_ = (call);                                        \
    if (r_ != ncclSuccess && r_ != ncclInProgress) return nccl_status(r_); \
  } while (0)

}  // namespace

struct Seg {
  int peer;
  int64_t a, b;  // x[a, b), global element indices
};

// One of the up to three row ranges a shard is cut into for the overlapped mode.
struct Part {
  int64_t a = 0, b = 0;  // local rows [a, b)
  void* rp = nullptr;    // rebased row offsets (device, owned)
  alphasparseSpMatDescr_t d = nullptr;
};

}  // namespace asp

struct alphasparseMg {
  alphasparseHandle_t h = nullptr;
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
  cudaStream_t comm_stream = nullptr;
  cudaEvent_t ev_ready = nullptr, ev_halo = nullptr;
  // the shard
  alphasparseSpMatDescr_t A = nullptr;  // the caller's descriptor (not owned)
  alphasparseMgExchange_t mode = ALPHASPARSE_MG_X_WINDOW;
  int root = 0;
  std::vector<int64_t> x_bounds;  // world + 1: rank p owns x[x_bounds[p], x_bounds[p+1])
  std::vector<int64_t> windows;   // 2 * world: rank p needs x[windows[2p], windows[2p+1])
  std::vector<asp::Seg> sends, recvs;
  int64_t lo = 0, hi = 0;         // this rank's window
  void* window = nullptr;         // device, (hi - lo) elements (BROADCAST on a non-root rank: the whole x)
  size_t es = 0;
  ncclDataType_t nt = ncclFloat32;
  alphasparseDnVecDescr_t xd = nullptr;  // x as a windowed vector over `window`
  int64_t i0 = 0, i1 = 0;         // interior rows [i0, i1)
  std::vector<asp::Part> parts;   // interior first
  int64_t bytes_received = 0;
};

namespace asp {
using Mg = ::alphasparseMg;
namespace {

void free_shard(Mg* m) {
  for (Part& p : m->parts) {
    if (p.d) alphasparseDestroySpMat(p.d);
    cudaFree(p.rp);
  }
  m->parts.clear();
  if (m->xd) alphasparseDestroyDnVec(m->xd);
  m->xd = nullptr;
  cudaFree(m->window);
  m->window = nullptr;
  m->sends.clear();
  m->recvs.clear();
  m->A = nullptr;
}

// Rows all of whose columns lie in [own_lo, own_hi) read nothing another rank owns.  First pass
// (from = 0, want_inside = true): the first such row.  Second pass (from = that row, want_inside =
// false): the first later row that does need a halo.  out starts at rows.
template <typename OffT>
__global__ void __launch_bounds__(256) first_row_kernel(const OffT* __restrict__ rp,
                                                        const int32_t* __restrict__ col, int64_t rows,
                                                        int64_t own_lo, int64_t own_hi, int64_t from,
                                                        bool want_inside,
                                                        unsigned long long* __restrict__ out) {
  unsigned long long best = ~0ull;
  for (int64_t r = from + blockIdx.x * (int64_t)blockDim.x + threadIdx.x; r < rows;
       r += (int64_t)gridDim.x * blockDim.x) {
    bool inside = true;
    for (int64_t k = (int64_t)rp[r]; k < (int64_t)rp[r + 1]; ++k) {
      const int64_t c = col[k];
      inside = inside && c >= own_lo && c < own_hi;
    }
    if (inside == want_inside) {
      best = (unsigned long long)r;
      break;  // rows ascend along a thread's stride: its first hit is its smallest
    }
  }
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long w = __shfl_xor_sync(0xffffffffu, best, o);
    if (w < best) best = w;
  }
  if ((threadIdx.x & 31) == 0 && best != ~0ull) atomicMin(out, best);
}

alphasparseStatus_t read_offset(const void* rp, bool o64, int64_t i, cudaStream_t st, int64_t* out) {
  if (o64) {
    ASP_CUDA(cudaMemcpyAsync(out, (const int64_t*)rp + i, 8, cudaMemcpyDeviceToHost, st));
    ASP_CUDA(cudaStreamSynchronize(st));
  } else {
    int32_t v = 0;
    ASP_CUDA(cudaMemcpyAsync(&v, (const int32_t*)rp + i, 4, cudaMemcpyDeviceToHost, st));
    ASP_CUDA(cudaStreamSynchronize(st));
    *out = v;
  }
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t enqueue_exchange(Mg* m, const NcclApi* nc, const char* x_own, int64_t o0,
                                     cudaStream_t st) {
  bool any = false;
  for (const Seg& s : m->recvs) any = any || s.peer != m->rank;
  for (const Seg& s : m->sends) any = any || s.peer != m->rank;
  if (!any) return ALPHA_SPARSE_STATUS_SUCCESS;
  ASP_NCCL(nc->GroupStart());
  ncclResult_t r = ncclSuccess;
  for (const Seg& s : m->recvs)
    if (s.peer != m->rank && r == ncclSuccess)
      r = nc->Recv((char*)m->window + (size_t)(s.a - m->lo) * m->es, (size_t)(s.b - s.a), m->nt, s.peer,
                   m->comm, st);
  for (const Seg& s : m->sends)
    if (s.peer != m->rank && r == ncclSuccess)
      r = nc->Send(x_own + (size_t)(s.a - o0) * m->es, (size_t)(s.b - s.a), m->nt, s.peer, m->comm, st);
  const ncclResult_t e = nc->GroupEnd();
  if (r != ncclSuccess) return nccl_status(r);
  ASP_NCCL(e);
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

}  // namespace
}  // namespace asp

using namespace asp;

extern "C" {

alphasparseStatus_t alphasparseMgExchangePlan(int world, int rank, const int64_t* own_bounds,
                                              const int64_t* windows, int64_t* sends, int* n_sends,
                                              int64_t* recvs, int* n_recvs) {
  if (!own_bounds || !windows || !sends || !n_sends || !recvs || !n_recvs)
    return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (world < 1 || rank < 0 || rank >= world) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  for (int p = 0; p < world; ++p)
    if (own_bounds[p + 1] < own_bounds[p]) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
  const int64_t my_lo = own_bounds[rank], my_hi = own_bounds[rank + 1];
  const int64_t w_lo = windows[2 * rank], w_hi = windows[2 * rank + 1];
  int ns = 0, nr = 0;
  for (int p = 0; p < world; ++p) {
    int64_t a = my_lo > windows[2 * p] ? my_lo : windows[2 * p];
    int64_t b = my_hi < windows[2 * p + 1] ? my_hi : windows[2 * p + 1];
    if (b > a) {
      sends[3 * ns] = p; sends[3 * ns + 1] = a; sends[3 * ns + 2] = b;
      ++ns;
    }
    a = w_lo > own_bounds[p] ? w_lo : own_bounds[p];
    b = w_hi < own_bounds[p + 1] ? w_hi : own_bounds[p + 1];
    if (b > a) {
      recvs[3 * nr] = p; recvs[3 * nr + 1] = a; recvs[3 * nr + 2] = b;
      ++nr;
    }
  }
  *n_sends = ns;
  *n_recvs = nr;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseMgGetUniqueId(void* id128) {
  if (!id128) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  const NcclApi* nc = nccl_api();
  if (!nc) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  ncclUniqueId id;
  ASP_NCCL(nc->GetUniqueId(&id));
  memcpy(id128, &id, sizeof id);
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseMgCommInitRank(void** comm, int world, const void* id128, int rank) {
  if (!comm || !id128) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (world < 1 || rank < 0 || rank >= world) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  const NcclApi* nc = nccl_api();
  if (!nc) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  ncclUniqueId id;
  memcpy(&id, id128, sizeof id);
  ncclComm_t c = nullptr;
  ASP_NCCL(nc->CommInitRank(&c, world, id, rank));
  *comm = c;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseMgCommDestroy(void* comm) {
  if (!comm) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  const NcclApi* nc = nccl_api();
  if (!nc) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  ASP_NCCL(nc->CommDestroy((ncclComm_t)comm));
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseMgCreate(alphasparseMgHandle_t* out, alphasparseHandle_t h, void* comm,
                                        int rank, int world) {
  if (!out) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  *out = nullptr;
  if (!h || !h->impl) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (world < 1 || rank < 0 || rank >= world) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (world > 1) {
    if (!comm) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    const NcclApi* nc = nccl_api();
    if (!nc) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    int n = 0, r = -1;
    ASP_NCCL(nc->CommCount((ncclComm_t)comm, &n));
    ASP_NCCL(nc->CommUserRank((ncclComm_t)comm, &r));
    if (n != world || r != rank) return ALPHA_SPARSE_STATUS_INVALID_VALUE;  // not this communicator's shape
  }
  Mg* m = new (std::nothrow) Mg();
  if (!m) return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  m->h = h;
  m->comm = (ncclComm_t)comm;
  m->rank = rank;
  m->world = world;
  int lo_prio = 0, hi_prio = 0;
  cudaError_t e = cudaDeviceGetStreamPriorityRange(&lo_prio, &hi_prio);
  // the few CTAs of a halo exchange must not queue behind a product that fills the GPU
  if (e == cudaSuccess)
    e = cudaStreamCreateWithPriority(&m->comm_stream, cudaStreamNonBlocking,
                                     env_int("ASP_MG_COMM_PRIORITY", 1) ? hi_prio : lo_prio);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&m->ev_ready, cudaEventDisableTiming);
  if (e == cudaSuccess) e = cudaEventCreateWithFlags(&m->ev_halo, cudaEventDisableTiming);
  if (e != cudaSuccess) {
    alphasparseMgDestroy(m);
    return asp::status_of(e);
  }
  *out = m;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseMgDestroy(alphasparseMgHandle_t m) {
  if (!m) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (m->comm_stream) cudaStreamSynchronize(m->comm_stream);
  free_shard(m);
  if (m->ev_ready) cudaEventDestroy(m->ev_ready);
  if (m->ev_halo) cudaEventDestroy(m->ev_halo);
  if (m->comm_stream) cudaStreamDestroy(m->comm_stream);
  delete m;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseMgSetShard(alphasparseMgHandle_t m, alphasparseSpMatDescr_t A,
                                          const int64_t* x_bounds, alphasparseMgExchange_t mode,
                                          int root) {
  if (!m) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!A) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  alphasparseStatus_t s = validate_csr(A);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  if (A->data_type != ALPHA_R_32F && A->data_type != ALPHA_R_64F) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (mode < ALPHASPARSE_MG_X_BROADCAST || mode > ALPHASPARSE_MG_X_WINDOW_OVERLAP)
    return ALPHA_SPARSE_STATUS_INVALID_VALUE;
  const int W = m->world;
  if (mode == ALPHASPARSE_MG_X_BROADCAST) {
    if (root < 0 || root >= W) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
  } else {
    if (!x_bounds) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    if (x_bounds[0] != 0 || x_bounds[W] != A->cols) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
    for (int p = 0; p < W; ++p)
      if (x_bounds[p + 1] < x_bounds[p]) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
  }
  alphasparseHandle_t h = m->h;
  cudaStream_t st = h->stream;
  ASP_CUDA(cudaStreamSynchronize(st));
  ASP_CUDA(cudaStreamSynchronize(m->comm_stream));
  free_shard(m);
  m->mode = mode;
  m->root = root;
  m->es = elem_size(A->data_type);
  m->nt = A->data_type == ALPHA_R_64F ? ncclFloat64 : ncclFloat32;
  if (!A->info) {
    s = analyse(h, A);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  }
  m->A = A;
  m->bytes_received = 0;
  m->i0 = m->i1 = 0;
  const NcclApi* nc = W > 1 ? nccl_api() : nullptr;
  if (W > 1 && !nc) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;

  if (mode == ALPHASPARSE_MG_X_BROADCAST) {
    m->lo = 0;
    m->hi = A->cols;
    if (W > 1 && m->rank != root && A->cols > 0) {
      ASP_CUDA(cudaMalloc(&m->window, (size_t)A->cols * m->es));
      m->bytes_received = A->cols * (int64_t)m->es;
    }
    return ALPHA_SPARSE_STATUS_SUCCESS;
  }

  m->x_bounds.assign(x_bounds, x_bounds + W + 1);
  const int64_t own_lo = x_bounds[m->rank], own_hi = x_bounds[m->rank + 1];
  // this rank's column window
  int64_t cmin = 0, cmax = -1;
  if (mode == ALPHASPARSE_MG_X_ALLGATHER) {
    cmin = 0;
    cmax = A->cols - 1;
  } else {
    s = alphasparseCsrColumnRange(h, A->nnz, A->const_col_data, ALPHA_SPARSE_INDEXTYPE_I32, &cmin, &cmax);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  }
  constexpr int64_t kAlign = 32;  // the window starts on a multiple of 32 elements: keeps 128-byte alignment
  m->lo = cmax >= cmin ? (cmin / kAlign) * kAlign : 0;
  m->hi = cmax >= cmin ? cmax + 1 : 0;
  // every rank learns every window
  m->windows.assign(2 * (size_t)W, 0);
  if (W > 1) {
    int64_t* d = nullptr;
    ASP_CUDA(cudaMalloc(&d, sizeof(int64_t) * 2 * (size_t)(W + 1)));
    const int64_t mine[2] = {m->lo, m->hi};
    cudaError_t e = cudaMemcpyAsync(d, mine, sizeof mine, cudaMemcpyHostToDevice, st);
    ncclResult_t r = ncclSuccess;
    if (e == cudaSuccess) r = nc->AllGather(d, d + 2, 2, ncclInt64, m->comm, st);
    if (e == cudaSuccess && r == ncclSuccess)
      e = cudaMemcpyAsync(m->windows.data(), d + 2, sizeof(int64_t) * 2 * (size_t)W, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d);
    if (r != ncclSuccess) return nccl_status(r);
    if (e != cudaSuccess) return asp::status_of(e);
  } else {
    m->windows[0] = m->lo;
    m->windows[1] = m->hi;
  }
  {
    std::vector<int64_t> sb(3 * (size_t)W), rb(3 * (size_t)W);
    int ns = 0, nr = 0;
    s = alphasparseMgExchangePlan(W, m->rank, m->x_bounds.data(), m->windows.data(), sb.data(), &ns,
                                  rb.data(), &nr);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    for (int i = 0; i < ns; ++i) m->sends.push_back({(int)sb[3 * i], sb[3 * i + 1], sb[3 * i + 2]});
    for (int i = 0; i < nr; ++i) {
      m->recvs.push_back({(int)rb[3 * i], rb[3 * i + 1], rb[3 * i + 2]});
      if (rb[3 * i] != m->rank) m->bytes_received += (rb[3 * i + 2] - rb[3 * i + 1]) * (int64_t)m->es;
    }
  }
  if (m->hi > m->lo) ASP_CUDA(cudaMalloc(&m->window, (size_t)(m->hi - m->lo) * m->es));
  s = alphasparseCreateDnVecWindow(&m->xd, A->cols, m->lo, m->hi - m->lo, m->window, A->data_type);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;

  if (mode != ALPHASPARSE_MG_X_WINDOW_OVERLAP || W == 1 || A->rows == 0) return ALPHA_SPARSE_STATUS_SUCCESS;

  // interior rows: the first contiguous run of rows that read only this rank's own part of x
  const bool o64 = A->row_type == ALPHA_SPARSE_INDEXTYPE_I64;
  unsigned long long* d_out = nullptr;
  ASP_CUDA(cudaMalloc(&d_out, sizeof(unsigned long long)));
  auto first_row = [&](int64_t from, bool want_inside, int64_t* res) -> alphasparseStatus_t {
    const unsigned long long init = (unsigned long long)A->rows;
    ASP_CUDA(cudaMemcpyAsync(d_out, &init, sizeof init, cudaMemcpyHostToDevice, st));
    int64_t g = (A->rows - from + 255) / 256;
    const int64_t cap = (int64_t)impl(h)->sm_count * 16;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    if (o64)
      first_row_kernel<int64_t><<<(unsigned)g, 256, 0, st>>>((const int64_t*)A->row_offsets, A->const_col_data,
                                                            A->rows, own_lo, own_hi, from, want_inside, d_out);
    else
      first_row_kernel<int32_t><<<(unsigned)g, 256, 0, st>>>((const int32_t*)A->row_offsets, A->const_col_data,
                                                            A->rows, own_lo, own_hi, from, want_inside, d_out);
    impl(h)->launches++;
    unsigned long long v = 0;
    ASP_CUDA(cudaMemcpyAsync(&v, d_out, sizeof v, cudaMemcpyDeviceToHost, st));
    ASP_CUDA(cudaStreamSynchronize(st));
    *res = (int64_t)v;
    return ALPHA_SPARSE_STATUS_SUCCESS;
  };
  int64_t i0 = 0, i1 = 0;
  s = first_row(0, true, &i0);
  if (s == ALPHA_SPARSE_STATUS_SUCCESS) {
    if (i0 >= A->rows) i0 = i1 = 0;
    else s = first_row(i0, false, &i1);
  }
  cudaFree(d_out);
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  // The interior and bottom parts are slices of the shard's arrays: move the two cuts to rows whose
  // first entry sits on a 16-byte boundary of both arrays (a multiple of four entries), or those
  // parts lose the bulk-copy kernels.  Rows that leave the interior this way simply count as
  // boundary rows.
  if (i1 > i0) {
    constexpr int kLook = 4096;  // far enough to get past a run of even-length rows that starts on an odd entry
    auto align_cut = [&](int64_t from, int dir, int64_t* cut) -> alphasparseStatus_t {
      int64_t a = dir > 0 ? from : from - kLook + 1;
      if (a < 0) a = 0;
      int64_t b = dir > 0 ? from + kLook : from + 1;  // offsets of rows [a, b)
      if (b > A->rows + 1) b = A->rows + 1;
      std::vector<int64_t> host((size_t)kLook);
      const int64_t cnt = b - a;
      if (o64) {
        ASP_CUDA(cudaMemcpyAsync(host.data(), (const int64_t*)A->row_offsets + a, sizeof(int64_t) * cnt, cudaMemcpyDeviceToHost, st));
        ASP_CUDA(cudaStreamSynchronize(st));
      } else {
        std::vector<int32_t> h32((size_t)kLook);
        ASP_CUDA(cudaMemcpyAsync(h32.data(), (const int32_t*)A->row_offsets + a, sizeof(int32_t) * cnt, cudaMemcpyDeviceToHost, st));
        ASP_CUDA(cudaStreamSynchronize(st));
        for (int64_t j = 0; j < cnt; ++j) host[j] = h32[j];
      }
      *cut = -1;
      if (dir > 0) {
        for (int64_t j = 0; j < cnt; ++j)
          if (host[j] % 4 == 0) { *cut = a + j; break; }
      } else {
        for (int64_t j = cnt - 1; j >= 0; --j)
          if (host[j] % 4 == 0) { *cut = a + j; break; }
      }
      return ALPHA_SPARSE_STATUS_SUCCESS;
    };
    int64_t c0 = i0, c1 = i1;
    if (i0 > 0) s = align_cut(i0, +1, &c0);
    if (s == ALPHA_SPARSE_STATUS_SUCCESS && i1 < A->rows) s = align_cut(i1, -1, &c1);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    if (c0 < 0 || c1 < 0 || c1 <= c0) i0 = i1 = 0;  // no aligned cut nearby: run as WINDOW
    else {
      i0 = c0;
      i1 = c1;
    }
  }
  m->i0 = i0;
  m->i1 = i1;
  if (i1 <= i0) return ALPHA_SPARSE_STATUS_SUCCESS;  // no interior: the overlapped mode runs as WINDOW

  const size_t ob = o64 ? 8 : 4;
  const int64_t cut[3][2] = {{i0, i1}, {0, i0}, {i1, A->rows}};
  for (int c = 0; c < 3; ++c) {
    const int64_t a = cut[c][0], b = cut[c][1];
    if (b <= a) continue;
    Part p;
    p.a = a;
    p.b = b;
    int64_t k0 = 0, k1 = 0;
    s = read_offset(A->row_offsets, o64, a, st, &k0);
    if (s == ALPHA_SPARSE_STATUS_SUCCESS) s = read_offset(A->row_offsets, o64, b, st, &k1);
    if (s == ALPHA_SPARSE_STATUS_SUCCESS) s = asp::status_of(cudaMalloc(&p.rp, (size_t)(b - a + 1) * ob));
    if (s == ALPHA_SPARSE_STATUS_SUCCESS)
      s = alphasparseCsrRebaseRowOffsets(h, A->row_offsets, A->row_type, a, b, p.rp, A->row_type);
    if (s == ALPHA_SPARSE_STATUS_SUCCESS)
      s = alphasparseCreateCsr(&p.d, b - a, A->cols, k1 - k0, p.rp, (void*)(A->const_col_data + k0),
                               (void*)((const char*)A->const_val_data + (size_t)k0 * m->es), A->row_type,
                               ALPHA_SPARSE_INDEXTYPE_I32, ALPHA_SPARSE_INDEX_BASE_ZERO, A->data_type);
    if (s == ALPHA_SPARSE_STATUS_SUCCESS) s = analyse(h, p.d);
    m->parts.push_back(p);  // owned from here on, also when a step above failed
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  }
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseMgOwnView(alphasparseMgHandle_t m, void** ptr, int64_t* first, int64_t* count) {
  if (!m) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!ptr || !first || !count) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (!m->A || m->mode == ALPHASPARSE_MG_X_BROADCAST) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
  const int64_t o0 = m->x_bounds[m->rank], o1 = m->x_bounds[m->rank + 1];
  // offered only when the window holds the whole own part: what peers are sent is read from there too
  if (o1 <= o0 || m->lo > o0 || m->hi < o1) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  *ptr = (char*)m->window + (size_t)(o0 - m->lo) * m->es;
  *first = o0;
  *count = o1 - o0;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseMgGetInfo(alphasparseMgHandle_t m, int64_t* info) {
  if (!m) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!info) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  for (int i = 0; i < ASP_MG_INFO_COUNT; ++i) info[i] = 0;
  info[ASP_MG_INFO_WINDOW_LO] = m->lo;
  info[ASP_MG_INFO_WINDOW_HI] = m->hi;
  info[ASP_MG_INFO_BYTES_RECEIVED] = m->bytes_received;
  info[ASP_MG_INFO_INTERIOR_BEGIN] = m->i0;
  info[ASP_MG_INFO_INTERIOR_END] = m->i1;
  info[ASP_MG_INFO_NUM_SENDS] = 0;
  info[ASP_MG_INFO_NUM_RECVS] = 0;
  for (const Seg& s : m->sends) info[ASP_MG_INFO_NUM_SENDS] += s.peer != m->rank;
  for (const Seg& s : m->recvs) info[ASP_MG_INFO_NUM_RECVS] += s.peer != m->rank;
  info[ASP_MG_INFO_MODE] = m->mode;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseMgExchange(alphasparseMgHandle_t m, const void* x) {
  if (!m) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!m->A) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
  cudaStream_t st = m->h->stream;
  const NcclApi* nc = m->world > 1 ? nccl_api() : nullptr;
  if (m->mode == ALPHASPARSE_MG_X_BROADCAST) {
    if (m->world == 1) return ALPHA_SPARSE_STATUS_SUCCESS;
    const int64_t n = m->A->cols;
    if (n == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
    if (m->rank == m->root) {
      if (!x) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
      ASP_NCCL(nc->Broadcast(x, (void*)x, (size_t)n, m->nt, m->root, m->comm, st));
    } else {
      ASP_NCCL(nc->Broadcast(m->window, m->window, (size_t)n, m->nt, m->root, m->comm, st));
    }
    return ALPHA_SPARSE_STATUS_SUCCESS;
  }
  const int64_t o0 = m->x_bounds[m->rank], o1 = m->x_bounds[m->rank + 1];
  if (o1 > o0 && !x) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  const char* xo = (const char*)x;
  const bool in_place = m->window && m->lo <= o0 && xo == (const char*)m->window + (size_t)(o0 - m->lo) * m->es;
  if (!in_place)
    for (const Seg& s : m->recvs)
      if (s.peer == m->rank)
        ASP_CUDA(cudaMemcpyAsync((char*)m->window + (size_t)(s.a - m->lo) * m->es, xo + (size_t)(s.a - o0) * m->es,
                                 (size_t)(s.b - s.a) * m->es, cudaMemcpyDeviceToDevice, st));
  if (m->world == 1) return ALPHA_SPARSE_STATUS_SUCCESS;
  return enqueue_exchange(m, nc, xo, o0, st);
}

alphasparseStatus_t alphasparseMgSpMV(alphasparseMgHandle_t m, const void* alpha, const void* x,
                                      const void* beta, void* y, alphasparseSpMVAlg_t alg) {
  if (!m) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!alpha || !beta) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (!m->A) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
  alphasparseSpMatDescr_t A = m->A;
  if (A->rows > 0 && !y) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  alphasparseHandle_t h = m->h;
  cudaStream_t st = h->stream;
  const alphasparseDataType dt = A->data_type;
  const NcclApi* nc = m->world > 1 ? nccl_api() : nullptr;
  if (m->world > 1 && !nc) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  alphasparseStatus_t s;
  _alphasparse_dnvec_descr yv{true, A->rows, y, dt};
  if (m->world == 1) {  // the rank owns all of x: nothing to exchange, nothing to stage
    if (A->cols > 0 && !x) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    _alphasparse_dnvec_descr xv{true, A->cols, const_cast<void*>(x), dt};
    return alphasparseSpMV(h, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, alpha, A, &xv, beta, &yv, dt, alg, nullptr);
  }

  if (m->mode == ALPHASPARSE_MG_X_BROADCAST) {
    s = alphasparseMgExchange(m, x);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    const void* xs = (m->world == 1 || m->rank == m->root) ? x : m->window;
    if (A->cols > 0 && !xs) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    _alphasparse_dnvec_descr xv{true, A->cols, const_cast<void*>(xs), dt};
    s = alphasparseSpMV(h, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, alpha, A, &xv, beta, &yv, dt, alg, nullptr);
  } else if (m->mode != ALPHASPARSE_MG_X_WINDOW_OVERLAP || m->parts.empty()) {
    s = alphasparseMgExchange(m, x);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    s = alphasparseSpMV(h, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, alpha, A, m->xd, beta, &yv, dt, alg, nullptr);
  } else {
    // own part into the window on the compute stream (the interior rows read only this), the halo on
    // the side stream meanwhile, then the boundary rows
    const int64_t o0 = m->x_bounds[m->rank], o1 = m->x_bounds[m->rank + 1];
    if (o1 > o0 && !x) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    const char* xo = (const char*)x;
    const bool in_place = m->lo <= o0 && xo == (const char*)m->window + (size_t)(o0 - m->lo) * m->es;
    if (!in_place)
      for (const Seg& g : m->recvs)
        if (g.peer == m->rank)
          ASP_CUDA(cudaMemcpyAsync((char*)m->window + (size_t)(g.a - m->lo) * m->es, xo + (size_t)(g.a - o0) * m->es,
                                   (size_t)(g.b - g.a) * m->es, cudaMemcpyDeviceToDevice, st));
    // the side stream starts after everything enqueued so far: the caller's x is complete and the
    // previous step's boundary rows no longer read the halo that is about to be overwritten
    ASP_CUDA(cudaEventRecord(m->ev_ready, st));
    ASP_CUDA(cudaStreamWaitEvent(m->comm_stream, m->ev_ready, 0));
    // the interior rows are enqueued before the exchange: the host's time inside NCCL then passes
    // while the GPU already multiplies
    bool exchanged = false;
    for (const Part& p : m->parts) {
      const bool interior = p.a == m->i0 && p.b == m->i1;
      if (!interior && !exchanged) {
        s = enqueue_exchange(m, nc, xo, o0, m->comm_stream);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        ASP_CUDA(cudaEventRecord(m->ev_halo, m->comm_stream));
        exchanged = true;
      }
      if (!interior) ASP_CUDA(cudaStreamWaitEvent(st, m->ev_halo, 0));  // boundary rows need the halo
      _alphasparse_dnvec_descr yp{true, p.b - p.a, (char*)y + (size_t)p.a * m->es, dt};
      s = alphasparseSpMV(h, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, alpha, p.d, m->xd, beta, &yp, dt, alg, nullptr);
      if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    }
    if (!exchanged) {  // a shard without boundary rows still owes its peers their halos
      s = enqueue_exchange(m, nc, xo, o0, m->comm_stream);
      if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
      ASP_CUDA(cudaEventRecord(m->ev_halo, m->comm_stream));
    }
    // whatever the caller enqueues next on its stream (e.g. an update of x) comes after the sends
    ASP_CUDA(cudaStreamWaitEvent(st, m->ev_halo, 0));
    s = ALPHA_SPARSE_STATUS_SUCCESS;
  }
  if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
  if (m->world > 1) {
    ncclResult_t async = ncclSuccess;
    ASP_NCCL(nc->CommGetAsyncError(m->comm, &async));  // one non-blocking look, never a wait
    if (async != ncclSuccess && async != ncclInProgress) return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
  }
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

}  // extern "C"
