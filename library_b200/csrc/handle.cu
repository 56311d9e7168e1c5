// Handle, stream and descriptor management plus the timers the reference's drivers call.
// Replaces cuda/util/handle.cu (handle :52-175, timers :547-599, dense descriptors
// :657-738) and cuda/format/alphasparse_create_csr.h:6-63 of the reference.
#include <sys/time.h>

#include <algorithm>
#include <new>
#include <vector>

#include "asp_internal.h"

using namespace asp;

namespace {
__global__ void asp_init_kernel() {}
}  // namespace

extern "C" {

alphasparseStatus_t initHandle(alphasparseHandle_t* handle) {
  if (!handle) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  auto* h = new (std::nothrow) alphasparse_handle();
  if (!h) return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  *h = alphasparse_handle{};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    delete h;
    return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
  }
  h->device = dev;  // the reference hard-codes device 0; one process per GPU needs the current one
  h->stream = nullptr;
  h->pointer_mode = ALPHA_SPARSE_POINTER_MODE_HOST;
  h->impl = new (std::nothrow) HandleImpl();
  if (!h->impl) {
    delete h;
    return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  }
  for (int i = 0; i < 6; ++i) {
    if (cudaStreamCreateWithFlags(&h->streams[i], cudaStreamNonBlocking) != cudaSuccess) {
      h->streams[i] = nullptr;
    }
  }
  *handle = h;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseGetHandle(alphasparseHandle_t* handle) {
  if (!handle) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (*handle == nullptr) {
    alphasparseStatus_t st = initHandle(handle);
    if (st != ALPHA_SPARSE_STATUS_SUCCESS) return st;
  }
  alphasparseHandle_t h = *handle;
  ASP_CUDA(cudaSetDevice(h->device));
  cudaDeviceProp prop;
  ASP_CUDA(cudaGetDeviceProperties(&prop, h->device));
  if (prop.major < 10) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;  // sm_100a code only
  h->wavefront_size = prop.warpSize;
  impl(h)->sm_count = prop.multiProcessorCount;
  impl(h)->smem_optin = prop.sharedMemPerBlockOptin;
  {
    // dense bf16: 8192 flop per clock per SM on this architecture, of which a long-running kernel
    // sustains about 0.62 under the power cap; HBM: double data rate over the bus, of which a
    // streaming kernel sustains about 0.8
    int sm_khz = 0, mem_khz = 0, bus_bits = 0;
    if (cudaDeviceGetAttribute(&sm_khz, cudaDevAttrClockRate, h->device) == cudaSuccess &&
        cudaDeviceGetAttribute(&mem_khz, cudaDevAttrMemoryClockRate, h->device) == cudaSuccess &&
        cudaDeviceGetAttribute(&bus_bits, cudaDevAttrGlobalMemoryBusWidth, h->device) == cudaSuccess &&
        sm_khz > 0 && mem_khz > 0 && bus_bits > 0) {
      impl(h)->bf16_flops = 0.62 * 8192.0 * prop.multiProcessorCount * (double)sm_khz * 1e3;
      impl(h)->hbm_bytes = 0.8 * 2.0 * (double)mem_khz * 1e3 * (bus_bits / 8.0);
    }
  }
  const char* layer = getenv("ALPHA_SPARSE_LAYER");
  h->layer_mode = layer ? (alphasparse_layer_mode_t)atoi(layer) : ALPHA_SPARSE_LAYER_MODE_NONE;
  if (!h->buffer) {
    h->buffer_size = 1 << 20;
    ASP_CUDA(cudaMalloc(&h->buffer, h->buffer_size));
    ASP_CUDA(cudaMalloc((void**)&h->sone, sizeof(float)));
    ASP_CUDA(cudaMalloc((void**)&h->done, sizeof(double)));
    const float s1 = 1.0f;
    const double d1 = 1.0;
    ASP_CUDA(cudaMemcpyAsync(h->sone, &s1, sizeof s1, cudaMemcpyHostToDevice, h->stream));
    ASP_CUDA(cudaMemcpyAsync(h->done, &d1, sizeof d1, cudaMemcpyHostToDevice, h->stream));
  }
  asp_init_kernel<<<1, 1, 0, h->stream>>>();
  ASP_CUDA(cudaGetLastError());
  ASP_CUDA(cudaStreamSynchronize(h->stream));
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparse_destory_handle(alphasparseHandle_t h) {
  if (!h) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  cudaFree(h->buffer);
  cudaFree(h->sone);
  cudaFree(h->done);
  for (int i = 0; i < 6; ++i)
    if (h->streams[i]) cudaStreamDestroy(h->streams[i]);
  delete impl(h);
  delete h;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseSetStream(alphasparseHandle_t h, cudaStream_t stream) {
  if (!h) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  h->stream = stream;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseGetStream(alphasparseHandle_t h, cudaStream_t* stream) {
  if (!h) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
  if (!stream) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  *stream = h->stream;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

int64_t alphasparseGetLaunchCount(alphasparseHandle_t h) { return h ? impl(h)->launches : -1; }

// ---- descriptors -------------------------------------------------------------------------

alphasparseStatus_t alphasparseCreateCsr(alphasparseSpMatDescr_t* out, int64_t rows, int64_t cols,
                                         int64_t nnz, void* rowOffsets, void* colInd,
                                         void* values, alphasparseIndexType_t rowT,
                                         alphasparseIndexType_t colT,
                                         alphasparseIndexBase_t base,
                                         alphasparseDataType valueType) {
  if (!out) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  *out = nullptr;
  if (rows < 0 || cols < 0 || nnz < 0) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (rows >= (int64_t(1) << 31) || cols >= (int64_t(1) << 31)) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (!rowOffsets) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (nnz > 0 && (!colInd || !values)) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (rowT != ALPHA_SPARSE_INDEXTYPE_I32 && rowT != ALPHA_SPARSE_INDEXTYPE_I64)
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (colT != ALPHA_SPARSE_INDEXTYPE_I32) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (rowT == ALPHA_SPARSE_INDEXTYPE_I32 && nnz >= (int64_t(1) << 31))
    return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (base != ALPHA_SPARSE_INDEX_BASE_ZERO) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  if (valueType != ALPHA_R_32F && valueType != ALPHA_R_64F && valueType != ALPHA_R_16BF && valueType != ALPHA_R_16F &&
      valueType != ALPHA_C_32F && valueType != ALPHA_C_64F && valueType != ALPHA_R_8I)
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  auto* d = new (std::nothrow) _alphasparseSpMatDescr();
  if (!d) return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  *d = _alphasparseSpMatDescr{};
  d->init = true;
  d->rows = rows;
  d->cols = cols;
  d->nnz = nnz;
  d->row_offsets = rowOffsets;
  if (rowT == ALPHA_SPARSE_INDEXTYPE_I32) {
    d->row_data = (int*)rowOffsets;
    d->const_row_data = (const int*)rowOffsets;
  }
  d->col_data = (int*)colInd;
  d->const_col_data = (const int*)colInd;
  d->val_data = values;
  d->const_val_data = values;
  d->row_type = rowT;
  d->col_type = colT;
  d->data_type = valueType;
  d->idx_base = base;
  d->format = ALPHA_SPARSE_FORMAT_CSR;
  d->batch_count = 1;
  *out = d;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseCreateDnVec(alphasparseDnVecDescr_t* descr, int64_t size,
                                           void* values, alphasparseDataType data_type) {
  if (!descr) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (size < 0) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (size > 0 && !values) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  *descr = nullptr;
  auto* d = new (std::nothrow) _alphasparse_dnvec_descr();
  if (!d) return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  d->init = true;
  d->size = size;
  d->values = values;
  d->data_type = data_type;
  *descr = d;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseCreateDnVecWindow(alphasparseDnVecDescr_t* descr, int64_t size,
                                                 int64_t first, int64_t count, void* window_values,
                                                 alphasparseDataType data_type) {
  if (!descr) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (size < 0 || first < 0 || count < 0 || first + count > size) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (count > 0 && !window_values) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  const size_t es = asp::elem_size(data_type);
  if (es == 0) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  // Element i of the logical vector lives at window_values[i - first]: the descriptor carries the
  // address element 0 would have.  Only elements inside the window may be touched by a kernel.
  const uintptr_t base = reinterpret_cast<uintptr_t>(window_values) - (uintptr_t)first * es;
  return alphasparseCreateDnVec(descr, size, size > 0 ? reinterpret_cast<void*>(base) : window_values,
                                data_type);
}

alphasparseStatus_t alphasparseCreateDnMat(alphasparseDnMatDescr_t* descr, int64_t rows,
                                           int64_t cols, int64_t ld, void* values,
                                           alphasparseDataType valueType,
                                           alphasparseOrder_t order) {
  if (!descr) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (rows < 0 || cols < 0) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (!values && rows > 0 && cols > 0) return ALPHA_SPARSE_STATUS_INVALID_POINTER;  // an empty matrix needs no storage
  // The reference stores ld unchecked; a leading dimension shorter than a row (or column)
  // would make rows overlap, so it is rejected here.
  if (ld < (order == ALPHASPARSE_ORDER_ROW ? cols : rows)) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  *descr = nullptr;
  auto* d = new (std::nothrow) _alphasparse_dnmat_descr();
  if (!d) return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  d->init = true;
  d->rows = rows;
  d->cols = cols;
  d->ld = ld;
  d->values = values;
  d->data_type = valueType;
  d->order = order;
  *descr = d;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseDestroySpMat(alphasparseSpMatDescr_t A) {
  if (!A) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (A->info) {
    free_plan(plan_of(A));
    A->info = nullptr;
  }
  delete A;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseDestroyDnVec(alphasparseDnVecDescr_t d) {
  if (!d) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  delete d;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseDestroyDnMat(alphasparseDnMatDescr_t d) {
  if (!d) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  delete d;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseDnVecSetValues(alphasparseDnVecDescr_t d, void* values) {
  if (!d || !values) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  d->values = values;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseDnMatSetValues(alphasparseDnMatDescr_t d, void* values) {
  if (!d || !values) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  d->values = values;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

// ---- timers ------------------------------------------------------------------------------

double get_time_us(void) {
  cudaDeviceSynchronize();
  struct timeval tv;
  gettimeofday(&tv, nullptr);
  return (double)tv.tv_sec * 1e6 + (double)tv.tv_usec;
}

// Mean of the samples below twice the plain mean (cuda/util/handle.cu:556-573).
double get_avg_time_n(const double* t, int n) {
  if (!t || n <= 0) return 0.0;
  double avg = 0;
  for (int i = 0; i < n; ++i) avg += t[i];
  avg /= n;
  double s = 0;
  int cnt = 0;
  for (int i = 0; i < n; ++i)
    if (t[i] < 2 * avg) {
      s += t[i];
      ++cnt;
    }
  return cnt ? s / cnt : avg;
}

}  // extern "C"
