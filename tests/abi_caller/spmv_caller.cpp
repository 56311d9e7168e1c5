// A C++ caller of the SpMV path written the way the reference's own test driver calls it
// (cuda/test/level2/spmv_csr_r_f32_test.cu:175-262): initHandle + alphasparseGetHandle, COO rows to
// CSR offsets with the template alphasparseXcoo2csr(row, nnz, m, ptr), template
// alphasparseCreateCsr with int sizes, alphasparseSpMV_bufferSize, cudaMalloc of that size, warm-up
// and timed calls with ALPHA_SPARSE_SPMV_ALG_COO (what the reference's CSR drivers pass), the
// get_time_us / get_avg_time timers, result copied back.  It compiles against
// include/alphasparse_b200.h alone and links libalphasparse_b200.so: the proof that a caller of
// the reference builds against this library.
//
//   spmv_caller <input file> <output file>        (file layout: caller_io.h)
#include <alphasparse_b200.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <vector>

#include "caller_io.h"

#define CHECK_CUDA(call)                                                        \
  do {                                                                          \
    cudaError_t e_ = (call);                                                    \
    if (e_ != cudaSuccess) {                                                    \
      fprintf(stderr, "%s:%d CUDA error %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
      return 2;                                                                 \
    }                                                                           \
  } while (0)
#define CHECK_ALPHA(call)                                                       \
  do {                                                                          \
    alphasparseStatus_t s_ = (call);                                            \
    if (s_ != ALPHA_SPARSE_STATUS_SUCCESS) {                                    \
      fprintf(stderr, "%s:%d alphasparse status %d\n", __FILE__, __LINE__, (int)s_); \
      return 3;                                                                 \
    }                                                                           \
  } while (0)

int main(int argc, char** argv) {
  if (argc != 3) return 1;
  CallerInput in;
  if (!read_input(argv[1], &in) || in.kind != 0) return 1;
  const int m = (int)in.rows, n = (int)in.cols, nnz = (int)in.nnz;
  const float alpha = in.alpha, beta = in.beta;
  const int warm_up = 2, trials = 5;

  alphasparseHandle_t handle = NULL;
  CHECK_ALPHA(initHandle(&handle));
  CHECK_ALPHA(alphasparseGetHandle(&handle));
  cudaStream_t stream = NULL;
  CHECK_CUDA(cudaStreamCreate(&stream));
  handle->stream = stream;  // the reference has no setter: callers write the field

  int *dArow = NULL, *dAcol = NULL, *dCsrRowPtr = NULL;
  float *dAval = NULL, *dX = NULL, *dY = NULL;
  CHECK_CUDA(cudaMalloc((void**)&dArow, sizeof(int) * (nnz > 0 ? nnz : 1)));
  CHECK_CUDA(cudaMalloc((void**)&dAcol, sizeof(int) * (nnz > 0 ? nnz : 1)));
  CHECK_CUDA(cudaMalloc((void**)&dAval, sizeof(float) * (nnz > 0 ? nnz : 1)));
  CHECK_CUDA(cudaMalloc((void**)&dCsrRowPtr, sizeof(int) * (m + 1)));
  CHECK_CUDA(cudaMalloc((void**)&dX, sizeof(float) * (n > 0 ? n : 1)));
  CHECK_CUDA(cudaMalloc((void**)&dY, sizeof(float) * (m > 0 ? m : 1)));
  CHECK_CUDA(cudaMemcpy(dArow, in.coo_row.data(), sizeof(int) * nnz, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dAcol, in.coo_col.data(), sizeof(int) * nnz, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dAval, in.val.data(), sizeof(float) * nnz, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dX, in.dense_in.data(), sizeof(float) * n, cudaMemcpyHostToDevice));
  CHECK_ALPHA(alphasparseXcoo2csr(dArow, nnz, m, dCsrRowPtr));  // template overload, default stream
  CHECK_CUDA(cudaDeviceSynchronize());

  alphasparseDnVecDescr_t x{}, y{};
  CHECK_ALPHA(alphasparseCreateDnVec(&x, n, (void*)dX, ALPHA_R_32F));
  CHECK_ALPHA(alphasparseCreateDnVec(&y, m, (void*)dY, ALPHA_R_32F));
  alphasparseSpMatDescr_t csr;
  CHECK_ALPHA(alphasparseCreateCsr(&csr, m, n, nnz, dCsrRowPtr, dAcol, dAval, ALPHA_SPARSE_INDEXTYPE_I32,
                                   ALPHA_SPARSE_INDEXTYPE_I32, ALPHA_SPARSE_INDEX_BASE_ZERO, ALPHA_R_32F));
  size_t bufferSize = 0;
  void* dBuffer = NULL;
  CHECK_ALPHA(alphasparseSpMV_bufferSize(handle, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, &alpha, csr, x, &beta, y,
                                         ALPHA_R_32F, ALPHA_SPARSE_SPMV_ALG_COO, &bufferSize));
  CHECK_CUDA(cudaMalloc(&dBuffer, bufferSize));

  std::vector<double> times;
  for (int i = 0; i < warm_up + trials; ++i) {
    // y = alpha*A*x + beta*y overwrites its input: every call starts from the same y0
    CHECK_CUDA(cudaMemcpyAsync(dY, in.dense_out.data(), sizeof(float) * m, cudaMemcpyHostToDevice, stream));
    const double t0 = get_time_us();
    CHECK_ALPHA(alphasparseSpMV(handle, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, &alpha, csr, x, &beta, y, ALPHA_R_32F,
                                ALPHA_SPARSE_SPMV_ALG_COO, dBuffer));
    CHECK_CUDA(cudaDeviceSynchronize());
    if (i >= warm_up) times.push_back((get_time_us() - t0) / 1e3);
  }
  printf("alphasparse: %lf ms (filtered mean), %lf ms (around the median)\n", get_avg_time(times), get_avg_time_2(times));

  std::vector<float> out((size_t)m);
  CHECK_CUDA(cudaMemcpy(out.data(), dY, sizeof(float) * m, cudaMemcpyDeviceToHost));
  if (!write_output(argv[2], out)) return 1;
  alphasparseDestroySpMat(csr);
  alphasparseDestroyDnVec(x);
  alphasparseDestroyDnVec(y);
  cudaFree(dBuffer); cudaFree(dArow); cudaFree(dAcol); cudaFree(dAval); cudaFree(dCsrRowPtr); cudaFree(dX); cudaFree(dY);
  alphasparse_destory_handle(handle);
  cudaStreamDestroy(stream);
  return 0;
}
