// A C++ caller of the SpMM path written the way the reference's own test driver calls it
// (cuda/test/level3/spmm_csr_row_r_f32_test.cu:169-262): handle, COO rows to CSR offsets, row-major
// dense descriptors, template alphasparseCreateCsr, alphasparseSpMM_bufferSize, cudaMalloc of that
// size, one alphasparseSpMM with ALPHASPARSE_SPMM_CSR_ALG2 (the reference's default algorithm),
// the get_avg_time timer, result copied back.  Compiles against include/alphasparse_b200.h alone.
//
//   spmm_caller <input file> <output file>        (file layout: caller_io.h)
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
  if (!read_input(argv[1], &in) || in.kind != 1) return 1;
  const int A_rows = (int)in.rows, A_cols = (int)in.cols, nnz = (int)in.nnz, C_cols = (int)in.n;
  const int ldb = C_cols, ldc = C_cols;
  const size_t B_size = (size_t)A_cols * ldb, C_size = (size_t)A_rows * ldc;
  const float alpha = in.alpha, beta = in.beta;
  const alphasparseSpMMAlg_t alpha_alg = ALPHASPARSE_SPMM_CSR_ALG2;

  alphasparseHandle_t handle = NULL;
  CHECK_ALPHA(initHandle(&handle));
  CHECK_ALPHA(alphasparseGetHandle(&handle));

  int *dArow = NULL, *dAcol = NULL, *dCsrRowPtr = NULL;
  float *dAval = NULL, *dmatB = NULL, *dmatC = NULL;
  CHECK_CUDA(cudaMalloc((void**)&dmatB, sizeof(float) * (B_size ? B_size : 1)));
  CHECK_CUDA(cudaMalloc((void**)&dmatC, sizeof(float) * (C_size ? C_size : 1)));
  CHECK_CUDA(cudaMalloc((void**)&dArow, sizeof(int) * (nnz > 0 ? nnz : 1)));
  CHECK_CUDA(cudaMalloc((void**)&dAcol, sizeof(int) * (nnz > 0 ? nnz : 1)));
  CHECK_CUDA(cudaMalloc((void**)&dAval, sizeof(float) * (nnz > 0 ? nnz : 1)));
  CHECK_CUDA(cudaMalloc((void**)&dCsrRowPtr, sizeof(int) * (A_rows + 1)));
  CHECK_CUDA(cudaMemcpy(dArow, in.coo_row.data(), sizeof(int) * nnz, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dAcol, in.coo_col.data(), sizeof(int) * nnz, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dAval, in.val.data(), sizeof(float) * nnz, cudaMemcpyHostToDevice));
  CHECK_ALPHA(alphasparseXcoo2csr(dArow, nnz, A_rows, dCsrRowPtr));
  CHECK_CUDA(cudaMemcpy(dmatB, in.dense_in.data(), sizeof(float) * B_size, cudaMemcpyHostToDevice));
  CHECK_CUDA(cudaMemcpy(dmatC, in.dense_out.data(), sizeof(float) * C_size, cudaMemcpyHostToDevice));

  alphasparseDnMatDescr_t matB, matC;
  CHECK_ALPHA(alphasparseCreateDnMat(&matB, A_cols, C_cols, ldb, dmatB, ALPHA_R_32F, ALPHASPARSE_ORDER_ROW));
  CHECK_ALPHA(alphasparseCreateDnMat(&matC, A_rows, C_cols, ldc, dmatC, ALPHA_R_32F, ALPHASPARSE_ORDER_ROW));
  alphasparseSpMatDescr_t matA;
  CHECK_ALPHA(alphasparseCreateCsr(&matA, A_rows, A_cols, nnz, dCsrRowPtr, dAcol, dAval, ALPHA_SPARSE_INDEXTYPE_I32,
                                   ALPHA_SPARSE_INDEXTYPE_I32, ALPHA_SPARSE_INDEX_BASE_ZERO, ALPHA_R_32F));
  std::vector<double> times;
  const double t0 = get_time_us();
  size_t bufferSize = 0;
  CHECK_ALPHA(alphasparseSpMM_bufferSize(handle, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE,
                                         &alpha, matA, matB, &beta, matC, ALPHA_R_32F, alpha_alg, &bufferSize));
  void* dBuffer = NULL;
  CHECK_CUDA(cudaMalloc(&dBuffer, bufferSize));
  CHECK_ALPHA(alphasparseSpMM(handle, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, &alpha,
                              matA, matB, &beta, matC, ALPHA_R_32F, alpha_alg, dBuffer));
  CHECK_CUDA(cudaDeviceSynchronize());
  times.push_back((get_time_us() - t0) / 1e3);
  printf("alphasparse: %lf\n", get_avg_time(times));

  std::vector<float> out(C_size);
  CHECK_CUDA(cudaMemcpy(out.data(), dmatC, sizeof(float) * C_size, cudaMemcpyDeviceToHost));
  if (!write_output(argv[2], out)) return 1;
  alphasparseDestroySpMat(matA);
  alphasparseDestroyDnMat(matB);
  alphasparseDestroyDnMat(matC);
  cudaFree(dBuffer); cudaFree(dArow); cudaFree(dAcol); cudaFree(dAval); cudaFree(dCsrRowPtr); cudaFree(dmatB); cudaFree(dmatC);
  alphasparse_destory_handle(handle);
  return 0;
}
