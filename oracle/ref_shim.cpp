// TEST INFRASTRUCTURE ONLY (also the timed CPU baseline of bench.py). Flat C entry points over the reference's own x86 (hygon)
// CSR mv / mm code, which oracle/Makefile compiles in place from the reference tree into
// oracle/_ref/libasp_ref.so.  Nothing in the product path links or loads this file.
//
// The reference calls wrapped here:
//   alphasparse_{s,d,c,z}_create_csr  hygon/format/alphasparse_create_csr.cpp:12-25
//   alphasparse_{s,d,c,z}_mv          hygon/kernel/level2/alphasparse_mv.cpp:1219-1239
//   alphasparse_{s,d}_mm          hygon/kernel/level3/alphasparse_mm.cpp:2588-2617
//   alphasparse_destroy           hygon/format/alphasparse_destroy.cpp
//   alpha_set_thread_num          hygon/util/thread.cpp:23-31
#include <alphasparse.h>
#include <cstdint>
#include <chrono>

static inline double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

extern "C" {

void ref_set_threads(int n) { alpha_set_thread_num(n); }
int ref_get_threads(void) { return alpha_get_thread_num(); }

#define REF_MV(NAME, T, CREATE, MV)                                                        \
  int NAME(int rows, int cols, const int* row_ptr, const int* col_idx, const T* val,       \
           const T* x, T alpha, T beta, T* y, int repeats,     \
           double* times) {                               \
    alphasparse_matrix_t A = nullptr;                                                      \
    int st = (int)CREATE(&A, ALPHA_SPARSE_INDEX_BASE_ZERO, rows, cols, (int*)row_ptr,      \
                         (int*)row_ptr + 1, (int*)col_idx, (T*)val);                       \
    if (st != 0) return 100 + st;                                                          \
    struct alpha_matrix_descr d;                                                           \
    d.type = ALPHA_SPARSE_MATRIX_TYPE_GENERAL;                                             \
    d.mode = ALPHA_SPARSE_FILL_MODE_LOWER;                                                 \
    d.diag = ALPHA_SPARSE_DIAG_NON_UNIT;                                                   \
    for (int r = 0; r < (repeats < 1 ? 1 : repeats) && st == 0; ++r) {                     \
      double t0 = now_s();                                                                 \
      st = (int)MV(ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, alpha, A, d, x, beta, y);         \
      if (times) times[r] = now_s() - t0;                                                  \
    }                                                                                      \
    alphasparse_destroy(A);                                                                \
    return st;                                                                             \
  }

REF_MV(ref_s_mv, float, alphasparse_s_create_csr, alphasparse_s_mv)
REF_MV(ref_d_mv, double, alphasparse_d_create_csr, alphasparse_d_mv)

// complex: alpha, beta and the arrays as interleaved (re, im) pairs
#define REF_MV_CPLX(NAME, T, CT, CREATE, MV)                                               \
  int NAME(int rows, int cols, const int* row_ptr, const int* col_idx, const T* val,       \
           const T* x, const T* alpha, const T* beta, T* y) {                              \
    alphasparse_matrix_t A = nullptr;                                                      \
    int st = (int)CREATE(&A, ALPHA_SPARSE_INDEX_BASE_ZERO, rows, cols, (int*)row_ptr,      \
                         (int*)row_ptr + 1, (int*)col_idx, (CT*)val);                      \
    if (st != 0) return 100 + st;                                                          \
    struct alpha_matrix_descr d;                                                           \
    d.type = ALPHA_SPARSE_MATRIX_TYPE_GENERAL;                                             \
    d.mode = ALPHA_SPARSE_FILL_MODE_LOWER;                                                 \
    d.diag = ALPHA_SPARSE_DIAG_NON_UNIT;                                                   \
    CT a, b;                                                                               \
    a.real = alpha[0]; a.imag = alpha[1]; b.real = beta[0]; b.imag = beta[1];              \
    st = (int)MV(ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, a, A, d, (const CT*)x, b, (CT*)y);  \
    alphasparse_destroy(A);                                                                \
    return st;                                                                             \
  }
REF_MV_CPLX(ref_c_mv, float, ALPHA_Complex8, alphasparse_c_create_csr, alphasparse_c_mv)
REF_MV_CPLX(ref_z_mv, double, ALPHA_Complex16, alphasparse_z_create_csr, alphasparse_z_mv)

#define REF_MM(NAME, T, CREATE, MM)                                                        \
  int NAME(int rows, int cols, const int* row_ptr, const int* col_idx, const T* val,       \
           const T* X, int n, int ldx, T alpha, T beta, T* Y, int ldy, int repeats,     \
           double* times) {      \
    alphasparse_matrix_t A = nullptr;                                                      \
    int st = (int)CREATE(&A, ALPHA_SPARSE_INDEX_BASE_ZERO, rows, cols, (int*)row_ptr,      \
                         (int*)row_ptr + 1, (int*)col_idx, (T*)val);                       \
    if (st != 0) return 100 + st;                                                          \
    struct alpha_matrix_descr d;                                                           \
    d.type = ALPHA_SPARSE_MATRIX_TYPE_GENERAL;                                             \
    d.mode = ALPHA_SPARSE_FILL_MODE_LOWER;                                                 \
    d.diag = ALPHA_SPARSE_DIAG_NON_UNIT;                                                   \
    for (int r = 0; r < (repeats < 1 ? 1 : repeats) && st == 0; ++r) {                     \
      double t0 = now_s();                                                                 \
      st = (int)MM(ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, alpha, A, d,                      \
                   ALPHA_SPARSE_LAYOUT_ROW_MAJOR, X, n, ldx, beta, Y, ldy);                \
      if (times) times[r] = now_s() - t0;                                                  \
    }                                                                                      \
    alphasparse_destroy(A);                                                                \
    return st;                                                                             \
  }

REF_MM(ref_s_mm, float, alphasparse_s_create_csr, alphasparse_s_mm)
REF_MM(ref_d_mm, double, alphasparse_d_create_csr, alphasparse_d_mm)

#define REF_MM_CPLX(NAME, T, CT, CREATE, MM)                                               \
  int NAME(int rows, int cols, const int* row_ptr, const int* col_idx, const T* val,       \
           const T* X, int n, int ldx, const T* alpha, const T* beta, T* Y, int ldy) {     \
    alphasparse_matrix_t A = nullptr;                                                      \
    int st = (int)CREATE(&A, ALPHA_SPARSE_INDEX_BASE_ZERO, rows, cols, (int*)row_ptr,      \
                         (int*)row_ptr + 1, (int*)col_idx, (CT*)val);                      \
    if (st != 0) return 100 + st;                                                          \
    struct alpha_matrix_descr d;                                                           \
    d.type = ALPHA_SPARSE_MATRIX_TYPE_GENERAL;                                             \
    d.mode = ALPHA_SPARSE_FILL_MODE_LOWER;                                                 \
    d.diag = ALPHA_SPARSE_DIAG_NON_UNIT;                                                   \
    CT a, b;                                                                               \
    a.real = alpha[0]; a.imag = alpha[1]; b.real = beta[0]; b.imag = beta[1];              \
    st = (int)MM(ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, a, A, d, ALPHA_SPARSE_LAYOUT_ROW_MAJOR,\
                 (const CT*)X, n, ldx, b, (CT*)Y, ldy);                                    \
    alphasparse_destroy(A);                                                                \
    return st;                                                                             \
  }
REF_MM_CPLX(ref_c_mm, float, ALPHA_Complex8, alphasparse_c_create_csr, alphasparse_c_mm)
REF_MM_CPLX(ref_z_mm, double, ALPHA_Complex16, alphasparse_z_create_csr, alphasparse_z_mm)

}  // extern "C"
