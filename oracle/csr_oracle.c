/* TEST INFRASTRUCTURE ONLY: the CPU oracle for the CSR SpMV / SpMM path.
 *
 * A plain-C restatement of the arithmetic the reference's x86 (hygon) backend performs for
 * y = alpha*A*x + beta*y and Y = alpha*A*X + beta*Y on a general CSR matrix.  Only tests,
 * the smoke check and the CPU-baseline leg of the benchmark may load this library; the
 * product (the CUDA library) never does.
 *
 * Pinning: the reference holds no golden vectors for this path (its tests are differential
 * against MKL / cuSPARSE).  The pin is the reference code itself: oracle/Makefile compiles
 * the hygon sources in place into oracle/_ref/libasp_ref.so, tests/golden/make_golden.py ran
 * it on seeded inputs and committed input seeds + output digests/vectors, and
 * tests/test_oracle.py checks this restatement against those vectors (bit-exact for SpMV,
 * where the summation order below is the assembly's) and against the live library when it
 * is present.
 *
 * Reference code restated (paths within the reference project):
 *   hygon/kernel/level2/mv/gemv/gemv_csr.hpp:14-78        row loop, one call per thread range
 *   hygon/kernel/level2/mv/gemv/csrmv/gemv_csr_serial_fma_fp64_u4.S:47-150
 *        fp64 row: four FMA partial sums p0..p3 over groups of four entries,
 *        s = (p0+p2)+(p1+p3), then up to three scalar-FMA tail entries,
 *        y = fma(alpha, s, beta*y)
 *   hygon/kernel/level2/mv/gemv/csrmv/gemv_sload_shuffle_shuffle_reduce_128.S:15-185
 *        fp32 row: the same with s = (p0+p1)+(p2+p3)
 *   hygon/kernel/level3/mm/gemm/gemm_csr_row.hpp:15-73,124-158
 *        Y[r,:] *= beta, then for each entry of row r in storage order
 *        Y[r,c] = fma(alpha*a, X[col,c], Y[r,c])
 *   hygon/util/partition.cpp:83-96    balanced_partition_row_by_nnz (lifted to int64 here)
 *
 * The reference is int32-only; the _i64 variants take 64-bit row offsets with the same
 * per-row arithmetic, for matrices whose nnz does not fit 32 bits.
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>
#include <string.h>

#define DEF_SPMV_F64(NAME, OFF_T)                                                          \
  void NAME(int64_t rows, const OFF_T* row_ptr, const int32_t* col, const double* val,     \
            const double* x, double alpha, double beta, double* y) {                       \
    _Pragma("omp parallel for schedule(static)")                                           \
    for (int64_t i = 0; i < rows; ++i) {                                                   \
      int64_t k = (int64_t)row_ptr[i], e = (int64_t)row_ptr[i + 1];                        \
      double p0 = 0, p1 = 0, p2 = 0, p3 = 0, s = 0;                                        \
      if (k < e - 3) {                                                                     \
        for (; k < e - 3; k += 4) {                                                        \
          p0 = fma(val[k], x[col[k]], p0);                                                 \
          p1 = fma(val[k + 1], x[col[k + 1]], p1);                                         \
          p2 = fma(val[k + 2], x[col[k + 2]], p2);                                         \
          p3 = fma(val[k + 3], x[col[k + 3]], p3);                                         \
        }                                                                                  \
        s = (p0 + p2) + (p1 + p3);                                                         \
      }                                                                                    \
      for (; k < e; ++k) s = fma(val[k], x[col[k]], s);                                    \
      y[i] = fma(alpha, s, beta * y[i]);                                                   \
    }                                                                                      \
  }

#define DEF_SPMV_F32(NAME, OFF_T)                                                          \
  void NAME(int64_t rows, const OFF_T* row_ptr, const int32_t* col, const float* val,      \
            const float* x, float alpha, float beta, float* y) {                           \
    _Pragma("omp parallel for schedule(static)")                                           \
    for (int64_t i = 0; i < rows; ++i) {                                                   \
      int64_t k = (int64_t)row_ptr[i], e = (int64_t)row_ptr[i + 1];                        \
      float p0 = 0, p1 = 0, p2 = 0, p3 = 0, s = 0;                                         \
      if (k < e - 3) {                                                                     \
        for (; k < e - 3; k += 4) {                                                        \
          p0 = fmaf(val[k], x[col[k]], p0);                                                \
          p1 = fmaf(val[k + 1], x[col[k + 1]], p1);                                        \
          p2 = fmaf(val[k + 2], x[col[k + 2]], p2);                                        \
          p3 = fmaf(val[k + 3], x[col[k + 3]], p3);                                        \
        }                                                                                  \
        s = (p0 + p1) + (p2 + p3);                                                         \
      }                                                                                    \
      for (; k < e; ++k) s = fmaf(val[k], x[col[k]], s);                                   \
      y[i] = fmaf(alpha, s, beta * y[i]);                                                  \
    }                                                                                      \
  }

DEF_SPMV_F64(oracle_spmv_f64_i32, int32_t)
DEF_SPMV_F64(oracle_spmv_f64_i64, int64_t)
DEF_SPMV_F32(oracle_spmv_f32_i32, int32_t)
DEF_SPMV_F32(oracle_spmv_f32_i64, int64_t)

/* Complex SpMV (interleaved re, im).  The reference's CPU kernels for it are assembly
 * (hygon/kernel/level2/mv/gemv/gemv_csr.hpp:80-139 -> csrmv/gemv_csr_serial_fma_c8_u2.S,
 * gemv_csr_serial_fma_c16_u1.S); this restatement keeps their structure - per row a sum over the
 * entries in storage order, then y = alpha*sum + beta*y - with fused multiply-adds on the real and
 * imaginary parts, and is checked against the compiled reference within rounding (its unrolled
 * partial sums make the last bits differ), not bit for bit. */
#define DEF_SPMV_CPLX(NAME, T, OFF_T, FMA)                                                 \
  void NAME(int64_t rows, const OFF_T* row_ptr, const int32_t* col, const T* val,          \
            const T* x, const T* alpha, const T* beta, T* y) {                             \
    _Pragma("omp parallel for schedule(static)")                                           \
    for (int64_t i = 0; i < rows; ++i) {                                                   \
      T sr = 0, si = 0;                                                                    \
      for (int64_t k = (int64_t)row_ptr[i]; k < (int64_t)row_ptr[i + 1]; ++k) {            \
        const T ar = val[2 * k], ai = val[2 * k + 1];                                      \
        const T xr = x[2 * (int64_t)col[k]], xi = x[2 * (int64_t)col[k] + 1];              \
        sr = FMA(-ai, xi, FMA(ar, xr, sr));                                                \
        si = FMA(ai, xr, FMA(ar, xi, si));                                                 \
      }                                                                                    \
      const T yr = y[2 * i], yi = y[2 * i + 1];                                            \
      const T tr = FMA(-alpha[1], si, alpha[0] * sr), ti = FMA(alpha[1], sr, alpha[0] * si); \
      const T ur = FMA(-beta[1], yi, beta[0] * yr), ui = FMA(beta[1], yr, beta[0] * yi);   \
      y[2 * i] = tr + ur;                                                                  \
      y[2 * i + 1] = ti + ui;                                                              \
    }                                                                                      \
  }
DEF_SPMV_CPLX(oracle_spmv_c32_i32, float, int32_t, fmaf)
DEF_SPMV_CPLX(oracle_spmv_c32_i64, float, int64_t, fmaf)
DEF_SPMV_CPLX(oracle_spmv_c64_i32, double, int32_t, fma)
DEF_SPMV_CPLX(oracle_spmv_c64_i64, double, int64_t, fma)

/* int8 A and x.  The reference has no CPU path for these instances (its hygon backend knows s, d, c, z
 * only), so nothing pins them beyond the arithmetic its CUDA dispatcher instantiates
 * (cuda/kernel/level2/alphasparse_spmv.cu:276-287): int32 products and sums with int32 alpha / beta
 * and y, or values widened to float with float alpha / beta and y.  Parity unpinned for these two. */
#define DEF_SPMV_I8(NAME, OFF_T, TY, ACC)                                                  \
  void NAME(int64_t rows, const OFF_T* row_ptr, const int32_t* col, const int8_t* val,     \
            const int8_t* x, TY alpha, TY beta, TY* y) {                                   \
    _Pragma("omp parallel for schedule(static)")                                           \
    for (int64_t i = 0; i < rows; ++i) {                                                   \
      TY s = 0;                                                                            \
      for (int64_t k = (int64_t)row_ptr[i]; k < (int64_t)row_ptr[i + 1]; ++k) ACC;         \
      y[i] = alpha * s + beta * y[i];                                                      \
    }                                                                                      \
  }
DEF_SPMV_I8(oracle_spmv_i8_i32_i32, int32_t, int32_t, s += (int32_t)val[k] * (int32_t)x[col[k]])
DEF_SPMV_I8(oracle_spmv_i8_i32_i64, int64_t, int32_t, s += (int32_t)val[k] * (int32_t)x[col[k]])
DEF_SPMV_I8(oracle_spmv_i8_f32_i32, int32_t, float, s = fmaf((float)val[k], (float)x[col[k]], s))
DEF_SPMV_I8(oracle_spmv_i8_f32_i64, int64_t, float, s = fmaf((float)val[k], (float)x[col[k]], s))

/* Row-major SpMM, X is cols x n with leading dimension ldx, Y is rows x n with ldy. */
#define DEF_SPMM(NAME, T, OFF_T, FMA)                                                      \
  void NAME(int64_t rows, const OFF_T* row_ptr, const int32_t* col, const T* val,          \
            const T* X, int64_t n, int64_t ldx, T alpha, T beta, T* Y, int64_t ldy) {      \
    _Pragma("omp parallel for schedule(static)")                                           \
    for (int64_t i = 0; i < rows; ++i) {                                                   \
      T* yr = Y + i * ldy;                                                                 \
      for (int64_t c = 0; c < n; ++c) yr[c] = yr[c] * beta;                                \
      for (int64_t k = (int64_t)row_ptr[i]; k < (int64_t)row_ptr[i + 1]; ++k) {            \
        const T a = alpha * val[k];                                                        \
        const T* xr = X + (int64_t)col[k] * ldx;                                           \
        for (int64_t c = 0; c < n; ++c) yr[c] = FMA(a, xr[c], yr[c]);                      \
      }                                                                                    \
    }                                                                                      \
  }

DEF_SPMM(oracle_spmm_f32_i32, float, int32_t, fmaf)
DEF_SPMM(oracle_spmm_f32_i64, float, int64_t, fmaf)
DEF_SPMM(oracle_spmm_f64_i32, double, int32_t, fma)
DEF_SPMM(oracle_spmm_f64_i64, double, int64_t, fma)

/* bf16 operands (A values and X stored as the upper 16 bits of an IEEE float), fp32
 * accumulation and fp32 Y: the arithmetic of the tensor-core SpMM variant, which the
 * reference does not have (its bf16 dispatch is commented out,
 * cuda/kernel/level3/alphasparse_spmm.cu:597-610).  Same loop as above after widening. */
static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
void oracle_spmm_bf16_i32(int64_t rows, const int32_t* row_ptr, const int32_t* col,
                          const uint16_t* val, const uint16_t* X, int64_t n, int64_t ldx,
                          float alpha, float beta, float* Y, int64_t ldy) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < rows; ++i) {
    float* yr = Y + i * ldy;
    for (int64_t c = 0; c < n; ++c) yr[c] = yr[c] * beta;
    for (int64_t k = row_ptr[i]; k < row_ptr[i + 1]; ++k) {
      const float a = alpha * bf16_to_f32(val[k]);
      const uint16_t* xr = X + (int64_t)col[k] * ldx;
      for (int64_t c = 0; c < n; ++c) yr[c] = fmaf(a, bf16_to_f32(xr[c]), yr[c]);
    }
  }
}

/* Complex SpMM (interleaved re, im), the generic row kernel of the reference's CPU backend
 * (hygon/kernel/level3/mm/gemm/gemm_csr_row.hpp:76-122 with J = complex): Y[r,:] = Y[r,:]*beta,
 * then for each entry of row r in storage order t = alpha*a and Y[r,c] = X[col,c]*t + Y[r,c].
 * Checked against the compiled reference within rounding (the compiler is free to contract its
 * complex products), not bit for bit. */
#define DEF_SPMM_CPLX(NAME, T, OFF_T, FMA)                                                 \
  void NAME(int64_t rows, const OFF_T* row_ptr, const int32_t* col, const T* val,          \
            const T* X, int64_t n, int64_t ldx, const T* alpha, const T* beta, T* Y,       \
            int64_t ldy) {                                                                 \
    _Pragma("omp parallel for schedule(static)")                                           \
    for (int64_t i = 0; i < rows; ++i) {                                                   \
      T* yr = Y + 2 * i * ldy;                                                             \
      for (int64_t c = 0; c < n; ++c) {                                                    \
        const T a = yr[2 * c], b = yr[2 * c + 1];                                          \
        yr[2 * c] = FMA(-b, beta[1], a * beta[0]);                                         \
        yr[2 * c + 1] = FMA(b, beta[0], a * beta[1]);                                      \
      }                                                                                    \
      for (int64_t k = (int64_t)row_ptr[i]; k < (int64_t)row_ptr[i + 1]; ++k) {            \
        const T ar = val[2 * k], ai = val[2 * k + 1];                                      \
        const T tr = FMA(-alpha[1], ai, alpha[0] * ar), ti = FMA(alpha[1], ar, alpha[0] * ai); \
        const T* xr = X + 2 * (int64_t)col[k] * ldx;                                       \
        for (int64_t c = 0; c < n; ++c) {                                                  \
          const T xa = xr[2 * c], xb = xr[2 * c + 1];                                      \
          yr[2 * c] = FMA(-xb, ti, FMA(xa, tr, yr[2 * c]));                                \
          yr[2 * c + 1] = FMA(xb, tr, FMA(xa, ti, yr[2 * c + 1]));                         \
        }                                                                                  \
      }                                                                                    \
    }                                                                                      \
  }
DEF_SPMM_CPLX(oracle_spmm_c32_i32, float, int32_t, fmaf)
DEF_SPMM_CPLX(oracle_spmm_c32_i64, float, int64_t, fmaf)
DEF_SPMM_CPLX(oracle_spmm_c64_i32, double, int32_t, fma)
DEF_SPMM_CPLX(oracle_spmm_c64_i64, double, int64_t, fma)

/* int8 and fp16 SpMM.  The reference has no CPU path for these instances, so nothing pins them
 * beyond the arithmetic its CUDA dispatcher instantiates (cuda/kernel/level3/alphasparse_spmm.cu:
 * 572-596): per element of Y a sum over the row's entries in storage order, then
 * alpha*sum + beta*y -  int32 products and sums (wrapping, as the device's), or values widened to
 * float with float sums, alpha and beta; the fp16 -> fp16 instance rounds once at the end (to
 * nearest even).  Parity unpinned for these four. */
static inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, u;
  if (exp == 0) {
    if (man == 0) u = sign;
    else {                                  /* subnormal: normalise */
      int sh = 0;
      while (!(man & 0x400u)) { man <<= 1; ++sh; }
      man &= 0x3FFu;
      u = sign | ((uint32_t)(127 - 15 - sh + 1) << 23) | (man << 13);
    }
  } else if (exp == 31) u = sign | 0x7F800000u | (man << 13);
  else u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  float f;
  memcpy(&f, &u, 4);
  return f;
}
static inline uint16_t f32_to_f16(float f) {   /* round to nearest even */
  uint32_t u;
  memcpy(&u, &f, 4);
  const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  const uint32_t a = u & 0x7FFFFFFFu;
  if (a >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (a > 0x7F800000u ? 0x200u : 0u));
  if (a >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);            /* rounds to infinity */
  if (a < 0x33000001u) return sign;                                    /* rounds to zero */
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
  int shift = e < -14 ? 13 + (-14 - e) : 13;                           /* subnormal halves lose more bits */
  uint32_t q = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q;
  if (e < -14) return (uint16_t)(sign | q);                            /* q may carry into the exponent: still right */
  return (uint16_t)(sign | (uint16_t)((((uint32_t)(e + 15)) << 10) + (q - 0x400u)));
}
#define DEF_SPMM_WIDE(NAME, OFF_T, TA, TY, TS, LOAD, MAD, FINISH)                          \
  void NAME(int64_t rows, const OFF_T* row_ptr, const int32_t* col, const TA* val,         \
            const TA* X, int64_t n, int64_t ldx, TS alpha, TS beta, TY* Y, int64_t ldy) {  \
    _Pragma("omp parallel for schedule(static)")                                           \
    for (int64_t i = 0; i < rows; ++i)                                                     \
      for (int64_t c = 0; c < n; ++c) {                                                    \
        TS s = 0;                                                                          \
        for (int64_t k = (int64_t)row_ptr[i]; k < (int64_t)row_ptr[i + 1]; ++k) {          \
          const TS a = LOAD(val[k]), x = LOAD(X[(int64_t)col[k] * ldx + c]);               \
          s = MAD;                                                                         \
        }                                                                                  \
        TY* y = Y + i * ldy + c;                                                           \
        *y = FINISH;                                                                       \
      }                                                                                    \
  }
#define ID_(v) (v)
#define I32_(v) ((int32_t)(v))
#define F32_(v) ((float)(v))
#define WRAP_MAD_ (int32_t)((uint32_t)s + (uint32_t)a * (uint32_t)x)
#define WRAP_FIN_ (int32_t)((uint32_t)alpha * (uint32_t)s + (beta == 0 ? 0u : (uint32_t)beta * (uint32_t)*y))
#define F_FIN_ (beta == 0.f ? alpha * s : fmaf(alpha, s, beta * *y))
#define H_FIN_ f32_to_f16(beta == 0.f ? alpha * s : fmaf(alpha, s, beta * f16_to_f32(*y)))
DEF_SPMM_WIDE(oracle_spmm_i8_i32_i32, int32_t, int8_t, int32_t, int32_t, I32_, WRAP_MAD_, WRAP_FIN_)
DEF_SPMM_WIDE(oracle_spmm_i8_i32_i64, int64_t, int8_t, int32_t, int32_t, I32_, WRAP_MAD_, WRAP_FIN_)
DEF_SPMM_WIDE(oracle_spmm_i8_f32_i32, int32_t, int8_t, float, float, F32_, fmaf(a, x, s), F_FIN_)
DEF_SPMM_WIDE(oracle_spmm_i8_f32_i64, int64_t, int8_t, float, float, F32_, fmaf(a, x, s), F_FIN_)
DEF_SPMM_WIDE(oracle_spmm_f16_f32_i32, int32_t, uint16_t, float, float, f16_to_f32, fmaf(a, x, s), F_FIN_)
DEF_SPMM_WIDE(oracle_spmm_f16_f32_i64, int64_t, uint16_t, float, float, f16_to_f32, fmaf(a, x, s), F_FIN_)
DEF_SPMM_WIDE(oracle_spmm_f16_f16_i32, int32_t, uint16_t, uint16_t, float, f16_to_f32, fmaf(a, x, s), H_FIN_)
DEF_SPMM_WIDE(oracle_spmm_f16_f16_i64, int64_t, uint16_t, uint16_t, float, f16_to_f32, fmaf(a, x, s), H_FIN_)

/* Contiguous row ranges of near-equal nnz: bound[0]=0, bound[parts]=rows and
 * bound[i] = first index j in [0, rows-1] with row_end[j] >= (nnz/parts)*i, where
 * row_end = row_ptr+1 (hygon/util/partition.cpp:83-96 with lower_bound_int :41-57). */
#define DEF_PARTITION(NAME, OFF_T)                                                         \
  void NAME(const OFF_T* row_ptr, int64_t rows, int64_t parts, int64_t* bound) {           \
    const OFF_T* row_end = row_ptr + 1;                                                    \
    bound[0] = 0;                                                                          \
    if (rows <= 0) {                                                                       \
      for (int64_t i = 1; i <= parts; ++i) bound[i] = 0;                                   \
      return;                                                                              \
    }                                                                                      \
    int64_t nnz = (int64_t)row_end[rows - 1];                                              \
    int64_t ave = nnz / parts;                                                             \
    for (int64_t i = 1; i < parts; ++i) {                                                  \
      int64_t l = 0, r = rows - 1, v = ave * i;                                            \
      while (r > l) {                                                                      \
        int64_t m = (l + r) / 2;                                                           \
        if ((int64_t)row_end[m] < v) l = m + 1; else r = m;                                \
      }                                                                                    \
      bound[i] = l;                                                                        \
    }                                                                                      \
    bound[parts] = rows;                                                                   \
  }

DEF_PARTITION(oracle_partition_rows_by_nnz_i32, int32_t)
DEF_PARTITION(oracle_partition_rows_by_nnz_i64, int64_t)
