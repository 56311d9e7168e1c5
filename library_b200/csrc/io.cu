// Host-side readers for the step before the path: a MatrixMarket coordinate file to COO arrays, and
// the (row, column) ordering that CSR conversion needs.  They replace what the reference's test
// drivers use before alphasparseXcoo2csr: alpha_read_coo<T> (cuda/test/io.cu:1227-1238 and the
// MatrixMarket parser :103-184, :490-575) and coo_order (cuda/format/coo_order.h:25-43).
// Behaviour kept from the reference's reader: indices become zero-based; a "pattern" entry gets the
// value 1; for symmetric, Hermitian and skew-symmetric files every off-diagonal entry is followed by
// its mirror image WITH THE SAME VALUE (the reference does not negate for skew-symmetric files).
// Differences: errors are returned as status codes (the reference prints and calls exit), 64-bit
// counts, bounds of every index are checked.  alphasparseReadBinCoo reads the binary dump format of the
// reference's drivers (bin_header, cuda/test/include/io.h:41-50; records, cuda/test/io.cu:596-725).
#include <algorithm>
#include <cctype>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <numeric>
#include <string>
#include <vector>

#include "alphasparse_b200.h"

namespace {

bool next_data_line(FILE* fp, std::string& line) {
  char buf[1024];
  for (;;) {
    line.clear();
    bool got = false;
    while (fgets(buf, sizeof buf, fp)) {
      got = true;
      line += buf;
      if (!line.empty() && line.back() == '\n') break;
    }
    if (!got) return false;
    size_t i = 0;
    while (i < line.size() && isspace((unsigned char)line[i])) ++i;
    if (i == line.size() || line[i] == '%') continue;  // blank or comment
    return true;
  }
}

std::string lower(std::string s) {
  for (auto& c : s) c = (char)tolower((unsigned char)c);
  return s;
}

template <typename T>
alphasparseStatus_t read_t(FILE* fp, bool mirror, int64_t m, int64_t n, int64_t lines, int32_t** ri, int32_t** ci,
                           void** vals, int64_t* nnz) {
  std::vector<int32_t> r, c;
  std::vector<T> v;
  // the announced count comes from the file: reserve at most 64 M entries ahead, the vectors grow beyond that
  const size_t ahead = (size_t)(lines < (1ll << 26) ? lines : (1ll << 26)) * (mirror ? 2 : 1);
  r.reserve(ahead);
  c.reserve(ahead);
  v.reserve(ahead);
  std::string line;
  for (int64_t i = 0; i < lines; ++i) {
    if (!next_data_line(fp, line)) return ALPHA_SPARSE_STATUS_INVALID_VALUE;  // fewer entries than announced
    char* p = nullptr;
    const long long row = strtoll(line.c_str(), &p, 10);
    char* q = nullptr;
    const long long col = strtoll(p, &q, 10);
    if (p == line.c_str() || q == p) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (row < 1 || row > m || col < 1 || col > n) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    char* e = nullptr;
    const double x = strtod(q, &e);
    const T val = e == q ? T(1) : (T)x;  // no value field: a pattern entry
    r.push_back((int32_t)(row - 1));
    c.push_back((int32_t)(col - 1));
    v.push_back(val);
    if (mirror && row != col) {
      r.push_back((int32_t)(col - 1));
      c.push_back((int32_t)(row - 1));
      v.push_back(val);
    }
  }
  const size_t k = r.size();
  *ri = (int32_t*)malloc((k ? k : 1) * sizeof(int32_t));
  *ci = (int32_t*)malloc((k ? k : 1) * sizeof(int32_t));
  *vals = malloc((k ? k : 1) * sizeof(T));
  if (!*ri || !*ci || !*vals) {
    free(*ri);
    free(*ci);
    free(*vals);
    *ri = *ci = nullptr;
    *vals = nullptr;
    return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  }
  if (k) {
    memcpy(*ri, r.data(), k * sizeof(int32_t));
    memcpy(*ci, c.data(), k * sizeof(int32_t));
    memcpy(*vals, v.data(), k * sizeof(T));
  }
  *nnz = (int64_t)k;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

template <typename T>
void order_t(int64_t nnz, int32_t* ri, int32_t* ci, T* v) {
  std::vector<int64_t> idx((size_t)nnz);
  std::iota(idx.begin(), idx.end(), (int64_t)0);
  std::stable_sort(idx.begin(), idx.end(), [&](int64_t a, int64_t b) {
    return ri[a] != ri[b] ? ri[a] < ri[b] : ci[a] < ci[b];
  });
  std::vector<int32_t> r2((size_t)nnz), c2((size_t)nnz);
  std::vector<T> v2((size_t)nnz);
  for (int64_t i = 0; i < nnz; ++i) {
    r2[i] = ri[idx[i]];
    c2[i] = ci[idx[i]];
    v2[i] = v[idx[i]];
  }
  memcpy(ri, r2.data(), (size_t)nnz * sizeof(int32_t));
  memcpy(ci, c2.data(), (size_t)nnz * sizeof(int32_t));
  memcpy(v, v2.data(), (size_t)nnz * sizeof(T));
}

}  // namespace

extern "C" {

alphasparseStatus_t alphasparseReadMtxCoo(const char* file, int64_t* rows, int64_t* cols, int64_t* nnz,
                                          int32_t** row_index, int32_t** col_index, void** values,
                                          alphasparseDataType valueType) {
  if (!file || !rows || !cols || !nnz || !row_index || !col_index || !values) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (valueType != ALPHA_R_32F && valueType != ALPHA_R_64F) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  *row_index = *col_index = nullptr;
  *values = nullptr;
  *rows = *cols = *nnz = 0;
  FILE* fp = fopen(file, "r");
  if (!fp) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
  alphasparseStatus_t st = ALPHA_SPARSE_STATUS_SUCCESS;
  bool mirror = false;
  char head[1024];
  if (!fgets(head, sizeof head, fp)) {
    fclose(fp);
    return ALPHA_SPARSE_STATUS_INVALID_VALUE;
  }
  if (head[0] == '%') {
    // %%MatrixMarket matrix coordinate <field> <symmetry>
    char banner[64] = "", object[64] = "", format[64] = "", field[64] = "", symm[64] = "";
    sscanf(head, "%63s %63s %63s %63s %63s", banner, object, format, field, symm);
    if (lower(format) == "array") st = ALPHA_SPARSE_STATUS_NOT_SUPPORTED;   // dense files
    if (lower(field) == "complex") st = ALPHA_SPARSE_STATUS_NOT_SUPPORTED;  // real value types only
    const std::string sy = lower(symm);
    mirror = sy == "symmetric" || sy == "hermitian" || sy == "skew-symmetric";
  } else {
    rewind(fp);  // no banner: the first data line is the size line of a general real matrix
  }
  std::string line;
  long long m = 0, n = 0, lines = 0;
  if (st == ALPHA_SPARSE_STATUS_SUCCESS &&
      (!next_data_line(fp, line) || sscanf(line.c_str(), "%lld %lld %lld", &m, &n, &lines) != 3 || m < 0 || n < 0 ||
       lines < 0 || m >= (1ll << 31) || n >= (1ll << 31)))
    st = ALPHA_SPARSE_STATUS_INVALID_VALUE;
  if (st == ALPHA_SPARSE_STATUS_SUCCESS) {
    try {  // no C++ exception may cross the C boundary
      st = valueType == ALPHA_R_32F ? read_t<float>(fp, mirror, m, n, lines, row_index, col_index, values, nnz)
                                    : read_t<double>(fp, mirror, m, n, lines, row_index, col_index, values, nnz);
    } catch (...) {
      st = ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
  }
  fclose(fp);
  if (st == ALPHA_SPARSE_STATUS_SUCCESS) {
    *rows = m;
    *cols = n;
  }
  return st;
}

// The reference's binary matrix dump: a header of eight int64 (rows, cols, records, entries after
// mirroring, value fields per record - 0 pattern, 1 real, 2 complex -, number type, symmetry - 0
// general -, reserved), then one record per stored entry: int32 row and column (one-based) followed
// by that many doubles.  As in the reference's reader (cuda/test/io.cu:603-725) a pattern entry gets
// the value 1, a complex entry contributes its real part, and for a symmetric file every
// off-diagonal record is followed by its mirror image with the same value.
alphasparseStatus_t alphasparseReadBinCoo(const char* file, int64_t* rows, int64_t* cols, int64_t* nnz,
                                          int32_t** row_index, int32_t** col_index, void** values,
                                          alphasparseDataType valueType) {
  if (!file || !rows || !cols || !nnz || !row_index || !col_index || !values) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  if (valueType != ALPHA_R_32F && valueType != ALPHA_R_64F) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  *row_index = *col_index = nullptr;
  *values = nullptr;
  FILE* fp = fopen(file, "rb");
  if (!fp) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
  int64_t hdr[8];
  if (fread(hdr, sizeof(int64_t), 8, fp) != 8) {
    fclose(fp);
    return ALPHA_SPARSE_STATUS_INVALID_VALUE;
  }
  const int64_t m = hdr[0], n = hdr[1], records = hdr[2], fields = hdr[4];
  const bool mirror = hdr[6] != 0;
  if (m < 0 || n < 0 || records < 0 || m >= (int64_t(1) << 31) || n >= (int64_t(1) << 31) || fields < 0 || fields > 2) {
    fclose(fp);
    return fields > 2 ? ALPHA_SPARSE_STATUS_NOT_SUPPORTED : ALPHA_SPARSE_STATUS_INVALID_VALUE;
  }
  const size_t es = valueType == ALPHA_R_64F ? 8 : 4;
  const int64_t cap = mirror ? 2 * records : records;
  int32_t* ri = (int32_t*)malloc(sizeof(int32_t) * (size_t)(cap > 0 ? cap : 1));
  int32_t* ci = (int32_t*)malloc(sizeof(int32_t) * (size_t)(cap > 0 ? cap : 1));
  void* v = malloc(es * (size_t)(cap > 0 ? cap : 1));
  alphasparseStatus_t st = (ri && ci && v) ? ALPHA_SPARSE_STATUS_SUCCESS : ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  int64_t k = 0;
  for (int64_t i = 0; i < records && st == ALPHA_SPARSE_STATUS_SUCCESS; ++i) {
    int32_t rc[2];
    double f[2] = {1.0, 0.0};
    if (fread(rc, sizeof(int32_t), 2, fp) != 2 || (fields > 0 && fread(f, sizeof(double), (size_t)fields, fp) != (size_t)fields)) {
      st = ALPHA_SPARSE_STATUS_INVALID_VALUE;  // the file ends before the announced records do
      break;
    }
    const int64_t r = (int64_t)rc[0] - 1, c = (int64_t)rc[1] - 1;
    if (r < 0 || r >= m || c < 0 || c >= n) {
      st = ALPHA_SPARSE_STATUS_INVALID_VALUE;
      break;
    }
    for (int copy = 0; copy < ((mirror && r != c) ? 2 : 1); ++copy) {
      ri[k] = (int32_t)(copy ? c : r);
      ci[k] = (int32_t)(copy ? r : c);
      if (es == 8) ((double*)v)[k] = f[0];
      else ((float*)v)[k] = (float)f[0];
      ++k;
    }
  }
  fclose(fp);
  if (st != ALPHA_SPARSE_STATUS_SUCCESS) {
    free(ri);
    free(ci);
    free(v);
    return st;
  }
  *rows = m;
  *cols = n;
  *nnz = k;
  *row_index = ri;
  *col_index = ci;
  *values = v;
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparseStatus_t alphasparseCooOrder(int64_t nnz, int32_t* row_index, int32_t* col_index, void* values,
                                        alphasparseDataType valueType) {
  if (nnz < 0) return ALPHA_SPARSE_STATUS_INVALID_SIZE;
  if (nnz > 0 && (!row_index || !col_index || !values)) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
  try {
    if (valueType == ALPHA_R_32F) order_t<float>(nnz, row_index, col_index, (float*)values);
    else if (valueType == ALPHA_R_64F) order_t<double>(nnz, row_index, col_index, (double*)values);
    else return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
  } catch (...) {
    return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
  }
  return ALPHA_SPARSE_STATUS_SUCCESS;
}

void alphasparseFreeHost(void* p) { free(p); }

}  // extern "C"
