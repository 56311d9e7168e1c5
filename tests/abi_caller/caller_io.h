// Input / output files of the two compiled callers (tests/test_compiled_caller.py writes and reads them).
//   input : int64 header[6] = {kind (0 SpMV, 1 SpMM), rows, cols, nnz, n, reserved}, float alpha, float beta,
//           int32 coo_row[nnz] (ascending), int32 coo_col[nnz], float val[nnz],
//           float dense_in[cols * n] (x, or row-major B), float dense_out[rows * n] (y0, or row-major C0)
//   output: float dense_out[rows * n]
#pragma once
#include <cstdint>
#include <cstdio>
#include <vector>

struct CallerInput {
  int64_t kind = 0, rows = 0, cols = 0, nnz = 0, n = 1;
  float alpha = 1.f, beta = 0.f;
  std::vector<int> coo_row, coo_col;
  std::vector<float> val, dense_in, dense_out;
};

inline bool read_input(const char* path, CallerInput* in) {
  FILE* f = fopen(path, "rb");
  if (!f) return false;
  int64_t hdr[6];
  bool ok = fread(hdr, sizeof(int64_t), 6, f) == 6;
  if (ok) {
    in->kind = hdr[0]; in->rows = hdr[1]; in->cols = hdr[2]; in->nnz = hdr[3]; in->n = hdr[4];
    ok = fread(&in->alpha, 4, 1, f) == 1 && fread(&in->beta, 4, 1, f) == 1;
  }
  auto rd = [&](auto& v, size_t count) {
    v.resize(count);
    return count == 0 || fread(v.data(), sizeof(v[0]), count, f) == count;
  };
  ok = ok && rd(in->coo_row, (size_t)in->nnz) && rd(in->coo_col, (size_t)in->nnz) && rd(in->val, (size_t)in->nnz) &&
       rd(in->dense_in, (size_t)(in->cols * in->n)) && rd(in->dense_out, (size_t)(in->rows * in->n));
  fclose(f);
  return ok;
}

inline bool write_output(const char* path, const std::vector<float>& out) {
  FILE* f = fopen(path, "wb");
  if (!f) return false;
  const bool ok = out.empty() || fwrite(out.data(), sizeof(float), out.size(), f) == out.size();
  fclose(f);
  return ok;
}
