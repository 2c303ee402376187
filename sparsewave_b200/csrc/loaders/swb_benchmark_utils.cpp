// libsparsewave_benchmark_utils.so: benchmark input loaders with the symbols and behaviour of the library the
// SparseWave tree builds from benchmark/SparseBenchmarkUtils.cpp, plus a Matrix Market converter.  Host C++ only.
#include "../../../include/sparsewave_benchmark_utils.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <numeric>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

constexpr uint64_t kI64Max = (uint64_t)std::numeric_limits<int64_t>::max();

// Every loader failure is fatal for the benchmark program that called it.
[[noreturn]] void die(const std::string &why) {
  fprintf(stderr, "SparseWave benchmark input error: %s\n", why.c_str());
  fflush(stderr);
  abort();
}

// A binary matrix file being consumed front to back.
class InputFile {
 public:
  InputFile(const char *env_name) {
    const char *path = getenv(env_name);
    if (!path) die(std::string(env_name) + " is not set");
    f_ = fopen(path, "rb");
    if (!f_) die(std::string("could not open ") + path);
  }
  ~InputFile() { if (f_) fclose(f_); }
  InputFile(const InputFile &) = delete;
  InputFile &operator=(const InputFile &) = delete;

  void bytes(void *dst, uint64_t n, const std::string &what) {
    if (n > 0 && fread(dst, 1, n, f_) != n) die("could not read " + what);
  }
  uint64_t u64(const char *what) {
    uint64_t v = 0;
    bytes(&v, sizeof v, what);
    return v;
  }
  // magic + rows, columns, nnz
  void header(const char *magic, const char *format, uint64_t &rows, uint64_t &cols, uint64_t &nnz) {
    char got[8];
    if (fread(got, 1, 8, f_) != 8 || memcmp(got, magic, 8) != 0)
      die(std::string("invalid ") + format + " binary header");
    rows = u64("row count");
    cols = u64("column count");
    nnz = u64("NNZ count");
    if (rows > kI64Max || cols > kI64Max || nnz > kI64Max)
      die(std::string(format) + " dimensions exceed the runner limits");
  }
  // `count` elements into a unit-stride rank-1 memref of exactly that size
  template <typename M>
  void into(M *m, uint64_t count, const char *what) {
    if (m->sizes[0] != (int64_t)count || m->strides[0] != 1) die(std::string(what) + " memref has an unexpected layout");
    bytes(m->data + m->offset, count * sizeof(*m->data), what);
  }
  template <typename T>
  std::vector<T> vec(uint64_t count, const char *what) {
    if (count > kI64Max) die(std::string(what) + " exceeds the runner limits");
    std::vector<T> v(count);
    bytes(v.data(), count * sizeof(T), what);
    return v;
  }

 private:
  FILE *f_ = nullptr;
};

template <typename M>
auto *at(M *m) { return m->data + m->offset; }

void ones(swbu_memref_f32 *vector, uint64_t n) {
  if (vector->sizes[0] != (int64_t)n || vector->strides[0] != 1) die("vector memref has an unexpected layout");
  std::fill_n(at(vector), n, 1.0f);
}

void zeros(swbu_memref_f32 *expected, uint64_t n) {
  if (expected->sizes[0] != (int64_t)n || expected->strides[0] != 1)
    die("expected-output memref has an unexpected layout");
  std::fill_n(at(expected), n, 0.0f);
}

// Row-major identity layout of the two dense operands of SpMM, and the fixed right-hand side.
void check_dense_pair(swbu_memref_f32_2d *rhs, swbu_memref_f32_2d *expected, uint64_t rows, uint64_t cols) {
  const bool rhs_ok = rhs->sizes[0] == (int64_t)cols && rhs->sizes[1] >= 1 && rhs->strides[1] == 1 &&
                      rhs->strides[0] == rhs->sizes[1];
  if (!rhs_ok) die("RHS memref has an unexpected layout");
  const bool out_ok = expected->sizes[0] == (int64_t)rows && expected->sizes[1] == rhs->sizes[1] &&
                      expected->strides[1] == 1 && expected->strides[0] == expected->sizes[1];
  if (!out_ok) die("expected-output memref has an unexpected layout");
}

void fill_rhs_pattern(swbu_memref_f32_2d *rhs) {
  float *b = at(rhs);
  const int64_t k_count = rhs->sizes[0], n = rhs->sizes[1];
  for (int64_t k = 0; k < k_count; ++k)
    for (int64_t j = 0; j < n; ++j) b[k * n + j] = 1.0f + (float)((uint64_t)(k + j) % 7) * 0.125f;
}

struct Csr { uint64_t rows, cols, nnz; };

Csr read_csr(swbu_memref_i32 *row_offsets, swbu_memref_i32 *column_indices, swbu_memref_f32 *values) {
  InputFile in("SPARSEWAVE_BENCHMARK_CSR");
  Csr d{};
  in.header("SWCSR001", "CSR", d.rows, d.cols, d.nnz);
  in.into(row_offsets, d.rows + 1, "row offsets");
  in.into(column_indices, d.nnz, "column indices");
  in.into(values, d.nnz, "values");
  return d;
}

}  // namespace

extern "C" {

void _mlir_ciface_loadCSRSpMVBenchmarkInputs(swbu_memref_i32 *row_offsets, swbu_memref_i32 *column_indices,
                                             swbu_memref_f32 *values, swbu_memref_f32 *vector,
                                             swbu_memref_f32 *expected) {
  const Csr d = read_csr(row_offsets, column_indices, values);
  ones(vector, d.cols);
  zeros(expected, d.rows);
  const int32_t *rp = at(row_offsets);
  const float *v = at(values);
  float *y = at(expected);
  for (uint64_t r = 0; r < d.rows; ++r) {  // x == 1: the row sum, single precision, position order
    float sum = 0.0f;
    for (int32_t p = rp[r]; p < rp[r + 1]; ++p) sum += v[p];
    y[r] = sum;
  }
}

void _mlir_ciface_loadCOOSpMVBenchmarkInputs(swbu_memref_i32 *row_indices, swbu_memref_i32 *column_indices,
                                             swbu_memref_f32 *values, swbu_memref_f32 *vector,
                                             swbu_memref_f32 *expected) {
  uint64_t rows, cols, nnz;
  {
    InputFile in("SPARSEWAVE_BENCHMARK_COO");
    in.header("SWCOO001", "COO", rows, cols, nnz);
    in.into(row_indices, nnz, "row indices");
    in.into(column_indices, nnz, "column indices");
    in.into(values, nnz, "values");
  }
  ones(vector, cols);
  zeros(expected, rows);
  const int32_t *ri = at(row_indices), *ci = at(column_indices);
  const float *v = at(values);
  float *y = at(expected);
  for (uint64_t p = 0; p < nnz; ++p) {
    if (ri[p] < 0 || (uint64_t)ri[p] >= rows || ci[p] < 0 || (uint64_t)ci[p] >= cols)
      die("COO coordinate is out of bounds");
    y[ri[p]] += v[p];
  }
}

void _mlir_ciface_loadSpMMBenchmarkInputs(swbu_memref_i32 *row_offsets, swbu_memref_i32 *column_indices,
                                          swbu_memref_f32 *values, swbu_memref_f32_2d *rhs,
                                          swbu_memref_f32_2d *expected) {
  const Csr d = read_csr(row_offsets, column_indices, values);
  check_dense_pair(rhs, expected, d.rows, d.cols);
  fill_rhs_pattern(rhs);
  const int32_t *rp = at(row_offsets), *ci = at(column_indices);
  const float *v = at(values), *b = at(rhs);
  float *c = at(expected);
  const int64_t n = rhs->sizes[1];
  for (uint64_t r = 0; r < d.rows; ++r)
    for (int64_t j = 0; j < n; ++j) {
      float sum = 0.0f;
      for (int32_t p = rp[r]; p < rp[r + 1]; ++p) sum += v[p] * b[(int64_t)ci[p] * n + j];
      c[r * n + j] = sum;
    }
}

void _mlir_ciface_loadBSRSpMMBenchmarkInputs(swbu_memref_i32 *block_row_offsets, swbu_memref_i32 *block_column_indices,
                                             swbu_memref_f32 *block_values, swbu_memref_f32_2d *rhs,
                                             swbu_memref_f32_2d *expected) {
  uint64_t rows, cols, nnzb, bs, orig_rows, orig_cols, orig_nnz;
  std::vector<int32_t> in_rows, in_cols;
  std::vector<float> in_vals;
  {
    InputFile in("SPARSEWAVE_BENCHMARK_BSR");
    in.header("SWBSR001", "BSR", rows, cols, nnzb);
    bs = in.u64("block size");
    orig_rows = in.u64("original row count");
    orig_cols = in.u64("original column count");
    orig_nnz = in.u64("original NNZ count");
    if (bs == 0 || rows % bs != 0 || cols % bs != 0) die("BSR dimensions must be divisible by a positive block size");
    if (orig_rows > rows || orig_cols > cols) die("original BSR dimensions exceed the padded dimensions");
    if (bs > kI64Max || nnzb > kI64Max / bs / bs) die("BSR block values exceed the runner limits");
    in.into(block_row_offsets, rows / bs + 1, "block-row offsets");
    in.into(block_column_indices, nnzb, "block-column indices");
    in.into(block_values, nnzb * bs * bs, "block values");
    in_rows = in.vec<int32_t>(orig_nnz, "input row indices");
    in_cols = in.vec<int32_t>(orig_nnz, "input column indices");
    in_vals = in.vec<float>(orig_nnz, "input values");
  }
  check_dense_pair(rhs, expected, rows, cols);
  fill_rhs_pattern(rhs);
  const float *b = at(rhs);
  float *c = at(expected);
  const int64_t n = rhs->sizes[1];
  std::fill_n(c, rows * (uint64_t)n, 0.0f);
  // The expected output comes from the entries the blocks were built from, not from the padded blocks.
  for (uint64_t e = 0; e < orig_nnz; ++e) {
    const int32_t r = in_rows[e], k = in_cols[e];
    if (r < 0 || (uint64_t)r >= orig_rows || k < 0 || (uint64_t)k >= orig_cols)
      die("original BSR input coordinate is out of bounds");
    for (int64_t j = 0; j < n; ++j) c[(int64_t)r * n + j] += in_vals[e] * b[(int64_t)k * n + j];
  }
}

}  // extern "C"
