// Matrix Market -> SWCSR001 / SWCOO001 / SWBSR001, the C++ form of the conversion the SparseWave benchmark
// drivers do in Python (benchmark/benchmark_utils.py:56-379).  Part of libsparsewave_benchmark_utils.so.
#include "../../../include/sparsewave_benchmark_utils.h"

#include <algorithm>
#include <cctype>
#include <cerrno>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <numeric>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

namespace {

constexpr int64_t kI32Max = 2147483647LL;

// Entries in (row, column) order (stable: equal coordinates keep their file order, a mirrored entry follows
// its original), values still in double: they are rounded to f32 when a file is written, as the reference's
// struct.pack("<f") does, so that sums of duplicates (BSR) see the unrounded values.
struct Coo {
  int64_t rows = 0, cols = 0;
  std::vector<int32_t> row, col;
  std::vector<double> val;
};

std::string lower(std::string s) {
  for (char &c : s) c = (char)tolower((unsigned char)c);
  return s;
}

std::vector<std::string> split(const std::string &line) {
  std::istringstream in(line);
  std::vector<std::string> out;
  for (std::string t; in >> t;) out.push_back(t);
  return out;
}

bool blank_or_comment(const std::string &line) {
  for (char c : line) {
    if (isspace((unsigned char)c)) continue;
    return c == '%';
  }
  return true;
}

bool to_int(const std::string &t, int64_t &out) {
  char *end = nullptr;
  errno = 0;
  const long long v = strtoll(t.c_str(), &end, 10);
  if (end == t.c_str() || *end != '\0' || errno == ERANGE) return false;
  out = v;
  return true;
}

bool to_double(const std::string &t, double &out) {
  char *end = nullptr;
  const double v = strtod(t.c_str(), &end);
  if (end == t.c_str() || *end != '\0') return false;
  out = v;
  return true;
}

// double -> f32 as struct.pack("<f") does: round to nearest, refuse what rounds to infinity
bool fits_f32(double v) { return std::isfinite((double)(float)v) || !std::isfinite(v); }

[[noreturn]] void fail(const std::string &path, const std::string &what) { throw std::runtime_error(path + ": " + what); }
[[noreturn]] void fail_at(const std::string &path, int64_t line, const std::string &what) {
  throw std::runtime_error(path + ":" + std::to_string(line) + ": " + what);
}

// read_matrix_market of the reference drivers (benchmark/benchmark_utils.py:56-177), check for check and
// message for message: coordinate files only; fields real, integer, pattern (value 1); symmetry general or
// symmetric (expanded, square matrices only); blank and comment lines are skipped anywhere; every entry line
// has exactly the expected number of fields, indices in range, a finite value that fits f32; the number of
// entries read equals the declared one; the entries are then ordered by (row, column).
Coo read_matrix_market(const char *path_c) {
  const std::string path = path_c;
  std::ifstream f(path_c);
  if (!f) throw std::runtime_error("could not open " + path);
  std::string line;
  std::getline(f, line);
  const std::vector<std::string> head = split(line);
  if (head.size() != 5 || head[0] != "%%MatrixMarket" || head[1] != "matrix" || head[2] != "coordinate")
    fail(path, "expected a Matrix Market coordinate matrix");
  const std::string field = lower(head[3]), symmetry = lower(head[4]);
  if (field != "real" && field != "integer" && field != "pattern") fail(path, "unsupported Matrix Market field '" + field + "'");
  if (symmetry != "general" && symmetry != "symmetric") fail(path, "unsupported Matrix Market symmetry '" + symmetry + "'");
  const bool pattern = field == "pattern", integer = field == "integer", mirrored = symmetry == "symmetric";

  bool have_size = false;
  while (std::getline(f, line)) {
    if (!blank_or_comment(line)) {
      have_size = true;
      break;
    }
  }
  if (!have_size) fail(path, "missing matrix dimensions");
  const std::vector<std::string> size = split(line);
  Coo m;
  int64_t declared = 0;
  if (size.size() != 3 || !to_int(size[0], m.rows) || !to_int(size[1], m.cols) || !to_int(size[2], declared))
    fail(path, "invalid matrix dimensions");
  if (m.rows <= 0 || m.cols <= 0 || declared < 0) fail(path, "matrix dimensions must be nonnegative");
  if (mirrored && m.rows != m.cols) fail(path, "a symmetric matrix must be square");

  std::vector<int32_t> row, col;
  std::vector<double> val;
  int64_t read = 0;
  const size_t expected = pattern ? 2 : 3;
  for (int64_t line_number = 3; std::getline(f, line); ++line_number) {  // the reference counts from 3 after the size line
    if (blank_or_comment(line)) continue;
    const std::vector<std::string> t = split(line);
    if (t.size() != expected) fail_at(path, line_number, "expected " + std::to_string(expected) + " fields");
    int64_t r = 0, c = 0, whole = 0;
    double v = 1.0;
    bool ok = to_int(t[0], r) && to_int(t[1], c);
    if (ok && integer) {
      ok = to_int(t[2], whole);
      v = (double)whole;
    } else if (ok && !pattern) {
      ok = to_double(t[2], v);
    }
    if (!ok) fail_at(path, line_number, "invalid matrix entry");
    --r;
    --c;
    if (r < 0 || r >= m.rows || c < 0 || c >= m.cols) fail_at(path, line_number, "matrix index is out of bounds");
    if (!std::isfinite(v)) fail_at(path, line_number, "matrix value must be finite");
    if (!fits_f32(v)) fail_at(path, line_number, "matrix value must fit in f32");
    row.push_back((int32_t)r); col.push_back((int32_t)c); val.push_back(v);
    ++read;
    if (mirrored && r != c) {
      row.push_back((int32_t)c); col.push_back((int32_t)r); val.push_back(v);
    }
  }
  if (read != declared)
    fail(path, "header declares " + std::to_string(declared) + " entries, but the file contains " + std::to_string(read));

  std::vector<size_t> order(val.size());
  std::iota(order.begin(), order.end(), (size_t)0);
  std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
    return row[a] != row[b] ? row[a] < row[b] : col[a] < col[b];
  });
  m.row.resize(val.size()); m.col.resize(val.size()); m.val.resize(val.size());
  for (size_t i = 0; i < order.size(); ++i) {
    m.row[i] = row[order[i]]; m.col[i] = col[order[i]]; m.val[i] = val[order[i]];
  }
  return m;
}

std::vector<float> to_f32(const std::vector<double> &v) {
  std::vector<float> out(v.size());
  for (size_t i = 0; i < v.size(); ++i) out[i] = (float)v[i];
  return out;
}

class Output {
 public:
  explicit Output(const char *path) : f_(fopen(path, "wb")), path_(path) {
    if (!f_) throw std::runtime_error(std::string("could not create ") + path);
  }
  ~Output() { if (f_) fclose(f_); }
  void raw(const void *p, size_t n) {
    if (n > 0 && fwrite(p, 1, n, f_) != n) throw std::runtime_error("could not write " + path_);
  }
  void u64(uint64_t v) { raw(&v, sizeof v); }
  template <typename T>
  void array(const std::vector<T> &v) { raw(v.data(), v.size() * sizeof(T)); }
  void close() {
    FILE *f = f_;
    f_ = nullptr;
    if (fclose(f) != 0) throw std::runtime_error("could not write " + path_);
  }

 private:
  FILE *f_;
  std::string path_;
};

void write_coo(const Coo &m, const char *path) {
  if (m.rows > kI32Max || m.cols > kI32Max || (int64_t)m.val.size() > kI32Max)
    throw std::runtime_error("matrix dimensions and NNZ must fit in the i32 COO type");
  Output out(path);
  out.raw("SWCOO001", 8);
  out.u64(m.rows); out.u64(m.cols); out.u64(m.val.size());
  out.array(m.row); out.array(m.col); out.array(to_f32(m.val));
  out.close();
}

void write_csr(const Coo &m, const char *path) {
  const size_t nnz = m.val.size();
  if (m.rows > kI32Max || (int64_t)nnz > kI32Max) throw std::runtime_error("matrix rows and NNZ must fit in the i32 CSR type");
  std::vector<int32_t> row_ptr(m.rows + 1, 0);
  for (size_t e = 0; e < nnz; ++e) ++row_ptr[m.row[e] + 1];
  for (int64_t r = 0; r < m.rows; ++r) row_ptr[r + 1] += row_ptr[r];
  Output out(path);
  out.raw("SWCSR001", 8);
  out.u64(m.rows); out.u64(m.cols); out.u64(nnz);
  out.array(row_ptr); out.array(m.col); out.array(to_f32(m.val));
  out.close();
}

// Dimensions padded up to the block size; blocks ordered by (block row, block column); entries with the
// same coordinate are summed in double, in (row, column) order, into their slot and rounded once; the entries
// themselves follow the blocks (benchmark_utils.py:241-379).
void write_bsr(const Coo &m, int64_t bs, const char *path) {
  if (bs <= 0) throw std::runtime_error("BSR block size must be positive");
  const int64_t prow = (m.rows + bs - 1) / bs * bs, pcol = (m.cols + bs - 1) / bs * bs;
  const int64_t brows = prow / bs, bcols = pcol / bs, stride = bcols > 0 ? bcols : 1;
  const size_t nnz = m.val.size();
  std::vector<int64_t> key(nnz);
  for (size_t e = 0; e < nnz; ++e) key[e] = (m.row[e] / bs) * stride + m.col[e] / bs;
  std::vector<int64_t> uniq(key);
  std::sort(uniq.begin(), uniq.end());
  uniq.erase(std::unique(uniq.begin(), uniq.end()), uniq.end());
  const size_t nnzb = uniq.size();
  if (prow > kI32Max || pcol > kI32Max || (int64_t)nnzb > kI32Max || (int64_t)nnz > kI32Max)
    throw std::runtime_error("BSR dimensions and NNZ blocks must fit in i32");
  std::vector<double> acc(nnzb * bs * bs, 0.0);
  for (size_t e = 0; e < nnz; ++e) {
    const size_t slot = std::lower_bound(uniq.begin(), uniq.end(), key[e]) - uniq.begin();
    acc[(slot * bs + m.row[e] % bs) * bs + m.col[e] % bs] += m.val[e];
  }
  std::vector<int32_t> brp(brows + 1, 0), bci(nnzb);
  for (size_t b = 0; b < nnzb; ++b) {
    ++brp[uniq[b] / stride + 1];
    bci[b] = (int32_t)(uniq[b] % stride);
  }
  for (int64_t r = 0; r < brows; ++r) brp[r + 1] += brp[r];
  for (double v : acc)
    if (!fits_f32(v)) throw std::runtime_error("coalesced BSR values must fit in f32");
  Output out(path);
  out.raw("SWBSR001", 8);
  out.u64(prow); out.u64(pcol); out.u64(nnzb); out.u64(bs); out.u64(m.rows); out.u64(m.cols); out.u64(nnz);
  out.array(brp); out.array(bci); out.array(to_f32(acc));
  out.array(m.row); out.array(m.col); out.array(to_f32(m.val));
  out.close();
}

}  // namespace

extern "C" int swbu_convert_matrix_market(const char *mtx_path, const char *format, int64_t block_size,
                                          const char *out_path, char *err, size_t err_len) {
  try {
    if (!mtx_path || !format || !out_path) throw std::runtime_error("NULL argument");
    const std::string fmt = format;
    if (fmt != "csr" && fmt != "coo" && fmt != "bsr") throw std::runtime_error("format must be csr, coo or bsr");
    const Coo m = read_matrix_market(mtx_path);
    if (fmt == "csr") write_csr(m, out_path);
    else if (fmt == "coo") write_coo(m, out_path);
    else write_bsr(m, block_size, out_path);
    return 0;
  } catch (const std::exception &e) {
    if (err && err_len > 0) snprintf(err, err_len, "%s", e.what());
    return -1;
  }
}
