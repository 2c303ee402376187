// Matrix Market -> SWCSR001 / SWCOO001 / SWBSR001, the C++ form of the conversion the SparseWave benchmark
// drivers do in Python (benchmark/benchmark_utils.py:56-379).  Part of libsparsewave_benchmark_utils.so.
#include "../../../include/sparsewave_benchmark_utils.h"

#include <algorithm>
#include <cctype>
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

struct Coo {
  int64_t rows = 0, cols = 0;
  std::vector<int32_t> row, col;
  std::vector<float> val;
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

int64_t to_int(const std::string &t) {
  char *end = nullptr;
  const long long v = strtoll(t.c_str(), &end, 10);
  if (end == t.c_str() || *end != '\0') throw std::runtime_error("malformed integer '" + t + "' in Matrix Market file");
  return v;
}

double to_double(const std::string &t) {
  char *end = nullptr;
  const double v = strtod(t.c_str(), &end);
  if (end == t.c_str() || *end != '\0') throw std::runtime_error("malformed value '" + t + "' in Matrix Market file");
  return v;
}

// Coordinate files only; symmetric and skew-symmetric files are expanded entry by entry (the mirrored
// entry directly after its original), pattern entries get the value 1; indices become 0-based.
Coo read_matrix_market(const char *path) {
  std::ifstream f(path);
  if (!f) throw std::runtime_error(std::string("could not open ") + path);
  std::string line;
  std::getline(f, line);
  const std::vector<std::string> head = split(line);
  if (head.size() != 5 || head[0] != "%%MatrixMarket" || head[1] != "matrix")
    throw std::runtime_error("expected a Matrix Market matrix header");
  const std::string layout = lower(head[2]), field = lower(head[3]), symmetry = lower(head[4]);
  if (layout != "coordinate") throw std::runtime_error("only coordinate Matrix Market files are supported");
  if (field != "real" && field != "integer" && field != "pattern")
    throw std::runtime_error("unsupported Matrix Market field: " + field);
  if (symmetry != "general" && symmetry != "symmetric" && symmetry != "skew-symmetric")
    throw std::runtime_error("unsupported Matrix Market symmetry: " + symmetry);
  const bool pattern = field == "pattern", mirrored = symmetry != "general", skew = symmetry == "skew-symmetric";

  std::vector<std::string> size;
  while (std::getline(f, line)) {
    if (!line.empty() && line[0] == '%') continue;
    size = split(line);
    if (!size.empty()) break;
  }
  if (size.size() != 3) throw std::runtime_error("expected the Matrix Market size line");
  Coo m;
  m.rows = to_int(size[0]);
  m.cols = to_int(size[1]);
  const int64_t entries = to_int(size[2]);
  if (m.rows < 0 || m.cols < 0 || entries < 0) throw std::runtime_error("negative Matrix Market dimensions");
  m.row.reserve(entries); m.col.reserve(entries); m.val.reserve(entries);
  for (int64_t e = 0; e < entries; ++e) {
    if (!std::getline(f, line)) throw std::runtime_error("Matrix Market file ends before its last entry");
    const std::vector<std::string> t = split(line);
    if (t.size() < (pattern ? 2u : 3u)) throw std::runtime_error("malformed Matrix Market entry");
    const int64_t r = to_int(t[0]) - 1, c = to_int(t[1]) - 1;
    const float v = pattern ? 1.0f : (float)to_double(t[2]);
    if (r < 0 || r >= m.rows || c < 0 || c >= m.cols) throw std::runtime_error("Matrix Market coordinate is out of bounds");
    m.row.push_back((int32_t)r); m.col.push_back((int32_t)c); m.val.push_back(v);
    if (mirrored && r != c) {
      m.row.push_back((int32_t)c); m.col.push_back((int32_t)r); m.val.push_back(skew ? -v : v);
    }
  }
  return m;
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
  out.array(m.row); out.array(m.col); out.array(m.val);
  out.close();
}

// Entries ordered by (row, column), equal coordinates in file order, duplicates kept.
void write_csr(const Coo &m, const char *path) {
  const size_t nnz = m.val.size();
  if (m.rows > kI32Max || (int64_t)nnz > kI32Max) throw std::runtime_error("matrix rows and NNZ must fit in the i32 CSR type");
  std::vector<size_t> order(nnz);
  std::iota(order.begin(), order.end(), (size_t)0);
  std::stable_sort(order.begin(), order.end(), [&](size_t a, size_t b) {
    return m.row[a] != m.row[b] ? m.row[a] < m.row[b] : m.col[a] < m.col[b];
  });
  std::vector<int32_t> row_ptr(m.rows + 1, 0), col(nnz);
  std::vector<float> val(nnz);
  for (size_t e = 0; e < nnz; ++e) ++row_ptr[m.row[e] + 1];
  for (int64_t r = 0; r < m.rows; ++r) row_ptr[r + 1] += row_ptr[r];
  for (size_t i = 0; i < nnz; ++i) { col[i] = m.col[order[i]]; val[i] = m.val[order[i]]; }
  Output out(path);
  out.raw("SWCSR001", 8);
  out.u64(m.rows); out.u64(m.cols); out.u64(nnz);
  out.array(row_ptr); out.array(col); out.array(val);
  out.close();
}

// Dimensions padded up to the block size; blocks ordered by (block row, block column); entries with the
// same coordinate are summed (in double, file order) into their slot; the original entries follow the blocks.
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
    acc[(slot * bs + m.row[e] % bs) * bs + m.col[e] % bs] += (double)m.val[e];
  }
  std::vector<int32_t> brp(brows + 1, 0), bci(nnzb);
  for (size_t b = 0; b < nnzb; ++b) {
    ++brp[uniq[b] / stride + 1];
    bci[b] = (int32_t)(uniq[b] % stride);
  }
  for (int64_t r = 0; r < brows; ++r) brp[r + 1] += brp[r];
  std::vector<float> bv(acc.size());
  for (size_t i = 0; i < acc.size(); ++i) bv[i] = (float)acc[i];
  Output out(path);
  out.raw("SWBSR001", 8);
  out.u64(prow); out.u64(pcol); out.u64(nnzb); out.u64(bs); out.u64(m.rows); out.u64(m.cols); out.u64(nnz);
  out.array(brp); out.array(bci); out.array(bv);
  out.array(m.row); out.array(m.col); out.array(m.val);
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
