// swb_runner - native benchmark runner over libsparsewave_b200.so.
//
// The B200 counterpart of the reference's native rocSPARSE runner
// (benchmark/SparseRocSparseBenchmark.cpp) and of its MLIR benchmark host
// (benchmark/spmv.mlir.in, spmm.mlir.in): reads an SWCSR001 matrix, fills the
// dense operand the way the reference's loaders do (x = 1 for SpMV,
// SparseBenchmarkUtils.cpp:187-193; B[k][j] = 1 + ((k + j) mod 7) / 8 for
// SpMM, :270-273), runs `warmup + iterations` dispatches of the chosen mapping
// with one CUDA-event pair per dispatch, and checks the device result against
// the host loop with the reference's criterion |actual - expected| <= 1e-4 *
// max(1, |expected|) (SparseRocSparseBenchmark.cpp:193-203).  The host loop
// only validates; nothing is ever computed on the host instead of the GPU.
//
//   swb_runner --csr FILE --operation spmv|spmm [--rhs-columns N]
//              [--options "spmv-mapping=... spmv-block-size=..."]
//              [--warmup 10] [--iterations 50] [--device 0]
//
// Output: key=value lines (timings_us, min_us, median_us, p95_us,
// gnnz_per_sec, gflops, gbps), then `[mismatches]`.  Exit 0 if the result
// matches, 2 if not, 1 on errors.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <fstream>
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../../include/sparsewave_b200.h"

namespace {

struct Arguments {
  std::string csr, operation = "spmv", options;
  int64_t rhsColumns = 4;
  int warmup = 10, iterations = 50, device = 0;
};

[[noreturn]] void usage(const std::string &why) {
  throw std::runtime_error(why + " (see the header of swb_runner.cpp for the options)");
}

Arguments parseArguments(int argc, char **argv) {
  Arguments a;
  for (int i = 1; i < argc; ++i) {
    std::string key = argv[i];
    auto value = [&]() -> std::string {
      if (i + 1 >= argc) usage("missing value for " + key);
      return argv[++i];
    };
    if (key == "--csr") a.csr = value();
    else if (key == "--operation") a.operation = value();
    else if (key == "--options") a.options = value();
    else if (key == "--rhs-columns") a.rhsColumns = std::stoll(value());
    else if (key == "--warmup") a.warmup = std::stoi(value());
    else if (key == "--iterations") a.iterations = std::stoi(value());
    else if (key == "--device") a.device = std::stoi(value());
    else usage("unknown argument " + key);
  }
  if (a.csr.empty()) usage("--csr is required");
  if (a.operation != "spmv" && a.operation != "spmm") usage("--operation must be spmv or spmm");
  if (a.rhsColumns < 1) usage("--rhs-columns must be positive");
  if (a.warmup < 0 || a.iterations < 1) usage("--warmup must be >= 0 and --iterations >= 1");
  return a;
}

struct CSRMatrix {
  uint64_t rows = 0, columns = 0, nnz = 0;
  std::vector<int32_t> rowOffsets, columnIndices;
  std::vector<float> values;
};

template <typename T>
void readArray(std::ifstream &in, std::vector<T> &out, uint64_t count, const char *name) {
  out.resize(count);
  in.read(reinterpret_cast<char *>(out.data()), (std::streamsize)(count * sizeof(T)));
  if (!in) throw std::runtime_error(std::string("could not read ") + name);
}

// SWCSR001: magic, <QQQ rows/columns/nnz, i32[rows+1], i32[nnz], f32[nnz]
// (benchmark/benchmark_utils.py:180-211).
CSRMatrix readCSR(const std::string &path) {
  std::ifstream in(path, std::ios::binary);
  if (!in) throw std::runtime_error("could not open " + path);
  char magic[8];
  in.read(magic, 8);
  if (!in || std::memcmp(magic, "SWCSR001", 8) != 0) throw std::runtime_error("invalid CSR binary header");
  CSRMatrix m;
  uint64_t header[3];
  in.read(reinterpret_cast<char *>(header), sizeof header);
  if (!in) throw std::runtime_error("could not read the CSR dimensions");
  m.rows = header[0], m.columns = header[1], m.nnz = header[2];
  if (m.rows >= 2147483647ull || m.nnz > 2147483647ull || m.columns > 2147483647ull)
    throw std::runtime_error("matrix rows and NNZ must fit in the i32 CSR type");
  readArray(in, m.rowOffsets, m.rows + 1, "row offsets");
  readArray(in, m.columnIndices, m.nnz, "column indices");
  readArray(in, m.values, m.nnz, "values");
  return m;
}

void checkCuda(cudaError_t e, const char *what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

void checkSwb(swb_context *ctx, int status, const char *what) {
  if (status != SWB_OK) throw std::runtime_error(std::string(what) + ": " + swb_last_error(ctx));
}

template <typename T>
T *toDevice(const std::vector<T> &host) {
  T *p = nullptr;
  checkCuda(cudaMalloc(&p, std::max<size_t>(host.size(), 1) * sizeof(T)), "cudaMalloc");
  if (!host.empty()) checkCuda(cudaMemcpy(p, host.data(), host.size() * sizeof(T), cudaMemcpyHostToDevice), "cudaMemcpy");
  return p;
}

// Expected output for validation (row-major, position order, f32).
std::vector<float> expectedOutput(const CSRMatrix &m, const std::vector<float> &rhs, int64_t n) {
  std::vector<float> out(m.rows * n, 0.0f);
  for (uint64_t r = 0; r < m.rows; ++r)
    for (int64_t j = 0; j < n; ++j) {
      float sum = 0.0f;
      for (int32_t p = m.rowOffsets[r]; p < m.rowOffsets[r + 1]; ++p)
        sum += m.values[p] * rhs[(int64_t)m.columnIndices[p] * n + j];
      out[r * n + j] = sum;
    }
  return out;
}

int64_t countMismatches(const std::vector<float> &actual, const std::vector<float> &expected) {
  int64_t bad = 0;
  for (size_t i = 0; i < expected.size(); ++i) {
    float scale = std::max(1.0f, std::fabs(expected[i]));
    if (!(std::fabs(actual[i] - expected[i]) <= 1e-4f * scale)) ++bad;
  }
  return bad;
}

}  // namespace

int main(int argc, char **argv) {
  swb_context *ctx = nullptr;
  try {
    Arguments args = parseArguments(argc, argv);
    CSRMatrix m = readCSR(args.csr);
    const bool spmv = args.operation == "spmv";
    const int64_t n = spmv ? 1 : args.rhsColumns;

    std::vector<float> rhs(m.columns * n);
    for (uint64_t k = 0; k < m.columns; ++k)
      for (int64_t j = 0; j < n; ++j) rhs[k * n + j] = spmv ? 1.0f : 1.0f + (float)((k + j) % 7) * 0.125f;

    checkCuda(cudaSetDevice(args.device), "cudaSetDevice");
    if (swb_create(&ctx, args.device) != SWB_OK) throw std::runtime_error(swb_last_error(nullptr));
    swb_options options;
    swb_options_default(&options);
    checkSwb(ctx, swb_options_parse(ctx, &options, args.options.c_str()), "options");
    checkSwb(ctx, swb_options_validate(ctx, &options), "options");
    // every dispatch must produce the whole result: with accumulate=1 the timed dispatches would keep adding
    if (options.accumulate) throw std::runtime_error("options: accumulate=1 is not accepted by the runner");
    checkSwb(ctx, swb_check_csr_host(ctx, (int64_t)m.rows, (int64_t)m.columns, (int64_t)m.nnz, m.rowOffsets.data(),
                                     m.columnIndices.data()),
             "matrix");

    int32_t *dRowOffsets = toDevice(m.rowOffsets), *dColumnIndices = toDevice(m.columnIndices);
    float *dValues = toDevice(m.values), *dRhs = toDevice(rhs), *dOutput = nullptr;
    std::vector<float> output(m.rows * n, -1.0f);
    dOutput = toDevice(output);

    cudaStream_t stream = nullptr;
    cudaEvent_t start = nullptr, end = nullptr;
    checkCuda(cudaStreamCreate(&stream), "cudaStreamCreate");
    checkCuda(cudaEventCreate(&start), "cudaEventCreate");
    checkCuda(cudaEventCreate(&end), "cudaEventCreate");
    auto dispatch = [&]() {
      int st = spmv ? swb_spmv(ctx, &options, (int64_t)m.rows, (int64_t)m.columns, (int64_t)m.nnz, dRowOffsets,
                               dColumnIndices, dValues, dRhs, dOutput, stream)
                    : swb_spmm(ctx, &options, (int64_t)m.rows, (int64_t)m.columns, (int64_t)m.nnz, n, dRowOffsets,
                               dColumnIndices, dValues, dRhs, dOutput, stream);
      checkSwb(ctx, st, "dispatch");
    };
    std::vector<float> timings;
    for (int i = 0; i < args.warmup + args.iterations; ++i) {
      checkCuda(cudaEventRecord(start, stream), "cudaEventRecord");
      dispatch();
      checkCuda(cudaEventRecord(end, stream), "cudaEventRecord");
      checkCuda(cudaEventSynchronize(end), "cudaEventSynchronize");
      float ms = 0.0f;
      checkCuda(cudaEventElapsedTime(&ms, start, end), "cudaEventElapsedTime");
      if (i >= args.warmup) timings.push_back(ms * 1000.0f);
    }
    checkCuda(cudaMemcpy(output.data(), dOutput, output.size() * sizeof(float), cudaMemcpyDeviceToHost), "cudaMemcpy");
    const int64_t mismatches = countMismatches(output, expectedOutput(m, rhs, n));

    std::vector<float> sorted = timings;
    std::sort(sorted.begin(), sorted.end());
    const double median = sorted.size() % 2 ? sorted[sorted.size() / 2]
                                            : 0.5 * (sorted[sorted.size() / 2 - 1] + sorted[sorted.size() / 2]);
    const double p95 = sorted[std::min(sorted.size() - 1, (size_t)std::ceil(0.95 * sorted.size()) - 1)];
    const double seconds = median * 1e-6;
    const double products = (double)m.nnz * (double)n;
    const double bytes = 8.0 * m.nnz + 4.0 * (m.rows + 1) + 4.0 * m.columns * n + 4.0 * m.rows * n;
    std::cout << "backend=" << swb_version() << '\n'
              << "operation=" << args.operation << '\n'
              << "options=" << args.options << '\n'
              << "rows=" << m.rows << "\ncols=" << m.columns << "\nnnz=" << m.nnz << "\nrhs_columns=" << n << '\n'
              << "kernels_launched=" << swb_kernel_launch_count(ctx) << '\n'
              << "timings_us=";
    for (size_t i = 0; i < timings.size(); ++i) std::cout << (i ? "," : "") << timings[i];
    std::cout << "\nmin_us=" << sorted.front() << "\nmedian_us=" << median << "\np95_us=" << p95
              << "\ngnnz_per_sec=" << products / seconds / 1e9 << "\ngflops=" << 2.0 * products / seconds / 1e9
              << "\ngbps=" << bytes / seconds / 1e9 << '\n'
              << '[' << mismatches << "]\n";

    cudaEventDestroy(start);
    cudaEventDestroy(end);
    cudaStreamDestroy(stream);
    cudaFree(dRowOffsets); cudaFree(dColumnIndices); cudaFree(dValues); cudaFree(dRhs); cudaFree(dOutput);
    swb_destroy(ctx);
    return mismatches == 0 ? 0 : 2;
  } catch (const std::exception &error) {
    std::cerr << "swb_runner error: " << error.what() << '\n';
    if (ctx) swb_destroy(ctx);
    return 1;
  }
}
