/* libsparsewave_benchmark_utils.so: host-side input loaders for SparseWave
 * benchmark programs, a stand-in for the shared library of the same name that
 * the SparseWave tree builds from benchmark/SparseBenchmarkUtils.cpp and loads
 * into mlir-runner (benchmark/run_spmv_benchmark.py:430-435).  Host code only;
 * no CUDA.
 *
 * The four loaders are called through MLIR's C interface: every argument is a
 * pointer to a strided memref descriptor.  Each reads the binary matrix named
 * by an environment variable into the caller's buffers, fills the dense
 * operand with a fixed pattern and computes the expected output on the host
 * with the single-precision loop of the reference.  Violations print
 * "SparseWave benchmark input error: <reason>" on stderr and abort, like the
 * reference (SparseBenchmarkUtils.cpp:31-34).
 */
#ifndef SPARSEWAVE_BENCHMARK_UTILS_H
#define SPARSEWAVE_BENCHMARK_UTILS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SWBU_API __attribute__((visibility("default")))

/* MLIR strided memref descriptors (mlir/ExecutionEngine/CRunnerUtils.h). */
typedef struct { int32_t *base, *data; int64_t offset, sizes[1], strides[1]; } swbu_memref_i32;
typedef struct { float *base, *data; int64_t offset, sizes[1], strides[1]; } swbu_memref_f32;
typedef struct { float *base, *data; int64_t offset, sizes[2], strides[2]; } swbu_memref_f32_2d;

/* SPARSEWAVE_BENCHMARK_CSR names an SWCSR001 file.  vector := 1, expected :=
 * row sums of the values (replaces SparseBenchmarkUtils.cpp:211-229). */
SWBU_API void _mlir_ciface_loadCSRSpMVBenchmarkInputs(swbu_memref_i32 *row_offsets, swbu_memref_i32 *column_indices,
                                                      swbu_memref_f32 *values, swbu_memref_f32 *vector,
                                                      swbu_memref_f32 *expected);

/* SPARSEWAVE_BENCHMARK_COO names an SWCOO001 file.  vector := 1, expected[row]
 * accumulates the values in file order (replaces :231-251). */
SWBU_API void _mlir_ciface_loadCOOSpMVBenchmarkInputs(swbu_memref_i32 *row_indices, swbu_memref_i32 *column_indices,
                                                      swbu_memref_f32 *values, swbu_memref_f32 *vector,
                                                      swbu_memref_f32 *expected);

/* SPARSEWAVE_BENCHMARK_CSR again; rhs[k][j] := 1 + ((k + j) mod 7) / 8,
 * expected := A * rhs by the sequential loop (replaces :253-289). */
SWBU_API void _mlir_ciface_loadSpMMBenchmarkInputs(swbu_memref_i32 *row_offsets, swbu_memref_i32 *column_indices,
                                                   swbu_memref_f32 *values, swbu_memref_f32_2d *rhs,
                                                   swbu_memref_f32_2d *expected);

/* SPARSEWAVE_BENCHMARK_BSR names an SWBSR001 file; same rhs pattern; expected
 * is accumulated from the file's original COO entries in file order (replaces
 * :291-326). */
SWBU_API void _mlir_ciface_loadBSRSpMMBenchmarkInputs(swbu_memref_i32 *block_row_offsets,
                                                      swbu_memref_i32 *block_column_indices,
                                                      swbu_memref_f32 *block_values, swbu_memref_f32_2d *rhs,
                                                      swbu_memref_f32_2d *expected);

/* Matrix Market (coordinate; real, integer or pattern; general, symmetric or
 * skew-symmetric) -> one of the binary formats, the C++ form of
 * benchmark/benchmark_utils.py:56-379: format is "csr", "coo" or "bsr"
 * (block_size > 0 for "bsr", ignored otherwise).  CSR entries are ordered by
 * (row, column) with duplicates kept; BSR blocks are ordered by (block row,
 * block column), duplicates summed into their slot, dimensions padded to the
 * block size.  Returns 0, or -1 with a message in err (never aborts).  Not a
 * symbol of the reference library. */
SWBU_API int swbu_convert_matrix_market(const char *mtx_path, const char *format, int64_t block_size,
                                        const char *out_path, char *err, size_t err_len);

#ifdef __cplusplus
}
#endif
#endif
