/*
 * swb_oracle.c - CPU restatement of the SparseWave reference arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA library is
 * compared against (tests/, the smoke test, and the CPU-baseline legs of the
 * benchmark).  Nothing in the product path links, loads or calls it.
 *
 * Parity pinned: the functions below reproduce every runtime golden vector
 * the reference's own tests hold for this path (test/Dialect/SparseWave/
 * spmv-runtime.mlir:64-71, sparse-tensor-runtime.mlir:29-35,
 * spmm-sparse-tensor-runtime.mlir:50-60, bsr-spmm-runtime.mlir:24-30,
 * test/TorchExport/csr_spmm_hip_runtime.mlir:12), the folded index answers of
 * position-space-lowering.mlir:200-222,226-243,343-356, and agree with the
 * reference's own CPU loops compiled from benchmark/SparseBenchmarkUtils.cpp
 * (oracle/build.py) on that file's fixed inputs.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (oracle/build.py).
 * -ffp-contract=off keeps every product and sum a separate f32 operation,
 * like the reference's `float sum; sum += v * b;` compiled without FMA
 * contraction and like its arith.mulf + arith.addf lowering.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

/* ---- CSR SpMM / SpMV: benchmark/SparseBenchmarkUtils.cpp:275-288 ---------
 * for row: for column: float sum = 0; for position in the row:
 *   sum += values[position] * rhs[col[position], column].
 * SpMV is the N == 1 case (same order as the thread-per-row lowering,
 * lib/Dialect/SparseWave/Transforms/SparseWaveToGPU.cpp:247-261). */
ORACLE_API void oracle_csr_spmm(int64_t rows, int64_t n, const int32_t *row_ptr,
                                const int32_t *col, const float *val,
                                const float *B, float *C) {
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t j = 0; j < n; ++j) {
      float sum = 0.0f;
      for (int32_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p)
        sum += val[p] * B[(int64_t)col[p] * n + j];
      C[r * n + j] = sum;
    }
}

ORACLE_API void oracle_csr_spmv(int64_t rows, const int32_t *row_ptr,
                                const int32_t *col, const float *val,
                                const float *x, float *y) {
  oracle_csr_spmm(rows, 1, row_ptr, col, val, x, y);
}

/* The same loops with rows spread over the host threads (the reference is
 * single-threaded; this is the "all host cores" CPU baseline).  Per-element
 * results are identical to the serial functions. */
ORACLE_API void oracle_csr_spmm_omp(int64_t rows, int64_t n, const int32_t *row_ptr,
                                    const int32_t *col, const float *val,
                                    const float *B, float *C) {
#pragma omp parallel for schedule(dynamic, 1024)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t j = 0; j < n; ++j) {
      float sum = 0.0f;
      for (int32_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p)
        sum += val[p] * B[(int64_t)col[p] * n + j];
      C[r * n + j] = sum;
    }
}

ORACLE_API void oracle_csr_spmv_omp(int64_t rows, const int32_t *row_ptr,
                                    const int32_t *col, const float *val,
                                    const float *x, float *y) {
  oracle_csr_spmm_omp(rows, 1, row_ptr, col, val, x, y);
}

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Thread count of the OpenMP loops above.  Launchers that start one process per GPU export
 * OMP_NUM_THREADS=1 to every rank; the timed CPU baseline sets the count it wants (the cores
 * the process may run on) explicitly instead of inheriting that. */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n >= 1) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* Per-output tolerance scale: sum_p |val[p] * B[col[p], j]| in f64. */
ORACLE_API void oracle_csr_abs_bound(int64_t rows, int64_t n, const int32_t *row_ptr,
                                     const int32_t *col, const float *val,
                                     const float *B, double *bound) {
#pragma omp parallel for schedule(dynamic, 1024)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t j = 0; j < n; ++j) {
      double s = 0.0;
      for (int32_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p)
        s += fabs((double)val[p] * (double)B[(int64_t)col[p] * n + j]);
      bound[r * n + j] = s;
    }
}

/* ---- BSR SpMM: SparseWaveToGPU.cpp:605-649 -------------------------------
 * per output (row, column): blocks of block row row/bs in storage order, then
 * local columns ascending: sum += bv[bp*bs*bs + (row%bs)*bs + lc] *
 * B[bc[bp]*bs + lc, column]. */
ORACLE_API void oracle_bsr_spmm_f32(int64_t rows, int64_t bs, int64_t n,
                                    const int32_t *brp, const int32_t *bci,
                                    const float *bv, const float *B, float *C) {
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t br = r / bs, lr = r % bs;
    for (int64_t j = 0; j < n; ++j) {
      float sum = 0.0f;
      for (int32_t bp = brp[br]; bp < brp[br + 1]; ++bp) {
        const float *a = bv + ((int64_t)bp * bs + lr) * bs;
        const float *b = B + ((int64_t)bci[bp] * bs) * n + j;
        for (int64_t lc = 0; lc < bs; ++lc) sum += a[lc] * b[lc * n];
      }
      C[r * n + j] = sum;
    }
  }
}

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Round to nearest even, NaN kept quiet. */
static inline uint16_t f32_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* Same order, bf16 operands widened to f32, f32 accumulation, one rounding to
 * bf16 at the store. */
ORACLE_API void oracle_bsr_spmm_bf16(int64_t rows, int64_t bs, int64_t n,
                                     const int32_t *brp, const int32_t *bci,
                                     const uint16_t *bv, const uint16_t *B,
                                     uint16_t *C, float *C_f32 /* optional */) {
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t br = r / bs, lr = r % bs;
    for (int64_t j = 0; j < n; ++j) {
      float sum = 0.0f;
      for (int32_t bp = brp[br]; bp < brp[br + 1]; ++bp) {
        const uint16_t *a = bv + ((int64_t)bp * bs + lr) * bs;
        const uint16_t *b = B + ((int64_t)bci[bp] * bs) * n + j;
        for (int64_t lc = 0; lc < bs; ++lc)
          sum += bf16_to_f32(a[lc]) * bf16_to_f32(b[lc * n]);
      }
      C[r * n + j] = f32_to_bf16(sum);
      if (C_f32) C_f32[r * n + j] = sum;
    }
  }
}

/* Size of what a bf16 BSR output is summed from: sum over the row's terms of
 * |a * b| in f64.  The bf16 tolerance of the tests is stated against it (an
 * output much smaller than this sum comes from cancellation). */
ORACLE_API void oracle_bsr_abs_bound_bf16(int64_t rows, int64_t bs, int64_t n,
                                          const int32_t *brp, const int32_t *bci,
                                          const uint16_t *bv, const uint16_t *B,
                                          double *bound) {
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t r = 0; r < rows; ++r) {
    const int64_t br = r / bs, lr = r % bs;
    for (int64_t j = 0; j < n; ++j) {
      double sum = 0.0;
      for (int32_t bp = brp[br]; bp < brp[br + 1]; ++bp) {
        const uint16_t *a = bv + ((int64_t)bp * bs + lr) * bs;
        const uint16_t *b = B + ((int64_t)bci[bp] * bs) * n + j;
        for (int64_t lc = 0; lc < bs; ++lc)
          sum += fabs((double)bf16_to_f32(a[lc]) * (double)bf16_to_f32(b[lc * n]));
      }
      bound[r * n + j] = sum;
    }
  }
}

/* ---- index arithmetic ----------------------------------------------------- */

/* sparsewave.position_space: SparsePositionToSCF.cpp:190-223. */
ORACLE_API void oracle_partition(int64_t lower, int64_t upper, int64_t worker,
                                 int64_t count, int64_t *begin, int64_t *end) {
  uint64_t span = (uint64_t)(upper - lower);
  uint64_t base = span / (uint64_t)count, rem = span % (uint64_t)count;
  int receives = (uint64_t)worker < rem;
  uint64_t before = receives ? (uint64_t)worker : rem;
  *begin = lower + (int64_t)((uint64_t)worker * base + before);
  *end = *begin + (int64_t)(base + (receives ? 1 : 0));
}

/* sparsewave.position_for: SparsePositionToSCF.cpp:38-98. */
ORACLE_API void oracle_chunk_bounds(int64_t lower, int64_t upper, int64_t worker,
                                    int64_t factor, int64_t *begin, int64_t *end) {
  uint64_t span = (uint64_t)(upper - lower), f = (uint64_t)factor;
  uint64_t count = span / f + (span % f != 0 ? 1 : 0);
  int active = (uint64_t)worker < count;
  uint64_t safe = active ? (uint64_t)worker : 0;
  *begin = lower + (int64_t)(safe * f);
  uint64_t remaining = (uint64_t)(upper - *begin);
  uint64_t bounded = remaining < f ? remaining : f;
  *end = *begin + (int64_t)(active ? bounded : 0);
}

/* sparsewave.csr_row_at_position: SparsePositionToSCF.cpp:225-271. */
ORACLE_API int64_t oracle_row_at_position(const int32_t *row_ptr, int64_t len,
                                          int64_t position) {
  uint64_t lo = 1, hi = (uint64_t)len;
  while (lo < hi) {
    uint64_t mid = lo + (hi - lo) / 2;
    if ((uint64_t)(int64_t)row_ptr[mid] <= (uint64_t)position)
      lo = mid + 1;
    else
      hi = mid;
  }
  return (int64_t)lo - 1;
}

/* ---- position schedules, executed sequentially -----------------------------
 * Each function zero-fills y (SparsePositionScheduling.cpp:31-47), walks the
 * workers in increasing order and applies their atomic adds in program order.
 * Optional traces (nnz entries each, may be NULL): the row recovered for each
 * position, the worker that processed it and whether an add was issued for a
 * segment ending there. */

/* ThreadPositionReducePattern, :135-194 (search per position, add per position). */
ORACLE_API void oracle_spmv_thread_position_atomic(
    int64_t rows, int64_t nnz, int64_t chunk, const int32_t *row_ptr,
    const int32_t *col, const float *val, const float *x, float *y,
    int32_t *t_row, int32_t *t_worker, int32_t *t_end) {
  for (int64_t r = 0; r < rows; ++r) y[r] = 0.0f;
  int64_t workers = nnz / chunk + (nnz % chunk != 0);
  for (int64_t w = 0; w < workers; ++w) {
    int64_t b, e;
    oracle_chunk_bounds(0, nnz, w, chunk, &b, &e);
    for (int64_t p = b; p < e; ++p) {
      int64_t row = oracle_row_at_position(row_ptr, rows + 1, p);
      y[row] += val[p] * x[col[p]];
      if (t_row) { t_row[p] = (int32_t)row; t_worker[p] = (int32_t)w; t_end[p] = 1; }
    }
  }
}

/* ThreadSegmentedPositionReducePattern, :196-316. */
ORACLE_API void oracle_spmv_thread_position_segmented(
    int64_t rows, int64_t nnz, int64_t chunk, const int32_t *row_ptr,
    const int32_t *col, const float *val, const float *x, float *y,
    int32_t *t_row, int32_t *t_worker, int32_t *t_end) {
  for (int64_t r = 0; r < rows; ++r) y[r] = 0.0f;
  if (t_end) memset(t_end, 0, (size_t)nnz * sizeof(int32_t));
  int64_t workers = nnz / chunk + (nnz % chunk != 0);
  for (int64_t w = 0; w < workers; ++w) {
    int64_t begin = w * chunk;
    int64_t remaining = nnz - begin;
    int64_t end = begin + (remaining < chunk ? remaining : chunk);
    int64_t key = oracle_row_at_position(row_ptr, rows + 1, begin);
    float value = val[begin] * x[col[begin]];
    int64_t boundary = row_ptr[key + 1];
    if (t_row) { t_row[begin] = (int32_t)key; t_worker[begin] = (int32_t)w; }
    for (int64_t p = begin + 1; p < end; ++p) {
      int64_t row = key;
      while (boundary <= p) { ++row; boundary = row_ptr[row + 1]; }
      float contribution = val[p] * x[col[p]];
      if (t_row) { t_row[p] = (int32_t)row; t_worker[p] = (int32_t)w; }
      if (row == key) {
        value = value + contribution;
      } else {
        y[key] += value;
        if (t_end) t_end[p - 1] = 1;
        value = contribution;
        key = row;
      }
    }
    y[key] += value;
    if (t_end) t_end[end - 1] = 1;
  }
}

/* WavePositionReducePattern, :318-403, with buildWavePrefixSegmentedReduction
 * (SparseGPUUtils.cpp:247-292) emulated lane by lane: wave count W =
 * max(ceil(nnz/B),1) * (B/32); wave w owns partition(0,nnz,w,W); inactive
 * lanes carry key 0 and value 0; five shuffle-up steps add the value `offset`
 * lanes below when that lane exists and has the same key; a lane is a segment
 * end when it is active and the next lane is absent, inactive or has another
 * key; segment ends add their inclusive value to y[key].
 * `batch` > 1 models this library's option of letting one warp walk `batch`
 * consecutive partitions: segment ends are then evaluated on the span (the
 * union of the partitions) instead of on each partition; values are summed
 * sequentially in that case. */
ORACLE_API void oracle_spmv_wave_position(
    int64_t rows, int64_t nnz, int64_t block, int64_t batch, const int32_t *row_ptr,
    const int32_t *col, const float *val, const float *x, float *y,
    int32_t *t_row, int32_t *t_worker, int32_t *t_end) {
  for (int64_t r = 0; r < rows; ++r) y[r] = 0.0f;
  if (t_end) memset(t_end, 0, (size_t)nnz * sizeof(int32_t));
  int64_t grid = nnz / block + (nnz % block != 0);
  if (grid < 1) grid = 1;
  int64_t waves = grid * (block / 32);
  if (batch <= 1) {
    for (int64_t w = 0; w < waves; ++w) {
      int64_t b, e;
      oracle_partition(0, nnz, w, waves, &b, &e);
      int64_t key[32];
      float v[32];
      int active[32];
      for (int l = 0; l < 32; ++l) {
        int64_t p = b + l;
        active[l] = p < e;
        key[l] = 0;
        v[l] = 0.0f;
        if (active[l]) {
          key[l] = oracle_row_at_position(row_ptr, rows + 1, p);
          v[l] = val[p] * x[col[p]];
          if (t_row) { t_row[p] = (int32_t)key[l]; t_worker[p] = (int32_t)w; }
        }
      }
      for (int off = 1; off < 32; off <<= 1) {
        float nv[32];
        for (int l = 0; l < 32; ++l) {
          nv[l] = v[l];
          if (l >= off && active[l] && key[l - off] == key[l]) nv[l] = v[l] + v[l - off];
        }
        memcpy(v, nv, sizeof v);
      }
      for (int l = 0; l < 32; ++l) {
        int next_same = (l + 1 < 32) && active[l + 1] && key[l + 1] == key[l];
        if (active[l] && !next_same) {
          y[key[l]] += v[l];
          if (t_end) t_end[b + l] = 1;
        }
      }
    }
    return;
  }
  for (int64_t w0 = 0; w0 < waves; w0 += batch) {
    int64_t w1 = w0 + batch < waves ? w0 + batch : waves;
    int64_t b, e, unused;
    oracle_partition(0, nnz, w0, waves, &b, &unused);
    oracle_partition(0, nnz, w1 - 1, waves, &unused, &e);
    int64_t key = -1;
    float value = 0.0f;
    for (int64_t w = w0; w < w1; ++w) {
      int64_t wb, we;
      oracle_partition(0, nnz, w, waves, &wb, &we);
      for (int64_t p = wb; p < we; ++p) {
        int64_t row = oracle_row_at_position(row_ptr, rows + 1, p);
        if (t_row) { t_row[p] = (int32_t)row; t_worker[p] = (int32_t)w; }
        float contribution = val[p] * x[col[p]];
        if (row == key) {
          value += contribution;
        } else {
          if (key >= 0) { y[key] += value; if (t_end) t_end[p - 1] = 1; }
          key = row;
          value = contribution;
        }
      }
    }
    if (key >= 0) { y[key] += value; if (t_end) t_end[e - 1] = 1; }
    (void)b;
  }
}

/* DecomposePositionSpMMPattern (PositionSpMMDecomposition.cpp:19-73) under the
 * thread/atomic schedule: iteration i in [0, nnz*N): position = i / N, column
 * = i % N, key = row*N + column. */
ORACLE_API void oracle_spmm_thread_position(
    int64_t rows, int64_t nnz, int64_t n, int64_t chunk, const int32_t *row_ptr,
    const int32_t *col, const float *val, const float *B, float *C) {
  for (int64_t i = 0; i < rows * n; ++i) C[i] = 0.0f;
  int64_t total = nnz * n;
  int64_t workers = total / chunk + (total % chunk != 0);
  for (int64_t w = 0; w < workers; ++w) {
    int64_t b, e;
    oracle_chunk_bounds(0, total, w, chunk, &b, &e);
    for (int64_t i = b; i < e; ++i) {
      int64_t p = i / n, j = i % n;
      int64_t row = oracle_row_at_position(row_ptr, rows + 1, p);
      C[row * n + j] += val[p] * B[(int64_t)col[p] * n + j];
    }
  }
}

/* COO SpMV: benchmark/SparseBenchmarkUtils.cpp:243-256 (expected output of
 * loadCOOSpMVBenchmarkInputs) and ThreadPerNonzeroCOOSpMVPattern
 * (SparseWaveToGPU.cpp:154-214): zero fill, then entries in storage order. */
ORACLE_API void oracle_coo_spmv(int64_t rows, int64_t nnz, const int32_t *row, const int32_t *col,
                                const float *val, const float *x, float *y) {
  for (int64_t r = 0; r < rows; ++r) y[r] = 0.0f;
  for (int64_t p = 0; p < nnz; ++p) y[row[p]] += val[p] * x[col[p]];
}

/* ---- mismatch counters ------------------------------------------------------ */

/* The reference's own criterion (benchmark/SparseRocSparseBenchmark.cpp:
 * 193-203, benchmark/spmv.mlir.in:25,86-91): |actual - expected| >
 * 1e-4 * max(1, |expected|) counts as a mismatch. */
ORACLE_API int64_t oracle_count_mismatches_reference(const float *actual, const float *expected,
                                                     int64_t n) {
  int64_t bad = 0;
  for (int64_t i = 0; i < n; ++i) {
    float scale = fabsf(expected[i]) > 1.0f ? fabsf(expected[i]) : 1.0f;
    if (!(fabsf(actual[i] - expected[i]) <= 1e-4f * scale)) ++bad;
  }
  return bad;
}

/* |actual - expected| <= rel * bound[i] (bound = sum |a*x|), else a mismatch. */
ORACLE_API int64_t oracle_count_mismatches_bound(const float *actual, const float *expected,
                                                 const double *bound, double rel, int64_t n) {
  int64_t bad = 0;
  for (int64_t i = 0; i < n; ++i)
    if (!(fabs((double)actual[i] - (double)expected[i]) <= rel * bound[i])) ++bad;
  return bad;
}
