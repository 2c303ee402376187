// Index arithmetic shared by host code and kernels.  Every function states the
// reference construct whose values it reproduces bit for bit.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define SWB_HD __host__ __device__ __forceinline__
#else
#define SWB_HD inline
#endif

namespace swb {

SWB_HD int64_t ceil_div(int64_t a, int64_t b) { return a / b + (a % b != 0); }
SWB_HD int64_t max1(int64_t v) { return v > 1 ? v : 1; }

// Largest x dimension of a CUDA grid.  `blocks` (at least one block is always launched) as a grid
// dimension, or false when it does not fit.
constexpr int64_t kMaxGridX = 2147483647LL;
inline bool grid_dim(int64_t blocks, unsigned *out) {
  const int64_t b = max1(blocks);
  if (b > kMaxGridX) return false;
  *out = (unsigned)b;
  return true;
}

// Balanced contiguous partition of [lower, upper) over `count` workers:
// base = span / count, rem = span % count; worker w starts at
// lower + w*base + min(w, rem) and takes base + (w < rem) positions
// (sparsewave.position_space, SparsePositionToSCF.cpp:190-223).
SWB_HD void partition(int64_t lower, int64_t upper, int64_t worker,
                      int64_t count, int64_t &begin, int64_t &end) {
  int64_t span = upper - lower;
  int64_t base = span / count;
  int64_t rem = span % count;
  bool extra = worker < rem;
  begin = lower + worker * base + (extra ? worker : rem);
  end = begin + base + (extra ? 1 : 0);
}

// Chunk of `factor` consecutive positions owned by `worker`; workers at or
// beyond ceil(span / factor) get the empty range [lower, lower)
// (sparsewave.position_for, SparsePositionToSCF.cpp:38-98).
SWB_HD void chunk_bounds(int64_t lower, int64_t upper, int64_t worker,
                         int64_t factor, int64_t &begin, int64_t &end) {
  int64_t span = upper - lower;
  int64_t chunks = span / factor + (span % factor != 0);
  bool active = worker >= 0 && worker < chunks;
  int64_t safe = active ? worker : 0;
  begin = lower + safe * factor;
  int64_t remaining = upper - begin;
  int64_t size = active ? (remaining < factor ? remaining : factor) : 0;
  end = begin + size;
}

// Row owning `position`: the predecessor of the first row offset greater than
// the position, searched over [1, len) so that empty rows are skipped
// (sparsewave.csr_row_at_position, SparsePositionToSCF.cpp:225-271).
SWB_HD int64_t row_at_position(const int32_t *row_ptr, int64_t len,
                               int64_t position) {
  int64_t lo = 1, hi = len;
  while (lo < hi) {
    int64_t mid = lo + (hi - lo) / 2;
    if ((int64_t)row_ptr[mid] <= position)
      lo = mid + 1;
    else
      hi = mid;
  }
  return lo - 1;
}

// Wave-per-position schedule (SparsePositionScheduling.cpp:340-362): the
// launch has G = max(ceil(nnz / B), 1) blocks, hence W = G * (B / 32) waves,
// and wave w owns partition(0, nnz, w, W), at most 32 positions.
SWB_HD int64_t wave_position_wave_count(int64_t nnz, int64_t block_size) {
  return max1(ceil_div(nnz, block_size)) * (block_size / 32);
}

}  // namespace swb
