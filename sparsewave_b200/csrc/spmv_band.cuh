// wave-per-position on large matrices: long rows through shared-memory bands of x
// (included by spmv_kernels.cu inside namespace swb::{anonymous}).
//
// The position mapping's cost on a large matrix is the gather of x: one 32-byte L2 sector per nonzero.
// Rows of the CSR format keep their columns sorted, so the part of a long row that falls into a band of
// BAND_COLS consecutive columns is one contiguous run of positions, and the band of x itself (128 KiB)
// fits in shared memory.  Rows of at least `long_min` positions (32 per band on average) are therefore
// taken out of the span kernel and handled band by band:
//   1. find_long_rows_kernel   zero fill of y fused with the list of long rows (row_ptr is read once),
//   2. band_bounds_kernel      for every (long row, band) the first position whose column lies in the band
//                              (binary search in the row's sorted columns),
//   3. spmv_band_kernel        one CTA per SM walks items = (band, group of long rows): the band of x is
//                              staged in shared memory once per band, a warp takes the run of one row in
//                              16-byte aligned chunks of 128 positions (one int4 + one float4 per lane, two
//                              chunks in flight), x read from shared memory, one atomicAdd per run.
// The span kernel skips the positions of those rows (spmv_wave_span.cuh, `long_min`).  The positions of a
// long row are still divided among warps and combined with atomicAdd, as the mapping prescribes
// (SparsePositionScheduling.cpp:318-403); only the division follows the bands instead of equal position
// counts.  An explicit wave-position-batch, a position trace or small operands keep the span kernel alone.
#pragma once

constexpr int BAND_COLS = 32768;          // floats of x per band
constexpr int BAND_THREADS = 1024;
constexpr int BAND_ITEM_ROWS = 1024;      // long rows per work item: one per thread
constexpr size_t BAND_SMEM = (size_t)BAND_COLS * 4 + 5 * (size_t)BAND_ITEM_ROWS * 4;
constexpr int BOUNDS_THREADS = 256;
constexpr int BOUNDS_SAMPLES = 1024;      // shared-memory samples of a row's columns, one every `stride` positions

// y = 0 (unless accumulating) and the list of rows with at least long_min positions, in any order.
__global__ void find_long_rows_kernel(float *__restrict__ y, int64_t rows, bool zero,
                                      const int32_t *__restrict__ row_ptr, int long_min, int cap,
                                      int *__restrict__ count, int *__restrict__ long_rows) {
  const int lane = threadIdx.x & 31;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t r0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x - lane; r0 < rows; r0 += stride) {
    const int64_t r = r0 + lane;
    bool is_long = false;
    if (r < rows) {
      if (zero) y[r] = 0.0f;
      is_long = __ldg(row_ptr + r + 1) - __ldg(row_ptr + r) >= long_min;
    }
    const unsigned m = __ballot_sync(FULL, is_long);
    if (m == 0) continue;
    int base = 0;
    if (lane == 0) base = atomicAdd(count, __popc(m));
    base = __shfl_sync(FULL, base, 0);
    const int slot = base + __popc(m & ((1u << lane) - 1u));
    if (is_long && slot < cap) long_rows[slot] = (int)r;
  }
}

// tab[b * cap + i] = a position of long row i at or before the first one whose column is >= b * BAND_COLS
// (b = 0 .. bands), at most one sampling stride before it; tab[bands * cap + i] = the row's end.  The band
// kernel reads the run [tab[b], tab[b + 1] + stride) and keeps the positions whose column lies in band b, so
// the brackets need not be exact and no search touches the row a second time.
// One CTA per long row: every `stride`-th column of the row is sampled into shared memory with independent
// loads (one memory latency) and each band boundary is bracketed by a binary search over the samples.
__global__ void __launch_bounds__(BOUNDS_THREADS) band_bounds_kernel(const int32_t *__restrict__ row_ptr,
                                                                     const int32_t *__restrict__ col, int bands, int cap,
                                                                     const int *__restrict__ count,
                                                                     const int *__restrict__ long_rows,
                                                                     int *__restrict__ tab, int *__restrict__ strides) {
  __shared__ int sample[BOUNDS_SAMPLES];
  const int n = min(*count, cap);
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const int r = long_rows[i];
    const int s = __ldg(row_ptr + r), e = __ldg(row_ptr + r + 1);
    const int len = e - s;
    const int stride = (len + BOUNDS_SAMPLES - 1) / BOUNDS_SAMPLES;  // >= 1
    const int ns = (len + stride - 1) / stride;                       // samples at s, s + stride, ...
    __syncthreads();  // the previous row's searches are done with the samples
    for (int k = threadIdx.x; k < ns; k += BOUNDS_THREADS) sample[k] = __ldg(col + s + (int64_t)k * stride);
    if (threadIdx.x == 0) strides[i] = stride;
    __syncthreads();
    for (int b = threadIdx.x; b <= bands; b += BOUNDS_THREADS) {
      int pos = s;
      if (b == bands) {
        pos = e;
      } else if (b > 0) {
        const int target = b * BAND_COLS;
        int lo = 0, hi = ns;  // first sample >= target
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (sample[mid] < target) lo = mid + 1; else hi = mid;
        }
        pos = lo == 0 ? s : s + (lo - 1) * stride;  // the last sample below the target: everything before it is too
      }
      tab[(int64_t)b * cap + i] = pos;
    }
  }
}

// One CTA per SM walks items = (band, group of up to BAND_ITEM_ROWS long rows).  The band of x is staged in
// shared memory once per band.  A warp takes whole runs (the positions of one long row inside the band):
// 16-byte aligned chunks of 128 positions, one int4 + one float4 per lane, two chunks in flight, x read from
// shared memory, partial sums kept per lane across the chunks of the run, one warp reduction and one
// atomicAdd per run.  The tables of the next item (row, run begin, run end per long row) are loaded while
// the current item is processed.
__global__ void __launch_bounds__(BAND_THREADS, 1) spmv_band_kernel(
    int64_t nnz, int64_t cols, const int32_t *__restrict__ col, const float *__restrict__ val,
    const float *__restrict__ x, float *__restrict__ y, int bands, int cap, const int *__restrict__ count,
    const int *__restrict__ long_rows, const int *__restrict__ tab, const int *__restrict__ strides) {
  extern __shared__ __align__(16) unsigned char band_smem[];
  float *xs = reinterpret_cast<float *>(band_smem);
  int *crow = reinterpret_cast<int *>(band_smem + (size_t)BAND_COLS * 4);
  int *cbeg = crow + BAND_ITEM_ROWS, *cend = cbeg + BAND_ITEM_ROWS;  // bracket of the run
  int *rbeg = cend + BAND_ITEM_ROWS, *rend = rbeg + BAND_ITEM_ROWS;  // the whole row
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int WARPS = BAND_THREADS / 32;

  const int n_long = min(*count, cap);
  if (n_long == 0) return;
  // The runs (band, long row), band-major, are split evenly over the CTAs; a CTA walks its share in items of
  // up to BAND_ITEM_ROWS rows of one band, so that it seldom changes band.
  const int64_t total = (int64_t)bands * n_long;
  int64_t at = total * blockIdx.x / gridDim.x;
  const int64_t stop = total * (blockIdx.x + 1) / gridDim.x;
  if (at >= stop) return;

  const int4 *col4 = reinterpret_cast<const int4 *>(col);
  const float4 *val4 = reinterpret_cast<const float4 *>(val);

  auto item_rows = [&](int64_t from) -> int {  // rows of the item that starts at run `from`
    const int64_t in_band = n_long - from % n_long, left = stop - from;
    const int64_t n = in_band < left ? in_band : left;
    return (int)(n < BAND_ITEM_ROWS ? n : BAND_ITEM_ROWS);
  };
  // this thread's entry of an item's tables
  int t_row = 0, t_beg = 0, t_end = 0, t_rbeg = 0, t_rend = 0;
  auto fetch = [&](int64_t from, int n) {
    const int b = (int)(from / n_long), i = (int)(from % n_long) + tid;
    t_row = t_beg = t_end = t_rbeg = t_rend = 0;
    if (tid < n) {
      t_row = __ldg(long_rows + i);
      t_rbeg = __ldg(tab + i);
      t_rend = __ldg(tab + (int64_t)bands * cap + i);
      t_beg = __ldg(tab + (int64_t)b * cap + i);
      // the bracket of the next boundary starts up to one stride before it
      t_end = b + 1 == bands ? t_rend : min(__ldg(tab + (int64_t)(b + 1) * cap + i) + __ldg(strides + i), t_rend);
    }
  };
  int nrows = item_rows(at);
  fetch(at, nrows);
  int cur_band = -1;
  while (at < stop) {
    const int b = (int)(at / n_long);
    __syncthreads();  // everyone is done with the previous item's tables (and band)
    crow[tid] = t_row;
    cbeg[tid] = t_beg;
    cend[tid] = t_end;
    rbeg[tid] = t_rbeg;
    rend[tid] = t_rend;
    if (b != cur_band) {
      const int64_t c0 = (int64_t)b * BAND_COLS;
      const int64_t n = min((int64_t)BAND_COLS, cols - c0);
      const float4 *src = reinterpret_cast<const float4 *>(x + c0);
      for (int i = tid; i < BAND_COLS / 4; i += BAND_THREADS) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (4 * (int64_t)i + 3 < n) {
          v = ld_x4(src + i);
        } else {
          if (4 * (int64_t)i + 0 < n) v.x = __ldg(x + c0 + 4 * i + 0);
          if (4 * (int64_t)i + 1 < n) v.y = __ldg(x + c0 + 4 * i + 1);
          if (4 * (int64_t)i + 2 < n) v.z = __ldg(x + c0 + 4 * i + 2);
        }
        reinterpret_cast<float4 *>(xs)[i] = v;
      }
      cur_band = b;
    }
    __syncthreads();
    const int rows_now = nrows;
    at += rows_now;
    if (at < stop) {  // the next item's tables travel while this item is processed
      nrows = item_rows(at);
      fetch(at, nrows);
    }

    const int cbase = b * BAND_COLS;
    // The bracket reaches into the neighbouring bands, and a whole chunk is loaded even where the bracket
    // ends inside it: a position counts where its column lies in this band.  Only a chunk that sticks out
    // of the row itself (the row's first and last chunk) needs its positions checked against the row.
    auto term = [&](const int4 &c, const float4 &v) -> float {
      const unsigned k0 = (unsigned)(c.x - cbase), k1 = (unsigned)(c.y - cbase), k2 = (unsigned)(c.z - cbase),
                     k3 = (unsigned)(c.w - cbase);
      const float q0 = k0 < (unsigned)BAND_COLS ? mul(v.x, xs[k0]) : 0.0f;
      const float q1 = k1 < (unsigned)BAND_COLS ? mul(v.y, xs[k1]) : 0.0f;
      const float q2 = k2 < (unsigned)BAND_COLS ? mul(v.z, xs[k2]) : 0.0f;
      const float q3 = k3 < (unsigned)BAND_COLS ? mul(v.w, xs[k3]) : 0.0f;
      return add(add(q0, q1), add(q2, q3));
    };
    auto load_edge = [&](int p, int rs, int re, int4 &c, float4 &v) {  // a chunk that sticks out of the row
      c = make_int4(-1, -1, -1, -1);  // no band holds column -1
      v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (p + 0 >= rs && p + 0 < re) { c.x = ld_stream(col + p + 0); v.x = ld_stream(val + p + 0); }
      if (p + 1 >= rs && p + 1 < re) { c.y = ld_stream(col + p + 1); v.y = ld_stream(val + p + 1); }
      if (p + 2 >= rs && p + 2 < re) { c.z = ld_stream(col + p + 2); v.z = ld_stream(val + p + 2); }
      if (p + 3 >= rs && p + 3 < re) { c.w = ld_stream(col + p + 3); v.w = ld_stream(val + p + 3); }
    };
    for (int j = warp; j < rows_now; j += WARPS) {
      const int s = cbeg[j], e = cend[j];
      if (e <= s) continue;  // uniform
      const int rs = rbeg[j], re = rend[j];
      float acc = 0.0f;
      for (int cs = s & ~3; cs < e; cs += 256) {  // two chunks of 128 positions per step; cs is uniform
        const int p = cs + 4 * lane;
        const bool second = cs + 128 < e;
        int4 c0, c1 = make_int4(-1, -1, -1, -1);
        float4 v0, v1 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (cs >= rs && cs + 256 <= re) {  // uniform: both chunks inside the row (and the arrays)
          c0 = ld_stream(col4 + (p >> 2));
          v0 = ld_stream(val4 + (p >> 2));
          if (second) {
            c1 = ld_stream(col4 + ((p + 128) >> 2));
            v1 = ld_stream(val4 + ((p + 128) >> 2));
          }
        } else {
          load_edge(p, rs, re, c0, v0);
          if (second) load_edge(p + 128, rs, re, c1, v1);
        }
        acc = add(acc, term(c0, v0));
        if (second) acc = add(acc, term(c1, v1));
      }
      acc = warp_sum(acc);
      if (lane == 0) atomicAdd(y + crow[j], acc);
    }
  }
}
