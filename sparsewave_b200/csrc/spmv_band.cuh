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
//                              staged in shared memory once per band, the runs of the group's rows are cut
//                              into 16-byte aligned chunks of 128 positions, every chunk is one int4 + one
//                              float4 per lane, four chunks in flight per warp, x read from shared memory,
//                              one atomicAdd per chunk.
// The span kernel skips the positions of those rows (spmv_wave_span.cuh, `long_min`).  The positions of a
// long row are still divided among warps and combined with atomicAdd, as the mapping prescribes
// (SparsePositionScheduling.cpp:318-403); only the division follows the bands instead of equal position
// counts.  An explicit wave-position-batch, a position trace or small operands keep the span kernel alone.
#pragma once

constexpr int BAND_COLS = 32768;          // floats of x per band
constexpr int BAND_THREADS = 1024;
constexpr int BAND_ITEM_ROWS = 512;       // long rows per work item
constexpr int BAND_UNROLL = 4;            // chunks in flight per warp
constexpr int BAND_TABLE_INTS = 4 * BAND_ITEM_ROWS + 8;  // per buffer: chunk starts (+1), row, run begin, run end
constexpr size_t BAND_SMEM = (size_t)BAND_COLS * 4 + 2 * (size_t)BAND_TABLE_INTS * 4;

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

// tab[b * cap + i] = first position of long row i whose column is >= b * BAND_COLS (b = 0 .. bands).
// One CTA per long row, one thread per band: the upper levels of the row's search tree are shared by its
// bands and stay in L1, so a row costs a few hundred L2 sectors instead of 16 per (row, band) pair.
__global__ void __launch_bounds__(128) band_bounds_kernel(const int32_t *__restrict__ row_ptr,
                                                          const int32_t *__restrict__ col, int bands, int cap,
                                                          const int *__restrict__ count,
                                                          const int *__restrict__ long_rows, int *__restrict__ tab) {
  const int n = min(*count, cap);
  for (int i = blockIdx.x; i < n; i += gridDim.x) {
    const int r = long_rows[i];
    const int s = __ldg(row_ptr + r), e = __ldg(row_ptr + r + 1);
    for (int b = threadIdx.x; b <= bands; b += blockDim.x) {
      int lo = s, hi = e;
      if (b == 0) hi = lo;
      else if (b == bands) lo = hi;
      const int target = b * BAND_COLS;
      while (lo < hi) {
        const int mid = lo + ((hi - lo) >> 1);
        if (__ldg(col + mid) < target) lo = mid + 1; else hi = mid;
      }
      tab[(int64_t)b * cap + i] = lo;
    }
  }
}

__global__ void __launch_bounds__(BAND_THREADS, 1) spmv_band_kernel(
    int64_t nnz, int64_t cols, const int32_t *__restrict__ col, const float *__restrict__ val,
    const float *__restrict__ x, float *__restrict__ y, int bands, int cap, const int *__restrict__ count,
    const int *__restrict__ long_rows, const int *__restrict__ tab) {
  extern __shared__ __align__(16) unsigned char band_smem[];
  float *xs = reinterpret_cast<float *>(band_smem);
  int *tables = reinterpret_cast<int *>(band_smem + (size_t)BAND_COLS * 4);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int WORKERS = BAND_THREADS / 32 - 1;  // the last warp prepares the next item's tables

  const int n_long = min(*count, cap);
  if (n_long == 0) return;
  const int groups = (n_long + BAND_ITEM_ROWS - 1) / BAND_ITEM_ROWS;
  const int64_t items = (int64_t)bands * groups;
  // contiguous share of the band-major item list, so that a CTA seldom changes band
  const int64_t it0 = items * blockIdx.x / gridDim.x, it1 = items * (blockIdx.x + 1) / gridDim.x;
  if (it0 >= it1) return;

  const int4 *col4 = reinterpret_cast<const int4 *>(col);
  const float4 *val4 = reinterpret_cast<const float4 *>(val);

  // Tables of one item: T[0 .. BAND_ITEM_ROWS] chunk starts (exclusive prefix sums, the total last), then
  // row, run begin and run end per long row of the group.
  auto prepare = [&](int64_t item, int *T) {  // executed by one warp
    const int b = (int)(item / groups), g = (int)(item % groups);
    const int i0 = g * BAND_ITEM_ROWS, nrows = min(BAND_ITEM_ROWS, n_long - i0);
    int *crow = T + BAND_ITEM_ROWS + 8, *cbeg = crow + BAND_ITEM_ROWS, *cend = cbeg + BAND_ITEM_ROWS;
    // all loads first (three per row, 16 rows per lane), then the scan
    constexpr int PER = BAND_ITEM_ROWS / 32;
    int nch[PER];
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int j = k * 32 + lane;
      int s = 0, e = 0, r = 0;
      if (j < nrows) {
        s = __ldg(tab + (int64_t)b * cap + i0 + j);
        e = __ldg(tab + (int64_t)(b + 1) * cap + i0 + j);
        r = __ldg(long_rows + i0 + j);
      }
      crow[j] = r;
      cbeg[j] = s;
      cend[j] = e;
      nch[k] = e > s ? (e - (s & ~3) + 127) >> 7 : 0;
    }
    int base = 0;
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      int incl = nch[k];
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int t = __shfl_up_sync(FULL, incl, off);
        if (lane >= off) incl += t;
      }
      T[k * 32 + lane] = base + incl - nch[k];
      base += __shfl_sync(FULL, incl, 31);
    }
    if (lane == 0) T[BAND_ITEM_ROWS] = base;  // total
  };

  int cur_band = -1;
  if (warp == WORKERS) prepare(it0, tables);
  for (int64_t item = it0; item < it1; ++item) {
    const int buf = (int)((item - it0) & 1);
    int *T = tables + buf * BAND_TABLE_INTS;
    const int b = (int)(item / groups);
    if (b != cur_band) {
      __syncthreads();  // everyone is done with the previous band
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
    __syncthreads();  // tables of `item` and the band are in shared memory

    if (warp == WORKERS) {
      if (item + 1 < it1) prepare(item + 1, tables + (buf ^ 1) * BAND_TABLE_INTS);
    } else {
      const int g = (int)(item % groups);
      const int nrows = min(BAND_ITEM_ROWS, n_long - g * BAND_ITEM_ROWS);
      const int *crow = T + BAND_ITEM_ROWS + 8, *cbeg = crow + BAND_ITEM_ROWS, *cend = cbeg + BAND_ITEM_ROWS;
      const int total = T[BAND_ITEM_ROWS];
      const int cbase = b * BAND_COLS;
      for (int c0 = warp * BAND_UNROLL; c0 < total; c0 += WORKERS * BAND_UNROLL) {
        int4 cc[BAND_UNROLL];
        float4 vv[BAND_UNROLL];
        int jj[BAND_UNROLL], p0[BAND_UNROLL];
#pragma unroll
        for (int u = 0; u < BAND_UNROLL; ++u) {
          const int c = c0 + u;
          jj[u] = -1;
          p0[u] = 0;
          cc[u] = make_int4(cbase, cbase, cbase, cbase);
          vv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (c < total) {  // uniform
            // last row j with T[j] <= c: two 32-ary steps over the chunk starts
            const int coarse = T[16 * (lane + 1)];
            const int k = __popc(__ballot_sync(FULL, coarse <= c));  // block of 16 starts; k <= 31 as T[512] > c
            const int fine = (lane < 16) ? T[16 * k + lane] : 0x7fffffff;
            const int j = min(16 * k + __popc(__ballot_sync(FULL, fine <= c)) - 1, nrows - 1);
            jj[u] = j;
            p0[u] = (cbeg[j] & ~3) + ((c - T[j]) << 7) + 4 * lane;
            if (p0[u] < cend[j]) {
              if ((int64_t)p0[u] + 3 < nnz) {
                cc[u] = ld_stream(col4 + (p0[u] >> 2));
                vv[u] = ld_stream(val4 + (p0[u] >> 2));
              } else {
                if (p0[u] + 0 < nnz) { cc[u].x = ld_stream(col + p0[u] + 0); vv[u].x = ld_stream(val + p0[u] + 0); }
                if (p0[u] + 1 < nnz) { cc[u].y = ld_stream(col + p0[u] + 1); vv[u].y = ld_stream(val + p0[u] + 1); }
                if (p0[u] + 2 < nnz) { cc[u].z = ld_stream(col + p0[u] + 2); vv[u].z = ld_stream(val + p0[u] + 2); }
              }
            }
          }
        }
#pragma unroll
        for (int u = 0; u < BAND_UNROLL; ++u) {
          if (jj[u] < 0) continue;  // uniform
          const int p = p0[u], s = cbeg[jj[u]], e = cend[jj[u]];
          // positions outside the run are dropped (their columns may lie in another band)
          const bool m0 = p + 0 >= s && p + 0 < e, m1 = p + 1 >= s && p + 1 < e;
          const bool m2 = p + 2 >= s && p + 2 < e, m3 = p + 3 >= s && p + 3 < e;
          const float q0 = m0 ? mul(vv[u].x, xs[cc[u].x - cbase]) : 0.0f;
          const float q1 = m1 ? mul(vv[u].y, xs[cc[u].y - cbase]) : 0.0f;
          const float q2 = m2 ? mul(vv[u].z, xs[cc[u].z - cbase]) : 0.0f;
          const float q3 = m3 ? mul(vv[u].w, xs[cc[u].w - cbase]) : 0.0f;
          const float total_u = warp_sum(add(add(q0, q1), add(q2, q3)));
          if (lane == 0) atomicAdd(y + crow[jj[u]], total_u);
        }
      }
    }
  }
}
