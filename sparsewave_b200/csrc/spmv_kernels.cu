// CSR SpMV kernels for sm_100a: the three row mappings and the two position
// mappings of sparsewave.spmv.  A reference "wave" (Wave32) is a CUDA warp.
//
// Arithmetic: products and sums are separate IEEE f32 operations
// (__fmul_rn / __fadd_rn, never contracted to FMA), like the reference's
// arith.mulf + arith.addf (SparseWaveToGPU.cpp:252-256).  thread-per-row adds
// in position order, so it reproduces the CPU CSR loop bit for bit; the
// cooperative mappings add the same products in a tree order.
#include <atomic>

#include "swb_index.h"
#include "swb_kernels.h"

namespace swb {
namespace {

constexpr unsigned FULL = 0xffffffffu;

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }

// L2 eviction priorities per instruction: the col/val streams of the vectorised kernels are marked
// evict-first and the gathered vector evict-last, so that a stream far larger than L2 does not push the
// vector's lines out (measured on a 92 M-nonzero SpMV: 1.39x the algorithmic DRAM bytes without the
// hints, 1.01x with them).  No device-wide setting is involved.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// Streaming loads for data read once (col/val).
__device__ __forceinline__ int ld_stream(const int32_t *p) { return __ldcs(p); }
__device__ __forceinline__ float ld_stream(const float *p) { return __ldcs(p); }
__device__ __forceinline__ int4 ld_stream(const int4 *p) {
  int4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.s32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(l2_policy_evict_first()));
  return v;
}
__device__ __forceinline__ float4 ld_stream(const float4 *p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p), "l"(l2_policy_evict_first()));
  return v;
}

// Gather of one x element: read-only path, no L1 allocation (the 13 % L1 hit rate of a random gather
// does not pay for the fills), kept in L2.
__device__ __forceinline__ float ld_x(const float *p) {
  float v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.f32 %0, [%1], %2;"
               : "=f"(v) : "l"(p), "l"(l2_policy_evict_last()));
  return v;
}
__device__ __forceinline__ float4 ld_x4(const float4 *p) {
  float4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p), "l"(l2_policy_evict_last()));
  return v;
}

// XOR butterfly, offsets 1,2,4,8,16: every lane ends with the warp sum
// (buildWaveReduction, SparseGPUUtils.cpp:236-245).
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) v = add(v, __shfl_xor_sync(FULL, v, off));
  return v;
}

// ---------------------------------------------------------------------------
// zero fill (buildOutputInitialization, SparsePositionScheduling.cpp:31-47)
// ---------------------------------------------------------------------------
__global__ void fill_zero_kernel(float *__restrict__ y, int64_t n) {
  // A kernel launched behind this one with programmatic stream serialisation may start its prologue now
  // (it waits with griddepcontrol.wait before it touches y).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) y[i] = 0.0f;
}

// ---------------------------------------------------------------------------
// thread-per-row (ThreadPerRowSpMVPattern, SparseWaveToGPU.cpp:216-274)
// row = blockIdx * blockDim + threadIdx; sequential sum from 0.0f in position
// order; plain store.
// ---------------------------------------------------------------------------
__global__ void spmv_thread_per_row_kernel(int64_t rows,
                                           const int32_t *__restrict__ row_ptr,
                                           const int32_t *__restrict__ col,
                                           const float *__restrict__ val,
                                           const float *__restrict__ x,
                                           float *__restrict__ y) {
  int64_t row = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  int p = row_ptr[row];
  const int end = row_ptr[row + 1];
  float sum = 0.0f;
  // Four independent (col, val, x) loads in flight, summed in position order.
  for (; p + 4 <= end; p += 4) {
    int c0 = ld_stream(col + p), c1 = ld_stream(col + p + 1);
    int c2 = ld_stream(col + p + 2), c3 = ld_stream(col + p + 3);
    float v0 = ld_stream(val + p), v1 = ld_stream(val + p + 1);
    float v2 = ld_stream(val + p + 2), v3 = ld_stream(val + p + 3);
    float x0 = __ldg(x + c0), x1 = __ldg(x + c1), x2 = __ldg(x + c2), x3 = __ldg(x + c3);
    sum = add(sum, mul(v0, x0));
    sum = add(sum, mul(v1, x1));
    sum = add(sum, mul(v2, x2));
    sum = add(sum, mul(v3, x3));
  }
  for (; p < end; ++p) sum = add(sum, mul(ld_stream(val + p), __ldg(x + ld_stream(col + p))));
  y[row] = sum;
}

// Partial sum of positions [start, end) taken by participant `who` of `count`
// participants with stride `count`.  Rows of at least VEC_MIN positions use
// 128-bit loads of the col/val streams: a scalar head up to the next 16-byte
// boundary, int4/float4 groups strided over the participants, a scalar tail.
constexpr int VEC_MIN = 128;

__device__ __forceinline__ float strided_row_partial(int start, int end, int who, int count,
                                                     const int32_t *__restrict__ col,
                                                     const float *__restrict__ val,
                                                     const float *__restrict__ x,
                                                     bool vec_ok) {
  float sum = 0.0f;
  if (vec_ok && end - start >= VEC_MIN) {
    const int a0 = (start + 3) & ~3;  // first 16-byte aligned position
    int p = start + who;
    if (p < a0) sum = add(sum, mul(ld_stream(val + p), __ldg(x + ld_stream(col + p))));
    const int g1 = end >> 2;
    const int4 *col4 = reinterpret_cast<const int4 *>(col);
    const float4 *val4 = reinterpret_cast<const float4 *>(val);
    int g = (a0 >> 2) + who;
    for (; g + count < g1; g += 2 * count) {
      int4 ca = ld_stream(col4 + g), cb = ld_stream(col4 + g + count);
      float4 va = ld_stream(val4 + g), vb = ld_stream(val4 + g + count);
      float xa0 = __ldg(x + ca.x), xa1 = __ldg(x + ca.y), xa2 = __ldg(x + ca.z), xa3 = __ldg(x + ca.w);
      float xb0 = __ldg(x + cb.x), xb1 = __ldg(x + cb.y), xb2 = __ldg(x + cb.z), xb3 = __ldg(x + cb.w);
      sum = add(sum, mul(va.x, xa0)); sum = add(sum, mul(va.y, xa1));
      sum = add(sum, mul(va.z, xa2)); sum = add(sum, mul(va.w, xa3));
      sum = add(sum, mul(vb.x, xb0)); sum = add(sum, mul(vb.y, xb1));
      sum = add(sum, mul(vb.z, xb2)); sum = add(sum, mul(vb.w, xb3));
    }
    for (; g < g1; g += count) {
      int4 ca = ld_stream(col4 + g);
      float4 va = ld_stream(val4 + g);
      float xa0 = __ldg(x + ca.x), xa1 = __ldg(x + ca.y), xa2 = __ldg(x + ca.z), xa3 = __ldg(x + ca.w);
      sum = add(sum, mul(va.x, xa0)); sum = add(sum, mul(va.y, xa1));
      sum = add(sum, mul(va.z, xa2)); sum = add(sum, mul(va.w, xa3));
    }
    p = (g1 << 2) + who;
    if (p < end) sum = add(sum, mul(ld_stream(val + p), __ldg(x + ld_stream(col + p))));
    return sum;
  }
  // Reference traversal: p = start + who, step count
  // (buildStridedPositionRange, SparseGPUUtils.cpp:70-78), two loads in flight.
  int p = start + who;
  for (; p + count < end; p += 2 * count) {
    int c0 = ld_stream(col + p), c1 = ld_stream(col + p + count);
    float v0 = ld_stream(val + p), v1 = ld_stream(val + p + count);
    float x0 = __ldg(x + c0), x1 = __ldg(x + c1);
    sum = add(sum, mul(v0, x0));
    sum = add(sum, mul(v1, x1));
  }
  if (p < end) sum = add(sum, mul(ld_stream(val + p), __ldg(x + ld_stream(col + p))));
  return sum;
}

// ---------------------------------------------------------------------------
// wave-per-row (WavePerRowSpMVPattern, SparseWaveToGPU.cpp:276-354)
// row = blockIdx * (blockDim/32) + threadIdx/32; lane-strided positions;
// butterfly; lane 0 stores.
// ---------------------------------------------------------------------------
__global__ void spmv_wave_per_row_kernel(int64_t rows, const int32_t *__restrict__ row_ptr,
                                         const int32_t *__restrict__ col,
                                         const float *__restrict__ val,
                                         const float *__restrict__ x, float *__restrict__ y,
                                         bool vec_ok) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int start = row_ptr[row], end = row_ptr[row + 1];
  float sum = strided_row_partial(start, end, lane, 32, col, val, x, vec_ok);
  sum = warp_sum(sum);
  if (lane == 0) y[row] = sum;
}

// ---------------------------------------------------------------------------
// block-per-row (BlockPerRowSpMVPattern, SparseWaveToGPU.cpp:356-487)
// row = blockIdx; thread-strided positions; warp butterfly -> shared
// wave_sums[blockDim/32] -> barrier -> warp 0 butterfly over the partials ->
// lane 0 stores.
// ---------------------------------------------------------------------------
__global__ void spmv_block_per_row_kernel(int64_t rows, const int32_t *__restrict__ row_ptr,
                                          const int32_t *__restrict__ col,
                                          const float *__restrict__ val,
                                          const float *__restrict__ x, float *__restrict__ y,
                                          bool vec_ok) {
  __shared__ float wave_sums[32];
  const int64_t row = blockIdx.x;
  if (row >= rows) return;  // uniform for the block
  const int lane = threadIdx.x & 31, wave = threadIdx.x >> 5;
  const int waves = blockDim.x >> 5;
  const int start = row_ptr[row], end = row_ptr[row + 1];
  float sum = strided_row_partial(start, end, threadIdx.x, blockDim.x, col, val, x, vec_ok);
  sum = warp_sum(sum);
  if (lane == 0) wave_sums[wave] = sum;
  __syncthreads();
  if (wave == 0) {
    float v = lane < waves ? wave_sums[lane] : 0.0f;
    v = warp_sum(v);
    if (lane == 0) y[row] = v;
  }
}

// ---------------------------------------------------------------------------
// thread-per-position (ThreadPositionReducePattern and
// ThreadSegmentedPositionReducePattern, SparsePositionScheduling.cpp:135-316)
// worker = blockIdx * blockDim + threadIdx owns positions
// [worker*chunk, min(nnz, (worker+1)*chunk)).  The row of the first position
// comes from the upper-bound search; later rows by advancing over row
// boundaries (buildNextCSRRowState, :108-133), which yields the same row the
// per-position search would.  atomic: one atomicAdd per position.  segmented:
// one atomicAdd per row change plus one at the chunk end.
// ---------------------------------------------------------------------------
__device__ __forceinline__ int warp_row_search(const int32_t *__restrict__ row_ptr, int len, int pos, int lane);

// Row of the first position of every worker of a block, found by the block
// together instead of one 22-step binary search per thread: warp 0 searches
// the row of the block's first position (32-ary, five dependent loads for 4 M
// rows); the block then streams the row offsets that follow with coalesced
// loads, each offset b inside the block's position range [cb, ce) marks the
// first worker that starts at or after b (atomicMax keeps the last of several
// rows that start at one position, i.e. skips empty rows), and a block-wide
// prefix maximum gives every worker the last row that starts at or before its
// first position - the value of the reference's upper-bound search
// (SparsePositionToSCF.cpp:225-271).  Needs blockDim.x to be a multiple of 32.
__device__ __forceinline__ int block_first_rows(const int32_t *__restrict__ row_ptr, int64_t rows, int64_t cb,
                                                int64_t ce, int64_t chunk, int *marks, int *warp_tot) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  __shared__ int first_row;
  if (warp == 0) {
    const int r = warp_row_search(row_ptr, (int)rows + 1, (int)cb, lane);
    if (lane == 0) first_row = r;
  }
  marks[tid] = -1;
  __syncthreads();
  const int R0 = first_row;
  if (tid == 0) marks[0] = R0;
  __syncthreads();
  for (int64_t r0 = (int64_t)R0 + 1;; r0 += blockDim.x) {
    const int64_t r = r0 + tid;
    int64_t b = INT64_MAX;
    if (r <= rows) b = __ldg(row_ptr + r);
    const bool inside = b < ce;
    if (inside) {
      const int64_t w = (b - cb + chunk - 1) / chunk;  // first worker whose chunk starts at or after b
      if (w < blockDim.x) atomicMax(&marks[w], (int)r);
    }
    if (!__syncthreads_and(inside)) break;
  }
  // inclusive prefix maximum over the block
  int v = marks[tid];
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const int t = __shfl_up_sync(FULL, v, off);
    if (lane >= off) v = max(v, t);
  }
  if (lane == 31) warp_tot[warp] = v;
  __syncthreads();
  if (warp == 0) {
    int t = lane < nwarps ? warp_tot[lane] : -1;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int u = __shfl_up_sync(FULL, t, off);
      if (lane >= off) t = max(t, u);
    }
    warp_tot[lane] = t;  // inclusive over warps
  }
  __syncthreads();
  if (warp > 0) v = max(v, warp_tot[warp - 1]);
  return v;
}

// y[key] += value for every lane with key >= 0, all 32 lanes calling.  Each run of adjacent lanes with the
// same key is added up with a segmented shuffle scan and its last lane issues the one atomicAdd of the
// run (keys in any order are handled; sorted keys give the longest runs).
__device__ __forceinline__ void warp_add_runs(float *__restrict__ y, int key, float value, int lane) {
  const int below = __shfl_up_sync(FULL, key, 1);
  const bool head = lane == 0 || below != key;
  const unsigned hmask = __ballot_sync(FULL, head);
  const unsigned le = (lane == 31) ? FULL : ((1u << (lane + 1)) - 1u);
  const int dist = lane - (31 - __clz(hmask & le));
  float S = value;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float t = __shfl_up_sync(FULL, S, off);
    if (off <= dist) S = add(S, t);
  }
  const bool last = lane == 31 || ((hmask >> (lane + 1)) & 1u);
  if (key >= 0 && last) atomicAdd(y + key, S);
}

template <bool SEGMENTED, bool TRACE, bool COOP>
__global__ void spmv_thread_per_position_kernel(int64_t rows, int64_t nnz, int64_t chunk,
                                                const int32_t *__restrict__ row_ptr,
                                                const int32_t *__restrict__ col,
                                                const float *__restrict__ val,
                                                const float *__restrict__ x,
                                                float *__restrict__ y, PositionTrace trace) {
  const int64_t worker = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t begin, end;
  chunk_bounds(0, nnz, worker, chunk, begin, end);
  int64_t row;
  if (COOP) {
    __shared__ int marks[1024];
    __shared__ int warp_tot[32];
    // positions of this block: workers blockIdx*B .. +B, clipped to nnz (uniform for the block)
    const int64_t w0 = (int64_t)blockIdx.x * blockDim.x;
    int64_t cb, ce, unused;
    chunk_bounds(0, nnz, w0, chunk, cb, unused);
    const int64_t last = w0 + blockDim.x - 1;
    chunk_bounds(0, nnz, last, chunk, unused, ce);
    if (ce <= cb) ce = nnz;  // the last worker of the block is past the end: the block reaches nnz
    if (w0 * chunk >= nnz) return;  // whole block inactive (only the clamped grid of an empty matrix)
    row = block_first_rows(row_ptr, rows, cb, ce, chunk, marks, warp_tot);
    if constexpr (!SEGMENTED) {
      // Atomic schedule on whole warps: at step j the lanes hold positions `chunk` apart, so their rows
      // are non-decreasing and equal rows sit in adjacent lanes.  The products of such a run are added
      // by warp_add_runs and the run's last lane issues one atomicAdd for all of them: the same additions
      // into y as one atomicAdd per position, far fewer of them on the same address.
      const int lane = threadIdx.x & 31;
      int64_t nxt = begin < end ? row_ptr[row + 1] : 0;
      for (int64_t j = 0; j < chunk; ++j) {
        const int64_t p = begin + j;
        const bool valid = p < end;
        if (__ballot_sync(FULL, valid) == 0) break;
        float prod = 0.0f;
        if (valid) {
          while (nxt <= p) {
            ++row;
            nxt = row_ptr[row + 1];
          }
          prod = mul(ld_stream(val + p), __ldg(x + ld_stream(col + p)));
          if (TRACE) {
            trace.row_of_position[p] = (int32_t)row;
            trace.worker_of_position[p] = (int32_t)worker;
            trace.segment_end[p] = 1;
          }
        }
        warp_add_runs(y, valid ? (int)row : -1, prod, lane);
      }
      return;
    }
  } else {
    if (begin >= end) return;
    row = row_at_position(row_ptr, rows + 1, begin);
  }
  // From here: the segmented schedule, and the atomic one on blocks that are not made of whole warps.
  // With whole warps the threads past the last position stay for the warp-wide flush at the end.
  const bool live = begin < end;
  int64_t next = live ? row_ptr[row + 1] : 0;
  float acc = 0.0f;
  int64_t acc_row = row;
  for (int64_t p = begin; p < end; ++p) {
    while (next <= p) {
      ++row;
      next = row_ptr[row + 1];
    }
    float prod = mul(ld_stream(val + p), __ldg(x + ld_stream(col + p)));
    if (TRACE) {
      trace.row_of_position[p] = (int32_t)row;
      trace.worker_of_position[p] = (int32_t)worker;
    }
    if (SEGMENTED) {
      if (row != acc_row) {
        atomicAdd(y + acc_row, acc);
        if (TRACE) trace.segment_end[p - 1] = 1;
        acc = prod;
        acc_row = row;
      } else {
        acc = (p == begin) ? prod : add(acc, prod);
      }
    } else {
      atomicAdd(y + row, prod);
      if (TRACE) trace.segment_end[p] = 1;
    }
  }
  if (SEGMENTED) {
    // Last open segment of every worker.  On whole warps the workers' last rows are non-decreasing over
    // the lanes, so workers that end inside the same long row share one atomicAdd.
    if (COOP) warp_add_runs(y, live ? (int)acc_row : -1, acc, threadIdx.x & 31);
    else atomicAdd(y + acc_row, acc);
    if (TRACE && live) trace.segment_end[end - 1] = 1;
  }
}

// ---------------------------------------------------------------------------
// COO SpMV, thread-per-nonzero (ThreadPerNonzeroCOOSpMVPattern,
// SparseWaveToGPU.cpp:154-214): zero fill, then position = blockIdx * blockDim
// + threadIdx adds val * x[col] to y[row] with one atomicAdd; duplicate
// coordinates simply add twice.
// ---------------------------------------------------------------------------
template <bool WHOLE_WARPS>
__global__ void coo_spmv_thread_per_nonzero_kernel(int64_t nnz, const int32_t *__restrict__ row,
                                                   const int32_t *__restrict__ col,
                                                   const float *__restrict__ val,
                                                   const float *__restrict__ x, float *__restrict__ y) {
  const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (WHOLE_WARPS) {
    // Entries of one row that sit in adjacent lanes (row-sorted files) share one atomicAdd.
    if (p - (threadIdx.x & 31) >= nnz) return;  // whole warp past the end
    const bool valid = p < nnz;
    const int r = valid ? ld_stream(row + p) : -1;
    const float prod = valid ? mul(ld_stream(val + p), __ldg(x + ld_stream(col + p))) : 0.0f;
    warp_add_runs(y, r, prod, threadIdx.x & 31);
    return;
  }
  if (p >= nnz) return;
  atomicAdd(y + ld_stream(row + p), mul(ld_stream(val + p), __ldg(x + ld_stream(col + p))));
}

// ---------------------------------------------------------------------------
// wave-per-position (WavePositionReducePattern, SparsePositionScheduling.cpp:
// 318-403; segmented scan buildWavePrefixSegmentedReduction,
// SparseGPUUtils.cpp:247-292).
//
// Reference schedule: W = max(ceil(nnz/B),1) * (B/32) waves; wave w owns
// partition(0, nnz, w, W), at most 32 positions, lane = position - begin; a
// segmented inclusive scan keyed on the row sums each row segment and the
// segment-end lane issues one atomicAdd.
//
// Here one warp walks `batch` consecutive wave partitions (a contiguous span
// of positions).  Rows are recovered once per tile of TILE_WAVES partitions:
// one warp-cooperative 32-ary upper-bound search at the span start, then the
// row offsets that follow are streamed with coalesced loads and each offset
// that falls inside the tile marks its position in shared memory; a prefix
// maximum turns the marks into the row of every position (the last row that
// starts at or before it, so empty rows are skipped like the reference's
// search does).  Inside a partition the reduction is the reference's:
// segment heads from the row keys, a 5-step shuffle-up inclusive scan, one
// atomicAdd per segment end.  The last, still open segment of a partition is
// carried in registers into the next partition of the same warp and flushed
// when its row ends or the span ends; with batch == 1 this is exactly one
// atomicAdd per (partition, row) segment, the reference's count.
// ---------------------------------------------------------------------------
constexpr int TILE_WAVES = 8;
constexpr int TILE_POS = TILE_WAVES * 32;

// Smallest idx in [1, len) with row_ptr[idx] > pos, minus one; all lanes of the
// warp take part and get the result.
__device__ __forceinline__ int warp_row_search(const int32_t *__restrict__ row_ptr, int len,
                                               int pos, int lane) {
  int lo = 1, hi = len;
  while (lo < hi) {
    const int n = hi - lo;
    const int step = (n + 31) >> 5;
    const int64_t idx = (int64_t)lo + (int64_t)(lane + 1) * step - 1;
    bool gt = true;
    if (idx < hi) gt = __ldg(row_ptr + idx) > pos;
    const unsigned m = __ballot_sync(FULL, gt);
    if (m == 0) {
      lo = hi;
      break;
    }
    const int f = __ffs(m) - 1;
    const int64_t nlo = (int64_t)lo + (int64_t)f * step;
    int64_t nhi = nlo + step - 1;
    if (nhi > hi) nhi = hi;
    lo = (int)nlo;
    hi = (int)nhi;
  }
  return lo - 1;
}

template <bool TRACE, int MAX_BLOCK>
__global__ void __launch_bounds__(MAX_BLOCK) spmv_wave_per_position_kernel(int64_t rows, int64_t nnz, int64_t wave_count,
                                              int64_t batch, const int32_t *__restrict__ row_ptr,
                                              const int32_t *__restrict__ col,
                                              const float *__restrict__ val,
                                              const float *__restrict__ x, float *__restrict__ y,
                                              PositionTrace trace) {
  extern __shared__ int smem_rows[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int wpb = blockDim.x >> 5;
  int *rowof = smem_rows + warp * TILE_POS;

  const int64_t span_id = (int64_t)blockIdx.x * wpb + warp;
  const int64_t w0 = span_id * batch;
  if (w0 >= wave_count) return;
  const int64_t w1 = (w0 + batch < wave_count) ? w0 + batch : wave_count;
  const int64_t base = nnz / wave_count, rem = nnz % wave_count;
  auto wave_begin = [&](int64_t w) { return w * base + (w < rem ? w : rem); };
  const int64_t span_begin = wave_begin(w0), span_end = wave_begin(w1);
  if (span_begin >= span_end) return;

  // Row of the first position of the span.
  int R = warp_row_search(row_ptr, (int)rows + 1, (int)span_begin, lane);

  int carry_row = -1;   // row of the open segment, -1 if none
  float acc = 0.0f;     // per-lane partial of the open segment
  int64_t carry_last = span_begin - 1;  // last position folded into the carry

  for (int64_t wt = w0; wt < w1; wt += TILE_WAVES) {
    const int64_t wte = (wt + TILE_WAVES < w1) ? wt + TILE_WAVES : w1;
    const int tile_begin = (int)wave_begin(wt), tile_end = (int)wave_begin(wte);
    const int n = tile_end - tile_begin;
    if (n <= 0) continue;

    // 1. Issue the col/val loads of every partition of the tile.
    int c[TILE_WAVES];
    float v[TILE_WAVES];
    int pos[TILE_WAVES];
    bool act[TILE_WAVES];
#pragma unroll
    for (int j = 0; j < TILE_WAVES; ++j) {
      const int64_t w = wt + j;
      int b = tile_end, e = tile_end;
      if (w < wte) {
        b = (int)wave_begin(w);
        e = (int)wave_begin(w + 1);
      }
      pos[j] = b + lane;
      act[j] = pos[j] < e;
      c[j] = 0;
      v[j] = 0.0f;
      if (act[j]) {
        c[j] = ld_stream(col + pos[j]);
        v[j] = ld_stream(val + pos[j]);
      }
    }

    // 2. Row of every position of the tile.
    __syncwarp();  // the previous tile's reads are done
#pragma unroll
    for (int i = 0; i < TILE_POS / 32; ++i) rowof[i * 32 + lane] = (i == 0 && lane == 0) ? R : -1;
    __syncwarp();
    bool any_boundary = false;
    for (int64_t r0 = (int64_t)R + 1;; r0 += 32) {
      const int64_t r = r0 + lane;
      int b = 0x7fffffff;
      if (r <= rows) b = __ldg(row_ptr + r);
      const bool inside = b < tile_end;
      if (inside) atomicMax(&rowof[b - tile_begin], (int)r);
      const unsigned m = __ballot_sync(FULL, inside);
      any_boundary |= (m != 0);
      if (m != FULL) break;
    }
    __syncwarp();
    if (any_boundary) {
      // Inclusive prefix maximum over the tile, TILE_POS/32 entries per lane.
      constexpr int PER = TILE_POS / 32;
      int loc[PER];
      int run = -1;
#pragma unroll
      for (int i = 0; i < PER; ++i) {
        run = max(run, rowof[lane * PER + i]);
        loc[i] = run;
      }
      int incl = run;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        int t = __shfl_up_sync(FULL, incl, off);
        if (lane >= off) incl = max(incl, t);
      }
      int excl = __shfl_up_sync(FULL, incl, 1);
      if (lane == 0) excl = -1;
      __syncwarp();
#pragma unroll
      for (int i = 0; i < PER; ++i) rowof[lane * PER + i] = max(loc[i], excl);
      __syncwarp();
      R = rowof[n - 1];
    }

    // 3. Gathers of x.
    float prod[TILE_WAVES];
#pragma unroll
    for (int j = 0; j < TILE_WAVES; ++j) {
      float xv = act[j] ? __ldg(x + c[j]) : 0.0f;
      prod[j] = mul(v[j], xv);
    }

    // 4. Reduce partition by partition.
#pragma unroll
    for (int j = 0; j < TILE_WAVES; ++j) {
      const unsigned amask = __ballot_sync(FULL, act[j]);
      if (amask == 0) continue;  // uniform
      const int idx = pos[j] - tile_begin;
      const int row = act[j] ? (any_boundary ? rowof[idx] : R) : -2;
      if (TRACE && act[j]) {
        trace.row_of_position[pos[j]] = row;
        trace.worker_of_position[pos[j]] = (int32_t)(wt + j);
      }
      const int nact = __popc(amask);  // active lanes form a prefix
      const bool same = __all_sync(FULL, !act[j] || row == carry_row);
      if (same) {
        acc = add(acc, prod[j]);
        carry_last = pos[0 + j] - lane + nact - 1;
        continue;
      }
      // Close or merge the carried segment.
      float val_j = prod[j];
      const int first_row = __shfl_sync(FULL, row, 0);
      if (carry_row >= 0) {
        const float total = warp_sum(acc);
        if (first_row == carry_row) {
          if (lane == 0) val_j = add(total, val_j);
        } else if (lane == 0) {
          atomicAdd(y + carry_row, total);
          if (TRACE) trace.segment_end[carry_last] = 1;
        }
      }
      // Segment heads: lane 0, a row change, or an inactive lane.
      const int prev_row = __shfl_up_sync(FULL, row, 1);
      const bool head = (lane == 0) || (row != prev_row) || !act[j];
      const unsigned hmask = __ballot_sync(FULL, head);
      const unsigned le = (lane == 31) ? FULL : ((1u << (lane + 1)) - 1u);
      const int dist = lane - (31 - __clz(hmask & le));
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const float t = __shfl_up_sync(FULL, val_j, off);
        if (off <= dist) val_j = add(val_j, t);
      }
      const bool next_head = (lane == 31) || ((hmask >> (lane + 1)) & 1u);
      const bool last_active = (lane == nact - 1);
      if (act[j] && next_head && !last_active) {
        atomicAdd(y + row, val_j);
        if (TRACE) trace.segment_end[pos[j]] = 1;
      }
      // The segment of the last active lane stays open.
      carry_row = __shfl_sync(FULL, row, nact - 1);
      acc = last_active ? val_j : 0.0f;
      carry_last = pos[j] - lane + nact - 1;
    }
  }
  if (carry_row >= 0) {
    const float total = warp_sum(acc);
    if (lane == 0) {
      atomicAdd(y + carry_row, total);
      if (TRACE) trace.segment_end[carry_last] = 1;
    }
  }
}

#include "spmv_wave_span.cuh"
#include "spmv_band.cuh"

// ---------------------------------------------------------------------------
// Roofline probe: the col/val streams and the gather of x with no row logic at all (every warp adds its
// products into one of 1024 sinks).  What this kernel takes on a matrix's own arrays is the floor of any
// SpMV mapping that reads x[col[p]] through the cache hierarchy: on a vector much larger than L1 the
// rate of 32-byte sector requests, not HBM, sets it.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) stream_gather_probe_kernel(const int4 *__restrict__ col4,
                                                                  const float4 *__restrict__ val4,
                                                                  const float *__restrict__ x, int64_t n4,
                                                                  float *__restrict__ sink) {
  float s = 0.0f;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const int4 c = ld_stream(col4 + i);
    const float4 v = ld_stream(val4 + i);
    const float x0 = ld_x(x + c.x), x1 = ld_x(x + c.y), x2 = ld_x(x + c.z), x3 = ld_x(x + c.w);
    s = add(s, add(add(mul(v.x, x0), mul(v.y, x1)), add(mul(v.z, x2), mul(v.w, x3))));
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) atomicAdd(sink + (blockIdx.x & 1023), s);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline unsigned grid_of(int64_t blocks) { return (unsigned)max1(blocks); }

}  // namespace

cudaError_t launch_stream_gather_probe(int64_t nnz, const int32_t *col, const float *val, const float *x, float *sink,
                                       const DeviceInfo &dev, cudaStream_t s, int64_t *launches) {
  if (!aligned16(col) || !aligned16(val)) return cudaErrorMisalignedAddress;
  stream_gather_probe_kernel<<<(unsigned)(dev.sm_count * 16), 256, 0, s>>>(
      reinterpret_cast<const int4 *>(col), reinterpret_cast<const float4 *>(val), x, nnz / 4, sink);
  ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_fill_zero(float *y, int64_t n, int block, cudaStream_t s, int64_t *launches) {
  // Thread mapping over len(y) (SparsePositionScheduling.cpp:31-47); the grid
  // is capped and threads stride, which stores the same zeros.
  int64_t blocks = max1(ceil_div(n, block));
  if (blocks > 148 * 32) blocks = 148 * 32;
  fill_zero_kernel<<<(unsigned)blocks, block, 0, s>>>(y, n);
  ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_coo_spmv_thread_per_nonzero(int64_t rows, int64_t nnz, const int32_t *row, const int32_t *col,
                                               const float *val, const float *x, float *y, int block,
                                               cudaStream_t s, int64_t *launches) {
  cudaError_t e = launch_fill_zero(y, rows, block, s, launches);
  if (e != cudaSuccess) return e;
  if (block % 32 == 0)
    coo_spmv_thread_per_nonzero_kernel<true><<<grid_of(ceil_div(nnz, block)), block, 0, s>>>(nnz, row, col, val, x, y);
  else
    coo_spmv_thread_per_nonzero_kernel<false><<<grid_of(ceil_div(nnz, block)), block, 0, s>>>(nnz, row, col, val, x, y);
  ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_spmv_thread_per_row(const CsrSpmvArgs &a, int block, cudaStream_t s,
                                       int64_t *launches) {
  spmv_thread_per_row_kernel<<<grid_of(ceil_div(a.rows, block)), block, 0, s>>>(
      a.rows, a.row_ptr, a.col_idx, a.val, a.x, a.y);
  ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_spmv_wave_per_row(const CsrSpmvArgs &a, int block, cudaStream_t s,
                                     int64_t *launches) {
  const bool vec_ok = aligned16(a.col_idx) && aligned16(a.val);
  spmv_wave_per_row_kernel<<<grid_of(ceil_div(a.rows, block / 32)), block, 0, s>>>(
      a.rows, a.row_ptr, a.col_idx, a.val, a.x, a.y, vec_ok);
  ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_spmv_block_per_row(const CsrSpmvArgs &a, int block, cudaStream_t s,
                                      int64_t *launches) {
  const bool vec_ok = aligned16(a.col_idx) && aligned16(a.val);
  spmv_block_per_row_kernel<<<grid_of(a.rows), block, 0, s>>>(a.rows, a.row_ptr, a.col_idx,
                                                               a.val, a.x, a.y, vec_ok);
  ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_spmv_thread_per_position(const CsrSpmvArgs &a, int block, int64_t chunk,
                                            bool segmented, const PositionTrace &trace,
                                            cudaStream_t s, int64_t *launches) {
  if (!a.accumulate) {
    cudaError_t e = launch_fill_zero(a.y, a.rows, block, s, launches);
    if (e != cudaSuccess) return e;
  }
  const int64_t workers = ceil_div(a.nnz, chunk);
  const unsigned grid = grid_of(ceil_div(workers, block));
  // Blocks made of whole warps recover rows cooperatively; other block sizes search per thread.
  const bool coop = block % 32 == 0;
#define SWB_TPP(SEG, TR)                                                                         \
  do {                                                                                           \
    if (coop)                                                                                    \
      spmv_thread_per_position_kernel<SEG, TR, true><<<grid, block, 0, s>>>(                      \
          a.rows, a.nnz, chunk, a.row_ptr, a.col_idx, a.val, a.x, a.y, trace);                    \
    else                                                                                         \
      spmv_thread_per_position_kernel<SEG, TR, false><<<grid, block, 0, s>>>(                     \
          a.rows, a.nnz, chunk, a.row_ptr, a.col_idx, a.val, a.x, a.y, trace);                    \
  } while (0)
  if (trace.enabled()) {
    if (segmented) SWB_TPP(true, true); else SWB_TPP(false, true);
  } else {
    if (segmented) SWB_TPP(true, false); else SWB_TPP(false, false);
  }
#undef SWB_TPP
  ++*launches;
  return cudaGetLastError();
}

int64_t wave_per_position_auto_batch(int64_t nnz, int block, const DeviceInfo &dev) {
  // Spans long enough that the one row search per span is amortised, short enough that the warps fill the
  // SMs many times over.  Measured on a power-law SpMV: 92 M nonzeros want 32 to 48 partitions per span
  // (0.397 ms; 0.400 at 64, 0.413 at 16), a quarter of it 12 to 16 (0.110 ms; 0.115 at 9), an eighth 8 (0.059 ms;
  // 0.065 at 4, 0.062 at 16).  Small problems keep at least 16 warps per SM.
  const int64_t waves = wave_position_wave_count(nnz, block);
  int64_t batch = waves / ((int64_t)dev.sm_count * 64 * 6);
  if (batch > 48) batch = 48;
  if (batch < 8) {
    const int64_t by_occupancy = waves / ((int64_t)dev.sm_count * 16);
    batch = by_occupancy < 8 ? by_occupancy : 8;
  }
  if (batch < 1) batch = 1;
  return batch;
}

int64_t wave_per_position_physical_grid(int64_t nnz, int block, int64_t batch) {
  const int64_t waves = wave_position_wave_count(nnz, block);
  const int64_t spans = ceil_div(waves, batch);
  return max1(ceil_div(spans, block / 32));
}

// Shape of the long-row path for a matrix, or false when the span kernel alone is used: small problems
// (the three extra launches would cost more than they save), more bands than a grid dimension holds, or
// operands without the 16-byte alignment of the 128-bit loads.
bool band_path_plan(const CsrSpmvArgs &a, int64_t min_nnz, BandPlan *plan) {
  if (a.nnz < min_nnz || a.nnz < 1 || a.cols < 1) return false;
  const int64_t bands = ceil_div(a.cols, BAND_COLS);
  if (bands > 4096) return false;
  if (!aligned16(a.col_idx) || !aligned16(a.val) || !aligned16(a.x)) return false;
  plan->bands = (int)bands;
  plan->long_min = (int)(32 * bands < 256 ? 256 : 32 * bands);
  plan->cap = (int)(a.nnz / plan->long_min) + 1;
  return true;
}

size_t band_scratch_bytes(const BandPlan &plan) {
  // counter (padded), list of long rows, their sampling strides, (bands + 1) x cap table of run brackets
  return 256 + 2 * (size_t)plan.cap * 4 + (size_t)(plan.bands + 1) * (size_t)plan.cap * 4;
}

cudaError_t launch_spmv_wave_per_position(const CsrSpmvArgs &a, int block, int64_t batch,
                                          const PositionTrace &trace, cudaStream_t s,
                                          int64_t *launches, int64_t *physical_grid,
                                          const BandPlan *band, void *band_scratch, const DeviceInfo &dev) {
  const int64_t waves = wave_position_wave_count(a.nnz, block);
  const int64_t grid = wave_per_position_physical_grid(a.nnz, block, batch);
  if (physical_grid) *physical_grid = grid;
  // Spans of two or more partitions take the chunked span kernel (needs
  // 16-byte aligned col/val); batch == 1 is the reference schedule, one
  // partition per warp and lane == position.  Blocks above 512 threads need
  // the register-capped instantiation.
  // col and val views that start the same number of elements past a 16-byte boundary take the span kernel
  // too (it reads from that boundary); other misalignments take the scalar kernel.
  const uintptr_t col_off = reinterpret_cast<uintptr_t>(a.col_idx) & 15u, val_off = reinterpret_cast<uintptr_t>(a.val) & 15u;
  const bool span = batch >= 2 && col_off == val_off && col_off % 4 == 0 && a.nnz > 0;
  const int shift = span ? (int)(col_off / 4) : 0;
  const bool banded = span && shift == 0 && band && band_scratch && !trace.enabled();
  int long_min = 0;
  int *count = nullptr, *long_rows = nullptr, *strides = nullptr, *tab = nullptr;
  if (banded) {
    // zero fill fused with the search for long rows, then the band boundaries of those rows
    static std::atomic<bool> configured[64];
    int device = 0;
    cudaGetDevice(&device);
    if (device < 0 || device >= 64 || !configured[device].load(std::memory_order_acquire)) {
      cudaError_t e = cudaFuncSetAttribute(spmv_band_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)BAND_SMEM);
      if (e != cudaSuccess) return e;
      if (device >= 0 && device < 64) configured[device].store(true, std::memory_order_release);
    }
    long_min = band->long_min;
    count = static_cast<int *>(band_scratch);
    long_rows = count + 64;
    strides = long_rows + band->cap;
    tab = strides + band->cap;
    cudaError_t e = cudaMemsetAsync(count, 0, sizeof(int), s);
    if (e != cudaSuccess) return e;
    int64_t blocks = max1(ceil_div(a.rows, 256));
    if (blocks > 148 * 32) blocks = 148 * 32;
    find_long_rows_kernel<<<(unsigned)blocks, 256, 0, s>>>(a.y, a.rows, !a.accumulate, a.row_ptr, long_min, band->cap,
                                                          count, long_rows);
    ++*launches;
    band_bounds_kernel<<<(unsigned)(band->cap < 148 * 16 ? band->cap : 148 * 16), BOUNDS_THREADS, 0, s>>>(
        a.row_ptr, a.col_idx, band->bands, band->cap, count, long_rows, tab, strides);
    ++*launches;
    e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  } else if (!a.accumulate) {
    cudaError_t e = launch_fill_zero(a.y, a.rows, block, s, launches);
    if (e != cudaSuccess) return e;
  }
  const size_t smem = (size_t)(block / 32) * TILE_POS * sizeof(int);
  const size_t span_smem = (size_t)(block / 32) * SPAN_CHUNK * sizeof(int);
  // Directly behind this call's own zero fill (or the library's exchange kernel, which fills y too) the
  // span kernel is launched with programmatic stream serialisation: its row search and first loads
  // overlap the end of that kernel, and it waits (griddepcontrol.wait) before it reads x or adds to y.
  cudaLaunchAttribute pdl[1];
  pdl[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  pdl[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3((unsigned)block);
  cfg.dynamicSmemBytes = span_smem;
  cfg.stream = s;
  cfg.attrs = pdl;
  cfg.numAttrs = (!banded && (!a.accumulate || a.behind_exchange)) ? 1 : 0;
#define SWB_WPP(TR, MB)                                                                   \
  do {                                                                                    \
    if (span)                                                                             \
      cudaLaunchKernelEx(&cfg, spmv_wave_span_kernel<TR, MB>, a.rows, a.nnz, waves, batch, a.row_ptr, a.col_idx, \
                         a.val, a.x, a.y, trace, long_min, shift);                         \
    else                                                                                  \
      spmv_wave_per_position_kernel<TR, MB><<<(unsigned)grid, block, smem, s>>>(           \
          a.rows, a.nnz, waves, batch, a.row_ptr, a.col_idx, a.val, a.x, a.y, trace);      \
  } while (0)
  if (trace.enabled()) {
    if (block > 512) SWB_WPP(true, 1024); else SWB_WPP(true, 512);
  } else {
    if (block > 512) SWB_WPP(false, 1024); else SWB_WPP(false, 512);
  }
#undef SWB_WPP
  ++*launches;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess || !banded) return e;
  spmv_band_kernel<<<(unsigned)dev.sm_count, BAND_THREADS, BAND_SMEM, s>>>(
      a.nnz, a.cols, a.col_idx, a.val, a.x, a.y, band->bands, band->cap, count, long_rows, tab, strides);
  ++*launches;
  return cudaGetLastError();
}

}  // namespace swb
