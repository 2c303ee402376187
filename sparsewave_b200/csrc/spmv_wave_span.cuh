// wave-per-position, span form (included by spmv_kernels.cu inside namespace
// swb::{anonymous}).
//
// One warp owns the union of `batch` consecutive reference wave partitions:
// a contiguous span [span_begin, span_end) of positions whose two ends are
// partition boundaries of the reference schedule
// (SparsePositionScheduling.cpp:340-362).  Inside the span the per-partition
// boundaries do not influence any result (the open row segment is carried
// from one partition into the next), so the span is walked in 16-byte aligned
// chunks of 128 positions: lane l holds positions chunk + 4l .. 4l+3, loaded
// with one int4 and one float4.  Positions of the first and last chunk that
// lie outside the span are masked to value 0.
//
// Rows: one warp-cooperative upper-bound search at the span start.  A chunk
// that ends before the current row does (the common case on long rows) is
// accumulated lane-locally with no shuffle at all.  A chunk containing row
// boundaries streams the row offsets that follow with coalesced loads, marks
// each offset inside the chunk in shared memory (atomicMax, so that of several
// rows starting at one position the last, non-empty one wins) and takes a
// prefix maximum: the row of every position, equal to the reference's
// upper-bound search (SparsePositionToSCF.cpp:225-271).
//
// Reduction in a boundary chunk: runs of equal rows that begin and end inside
// one lane are added to y directly; the lane's last run takes part in a
// segmented inclusive shuffle-up scan across lanes (segment heads from the row
// keys, as buildWavePrefixSegmentedReduction does per position,
// SparseGPUUtils.cpp:247-292); a lane's first run closes with the scanned value
// of the lane below.  One atomicAdd per (row, span) segment; the segment still
// open at the end of a chunk is carried in registers.
//
// shift (0..3): col and val are views that start `shift` elements past a 16-byte boundary (the same for
// both).  The kernel then reads from the boundary before them and works in positions p + shift, which keeps
// every 128-bit load aligned; the up to three elements in front of the arrays share their 16-byte granule
// with the first element and are masked like any position outside the span.
//
// long_min > 0: rows of at least long_min (>= 256) positions belong to the band kernel
// (spmv_band.cuh) and are left out here.  A row that long is never inside one chunk, so only the row that
// enters a chunk and the row that leaves it can be long: chunks that lie wholly in such a row are jumped
// over without a load, and in a chunk with row boundaries their positions count as zero (the reduction
// then adds 0.0f to that row, which changes nothing).
#pragma once

constexpr int SPAN_CHUNK = 128;

template <bool TRACE>
struct SpanEmit {
  float *y;
  PositionTrace trace;
  int lo, hi;  // valid positions of the span: [lo, hi)
  __device__ __forceinline__ void operator()(int row, float v, int last_pos) const {
    atomicAdd(y + row, v);
    if (TRACE) {
      int p = last_pos < lo ? lo : (last_pos >= hi ? hi - 1 : last_pos);
      trace.segment_end[p] = 1;
    }
  }
};

template <bool TRACE, int MAX_BLOCK>
__global__ void __launch_bounds__(MAX_BLOCK) spmv_wave_span_kernel(
    int64_t rows, int64_t nnz, int64_t wave_count, int64_t batch, const int32_t *__restrict__ row_ptr,
    const int32_t *__restrict__ col, const float *__restrict__ val, const float *__restrict__ x,
    float *__restrict__ y, PositionTrace trace, int long_min, int shift) {
  extern __shared__ int smem_rows[];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int wpb = blockDim.x >> 5;
  int *marks = smem_rows + warp * SPAN_CHUNK;

  const int64_t span_id = (int64_t)blockIdx.x * wpb + warp;
  const int64_t w0 = span_id * batch;
  if (w0 >= wave_count) return;
  const int64_t w1 = (w0 + batch < wave_count) ? w0 + batch : wave_count;
  const int64_t base = nnz / wave_count, rem = nnz % wave_count;
  auto wave_begin = [&](int64_t w) { return w * base + (w < rem ? w : rem); };
  // from here on positions are shifted: p + shift, array element p + shift of the aligned views below
  const int sb = (int)wave_begin(w0) + shift, se = (int)wave_begin(w1) + shift;
  if (sb >= se) return;
  nnz += shift;
  col -= shift;
  val -= shift;
  if (TRACE) {
    trace.row_of_position -= shift;
    trace.worker_of_position -= shift;
    trace.segment_end -= shift;
  }
  // Reference wave that owns a (shifted) position (inverse of wave_begin), for the trace.
  auto wave_of = [&](int ps) -> int {
    const int64_t p = ps - shift, split = rem * (base + 1);
    return (int)(p < split ? p / (base + 1) : rem + (p - split) / base);
  };

  const SpanEmit<TRACE> emit{y, trace, sb, se};
  const int4 *col4 = reinterpret_cast<const int4 *>(col);
  const float4 *val4 = reinterpret_cast<const float4 *>(val);

  int R = warp_row_search(row_ptr, (int)rows + 1, sb - shift, lane);
  int next_b = __ldg(row_ptr + R + 1) + shift;  // first position of the next non-empty row (or nnz)
  // the row that enters the current chunk belongs to the band kernel
  bool head_long = long_min > 0 && next_b - shift - __ldg(row_ptr + R) >= long_min;
  if (head_long && next_b >= se) return;  // the whole span lies inside a long row
  int carry_row = -1;
  float acc = 0.0f;
  int carry_last = sb;

  // col/val of a chunk: one int4 + one float4 per lane (scalar loads only at the
  // very end of the arrays).  The next chunk's streams are requested before the
  // current chunk's x gathers so that both latencies overlap.
  auto load_chunk = [&](int cbase, int4 &c, float4 &v) {
    c = make_int4(0, 0, 0, 0);
    v = make_float4(0.f, 0.f, 0.f, 0.f);
    const int q0 = cbase + 4 * lane;
    if (cbase < se && q0 < se) {
      if ((int64_t)q0 + 3 < nnz) {
        c = ld_stream(col4 + (q0 >> 2));
        v = ld_stream(val4 + (q0 >> 2));
      } else {
        if (q0 + 0 < nnz) { c.x = ld_stream(col + q0 + 0); v.x = ld_stream(val + q0 + 0); }
        if (q0 + 1 < nnz) { c.y = ld_stream(col + q0 + 1); v.y = ld_stream(val + q0 + 1); }
        if (q0 + 2 < nnz) { c.z = ld_stream(col + q0 + 2); v.z = ld_stream(val + q0 + 2); }
      }
    }
  };
  int4 cn;
  float4 vn;
  load_chunk(sb & ~3, cn, vn);
  // Launched behind the zero fill with programmatic stream serialisation, the kernel has come this far
  // while the fill may still be running: y is touched only after it has finished.  (Without that launch
  // attribute this returns at once.)
  asm volatile("griddepcontrol.wait;" ::: "memory");

  for (int cb = sb & ~3; cb < se; cb += SPAN_CHUNK) {
    const int ce = (cb + SPAN_CHUNK < se) ? cb + SPAN_CHUNK : se;
    if (head_long && next_b >= ce) {
      // The chunk lies in a long row: go on at the chunk that holds the row's end (or stop).
      if (next_b >= se) break;
      const int skip = (next_b - cb) / SPAN_CHUNK;  // >= 1 whole chunks to leave out, this one included
      cb += (skip - 1) * SPAN_CHUNK;
      load_chunk(cb + SPAN_CHUNK, cn, vn);  // the chunk the loop goes on with
      continue;
    }
    const int p0 = cb + 4 * lane;
    const int4 c = cn;
    const float4 v = vn;
    load_chunk(cb + SPAN_CHUNK, cn, vn);
    const bool m0 = p0 + 0 >= sb && p0 + 0 < ce, m1 = p0 + 1 >= sb && p0 + 1 < ce;
    const bool m2 = p0 + 2 >= sb && p0 + 2 < ce, m3 = p0 + 3 >= sb && p0 + 3 < ce;
    const float q0 = m0 ? mul(v.x, ld_x(x + c.x)) : 0.0f;
    const float q1 = m1 ? mul(v.y, ld_x(x + c.y)) : 0.0f;
    const float q2 = m2 ? mul(v.z, ld_x(x + c.z)) : 0.0f;
    const float q3 = m3 ? mul(v.w, ld_x(x + c.w)) : 0.0f;

    if (next_b >= ce) {
      // The whole chunk lies in row R.
      if (carry_row != R) {
        if (carry_row >= 0) {
          const float total = warp_sum(acc);
          if (lane == 0) emit(carry_row, total, carry_last);
        }
        carry_row = R;
        acc = 0.0f;
      }
      acc = add(acc, add(add(q0, q1), add(q2, q3)));
      carry_last = ce - 1;
      if (TRACE) {
        if (m0) { trace.row_of_position[p0 + 0] = R; trace.worker_of_position[p0 + 0] = wave_of(p0 + 0); }
        if (m1) { trace.row_of_position[p0 + 1] = R; trace.worker_of_position[p0 + 1] = wave_of(p0 + 1); }
        if (m2) { trace.row_of_position[p0 + 2] = R; trace.worker_of_position[p0 + 2] = wave_of(p0 + 2); }
        if (m3) { trace.row_of_position[p0 + 3] = R; trace.worker_of_position[p0 + 3] = wave_of(p0 + 3); }
      }
      continue;
    }

    // ---- chunk with row boundaries: row of every position -------------------
    __syncwarp();
    *reinterpret_cast<int4 *>(marks + 4 * lane) = make_int4(lane == 0 ? R : -1, -1, -1, -1);
    __syncwarp();
    for (int64_t r0 = (int64_t)R + 1;; r0 += 32) {
      const int64_t r = r0 + lane;
      int b = 0x7fffffff;
      if (r <= rows) b = __ldg(row_ptr + r) + shift;
      const bool inside = b < ce;
      if (inside) atomicMax(&marks[b - cb], (int)r);
      if (__ballot_sync(FULL, inside) != FULL) break;
    }
    __syncwarp();
    const int4 mk = *reinterpret_cast<const int4 *>(marks + 4 * lane);
    int r0 = mk.x, r1 = max(r0, mk.y), r2 = max(r1, mk.z), r3 = max(r2, mk.w);
    int incl = r3;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int t = __shfl_up_sync(FULL, incl, off);
      if (lane >= off) incl = max(incl, t);
    }
    int excl = __shfl_up_sync(FULL, incl, 1);
    if (lane == 0) excl = -1;
    r0 = max(r0, excl); r1 = max(r1, excl); r2 = max(r2, excl); r3 = max(r3, excl);
    const int R_last = __shfl_sync(FULL, r3, 31);
    if (TRACE) {
      if (m0) { trace.row_of_position[p0 + 0] = r0; trace.worker_of_position[p0 + 0] = wave_of(p0 + 0); }
      if (m1) { trace.row_of_position[p0 + 1] = r1; trace.worker_of_position[p0 + 1] = wave_of(p0 + 1); }
      if (m2) { trace.row_of_position[p0 + 2] = r2; trace.worker_of_position[p0 + 2] = wave_of(p0 + 2); }
      if (m3) { trace.row_of_position[p0 + 3] = r3; trace.worker_of_position[p0 + 3] = wave_of(p0 + 3); }
    }

    // ---- positions of long rows count as zero here (the band kernel adds them) ----------
    float z0 = q0, z1 = q1, z2 = q2, z3 = q3;
    bool tail_long = false;
    if (long_min > 0) {
      tail_long = __ldg(row_ptr + R_last + 1) - __ldg(row_ptr + R_last) >= long_min;
      if (head_long || tail_long) {
        const int ra = head_long ? R : -1, rb = tail_long ? R_last : -1;
        if (r0 == ra || r0 == rb) z0 = 0.0f;
        if (r1 == ra || r1 == rb) z1 = 0.0f;
        if (r2 == ra || r2 == rb) z2 = 0.0f;
        if (r3 == ra || r3 == rb) z3 = 0.0f;
      }
    }

    // ---- runs inside the lane --------------------------------------------------
    const int head_row = r0;
    float head = z0, cur = z0;
    int cur_row = r0;
    bool in_head = true;
    int head_last = p0 + 3;  // last position of the head run
#define SWB_RUN_STEP(RJ, QJ, J)                              \
    if ((RJ) == cur_row) {                                     \
      cur = add(cur, (QJ));                                    \
    } else {                                                   \
      if (in_head) { head = cur; head_last = p0 + (J) - 1; in_head = false; } \
      else emit(cur_row, cur, p0 + (J) - 1);                   \
      cur_row = (RJ);                                          \
      cur = (QJ);                                              \
    }
    SWB_RUN_STEP(r1, z1, 1)
    SWB_RUN_STEP(r2, z2, 2)
    SWB_RUN_STEP(r3, z3, 3)
#undef SWB_RUN_STEP
    const bool single = in_head;
    const int tail_row = cur_row;
    float tail = cur;

    // ---- the carried segment meets lane 0 -----------------------------------------
    int prev_tail_row = __shfl_up_sync(FULL, tail_row, 1);
    if (lane == 0) prev_tail_row = carry_row;
    const bool continues = (head_row == prev_tail_row);
    if (carry_row >= 0) {  // uniform
      const float total = warp_sum(acc);
      if (lane == 0) {
        if (continues) {
          if (single) tail = add(total, tail); else head = add(total, head);
        } else {
          emit(carry_row, total, carry_last);
        }
      }
    }

    // ---- segmented inclusive scan of the lanes' last runs -------------------------
    const bool seg_head = (lane == 0) || !(single && continues);
    const unsigned hmask = __ballot_sync(FULL, seg_head);
    const unsigned le = (lane == 31) ? FULL : ((1u << (lane + 1)) - 1u);
    const int dist = lane - (31 - __clz(hmask & le));
    float S = tail;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float t = __shfl_up_sync(FULL, S, off);
      if (off <= dist) S = add(S, t);
    }
    const float prevS = __shfl_up_sync(FULL, S, 1);
    if (!single) {
      // The lane's first run ends here: add what the lanes below carried into it.
      const float h = (continues && lane > 0) ? add(prevS, head) : head;
      emit(head_row, h, head_last);
    }
    const int next_head_row = __shfl_down_sync(FULL, head_row, 1);
    if (lane < 31 && next_head_row != tail_row) emit(tail_row, S, p0 + 3);
    carry_row = __shfl_sync(FULL, tail_row, 31);
    acc = (lane == 31) ? S : 0.0f;
    carry_last = ce - 1;
    R = R_last;
    next_b = __ldg(row_ptr + R + 1) + shift;
    head_long = tail_long;
  }
  if (carry_row >= 0) {
    const float total = warp_sum(acc);
    if (lane == 0) emit(carry_row, total, carry_last);
  }
}
