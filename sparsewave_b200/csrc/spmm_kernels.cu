// CSR SpMM kernels for sm_100a: thread-per-output, wave-per-row-tile and
// thread-per-position mappings of sparsewave.spmm.  B is cols x N and C is
// rows x N, row-major.  Products and sums are separate f32 operations.
#include "swb_index.h"
#include "swb_kernels.h"

namespace swb {
namespace {

constexpr unsigned FULL = 0xffffffffu;

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }

// ---------------------------------------------------------------------------
// thread-per-output (ThreadPerOutputSpMMPattern, SparseWaveToGPU.cpp:489-558)
// element = blockIdx * blockDim + threadIdx; row = element / N; column =
// element % N; sequential sum in position order (bit-identical to the CPU
// CSR loop).
// ---------------------------------------------------------------------------
__global__ void spmm_thread_per_output_kernel(int64_t rows, int64_t N,
                                              const int32_t *__restrict__ row_ptr,
                                              const int32_t *__restrict__ col,
                                              const float *__restrict__ val,
                                              const float *__restrict__ B, float *__restrict__ C) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= rows * N) return;
  const int64_t row = e / N, j = e % N;
  int p = row_ptr[row];
  const int end = row_ptr[row + 1];
  const float *Bj = B + j;
  float sum = 0.0f;
  for (; p + 4 <= end; p += 4) {
    int c0 = __ldg(col + p), c1 = __ldg(col + p + 1), c2 = __ldg(col + p + 2), c3 = __ldg(col + p + 3);
    float v0 = __ldg(val + p), v1 = __ldg(val + p + 1), v2 = __ldg(val + p + 2), v3 = __ldg(val + p + 3);
    float b0 = __ldg(Bj + (int64_t)c0 * N), b1 = __ldg(Bj + (int64_t)c1 * N);
    float b2 = __ldg(Bj + (int64_t)c2 * N), b3 = __ldg(Bj + (int64_t)c3 * N);
    sum = add(sum, mul(v0, b0));
    sum = add(sum, mul(v1, b1));
    sum = add(sum, mul(v2, b2));
    sum = add(sum, mul(v3, b3));
  }
  for (; p < end; ++p) sum = add(sum, mul(__ldg(val + p), __ldg(Bj + (int64_t)__ldg(col + p) * N)));
  C[e] = sum;
}

// The same mapping where N and the block size are multiples of 32: the 32 outputs of a warp lie in one
// matrix row, so the warp reads 32 positions of col and val with one coalesced load each and passes them
// around by shuffles instead of every lane loading every position (three L1 requests per position become
// one).  Each thread still adds its products in position order: bit-identical to the kernel above.
__global__ void spmm_thread_per_output_warp_row_kernel(int64_t rows, int64_t N,
                                                       const int32_t *__restrict__ row_ptr,
                                                       const int32_t *__restrict__ col,
                                                       const float *__restrict__ val,
                                                       const float *__restrict__ B, float *__restrict__ C) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= rows * N) return;  // rows * N is a multiple of 32: whole warps leave
  const int lane = threadIdx.x & 31;
  const int64_t row = e / N, j = e % N;
  const int start = row_ptr[row], end = row_ptr[row + 1];
  const float *Bj = B + j;
  float sum = 0.0f;
  for (int base = start; base < end; base += 32) {
    const int left = end - base < 32 ? end - base : 32;
    const int cl = lane < left ? __ldg(col + base + lane) : 0;
    const float vl = lane < left ? __ldg(val + base + lane) : 0.0f;
    int k = 0;
    for (; k + 4 <= left; k += 4) {
      const int c0 = __shfl_sync(FULL, cl, k), c1 = __shfl_sync(FULL, cl, k + 1);
      const int c2 = __shfl_sync(FULL, cl, k + 2), c3 = __shfl_sync(FULL, cl, k + 3);
      const float b0 = __ldg(Bj + (int64_t)c0 * N), b1 = __ldg(Bj + (int64_t)c1 * N);
      const float b2 = __ldg(Bj + (int64_t)c2 * N), b3 = __ldg(Bj + (int64_t)c3 * N);
      sum = add(sum, mul(__shfl_sync(FULL, vl, k), b0));
      sum = add(sum, mul(__shfl_sync(FULL, vl, k + 1), b1));
      sum = add(sum, mul(__shfl_sync(FULL, vl, k + 2), b2));
      sum = add(sum, mul(__shfl_sync(FULL, vl, k + 3), b3));
    }
    for (; k < left; ++k)
      sum = add(sum, mul(__shfl_sync(FULL, vl, k), __ldg(Bj + (int64_t)__shfl_sync(FULL, cl, k) * N)));
  }
  C[e] = sum;
}

// ---------------------------------------------------------------------------
// wave-per-row-tile (WavePerRowTileSpMMPattern, SparseWaveToGPU.cpp:1057-1256)
// tiles = ceil(N / T); unit = blockIdx * (blockDim/32) + threadIdx/32;
// row = unit / tiles; tile = unit % tiles; first column = tile * T.  Lanes
// stride the row's positions; each position's value is loaded once and used
// for the T right-hand-side columns of the tile.  A tile that reaches past N
// runs the guarded path.
//
// TCAP is T rounded up to a power of two (columns k >= T are inactive).  Full
// tiles of 4, 8, 16 or 32 columns on 16-byte aligned operands take the
// vectorised kernel further below instead.
//
// Reduction: instead of T independent 5-step butterflies (5*T shuffles) the
// warp does a halving exchange: at the step with lane distance `off` each
// lane keeps one half of its accumulators and sends the other half to its
// partner, so the accumulator count halves per step until one is left
// (TCAP-1 shuffles), then plain butterfly steps finish.  Lane l ends with the
// full sum of column (l >> (5 - log2 TCAP)) of the tile.
// ---------------------------------------------------------------------------
template <int TCAP>
__device__ __forceinline__ void tile_reduce(float (&acc)[TCAP], int lane) {
  int w = TCAP;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    if (w > 1) {
      const int half = w >> 1;
      const bool upper = (lane & off) != 0;
#pragma unroll
      for (int i = 0; i < TCAP / 2; ++i) {
        if (i < half) {
          const float send = upper ? acc[i] : acc[i + half];
          const float keep = upper ? acc[i + half] : acc[i];
          acc[i] = add(keep, __shfl_xor_sync(FULL, send, off));
        }
      }
      w = half;
    } else {
      acc[0] = add(acc[0], __shfl_xor_sync(FULL, acc[0], off));
    }
  }
}

// Column (within the tile) whose sum lane `lane` holds after tile_reduce.
template <int TCAP>
__device__ __forceinline__ int tile_column_of_lane(int lane) {
  int k = 0, w = TCAP;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    if (w > 1) {
      w >>= 1;
      if (lane & off) k += w;
    }
  }
  return k;
}

// Lowest lane holding column k: the lanes whose "kept" bits spell k and whose
// remaining low bits are zero.
template <int TCAP>
__device__ __forceinline__ bool lane_is_column_writer(int lane) {
  int w = TCAP, used = 0;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    if (w > 1) {
      w >>= 1;
      used |= off;
    }
  }
  return (lane & ~used) == 0;
}

template <int TCAP>
__global__ void spmm_wave_per_row_tile_kernel(int64_t rows, int64_t N, int T, int64_t tiles,
                                              const int32_t *__restrict__ row_ptr,
                                              const int32_t *__restrict__ col,
                                              const float *__restrict__ val,
                                              const float *__restrict__ B, float *__restrict__ C,
                                              bool accumulate) {
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= rows * tiles) return;
  const int64_t row = unit / tiles;
  const int64_t j0 = (unit % tiles) * T;
  const int start = row_ptr[row], end = row_ptr[row + 1];
  const bool full = j0 + T <= N;

  float acc[TCAP];
#pragma unroll
  for (int k = 0; k < TCAP; ++k) acc[k] = 0.0f;

  if (full && T == TCAP) {
    for (int p = start + lane; p < end; p += 32) {
      const int c = __ldcs(col + p);
      const float v = __ldcs(val + p);
      const float *b = B + (int64_t)c * N + j0;
#pragma unroll
      for (int k = 0; k < TCAP; ++k) acc[k] = add(acc[k], mul(v, __ldg(b + k)));
    }
  } else {
    // Guarded path: tail tile (or T below the register capacity).
    for (int p = start + lane; p < end; p += 32) {
      const int c = __ldcs(col + p);
      const float v = __ldcs(val + p);
      const float *b = B + (int64_t)c * N + j0;
#pragma unroll
      for (int k = 0; k < TCAP; ++k)
        if (k < T && j0 + k < N) acc[k] = add(acc[k], mul(v, __ldg(b + k)));
    }
  }

  tile_reduce<TCAP>(acc, lane);
  const int k = tile_column_of_lane<TCAP>(lane);
  if (lane_is_column_writer<TCAP>(lane) && k < T && j0 + k < N) {
    float *out = C + row * N + j0 + k;
    *out = accumulate ? add(*out, acc[0]) : acc[0];
  }
}

// Full tiles of 4, 8, 16 or 32 columns with 16-byte aligned B and C rows.  The
// unit <-> (row, tile) assignment is the same; inside the warp G = T/4 adjacent
// lanes share a position and read the tile's T floats of that B row as one
// contiguous run of G float4 (64 contiguous bytes per position for T = 16), and
// the 32/G lane groups stride the row's positions.  Each lane keeps one float4
// of partial sums.  Reduction over the lane groups: two halving exchanges (lane
// distance 16 keeps two of the four components, distance 8 keeps one), then
// plain butterfly steps down to distance G: 3 + log2(8/G) shuffles.
template <int G>
__global__ void spmm_wave_per_row_tile_vec_kernel(int64_t rows, int64_t N, int64_t tiles,
                                                  const int32_t *__restrict__ row_ptr,
                                                  const int32_t *__restrict__ col,
                                                  const float *__restrict__ val,
                                                  const float *__restrict__ B, float *__restrict__ C,
                                                  bool accumulate) {
  constexpr int T = 4 * G, PG = 32 / G;
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= rows * tiles) return;
  const int64_t row = unit / tiles;
  const int64_t j0 = (unit % tiles) * T;
  const int cq = lane % G, pg = lane / G;
  const int start = row_ptr[row], end = row_ptr[row + 1];
  const float *Bt = B + j0 + 4 * cq;

  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if constexpr (G >= 4) {
    // 32 positions per pass, read by the whole warp with one coalesced load of col and one of val and
    // handed to the lane groups by shuffles (see the fused-row kernel below); same order of additions
    auto fma4 = [&](float v, const float4 &b) {
      acc.x = add(acc.x, mul(v, b.x)); acc.y = add(acc.y, mul(v, b.y));
      acc.z = add(acc.z, mul(v, b.z)); acc.w = add(acc.w, mul(v, b.w));
    };
    int cn = start + lane < end ? __ldg(col + start + lane) : 0;
    float vn = start + lane < end ? __ldg(val + start + lane) : 0.0f;
    for (int base = start; base < end; base += 32) {
      const int cl = cn;
      const float vl = vn;
      const int mine = base + 32 + lane;
      cn = mine < end ? __ldg(col + mine) : 0;
      vn = mine < end ? __ldg(val + mine) : 0.0f;
      const int left = end - base < 32 ? end - base : 32;
      int j = 0;
      for (; j + 4 * PG <= left; j += 4 * PG) {
        const int k = j + pg;
        const int c0 = __shfl_sync(FULL, cl, k), c1 = __shfl_sync(FULL, cl, k + PG);
        const int c2 = __shfl_sync(FULL, cl, k + 2 * PG), c3 = __shfl_sync(FULL, cl, k + 3 * PG);
        const float4 b0 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c0 * N));
        const float4 b1 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c1 * N));
        const float4 b2 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c2 * N));
        const float4 b3 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c3 * N));
        const float v0 = __shfl_sync(FULL, vl, k), v1 = __shfl_sync(FULL, vl, k + PG);
        const float v2 = __shfl_sync(FULL, vl, k + 2 * PG), v3 = __shfl_sync(FULL, vl, k + 3 * PG);
        fma4(v0, b0); fma4(v1, b1); fma4(v2, b2); fma4(v3, b3);
      }
      for (; j < left; j += PG) {
        const int kk = j + pg;
        const int c0 = __shfl_sync(FULL, cl, kk & 31);
        const float v0 = __shfl_sync(FULL, vl, kk & 31);
        if (kk < left) fma4(v0, __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c0 * N)));
      }
    }
  } else {
  int p = start + pg;
  for (; p + PG < end; p += 2 * PG) {
    const int c0 = __ldg(col + p), c1 = __ldg(col + p + PG);
    const float v0 = __ldg(val + p), v1 = __ldg(val + p + PG);
    const float4 b0 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c0 * N));
    const float4 b1 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c1 * N));
    acc.x = add(acc.x, mul(v0, b0.x)); acc.y = add(acc.y, mul(v0, b0.y));
    acc.z = add(acc.z, mul(v0, b0.z)); acc.w = add(acc.w, mul(v0, b0.w));
    acc.x = add(acc.x, mul(v1, b1.x)); acc.y = add(acc.y, mul(v1, b1.y));
    acc.z = add(acc.z, mul(v1, b1.z)); acc.w = add(acc.w, mul(v1, b1.w));
  }
  if (p < end) {
    const int c0 = __ldg(col + p);
    const float v0 = __ldg(val + p);
    const float4 b0 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c0 * N));
    acc.x = add(acc.x, mul(v0, b0.x)); acc.y = add(acc.y, mul(v0, b0.y));
    acc.z = add(acc.z, mul(v0, b0.z)); acc.w = add(acc.w, mul(v0, b0.w));
  }
  }

  // distance 16: lanes with bit 4 set keep (z, w), the others (x, y)
  const bool up16 = (lane & 16) != 0;
  float k0 = up16 ? acc.z : acc.x, k1 = up16 ? acc.w : acc.y;
  const float s0 = up16 ? acc.x : acc.z, s1 = up16 ? acc.y : acc.w;
  k0 = add(k0, __shfl_xor_sync(FULL, s0, 16));
  k1 = add(k1, __shfl_xor_sync(FULL, s1, 16));
  // distance 8: lanes with bit 3 set keep the second of the two
  const bool up8 = (lane & 8) != 0;
  float r = up8 ? k1 : k0;
  const float s = up8 ? k0 : k1;
  r = add(r, __shfl_xor_sync(FULL, s, 8));
#pragma unroll
  for (int off = 4; off >= G; off >>= 1) r = add(r, __shfl_xor_sync(FULL, r, off));
  const int comp = (up16 ? 2 : 0) + (up8 ? 1 : 0);
  if ((lane & 7 & ~(G - 1)) == 0) {
    float *out = C + row * N + j0 + 4 * cq + comp;
    *out = accumulate ? add(*out, r) : r;
  }
}

// Whole rows of B of 16 to 128 floats (G = N/4 = 4 to 32 lanes per row): every tile of a matrix row is
// computed by one warp in one pass - the (row, tile) units of a row are fused - so the row's col/val
// stream is read once instead of once per tile and each nonzero fetches its B row as one contiguous
// run of 64 to 512 bytes.  The warp reads 32 positions of col and val with one coalesced load each (the
// next 32 are requested before the rows of B of the current ones) and hands them to the 32/G lane groups
// by shuffles; a group takes every (32/G)-th position, four rows of B in flight per group.  Reading col
// and val per group with broadcast loads instead costs one L1 request per position and group and was
// 16 % slower on 2 M rows of 64 nonzeros with N = 64 (3.46 -> 2.90 ms).  The partial float4 sums of the
// groups are added with butterfly steps and group 0 stores the row of C.
template <int G>
__global__ void spmm_wave_per_row_fused_kernel(int64_t rows, int64_t N, const int32_t *__restrict__ row_ptr,
                                               const int32_t *__restrict__ col, const float *__restrict__ val,
                                               const float *__restrict__ B, float *__restrict__ C,
                                               bool accumulate) {
  constexpr int PG = 32 / G;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int cq = lane % G, pg = lane / G;
  const int start = row_ptr[row], end = row_ptr[row + 1];
  const float *Bt = B + 4 * cq;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  auto fma4 = [&](float v, const float4 &b) {
    acc.x = add(acc.x, mul(v, b.x)); acc.y = add(acc.y, mul(v, b.y));
    acc.z = add(acc.z, mul(v, b.z)); acc.w = add(acc.w, mul(v, b.w));
  };
  // 32 positions per pass: one coalesced load of col and of val by the whole warp, handed to the lane
  // groups by shuffles (group pg takes positions base + pg, base + pg + PG, ... as before: same sums)
  int cn = start + lane < end ? __ldg(col + start + lane) : 0;
  float vn = start + lane < end ? __ldg(val + start + lane) : 0.0f;
  for (int base = start; base < end; base += 32) {
    const int cl = cn;
    const float vl = vn;
    const int mine = base + 32 + lane;  // the next pass is requested before this one's rows of B
    cn = mine < end ? __ldg(col + mine) : 0;
    vn = mine < end ? __ldg(val + mine) : 0.0f;
    const int left = end - base < 32 ? end - base : 32;  // positions of this pass
    int j = 0;  // warp-uniform: positions of the pass handed out so far (every lane joins every shuffle)
    for (; j + 4 * PG <= left; j += 4 * PG) {
      const int k = j + pg;  // position of this group inside the pass
      const int c0 = __shfl_sync(FULL, cl, k), c1 = __shfl_sync(FULL, cl, k + PG);
      const int c2 = __shfl_sync(FULL, cl, k + 2 * PG), c3 = __shfl_sync(FULL, cl, k + 3 * PG);
      const float4 b0 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c0 * N));
      const float4 b1 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c1 * N));
      const float4 b2 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c2 * N));
      const float4 b3 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c3 * N));
      const float v0 = __shfl_sync(FULL, vl, k), v1 = __shfl_sync(FULL, vl, k + PG);
      const float v2 = __shfl_sync(FULL, vl, k + 2 * PG), v3 = __shfl_sync(FULL, vl, k + 3 * PG);
      fma4(v0, b0); fma4(v1, b1); fma4(v2, b2); fma4(v3, b3);
    }
    for (; j + 2 * PG <= left; j += 2 * PG) {  // short rows and row ends: two rows of B in flight
      const int k = j + pg;
      const int c0 = __shfl_sync(FULL, cl, k), c1 = __shfl_sync(FULL, cl, k + PG);
      const float4 b0 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c0 * N));
      const float4 b1 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c1 * N));
      const float v0 = __shfl_sync(FULL, vl, k), v1 = __shfl_sync(FULL, vl, k + PG);
      fma4(v0, b0); fma4(v1, b1);
    }
    // the ragged end of the pass: every lane takes part in the shuffles, only lanes with a position add
    for (; j < left; j += PG) {
      const int kk = j + pg;
      const int c0 = __shfl_sync(FULL, cl, kk & 31);
      const float v0 = __shfl_sync(FULL, vl, kk & 31);
      if (kk < left) fma4(v0, __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c0 * N)));
    }
  }
#pragma unroll
  for (int off = G; off < 32; off <<= 1) {
    acc.x = add(acc.x, __shfl_xor_sync(FULL, acc.x, off));
    acc.y = add(acc.y, __shfl_xor_sync(FULL, acc.y, off));
    acc.z = add(acc.z, __shfl_xor_sync(FULL, acc.z, off));
    acc.w = add(acc.w, __shfl_xor_sync(FULL, acc.w, off));
  }
  if (pg == 0) {
    float4 *out = reinterpret_cast<float4 *>(C + row * N) + cq;
    if (accumulate) {
      const float4 old = *out;
      acc.x = add(old.x, acc.x); acc.y = add(old.y, acc.y); acc.z = add(old.z, acc.z); acc.w = add(old.w, acc.w);
    }
    *out = acc;
  }
}

// Rows of B of 4 * G floats with G no power of two (N = 12, 20, 24, 28, 36 ... 124): the same fusion with
// PG = 32 / G (rounded down) lane groups on PG * G of the warp's lanes; the other lanes only take part in the
// shuffles.  The groups' partial sums are added into group 0 one after the other.
__global__ void spmm_wave_per_row_any_kernel(int64_t rows, int64_t N, int G, const int32_t *__restrict__ row_ptr,
                                             const int32_t *__restrict__ col, const float *__restrict__ val,
                                             const float *__restrict__ B, float *__restrict__ C,
                                             bool accumulate) {
  const int PG = 32 / G;
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const bool active = lane < PG * G;
  const int cq = lane % G, pg = active ? lane / G : 0;
  const int start = row_ptr[row], end = row_ptr[row + 1];
  const float *Bt = B + 4 * cq;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  auto fma4 = [&](float v, const float4 &b) {
    acc.x = add(acc.x, mul(v, b.x)); acc.y = add(acc.y, mul(v, b.y));
    acc.z = add(acc.z, mul(v, b.z)); acc.w = add(acc.w, mul(v, b.w));
  };
  int cn = start + lane < end ? __ldg(col + start + lane) : 0;
  float vn = start + lane < end ? __ldg(val + start + lane) : 0.0f;
  for (int base = start; base < end; base += 32) {
    const int cl = cn;
    const float vl = vn;
    const int mine = base + 32 + lane;
    cn = mine < end ? __ldg(col + mine) : 0;
    vn = mine < end ? __ldg(val + mine) : 0.0f;
    const int left = end - base < 32 ? end - base : 32;
    int j = 0;  // warp-uniform
    for (; j + 4 * PG <= left; j += 4 * PG) {
      const int k = j + pg;
      const int c0 = __shfl_sync(FULL, cl, k), c1 = __shfl_sync(FULL, cl, k + PG);
      const int c2 = __shfl_sync(FULL, cl, k + 2 * PG), c3 = __shfl_sync(FULL, cl, k + 3 * PG);
      const float v0 = __shfl_sync(FULL, vl, k), v1 = __shfl_sync(FULL, vl, k + PG);
      const float v2 = __shfl_sync(FULL, vl, k + 2 * PG), v3 = __shfl_sync(FULL, vl, k + 3 * PG);
      if (active) {
        const float4 b0 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c0 * N));
        const float4 b1 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c1 * N));
        const float4 b2 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c2 * N));
        const float4 b3 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c3 * N));
        fma4(v0, b0); fma4(v1, b1); fma4(v2, b2); fma4(v3, b3);
      }
    }
    for (; j < left; j += PG) {
      const int kk = j + pg;
      const int c0 = __shfl_sync(FULL, cl, kk & 31);
      const float v0 = __shfl_sync(FULL, vl, kk & 31);
      if (active && kk < left) fma4(v0, __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c0 * N)));
    }
  }
  for (int g = 1; g < PG; ++g) {  // group g's sums into group 0, in group order
    const int src = (lane + g * G) & 31;
    const float tx = __shfl_sync(FULL, acc.x, src), ty = __shfl_sync(FULL, acc.y, src);
    const float tz = __shfl_sync(FULL, acc.z, src), tw = __shfl_sync(FULL, acc.w, src);
    if (lane < G) { acc.x = add(acc.x, tx); acc.y = add(acc.y, ty); acc.z = add(acc.z, tz); acc.w = add(acc.w, tw); }
  }
  if (lane < G) {
    float4 *out = reinterpret_cast<float4 *>(C + row * N) + cq;
    if (accumulate) {
      const float4 old = *out;
      acc.x = add(old.x, acc.x); acc.y = add(old.y, acc.y); acc.z = add(old.z, acc.z); acc.w = add(old.w, acc.w);
    }
    *out = acc;
  }
}

// Rows of B of 128 * R floats (R = 2, 3, 4): the same fusion with the whole warp on one position; a lane
// holds R float4 of the row of C (columns 4 * lane + 128 * r) and reads the position's row of B as R
// coalesced 512-byte runs.  Two positions are in flight for R = 2, one for wider rows (as many bytes per
// lane as in the kernel above).
template <int R>
__global__ void spmm_wave_per_row_wide_kernel(int64_t rows, int64_t N, const int32_t *__restrict__ row_ptr,
                                              const int32_t *__restrict__ col, const float *__restrict__ val,
                                              const float *__restrict__ B, float *__restrict__ C,
                                              bool accumulate) {
  constexpr int U = R == 2 ? 2 : 1;  // positions in flight
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int start = row_ptr[row], end = row_ptr[row + 1];
  const float4 *Bt = reinterpret_cast<const float4 *>(B) + lane;
  const int64_t N4 = N / 4;
  float4 acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = make_float4(0.f, 0.f, 0.f, 0.f);
  auto fma4 = [&](float4 &a, float v, const float4 &b) {
    a.x = add(a.x, mul(v, b.x)); a.y = add(a.y, mul(v, b.y));
    a.z = add(a.z, mul(v, b.z)); a.w = add(a.w, mul(v, b.w));
  };
  int cn = start + lane < end ? __ldg(col + start + lane) : 0;
  float vn = start + lane < end ? __ldg(val + start + lane) : 0.0f;
  for (int base = start; base < end; base += 32) {
    const int cl = cn;
    const float vl = vn;
    const int mine = base + 32 + lane;
    cn = mine < end ? __ldg(col + mine) : 0;
    vn = mine < end ? __ldg(val + mine) : 0.0f;
    const int left = end - base < 32 ? end - base : 32;
    int j = 0;
    for (; j + U <= left; j += U) {
      float4 b[U][R];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float4 *brow = Bt + (int64_t)__shfl_sync(FULL, cl, j + u) * N4;
#pragma unroll
        for (int r = 0; r < R; ++r) b[u][r] = __ldg(brow + 32 * r);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const float v = __shfl_sync(FULL, vl, j + u);
#pragma unroll
        for (int r = 0; r < R; ++r) fma4(acc[r], v, b[u][r]);
      }
    }
    if (U > 1 && j < left) {  // U == 2: one position left over
      const float4 *brow = Bt + (int64_t)__shfl_sync(FULL, cl, j) * N4;
      const float v = __shfl_sync(FULL, vl, j);
#pragma unroll
      for (int r = 0; r < R; ++r) fma4(acc[r], v, __ldg(brow + 32 * r));
    }
  }
  float4 *out = reinterpret_cast<float4 *>(C + row * N) + lane;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float4 a = acc[r];
    if (accumulate) {
      const float4 old = out[32 * r];
      a.x = add(old.x, a.x); a.y = add(old.y, a.y); a.z = add(old.z, a.z); a.w = add(old.w, a.w);
    }
    out[32 * r] = a;
  }
}

// Short matrix rows with rows of B of up to 32 floats: a full warp per row leaves most lanes with one
// position or none and the kernel waits on three dependent loads per warp.  Here L = 4, 8 or 16 lanes
// serve one matrix row (32/L rows per warp): G = N/4 adjacent lanes cover the row of B with one float4
// each, the L/G lane groups stride the row's positions with four positions in flight, butterfly steps
// over the lane distances G ... L/2 add the groups' partial sums, group 0 stores the row of C.
template <int G, int L>
__global__ void spmm_subwarp_row_kernel(int64_t rows, int64_t N, const int32_t *__restrict__ row_ptr,
                                        const int32_t *__restrict__ col, const float *__restrict__ val,
                                        const float *__restrict__ B, float *__restrict__ C, bool accumulate) {
  constexpr int PG = L / G, RW = 32 / L;
  static_assert(L >= G && L < 32 && PG >= 1, "lanes per row");
  const int lane = threadIdx.x & 31;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (warp * RW >= rows) return;  // whole warp out of range
  const int l = lane % L, cq = l % G, pg = l / G;
  const int64_t row = warp * RW + lane / L;
  const bool live = row < rows;  // lanes past the last row still take part in the shuffles
  const int start = live ? row_ptr[row] : 0, end = live ? row_ptr[row + 1] : 0;
  const float *Bt = B + 4 * cq;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  auto fma4 = [&](float v, const float4 &b) {
    acc.x = add(acc.x, mul(v, b.x)); acc.y = add(acc.y, mul(v, b.y));
    acc.z = add(acc.z, mul(v, b.z)); acc.w = add(acc.w, mul(v, b.w));
  };
  int p = start + pg;
  for (; p + 3 * PG < end; p += 4 * PG) {
    const int c0 = __ldg(col + p), c1 = __ldg(col + p + PG), c2 = __ldg(col + p + 2 * PG), c3 = __ldg(col + p + 3 * PG);
    const float v0 = __ldg(val + p), v1 = __ldg(val + p + PG), v2 = __ldg(val + p + 2 * PG), v3 = __ldg(val + p + 3 * PG);
    const float4 b0 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c0 * N));
    const float4 b1 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c1 * N));
    const float4 b2 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c2 * N));
    const float4 b3 = __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c3 * N));
    fma4(v0, b0); fma4(v1, b1); fma4(v2, b2); fma4(v3, b3);
  }
  for (; p < end; p += PG) {
    const int c0 = __ldg(col + p);
    const float v0 = __ldg(val + p);
    fma4(v0, __ldg(reinterpret_cast<const float4 *>(Bt + (int64_t)c0 * N)));
  }
#pragma unroll
  for (int off = G; off < L; off <<= 1) {
    acc.x = add(acc.x, __shfl_xor_sync(FULL, acc.x, off));
    acc.y = add(acc.y, __shfl_xor_sync(FULL, acc.y, off));
    acc.z = add(acc.z, __shfl_xor_sync(FULL, acc.z, off));
    acc.w = add(acc.w, __shfl_xor_sync(FULL, acc.w, off));
  }
  if (live && pg == 0) {
    float4 *out = reinterpret_cast<float4 *>(C + row * N) + cq;
    if (accumulate) {
      const float4 old = *out;
      acc.x = add(old.x, acc.x); acc.y = add(old.y, acc.y); acc.z = add(old.z, acc.z); acc.w = add(old.w, acc.w);
    }
    *out = acc;
  }
}

// ---------------------------------------------------------------------------
// thread-per-position (DecomposePositionSpMMPattern,
// PositionSpMMDecomposition.cpp:19-73, scheduled with the thread/atomic
// schedule, Pipelines.cpp:262-271).  The iteration space is [0, nnz*N):
// position = i / N, column = i % N, key = row*N + column; worker w owns
// iterations [w*chunk, min(nnz*N, (w+1)*chunk)) and issues one atomicAdd per
// iteration.
// ---------------------------------------------------------------------------
__global__ void spmm_thread_per_position_kernel(int64_t rows, int64_t nnz, int64_t N, int64_t chunk,
                                                const int32_t *__restrict__ row_ptr,
                                                const int32_t *__restrict__ col,
                                                const float *__restrict__ val,
                                                const float *__restrict__ B, float *__restrict__ C) {
  const int64_t worker = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  int64_t begin, end;
  chunk_bounds(0, nnz * N, worker, chunk, begin, end);
  if (begin >= end) return;
  int64_t p = begin / N, j = begin % N;
  int64_t row = row_at_position(row_ptr, rows + 1, p);
  int64_t next = row_ptr[row + 1];
  int c = __ldg(col + p);
  float v = __ldg(val + p);
  for (int64_t i = begin; i < end; ++i) {
    atomicAdd(C + row * N + j, mul(v, __ldg(B + (int64_t)c * N + j)));
    if (++j == N) {
      j = 0;
      ++p;
      if (i + 1 < end) {
        while (next <= p) {
          ++row;
          next = row_ptr[row + 1];
        }
        c = __ldg(col + p);
        v = __ldg(val + p);
      }
    }
  }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// CUDA grids hold at most 2^31 - 1 blocks in x; a launch that needs more is refused instead of truncated.
#define SWB_GRID(name, blocks)                                      \
  unsigned name = 0;                                                 \
  if (!grid_dim(blocks, &name)) return cudaErrorInvalidConfiguration

template <int TCAP>
cudaError_t launch_tile(const CsrSpmmArgs &a, int block, int T, cudaStream_t s) {
  const int64_t tiles = ceil_div(a.n_rhs, T);
  const int64_t units = a.rows * tiles;
  SWB_GRID(grid, ceil_div(units, block / 32));
  const bool vec = (T == TCAP) && (TCAP % 4 == 0) && (a.n_rhs % 4 == 0) && (a.n_rhs % T == 0) &&
                   aligned16(a.B) && aligned16(a.C);
  if (vec) {
    if constexpr (TCAP >= 4)
      spmm_wave_per_row_tile_vec_kernel<TCAP / 4><<<grid, block, 0, s>>>(a.rows, a.n_rhs, tiles, a.row_ptr,
                                                                          a.col_idx, a.val, a.B, a.C, a.accumulate);
  } else {
    spmm_wave_per_row_tile_kernel<TCAP><<<grid, block, 0, s>>>(
        a.rows, a.n_rhs, T, tiles, a.row_ptr, a.col_idx, a.val, a.B, a.C, a.accumulate);
  }
  return cudaGetLastError();
}

template <int G, int L>
cudaError_t launch_subwarp(const CsrSpmmArgs &a, int block, cudaStream_t s) {
  const int64_t warps = ceil_div(a.rows, 32 / L);
  SWB_GRID(grid, ceil_div(warps, block / 32));
  spmm_subwarp_row_kernel<G, L><<<grid, block, 0, s>>>(
      a.rows, a.n_rhs, a.row_ptr, a.col_idx, a.val, a.B, a.C, a.accumulate);
  return cudaGetLastError();
}

// Lanes per matrix row for rows of B of 4*G floats: at least 4 lanes (and at least G), at most the warp,
// doubled while a lane group would get more than positions_per_lane_group(G) of the mean row's positions.
// The figures are measured (1 M and 2 M rows, uniform columns, 2 to 64 positions per row): few lanes per row
// mean more rows in flight per warp and fewer butterfly steps, and win until the per-group chain of
// positions gets long.  Against four positions per group for every width: N = 8, 24 per row 0.226 -> 0.125 ms;
// N = 16, 24 per row 0.492 -> 0.205 ms; N = 32, 10 per row 0.514 -> 0.246 ms; N = 64, 5 per row (half a warp
// instead of a warp) 1.02 -> 0.53 ms.
constexpr int64_t positions_per_lane_group(int G) { return G == 1 ? 6 : G == 2 ? 12 : G <= 8 ? 16 : 12; }

template <int G>
cudaError_t launch_row_of_tiles(const CsrSpmmArgs &a, int block, cudaStream_t s) {
  const int64_t mean = a.rows > 0 ? a.nnz / a.rows : 0;
  int lanes = G > 4 ? G : 4;
  constexpr int64_t kPerGroup = positions_per_lane_group(G);
  while (lanes < 32 && (int64_t)(lanes / G) * kPerGroup < mean) lanes *= 2;
  if constexpr (G <= 4) if (lanes == 4) return launch_subwarp<G, 4>(a, block, s);
  if constexpr (G <= 8) if (lanes == 8) return launch_subwarp<G, 8>(a, block, s);
  if (lanes == 16) return launch_subwarp<G, 16>(a, block, s);
  if constexpr (G >= 4) {  // a warp per row, col/val handed to the lane groups by shuffles
    SWB_GRID(grid, ceil_div(a.rows, block / 32));
    spmm_wave_per_row_fused_kernel<G><<<grid, block, 0, s>>>(a.rows, a.n_rhs, a.row_ptr, a.col_idx, a.val, a.B, a.C,
                                                             a.accumulate);
    return cudaGetLastError();
  } else {
    return launch_tile<4 * G>(a, block, 4 * G, s);
  }
}

}  // namespace

cudaError_t launch_spmm_thread_per_output(const CsrSpmmArgs &a, int block, cudaStream_t s,
                                          int64_t *launches) {
  SWB_GRID(grid, ceil_div(a.rows * a.n_rhs, block));
  if (a.n_rhs % 32 == 0 && block % 32 == 0)
    spmm_thread_per_output_warp_row_kernel<<<grid, block, 0, s>>>(a.rows, a.n_rhs, a.row_ptr, a.col_idx, a.val, a.B,
                                                                  a.C);
  else
    spmm_thread_per_output_kernel<<<grid, block, 0, s>>>(a.rows, a.n_rhs, a.row_ptr, a.col_idx, a.val, a.B, a.C);
  ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_spmm_wave_per_row_tile(const CsrSpmmArgs &a, int block, int tile,
                                          cudaStream_t s, int64_t *launches) {
  ++*launches;
  // Rows of B of 4, 8, ... 128 floats on 16-byte aligned operands: all tiles of a matrix row are fused
  // into one pass (the tile size then only names the logical units, SparseWaveToGPU.cpp:1078-1084), by a
  // warp, or by part of a warp where the rows are short.
  const int64_t N = a.n_rhs;
  const bool pow2_row = N >= 4 && N <= 128 && (N & (N - 1)) == 0;
  if ((N == 256 || N == 384 || N == 512) && aligned16(a.B) && aligned16(a.C)) {
    SWB_GRID(grid, ceil_div(a.rows, block / 32));
    if (N == 256)
      spmm_wave_per_row_wide_kernel<2><<<grid, block, 0, s>>>(a.rows, N, a.row_ptr, a.col_idx, a.val, a.B, a.C, a.accumulate);
    else if (N == 384)
      spmm_wave_per_row_wide_kernel<3><<<grid, block, 0, s>>>(a.rows, N, a.row_ptr, a.col_idx, a.val, a.B, a.C, a.accumulate);
    else
      spmm_wave_per_row_wide_kernel<4><<<grid, block, 0, s>>>(a.rows, N, a.row_ptr, a.col_idx, a.val, a.B, a.C, a.accumulate);
    return cudaGetLastError();
  }
  // other multiples of 4 up to 124 (rows of B of 12, 20, 24 ... floats) where a matrix row has enough positions
  // for a warp: one warp per row as well
  if (N >= 12 && N < 128 && N % 4 == 0 && !pow2_row && a.rows > 0 && a.nnz / a.rows >= 8 && aligned16(a.B) &&
      aligned16(a.C)) {
    SWB_GRID(grid, ceil_div(a.rows, block / 32));
    spmm_wave_per_row_any_kernel<<<grid, block, 0, s>>>(a.rows, N, (int)(N / 4), a.row_ptr, a.col_idx, a.val, a.B,
                                                       a.C, a.accumulate);
    return cudaGetLastError();
  }
  if (pow2_row && aligned16(a.B) && aligned16(a.C)) {
    if (N == 4) return launch_row_of_tiles<1>(a, block, s);
    if (N == 8) return launch_row_of_tiles<2>(a, block, s);
    if (N == 16) return launch_row_of_tiles<4>(a, block, s);
    if (N == 32) return launch_row_of_tiles<8>(a, block, s);
    if (N == 64) return launch_row_of_tiles<16>(a, block, s);  // half a warp per row where rows are short
    SWB_GRID(grid, ceil_div(a.rows, block / 32));
    spmm_wave_per_row_fused_kernel<32><<<grid, block, 0, s>>>(a.rows, N, a.row_ptr, a.col_idx, a.val, a.B, a.C,
                                                               a.accumulate);
    return cudaGetLastError();
  }
  if (tile <= 1) return launch_tile<1>(a, block, tile, s);
  if (tile <= 2) return launch_tile<2>(a, block, tile, s);
  if (tile <= 4) return launch_tile<4>(a, block, tile, s);
  if (tile <= 8) return launch_tile<8>(a, block, tile, s);
  if (tile <= 16) return launch_tile<16>(a, block, tile, s);
  return launch_tile<32>(a, block, tile, s);
}

int64_t wave_per_row_tile_physical_grid(int64_t rows, int64_t nnz, int64_t n_rhs, int block, int tile) {
  // Mirrors launch_spmm_wave_per_row_tile and launch_row_of_tiles for 16-byte aligned operands.
  const int64_t wpb = block / 32;
  const bool pow2_row = n_rhs >= 4 && n_rhs <= 128 && (n_rhs & (n_rhs - 1)) == 0;
  if (n_rhs == 256 || n_rhs == 384 || n_rhs == 512) return max1(ceil_div(rows, wpb));
  if (n_rhs >= 12 && n_rhs < 128 && n_rhs % 4 == 0 && !pow2_row && rows > 0 && nnz / rows >= 8)
    return max1(ceil_div(rows, wpb));
  if (!pow2_row) return max1(ceil_div(rows * ceil_div(n_rhs, tile), wpb));
  if (n_rhs > 64) return max1(ceil_div(rows, wpb));
  const int64_t G = n_rhs / 4, mean = rows > 0 ? nnz / rows : 0;
  int64_t lanes = G > 4 ? G : 4;
  while (lanes < 32 && (lanes / G) * positions_per_lane_group((int)G) < mean) lanes *= 2;
  return max1(ceil_div(ceil_div(rows, 32 / lanes), wpb));
}

cudaError_t launch_spmm_thread_per_position(const CsrSpmmArgs &a, int block, int64_t chunk,
                                            cudaStream_t s, int64_t *launches) {
  // Zero fill of the flattened output, then the atomic schedule.
  const int64_t workers = ceil_div(a.nnz * a.n_rhs, chunk);
  SWB_GRID(grid, ceil_div(workers, block));
  if (!a.accumulate) {
    cudaError_t e = launch_fill_zero(a.C, a.rows * a.n_rhs, block, s, launches);
    if (e != cudaSuccess) return e;
  }
  spmm_thread_per_position_kernel<<<grid, block, 0, s>>>(a.rows, a.nnz, a.n_rhs, chunk, a.row_ptr,
                                                         a.col_idx, a.val, a.B, a.C);
  ++*launches;
  return cudaGetLastError();
}

}  // namespace swb
