// wave-per-row-tile SpMM with a TMA-staged slice of B in shared memory, for matrices whose nonzeros
// cluster around the diagonal (banded or banded-plus-random structure).
//
// Reference mapping: WavePerRowTileSpMMPattern (SparseWaveToGPU.cpp:1057-1256): a wave owns one (row, tile
// of T right-hand-side columns) unit and reuses each loaded value across the tile; the reference reads B
// with T scalar loads per position (:1140-1151).  Here a CTA owns STAGED_ROWS adjacent matrix rows and
// one tile of 16 columns: the rows of B that the band of those matrix rows can touch, B[r0 - HALO,
// r0 + STAGED_ROWS + HALO) x 16 columns (3072 x 64 bytes = 192 KiB), are brought into shared memory once by
// TMA (cp.async.bulk.tensor.2d, twelve boxes of 256 rows, no multicast), and every position whose column
// falls into that window reads its 64-byte piece of B from shared memory; the others read it from global
// memory as before.  A warp walks whole matrix rows: four lanes cover the 16 columns of a position with one
// float4 each, the eight lane groups stride the row's positions with four positions in flight per group,
// butterfly steps add the groups' partial sums, and lanes 0-3 store the row's 16 outputs.  The four column
// tiles of a row block are adjacent CTAs, so that the col/val stream they share is read from DRAM once.
//
// The result does not depend on where the window lies, only the traffic does: on a matrix without band
// structure the staging is wasted.  The TMA wait is bounded; when it runs out the kernel raises the
// context's status word and returns.
#include <cuda.h>

#include <atomic>

#include "swb_index.h"
#include "swb_kernels.h"

namespace swb {
namespace {

constexpr unsigned FULL = 0xffffffffu;
constexpr int STAGED_ROWS = 1024;   // matrix rows per CTA
constexpr int STAGED_HALO = 1024;   // rows of B staged on either side of them
constexpr int STAGED_WINDOW = STAGED_ROWS + 2 * STAGED_HALO;
constexpr int STAGED_TILE = 16;     // right-hand-side columns per CTA
constexpr int STAGED_BOX_ROWS = 256;
constexpr int STAGED_THREADS = 1024;
constexpr size_t STAGED_SMEM = (size_t)STAGED_WINDOW * STAGED_TILE * 4 + 128;
constexpr uint32_t STAGED_WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__global__ void __launch_bounds__(STAGED_THREADS, 1) spmm_row_block_staged_kernel(
    const __grid_constant__ CUtensorMap map_B, int64_t rows, int64_t N, int64_t tiles,
    const int32_t *__restrict__ row_ptr, const int32_t *__restrict__ col, const float *__restrict__ val,
    const float *__restrict__ B, float *__restrict__ C, bool accumulate, int *status) {
  extern __shared__ __align__(128) unsigned char staged_smem[];
  __shared__ __align__(8) uint64_t bar;
  float4 *win = reinterpret_cast<float4 *>((reinterpret_cast<uintptr_t>(staged_smem) + 127) & ~(uintptr_t)127);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t rb = blockIdx.x / tiles;
  const int j0 = (int)(blockIdx.x % tiles) * STAGED_TILE;
  const int64_t r0 = rb * STAGED_ROWS;
  const int64_t r1 = r0 + STAGED_ROWS < rows ? r0 + STAGED_ROWS : rows;
  const int w0 = (int)r0 - STAGED_HALO;  // first row of B in the window (may be negative: zero filled)

  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&bar)),
                 "r"((uint32_t)(STAGED_WINDOW * STAGED_TILE * 4))
                 : "memory");
#pragma unroll 1
    for (int k = 0; k < STAGED_WINDOW / STAGED_BOX_ROWS; ++k)
      asm volatile(
          "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
              smem_u32(win) + (uint32_t)k * STAGED_BOX_ROWS * STAGED_TILE * 4),
          "l"(&map_B), "r"(j0), "r"(w0 + k * STAGED_BOX_ROWS), "r"(smem_u32(&bar))
          : "memory");
  }
  __syncthreads();  // the barrier is initialised before anyone polls it
  bool ok = false;
  for (uint32_t i = 0; i < STAGED_WAIT_LIMIT && !ok; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(&bar)), "r"(0u)
        : "memory");
    ok = done != 0;
  }
  if (!__syncthreads_and(ok)) {  // bounded wait ran out: the window is not valid
    if (tid == 0) atomicExch(status, 5);
    // copies of this CTA may still be in flight: a bounded time (1 ms) for them to land before the shared
    // memory goes back to the SM
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    return;
  }

  const int q = lane & 3, g = lane >> 2;  // float4 of the tile, lane group
  const float *Bq = B + j0 + 4 * q;
  auto piece = [&](int c) -> float4 {  // the tile's columns 4q .. 4q+3 of row c of B
    const unsigned w = (unsigned)(c - w0);
    if (w < (unsigned)STAGED_WINDOW) return win[w * (STAGED_TILE / 4) + q];
    return __ldg(reinterpret_cast<const float4 *>(Bq + (int64_t)c * N));
  };
  for (int64_t row = r0 + warp; row < r1; row += STAGED_THREADS / 32) {
    const int start = __ldg(row_ptr + row), end = __ldg(row_ptr + row + 1);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    auto fma4 = [&](float v, const float4 &b) {
      acc.x = add(acc.x, mul(v, b.x)); acc.y = add(acc.y, mul(v, b.y));
      acc.z = add(acc.z, mul(v, b.z)); acc.w = add(acc.w, mul(v, b.w));
    };
    int p = start + g;
    for (; p + 24 < end; p += 32) {
      const int c0 = __ldg(col + p), c1 = __ldg(col + p + 8), c2 = __ldg(col + p + 16), c3 = __ldg(col + p + 24);
      const float v0 = __ldg(val + p), v1 = __ldg(val + p + 8), v2 = __ldg(val + p + 16), v3 = __ldg(val + p + 24);
      const float4 b0 = piece(c0), b1 = piece(c1), b2 = piece(c2), b3 = piece(c3);
      fma4(v0, b0); fma4(v1, b1); fma4(v2, b2); fma4(v3, b3);
    }
    for (; p < end; p += 8) fma4(__ldg(val + p), piece(__ldg(col + p)));
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      acc.x = add(acc.x, __shfl_xor_sync(FULL, acc.x, off));
      acc.y = add(acc.y, __shfl_xor_sync(FULL, acc.y, off));
      acc.z = add(acc.z, __shfl_xor_sync(FULL, acc.z, off));
      acc.w = add(acc.w, __shfl_xor_sync(FULL, acc.w, off));
    }
    if (g == 0) {
      float4 *out = reinterpret_cast<float4 *>(C + row * N + j0) + q;
      if (accumulate) {
        const float4 old = *out;
        acc.x = add(old.x, acc.x); acc.y = add(old.y, acc.y); acc.z = add(old.z, acc.z); acc.w = add(old.w, acc.w);
      }
      *out = acc;
    }
  }
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static std::atomic<EncodeTiledFn> cached{nullptr};
  EncodeTiledFn fn = cached.load(std::memory_order_acquire);
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult qr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qr) == cudaSuccess &&
        qr == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
      cached.store(fn, std::memory_order_release);
    }
  }
  return fn;
}

}  // namespace

bool spmm_staged_supported(const CsrSpmmArgs &a) {
  // TMA: 16-byte aligned base and row pitch, 32-bit box coordinates; whole tiles of 16 columns
  return a.n_rhs >= STAGED_TILE && a.n_rhs % STAGED_TILE == 0 && a.rows > 0 && a.cols > 0 && a.cols < 2147483647LL - 4096 &&
         a.rows < 2147483647LL - 4096 && (reinterpret_cast<uintptr_t>(a.B) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(a.C) & 15u) == 0;
}

cudaError_t launch_spmm_row_block_staged(const CsrSpmmArgs &a, int *status_flag, cudaStream_t s, int64_t *launches) {
  static std::atomic<bool> configured[64];
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(spmm_row_block_staged_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)STAGED_SMEM);
    if (e != cudaSuccess) return e;
    if (device >= 0 && device < 64) configured[device].store(true, std::memory_order_release);
  }
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return cudaErrorNotSupported;
  CUtensorMap map_B;
  cuuint64_t dims[2] = {(cuuint64_t)a.n_rhs, (cuuint64_t)a.cols};
  cuuint64_t strides[1] = {(cuuint64_t)a.n_rhs * 4};
  cuuint32_t box[2] = {STAGED_TILE, STAGED_BOX_ROWS};
  cuuint32_t elem[2] = {1, 1};
  if (encode(&map_B, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(a.B), dims, strides, box, elem,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  const int64_t tiles = a.n_rhs / STAGED_TILE;
  unsigned grid = 0;
  if (!grid_dim(ceil_div(a.rows, STAGED_ROWS) * tiles, &grid)) return cudaErrorInvalidConfiguration;
  spmm_row_block_staged_kernel<<<grid, STAGED_THREADS, STAGED_SMEM, s>>>(map_B, a.rows, a.n_rhs, tiles, a.row_ptr,
                                                                           a.col_idx, a.val, a.B, a.C, a.accumulate,
                                                                           status_flag);
  ++*launches;
  return cudaGetLastError();
}

}  // namespace swb
