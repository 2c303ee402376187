// BSR SpMM for 16x16 bf16 blocks on the Blackwell tensor cores (tcgen05 + TMEM).
//
// Reference arithmetic (ThreadPerOutputBSRSpMMPattern, SparseWaveToGPU.cpp:560-665):
//   C[br*16 + r, j] = sum over blocks bp of block row br, sum over lc:
//                     bv[bp][r][lc] * B[bci[bp]*16 + lc, j]
// with bf16 operands, f32 accumulation and one rounding to bf16 at the store.
//
// Mapping to the MMA.  A 16-row block would waste the M dimension (64 or 128)
// of tcgen05.mma, so the product is formed transposed: for one block row and a
// tile of 128 right-hand-side columns,
//   D[m, r] (+)= sum_k  Bt[m, k] * At[k, r],   m = column in the tile, k = lc,
// one tcgen05.mma of shape M=128, N=16, K=16 per nonzero block, all blocks of
// the block row accumulating into one 128-lane x 16-column f32 tile in TMEM.
//   - MMA operand A = the 16 x 128 slab B[bci*16 .. +16, n0 .. n0+128): row k is
//     contiguous in memory along m, i.e. MN-major.
//   - MMA operand B = the block itself, [r][lc] row-major: K-major.
// Both operands are staged in shared memory in the canonical no-swizzle layouts
// of 8 x 16-byte core matrices by 16-byte cp.async copies (the slab rows are
// gathered by block-column index, so there is no dense tile for a bulk tensor
// copy to fetch), double-buffered in chunks of CHUNK blocks.  One thread issues
// the MMAs; tcgen05.commit signals an mbarrier when a chunk's MMAs have read
// their operands.  The epilogue reads the accumulator with tcgen05.ld (each of
// the four warps its own 32 TMEM lanes), rounds to bf16 and stores C.
//
// Every mbarrier wait is bounded: when it runs out the kernel raises the status
// flag, drains its copies, frees its TMEM columns and returns.
#include <cuda_bf16.h>

#include "swb_index.h"
#include "swb_kernels.h"

namespace swb {
namespace {

constexpr int TILE_N = 128;                  // right-hand-side columns per CTA (MMA M)
constexpr int CHUNK = 8;                     // blocks per pipeline stage
constexpr int STAGES = 2;
constexpr int SLAB_BYTES = 16 * TILE_N * 2;  // 4096: one 16 x 128 bf16 slab
constexpr int BLOCK_BYTES = 16 * 16 * 2;     // 512
constexpr int ITEM_BYTES = SLAB_BYTES + BLOCK_BYTES;
constexpr int STAGE_BYTES = CHUNK * ITEM_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 128;  // + alignment slack
constexpr int TMEM_COLS = 32;                // minimum allocation; 16 are used
constexpr uint32_t WAIT_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Shared-memory matrix descriptor, no swizzle, version 1 (Blackwell):
// bits [0,14) address >> 4, [16,30) leading byte offset >> 4, [32,46) stride
// byte offset >> 4, [46,48) version, [61,64) layout type (0 = no swizzle).
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}

// Instruction descriptor for kind::f16: D f32 (bits 4-5 = 1), A and B bf16
// (bits 7-9 and 10-12 = 1), A MN-major (bit 15), B K-major (bit 16 = 0),
// N >> 3 at bits 17-22, M >> 4 at bits 24-28.
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((16u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

__global__ void __launch_bounds__(128) bsr16_spmm_tcgen05_kernel(
    int64_t n_tiles, int64_t N, const int32_t *__restrict__ brp, const int32_t *__restrict__ bci,
    const __nv_bfloat16 *__restrict__ bv, const __nv_bfloat16 *__restrict__ B, __nv_bfloat16 *__restrict__ C,
    int *status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t mbar[STAGES];
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t br = blockIdx.x / n_tiles;
  const int64_t n0 = (blockIdx.x % n_tiles) * TILE_N;
  const uint32_t stage0 = (smem_u32(smem_raw) + 127u) & ~127u;
  const int start = brp[br], end = brp[br + 1];
  const int nblk = end - start;

  if (nblk == 0) {  // empty block row: C = 0
    const int64_t col = n0 + tid;
    if (col < N)
      for (int r = 0; r < 16; ++r) C[(br * 16 + r) * N + col] = __float2bfloat16_rn(0.0f);
    return;
  }

  if (tid == 0) {
    failed = 0;
    for (int s = 0; s < STAGES; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&mbar[s])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_slot;

  // cp.async copies of chunk c into stage s.  Slab unit u (16 bytes) of a
  // block: ki = u % 8 (k within its group of 8), mg = (u / 8) % 16 (group of 8
  // columns), kg = u / 128; it lands at byte u * 16, which is the canonical
  // layout with 16 B between k rows, 128 B between column groups (stride byte
  // offset) and 2048 B between k groups (leading byte offset).  Block unit g
  // (row r = g / 2, k half kc = g % 2) lands at (kc * 16 + r) * 16: 16 B between
  // rows, 128 B between row groups (SBO), 256 B between k halves (LBO).
  auto issue_loads = [&](int c, int s) {
    const uint32_t sbase = stage0 + (uint32_t)s * STAGE_BYTES;
    const int first = start + c * CHUNK;
    const int count = min(CHUNK, end - first);
    // Block-column indices of the whole chunk first (independent loads), so that
    // the copies below do not wait for one index load per block.
    int bcs[CHUNK];
#pragma unroll
    for (int j = 0; j < CHUNK; ++j) bcs[j] = (j < count) ? __ldg(bci + first + j) : 0;
#pragma unroll
    for (int j = 0; j < CHUNK; ++j) {
      if (j >= count) break;
      const int bp = first + j;
      const int64_t bc = bcs[j];
      const uint32_t item = sbase + (uint32_t)j * ITEM_BYTES;
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int u = tid + 128 * i;
        const int ki = u & 7, mg = (u >> 3) & 15, kg = u >> 7;
        const int64_t col = n0 + mg * 8;
        const bool ok = col < N;
        const __nv_bfloat16 *src = ok ? B + (bc * 16 + kg * 8 + ki) * N + col : B;
        cp_async16(item + (uint32_t)u * 16, src, ok ? 16u : 0u);
      }
      if (tid < 32) {
        const int r = tid >> 1, kc = tid & 1;
        cp_async16(item + SLAB_BYTES + (uint32_t)(kc * 16 + r) * 16, bv + (int64_t)bp * 256 + tid * 8, 16u);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const int nchunks = (nblk + CHUNK - 1) / CHUNK;
  uint32_t uses[STAGES] = {0, 0};  // completed waits per stage -> wait parity
  bool ok = true;

  issue_loads(0, 0);
  for (int c = 0; c < nchunks && ok; ++c) {
    const int s = c & 1;
    if (c + 1 < nchunks) {
      if (c >= 1) {  // stage s^1 still feeds the MMAs of chunk c-1
        ok = mbar_wait(smem_u32(&mbar[s ^ 1]), uses[s ^ 1] & 1u);
        uses[s ^ 1]++;
        ok = __syncthreads_and(ok);  // one decision for the whole CTA
        if (!ok) break;
      }
      issue_loads(c + 1, s ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    // The copies were made through the generic proxy; the MMA reads through the async proxy.
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t sbase = stage0 + (uint32_t)s * STAGE_BYTES;
      const int count = min(CHUNK, nblk - c * CHUNK);
      for (int j = 0; j < count; ++j) {
        const uint32_t item = sbase + (uint32_t)j * ITEM_BYTES;
        const uint64_t adesc = make_desc(item, 2048u, 128u);
        const uint64_t bdesc = make_desc(item + SLAB_BYTES, 256u, 128u);
        const uint32_t accumulate = (c > 0 || j > 0) ? 1u : 0u;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem), "l"(adesc), "l"(bdesc), "r"(IDESC), "r"(accumulate)
            : "memory");
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                       smem_u32(&mbar[s]))
                   : "memory");
    }
  }
  if (ok) {  // the last chunk's MMAs
    const int s = (nchunks - 1) & 1;
    ok = mbar_wait(smem_u32(&mbar[s]), uses[s] & 1u);
  }
  ok = __syncthreads_and(ok);
  if (!ok) {
    failed = 1;
    atomicExch(status, 1);
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  __syncthreads();

  if (!failed) {
    uint32_t v[16];
    const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
        "%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    const int64_t col = n0 + warp * 32 + lane;  // TMEM lane m = column n0 + m of C
    if (col < N) {
#pragma unroll
      for (int r = 0; r < 16; ++r) C[(br * 16 + r) * N + col] = __float2bfloat16_rn(__uint_as_float(v[r]));
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

}  // namespace

bool bsr16_tcgen05_supported(const BsrSpmmArgs &a) {
  return a.block_size == 16 && a.n_rhs % 8 == 0 && (reinterpret_cast<uintptr_t>(a.B) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(a.block_values) & 15u) == 0;
}

cudaError_t launch_bsr16_spmm_tcgen05(const BsrSpmmArgs &a, int *status_flag, const DeviceInfo &dev,
                                      cudaStream_t s, int64_t *launches) {
  (void)dev;
  static bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device]) {
    cudaError_t e = cudaFuncSetAttribute(bsr16_spmm_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (device >= 0 && device < 64) configured[device] = true;
  }
  const int64_t brows = a.rows / 16;
  if (brows == 0) return cudaSuccess;
  const int64_t n_tiles = ceil_div(a.n_rhs, TILE_N);
  const int64_t grid = brows * n_tiles;
  if (grid > 2147483647LL) return cudaErrorInvalidConfiguration;
  bsr16_spmm_tcgen05_kernel<<<(unsigned)grid, 128, SMEM_BYTES, s>>>(
      n_tiles, a.n_rhs, a.block_row_ptr, a.block_col_idx, static_cast<const __nv_bfloat16 *>(a.block_values),
      static_cast<const __nv_bfloat16 *>(a.B), static_cast<__nv_bfloat16 *>(a.C), status_flag);
  ++*launches;
  return cudaGetLastError();
}

}  // namespace swb
