// BSR SpMM for 16x16 bf16 blocks on the Blackwell tensor cores:
// TMA (cp.async.bulk.tensor) -> shared memory -> tcgen05.mma -> TMEM -> tcgen05.ld.
//
// Reference arithmetic (ThreadPerOutputBSRSpMMPattern, SparseWaveToGPU.cpp:560-665):
//   C[br*16 + r, j] = sum over blocks bp of block row br, sum over lc:
//                     bv[bp][r][lc] * B[bci[bp]*16 + lc, j]
// with bf16 operands, f32 accumulation and one rounding to bf16 at the store.
//
// Mapping to the MMA.  A 16-row block would waste the M dimension (64 or 128)
// of tcgen05.mma, so the product is formed transposed: for one block row and
// 128 right-hand-side columns,
//   D[m, r] (+)= sum_k  Bt[m, k] * At[k, r],   m = column, k = lc,
// one tcgen05.mma of shape M=128, N=16, K=16 per nonzero block, all blocks of
// the block row accumulating into one 128-lane x 16-column f32 tile in TMEM.
// A CTA owns one block row and a tile of 256 right-hand-side columns, i.e. two
// such accumulators side by side in TMEM (columns 0-15 and 16-31), so that each
// block and each block-column index is fetched once per 256 columns.
//   - MMA operand A = a 16 x 128 slab B[bci*16 .. +16, n .. n+128).  Row k is
//     contiguous along m: MN-major.  Two TMA boxes of 64 columns x 16 rows with
//     the 128-byte swizzle land it as the canonical MN-major SWIZZLE_128B layout
//     (128-byte rows, 1024 bytes between groups of 8 k rows = stride byte
//     offset, 2048 bytes between the two 64-column halves = leading byte
//     offset).  Columns past N are zero-filled by the TMA unit; a tile whose
//     second 128 columns lie wholly past N skips them.
//   - MMA operand B = the block itself, [r][lc] row-major: K-major.  One TMA box
//     of 16 x 16 with the 32-byte swizzle over the block values viewed as a
//     (nnzb*16) x 16 matrix lands it as the canonical K-major SWIZZLE_32B layout
//     (32-byte rows, 256 bytes between groups of 8 rows = stride byte offset).
//     Both accumulators' MMAs read the same copy.
// The slab rows are gathered by block-column index, four boxes per block.
//
// Pipeline.  Lane 0 of warp 4 is the producer: per chunk of blocks it waits for
// the stage's `empty` mbarrier, loads the chunk's block-column indices, arms the
// stage's `full` mbarrier with the byte count and issues the TMA copies.  Lane 0
// of warp 5 issues the MMAs: it waits for `full`, issues the chunk's MMAs and
// lets tcgen05.commit arrive on `empty` when they have read their operands, so
// index loads and copies of later chunks never wait behind a commit.  After the
// last chunk the commit arrives on `done`; warps 0-3 then read both accumulators
// with tcgen05.ld (each warp its own 32 TMEM lanes), round to bf16 and store C.
//
// Every mbarrier wait is bounded: when one runs out the kernel raises the
// status word, frees its TMEM columns and returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include <atomic>
#include <cstdio>

#include "swb_index.h"
#include "swb_kernels.h"

namespace swb {
namespace {

constexpr int TILE_N = 256;                  // right-hand-side columns per CTA (two MMA M = 128 halves)
constexpr int HALF_N = 128;
// One block per stage, three stages (28 KiB of shared memory, seven CTAs per SM): on the 5 %-dense
// 1024 x 1024 block grid with 512 columns, 69.7 us; (2,2) 75.7, (2,3) 80.0, (1,2) 78.7, (1,4) 84.0, (4,2) 86.0.
// What counts is the number of CTAs in flight per SM, each being one serial chain of copies.
#ifndef SWB_BSR_CHUNK
#define SWB_BSR_CHUNK 1
#endif
#ifndef SWB_BSR_STAGES
#define SWB_BSR_STAGES 3
#endif
constexpr int CHUNK = SWB_BSR_CHUNK;         // blocks per pipeline stage
constexpr int STAGES = SWB_BSR_STAGES;
constexpr int BOX_BYTES = 16 * 64 * 2;       // 2048: 64 columns x 16 rows
constexpr int HALF_SLAB = 2 * BOX_BYTES;     // 4096: one 16 x 128 bf16 slab (one accumulator's operand)
constexpr int SLAB_BYTES = 2 * HALF_SLAB;    // 8192: 16 x 256
constexpr int BLOCK_BYTES = 16 * 16 * 2;     // 512
constexpr int STAGE_SLABS = CHUNK * SLAB_BYTES;
// slabs first (1024-aligned), then blocks, padded so that the next stage's slabs are 1024-aligned again
constexpr int STAGE_BYTES = (STAGE_SLABS + CHUNK * BLOCK_BYTES + 1023) / 1024 * 1024;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024;         // + alignment slack
constexpr int TMEM_COLS = 32;                // two accumulators of 16 columns
constexpr uint32_t WAIT_LIMIT = 1u << 22;
constexpr int PRODUCER_THREAD = 128;         // lane 0 of warp 4 issues the TMA copies
constexpr int MMA_THREAD = 160;              // lane 0 of warp 5 issues the MMAs
constexpr int THREADS = 192;
static_assert(STAGE_BYTES % 1024 == 0, "stages must keep the 1024-byte alignment of the swizzled slabs");

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Shared-memory matrix descriptor, version 1 (Blackwell): bits [0,14) address
// >> 4, [16,30) leading byte offset >> 4, [32,46) stride byte offset >> 4,
// [46,48) version, [61,64) layout type (2 = 128-byte swizzle, 6 = 32-byte).
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                              uint32_t layout) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
}

// Instruction descriptor for kind::f16: D f32 (bits 4-5 = 1), A and B bf16
// (bits 7-9 and 10-12 = 1), A MN-major (bit 15), B K-major (bit 16 = 0),
// N >> 3 at bits 17-22, M >> 4 at bits 24-28.
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | ((16u >> 3) << 17) | ((128u >> 4) << 24);

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

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// PER_CTA_STATUS: raise status[blockIdx.x] instead of status[0] when a wait gives up.
template <bool PER_CTA_STATUS>
__global__ void __launch_bounds__(THREADS) bsr16_spmm_tcgen05_kernel(
    const __grid_constant__ CUtensorMap map_B, const __grid_constant__ CUtensorMap map_A, int64_t n_tiles,
    int64_t N, const int32_t *__restrict__ brp, const int32_t *__restrict__ bci, __nv_bfloat16 *__restrict__ C,
    int *status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[STAGES];
  __shared__ __align__(8) uint64_t bar_empty[STAGES];
  __shared__ __align__(8) uint64_t bar_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int failed;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t br = blockIdx.x / n_tiles;
  const int n0 = (int)((blockIdx.x % n_tiles) * TILE_N);
  const int halves = ((int64_t)n0 + HALF_N < N) ? 2 : 1;  // the second 128 columns may lie wholly past N
  const uint32_t stage0 = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int start = brp[br], end = brp[br + 1];
  const int nblk = end - start;

  if (nblk == 0) {  // empty block row: C = 0
    for (int64_t col = (int64_t)n0 + tid; col < N && col < (int64_t)n0 + TILE_N; col += THREADS)
      for (int r = 0; r < 16; ++r) C[(br * 16 + r) * N + col] = __float2bfloat16_rn(0.0f);
    return;
  }

  if (tid == 0) {
    failed = 0;
    for (int s = 0; s < STAGES; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar_full[s])) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar_empty[s])) : "memory");
    }
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar_done)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_B) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_A) : "memory");
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
  const int nchunks = (nblk + CHUNK - 1) / CHUNK;

  if (tid == PRODUCER_THREAD) {
    for (int i = 0; i < nchunks; ++i) {
      const int s = i % STAGES;
      if (i >= STAGES && !mbar_wait(smem_u32(&bar_empty[s]), ((i / STAGES) - 1) & 1u)) {
        failed = 1;  // the MMAs of chunk i - STAGES never released this stage
        atomicExch(status + (PER_CTA_STATUS ? blockIdx.x : 0), 1);
        break;
      }
      const int first = start + i * CHUNK;
      const int count = min(CHUNK, end - first);
      int bcs[CHUNK];
#pragma unroll
      for (int j = 0; j < CHUNK; ++j) bcs[j] = (j < count) ? __ldg(bci + first + j) : 0;
      const uint32_t full = smem_u32(&bar_full[s]);
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full),
                   "r"((uint32_t)count * (uint32_t)(halves * HALF_SLAB + BLOCK_BYTES))
                   : "memory");
      const uint32_t sbase = stage0 + (uint32_t)s * STAGE_BYTES;
#pragma unroll
      for (int j = 0; j < CHUNK; ++j) {
        if (j >= count) break;
        const uint32_t slab = sbase + (uint32_t)j * SLAB_BYTES;
        tma_load_2d(slab, &map_B, n0, bcs[j] * 16, full);
        tma_load_2d(slab + BOX_BYTES, &map_B, n0 + 64, bcs[j] * 16, full);
        if (halves == 2) {
          tma_load_2d(slab + 2 * BOX_BYTES, &map_B, n0 + 128, bcs[j] * 16, full);
          tma_load_2d(slab + 3 * BOX_BYTES, &map_B, n0 + 192, bcs[j] * 16, full);
        }
        tma_load_2d(sbase + STAGE_SLABS + (uint32_t)j * BLOCK_BYTES, &map_A, 0, (first + j) * 16, full);
      }
    }
  } else if (tid == MMA_THREAD) {
    bool ok = true;
    for (int c = 0; c < nchunks; ++c) {
      const int s = c % STAGES;
      ok = mbar_wait(smem_u32(&bar_full[s]), (c / STAGES) & 1u);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t sbase = stage0 + (uint32_t)s * STAGE_BYTES;
      const int count = min(CHUNK, nblk - c * CHUNK);
      for (int j = 0; j < count; ++j) {
        const uint64_t bdesc = make_desc(sbase + STAGE_SLABS + (uint32_t)j * BLOCK_BYTES, 16u, 256u, 6u);
        const uint32_t accumulate = (c > 0 || j > 0) ? 1u : 0u;
        for (int h = 0; h < halves; ++h) {
          const uint64_t adesc = make_desc(sbase + (uint32_t)j * SLAB_BYTES + (uint32_t)h * HALF_SLAB, 2048u, 1024u, 2u);
          asm volatile(
              "{\n\t.reg .pred p;\n\t"
              "setp.ne.b32 p, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem + (uint32_t)h * 16u),
              "l"(adesc), "l"(bdesc), "r"(IDESC), "r"(accumulate)
              : "memory");
        }
      }
      const uint32_t arrive_on = (c == nchunks - 1) ? smem_u32(&bar_done) : smem_u32(&bar_empty[s]);
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(arrive_on)
                   : "memory");
    }
    if (!ok) {
      failed = 1;
      atomicExch(status + (PER_CTA_STATUS ? blockIdx.x : 0), 1);
      // Release the waiters below.
      asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&bar_done)) : "memory");
    }
  }
  // The four epilogue warps wait for the last MMA (or for the failure release).
  bool done_ok = warp < 4 ? mbar_wait(smem_u32(&bar_done), 0u) : true;
  done_ok = __syncthreads_and(done_ok);
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (!done_ok && tid == 0) atomicExch(status + (PER_CTA_STATUS ? blockIdx.x : 0), 1);
  if (!done_ok || failed) {
    // A wait gave up with copies or MMAs of this CTA possibly still in flight: give them a bounded time (1 ms)
    // to land before the shared memory and the TMEM columns go back to the SM.
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }

  if (done_ok && !failed && warp < 4) {
    // TMEM lane m of accumulator h = column n0 + 128 h + m of C; this warp reads lanes 32 warp .. +32
    for (int h = 0; h < halves; ++h) {
      uint32_t v[16];
      const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)h * 16u;
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
          "%15}, [%16];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
            "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
          : "r"(taddr)
          : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const int64_t col = (int64_t)n0 + h * HALF_N + warp * 32 + lane;
      if (col < N) {
#pragma unroll
        for (int r = 0; r < 16; ++r) C[(br * 16 + r) * N + col] = __float2bfloat16_rn(__uint_as_float(v[r]));
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements per row, `outer` rows.
bool make_map_2d(CUtensorMap *map, const void *base, uint64_t inner, uint64_t outer, uint32_t box_inner,
                 uint32_t box_outer, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {inner * 2};  // bytes between rows
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool bsr16_tcgen05_supported(const BsrSpmmArgs &a) {
  // TMA needs 16-byte aligned bases and row pitches.
  // ... and 32-bit box coordinates: block rows of the value matrix (nnzb * 16) and B's extents.
  if (a.nnzb > 2147483647LL / 16 || a.cols > 2147483647LL || a.n_rhs > 2147483647LL - 256) return false;
  return a.block_size == 16 && a.n_rhs % 8 == 0 && a.nnzb > 0 && a.cols > 0 &&
         (reinterpret_cast<uintptr_t>(a.B) & 15u) == 0 && (reinterpret_cast<uintptr_t>(a.block_values) & 15u) == 0;
}

cudaError_t launch_bsr16_spmm_tcgen05(const BsrSpmmArgs &a, int *status_flag, const DeviceInfo &dev,
                                      cudaStream_t s, int64_t *launches) {
  (void)dev;
  // Once per device; racing host threads at worst repeat the (idempotent) attribute call.
  static std::atomic<bool> configured[64];
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device].load(std::memory_order_acquire)) {
    cudaError_t e = cudaFuncSetAttribute(bsr16_spmm_tcgen05_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_BYTES);
    if (e != cudaSuccess) return e;
    if (device >= 0 && device < 64) configured[device].store(true, std::memory_order_release);
  }
  const int64_t brows = a.rows / 16;
  if (brows == 0) return cudaSuccess;
  const int64_t n_tiles = ceil_div(a.n_rhs, TILE_N);
  const int64_t grid = brows * n_tiles;
  if (grid > 2147483647LL) return cudaErrorInvalidConfiguration;
  CUtensorMap map_B, map_A;
  // B: cols x N bf16, boxes of 64 columns x 16 rows, 128-byte swizzle.
  if (!make_map_2d(&map_B, a.B, (uint64_t)a.n_rhs, (uint64_t)a.cols, 64, 16, CU_TENSOR_MAP_SWIZZLE_128B))
    return cudaErrorInvalidValue;
  // Block values as (nnzb*16) x 16 bf16, one 16 x 16 box per block, 32-byte swizzle.
  if (!make_map_2d(&map_A, a.block_values, 16, (uint64_t)a.nnzb * 16, 16, 16, CU_TENSOR_MAP_SWIZZLE_32B))
    return cudaErrorInvalidValue;
  bsr16_spmm_tcgen05_kernel<false><<<(unsigned)grid, THREADS, SMEM_BYTES, s>>>(
      map_B, map_A, n_tiles, a.n_rhs, a.block_row_ptr, a.block_col_idx, static_cast<__nv_bfloat16 *>(a.C),
      status_flag);
  ++*launches;
  return cudaGetLastError();
}

}  // namespace swb

// ---------------------------------------------------------------------------
// swb_bsr16_spmm_bf16_static: the tensor-core BSR SpMM for callers that must
// not allocate device memory.
//
// The regular entry point needs a context, and creating a context calls
// cudaMalloc for the status word its kernels raise when a bounded barrier wait
// gives up.  Some callers cannot do that: code running under a memory budget
// that was fixed at start-up (every byte handed out by the application's own
// pool), plug-ins that are loaded into a process which forbids driver
// allocations after initialisation, and code that runs while the allocator's
// lock may be held.  For them the status words live in the fixed array below,
// which is part of the library image: every GPU that loads the library holds
// its 128 KiB until the process exits, whether or not this entry point is used.
//
// One status word per CTA (block row x tile of 256 columns), hence the limit
// of SWB_STATIC_MAX_CTAS CTAs per call.  All calls share the array and a call
// begins by clearing the words it will use, so the array holds the outcome of
// the most recent call only, and two calls that overlap on the GPU (different
// streams) race on it.
// ---------------------------------------------------------------------------
namespace swb {
namespace {

constexpr int SWB_STATIC_MAX_CTAS = 32768;  // 32768 status words = 128 KiB

static __device__ __align__(256) int swb_static_status_words[SWB_STATIC_MAX_CTAS];

// In host code `swb_static_status_words` is only a handle for the symbol, not a
// device address; the address a kernel can use comes from
// cudaGetSymbolAddress, asked once per device with that device current.
// Host-side record per device: the array's device address and the number of words the most recent call
// on that device used.  Atomics, so that host threads may call concurrently (two threads that both find
// the address missing ask for it twice and store the same value).
struct StaticStatusSlot {
  std::atomic<int *> address{nullptr};
  std::atomic<int64_t> last_grid{0};
};
StaticStatusSlot g_static_slots[64];

int *static_status_address(cudaError_t *err, StaticStatusSlot **slot_out = nullptr) {
  int device = 0;
  *err = cudaGetDevice(&device);
  if (*err != cudaSuccess) return nullptr;
  if (device < 0 || device >= 64) {
    *err = cudaErrorInvalidDevice;
    return nullptr;
  }
  StaticStatusSlot &slot = g_static_slots[device];
  if (slot_out) *slot_out = &slot;
  int *address = slot.address.load(std::memory_order_acquire);
  if (!address) {
    void *p = nullptr;
    *err = cudaGetSymbolAddress(&p, swb_static_status_words);
    if (*err != cudaSuccess) return nullptr;
    address = static_cast<int *>(p);
    slot.address.store(address, std::memory_order_release);
  }
  return address;
}

// Counts the non-zero words among the first `grid` through pageable stack memory: no pinned or device
// allocation.  The stream must be idle.
cudaError_t count_status_words(const int *status, int64_t grid, int32_t *count_out) {
  int32_t count = 0;
  int piece[1024];
  for (int64_t off = 0; off < grid; off += 1024) {
    const int64_t n = grid - off < 1024 ? grid - off : 1024;
    cudaError_t e = cudaMemcpy(piece, status + off, (size_t)n * sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return e;
    for (int64_t i = 0; i < n; ++i) count += piece[i] != 0;
  }
  *count_out = count;
  return cudaSuccess;
}

int static_fail(int status, const char *fmt, long long a = 0, long long b = 0) {
  char buf[512];
  snprintf(buf, sizeof buf, fmt, a, b);
  set_thread_error(buf);
  return status;
}

}  // namespace
}  // namespace swb

extern "C" __attribute__((visibility("default"))) int swb_bsr16_spmm_bf16_static(
    int64_t rows, int64_t cols, int64_t nnzb, int64_t n_rhs, const int32_t *block_row_ptr,
    const int32_t *block_col_idx, const uint16_t *block_values, const uint16_t *B, uint16_t *C, void *stream,
    int32_t *gave_up_ctas) {
  using namespace swb;
  // Status codes are those of swb_status in sparsewave_b200.h.
  constexpr int kInvalidShape = -2, kInvalidArgument = -3, kCuda = -4, kUnsupported = -5, kCapacity = -7;
  if (rows < 0 || cols < 0 || nnzb < 0)
    return static_fail(kInvalidArgument, "bsr_spmm: rows, cols and nnzb must be non-negative");
  if (rows % 16 != 0)
    return static_fail(kInvalidShape, "output rows must be divisible by block size, but got %lld and 16", rows);
  if (cols % 16 != 0)
    return static_fail(kInvalidShape, "right-hand-side rows must be divisible by block size, but got %lld and 16", cols);
  if (n_rhs < 1) return static_fail(kInvalidShape, "bsr_spmm: right-hand side must have at least one column, but got %lld", n_rhs);
  if (rows > 2147483647LL || cols > 2147483647LL || nnzb > 2147483647LL / 16)
    return static_fail(kInvalidShape, "BSR dimensions and NNZ blocks must fit in i32");
  if (!block_row_ptr || (nnzb > 0 && (!block_col_idx || !block_values)) || (cols > 0 && !B) || (rows > 0 && !C))
    return static_fail(kInvalidArgument, "bsr_spmm: NULL operand pointer");
  BsrSpmmArgs a{rows, cols, nnzb, 16, n_rhs, block_row_ptr, block_col_idx, block_values, B, C};
  if (!bsr16_tcgen05_supported(a))
    return static_fail(kUnsupported,
                       "the static-scratch BSR entry point needs at least one block, a column count that is a "
                       "multiple of 8 and 16-byte aligned block values and right-hand side");
  const int64_t n_tiles = ceil_div(n_rhs, TILE_N);
  const int64_t grid = (rows / 16) * n_tiles;
  if (grid > SWB_STATIC_MAX_CTAS)
    return static_fail(kCapacity,
                       "the static-scratch BSR entry point handles at most %lld (block row, 256-column tile) pairs "
                       "per call, but this call needs %lld",
                       (long long)SWB_STATIC_MAX_CTAS, (long long)grid);
  if (grid == 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaSuccess;
  StaticStatusSlot *slot = nullptr;
  int *status = static_status_address(&e, &slot);
  if (!status) return static_fail(kCuda, cudaGetErrorString(e));
  e = cudaFuncSetAttribute(bsr16_spmm_tcgen05_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return static_fail(kCuda, cudaGetErrorString(e));
  CUtensorMap map_B, map_A;
  if (!make_map_2d(&map_B, B, (uint64_t)n_rhs, (uint64_t)cols, 64, 16, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_map_2d(&map_A, block_values, 16, (uint64_t)nnzb * 16, 16, 16, CU_TENSOR_MAP_SWIZZLE_32B))
    return static_fail(kCuda, "could not encode the TMA tensor maps");
  // The words keep the previous call's outcome: clear the ones this call uses.
  e = cudaMemsetAsync(status, 0, (size_t)grid * sizeof(int), s);
  if (e != cudaSuccess) return static_fail(kCuda, cudaGetErrorString(e));
  bsr16_spmm_tcgen05_kernel<true><<<(unsigned)grid, THREADS, SMEM_BYTES, s>>>(
      map_B, map_A, n_tiles, n_rhs, block_row_ptr, block_col_idx, reinterpret_cast<__nv_bfloat16 *>(C), status);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_fail(kCuda, cudaGetErrorString(e));
  slot->last_grid.store(grid, std::memory_order_release);
  if (gave_up_ctas) {
    e = cudaStreamSynchronize(s);
    if (e == cudaSuccess) e = count_status_words(status, grid, gave_up_ctas);
    if (e != cudaSuccess) return static_fail(kCuda, cudaGetErrorString(e));
  }
  return 0;
}

// Outcome of the most recent swb_bsr16_spmm_bf16_static call on the current device, for callers that
// passed gave_up_ctas == NULL: waits for `stream` and counts the CTAs of that call whose bounded wait
// gave up.  Allocates nothing.
extern "C" __attribute__((visibility("default"))) int swb_bsr16_static_status(void *stream, int32_t *gave_up_ctas) {
  using namespace swb;
  constexpr int kInvalidArgument = -3, kCuda = -4;
  if (!gave_up_ctas) return static_fail(kInvalidArgument, "bsr16 static status: gave_up_ctas is NULL");
  *gave_up_ctas = 0;
  cudaError_t e = cudaSuccess;
  StaticStatusSlot *slot = nullptr;
  int *status = static_status_address(&e, &slot);
  if (!status) return static_fail(kCuda, cudaGetErrorString(e));
  e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) e = count_status_words(status, slot->last_grid.load(std::memory_order_acquire), gave_up_ctas);
  if (e != cudaSuccess) return static_fail(kCuda, cudaGetErrorString(e));
  return 0;
}
