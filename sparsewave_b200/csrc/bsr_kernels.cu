// BSR SpMM, thread-per-output mapping (ThreadPerOutputBSRSpMMPattern,
// SparseWaveToGPU.cpp:560-665): element = blockIdx * blockDim + threadIdx;
// row = element / N, column = element % N, block row = row / bs, local row =
// row % bs; for every block of the block row, in storage order, and every
// local column in ascending order: sum += value * B[block_col*bs + lc, column].
// f32 blocks (the element type of the reference's runtime tests) and bf16
// blocks with f32 accumulation and one final rounding to bf16.
#include <cuda_bf16.h>

#include "swb_index.h"
#include "swb_kernels.h"

namespace swb {
namespace {

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void store(float *p, float v) { *p = v; }
__device__ __forceinline__ void store(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

// WARP_ROW: N and the block size of the launch are multiples of 32, so the 32 outputs of a warp lie in one
// matrix row and share the block row's values: lane l reads a[lc0 + l] once and the warp passes the values
// around by shuffles instead of 32 lanes reading each a[lc] (one L1 request per lc saved).  Every thread
// still adds its products in the reference's order: the result is the same bit for bit.  Used from block
// size 32 (512 x 512 blocks of 32 x 32 at 5 %, N = 512: 2.81 -> 2.59 ms; with 8 x 8 blocks it is 3 % slower).
template <typename T, bool WARP_ROW>
__global__ void bsr_spmm_thread_per_output_kernel(int64_t rows, int64_t N, int64_t bs,
                                                  const int32_t *__restrict__ brp,
                                                  const int32_t *__restrict__ bci,
                                                  const T *__restrict__ bv, const T *__restrict__ B,
                                                  T *__restrict__ C) {
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= rows * N) return;
  const int64_t row = e / N, j = e % N;
  const int64_t brow = row / bs, lrow = row % bs;
  const int start = brp[brow], end = brp[brow + 1];
  float sum = 0.0f;
  for (int bp = start; bp < end; ++bp) {
    const int64_t bc = bci[bp];
    const T *a = bv + ((int64_t)bp * bs + lrow) * bs;
    const T *b = B + (bc * bs) * N + j;
    if (WARP_ROW) {
      const int lane = threadIdx.x & 31;
      for (int64_t lc0 = 0; lc0 < bs; lc0 += 32) {  // uniform in the warp: same row, same block
        const int n = bs - lc0 < 32 ? (int)(bs - lc0) : 32;
        const float mine = lane < n ? to_f32(a[lc0 + lane]) : 0.0f;
        for (int k = 0; k < n; ++k)
          sum = add(sum, mul(__shfl_sync(0xffffffffu, mine, k), to_f32(b[(lc0 + k) * N])));
      }
    } else {
      for (int64_t lc = 0; lc < bs; ++lc) sum = add(sum, mul(to_f32(a[lc]), to_f32(b[lc * N])));
    }
  }
  store(C + e, sum);
}

}  // namespace

cudaError_t launch_bsr_spmm_thread_per_output_f32(const BsrSpmmArgs &a, int block, cudaStream_t s,
                                                  int64_t *launches) {
  unsigned grid = 0;  // refused, not truncated, beyond the CUDA grid limit
  if (!grid_dim(ceil_div(a.rows * a.n_rhs, block), &grid)) return cudaErrorInvalidConfiguration;
  if (a.n_rhs % 32 == 0 && block % 32 == 0 && a.block_size >= 32)
    bsr_spmm_thread_per_output_kernel<float, true><<<grid, block, 0, s>>>(
        a.rows, a.n_rhs, a.block_size, a.block_row_ptr, a.block_col_idx,
        static_cast<const float *>(a.block_values), static_cast<const float *>(a.B),
        static_cast<float *>(a.C));
  else
    bsr_spmm_thread_per_output_kernel<float, false><<<grid, block, 0, s>>>(
        a.rows, a.n_rhs, a.block_size, a.block_row_ptr, a.block_col_idx,
        static_cast<const float *>(a.block_values), static_cast<const float *>(a.B),
        static_cast<float *>(a.C));
  ++*launches;
  return cudaGetLastError();
}

cudaError_t launch_bsr_spmm_thread_per_output_bf16(const BsrSpmmArgs &a, int block, cudaStream_t s,
                                                   int64_t *launches) {
  unsigned grid = 0;  // refused, not truncated, beyond the CUDA grid limit
  if (!grid_dim(ceil_div(a.rows * a.n_rhs, block), &grid)) return cudaErrorInvalidConfiguration;
  if (a.n_rhs % 32 == 0 && block % 32 == 0 && a.block_size >= 32)
    bsr_spmm_thread_per_output_kernel<__nv_bfloat16, true><<<grid, block, 0, s>>>(
        a.rows, a.n_rhs, a.block_size, a.block_row_ptr, a.block_col_idx,
        static_cast<const __nv_bfloat16 *>(a.block_values), static_cast<const __nv_bfloat16 *>(a.B),
        static_cast<__nv_bfloat16 *>(a.C));
  else
    bsr_spmm_thread_per_output_kernel<__nv_bfloat16, false><<<grid, block, 0, s>>>(
        a.rows, a.n_rhs, a.block_size, a.block_row_ptr, a.block_col_idx,
        static_cast<const __nv_bfloat16 *>(a.block_values), static_cast<const __nv_bfloat16 *>(a.B),
        static_cast<__nv_bfloat16 *>(a.C));
  ++*launches;
  return cudaGetLastError();
}

}  // namespace swb
