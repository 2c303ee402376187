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

template <typename T>
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
    for (int64_t lc = 0; lc < bs; ++lc) sum = add(sum, mul(to_f32(a[lc]), to_f32(b[lc * N])));
  }
  store(C + e, sum);
}

}  // namespace

cudaError_t launch_bsr_spmm_thread_per_output_f32(const BsrSpmmArgs &a, int block, cudaStream_t s,
                                                  int64_t *launches) {
  unsigned grid = 0;  // refused, not truncated, beyond the CUDA grid limit
  if (!grid_dim(ceil_div(a.rows * a.n_rhs, block), &grid)) return cudaErrorInvalidConfiguration;
  bsr_spmm_thread_per_output_kernel<float><<<grid, block, 0, s>>>(
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
  bsr_spmm_thread_per_output_kernel<__nv_bfloat16><<<grid, block, 0, s>>>(
      a.rows, a.n_rhs, a.block_size, a.block_row_ptr, a.block_col_idx,
      static_cast<const __nv_bfloat16 *>(a.block_values), static_cast<const __nv_bfloat16 *>(a.B),
      static_cast<__nv_bfloat16 *>(a.C));
  ++*launches;
  return cudaGetLastError();
}

}  // namespace swb
