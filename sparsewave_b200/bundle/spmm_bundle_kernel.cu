// Stand-alone kernel of a SparseWave bundle: the fixed-shape CSR SpMM the
// reference's `sparsewave-bundle` packages for the lrrt runtime
// (tools/sparsewave-bundle/sparsewave_bundle_ir.py:4-17): mapping
// wave-per-row-tile, block 64, tile 4, four right-hand-side columns, five bare
// pointer arguments in the order rowOffsets, columnIndices, values, rhs,
// output (kernarg offsets 0/8/16/24/32), no shared memory, no workspace.
// The row count is fixed at compile time (-DSWB_BUNDLE_ROWS=<n>), like the
// reference's fixed-shape bundle (`fixed_output_rows`).
//
// Launch: block [64,1,1]; total work-items ceil_div(n, 2) * 64, i.e.
// ceil_div(n, 2) blocks, n = output rows (two warps = two rows per block).
#ifndef SWB_BUNDLE_ROWS
#error "compile with -DSWB_BUNDLE_ROWS=<output rows>"
#endif

extern "C" __global__ void __launch_bounds__(64)
spmm_kernel(const int *__restrict__ rowOffsets, const int *__restrict__ columnIndices,
            const float *__restrict__ values, const float *__restrict__ rhs, float *__restrict__ output) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 2 + (threadIdx.x >> 5);
  if (row >= (long long)SWB_BUNDLE_ROWS) return;
  const int start = rowOffsets[row], end = rowOffsets[row + 1];
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int p = start + lane; p < end; p += 32) {
    const int c = __ldg(columnIndices + p);
    const float v = __ldg(values + p);
    const float4 b = __ldg(reinterpret_cast<const float4 *>(rhs) + c);
    acc.x = __fadd_rn(acc.x, __fmul_rn(v, b.x));
    acc.y = __fadd_rn(acc.y, __fmul_rn(v, b.y));
    acc.z = __fadd_rn(acc.z, __fmul_rn(v, b.z));
    acc.w = __fadd_rn(acc.w, __fmul_rn(v, b.w));
  }
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    acc.x = __fadd_rn(acc.x, __shfl_xor_sync(0xffffffffu, acc.x, off));
    acc.y = __fadd_rn(acc.y, __shfl_xor_sync(0xffffffffu, acc.y, off));
    acc.z = __fadd_rn(acc.z, __shfl_xor_sync(0xffffffffu, acc.z, off));
    acc.w = __fadd_rn(acc.w, __shfl_xor_sync(0xffffffffu, acc.w, off));
  }
  if (lane == 0) reinterpret_cast<float4 *>(output)[row] = acc;
}
