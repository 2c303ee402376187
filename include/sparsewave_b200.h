/*
 * sparsewave_b200.h - C ABI of libsparsewave_b200.so
 *
 * A B200 (sm_100a) kernel backend for the SparseWave sparse operators
 * `sparsewave.spmv`, `sparsewave.spmm` and `sparsewave.bsr_spmm`.  The operand
 * lists and the option names are those of the SparseWave dialect and of its
 * `convert-sparsewave-to-gpu` / `schedule-sparsewave-position` passes; the
 * MLIR -> ROCDL -> HSACO code generation those passes feed is replaced by the
 * hand-written CUDA kernels behind these entry points.
 *
 * Conventions
 *   - Every function returns a swb_status (0 = success, negative = error).
 *     After an error, swb_last_error(ctx) holds the diagnostic; option and
 *     shape violations reproduce the reference's diagnostic text.
 *   - Unless the name ends in `_host`, data pointers are DEVICE pointers owned
 *     by the caller.  Kernels are enqueued on the caller's stream and the call
 *     returns without synchronising.  Nothing is retained after the call.
 *   - Outputs are fully overwritten; the caller never pre-zeroes them (row
 *     mappings store every element, position mappings zero-initialise first,
 *     SparsePositionScheduling.cpp:31-47,154-155).
 *   - rows == 0 and nnz == 0 are legal (the grid clamps to one inactive block,
 *     SparseGPUUtils.cpp:17-18).
 *   - A context belongs to one host thread and one device.
 *   - There is no CPU fallback: without a usable CUDA device every compute
 *     entry point fails with SWB_ERR_CUDA.
 *
 * Reference citations are paths inside the SparseWave source tree.
 */
#ifndef SPARSEWAVE_B200_H
#define SPARSEWAVE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SWB_API __attribute__((visibility("default")))

typedef struct swb_context swb_context;

/* CUDA stream handle (cudaStream_t) passed as an opaque pointer so that this
 * header needs no CUDA include.  NULL selects the legacy default stream. */
typedef void *swb_stream;

typedef enum swb_status {
  SWB_OK = 0,
  SWB_ERR_INVALID_OPTION = -1, /* option range / consistency violation      */
  SWB_ERR_INVALID_SHAPE = -2,  /* operand size contract violated            */
  SWB_ERR_INVALID_ARGUMENT = -3, /* NULL pointer, negative size, bad string */
  SWB_ERR_CUDA = -4,           /* CUDA runtime failure, text has the cause  */
  SWB_ERR_UNSUPPORTED = -5,    /* legal in the reference, not built here    */
  SWB_ERR_INVALID_DATA = -6,   /* host-side content check failed            */
  SWB_ERR_CAPACITY = -7        /* size exceeds a stated fixed maximum       */
} swb_status;

/* SpMV work mappings.  The three row mappings are the `mapping` option of
 * convert-sparsewave-to-gpu (SparseWaveToGPU.cpp:1265-1273); the two position
 * mappings are `spmv-mapping` values of the integrated pipeline
 * (Pipelines.cpp:243-256). */
typedef enum swb_spmv_mapping {
  SWB_THREAD_PER_ROW = 0,
  SWB_THREAD_PER_POSITION = 1,
  SWB_WAVE_PER_POSITION = 2,
  SWB_WAVE_PER_ROW = 3,
  SWB_BLOCK_PER_ROW = 4
} swb_spmv_mapping;

/* `thread-reduction` of schedule-sparsewave-position
 * (SparsePositionScheduling.cpp:447-453). */
typedef enum swb_position_reduction {
  SWB_REDUCTION_ATOMIC = 0,
  SWB_REDUCTION_SEGMENTED = 1
} swb_position_reduction;

/* `spmm-mapping` (SparseWaveToGPU.cpp:1274-1281, Pipelines.cpp:262-271). */
typedef enum swb_spmm_mapping {
  SWB_THREAD_PER_OUTPUT = 0,
  SWB_WAVE_PER_ROW_TILE = 1,
  SWB_SPMM_THREAD_PER_POSITION = 2
} swb_spmm_mapping;

/* Option block.  Names, defaults and ranges follow Passes.td:160-176,207-241
 * and Pipelines.h:114-190.  A wave is a CUDA warp, so wave_size must be 32 for
 * every cooperative mapping. */
typedef struct swb_options {
  int32_t mapping;                  /* swb_spmv_mapping, default thread-per-row  */
  int32_t position_reduction;       /* swb_position_reduction, default atomic    */
  int32_t spmm_mapping;             /* swb_spmm_mapping, default thread-per-output */
  /* Not a reference option.  0 (default): the output is overwritten, as every
   * reference lowering does.  1: the result is added to the existing output
   * (position mappings skip their zero fill; wave-per-row-tile adds on store).
   * Used by the multi-GPU layer to run the locally-owned columns of a row
   * shard while the all-gather of the remote part of x / B is in flight. */
  int32_t accumulate;
  int64_t block_size;               /* SpMV threads per block, default 256       */
  int64_t wave_size;                /* default 32                                */
  int64_t position_block_size;      /* position-parallel block size, default 256 */
  int64_t position_chunk_size;      /* thread-per-position chunk, default 1      */
  int64_t spmm_block_size;          /* default 256                               */
  int64_t spmm_tile_size;           /* wave-per-row-tile columns, 1..32, default 4 */
  int64_t spmm_position_chunk_size; /* default 1                                 */
  /* Not a reference option.  wave-per-position: number of consecutive
   * reference wave partitions one warp walks with a carried row segment.
   * 1 reproduces the reference schedule (one partition of <= 32 positions per
   * warp, one atomic per row segment of that partition); 0 picks a value from
   * the problem size. */
  int64_t wave_position_batch;
} swb_options;

/* ---- context ----------------------------------------------------------- */

/* Creates a context bound to CUDA device `device_ordinal`. */
SWB_API int swb_create(swb_context **out_ctx, int device_ordinal);
SWB_API void swb_destroy(swb_context *ctx);
/* Diagnostic of the last failing call on this context ("" if none).  With a
 * NULL context, the diagnostic of the last failing context-free call made by
 * this thread. */
SWB_API const char *swb_last_error(const swb_context *ctx);
/* Library version string. */
SWB_API const char *swb_version(void);
/* Number of kernels this context has launched since creation. */
SWB_API int64_t swb_kernel_launch_count(const swb_context *ctx);

/* Reads the context's device status word after the work queued on `stream`
 * has finished (synchronises that stream).  0 means no kernel gave up one of
 * its bounded waits; non-zero means a tensor-core BSR kernel abandoned a wait
 * on its pipeline barriers and its output is not valid. */
SWB_API int swb_device_status(swb_context *ctx, swb_stream stream,
                              int32_t *status);

/* ---- options (replaces the pass / pipeline option parsing) -------------- */

SWB_API void swb_options_default(swb_options *opts);
/* Parses a space- or comma-separated `key=value` list in the reference's own
 * spelling.  Pass-level keys (Passes.td:160-176,207-241): mapping, block-size,
 * wave-size, position-block-size, spmm-mapping, spmm-block-size,
 * spmm-tile-size, thread-chunk-size, thread-reduction.  Pipeline-level keys
 * (Pipelines.h:114-190): spmv-mapping, spmv-block-size,
 * spmv-position-chunk-size, spmv-position-reduction, wavefront-size,
 * spmm-position-chunk-size.  Keys of out-of-scope operators (sddmm-block-size
 * and the like) are accepted and ignored. */
SWB_API int swb_options_parse(swb_context *ctx, swb_options *opts,
                              const char *text);
/* Range and consistency checks with the reference's messages
 * (SparseWaveToGPU.cpp:1264-1397, SparsePositionScheduling.cpp:411-465). */
SWB_API int swb_options_validate(swb_context *ctx, const swb_options *opts);

/* ---- operators, device pointers ---------------------------------------- */

/* sparsewave.spmv (SparseWaveOps.td:17-52): y[r] = sum_p val[p] * x[col[p]]
 * over p in [row_ptr[r], row_ptr[r+1]).  row_ptr has rows+1 entries, col_idx
 * and val have nnz entries, x has cols entries, y has rows entries. */
SWB_API int swb_spmv(swb_context *ctx, const swb_options *opts, int64_t rows,
                     int64_t cols, int64_t nnz, const int32_t *row_ptr,
                     const int32_t *col_idx, const float *val, const float *x,
                     float *y, swb_stream stream);

/* Roofline probe for SpMV, not an operator: streams col_idx and val (nnz
 * rounded down to a multiple of 4; both arrays 16-byte aligned) and gathers
 * x[col_idx[p]] with no row logic, adding the products into the 1024 floats at
 * `sink`.  Its time on a matrix's own arrays is the floor of any mapping that
 * reads x through the cache hierarchy; the benchmark reports it beside the
 * kernel's time (the analogue of the reference runner's per-kernel bandwidth
 * columns, benchmark/run_spmv_benchmark.py:31-61).  No reference counterpart. */
SWB_API int swb_probe_stream_gather(swb_context *ctx, int64_t nnz,
                                    const int32_t *col_idx, const float *val,
                                    const float *x, float *sink,
                                    swb_stream stream);

/* sparsewave.coo_spmv (SparseWaveOps.td, COOSpMVOp; lowering
 * ThreadPerNonzeroCOOSpMVPattern, SparseWaveToGPU.cpp:154-214): y is zero
 * filled, then every entry adds val[p] * x[col_idx[p]] to y[row_idx[p]];
 * duplicate coordinates accumulate.  Uses opts->block_size. */
SWB_API int swb_coo_spmv(swb_context *ctx, const swb_options *opts, int64_t rows,
                         int64_t cols, int64_t nnz, const int32_t *row_idx,
                         const int32_t *col_idx, const float *val,
                         const float *x, float *y, swb_stream stream);

/* sparsewave.spmm (SparseWaveOps.td:91-124): C[r, j] = sum_p val[p] *
 * B[col[p], j].  B is cols x n_rhs and C is rows x n_rhs, both row-major with
 * identity layout (SparseBenchmarkUtils.cpp:261-268).  At most 2^31 - 257
 * nonzeros (SWB_ERR_UNSUPPORTED beyond). */
SWB_API int swb_spmm(swb_context *ctx, const swb_options *opts, int64_t rows,
                     int64_t cols, int64_t nnz, int64_t n_rhs,
                     const int32_t *row_ptr, const int32_t *col_idx,
                     const float *val, const float *B, float *C,
                     swb_stream stream);

/* sparsewave.bsr_spmm (SparseWaveOps.td:126-169) on f32 blocks, the element
 * type of the reference's own runtime tests; thread-per-output mapping
 * (SparseWaveToGPU.cpp:560-665).  block_values is [nnzb][bs][bs] row-major. */
SWB_API int swb_bsr_spmm_f32(swb_context *ctx, const swb_options *opts,
                             int64_t rows, int64_t cols, int64_t nnzb,
                             int64_t block_size, int64_t n_rhs,
                             const int32_t *block_row_ptr,
                             const int32_t *block_col_idx,
                             const float *block_values, const float *B,
                             float *C, swb_stream stream);

/* sparsewave.bsr_spmm on bf16 blocks with f32 accumulation and bf16 output
 * (the op requires one element type, SparseWaveOps.cpp:355-360).  Values are
 * raw bf16 bit patterns.  block_size 16 runs on the tcgen05 tensor cores;
 * other block sizes use the thread-per-output kernel. */
SWB_API int swb_bsr_spmm_bf16(swb_context *ctx, const swb_options *opts,
                              int64_t rows, int64_t cols, int64_t nnzb,
                              int64_t block_size, int64_t n_rhs,
                              const int32_t *block_row_ptr,
                              const int32_t *block_col_idx,
                              const uint16_t *block_values, const uint16_t *B,
                              uint16_t *C, swb_stream stream);

/* The tensor-core BSR SpMM (16x16 bf16 blocks, f32 accumulation, bf16 output)
 * for callers that must not allocate device memory.  It has no counterpart in
 * the reference; it exists because the entry point above needs a context, and
 * creating a context allocates the status word the kernel raises when one of
 * its bounded barrier waits gives up.  A caller that lives under a memory
 * budget fixed at start-up, that is loaded into a process which forbids
 * allocations after initialisation, or that may run while the allocator is
 * locked cannot do that.  This entry point takes no context, calls no
 * cudaMalloc / cudaFree and keeps its status words in a fixed 128 KiB array
 * inside the library image (held by every GPU that loads the library until
 * the process exits), one word per (block row, 256-column tile) pair.
 *   - Limit: (rows / 16) * ceil(n_rhs / 256) <= 32768, else SWB_ERR_CAPACITY.
 *   - Needs nnzb > 0, n_rhs % 8 == 0 and 16-byte aligned block_values and B,
 *     else SWB_ERR_UNSUPPORTED (there is no second kernel behind it).
 *   - The first call on a device looks up the array's device address; make
 *     that call before any stream capture begins.
 *   - Every call shares the array and first clears the words it uses, so it
 *     holds the outcome of the latest call only, and calls that overlap on
 *     the GPU race on it.
 *   - gave_up_ctas: NULL for an asynchronous call (check it later with
 *     swb_bsr16_static_status, before the next static call on that device);
 *     otherwise the call synchronises `stream` and stores how many CTAs
 *     abandoned a wait (0 = the output is valid).
 * Errors are reported through swb_last_error(NULL). */
SWB_API int swb_bsr16_spmm_bf16_static(int64_t rows, int64_t cols, int64_t nnzb,
                                       int64_t n_rhs,
                                       const int32_t *block_row_ptr,
                                       const int32_t *block_col_idx,
                                       const uint16_t *block_values,
                                       const uint16_t *B, uint16_t *C,
                                       swb_stream stream,
                                       int32_t *gave_up_ctas);
/* Outcome of the most recent swb_bsr16_spmm_bf16_static call on the current
 * device: synchronises `stream` (the stream that call was queued on) and
 * stores how many of its CTAs abandoned a wait (0 = its output is valid).
 * Like that call it allocates nothing (the fixed array is read back through
 * stack memory) and has no counterpart in the reference.  A later static call
 * on the same device overwrites the record, so ask before making one. */
SWB_API int swb_bsr16_static_status(swb_stream stream, int32_t *gave_up_ctas);

/* ---- operators, host buffers ------------------------------------------- */
/* Same contracts with HOST pointers: the call copies the operands to the
 * context's device workspace (grown on demand and kept), runs the kernel,
 * copies the result back and synchronises.  This is the call a host program
 * that keeps its matrices in host memory makes (the reference's benchmark
 * host code does gpu.alloc + gpu.memcpy around each @spmv call,
 * benchmark/spmv.mlir.in:37-70). */
SWB_API int swb_spmv_host(swb_context *ctx, const swb_options *opts,
                          int64_t rows, int64_t cols, int64_t nnz,
                          const int32_t *row_ptr, const int32_t *col_idx,
                          const float *val, const float *x, float *y);
SWB_API int swb_spmm_host(swb_context *ctx, const swb_options *opts,
                          int64_t rows, int64_t cols, int64_t nnz,
                          int64_t n_rhs, const int32_t *row_ptr,
                          const int32_t *col_idx, const float *val,
                          const float *B, float *C);
SWB_API int swb_bsr_spmm_bf16_host(swb_context *ctx, const swb_options *opts,
                                   int64_t rows, int64_t cols, int64_t nnzb,
                                   int64_t block_size, int64_t n_rhs,
                                   const int32_t *block_row_ptr,
                                   const int32_t *block_col_idx,
                                   const uint16_t *block_values,
                                   const uint16_t *B, uint16_t *C);

/* Matrix resident on the device, dense operands in host memory: the shape of
 * the reference's own host programs, which copy the matrix to the device once
 * and then call the operator in a loop (benchmark/spmv.mlir.in:37-65).
 * swb_csr_upload checks the index arrays (as swb_check_csr_host does) and
 * copies the matrix; the per-call functions copy x (or B) in, run the kernel,
 * copy y (or C) out and synchronise.  Large matrices are cut into row panels
 * at upload (swb_plan_row_panels) and the rows of the result start their copy
 * to the host as soon as their panel is done, while later panels compute;
 * matrices of 40 M nonzeros or more (SWB_RESIDENT_SPLIT_NNZ) are also kept as
 * two column parts (twice the device memory) so that the first part computes
 * while the rest of the dense operand is still being copied in.  Use
 * pinned host buffers to benefit.  The handle belongs to the context's device
 * and is released with swb_csr_release. */
typedef struct swb_csr_handle swb_csr_handle;
SWB_API int swb_csr_upload(swb_context *ctx, int64_t rows, int64_t cols,
                           int64_t nnz, const int32_t *row_ptr,
                           const int32_t *col_idx, const float *val,
                           swb_csr_handle **out);
SWB_API void swb_csr_release(swb_context *ctx, swb_csr_handle *matrix);
SWB_API int swb_spmv_resident_host(swb_context *ctx, const swb_options *opts,
                                   const swb_csr_handle *matrix,
                                   const float *x, float *y);
SWB_API int swb_spmm_resident_host(swb_context *ctx, const swb_options *opts,
                                   const swb_csr_handle *matrix, int64_t n_rhs,
                                   const float *B, float *C);

/* The same for a bf16 BSR matrix: swb_bsr_upload checks the block structure on
 * the host (offsets start at 0, are monotone and end at nnzb; block columns in
 * range) and copies it to the device once; swb_bsr_spmm_bf16_resident_host
 * copies B (cols x n_rhs bf16) in, runs the BSR SpMM (the tensor-core kernel
 * for 16 x 16 blocks), copies C (rows x n_rhs bf16) out and synchronises. */
typedef struct swb_bsr_handle swb_bsr_handle;
SWB_API int swb_bsr_upload(swb_context *ctx, int64_t rows, int64_t cols,
                           int64_t nnzb, int64_t block_size,
                           const int32_t *block_row_ptr,
                           const int32_t *block_col_idx,
                           const uint16_t *block_values, swb_bsr_handle **out);
SWB_API void swb_bsr_release(swb_context *ctx, swb_bsr_handle *matrix);
SWB_API int swb_bsr_spmm_bf16_resident_host(swb_context *ctx,
                                            const swb_options *opts,
                                            const swb_bsr_handle *matrix,
                                            int64_t n_rhs, const uint16_t *B,
                                            uint16_t *C);

/* ---- sharded operators -------------------------------------------------- */
/* One row shard per rank of the context's communicator (swb_comm_init), the
 * dense operand owned in equal contiguous chunks of ceil(cols / n_ranks) rows
 * (rank k owns rows [k * chunk, min(cols, (k + 1) * chunk)) of x or B).  A call
 * gathers every rank's chunk into a full copy on this device - with the
 * peer-store kernel when the context has a window of exactly that chunk size
 * (swb_comm_window_create), else with ncclAllGather into a buffer the context
 * keeps - and then runs the operator on this rank's rows: y / C hold the
 * shard's rows only.  Collective: every rank makes the same call.  The buffers
 * are allocated by the first call that needs them (make it outside stream
 * capture).  Without a communicator the calls are the plain operators.  Not a
 * reference feature (the reference is single GPU).
 *
 * swb_spmv_sharded / swb_spmm_sharded take the shard's CSR arrays (row offsets
 * rebased to zero, global column numbers) and this rank's chunk as DEVICE
 * pointers and queue everything on `stream`. */
SWB_API int swb_spmv_sharded(swb_context *ctx, const swb_options *opts,
                             int64_t rows, int64_t cols, int64_t nnz,
                             const int32_t *row_ptr, const int32_t *col_idx,
                             const float *val, const float *x_owned, float *y,
                             swb_stream stream);
SWB_API int swb_spmm_sharded(swb_context *ctx, const swb_options *opts,
                             int64_t rows, int64_t cols, int64_t nnz,
                             int64_t n_rhs, const int32_t *row_ptr,
                             const int32_t *col_idx, const float *val,
                             const float *B_owned, float *C,
                             swb_stream stream);
/* swb_csr_upload_rows keeps rows [row_begin, row_end) of a HOST matrix on the
 * device (offsets rebased to zero, checked like swb_csr_upload, one copy, no
 * panels): the shard of a rank whose boundaries come from
 * swb_shard_rows_by_nnz.  The *_sharded_host calls then take this rank's
 * chunk of the dense operand and return this rank's rows in HOST memory: chunk
 * in, exchange on the device, kernel, rows out, synchronised. */
SWB_API int swb_csr_upload_rows(swb_context *ctx, int64_t rows_total,
                                int64_t cols, const int32_t *row_ptr,
                                const int32_t *col_idx, const float *val,
                                int64_t row_begin, int64_t row_end,
                                swb_csr_handle **out);
SWB_API int swb_spmv_sharded_host(swb_context *ctx, const swb_options *opts,
                                  const swb_csr_handle *shard,
                                  const float *x_owned, float *y);
SWB_API int swb_spmm_sharded_host(swb_context *ctx, const swb_options *opts,
                                  const swb_csr_handle *shard, int64_t n_rhs,
                                  const float *B_owned, float *C);

/* Content checks the kernels rely on, run on HOST copies of the index arrays
 * before data is trusted: row_ptr[0] == 0, monotone, row_ptr[rows] == nnz,
 * 0 <= col < cols.  (The reference aborts on malformed benchmark inputs,
 * SparseBenchmarkUtils.cpp:31-34; here the call returns SWB_ERR_INVALID_DATA.) */
SWB_API int swb_check_csr_host(swb_context *ctx, int64_t rows, int64_t cols,
                               int64_t nnz, const int32_t *row_ptr,
                               const int32_t *col_idx);

/* ---- MLIR C-interface twins -------------------------------------------- */
/* What a `func.call` emitted with llvm.emit_c_interface binds: one pointer to
 * a memref descriptor per operand (the convention of
 * SparseBenchmarkUtils.cpp:211-216).  Data pointers are device pointers;
 * strides must be the identity layout.  These use a process-wide context on
 * the current device and the option string in the environment variable
 * SPARSEWAVE_B200_OPTIONS (pipeline spelling), synchronise before returning
 * and abort with a message on error, as the reference's helpers do. */
typedef struct swb_memref_1d_i32 { int32_t *base, *data; int64_t offset, sizes[1], strides[1]; } swb_memref_1d_i32;
typedef struct swb_memref_1d_f32 { float *base, *data; int64_t offset, sizes[1], strides[1]; } swb_memref_1d_f32;
typedef struct swb_memref_2d_f32 { float *base, *data; int64_t offset, sizes[2], strides[2]; } swb_memref_2d_f32;

/* Status-returning forms on an explicit context and stream; they apply the
 * operand-size checks of the op verifiers with their diagnostics
 * (SparseWaveOps.cpp:83-108, 144-207, 271-372) and do not synchronise. */
SWB_API int swb_spmv_memref(swb_context *ctx, const swb_options *opts,
                            swb_memref_1d_i32 *row_offsets,
                            swb_memref_1d_i32 *column_indices,
                            swb_memref_1d_f32 *values,
                            swb_memref_1d_f32 *vector,
                            swb_memref_1d_f32 *output, swb_stream stream);
SWB_API int swb_spmm_memref(swb_context *ctx, const swb_options *opts,
                            swb_memref_1d_i32 *row_offsets,
                            swb_memref_1d_i32 *column_indices,
                            swb_memref_1d_f32 *values, swb_memref_2d_f32 *rhs,
                            swb_memref_2d_f32 *output, swb_stream stream);
SWB_API int swb_bsr_spmm_memref(swb_context *ctx, const swb_options *opts,
                                swb_memref_1d_i32 *block_row_offsets,
                                swb_memref_1d_i32 *block_column_indices,
                                swb_memref_1d_f32 *block_values,
                                swb_memref_2d_f32 *rhs,
                                swb_memref_2d_f32 *output, int64_t block_size,
                                swb_stream stream);

SWB_API void _mlir_ciface_sparsewave_spmv(swb_memref_1d_i32 *row_offsets,
                                          swb_memref_1d_i32 *column_indices,
                                          swb_memref_1d_f32 *values,
                                          swb_memref_1d_f32 *vector,
                                          swb_memref_1d_f32 *output);
SWB_API void _mlir_ciface_sparsewave_spmm(swb_memref_1d_i32 *row_offsets,
                                          swb_memref_1d_i32 *column_indices,
                                          swb_memref_1d_f32 *values,
                                          swb_memref_2d_f32 *rhs,
                                          swb_memref_2d_f32 *output);
SWB_API void _mlir_ciface_sparsewave_bsr_spmm(swb_memref_1d_i32 *block_row_offsets,
                                              swb_memref_1d_i32 *block_column_indices,
                                              swb_memref_1d_f32 *block_values,
                                              swb_memref_2d_f32 *rhs,
                                              swb_memref_2d_f32 *output,
                                              int64_t block_size);

/* ---- bundle-style launch ------------------------------------------------ */
/* The lrrt bundle launch contract for the fixed-shape SpMM kernel
 * (tools/sparsewave-bundle/sparsewave_bundle_ir.py:4-17,
 * sparsewave_bundle_manifest.py:64-120): five device pointers in the order
 * rowOffsets, columnIndices, values, rhs, output; n = output rows; mapping
 * wave-per-row-tile, block 64, tile 4, four right-hand-side columns.
 * `operation` must be "spmm". */
SWB_API int swb_bundle_launch(swb_context *ctx, const char *operation,
                              int64_t n, void *const args[5],
                              swb_stream stream);

/* ---- index helpers (host side of the shared host/device arithmetic) ----- */

/* sparsewave.position_space partition (SparsePositionToSCF.cpp:190-223). */
SWB_API void swb_partition(int64_t lower, int64_t upper, int64_t worker,
                           int64_t worker_count, int64_t *begin, int64_t *end);
/* sparsewave.position_for chunk bounds (SparsePositionToSCF.cpp:38-98); an
 * inactive worker gets begin == end. */
SWB_API void swb_chunk_bounds(int64_t lower, int64_t upper, int64_t worker,
                              int64_t factor, int64_t *begin, int64_t *end);
/* sparsewave.csr_row_at_position: upper-bound search over row offsets
 * (SparsePositionToSCF.cpp:225-271).  row_ptr is a HOST array of
 * row_ptr_len entries. */
SWB_API int64_t swb_row_at_position(const int32_t *row_ptr,
                                    int64_t row_ptr_len, int64_t position);

/* Launch geometry of an operator under `opts`: the reference's logical grid
 * and block (SparseGPUUtils.cpp:11-59, SparseWaveToGPU.cpp:380,
 * SparsePositionScheduling.cpp:340-350), the number of kernels per call and
 * the physical CUDA grid this library launches.  n_rhs == 0 selects SpMV. */
typedef struct swb_launch_shape {
  int64_t logical_grid;   /* blocks the reference would launch            */
  int64_t logical_block;  /* threads per block                            */
  int64_t work_units;     /* rows, outputs, workers or waves               */
  int64_t kernels;        /* launches per call (2 for position mappings)   */
  int64_t physical_grid;  /* CUDA blocks of the compute kernel (for 16-byte
                             aligned operands)                             */
} swb_launch_shape;
SWB_API int swb_launch_shape_query(swb_context *ctx, const swb_options *opts,
                                   int64_t rows, int64_t nnz, int64_t n_rhs,
                                   swb_launch_shape *out);

/* Debug variant of a position-mapped SpMV: besides y it records, per
 * position, the row it was attributed to, the worker (thread or wave) that
 * processed it and whether the position closed a segment (emitted an atomic
 * add).  Arrays have nnz entries (device pointers). */
SWB_API int swb_spmv_position_trace(swb_context *ctx, const swb_options *opts,
                                    int64_t rows, int64_t cols, int64_t nnz,
                                    const int32_t *row_ptr,
                                    const int32_t *col_idx, const float *val,
                                    const float *x, float *y,
                                    int32_t *row_of_position,
                                    int32_t *worker_of_position,
                                    int32_t *segment_end, swb_stream stream);

/* ---- multi-GPU communicator ------------------------------------------------ */
/* One NCCL communicator per context over the GPUs of one node (one process per
 * GPU).  Not a reference feature.  Rank 0 makes the 128-byte id with
 * swb_comm_unique_id and hands it to the other ranks by any host channel;
 * every rank then calls swb_comm_init (collective: it returns once all ranks
 * have joined).  swb_comm_allgather gathers `bytes_per_rank` bytes from every
 * rank into `recv` (rank k's bytes at offset k * bytes_per_rank) on `stream`:
 * the exchange of the dense operand (x or B) that precedes the local kernel
 * of a row shard.  swb_destroy releases the communicator. */
SWB_API int swb_comm_unique_id(uint8_t id[128]);
SWB_API int swb_comm_init(swb_context *ctx, const uint8_t id[128], int n_ranks,
                          int rank);
SWB_API int swb_comm_allgather(swb_context *ctx, const void *send, void *recv,
                               int64_t bytes_per_rank, swb_stream stream);
SWB_API void swb_comm_destroy(swb_context *ctx);

/* The same exchange as one kernel of peer stores over NVLink instead of
 * ncclAllGather.  swb_comm_window_create (collective over the communicator's
 * ranks, which must be processes of one node) allocates a window of n_ranks *
 * bytes_per_rank bytes on every rank (and a second buffer of the same size
 * behind it, which the sharded operators fill in turn with the first so that
 * their steps need no "no longer reading" round trip between the ranks), maps
 * the windows of the other ranks with CUDA IPC and returns this rank's window;
 * bytes_per_rank must be a multiple of 16.  swb_comm_window_allgather queues one kernel on `stream` that stores
 * the bytes_per_rank bytes at `send` (16-byte aligned device memory) into
 * every rank's window at offset rank * bytes_per_rank; work queued behind it
 * on the same stream finds the whole window filled.  A window must not be read
 * by other streams while a later all-gather may overwrite it.  The kernel's
 * waits on the other ranks are bounded: if one gives up (a rank that never
 * launches its step), swb_device_status reports 3 or 4 and the window content
 * is not valid.  One window per context; capturable in a CUDA graph.
 * swb_comm_window_allgather_next is the form the sharded operators use: it
 * fills the window's two buffers in turn (the first call after creation fills
 * the one swb_comm_window_create returned, the second buffer lies n_ranks *
 * bytes_per_rank bytes behind it) and stores the address of the buffer of this
 * call in *gathered.  Calls that take turns need no round trip between the
 * ranks before the stores; a call that meets the buffer of the call before it
 * (swb_comm_window_allgather twice, or a replayed graph with an odd number of
 * steps) waits for the peers first, decided on the device.
 * swb_comm_window_destroy is collective too (every rank unmaps before any
 * rank frees), so call it on every rank, while all ranks are still alive;
 * swb_destroy never runs a collective: on a context that still has a window
 * it only unmaps the peers' windows and leaves this rank's window allocated
 * until the process ends. */
SWB_API int swb_comm_window_create(swb_context *ctx, int64_t bytes_per_rank,
                                   void **window);
SWB_API int swb_comm_window_allgather(swb_context *ctx, const void *send,
                                      swb_stream stream);
SWB_API int swb_comm_window_allgather_next(swb_context *ctx, const void *send,
                                           swb_stream stream,
                                           const void **gathered);
SWB_API void swb_comm_window_destroy(swb_context *ctx);

/* ---- multi-GPU row sharding --------------------------------------------- */
/* nnz-balanced contiguous row shards: boundaries[k] = the first row r with
 * row_ptr[r] >= k * nnz / n_shards (exact integer arithmetic), boundaries[0]
 * = 0, boundaries[n_shards] = rows.  row_ptr is a HOST array; boundaries has
 * n_shards + 1 entries.  Not a reference feature (the reference is single
 * GPU). */
SWB_API int swb_shard_rows_by_nnz(swb_context *ctx, const int32_t *row_ptr,
                                  int64_t rows, int64_t n_shards,
                                  int64_t *boundaries);

/* ---- row panels of a resident matrix -------------------------------------- */
/* The cut swb_csr_upload makes for the pipelined result copy of the resident
 * host calls: min(8, nnz / panel_nnz) contiguous row panels of about equal
 * nnz each, every panel starting at a row whose first position is a multiple of
 * 4 (so its col/val slices stay 16-byte aligned).  row_ptr is a HOST array of
 * rows + 1 offsets starting at 0; panel_rows receives the first row of each
 * panel followed by `rows` (at most 9 entries); returns the number of panels
 * (>= 1).  Not a reference feature. */
SWB_API int swb_plan_row_panels(int64_t rows, int64_t nnz, const int32_t *row_ptr,
                                int64_t panel_nnz, int64_t *panel_rows);

#ifdef __cplusplus
}
#endif
#endif /* SPARSEWAVE_B200_H */
