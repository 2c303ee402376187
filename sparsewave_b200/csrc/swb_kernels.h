// Internal launch interface between the C-ABI dispatcher (swb_api.cu) and the
// kernel translation units.  All pointers are device pointers; every launcher
// enqueues on `stream`, adds the number of kernels it launched to *launches
// and returns the CUDA status of the launch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace swb {

struct CsrSpmvArgs {
  int64_t rows, cols, nnz;
  const int32_t *row_ptr;
  const int32_t *col_idx;
  const float *val;
  const float *x;
  float *y;
  bool accumulate = false;  // add to y instead of overwriting (position mappings: no zero fill)
  // The kernel queued directly before this call on the same stream is the library's own exchange kernel,
  // which produced x and the zeros of y and releases its dependents early: the span kernel may then be
  // launched with programmatic stream serialisation (it reads neither x nor y before its wait).
  bool behind_exchange = false;
};

struct CsrSpmmArgs {
  int64_t rows, cols, nnz, n_rhs;
  const int32_t *row_ptr;
  const int32_t *col_idx;
  const float *val;
  const float *B;
  float *C;
  bool accumulate = false;  // add to C instead of overwriting
};

struct BsrSpmmArgs {
  int64_t rows, cols, nnzb, block_size, n_rhs;
  const int32_t *block_row_ptr;
  const int32_t *block_col_idx;
  const void *block_values;  // f32 or bf16
  const void *B;
  void *C;
};

// Optional per-position trace of a position-mapped SpMV (all nnz entries).
struct PositionTrace {
  int32_t *row_of_position = nullptr;
  int32_t *worker_of_position = nullptr;
  int32_t *segment_end = nullptr;
  bool enabled() const { return row_of_position != nullptr; }
};

struct DeviceInfo {
  int sm_count = 148;
  int max_smem_optin = 0;
};

// y[i] = 0 (the separate initialisation launch of the position schedules).
cudaError_t launch_fill_zero(float *y, int64_t n, int block, cudaStream_t s,
                             int64_t *launches);

// Roofline probe: streams col/val (nnz rounded down to a multiple of 4, both 16-byte aligned) and gathers
// x[col[p]] with no row logic; products are added into the 1024 floats at `sink`.
cudaError_t launch_stream_gather_probe(int64_t nnz, const int32_t *col, const float *val, const float *x, float *sink,
                                       const DeviceInfo &dev, cudaStream_t s, int64_t *launches);

// --- COO SpMV (zero fill + one atomic per nonzero)
cudaError_t launch_coo_spmv_thread_per_nonzero(int64_t rows, int64_t nnz, const int32_t *row, const int32_t *col,
                                               const float *val, const float *x, float *y, int block,
                                               cudaStream_t s, int64_t *launches);

// --- SpMV row mappings
cudaError_t launch_spmv_thread_per_row(const CsrSpmvArgs &a, int block,
                                       cudaStream_t s, int64_t *launches);
cudaError_t launch_spmv_wave_per_row(const CsrSpmvArgs &a, int block,
                                     cudaStream_t s, int64_t *launches);
cudaError_t launch_spmv_block_per_row(const CsrSpmvArgs &a, int block,
                                      cudaStream_t s, int64_t *launches);

// --- SpMV position mappings (each also launches the zero fill)
cudaError_t launch_spmv_thread_per_position(const CsrSpmvArgs &a, int block,
                                            int64_t chunk, bool segmented,
                                            const PositionTrace &trace,
                                            cudaStream_t s, int64_t *launches);
// Long rows of a large matrix through shared-memory bands of x (spmv_band.cuh): `bands` bands of columns,
// rows of at least `long_min` positions, room for `cap` such rows in the scratch memory.
struct BandPlan {
  int bands = 0, long_min = 0, cap = 0;
};
bool band_path_plan(const CsrSpmvArgs &a, int64_t min_nnz, BandPlan *plan);  // false: not taken (nnz < min_nnz, ...)
size_t band_scratch_bytes(const BandPlan &plan);            // device scratch the path needs (256-byte aligned)
// `batch`: consecutive reference wave partitions walked by one warp (>= 1).  `band` + `band_scratch`
// (or NULL) switch the long-row path on; it replaces the zero-fill launch by three kernels.
cudaError_t launch_spmv_wave_per_position(const CsrSpmvArgs &a, int block,
                                          int64_t batch,
                                          const PositionTrace &trace,
                                          cudaStream_t s, int64_t *launches,
                                          int64_t *physical_grid,
                                          const BandPlan *band, void *band_scratch,
                                          const DeviceInfo &dev);
int64_t wave_per_position_auto_batch(int64_t nnz, int block,
                                     const DeviceInfo &dev);
int64_t wave_per_position_physical_grid(int64_t nnz, int block, int64_t batch);

// --- SpMM
cudaError_t launch_spmm_thread_per_output(const CsrSpmmArgs &a, int block,
                                          cudaStream_t s, int64_t *launches);
cudaError_t launch_spmm_wave_per_row_tile(const CsrSpmmArgs &a, int block,
                                          int tile, cudaStream_t s,
                                          int64_t *launches);
// CUDA blocks launch_spmm_wave_per_row_tile uses when B and C are 16-byte aligned.
int64_t wave_per_row_tile_physical_grid(int64_t rows, int64_t nnz, int64_t n_rhs, int block, int tile);
// wave-per-row-tile with a TMA-staged window of B rows around the diagonal in shared memory (spmm_staged.cu):
// 1024 matrix rows x 16 right-hand-side columns per CTA.  `status_flag`: device int raised when the bounded
// TMA wait gives up.
bool spmm_staged_supported(const CsrSpmmArgs &a);
cudaError_t launch_spmm_row_block_staged(const CsrSpmmArgs &a, int *status_flag, cudaStream_t s, int64_t *launches);
cudaError_t launch_spmm_thread_per_position(const CsrSpmmArgs &a, int block,
                                            int64_t chunk, cudaStream_t s,
                                            int64_t *launches);

// --- BSR SpMM
cudaError_t launch_bsr_spmm_thread_per_output_f32(const BsrSpmmArgs &a,
                                                  int block, cudaStream_t s,
                                                  int64_t *launches);
cudaError_t launch_bsr_spmm_thread_per_output_bf16(const BsrSpmmArgs &a,
                                                   int block, cudaStream_t s,
                                                   int64_t *launches);
// 16x16 bf16 blocks on the tcgen05 tensor cores.  `status_flag` is a device
// int the kernel sets non-zero when one of its bounded waits gives up.
bool bsr16_tcgen05_supported(const BsrSpmmArgs &a);
cudaError_t launch_bsr16_spmm_tcgen05(const BsrSpmmArgs &a, int *status_flag,
                                      const DeviceInfo &dev, cudaStream_t s,
                                      int64_t *launches);

// Context accessors for translation units that do not see the context's layout.
}  // namespace swb
struct swb_context;
namespace swb {
void set_context_error(swb_context *ctx, const char *message);
int context_device(const swb_context *ctx);
void *context_comm(const swb_context *ctx);
void set_context_comm(swb_context *ctx, void *comm, int n_ranks, int rank);
bool context_comm_shape(const swb_context *ctx, int *n_ranks, int *rank);  // false without a communicator
void *context_peer_window(const swb_context *ctx);
void set_context_peer_window(swb_context *ctx, void *window);
void *peer_window_data(const swb_context *ctx, int64_t *bytes_per_rank);  // NULL without a window
// swb_comm_window_allgather whose kernel also zero-fills zero[0 .. zero_count) (NULL: no fill)
int window_allgather_and_fill(swb_context *ctx, const void *send, float *zero, int64_t zero_count, cudaStream_t stream,
                              bool alternate, const void **gathered);
void abandon_peer_window(swb_context *ctx);  // non-collective tear-down (swb_peer_window.cu)
int *context_status_flag(const swb_context *ctx);
void count_launch(swb_context *ctx);

// Stores the diagnostic that swb_last_error(NULL) returns on this thread.
void set_thread_error(const char *message);

}  // namespace swb
