// C ABI of libsparsewave_b200.so: context, option parsing and validation with
// the reference's diagnostics, operand checks, dispatch to the kernels.
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "../../include/sparsewave_b200.h"
#include "swb_index.h"
#include "swb_kernels.h"

struct swb_context {
  int device = 0;
  swb::DeviceInfo dev;
  std::string error;
  int64_t launches = 0;
  // Device workspace of the *_host entry points: one allocation, grown on
  // demand, carved by a bump pointer per call.
  char *workspace = nullptr;
  size_t workspace_bytes = 0;
  size_t workspace_used = 0;
  cudaStream_t host_stream = nullptr;
  // Result copies of the resident-matrix host calls run here, behind the kernels of later row panels.
  cudaStream_t copy_stream = nullptr;
  cudaEvent_t panel_done[8] = {};
  // The dense operand of those calls travels here in two halves.
  cudaStream_t upload_stream = nullptr;
  cudaEvent_t upload_done[2] = {};
  // Scratch of the long-row path of wave-per-position SpMV (list of long rows and their band
  // boundaries): grown on demand by the first call that needs it, kept.
  void *band_scratch = nullptr;
  size_t band_scratch_bytes = 0;
  int *status_flag = nullptr;  // device int for kernels with bounded waits
  // Sharded operators: device copy of this rank's chunk of the dense operand padded to the common chunk
  // size, and the gathered operand when no peer window serves (both grown on demand, kept).
  char *shard_send = nullptr, *shard_full = nullptr;
  size_t shard_send_bytes = 0, shard_full_bytes = 0;
  bool behind_exchange = false;  // one-shot: the next swb_spmv is queued directly behind the exchange kernel
  void *comm = nullptr;        // NCCL communicator of the multi-GPU path (swb_comm.cu)
  void *peer_window = nullptr; // peer-store all-gather window (swb_peer_window.cu)
  int comm_ranks = 1, comm_rank = 0;
};

namespace {

thread_local std::string g_thread_error;

int fail(swb_context *ctx, int status, const char *fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (ctx)
    ctx->error = buf;
  else
    g_thread_error = buf;
  return status;
}

}  // namespace

namespace swb {
void set_thread_error(const char *message) { g_thread_error = message ? message : ""; }
void set_context_error(swb_context *ctx, const char *message) {
  if (ctx) ctx->error = message ? message : ""; else set_thread_error(message);
}
int context_device(const swb_context *ctx) { return ctx->device; }
void *context_comm(const swb_context *ctx) { return ctx->comm; }
void set_context_comm(swb_context *ctx, void *comm, int n_ranks, int rank) {
  ctx->comm = comm;
  ctx->comm_ranks = n_ranks;
  ctx->comm_rank = rank;
}
bool context_comm_shape(const swb_context *ctx, int *n_ranks, int *rank) {
  *n_ranks = ctx->comm_ranks;
  *rank = ctx->comm_rank;
  return ctx->comm != nullptr;
}
void *context_peer_window(const swb_context *ctx) { return ctx->peer_window; }
void set_context_peer_window(swb_context *ctx, void *window) { ctx->peer_window = window; }
int *context_status_flag(const swb_context *ctx) { return ctx->status_flag; }
void count_launch(swb_context *ctx) { ++ctx->launches; }
}  // namespace swb

namespace {

int cuda_fail(swb_context *ctx, cudaError_t e, const char *what) {
  return fail(ctx, SWB_ERR_CUDA, "CUDA error in %s: %s", what, cudaGetErrorString(e));
}

const char *spmv_mapping_name(int m) {
  switch (m) {
    case SWB_THREAD_PER_ROW: return "thread-per-row";
    case SWB_THREAD_PER_POSITION: return "thread-per-position";
    case SWB_WAVE_PER_POSITION: return "wave-per-position";
    case SWB_WAVE_PER_ROW: return "wave-per-row";
    case SWB_BLOCK_PER_ROW: return "block-per-row";
  }
  return nullptr;
}

bool is_position_mapping(int m) {
  return m == SWB_THREAD_PER_POSITION || m == SWB_WAVE_PER_POSITION;
}

// Keys of operators outside this library: parsed, range-checked with the
// reference's message (SparseWaveToGPU.cpp:1315-1346), otherwise unused.
struct ForeignBlockSize {
  const char *key;
  const char *label;
};
const ForeignBlockSize kForeign[] = {
    {"sddmm-block-size", "SDDMM block size"},
    {"row-reduction-block-size", "CSR row-reduction block size"},
    {"rowwise-map-block-size", "CSR row-wise map block size"},
    {"elementwise-block-size", "elementwise block size"},
};

bool parse_int(const std::string &s, int64_t &out) {
  if (s.empty()) return false;
  char *end = nullptr;
  long long v = strtoll(s.c_str(), &end, 10);
  if (*end != '\0') return false;
  out = v;
  return true;
}

constexpr int64_t kI32Max = 2147483647LL;

int check_ctx(swb_context *ctx) {
  if (!ctx) return fail(nullptr, SWB_ERR_INVALID_ARGUMENT, "context is NULL");
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaSetDevice");
  return SWB_OK;
}

int check_csr_sizes(swb_context *ctx, const char *op, int64_t rows, int64_t cols, int64_t nnz) {
  if (rows < 0 || cols < 0 || nnz < 0)
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "%s: rows, cols and nnz must be non-negative", op);
  // i32 row offsets and column indices (benchmark/run_spmv_benchmark.py:581-600).
  if (rows >= kI32Max || cols > kI32Max || nnz > kI32Max)
    return fail(ctx, SWB_ERR_INVALID_SHAPE, "%s: matrix rows and NNZ must fit in the i32 CSR type", op);
  return SWB_OK;
}

// Workspace -----------------------------------------------------------------
int workspace_reserve(swb_context *ctx, size_t bytes) {
  ctx->workspace_used = 0;
  if (bytes <= ctx->workspace_bytes) return SWB_OK;
  if (ctx->workspace) {
    cudaFree(ctx->workspace);
    ctx->workspace = nullptr;
    ctx->workspace_bytes = 0;
  }
  cudaError_t e = cudaMalloc(&ctx->workspace, bytes);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMalloc(workspace)");
  ctx->workspace_bytes = bytes;
  return SWB_OK;
}

size_t pad256(size_t b) { return (b + 255) & ~(size_t)255; }

template <typename T>
T *workspace_take(swb_context *ctx, size_t count) {
  T *p = reinterpret_cast<T *>(ctx->workspace + ctx->workspace_used);
  ctx->workspace_used += pad256(count * sizeof(T));
  return p;
}

int ensure_host_stream(swb_context *ctx) {
  if (ctx->host_stream) return SWB_OK;
  cudaError_t e = cudaStreamCreateWithFlags(&ctx->host_stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaStreamCreate");
  return SWB_OK;
}

int ensure_copy_stream(swb_context *ctx) {
  if (ctx->copy_stream) return SWB_OK;
  cudaError_t e = cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->upload_stream, cudaStreamNonBlocking);
  for (int k = 0; e == cudaSuccess && k < 8; ++k)
    e = cudaEventCreateWithFlags(&ctx->panel_done[k], cudaEventDisableTiming);
  for (int k = 0; e == cudaSuccess && k < 2; ++k)
    e = cudaEventCreateWithFlags(&ctx->upload_done[k], cudaEventDisableTiming);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaStreamCreate(copy)");
  return SWB_OK;
}

int64_t env_i64(const char *name, int64_t fallback) {
  const char *text = getenv(name);
  if (!text || !*text) return fallback;
  char *end = nullptr;
  long long v = strtoll(text, &end, 10);
  return (*end == '\0' && v > 0) ? v : fallback;
}

// like env_i64, but "0" is a value
int64_t env_i64_or_zero(const char *name, int64_t fallback) {
  const char *text = getenv(name);
  if (!text || !*text) return fallback;
  char *end = nullptr;
  long long v = strtoll(text, &end, 10);
  return (*end == '\0' && v >= 0) ? v : fallback;
}

#define SWB_CUDA(ctx, call)                                   \
  do {                                                        \
    cudaError_t e__ = (call);                                 \
    if (e__ != cudaSuccess) return cuda_fail(ctx, e__, #call); \
  } while (0)

}  // namespace

extern "C" {

const char *swb_version(void) { return "sparsewave_b200 0.1 (sm_100a)"; }

int swb_create(swb_context **out_ctx, int device_ordinal) {
  if (!out_ctx) return fail(nullptr, SWB_ERR_INVALID_ARGUMENT, "out_ctx is NULL");
  *out_ctx = nullptr;
  int count = 0;
  cudaError_t e = cudaGetDeviceCount(&count);
  if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaGetDeviceCount");
  if (device_ordinal < 0 || device_ordinal >= count)
    return fail(nullptr, SWB_ERR_CUDA, "CUDA device %d is not available (%d devices)", device_ordinal, count);
  e = cudaSetDevice(device_ordinal);
  if (e != cudaSuccess) return cuda_fail(nullptr, e, "cudaSetDevice");
  swb_context *ctx = new swb_context();
  ctx->device = device_ordinal;
  cudaDeviceGetAttribute(&ctx->dev.sm_count, cudaDevAttrMultiProcessorCount, device_ordinal);
  cudaDeviceGetAttribute(&ctx->dev.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device_ordinal);
  // Status word of kernels with bounded waits (0 = no wait ever gave up).
  e = cudaMalloc(&ctx->status_flag, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(ctx->status_flag, 0, sizeof(int));
  if (e != cudaSuccess) {
    delete ctx;
    return cuda_fail(nullptr, e, "cudaMalloc(status)");
  }
  *out_ctx = ctx;
  return SWB_OK;
}

int swb_device_status(swb_context *ctx, swb_stream stream, int32_t *status) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  if (!status) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "status is NULL");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int v = 0;
  SWB_CUDA(ctx, cudaMemcpyAsync(&v, ctx->status_flag, sizeof(int), cudaMemcpyDeviceToHost, s));
  SWB_CUDA(ctx, cudaStreamSynchronize(s));
  *status = v;
  return SWB_OK;
}

void swb_destroy(swb_context *ctx) {
  if (!ctx) return;
  cudaSetDevice(ctx->device);
  swb::abandon_peer_window(ctx);  // never a collective here: the other ranks may be gone
  swb_comm_destroy(ctx);
  if (ctx->workspace) cudaFree(ctx->workspace);
  if (ctx->band_scratch) cudaFree(ctx->band_scratch);
  if (ctx->shard_send) cudaFree(ctx->shard_send);
  if (ctx->shard_full) cudaFree(ctx->shard_full);
  if (ctx->status_flag) cudaFree(ctx->status_flag);
  if (ctx->host_stream) cudaStreamDestroy(ctx->host_stream);
  if (ctx->copy_stream) cudaStreamDestroy(ctx->copy_stream);
  if (ctx->upload_stream) cudaStreamDestroy(ctx->upload_stream);
  for (cudaEvent_t ev : ctx->panel_done)
    if (ev) cudaEventDestroy(ev);
  for (cudaEvent_t ev : ctx->upload_done)
    if (ev) cudaEventDestroy(ev);
  delete ctx;
}

const char *swb_last_error(const swb_context *ctx) {
  return ctx ? ctx->error.c_str() : g_thread_error.c_str();
}

int64_t swb_kernel_launch_count(const swb_context *ctx) { return ctx ? ctx->launches : 0; }

// ---- options ---------------------------------------------------------------

void swb_options_default(swb_options *o) {
  if (!o) return;
  memset(o, 0, sizeof *o);
  o->mapping = SWB_THREAD_PER_ROW;
  o->position_reduction = SWB_REDUCTION_ATOMIC;
  o->spmm_mapping = SWB_THREAD_PER_OUTPUT;
  o->block_size = 256;
  o->wave_size = 32;
  o->position_block_size = 256;
  o->position_chunk_size = 1;
  o->spmm_block_size = 256;
  o->spmm_tile_size = 4;
  o->spmm_position_chunk_size = 1;
  o->wave_position_batch = 0;
}

int swb_options_parse(swb_context *ctx, swb_options *o, const char *text) {
  if (!o) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "options is NULL");
  if (!text) return SWB_OK;
  std::string s(text);
  size_t i = 0;
  while (i < s.size()) {
    while (i < s.size() && (s[i] == ' ' || s[i] == ',' || s[i] == '\t' || s[i] == '\n')) ++i;
    if (i >= s.size()) break;
    size_t j = i;
    while (j < s.size() && s[j] != ' ' && s[j] != ',' && s[j] != '\t' && s[j] != '\n') ++j;
    std::string tok = s.substr(i, j - i);
    i = j;
    size_t eq = tok.find('=');
    if (eq == std::string::npos)
      return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "expected key=value, but got '%s'", tok.c_str());
    std::string key = tok.substr(0, eq), value = tok.substr(eq + 1);
    int64_t n = 0;
    auto want_int = [&](int64_t &dst) -> int {
      if (!parse_int(value, n))
        return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "option '%s' expects an integer, but got '%s'", key.c_str(), value.c_str());
      dst = n;
      return SWB_OK;
    };
    int st = SWB_OK;
    if (key == "mapping" || key == "spmv-mapping") {
      if (value == "thread-per-row") o->mapping = SWB_THREAD_PER_ROW;
      else if (value == "wave-per-row") o->mapping = SWB_WAVE_PER_ROW;
      else if (value == "block-per-row") o->mapping = SWB_BLOCK_PER_ROW;
      else if (value == "thread-per-position" || (key == "mapping" && value == "thread")) o->mapping = SWB_THREAD_PER_POSITION;
      else if (value == "wave-per-position" || (key == "mapping" && value == "wave")) o->mapping = SWB_WAVE_PER_POSITION;
      else if (key == "mapping" && value == "block")
        // schedule-sparsewave-position mapping (SparsePositionScheduling.cpp:412-417)
        return fail(ctx, SWB_ERR_INVALID_OPTION, "unsupported position mapping '%s'; expected 'thread' or 'wave'", value.c_str());
      else
        return fail(ctx, SWB_ERR_INVALID_OPTION,
                    "unsupported SpMV mapping strategy '%s'; expected 'thread-per-row', 'wave-per-row', or 'block-per-row'",
                    value.c_str());
    } else if (key == "spmm-mapping") {
      if (value == "thread-per-output") o->spmm_mapping = SWB_THREAD_PER_OUTPUT;
      else if (value == "wave-per-row-tile") o->spmm_mapping = SWB_WAVE_PER_ROW_TILE;
      else if (value == "thread-per-position") o->spmm_mapping = SWB_SPMM_THREAD_PER_POSITION;
      else
        return fail(ctx, SWB_ERR_INVALID_OPTION,
                    "unsupported SpMM mapping strategy '%s'; expected 'thread-per-output' or 'wave-per-row-tile'",
                    value.c_str());
    } else if (key == "thread-reduction" || key == "spmv-position-reduction") {
      if (value == "atomic") o->position_reduction = SWB_REDUCTION_ATOMIC;
      else if (value == "segmented") o->position_reduction = SWB_REDUCTION_SEGMENTED;
      else
        return fail(ctx, SWB_ERR_INVALID_OPTION,
                    "unsupported thread position reduction '%s'; expected 'atomic' or 'segmented'", value.c_str());
    } else if (key == "block-size" || key == "spmv-block-size") st = want_int(o->block_size);
    else if (key == "wave-size" || key == "wavefront-size") st = want_int(o->wave_size);
    else if (key == "position-block-size") st = want_int(o->position_block_size);
    else if (key == "thread-chunk-size" || key == "spmv-position-chunk-size") st = want_int(o->position_chunk_size);
    else if (key == "spmm-block-size") st = want_int(o->spmm_block_size);
    else if (key == "spmm-tile-size") st = want_int(o->spmm_tile_size);
    else if (key == "spmm-position-chunk-size") st = want_int(o->spmm_position_chunk_size);
    else if (key == "wave-position-batch") st = want_int(o->wave_position_batch);
    else if (key == "accumulate") {
      int64_t v = 0;
      st = want_int(v);
      o->accumulate = v != 0;
    }
    else {
      bool foreign = false;
      for (const ForeignBlockSize &f : kForeign) {
        if (key == f.key) {
          foreign = true;
          int64_t v = 0;
          st = want_int(v);
          if (st == SWB_OK && (v < 1 || v > 1024))
            return fail(ctx, SWB_ERR_INVALID_OPTION, "%s must be between 1 and 1024, but got %lld", f.label, (long long)v);
        }
      }
      if (!foreign) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "unknown option '%s'", key.c_str());
    }
    if (st != SWB_OK) return st;
  }
  return SWB_OK;
}

int swb_options_validate(swb_context *ctx, const swb_options *o) {
  if (!o) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "options is NULL");
  const char *name = spmv_mapping_name(o->mapping);
  if (!name)
    return fail(ctx, SWB_ERR_INVALID_OPTION,
                "unsupported SpMV mapping strategy '%d'; expected 'thread-per-row', 'wave-per-row', or 'block-per-row'",
                o->mapping);
  if (o->spmm_mapping < SWB_THREAD_PER_OUTPUT || o->spmm_mapping > SWB_SPMM_THREAD_PER_POSITION)
    return fail(ctx, SWB_ERR_INVALID_OPTION,
                "unsupported SpMM mapping strategy '%d'; expected 'thread-per-output' or 'wave-per-row-tile'",
                o->spmm_mapping);
  if (o->position_reduction != SWB_REDUCTION_ATOMIC && o->position_reduction != SWB_REDUCTION_SEGMENTED)
    return fail(ctx, SWB_ERR_INVALID_OPTION,
                "unsupported thread position reduction '%d'; expected 'atomic' or 'segmented'", o->position_reduction);

  // schedule-sparsewave-position (SparsePositionScheduling.cpp:411-465); the
  // pipeline feeds it spmv-block-size (Pipelines.cpp:249).
  if (is_position_mapping(o->mapping)) {
    const bool wave = o->mapping == SWB_WAVE_PER_POSITION;
    if (o->block_size < 1 || o->block_size > 1024)
      return fail(ctx, SWB_ERR_INVALID_OPTION, "position block size must be between 1 and 1024, but got %lld", (long long)o->block_size);
    if (wave && o->wave_size != 32)
      return fail(ctx, SWB_ERR_INVALID_OPTION, "wave position mapping currently requires Wave32, but got %lld", (long long)o->wave_size);
    if (wave && o->block_size % o->wave_size != 0)
      return fail(ctx, SWB_ERR_INVALID_OPTION,
                  "wave position mapping requires the block size to be a multiple of %lld, but got %lld",
                  (long long)o->wave_size, (long long)o->block_size);
    if (o->position_chunk_size < 1)
      return fail(ctx, SWB_ERR_INVALID_OPTION, "thread position chunk size must be positive, but got %lld", (long long)o->position_chunk_size);
    if (wave && o->position_chunk_size != 1)
      return fail(ctx, SWB_ERR_INVALID_OPTION, "thread position chunk size applies only to thread mapping");
    if (wave && o->position_reduction != SWB_REDUCTION_ATOMIC)
      return fail(ctx, SWB_ERR_INVALID_OPTION, "thread position reduction applies only to thread mapping");
    if (o->wave_position_batch < 0)
      return fail(ctx, SWB_ERR_INVALID_OPTION, "wave position batch must be non-negative, but got %lld", (long long)o->wave_position_batch);
  }
  if (o->spmm_mapping == SWB_SPMM_THREAD_PER_POSITION) {
    if (o->spmm_block_size < 1 || o->spmm_block_size > 1024)
      return fail(ctx, SWB_ERR_INVALID_OPTION, "position block size must be between 1 and 1024, but got %lld", (long long)o->spmm_block_size);
    if (o->spmm_position_chunk_size < 1)
      return fail(ctx, SWB_ERR_INVALID_OPTION, "thread position chunk size must be positive, but got %lld", (long long)o->spmm_position_chunk_size);
  }

  // convert-sparsewave-to-gpu (SparseWaveToGPU.cpp:1282-1372).
  if (o->block_size < 1 || o->block_size > 1024)
    return fail(ctx, SWB_ERR_INVALID_OPTION, "SpMV block size must be between 1 and 1024, but got %lld", (long long)o->block_size);
  if (o->position_block_size < 1 || o->position_block_size > 1024)
    return fail(ctx, SWB_ERR_INVALID_OPTION, "position-parallel block size must be between 1 and 1024, but got %lld", (long long)o->position_block_size);
  if (o->spmm_block_size < 1 || o->spmm_block_size > 1024)
    return fail(ctx, SWB_ERR_INVALID_OPTION, "SpMM block size must be between 1 and 1024, but got %lld", (long long)o->spmm_block_size);
  if (o->spmm_tile_size < 1 || o->spmm_tile_size > 32)
    return fail(ctx, SWB_ERR_INVALID_OPTION, "SpMM tile size must be between 1 and 32, but got %lld", (long long)o->spmm_tile_size);
  if (o->spmm_mapping == SWB_WAVE_PER_ROW_TILE && o->wave_size != 32)
    return fail(ctx, SWB_ERR_INVALID_OPTION, "wave-per-row-tile currently requires Wave32, but got wave size %lld", (long long)o->wave_size);
  if (o->spmm_mapping == SWB_WAVE_PER_ROW_TILE && o->spmm_block_size % o->wave_size != 0)
    return fail(ctx, SWB_ERR_INVALID_OPTION,
                "wave-per-row-tile requires the SpMM block size to be a multiple of %lld, but got %lld",
                (long long)o->wave_size, (long long)o->spmm_block_size);
  const bool cooperative = o->mapping == SWB_WAVE_PER_ROW || o->mapping == SWB_BLOCK_PER_ROW;
  if (cooperative && o->wave_size != 32)
    return fail(ctx, SWB_ERR_INVALID_OPTION, "%s currently requires Wave32, but got wave size %lld", name, (long long)o->wave_size);
  if (cooperative && o->block_size % o->wave_size != 0)
    return fail(ctx, SWB_ERR_INVALID_OPTION, "%s requires the SpMV block size to be a multiple of %lld, but got %lld",
                name, (long long)o->wave_size, (long long)o->block_size);
  return SWB_OK;
}

// ---- index helpers -----------------------------------------------------------

void swb_partition(int64_t lower, int64_t upper, int64_t worker, int64_t count, int64_t *b, int64_t *e) {
  int64_t bb, ee;
  swb::partition(lower, upper, worker, count, bb, ee);
  if (b) *b = bb;
  if (e) *e = ee;
}

void swb_chunk_bounds(int64_t lower, int64_t upper, int64_t worker, int64_t factor, int64_t *b, int64_t *e) {
  int64_t bb, ee;
  swb::chunk_bounds(lower, upper, worker, factor, bb, ee);
  if (b) *b = bb;
  if (e) *e = ee;
}

int64_t swb_row_at_position(const int32_t *row_ptr, int64_t len, int64_t position) {
  return swb::row_at_position(row_ptr, len, position);
}

int swb_launch_shape_query(swb_context *ctx, const swb_options *o, int64_t rows, int64_t nnz,
                           int64_t n_rhs, swb_launch_shape *out) {
  if (!out) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "out is NULL");
  int st = swb_options_validate(ctx, o);
  if (st != SWB_OK) return st;
  swb::DeviceInfo dev;
  if (ctx) dev = ctx->dev;
  swb_launch_shape r = {0, 0, 0, 1, 0};
  using swb::ceil_div;
  using swb::max1;
  if (n_rhs == 0) {
    const int64_t B = o->block_size;
    r.logical_block = B;
    switch (o->mapping) {
      case SWB_THREAD_PER_ROW:
        r.work_units = rows;
        r.logical_grid = max1(ceil_div(rows, B));
        r.physical_grid = r.logical_grid;
        break;
      case SWB_WAVE_PER_ROW:
        r.work_units = rows;
        r.logical_grid = max1(ceil_div(rows, B / 32));
        r.physical_grid = r.logical_grid;
        break;
      case SWB_BLOCK_PER_ROW:
        r.work_units = rows;
        r.logical_grid = max1(rows);
        r.physical_grid = r.logical_grid;
        break;
      case SWB_THREAD_PER_POSITION:
        r.work_units = ceil_div(nnz, o->position_chunk_size);
        r.logical_grid = max1(ceil_div(r.work_units, B));
        r.physical_grid = r.logical_grid;
        r.kernels = 2;
        break;
      case SWB_WAVE_PER_POSITION: {
        r.work_units = swb::wave_position_wave_count(nnz, B);
        r.logical_grid = max1(ceil_div(nnz, B));
        int64_t batch = o->wave_position_batch > 0 ? o->wave_position_batch
                                                   : swb::wave_per_position_auto_batch(nnz, (int)B, dev);
        r.physical_grid = swb::wave_per_position_physical_grid(nnz, (int)B, batch);
        r.kernels = 2;
        break;
      }
    }
  } else {
    const int64_t B = o->spmm_block_size;
    r.logical_block = B;
    switch (o->spmm_mapping) {
      case SWB_THREAD_PER_OUTPUT:
        r.work_units = rows * n_rhs;
        r.logical_grid = max1(ceil_div(r.work_units, B));
        break;
      case SWB_WAVE_PER_ROW_TILE:
        r.work_units = rows * ceil_div(n_rhs, o->spmm_tile_size);
        r.logical_grid = max1(ceil_div(r.work_units, B / 32));
        break;
      case SWB_SPMM_THREAD_PER_POSITION:
        r.work_units = ceil_div(nnz * n_rhs, o->spmm_position_chunk_size);
        r.logical_grid = max1(ceil_div(r.work_units, B));
        r.kernels = 2;
        break;
    }
    r.physical_grid = r.logical_grid;
    if (o->spmm_mapping == SWB_WAVE_PER_ROW_TILE)  // rows of B of 4 ... 128 floats: the tiles of a row are fused
      r.physical_grid = swb::wave_per_row_tile_physical_grid(rows, nnz, n_rhs, (int)B, (int)o->spmm_tile_size);
  }
  if (r.physical_grid > swb::kMaxGridX)
    return fail(ctx, SWB_ERR_UNSUPPORTED,
                "the launch needs %lld blocks, more than a CUDA grid holds (%lld); use a larger block or tile size",
                (long long)r.physical_grid, (long long)swb::kMaxGridX);
  *out = r;
  return SWB_OK;
}

// ---- operators ----------------------------------------------------------------

static int spmv_impl(swb_context *ctx, const swb_options *o, int64_t rows, int64_t cols, int64_t nnz,
                     const int32_t *row_ptr, const int32_t *col_idx, const float *val, const float *x,
                     float *y, const swb::PositionTrace &trace, cudaStream_t stream) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  st = swb_options_validate(ctx, o);
  if (st != SWB_OK) return st;
  st = check_csr_sizes(ctx, "spmv", rows, cols, nnz);
  if (st != SWB_OK) return st;
  if (!row_ptr || (nnz > 0 && (!col_idx || !val)) || (cols > 0 && !x) || (rows > 0 && !y))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "spmv: NULL operand pointer");
  if (trace.enabled() && !is_position_mapping(o->mapping))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "position trace requires a position mapping");
  // The position kernels step through positions in 32-bit chunks of up to 4096 past the end.
  if (is_position_mapping(o->mapping) && nnz > kI32Max - 65536)
    return fail(ctx, SWB_ERR_UNSUPPORTED, "position mappings support at most %lld nonzeros, but got %lld",
                (long long)(kI32Max - 65536), (long long)nnz);
  if (o->accumulate && !is_position_mapping(o->mapping))
    return fail(ctx, SWB_ERR_UNSUPPORTED, "accumulate is available for the position mappings of SpMV only");
  swb::CsrSpmvArgs a{rows, cols, nnz, row_ptr, col_idx, val, x, y};
  a.accumulate = o->accumulate != 0;
  a.behind_exchange = ctx->behind_exchange && a.accumulate;
  ctx->behind_exchange = false;
  const int B = (int)o->block_size;
  cudaError_t e = cudaSuccess;
  switch (o->mapping) {
    case SWB_THREAD_PER_ROW: e = swb::launch_spmv_thread_per_row(a, B, stream, &ctx->launches); break;
    case SWB_WAVE_PER_ROW: e = swb::launch_spmv_wave_per_row(a, B, stream, &ctx->launches); break;
    case SWB_BLOCK_PER_ROW: e = swb::launch_spmv_block_per_row(a, B, stream, &ctx->launches); break;
    case SWB_THREAD_PER_POSITION:
      e = swb::launch_spmv_thread_per_position(a, B, o->position_chunk_size,
                                               o->position_reduction == SWB_REDUCTION_SEGMENTED, trace,
                                               stream, &ctx->launches);
      break;
    case SWB_WAVE_PER_POSITION: {
      int64_t batch = o->wave_position_batch > 0 ? o->wave_position_batch
                                                 : swb::wave_per_position_auto_batch(nnz, B, ctx->dev);
      // Automatic batch on a large matrix: long rows can go through shared-memory bands of x.  The scratch
      // memory is allocated by the first call that needs it (make that call outside stream capture).
      swb::BandPlan plan;
      // Opt-in: SWB_BAND_MIN_NNZ = nonzeros from which the path is taken (unset or 0: never; on a 92 M-nonzero
      // power-law matrix it is correct but 8 % slower than the span kernel alone).
      const int64_t band_min_nnz = env_i64_or_zero("SWB_BAND_MIN_NNZ", 0);
      const bool banded = o->wave_position_batch == 0 && !trace.enabled() && band_min_nnz > 0 &&
                          swb::band_path_plan(a, band_min_nnz, &plan);
      if (banded) {
        const size_t need = swb::band_scratch_bytes(plan);
        if (need > ctx->band_scratch_bytes) {
          if (ctx->band_scratch) cudaFree(ctx->band_scratch);
          ctx->band_scratch = nullptr;
          ctx->band_scratch_bytes = 0;
          cudaError_t me = cudaMalloc(&ctx->band_scratch, need);
          if (me != cudaSuccess) return cuda_fail(ctx, me, "cudaMalloc(long-row scratch)");
          ctx->band_scratch_bytes = need;
        }
      }
      e = swb::launch_spmv_wave_per_position(a, B, batch, trace, stream, &ctx->launches, nullptr,
                                             banded ? &plan : nullptr, banded ? ctx->band_scratch : nullptr, ctx->dev);
      break;
    }
  }
  if (e != cudaSuccess) return cuda_fail(ctx, e, "spmv launch");
  return SWB_OK;
}

int swb_spmv(swb_context *ctx, const swb_options *o, int64_t rows, int64_t cols, int64_t nnz,
             const int32_t *row_ptr, const int32_t *col_idx, const float *val, const float *x, float *y,
             swb_stream stream) {
  return spmv_impl(ctx, o, rows, cols, nnz, row_ptr, col_idx, val, x, y, swb::PositionTrace(),
                   static_cast<cudaStream_t>(stream));
}

int swb_probe_stream_gather(swb_context *ctx, int64_t nnz, const int32_t *col_idx, const float *val, const float *x,
                            float *sink, swb_stream stream) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  if (nnz < 0 || !col_idx || !val || !x || !sink)
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "gather probe: NULL pointer or negative size");
  cudaError_t e = swb::launch_stream_gather_probe(nnz, col_idx, val, x, sink, ctx->dev, static_cast<cudaStream_t>(stream),
                                                  &ctx->launches);
  if (e == cudaErrorMisalignedAddress)
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "gather probe: col_idx and val must be 16-byte aligned");
  if (e != cudaSuccess) return cuda_fail(ctx, e, "gather probe launch");
  return SWB_OK;
}

int swb_coo_spmv(swb_context *ctx, const swb_options *o, int64_t rows, int64_t cols, int64_t nnz,
                 const int32_t *row_idx, const int32_t *col_idx, const float *val, const float *x, float *y,
                 swb_stream stream) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  st = swb_options_validate(ctx, o);
  if (st != SWB_OK) return st;
  if (rows < 0 || cols < 0 || nnz < 0)
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "coo_spmv: rows, cols and nnz must be non-negative");
  // i32 coordinates (benchmark/benchmark_utils.py:214-223)
  if (rows > kI32Max || cols > kI32Max || nnz > kI32Max)
    return fail(ctx, SWB_ERR_INVALID_SHAPE, "coo_spmv: matrix dimensions and NNZ must fit in the i32 COO type");
  if ((nnz > 0 && (!row_idx || !col_idx || !val)) || (cols > 0 && !x) || (rows > 0 && !y))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "coo_spmv: NULL operand pointer");
  cudaError_t e = swb::launch_coo_spmv_thread_per_nonzero(rows, nnz, row_idx, col_idx, val, x, y,
                                                          (int)o->block_size, static_cast<cudaStream_t>(stream),
                                                          &ctx->launches);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "coo_spmv launch");
  return SWB_OK;
}

int swb_spmv_position_trace(swb_context *ctx, const swb_options *o, int64_t rows, int64_t cols, int64_t nnz,
                            const int32_t *row_ptr, const int32_t *col_idx, const float *val, const float *x,
                            float *y, int32_t *row_of_position, int32_t *worker_of_position,
                            int32_t *segment_end, swb_stream stream) {
  if (!ctx) return fail(nullptr, SWB_ERR_INVALID_ARGUMENT, "context is NULL");
  if (nnz > 0 && (!row_of_position || !worker_of_position || !segment_end))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "position trace: NULL trace pointer");
  swb::PositionTrace t;
  t.row_of_position = row_of_position;
  t.worker_of_position = worker_of_position;
  t.segment_end = segment_end;
  if (nnz > 0) {
    int st = check_ctx(ctx);
    if (st != SWB_OK) return st;
    SWB_CUDA(ctx, cudaMemsetAsync(segment_end, 0, (size_t)nnz * sizeof(int32_t), static_cast<cudaStream_t>(stream)));
  }
  return spmv_impl(ctx, o, rows, cols, nnz, row_ptr, col_idx, val, x, y, t, static_cast<cudaStream_t>(stream));
}

int swb_spmm(swb_context *ctx, const swb_options *o, int64_t rows, int64_t cols, int64_t nnz, int64_t n_rhs,
             const int32_t *row_ptr, const int32_t *col_idx, const float *val, const float *B, float *C,
             swb_stream stream) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  st = swb_options_validate(ctx, o);
  if (st != SWB_OK) return st;
  st = check_csr_sizes(ctx, "spmm", rows, cols, nnz);
  if (st != SWB_OK) return st;
  // The reference loaders require at least one right-hand-side column
  // (SparseBenchmarkUtils.cpp:262-263).
  if (n_rhs < 1) return fail(ctx, SWB_ERR_INVALID_SHAPE, "spmm: right-hand side must have at least one column, but got %lld", (long long)n_rhs);
  if (!row_ptr || (nnz > 0 && (!col_idx || !val)) || (cols > 0 && !B) || (rows > 0 && !C))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "spmm: NULL operand pointer");
  if (o->accumulate && o->spmm_mapping == SWB_THREAD_PER_OUTPUT)
    return fail(ctx, SWB_ERR_UNSUPPORTED, "accumulate is not available for the thread-per-output SpMM mapping");
  // The kernels step through a row's positions in 32-bit strides of up to 128 past its end.
  if (nnz > kI32Max - 256)
    return fail(ctx, SWB_ERR_UNSUPPORTED, "spmm: at most %lld nonzeros are supported, but got %lld",
                (long long)(kI32Max - 256), (long long)nnz);
  swb_launch_shape shape;
  st = swb_launch_shape_query(ctx, o, rows, nnz, n_rhs, &shape);  // refuses grids beyond the CUDA limit
  if (st != SWB_OK) return st;
  swb::CsrSpmmArgs a{rows, cols, nnz, n_rhs, row_ptr, col_idx, val, B, C};
  a.accumulate = o->accumulate != 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int Bs = (int)o->spmm_block_size;
  cudaError_t e = cudaSuccess;
  switch (o->spmm_mapping) {
    case SWB_THREAD_PER_OUTPUT: e = swb::launch_spmm_thread_per_output(a, Bs, s, &ctx->launches); break;
    case SWB_WAVE_PER_ROW_TILE:
      // Opt-in (SWB_SPMM_STAGED=1): the rows of B around the diagonal staged in shared memory by TMA, for
      // banded matrices.  Measured on a banded-plus-random matrix it does not beat the fused-row kernel (the
      // random half of the nonzeros keeps the step DRAM-bound), so it is not the default.
      if (env_i64_or_zero("SWB_SPMM_STAGED", 0) > 0 && swb::spmm_staged_supported(a))
        e = swb::launch_spmm_row_block_staged(a, ctx->status_flag, s, &ctx->launches);
      else
        e = swb::launch_spmm_wave_per_row_tile(a, Bs, (int)o->spmm_tile_size, s, &ctx->launches);
      break;
    case SWB_SPMM_THREAD_PER_POSITION:
      e = swb::launch_spmm_thread_per_position(a, Bs, o->spmm_position_chunk_size, s, &ctx->launches);
      break;
  }
  if (e != cudaSuccess) return cuda_fail(ctx, e, "spmm launch");
  return SWB_OK;
}

static int check_bsr(swb_context *ctx, int64_t rows, int64_t cols, int64_t nnzb, int64_t bs, int64_t n_rhs) {
  if (rows < 0 || cols < 0 || nnzb < 0)
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "bsr_spmm: rows, cols and nnzb must be non-negative");
  // verifyBSRStorage / BSRSpMMOp::verify (SparseWaveOps.cpp:144-207, 340-372)
  if (bs <= 0) return fail(ctx, SWB_ERR_INVALID_SHAPE, "block size must be positive, but got %lld", (long long)bs);
  if (rows % bs != 0)
    return fail(ctx, SWB_ERR_INVALID_SHAPE, "output rows must be divisible by block size, but got %lld and %lld", (long long)rows, (long long)bs);
  if (cols % bs != 0)
    return fail(ctx, SWB_ERR_INVALID_SHAPE, "right-hand-side rows must be divisible by block size, but got %lld and %lld", (long long)cols, (long long)bs);
  if (rows > kI32Max || cols > kI32Max || nnzb > kI32Max)
    return fail(ctx, SWB_ERR_INVALID_SHAPE, "BSR dimensions and NNZ blocks must fit in i32");
  if (n_rhs < 1) return fail(ctx, SWB_ERR_INVALID_SHAPE, "bsr_spmm: right-hand side must have at least one column, but got %lld", (long long)n_rhs);
  return SWB_OK;
}

int swb_bsr_spmm_f32(swb_context *ctx, const swb_options *o, int64_t rows, int64_t cols, int64_t nnzb,
                     int64_t bs, int64_t n_rhs, const int32_t *brp, const int32_t *bci, const float *bv,
                     const float *B, float *C, swb_stream stream) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  st = swb_options_validate(ctx, o);
  if (st != SWB_OK) return st;
  st = check_bsr(ctx, rows, cols, nnzb, bs, n_rhs);
  if (st != SWB_OK) return st;
  if (!brp || (nnzb > 0 && (!bci || !bv)) || (cols > 0 && !B) || (rows > 0 && !C))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "bsr_spmm: NULL operand pointer");
  swb::BsrSpmmArgs a{rows, cols, nnzb, bs, n_rhs, brp, bci, bv, B, C};
  cudaError_t e = swb::launch_bsr_spmm_thread_per_output_f32(a, (int)o->spmm_block_size,
                                                             static_cast<cudaStream_t>(stream), &ctx->launches);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "bsr_spmm launch");
  return SWB_OK;
}

int swb_bsr_spmm_bf16(swb_context *ctx, const swb_options *o, int64_t rows, int64_t cols, int64_t nnzb,
                      int64_t bs, int64_t n_rhs, const int32_t *brp, const int32_t *bci, const uint16_t *bv,
                      const uint16_t *B, uint16_t *C, swb_stream stream) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  st = swb_options_validate(ctx, o);
  if (st != SWB_OK) return st;
  st = check_bsr(ctx, rows, cols, nnzb, bs, n_rhs);
  if (st != SWB_OK) return st;
  if (!brp || (nnzb > 0 && (!bci || !bv)) || (cols > 0 && !B) || (rows > 0 && !C))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "bsr_spmm: NULL operand pointer");
  swb::BsrSpmmArgs a{rows, cols, nnzb, bs, n_rhs, brp, bci, bv, B, C};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  if (swb::bsr16_tcgen05_supported(a))
    e = swb::launch_bsr16_spmm_tcgen05(a, ctx->status_flag, ctx->dev, s, &ctx->launches);
  else
    e = swb::launch_bsr_spmm_thread_per_output_bf16(a, (int)o->spmm_block_size, s, &ctx->launches);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "bsr_spmm launch");
  return SWB_OK;
}

// ---- host-buffer entry points -----------------------------------------------------

int swb_check_csr_host(swb_context *ctx, int64_t rows, int64_t cols, int64_t nnz, const int32_t *row_ptr,
                       const int32_t *col_idx) {
  int st = check_csr_sizes(ctx, "csr", rows, cols, nnz);
  if (st != SWB_OK) return st;
  if (!row_ptr || (nnz > 0 && !col_idx)) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "csr: NULL operand pointer");
  if (row_ptr[0] != 0) return fail(ctx, SWB_ERR_INVALID_DATA, "row offsets must start at 0, but got %d", row_ptr[0]);
  for (int64_t r = 0; r < rows; ++r)
    if (row_ptr[r + 1] < row_ptr[r])
      return fail(ctx, SWB_ERR_INVALID_DATA, "row offsets must be non-decreasing, but row %lld has %d > %d",
                  (long long)r, row_ptr[r], row_ptr[r + 1]);
  if (row_ptr[rows] != nnz)
    return fail(ctx, SWB_ERR_INVALID_DATA, "last row offset must equal NNZ, but got %d and %lld", row_ptr[rows], (long long)nnz);
  for (int64_t p = 0; p < nnz; ++p)
    if (col_idx[p] < 0 || col_idx[p] >= cols)
      return fail(ctx, SWB_ERR_INVALID_DATA, "column index %d at position %lld is out of bounds for %lld columns",
                  col_idx[p], (long long)p, (long long)cols);
  return SWB_OK;
}

// The host-buffer calls treat the caller's result buffer as write-only (it is never copied to the
// device), so there is nothing for `accumulate` to add to.
static int reject_host_accumulate(swb_context *ctx, const swb_options *o) {
  if (o && o->accumulate)
    return fail(ctx, SWB_ERR_UNSUPPORTED,
                "accumulate is not available for the host-buffer calls: their result buffer is write-only");
  return SWB_OK;
}

int swb_spmv_host(swb_context *ctx, const swb_options *o, int64_t rows, int64_t cols, int64_t nnz,
                  const int32_t *row_ptr, const int32_t *col_idx, const float *val, const float *x, float *y) {
  int st = reject_host_accumulate(ctx, o);
  if (st != SWB_OK) return st;
  st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  st = check_csr_sizes(ctx, "spmv", rows, cols, nnz);
  if (st != SWB_OK) return st;
  if (!row_ptr || (nnz > 0 && (!col_idx || !val)) || (cols > 0 && !x) || (rows > 0 && !y))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "spmv: NULL operand pointer");
  st = ensure_host_stream(ctx);
  if (st != SWB_OK) return st;
  size_t need = pad256((rows + 1) * 4) + 2 * pad256(nnz * 4) + pad256(cols * 4) + pad256(rows * 4);
  st = workspace_reserve(ctx, need);
  if (st != SWB_OK) return st;
  int32_t *d_rp = workspace_take<int32_t>(ctx, rows + 1);
  int32_t *d_ci = workspace_take<int32_t>(ctx, nnz);
  float *d_v = workspace_take<float>(ctx, nnz);
  float *d_x = workspace_take<float>(ctx, cols);
  float *d_y = workspace_take<float>(ctx, rows);
  cudaStream_t s = ctx->host_stream;
  SWB_CUDA(ctx, cudaMemcpyAsync(d_rp, row_ptr, (rows + 1) * 4, cudaMemcpyHostToDevice, s));
  if (nnz > 0) {
    SWB_CUDA(ctx, cudaMemcpyAsync(d_ci, col_idx, nnz * 4, cudaMemcpyHostToDevice, s));
    SWB_CUDA(ctx, cudaMemcpyAsync(d_v, val, nnz * 4, cudaMemcpyHostToDevice, s));
  }
  if (cols > 0) SWB_CUDA(ctx, cudaMemcpyAsync(d_x, x, cols * 4, cudaMemcpyHostToDevice, s));
  st = swb_spmv(ctx, o, rows, cols, nnz, d_rp, d_ci, d_v, d_x, d_y, s);
  if (st != SWB_OK) return st;
  if (rows > 0) SWB_CUDA(ctx, cudaMemcpyAsync(y, d_y, rows * 4, cudaMemcpyDeviceToHost, s));
  SWB_CUDA(ctx, cudaStreamSynchronize(s));
  return SWB_OK;
}

int swb_spmm_host(swb_context *ctx, const swb_options *o, int64_t rows, int64_t cols, int64_t nnz, int64_t n_rhs,
                  const int32_t *row_ptr, const int32_t *col_idx, const float *val, const float *B, float *C) {
  int st = reject_host_accumulate(ctx, o);
  if (st != SWB_OK) return st;
  st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  st = check_csr_sizes(ctx, "spmm", rows, cols, nnz);
  if (st != SWB_OK) return st;
  if (n_rhs < 1) return fail(ctx, SWB_ERR_INVALID_SHAPE, "spmm: right-hand side must have at least one column, but got %lld", (long long)n_rhs);
  if (!row_ptr || (nnz > 0 && (!col_idx || !val)) || (cols > 0 && !B) || (rows > 0 && !C))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "spmm: NULL operand pointer");
  st = ensure_host_stream(ctx);
  if (st != SWB_OK) return st;
  size_t need = pad256((rows + 1) * 4) + 2 * pad256(nnz * 4) + pad256(cols * n_rhs * 4) + pad256(rows * n_rhs * 4);
  st = workspace_reserve(ctx, need);
  if (st != SWB_OK) return st;
  int32_t *d_rp = workspace_take<int32_t>(ctx, rows + 1);
  int32_t *d_ci = workspace_take<int32_t>(ctx, nnz);
  float *d_v = workspace_take<float>(ctx, nnz);
  float *d_B = workspace_take<float>(ctx, cols * n_rhs);
  float *d_C = workspace_take<float>(ctx, rows * n_rhs);
  cudaStream_t s = ctx->host_stream;
  SWB_CUDA(ctx, cudaMemcpyAsync(d_rp, row_ptr, (rows + 1) * 4, cudaMemcpyHostToDevice, s));
  if (nnz > 0) {
    SWB_CUDA(ctx, cudaMemcpyAsync(d_ci, col_idx, nnz * 4, cudaMemcpyHostToDevice, s));
    SWB_CUDA(ctx, cudaMemcpyAsync(d_v, val, nnz * 4, cudaMemcpyHostToDevice, s));
  }
  if (cols > 0) SWB_CUDA(ctx, cudaMemcpyAsync(d_B, B, cols * n_rhs * 4, cudaMemcpyHostToDevice, s));
  st = swb_spmm(ctx, o, rows, cols, nnz, n_rhs, d_rp, d_ci, d_v, d_B, d_C, s);
  if (st != SWB_OK) return st;
  if (rows > 0) SWB_CUDA(ctx, cudaMemcpyAsync(C, d_C, rows * n_rhs * 4, cudaMemcpyDeviceToHost, s));
  SWB_CUDA(ctx, cudaStreamSynchronize(s));
  return SWB_OK;
}

int swb_bsr_spmm_bf16_host(swb_context *ctx, const swb_options *o, int64_t rows, int64_t cols, int64_t nnzb,
                           int64_t bs, int64_t n_rhs, const int32_t *brp, const int32_t *bci,
                           const uint16_t *bv, const uint16_t *B, uint16_t *C) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  st = check_bsr(ctx, rows, cols, nnzb, bs, n_rhs);
  if (st != SWB_OK) return st;
  if (!brp || (nnzb > 0 && (!bci || !bv)) || (cols > 0 && !B) || (rows > 0 && !C))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "bsr_spmm: NULL operand pointer");
  st = ensure_host_stream(ctx);
  if (st != SWB_OK) return st;
  const int64_t brows = rows / bs;
  size_t need = pad256((brows + 1) * 4) + pad256(nnzb * 4) + pad256(nnzb * bs * bs * 2) +
                pad256(cols * n_rhs * 2) + pad256(rows * n_rhs * 2);
  st = workspace_reserve(ctx, need);
  if (st != SWB_OK) return st;
  int32_t *d_rp = workspace_take<int32_t>(ctx, brows + 1);
  int32_t *d_ci = workspace_take<int32_t>(ctx, nnzb);
  uint16_t *d_v = workspace_take<uint16_t>(ctx, nnzb * bs * bs);
  uint16_t *d_B = workspace_take<uint16_t>(ctx, cols * n_rhs);
  uint16_t *d_C = workspace_take<uint16_t>(ctx, rows * n_rhs);
  cudaStream_t s = ctx->host_stream;
  SWB_CUDA(ctx, cudaMemcpyAsync(d_rp, brp, (brows + 1) * 4, cudaMemcpyHostToDevice, s));
  if (nnzb > 0) {
    SWB_CUDA(ctx, cudaMemcpyAsync(d_ci, bci, nnzb * 4, cudaMemcpyHostToDevice, s));
    SWB_CUDA(ctx, cudaMemcpyAsync(d_v, bv, nnzb * bs * bs * 2, cudaMemcpyHostToDevice, s));
  }
  if (cols > 0) SWB_CUDA(ctx, cudaMemcpyAsync(d_B, B, cols * n_rhs * 2, cudaMemcpyHostToDevice, s));
  st = swb_bsr_spmm_bf16(ctx, o, rows, cols, nnzb, bs, n_rhs, d_rp, d_ci, d_v, d_B, d_C, s);
  if (st != SWB_OK) return st;
  if (rows > 0) SWB_CUDA(ctx, cudaMemcpyAsync(C, d_C, rows * n_rhs * 2, cudaMemcpyDeviceToHost, s));
  SWB_CUDA(ctx, cudaStreamSynchronize(s));
  return SWB_OK;
}

// ---- device-resident matrices, host dense operands ------------------------------------

// Row panels of a resident matrix.  The host calls below copy the result back to the host while later
// rows are still being computed: the rows are cut into up to 8 contiguous panels of about equal nnz, each
// panel is launched as a CSR problem of its own (its row offsets rebased to zero and stored once at upload,
// its slice of col/val, the whole dense operand, its rows of the output) and its rows of the result start
// their device-to-host copy on a second stream as soon as its kernels are done.  A panel starts at a row
// whose first position is a multiple of 4 (of 32 where one is near), so the col/val slices keep the
// 16-byte alignment the vectorised kernels ask for.  Environment: SWB_RESIDENT_PANEL_NNZ (nnz per panel
// that makes a matrix worth cutting, default 20000000) and SWB_RESIDENT_PANEL_BYTES (result bytes per
// panel below which a call runs uncut, default 524288), both read at upload.
constexpr int kMaxPanels = 8;

// Column parts.  A large matrix is also stored as two matrices over the same rows, one with the entries
// whose column lies below a cut (36 % of the columns by default) and one with the rest.  A call on a mapping that can accumulate then sends
// the first half of the dense operand, runs the first matrix while the second half is still on its way,
// and adds the second matrix (cut into row panels, as above) on top.  SWB_RESIDENT_SPLIT_NNZ: nnz from
// which a matrix is stored this way (default 40000000; it doubles the matrix's device memory).
struct CsrPart {
  int64_t nnz = 0;
  int32_t *row_ptr = nullptr, *col_idx = nullptr;
  float *val = nullptr;
  int panels = 1;
  int64_t panel_row[kMaxPanels + 1] = {};     // first row of each panel, then rows
  int64_t panel_pos[kMaxPanels + 1] = {};     // row_ptr[panel_row[k]]
  int64_t panel_rp_off[kMaxPanels] = {};      // start of panel k's rebased row offsets inside panel_row_ptr
  int32_t *panel_row_ptr = nullptr;           // device
};

struct swb_csr_handle {
  int64_t rows = 0, cols = 0, nnz = 0;
  int64_t panel_min_bytes = 0;
  CsrPart whole;
  bool split = false;
  int64_t split_col = 0;
  CsrPart low, high;  // columns [0, split_col) and [split_col, cols)
};

namespace {

// Panel boundaries on the host: boundary k is the first row at or after the nnz-balanced cut whose first
// position is aligned, looked for in a bounded window; a cut without one, or one that repeats the
// previous boundary, is dropped.
int plan_panels(int64_t rows, int64_t nnz, const int32_t *row_ptr, int64_t panel_nnz, int64_t *panel_row) {
  int64_t want = nnz / panel_nnz;
  if (want > kMaxPanels) want = kMaxPanels;
  panel_row[0] = 0;
  int count = 0;
  for (int64_t k = 1; k < want; ++k) {
    const int64_t target = (int64_t)((__int128)nnz * k / want);
    int64_t lo = 0, hi = rows;  // first row with row_ptr[row] >= target
    while (lo < hi) {
      const int64_t mid = lo + (hi - lo) / 2;
      if (row_ptr[mid] < target) lo = mid + 1; else hi = mid;
    }
    const int64_t window = lo + 4096 < rows ? lo + 4096 : rows;
    int64_t pick = -1;
    for (int64_t r = lo; r < window; ++r)
      if (row_ptr[r] % 32 == 0) { pick = r; break; }
    for (int64_t r = lo; pick < 0 && r < window; ++r)
      if (row_ptr[r] % 4 == 0) pick = r;
    if (pick <= panel_row[count] || pick >= rows) continue;
    panel_row[++count] = pick;
  }
  panel_row[++count] = rows;
  return count;
}

void free_part(CsrPart &p) {
  cudaFree(p.row_ptr); cudaFree(p.col_idx); cudaFree(p.val); cudaFree(p.panel_row_ptr);
  p = CsrPart();
}

// Copies one CSR matrix to the device and, when panel_nnz > 0, plans and stores its row panels.
cudaError_t upload_part(CsrPart &p, int64_t rows, int64_t nnz, const int32_t *row_ptr, const int32_t *col_idx,
                        const float *val, int64_t panel_nnz) {
  p.nnz = nnz;
  p.panel_row[1] = rows;
  p.panel_pos[1] = nnz;
  cudaError_t e = cudaMalloc(&p.row_ptr, (size_t)(rows + 1) * 4);
  if (e == cudaSuccess) e = cudaMalloc(&p.col_idx, (size_t)(nnz > 0 ? nnz : 1) * 4);
  if (e == cudaSuccess) e = cudaMalloc(&p.val, (size_t)(nnz > 0 ? nnz : 1) * 4);
  if (e == cudaSuccess) e = cudaMemcpy(p.row_ptr, row_ptr, (size_t)(rows + 1) * 4, cudaMemcpyHostToDevice);
  if (e == cudaSuccess && nnz > 0) e = cudaMemcpy(p.col_idx, col_idx, (size_t)nnz * 4, cudaMemcpyHostToDevice);
  if (e == cudaSuccess && nnz > 0) e = cudaMemcpy(p.val, val, (size_t)nnz * 4, cudaMemcpyHostToDevice);
  if (e != cudaSuccess || panel_nnz <= 0 || rows <= 0 || nnz <= 0) return e;
  const int count = plan_panels(rows, nnz, row_ptr, panel_nnz, p.panel_row);
  if (count <= 1) return e;
  std::vector<int32_t> rebased;
  for (int k = 0; k < count; ++k) {
    const int64_t r0 = p.panel_row[k], r1 = p.panel_row[k + 1];
    p.panel_pos[k] = row_ptr[r0];
    p.panel_rp_off[k] = (int64_t)rebased.size();
    for (int64_t r = r0; r <= r1; ++r) rebased.push_back(row_ptr[r] - row_ptr[r0]);
    while (rebased.size() % 64) rebased.push_back(0);  // every panel's offsets start 256-byte aligned
  }
  p.panel_pos[count] = nnz;
  e = cudaMalloc(&p.panel_row_ptr, rebased.size() * 4);
  if (e == cudaSuccess) e = cudaMemcpy(p.panel_row_ptr, rebased.data(), rebased.size() * 4, cudaMemcpyHostToDevice);
  if (e == cudaSuccess) p.panels = count;
  return e;
}

}  // namespace

int swb_plan_row_panels(int64_t rows, int64_t nnz, const int32_t *row_ptr, int64_t panel_nnz, int64_t *panel_rows) {
  if (!panel_rows) return 0;
  panel_rows[0] = 0;
  panel_rows[1] = rows > 0 ? rows : 0;
  if (rows <= 0 || nnz <= 0 || !row_ptr || panel_nnz <= 0) return 1;
  return plan_panels(rows, nnz, row_ptr, panel_nnz, panel_rows);
}

// `plain`: one copy of the matrix, no row panels and no column parts (the matrix of a sharded operator).
static int csr_upload_impl(swb_context *ctx, int64_t rows, int64_t cols, int64_t nnz, const int32_t *row_ptr,
                           const int32_t *col_idx, const float *val, bool plain, swb_csr_handle **out) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  if (!out) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "csr upload: out is NULL");
  *out = nullptr;
  st = swb_check_csr_host(ctx, rows, cols, nnz, row_ptr, col_idx);  // content is trusted from here on
  if (st != SWB_OK) return st;
  if (nnz > 0 && !val) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "csr upload: NULL operand pointer");
  swb_csr_handle *h = new swb_csr_handle();
  h->rows = rows; h->cols = cols; h->nnz = nnz;
  h->panel_min_bytes = env_i64("SWB_RESIDENT_PANEL_BYTES", 512 * 1024);
  const int64_t panel_nnz = plain ? 0 : env_i64("SWB_RESIDENT_PANEL_NNZ", 20000000);
  cudaError_t e = upload_part(h->whole, rows, nnz, row_ptr, col_idx, val, panel_nnz);

  if (!plain && e == cudaSuccess && rows > 0 && cols >= 2 && nnz >= env_i64("SWB_RESIDENT_SPLIT_NNZ", 40000000)) {
    // The two column parts, each a CSR matrix over all rows with the entries in their original order.  They
    // are an optimisation: without the host or device memory for them the matrix stays resident uncut.
    // Where the columns are cut: the first part should finish computing about when the rest of the operand
    // has arrived (SWB_RESIDENT_SPLIT_PERCENT of the columns go to the first part; 33 and 40 measured best
    // on a 92 M-nonzero SpMV over PCIe gen 5, 25 and 50 cost 6 % more).
    int64_t percent = env_i64("SWB_RESIDENT_SPLIT_PERCENT", 36);
    if (percent > 90) percent = 90;
    if (percent < 10) percent = 10;
    int64_t mid = (int64_t)((__int128)cols * percent / 100);
    mid -= mid % 4;  // the second part of the operand starts 16-byte aligned
    if (mid < 1) mid = 1;
    try {
      std::vector<int32_t> rp_lo(rows + 1, 0), rp_hi(rows + 1, 0);
      for (int64_t r = 0; r < rows; ++r) {
        int32_t below = 0;
        for (int32_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p) below += col_idx[p] < mid;
        rp_lo[r + 1] = rp_lo[r] + below;
        rp_hi[r + 1] = rp_hi[r] + (row_ptr[r + 1] - row_ptr[r] - below);
      }
      const int64_t nnz_lo = rp_lo[rows], nnz_hi = rp_hi[rows];
      std::vector<int32_t> ci_lo(nnz_lo), ci_hi(nnz_hi);
      std::vector<float> v_lo(nnz_lo), v_hi(nnz_hi);
      for (int64_t r = 0; r < rows; ++r) {
        int64_t a = rp_lo[r], b = rp_hi[r];
        for (int32_t p = row_ptr[r]; p < row_ptr[r + 1]; ++p) {
          if (col_idx[p] < mid) { ci_lo[a] = col_idx[p]; v_lo[a++] = val[p]; }
          else { ci_hi[b] = col_idx[p]; v_hi[b++] = val[p]; }
        }
      }
      cudaError_t es = upload_part(h->low, rows, nnz_lo, rp_lo.data(), ci_lo.data(), v_lo.data(), 0);
      // the second part finishes the result, so it is the one cut into row panels (about as many as the whole)
      if (es == cudaSuccess)
        es = upload_part(h->high, rows, nnz_hi, rp_hi.data(), ci_hi.data(), v_hi.data(), (panel_nnz + 1) / 2);
      if (es == cudaSuccess) {
        h->split = true;
        h->split_col = mid;
      } else {
        cudaGetLastError();  // out of device memory for the second copy: not an error of the upload
      }
    } catch (const std::bad_alloc &) {
      // no host memory for the temporary copies: the matrix stays uncut
    }
    if (!h->split) {
      free_part(h->low);
      free_part(h->high);
    }
  }
  if (e != cudaSuccess) {
    free_part(h->whole); free_part(h->low); free_part(h->high);
    delete h;
    return cuda_fail(ctx, e, "csr upload");
  }
  *out = h;
  return SWB_OK;
}

int swb_csr_upload(swb_context *ctx, int64_t rows, int64_t cols, int64_t nnz, const int32_t *row_ptr,
                   const int32_t *col_idx, const float *val, swb_csr_handle **out) {
  return csr_upload_impl(ctx, rows, cols, nnz, row_ptr, col_idx, val, false, out);
}

int swb_csr_upload_rows(swb_context *ctx, int64_t rows_total, int64_t cols, const int32_t *row_ptr,
                        const int32_t *col_idx, const float *val, int64_t row_begin, int64_t row_end,
                        swb_csr_handle **out) {
  if (!out) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "csr upload: out is NULL");
  *out = nullptr;
  if (!row_ptr || rows_total < 0 || row_begin < 0 || row_end < row_begin || row_end > rows_total)
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "csr upload: rows [%lld, %lld) are not a range of the %lld rows",
                (long long)row_begin, (long long)row_end, (long long)rows_total);
  const int64_t p0 = row_ptr[row_begin], p1 = row_ptr[row_end];
  if (p0 < 0 || p1 < p0)
    return fail(ctx, SWB_ERR_INVALID_DATA, "row offsets must be non-decreasing, but rows %lld and %lld start at %lld and %lld",
                (long long)row_begin, (long long)row_end, (long long)p0, (long long)p1);
  std::vector<int32_t> rebased((size_t)(row_end - row_begin) + 1);
  for (int64_t r = row_begin; r <= row_end; ++r) rebased[(size_t)(r - row_begin)] = (int32_t)(row_ptr[r] - p0);
  return csr_upload_impl(ctx, row_end - row_begin, cols, p1 - p0, rebased.data(), col_idx ? col_idx + p0 : nullptr,
                         val ? val + p0 : nullptr, true, out);
}

void swb_csr_release(swb_context *ctx, swb_csr_handle *h) {
  if (!h) return;
  if (ctx) cudaSetDevice(ctx->device);
  free_part(h->whole); free_part(h->low); free_part(h->high);
  delete h;
}

extern "C++" {
namespace {

// Queues the operator on `part` panel by panel on the host stream; behind each panel its rows of the
// result start their copy to the host on the copy stream.
template <typename Launch>
int run_panels_with_copy(swb_context *ctx, const swb_options *o, const CsrPart &part, int64_t width, float *d_out,
                         float *out_host, cudaError_t &e, Launch &launch) {
  int st = SWB_OK;
  for (int k = 0; k < part.panels && e == cudaSuccess; ++k) {
    const int64_t r0 = part.panel_row[k], r1 = part.panel_row[k + 1], p0 = part.panel_pos[k];
    const int32_t *rp = part.panels > 1 ? part.panel_row_ptr + part.panel_rp_off[k] : part.row_ptr;
    st = launch(o, r1 - r0, part.panel_pos[k + 1] - p0, rp, part.col_idx + p0, part.val + p0, d_out + r0 * width);
    if (st != SWB_OK) break;
    e = cudaEventRecord(ctx->panel_done[k], ctx->host_stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->copy_stream, ctx->panel_done[k], 0);
    if (e == cudaSuccess)
      e = cudaMemcpyAsync(out_host + r0 * width, d_out + r0 * width, (size_t)(r1 - r0) * width * 4,
                          cudaMemcpyDeviceToHost, ctx->copy_stream);
  }
  return st;
}

// Shared body of the two resident host calls.  `width` = floats per row of the dense operand and of the
// result (1 for SpMV); `can_accumulate` = the chosen mapping can add to an existing result;
// `launch(opts, rows, nnz, row_ptr, col, val, out)` queues one operator call on the host stream.
template <typename Launch>
int resident_host_call(swb_context *ctx, const swb_options *o, const swb_csr_handle *h, int64_t width,
                       bool can_accumulate, const float *dense_host, float *out_host, float **d_dense_out,
                       Launch launch) {
  int st = ensure_host_stream(ctx);
  if (st != SWB_OK) return st;
  const size_t dense_bytes = (size_t)h->cols * width * 4, out_bytes = (size_t)h->rows * width * 4;
  st = workspace_reserve(ctx, pad256(dense_bytes) + pad256(out_bytes));
  if (st != SWB_OK) return st;
  float *d_dense = workspace_take<float>(ctx, h->cols * width);
  float *d_out = workspace_take<float>(ctx, h->rows * width);
  *d_dense_out = d_dense;
  cudaStream_t s = ctx->host_stream;
  const bool halves = h->split && can_accumulate && !o->accumulate && out_bytes > 0;
  const CsrPart &last = halves ? h->high : h->whole;
  const bool cut = last.panels > 1 && (int64_t)(out_bytes / last.panels) >= h->panel_min_bytes;
  if (!halves && !cut) {
    if (dense_bytes > 0) SWB_CUDA(ctx, cudaMemcpyAsync(d_dense, dense_host, dense_bytes, cudaMemcpyHostToDevice, s));
    st = launch(o, h->rows, h->nnz, h->whole.row_ptr, h->whole.col_idx, h->whole.val, d_out);
    if (st != SWB_OK) return st;
    if (out_bytes > 0) SWB_CUDA(ctx, cudaMemcpyAsync(out_host, d_out, out_bytes, cudaMemcpyDeviceToHost, s));
    SWB_CUDA(ctx, cudaStreamSynchronize(s));
    return SWB_OK;
  }
  st = ensure_copy_stream(ctx);
  if (st != SWB_OK) return st;
  cudaError_t e = cudaSuccess;
  if (!halves) {
    e = cudaMemcpyAsync(d_dense, dense_host, dense_bytes, cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) st = run_panels_with_copy(ctx, o, h->whole, width, d_out, out_host, e, launch);
  } else {
    // first half of the operand, first matrix; the second half travels meanwhile; second matrix on top
    const size_t first = (size_t)h->split_col * width * 4;
    cudaStream_t up = ctx->upload_stream;
    e = cudaMemcpyAsync(d_dense, dense_host, first, cudaMemcpyHostToDevice, up);
    if (e == cudaSuccess) e = cudaEventRecord(ctx->upload_done[0], up);
    if (e == cudaSuccess)
      e = cudaMemcpyAsync(reinterpret_cast<char *>(d_dense) + first, reinterpret_cast<const char *>(dense_host) + first,
                          dense_bytes - first, cudaMemcpyHostToDevice, up);
    if (e == cudaSuccess) e = cudaEventRecord(ctx->upload_done[1], up);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(s, ctx->upload_done[0], 0);
    if (e == cudaSuccess)
      st = launch(o, h->rows, h->low.nnz, h->low.row_ptr, h->low.col_idx, h->low.val, d_out);
    if (e == cudaSuccess && st == SWB_OK) e = cudaStreamWaitEvent(s, ctx->upload_done[1], 0);
    if (e == cudaSuccess && st == SWB_OK) {
      swb_options add = *o;
      add.accumulate = 1;
      if (cut) {
        st = run_panels_with_copy(ctx, &add, h->high, width, d_out, out_host, e, launch);
      } else {
        st = launch(&add, h->rows, h->high.nnz, h->high.row_ptr, h->high.col_idx, h->high.val, d_out);
        if (st == SWB_OK) e = cudaMemcpyAsync(out_host, d_out, out_bytes, cudaMemcpyDeviceToHost, s);
      }
    }
  }
  // Every stream is drained before returning, also after an error: the copies touch caller memory.
  const cudaError_t e0 = ctx->upload_stream ? cudaStreamSynchronize(ctx->upload_stream) : cudaSuccess;
  const cudaError_t e1 = cudaStreamSynchronize(s), e2 = cudaStreamSynchronize(ctx->copy_stream);
  if (st != SWB_OK) return st;
  if (e == cudaSuccess) e = e0 != cudaSuccess ? e0 : (e1 != cudaSuccess ? e1 : e2);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "resident host call");
  return SWB_OK;
}

}  // namespace
}  // extern "C++"

int swb_spmv_resident_host(swb_context *ctx, const swb_options *o, const swb_csr_handle *h, const float *x, float *y) {
  int st = reject_host_accumulate(ctx, o);
  if (st != SWB_OK) return st;
  st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  if (!o) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "options is NULL");
  if (!h || (h->cols > 0 && !x) || (h->rows > 0 && !y))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "spmv: NULL matrix handle or operand pointer");
  float *d_x = nullptr;
  return resident_host_call(ctx, o, h, 1, is_position_mapping(o->mapping), x, y, &d_x,
                            [&](const swb_options *opts, int64_t rows, int64_t nnz, const int32_t *rp,
                                const int32_t *ci, const float *v, float *d_y) {
                              return swb_spmv(ctx, opts, rows, h->cols, nnz, rp, ci, v, d_x, d_y, ctx->host_stream);
                            });
}

int swb_spmm_resident_host(swb_context *ctx, const swb_options *o, const swb_csr_handle *h, int64_t n_rhs,
                           const float *B, float *C) {
  int st = reject_host_accumulate(ctx, o);
  if (st != SWB_OK) return st;
  st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  if (!o) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "options is NULL");
  if (n_rhs < 1) return fail(ctx, SWB_ERR_INVALID_SHAPE, "spmm: right-hand side must have at least one column, but got %lld", (long long)n_rhs);
  if (!h || (h->cols > 0 && !B) || (h->rows > 0 && !C))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "spmm: NULL matrix handle or operand pointer");
  float *d_B = nullptr;
  return resident_host_call(ctx, o, h, n_rhs, o->spmm_mapping != SWB_THREAD_PER_OUTPUT, B, C, &d_B,
                            [&](const swb_options *opts, int64_t rows, int64_t nnz, const int32_t *rp,
                                const int32_t *ci, const float *v, float *d_C) {
                              return swb_spmm(ctx, opts, rows, h->cols, nnz, n_rhs, rp, ci, v, d_B, d_C,
                                              ctx->host_stream);
                            });
}

// ---- device-resident bf16 BSR matrix, host dense operands ---------------------------------------

struct swb_bsr_handle {
  int64_t rows = 0, cols = 0, nnzb = 0, block_size = 0;
  int32_t *block_row_ptr = nullptr, *block_col_idx = nullptr;
  uint16_t *block_values = nullptr;
};

int swb_bsr_upload(swb_context *ctx, int64_t rows, int64_t cols, int64_t nnzb, int64_t bs, const int32_t *brp,
                   const int32_t *bci, const uint16_t *bv, swb_bsr_handle **out) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  if (!out) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "bsr upload: out is NULL");
  *out = nullptr;
  st = check_bsr(ctx, rows, cols, nnzb, bs, 1);
  if (st != SWB_OK) return st;
  if (!brp || (nnzb > 0 && (!bci || !bv))) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "bsr upload: NULL operand pointer");
  const int64_t brows = rows / bs, bcols = cols / bs;
  if (brp[0] != 0) return fail(ctx, SWB_ERR_INVALID_DATA, "block-row offsets must start at 0, but got %d", brp[0]);
  for (int64_t r = 0; r < brows; ++r)
    if (brp[r + 1] < brp[r])
      return fail(ctx, SWB_ERR_INVALID_DATA, "block-row offsets must be non-decreasing, but block row %lld has %d > %d",
                  (long long)r, brp[r], brp[r + 1]);
  if (brp[brows] != nnzb)
    return fail(ctx, SWB_ERR_INVALID_DATA, "last block-row offset must equal the number of blocks, but got %d and %lld",
                brp[brows], (long long)nnzb);
  for (int64_t b = 0; b < nnzb; ++b)
    if (bci[b] < 0 || bci[b] >= bcols)
      return fail(ctx, SWB_ERR_INVALID_DATA, "block column %d of block %lld is out of bounds for %lld block columns", bci[b],
                  (long long)b, (long long)bcols);
  swb_bsr_handle *h = new swb_bsr_handle();
  h->rows = rows; h->cols = cols; h->nnzb = nnzb; h->block_size = bs;
  const size_t value_bytes = (size_t)nnzb * bs * bs * 2;
  cudaError_t e = cudaMalloc(&h->block_row_ptr, (size_t)(brows + 1) * 4);
  if (e == cudaSuccess) e = cudaMalloc(&h->block_col_idx, (size_t)(nnzb > 0 ? nnzb : 1) * 4);
  if (e == cudaSuccess) e = cudaMalloc(&h->block_values, value_bytes > 0 ? value_bytes : 16);
  if (e == cudaSuccess) e = cudaMemcpy(h->block_row_ptr, brp, (size_t)(brows + 1) * 4, cudaMemcpyHostToDevice);
  if (e == cudaSuccess && nnzb > 0) e = cudaMemcpy(h->block_col_idx, bci, (size_t)nnzb * 4, cudaMemcpyHostToDevice);
  if (e == cudaSuccess && nnzb > 0) e = cudaMemcpy(h->block_values, bv, value_bytes, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    swb_bsr_release(ctx, h);
    return cuda_fail(ctx, e, "bsr upload");
  }
  *out = h;
  return SWB_OK;
}

void swb_bsr_release(swb_context *ctx, swb_bsr_handle *h) {
  if (!h) return;
  if (ctx) cudaSetDevice(ctx->device);
  cudaFree(h->block_row_ptr); cudaFree(h->block_col_idx); cudaFree(h->block_values);
  delete h;
}

int swb_bsr_spmm_bf16_resident_host(swb_context *ctx, const swb_options *o, const swb_bsr_handle *h, int64_t n_rhs,
                                    const uint16_t *B, uint16_t *C) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  if (!o) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "options is NULL");
  if (n_rhs < 1) return fail(ctx, SWB_ERR_INVALID_SHAPE, "bsr_spmm: right-hand side must have at least one column, but got %lld", (long long)n_rhs);
  if (!h || (h->cols > 0 && !B) || (h->rows > 0 && !C))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "bsr_spmm: NULL matrix handle or operand pointer");
  st = ensure_host_stream(ctx);
  if (st != SWB_OK) return st;
  const size_t b_bytes = (size_t)h->cols * n_rhs * 2, c_bytes = (size_t)h->rows * n_rhs * 2;
  st = workspace_reserve(ctx, pad256(b_bytes) + pad256(c_bytes));
  if (st != SWB_OK) return st;
  uint16_t *d_B = workspace_take<uint16_t>(ctx, h->cols * n_rhs);
  uint16_t *d_C = workspace_take<uint16_t>(ctx, h->rows * n_rhs);
  cudaStream_t s = ctx->host_stream;
  if (b_bytes > 0) SWB_CUDA(ctx, cudaMemcpyAsync(d_B, B, b_bytes, cudaMemcpyHostToDevice, s));
  st = swb_bsr_spmm_bf16(ctx, o, h->rows, h->cols, h->nnzb, h->block_size, n_rhs, h->block_row_ptr, h->block_col_idx,
                         h->block_values, d_B, d_C, s);
  cudaError_t e = cudaSuccess;
  if (st == SWB_OK && c_bytes > 0) e = cudaMemcpyAsync(C, d_C, c_bytes, cudaMemcpyDeviceToHost, s);
  const cudaError_t e1 = cudaStreamSynchronize(s);  // also after an error: the copies touch caller memory
  if (st != SWB_OK) return st;
  if (e == cudaSuccess) e = e1;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "bsr resident host call");
  return SWB_OK;
}

// ---- sharded operators: gather the dense operand, then the local kernel -----------------------

extern "C++" {
namespace {

int grow(swb_context *ctx, char **buf, size_t *have, size_t need, const char *what) {
  if (need <= *have) return SWB_OK;
  if (*buf) cudaFree(*buf);
  *buf = nullptr;
  *have = 0;
  cudaError_t e = cudaMalloc(buf, need);
  if (e != cudaSuccess) return cuda_fail(ctx, e, what);
  *have = need;
  return SWB_OK;
}

// Every rank's chunk of the dense operand (cols x width floats, ceil(cols / ranks) rows per rank, this
// rank's chunk at `owned`: device memory unless owned_on_host) gathered into one device copy, queued on
// `s`.  The exchange is the peer-store kernel when the context has a window of that chunk size, else
// ncclAllGather on the context's communicator; one rank needs neither.
// `zero` (or NULL): an output vector the consumer wants zero-filled first; the peer-store kernel does it
// on the side and *zero_filled says so.
int gather_dense_operand(swb_context *ctx, const float *owned, bool owned_on_host, int64_t cols, int64_t width,
                         cudaStream_t s, const float **full_out, float *zero = nullptr, int64_t zero_count = 0,
                         bool *zero_filled = nullptr) {
  if (zero_filled) *zero_filled = false;
  const int ranks = ctx->comm ? ctx->comm_ranks : 1, rank = ctx->comm ? ctx->comm_rank : 0;
  const int64_t chunk_rows = swb::ceil_div(cols, ranks);
  int64_t own_begin = (int64_t)rank * chunk_rows, own_end = own_begin + chunk_rows;
  if (own_begin > cols) own_begin = cols;
  if (own_end > cols) own_end = cols;
  const size_t own_bytes = (size_t)(own_end - own_begin) * width * 4, chunk_bytes = (size_t)chunk_rows * width * 4;
  if (own_bytes > 0 && !owned) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "sharded operator: NULL dense operand");
  const bool staged = owned_on_host || own_bytes != chunk_bytes || (reinterpret_cast<uintptr_t>(owned) & 15u) != 0;
  const char *send = reinterpret_cast<const char *>(owned);
  if (staged) {  // padded device copy of the chunk
    int st = grow(ctx, &ctx->shard_send, &ctx->shard_send_bytes, chunk_bytes > 0 ? chunk_bytes : 16, "cudaMalloc(chunk)");
    if (st != SWB_OK) return st;
    if (own_bytes > 0)
      SWB_CUDA(ctx, cudaMemcpyAsync(ctx->shard_send, owned, own_bytes,
                                    owned_on_host ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice, s));
    if (chunk_bytes > own_bytes) SWB_CUDA(ctx, cudaMemsetAsync(ctx->shard_send + own_bytes, 0, chunk_bytes - own_bytes, s));
    send = ctx->shard_send;
  }
  if (ranks == 1) {
    *full_out = reinterpret_cast<const float *>(send);
    return SWB_OK;
  }
  int64_t window_bytes = 0;
  void *window = swb::peer_window_data(ctx, &window_bytes);
  if (window && window_bytes == (int64_t)chunk_bytes && chunk_bytes % 16 == 0) {
    const void *gathered = nullptr;  // the two buffers of the window take turns: no ready-flag round trip
    int st = swb::window_allgather_and_fill(ctx, send, zero, zero_count, s, true, &gathered);
    if (st != SWB_OK) return st;
    if (zero && zero_filled) *zero_filled = true;
    *full_out = static_cast<const float *>(gathered);
    return SWB_OK;
  }
  int st = grow(ctx, &ctx->shard_full, &ctx->shard_full_bytes, chunk_bytes * (size_t)ranks, "cudaMalloc(gathered operand)");
  if (st != SWB_OK) return st;
  st = swb_comm_allgather(ctx, send, ctx->shard_full, (int64_t)chunk_bytes, s);
  if (st != SWB_OK) return st;
  *full_out = reinterpret_cast<const float *>(ctx->shard_full);
  return SWB_OK;
}

}  // namespace
}  // extern "C++"

int swb_spmv_sharded(swb_context *ctx, const swb_options *o, int64_t rows, int64_t cols, int64_t nnz,
                     const int32_t *row_ptr, const int32_t *col_idx, const float *val, const float *x_owned,
                     float *y, swb_stream stream) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  if (cols < 0) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "spmv: rows, cols and nnz must be non-negative");
  if (!o) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "options is NULL");
  const float *x = nullptr;
  // a position mapping starts from a zero-filled y: the exchange kernel fills it while it waits for the peers
  const bool wants_fill = is_position_mapping(o->mapping) && !o->accumulate && rows > 0 && y;
  bool filled = false;
  st = gather_dense_operand(ctx, x_owned, false, cols, 1, static_cast<cudaStream_t>(stream), &x,
                            wants_fill ? y : nullptr, rows, &filled);
  if (st != SWB_OK) return st;
  if (!filled) return swb_spmv(ctx, o, rows, cols, nnz, row_ptr, col_idx, val, x, y, stream);
  swb_options add = *o;
  add.accumulate = 1;
  ctx->behind_exchange = true;  // nothing was queued between the exchange kernel and this call's kernel
  st = swb_spmv(ctx, &add, rows, cols, nnz, row_ptr, col_idx, val, x, y, stream);
  ctx->behind_exchange = false;
  return st;
}

int swb_spmm_sharded(swb_context *ctx, const swb_options *o, int64_t rows, int64_t cols, int64_t nnz, int64_t n_rhs,
                     const int32_t *row_ptr, const int32_t *col_idx, const float *val, const float *B_owned,
                     float *C, swb_stream stream) {
  int st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  if (cols < 0) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "spmm: rows, cols and nnz must be non-negative");
  if (n_rhs < 1) return fail(ctx, SWB_ERR_INVALID_SHAPE, "spmm: right-hand side must have at least one column, but got %lld", (long long)n_rhs);
  const float *B = nullptr;
  st = gather_dense_operand(ctx, B_owned, false, cols, n_rhs, static_cast<cudaStream_t>(stream), &B);
  if (st != SWB_OK) return st;
  return swb_spmm(ctx, o, rows, cols, nnz, n_rhs, row_ptr, col_idx, val, B, C, stream);
}

// Host operands: this rank's chunk in, the exchange on the device, the local kernel, this rank's rows out.
static int sharded_host_call(swb_context *ctx, const swb_options *o, const swb_csr_handle *h, int64_t width,
                             const float *owned_host, float *out_host, bool spmv) {
  int st = reject_host_accumulate(ctx, o);
  if (st != SWB_OK) return st;
  st = check_ctx(ctx);
  if (st != SWB_OK) return st;
  if (!o) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "options is NULL");
  if (!h || (h->rows > 0 && !out_host))
    return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "sharded operator: NULL matrix handle or operand pointer");
  st = ensure_host_stream(ctx);
  if (st != SWB_OK) return st;
  const size_t out_bytes = (size_t)h->rows * width * 4;
  st = workspace_reserve(ctx, pad256(out_bytes));
  if (st != SWB_OK) return st;
  float *d_out = workspace_take<float>(ctx, h->rows * width);
  cudaStream_t s = ctx->host_stream;
  const float *dense = nullptr;
  const bool wants_fill = spmv && is_position_mapping(o->mapping) && h->rows > 0;
  bool filled = false;
  st = gather_dense_operand(ctx, owned_host, true, h->cols, width, s, &dense, wants_fill ? d_out : nullptr, h->rows, &filled);
  swb_options local = *o;
  if (filled) local.accumulate = 1;
  ctx->behind_exchange = filled && spmv;  // the kernel of swb_spmv comes directly behind the exchange kernel
  if (st == SWB_OK)
    st = spmv ? swb_spmv(ctx, &local, h->rows, h->cols, h->nnz, h->whole.row_ptr, h->whole.col_idx, h->whole.val, dense, d_out, s)
              : swb_spmm(ctx, &local, h->rows, h->cols, h->nnz, width, h->whole.row_ptr, h->whole.col_idx, h->whole.val, dense,
                         d_out, s);
  ctx->behind_exchange = false;
  cudaError_t e = cudaSuccess;
  if (st == SWB_OK && out_bytes > 0) e = cudaMemcpyAsync(out_host, d_out, out_bytes, cudaMemcpyDeviceToHost, s);
  const cudaError_t e1 = cudaStreamSynchronize(s);  // also after an error: the copies touch caller memory
  if (st != SWB_OK) return st;
  if (e == cudaSuccess) e = e1;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "sharded host call");
  return SWB_OK;
}

int swb_spmv_sharded_host(swb_context *ctx, const swb_options *o, const swb_csr_handle *h, const float *x_owned,
                          float *y) {
  return sharded_host_call(ctx, o, h, 1, x_owned, y, true);
}

int swb_spmm_sharded_host(swb_context *ctx, const swb_options *o, const swb_csr_handle *h, int64_t n_rhs,
                          const float *B_owned, float *C) {
  if (n_rhs < 1) return fail(ctx, SWB_ERR_INVALID_SHAPE, "spmm: right-hand side must have at least one column, but got %lld", (long long)n_rhs);
  return sharded_host_call(ctx, o, h, n_rhs, B_owned, C, false);
}

// ---- memref-descriptor entry points -------------------------------------------------

static swb_context *process_context() {
  static swb_context *ctx = nullptr;
  if (!ctx) {
    int device = 0;
    cudaGetDevice(&device);
    if (swb_create(&ctx, device) != SWB_OK) {
      fprintf(stderr, "sparsewave_b200: %s\n", swb_last_error(nullptr));
      abort();
    }
  }
  return ctx;
}

static void env_options(swb_context *ctx, swb_options *o) {
  swb_options_default(o);
  const char *text = getenv("SPARSEWAVE_B200_OPTIONS");
  if (text && swb_options_parse(ctx, o, text) != SWB_OK) {
    fprintf(stderr, "sparsewave_b200: %s\n", swb_last_error(ctx));
    abort();
  }
}

int swb_spmv_memref(swb_context *ctx, const swb_options *o, swb_memref_1d_i32 *rp, swb_memref_1d_i32 *ci,
                    swb_memref_1d_f32 *v, swb_memref_1d_f32 *x, swb_memref_1d_f32 *y, swb_stream stream) {
  if (!rp || !ci || !v || !x || !y) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "spmv: NULL memref descriptor");
  if (rp->strides[0] != 1 || ci->strides[0] != 1 || v->strides[0] != 1 || x->strides[0] != 1 || y->strides[0] != 1)
    return fail(ctx, SWB_ERR_INVALID_SHAPE, "spmv: memref has an unexpected layout");
  // SparseWaveOps.cpp:83-108
  if (ci->sizes[0] != v->sizes[0])
    return fail(ctx, SWB_ERR_INVALID_SHAPE,
                "'sparsewave.spmv' op column indices and values must have the same size, but got %lld and %lld",
                (long long)ci->sizes[0], (long long)v->sizes[0]);
  if (rp->sizes[0] != y->sizes[0] + 1)
    return fail(ctx, SWB_ERR_INVALID_SHAPE,
                "'sparsewave.spmv' op row offsets size must equal output size plus one, but got %lld and %lld",
                (long long)rp->sizes[0], (long long)y->sizes[0]);
  return swb_spmv(ctx, o, y->sizes[0], x->sizes[0], v->sizes[0], rp->data + rp->offset, ci->data + ci->offset,
                  v->data + v->offset, x->data + x->offset, y->data + y->offset, stream);
}

static bool identity2d(const swb_memref_2d_f32 *m) { return m->strides[1] == 1 && m->strides[0] == m->sizes[1]; }

int swb_spmm_memref(swb_context *ctx, const swb_options *o, swb_memref_1d_i32 *rp, swb_memref_1d_i32 *ci,
                    swb_memref_1d_f32 *v, swb_memref_2d_f32 *rhs, swb_memref_2d_f32 *out, swb_stream stream) {
  if (!rp || !ci || !v || !rhs || !out) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "spmm: NULL memref descriptor");
  if (rp->strides[0] != 1 || ci->strides[0] != 1 || v->strides[0] != 1)
    return fail(ctx, SWB_ERR_INVALID_SHAPE, "spmm: memref has an unexpected layout");
  if (!identity2d(rhs)) return fail(ctx, SWB_ERR_INVALID_SHAPE, "RHS memref has an unexpected layout");
  if (!identity2d(out)) return fail(ctx, SWB_ERR_INVALID_SHAPE, "output memref has an unexpected layout");
  if (ci->sizes[0] != v->sizes[0])
    return fail(ctx, SWB_ERR_INVALID_SHAPE,
                "'sparsewave.spmm' op column indices and values must have the same size, but got %lld and %lld",
                (long long)ci->sizes[0], (long long)v->sizes[0]);
  if (rp->sizes[0] != out->sizes[0] + 1)
    return fail(ctx, SWB_ERR_INVALID_SHAPE,
                "'sparsewave.spmm' op row offsets size must equal output rows plus one, but got %lld and %lld",
                (long long)rp->sizes[0], (long long)out->sizes[0]);
  if (rhs->sizes[1] != out->sizes[1])
    return fail(ctx, SWB_ERR_INVALID_SHAPE,
                "'sparsewave.spmm' op right-hand side and output must have the same number of columns");
  return swb_spmm(ctx, o, out->sizes[0], rhs->sizes[0], v->sizes[0], out->sizes[1], rp->data + rp->offset,
                  ci->data + ci->offset, v->data + v->offset, rhs->data + rhs->offset, out->data + out->offset,
                  stream);
}

int swb_bsr_spmm_memref(swb_context *ctx, const swb_options *o, swb_memref_1d_i32 *brp, swb_memref_1d_i32 *bci,
                        swb_memref_1d_f32 *bv, swb_memref_2d_f32 *rhs, swb_memref_2d_f32 *out, int64_t bs,
                        swb_stream stream) {
  if (!brp || !bci || !bv || !rhs || !out) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "bsr_spmm: NULL memref descriptor");
  if (brp->strides[0] != 1 || bci->strides[0] != 1 || bv->strides[0] != 1)
    return fail(ctx, SWB_ERR_INVALID_SHAPE, "bsr_spmm: memref has an unexpected layout");
  if (!identity2d(rhs)) return fail(ctx, SWB_ERR_INVALID_SHAPE, "RHS memref has an unexpected layout");
  if (!identity2d(out)) return fail(ctx, SWB_ERR_INVALID_SHAPE, "output memref has an unexpected layout");
  // verifyBSRStorage (SparseWaveOps.cpp:144-207)
  if (bs <= 0) return fail(ctx, SWB_ERR_INVALID_SHAPE, "'sparsewave.bsr_spmm' op block size must be positive, but got %lld", (long long)bs);
  if (out->sizes[0] % bs != 0)
    return fail(ctx, SWB_ERR_INVALID_SHAPE,
                "'sparsewave.bsr_spmm' op output rows must be divisible by block size, but got %lld and %lld",
                (long long)out->sizes[0], (long long)bs);
  if (brp->sizes[0] != out->sizes[0] / bs + 1)
    return fail(ctx, SWB_ERR_INVALID_SHAPE,
                "'sparsewave.bsr_spmm' op block-row offsets size must equal the number of block rows plus one, but got %lld and %lld",
                (long long)brp->sizes[0], (long long)(out->sizes[0] / bs));
  if (bv->sizes[0] != bci->sizes[0] * bs * bs)
    return fail(ctx, SWB_ERR_INVALID_SHAPE,
                "'sparsewave.bsr_spmm' op block values size must equal the number of blocks times block_size squared, but got %lld and %lld blocks",
                (long long)bv->sizes[0], (long long)bci->sizes[0]);
  if (rhs->sizes[1] != out->sizes[1])
    return fail(ctx, SWB_ERR_INVALID_SHAPE,
                "'sparsewave.bsr_spmm' op right-hand side and output must have the same number of columns");
  if (rhs->sizes[0] % bs != 0)
    return fail(ctx, SWB_ERR_INVALID_SHAPE,
                "'sparsewave.bsr_spmm' op right-hand-side rows must be divisible by block size, but got %lld and %lld",
                (long long)rhs->sizes[0], (long long)bs);
  return swb_bsr_spmm_f32(ctx, o, out->sizes[0], rhs->sizes[0], bci->sizes[0], bs, out->sizes[1],
                          brp->data + brp->offset, bci->data + bci->offset, bv->data + bv->offset,
                          rhs->data + rhs->offset, out->data + out->offset, stream);
}

static void finish_ciface(swb_context *ctx, int st) {
  if (st == SWB_OK) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) return;
    fprintf(stderr, "sparsewave_b200: CUDA error: %s\n", cudaGetErrorString(e));
    abort();
  }
  fprintf(stderr, "sparsewave_b200: %s\n", swb_last_error(ctx));
  abort();
}

void _mlir_ciface_sparsewave_spmv(swb_memref_1d_i32 *rp, swb_memref_1d_i32 *ci, swb_memref_1d_f32 *v,
                                  swb_memref_1d_f32 *x, swb_memref_1d_f32 *y) {
  swb_context *ctx = process_context();
  swb_options o;
  env_options(ctx, &o);
  finish_ciface(ctx, swb_spmv_memref(ctx, &o, rp, ci, v, x, y, nullptr));
}

void _mlir_ciface_sparsewave_spmm(swb_memref_1d_i32 *rp, swb_memref_1d_i32 *ci, swb_memref_1d_f32 *v,
                                  swb_memref_2d_f32 *rhs, swb_memref_2d_f32 *out) {
  swb_context *ctx = process_context();
  swb_options o;
  env_options(ctx, &o);
  finish_ciface(ctx, swb_spmm_memref(ctx, &o, rp, ci, v, rhs, out, nullptr));
}

void _mlir_ciface_sparsewave_bsr_spmm(swb_memref_1d_i32 *brp, swb_memref_1d_i32 *bci, swb_memref_1d_f32 *bv,
                                      swb_memref_2d_f32 *rhs, swb_memref_2d_f32 *out, int64_t bs) {
  swb_context *ctx = process_context();
  swb_options o;
  env_options(ctx, &o);
  finish_ciface(ctx, swb_bsr_spmm_memref(ctx, &o, brp, bci, bv, rhs, out, bs, nullptr));
}

// ---- bundle-style launch ----------------------------------------------------------------

int swb_bundle_launch(swb_context *ctx, const char *operation, int64_t n, void *const args[5], swb_stream stream) {
  if (!ctx) return fail(nullptr, SWB_ERR_INVALID_ARGUMENT, "context is NULL");
  if (!operation || strcmp(operation, "spmm") != 0)
    return fail(ctx, SWB_ERR_UNSUPPORTED, "input application is %s, but the bundle supports spmm", operation ? operation : "(null)");
  if (!args) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "bundle launch: args is NULL");
  if (n < 0) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "bundle launch: n must be non-negative");
  // Launch contract of the fixed-shape bundle: wave-per-row-tile, block 64,
  // tile 4, N == 4 (tools/sparsewave-bundle/sparsewave_bundle_ir.py:4-9).
  // The bundle kernel takes bare pointers, so the reduction extent (rows of
  // rhs) and NNZ are not part of the contract; they only matter for argument
  // checks here and are passed as upper bounds (with that NNZ the launcher
  // keeps a whole warp per row, the schedule the contract names).
  swb_options o;
  swb_options_default(&o);
  o.spmm_mapping = SWB_WAVE_PER_ROW_TILE;
  o.spmm_block_size = 64;
  o.spmm_tile_size = 4;
  return swb_spmm(ctx, &o, n, kI32Max, kI32Max - 256, 4, static_cast<const int32_t *>(args[0]),
                  static_cast<const int32_t *>(args[1]), static_cast<const float *>(args[2]),
                  static_cast<const float *>(args[3]), static_cast<float *>(args[4]), stream);
}

// ---- sharding -------------------------------------------------------------------------------

int swb_shard_rows_by_nnz(swb_context *ctx, const int32_t *row_ptr, int64_t rows, int64_t n_shards,
                          int64_t *boundaries) {
  if (!row_ptr || !boundaries) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "shard: NULL pointer");
  if (rows < 0 || n_shards < 1) return fail(ctx, SWB_ERR_INVALID_ARGUMENT, "shard: rows must be non-negative and n_shards positive");
  const int64_t nnz = row_ptr[rows];
  boundaries[0] = 0;
  for (int64_t k = 1; k < n_shards; ++k) {
    // floor(k * nnz / n_shards) without overflow: nnz < 2^31, k <= n_shards.
    const int64_t target = (int64_t)(((__int128)k * nnz) / n_shards);
    // first row r with row_ptr[r] >= target
    int64_t lo = 0, hi = rows;
    while (lo < hi) {
      int64_t mid = lo + (hi - lo) / 2;
      if (row_ptr[mid] < target) lo = mid + 1; else hi = mid;
    }
    boundaries[k] = lo < boundaries[k - 1] ? boundaries[k - 1] : lo;
  }
  boundaries[n_shards] = rows;
  return SWB_OK;
}

}  // extern "C"
