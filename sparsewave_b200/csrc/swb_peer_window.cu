// All-gather of the dense operand as one kernel of peer stores over NVLink.
//
// Every rank owns a window: a device allocation of [4 KiB header][2 buffers of n_ranks * bytes_per_rank data]
// exported to the other ranks of the node with CUDA IPC (the handles travel through the context's NCCL
// communicator at set-up).  A step names the buffer it fills and is one kernel per rank that
//   1. only when the step before it filled the same buffer: tells every peer "I no longer read my window"
//      (ready flag, epoch-numbered; stream order guarantees that the kernel that consumed the previous epoch
//      has finished) and
//   2. waits until every peer has said the same, so no buffer is overwritten while it is read,
//   3. stores its own chunk into that buffer of every rank's window (plain 16-byte peer stores; its own
//      window included); each CTA serves one destination,
//   4. per CTA: once its stores are ordered system-wide (one fence by one thread behind a CTA barrier), adds
//      one to the destination's arrival counter with a remote atomic,
//   5. the CTA of this rank that finishes last waits until this rank's own counter for that buffer shows
//      the arrivals of every rank's CTAs for this fill, so that the kernel after it finds the buffer complete.
// Steps that alternate between the two buffers need neither 1 nor 2: a rank starts epoch e only after its
// kernel of epoch e - 1 has seen every rank's arrivals of epoch e - 1, and a rank sends those only after (in
// its stream) the consumer of epoch e - 2 has finished, which was the last reader of the buffer that epoch e
// fills.  The sharded operators alternate; swb_comm_window_allgather always fills buffer 0 and therefore
// always takes steps 1 and 2.  Which of the two happens is decided on the device from the header (the
// buffer of the previous step), so that a replayed CUDA graph with an odd number of steps stays correct.
// Optionally the kernel also zero-fills an output vector (the separate fill launch of the position
// mappings) while it would otherwise wait.
// All waits poll counters in this GPU's own memory that the other ranks write, are bounded, and give up
// by setting the context's status word (swb_device_status) instead of spinning on; CTAs of one grid never
// wait for one another, so the grid needs no co-residency.
// Plain loads, stores and atomics only.  Not a reference feature.
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "../../include/sparsewave_b200.h"
#include "swb_kernels.h"

namespace swb {
namespace {

constexpr int kMaxRanks = 16;
constexpr int64_t kHeaderBytes = 4096;
// header words: ready[rank] at 0, arrivals[buffer] (of all ranks' CTAs, ever) at 256, epoch at 512, local CTA count
// at 516, 1 + the buffer of the last finished step at 520 (0: none yet), finished steps per buffer at 524
constexpr int kReadyOff = 0, kArrivalsOff = 256, kEpochOff = 512, kCountOff = 516, kLastBufferOff = 520, kFillsOff = 524;
constexpr unsigned kPollLimit = 1u << 24;  // polls of a word in local memory, 100 ns apart (a few seconds), before giving up
constexpr int kGridTarget = 128;           // CTAs of a step, split evenly over the destination ranks (four GPUs, 4 MB per rank:
                                           // 28.8 us with 64 to 128 CTAs, 32.7 with 256 or more)

struct PeerWindow {
  int ranks = 1, rank = 0, slices = 1;
  int next_buffer = 0;  // of the alternating (internal) steps
  int64_t bytes_per_rank = 0;
  char *local = nullptr;
  char *peer[kMaxRanks] = {};
  char **d_peer = nullptr;
};

// true when *word has reached `target` (compared modulo 2^32) before the poll limit
__device__ bool wait_word(const volatile unsigned *word, unsigned target) {
  for (unsigned n = 0; n < kPollLimit; ++n) {
    if ((int)(*word - target) >= 0) return true;
    __nanosleep(100);
  }
  return false;
}

__global__ void __launch_bounds__(256) peer_allgather_kernel(const int4 *__restrict__ send, int64_t n16,
                                                             char *const *__restrict__ peer, int rank, int ranks,
                                                             int64_t bytes_per_rank, int buffer,
                                                             float *__restrict__ zero, int64_t zero_count,
                                                             int *status) {
  char *local = peer[rank];
  __shared__ unsigned s_epoch;
  __shared__ int s_failed;
  __shared__ int s_last;
  __shared__ int s_same;
  __shared__ unsigned s_fill;
  if (threadIdx.x == 0) {
    s_epoch = *reinterpret_cast<volatile unsigned *>(local + kEpochOff) + 1u;
    s_fill = reinterpret_cast<volatile unsigned *>(local + kFillsOff)[buffer] + 1u;  // this is the n-th fill of the buffer
    // the step before this one filled the same buffer: its readers have to be waited for (steps 1 and 2)
    s_same = *reinterpret_cast<volatile unsigned *>(local + kLastBufferOff) == (unsigned)buffer + 1u;
    s_failed = 0;
    s_last = 0;
  }
  __syncthreads();
  const unsigned epoch = s_epoch;
  const bool handshake = s_same != 0;
  // A kernel launched behind this one with programmatic stream serialisation (the span kernel of the sharded
  // SpMV) may start its prologue now; it waits for the end of this grid before it reads x or touches y.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // 1. ready flags out (one CTA is enough)
  if (handshake && blockIdx.x == 0 && threadIdx.x < ranks)
    reinterpret_cast<volatile unsigned *>(peer[threadIdx.x] + kReadyOff)[rank] = epoch;
  // the zero fill of the consumer's output rides along while the flags travel
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < zero_count; i += (int64_t)gridDim.x * blockDim.x)
    zero[i] = 0.0f;
  // 2. ready flags in (every CTA looks for itself)
  if (handshake && threadIdx.x < ranks && threadIdx.x != rank &&
      !wait_word(reinterpret_cast<volatile unsigned *>(local + kReadyOff) + threadIdx.x, epoch))
    s_failed = 1;
  __syncthreads();

  // 3. this rank's chunk into the window of rank `dst`; the CTAs of one destination interleave by slice.
  // After a failed wait the stores still go out (they stay inside the windows) so that the counters below
  // remain consistent; the status word tells the host that the result is not to be trusted.
  const int dst = blockIdx.x % ranks, slice = blockIdx.x / ranks, slices = gridDim.x / ranks;
  int4 *out = reinterpret_cast<int4 *>(peer[dst] + kHeaderBytes + ((int64_t)buffer * ranks + rank) * bytes_per_rank);
  const int64_t stride = (int64_t)slices * blockDim.x;
  int64_t i = (int64_t)slice * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    const int4 a = __ldg(send + i), b = __ldg(send + i + stride), c = __ldg(send + i + 2 * stride),
               d = __ldg(send + i + 3 * stride);
    out[i] = a; out[i + stride] = b; out[i + 2 * stride] = c; out[i + 3 * stride] = d;
  }
  for (; i < n16; i += stride) out[i] = __ldg(send + i);

  // 4. the CTA's stores (ordered before thread 0 by the barrier, system-wide by its fence) precede its
  //    arrival at the destination; the CTA of this rank that counts last waits for the arrivals here
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    atomicAdd_system(reinterpret_cast<unsigned *>(peer[dst] + kArrivalsOff) + buffer, 1u);
    const unsigned before = atomicAdd(reinterpret_cast<unsigned *>(local + kCountOff), 1u);
    s_last = before == gridDim.x - 1;
    if (s_failed) atomicExch(status, 3);
  }
  __syncthreads();
  if (!s_last) return;

  // 5. every rank's CTAs aimed at this rank (slices per rank, so gridDim.x per fill) have arrived.  The
  //    arrivals are counted per buffer: a rank that is one step ahead already adds to the other buffer's
  //    counter, and none can be two steps ahead (it would need this rank's arrivals of the step between).
  if (threadIdx.x == 0) {
    if (!wait_word(reinterpret_cast<volatile unsigned *>(local + kArrivalsOff) + buffer, s_fill * gridDim.x))
      atomicExch(status, 4);
    __threadfence_system();
    reinterpret_cast<volatile unsigned *>(local + kFillsOff)[buffer] = s_fill;
    *reinterpret_cast<volatile unsigned *>(local + kCountOff) = 0u;
    *reinterpret_cast<volatile unsigned *>(local + kLastBufferOff) = (unsigned)buffer + 1u;
    *reinterpret_cast<volatile unsigned *>(local + kEpochOff) = epoch;
  }
}

int window_fail(swb_context *ctx, int status, const char *what, const char *detail) {
  char buf[512];
  snprintf(buf, sizeof buf, "%s: %s", what, detail);
  set_context_error(ctx, buf);
  return status;
}

void release(PeerWindow *w) {
  if (!w) return;
  for (int k = 0; k < w->ranks; ++k)
    if (k != w->rank && w->peer[k]) cudaIpcCloseMemHandle(w->peer[k]);
  if (w->d_peer) cudaFree(w->d_peer);
  if (w->local) cudaFree(w->local);
  delete w;
}

}  // namespace

// This rank's window (past its header) and the bytes every rank contributes, or NULL without a window.
void *peer_window_data(const swb_context *ctx, int64_t *bytes_per_rank) {
  PeerWindow *w = static_cast<PeerWindow *>(context_peer_window(ctx));
  if (!w) return nullptr;
  *bytes_per_rank = w->bytes_per_rank;
  return w->local + kHeaderBytes;
}

// Tear-down without a collective, for swb_destroy: the peers' windows are unmapped and the bookkeeping is
// freed, but this rank's window stays allocated (a peer may still map it, and memory that another process
// maps must not be freed), until the process ends.
void abandon_peer_window(swb_context *ctx) {
  PeerWindow *w = static_cast<PeerWindow *>(context_peer_window(ctx));
  if (!w) return;
  cudaSetDevice(context_device(ctx));
  w->local = nullptr;  // left allocated on purpose
  release(w);
  set_context_peer_window(ctx, nullptr);
}

}  // namespace swb

extern "C" {

int swb_comm_window_create(swb_context *ctx, int64_t bytes_per_rank, void **window) {
  using namespace swb;
  if (!ctx) {
    set_thread_error("context is NULL");
    return SWB_ERR_INVALID_ARGUMENT;
  }
  if (!window) return window_fail(ctx, SWB_ERR_INVALID_ARGUMENT, "window", "window is NULL");
  *window = nullptr;
  int ranks = 1, rank = 0;
  if (!context_comm_shape(ctx, &ranks, &rank))
    return window_fail(ctx, SWB_ERR_INVALID_ARGUMENT, "window", "the context has no communicator (swb_comm_init)");
  if (ranks > kMaxRanks) return window_fail(ctx, SWB_ERR_UNSUPPORTED, "window", "more than 16 ranks");
  if (bytes_per_rank <= 0 || bytes_per_rank % 16 != 0)
    return window_fail(ctx, SWB_ERR_INVALID_ARGUMENT, "window", "bytes_per_rank must be a positive multiple of 16");
  if (context_peer_window(ctx)) return window_fail(ctx, SWB_ERR_INVALID_ARGUMENT, "window", "the context already has a window");
  cudaError_t e = cudaSetDevice(context_device(ctx));
  if (e != cudaSuccess) return window_fail(ctx, SWB_ERR_CUDA, "cudaSetDevice", cudaGetErrorString(e));

  // Creation succeeds on every rank or on none: a rank whose allocation or mapping fails still takes part
  // in both exchanges (with an all-zero handle that no peer can open, then with its failure flag), so no
  // rank is left waiting in a collective and no rank ends up with a window that a peer lacks.
  PeerWindow *w = new PeerWindow();
  w->ranks = ranks; w->rank = rank; w->bytes_per_rank = bytes_per_rank;
  // SWB_WINDOW_CTAS (read at creation; the same on every rank, the arrival count relies on it): CTAs of a step
  int grid_target = kGridTarget;
  if (const char *env = getenv("SWB_WINDOW_CTAS")) {
    const long v = strtol(env, nullptr, 10);
    if (v >= ranks && v <= 1024) grid_target = (int)v;
  }
  w->slices = grid_target / ranks > 0 ? grid_target / ranks : 1;
  const size_t total = (size_t)kHeaderBytes + 2 * (size_t)ranks * (size_t)bytes_per_rank;  // header, two buffers
  struct Slot { cudaIpcMemHandle_t handle; int ok; int pad[3]; };  // one exchanged record, 80 bytes
  Slot *d_slots = nullptr;  // [0, ranks): gathered, [ranks]: this rank's
  Slot mine, all[kMaxRanks];
  memset(&mine, 0, sizeof mine);
  e = cudaMalloc(&d_slots, sizeof(Slot) * (size_t)(ranks + 1));
  if (e != cudaSuccess) {
    release(w);
    return window_fail(ctx, SWB_ERR_CUDA, "window exchange buffer", cudaGetErrorString(e));
  }
  std::string why;
  e = cudaMalloc(&w->local, total);
  if (e == cudaSuccess) e = cudaMemset(w->local, 0, (size_t)kHeaderBytes);
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&mine.handle, w->local);
  mine.ok = e == cudaSuccess;
  if (!mine.ok) why = std::string("window allocation: ") + cudaGetErrorString(e);

  auto exchange = [&]() -> int {  // this rank's slot to every rank; the header memset precedes it in stream order
    cudaError_t ce = cudaMemcpy(d_slots + ranks, &mine, sizeof mine, cudaMemcpyHostToDevice);
    if (ce != cudaSuccess) return window_fail(ctx, SWB_ERR_CUDA, "window exchange", cudaGetErrorString(ce));
    int st = swb_comm_allgather(ctx, d_slots + ranks, d_slots, (int64_t)sizeof(Slot), nullptr);
    if (st != SWB_OK) return st;
    ce = cudaStreamSynchronize(nullptr);
    if (ce == cudaSuccess) ce = cudaMemcpy(all, d_slots, sizeof(Slot) * (size_t)ranks, cudaMemcpyDeviceToHost);
    if (ce != cudaSuccess) return window_fail(ctx, SWB_ERR_CUDA, "window exchange", cudaGetErrorString(ce));
    return SWB_OK;
  };

  int st = exchange();  // 1. handles
  if (st == SWB_OK) {
    for (int k = 0; k < ranks && mine.ok; ++k) {
      if (k == rank) {
        w->peer[k] = w->local;
        continue;
      }
      void *p = nullptr;
      e = all[k].ok ? cudaIpcOpenMemHandle(&p, all[k].handle, cudaIpcMemLazyEnablePeerAccess) : cudaErrorInvalidValue;
      if (e != cudaSuccess) {
        mine.ok = 0;
        why = std::string("mapping the window of rank ") + std::to_string(k) + ": " + cudaGetErrorString(e);
        cudaGetLastError();
      }
      w->peer[k] = static_cast<char *>(p);
    }
    if (mine.ok) {
      e = cudaMalloc(&w->d_peer, sizeof(char *) * kMaxRanks);
      if (e == cudaSuccess) e = cudaMemcpy(w->d_peer, w->peer, sizeof(char *) * kMaxRanks, cudaMemcpyHostToDevice);
      if (e != cudaSuccess) {
        mine.ok = 0;
        why = std::string("window peer table: ") + cudaGetErrorString(e);
      }
    }
    st = exchange();  // 2. who succeeded
  }
  cudaFree(d_slots);
  if (st == SWB_OK) {
    for (int k = 0; k < ranks; ++k)
      if (!all[k].ok) {
        if (why.empty()) why = "rank " + std::to_string(k) + " could not create or map its window";
        st = window_fail(ctx, SWB_ERR_CUDA, "window", why.c_str());
        break;
      }
  }
  if (st != SWB_OK) {
    release(w);
    return st;
  }
  set_context_peer_window(ctx, w);
  *window = w->local + kHeaderBytes;
  return SWB_OK;
}

int swb_comm_window_allgather(swb_context *ctx, const void *send, swb_stream stream) {
  return swb::window_allgather_and_fill(ctx, send, nullptr, 0, static_cast<cudaStream_t>(stream), false, nullptr);
}

int swb_comm_window_allgather_next(swb_context *ctx, const void *send, swb_stream stream, const void **gathered) {
  return swb::window_allgather_and_fill(ctx, send, nullptr, 0, static_cast<cudaStream_t>(stream), true, gathered);
}

}  // extern "C"

namespace swb {

// The exchange of swb_comm_window_allgather; the same kernel also stores `zero_count` zeros at `zero`
// (the output vector of the operator that consumes the window), or nothing when zero is NULL.
// alternate: fill the buffer that the previous alternating call did not (no ready-flag round trip between
// such calls), else buffer 0, the one swb_comm_window_create returned.  *gathered (if not NULL): where the
// gathered operand of this call lies.
int window_allgather_and_fill(swb_context *ctx, const void *send, float *zero, int64_t zero_count, cudaStream_t stream,
                              bool alternate, const void **gathered) {
  if (!ctx) {
    set_thread_error("context is NULL");
    return SWB_ERR_INVALID_ARGUMENT;
  }
  PeerWindow *w = static_cast<PeerWindow *>(context_peer_window(ctx));
  if (!w) return window_fail(ctx, SWB_ERR_INVALID_ARGUMENT, "window all-gather", "the context has no window (swb_comm_window_create)");
  if (!send || (reinterpret_cast<uintptr_t>(send) & 15u))
    return window_fail(ctx, SWB_ERR_INVALID_ARGUMENT, "window all-gather", "send must be a 16-byte aligned device pointer");
  cudaError_t e = cudaSetDevice(context_device(ctx));
  if (e != cudaSuccess) return window_fail(ctx, SWB_ERR_CUDA, "cudaSetDevice", cudaGetErrorString(e));
  // enough 16-byte loads in flight (16 KiB per CTA) to keep the NVLink egress busy whatever the rank count;
  // the grid is the same on every rank and for every step of a window (the arrival count relies on it)
  const int buffer = alternate ? w->next_buffer : 0;
  if (alternate) w->next_buffer ^= 1;
  if (gathered) *gathered = w->local + kHeaderBytes + (int64_t)buffer * w->ranks * w->bytes_per_rank;
  peer_allgather_kernel<<<(unsigned)(w->ranks * w->slices), 256, 0, stream>>>(
      static_cast<const int4 *>(send), w->bytes_per_rank / 16, w->d_peer, w->rank, w->ranks, w->bytes_per_rank,
      buffer, zero, zero ? zero_count : 0, context_status_flag(ctx));
  count_launch(ctx);
  e = cudaGetLastError();
  if (e != cudaSuccess) return window_fail(ctx, SWB_ERR_CUDA, "window all-gather launch", cudaGetErrorString(e));
  return SWB_OK;
}

}  // namespace swb

extern "C" {

void swb_comm_window_destroy(swb_context *ctx) {
  using namespace swb;
  if (!ctx) return;
  PeerWindow *w = static_cast<PeerWindow *>(context_peer_window(ctx));
  if (!w) return;
  cudaSetDevice(context_device(ctx));
  cudaDeviceSynchronize();
  // Unmap the peers' windows, then make sure every rank has done so before any window is freed (memory
  // must not be freed while another process still maps it): a 4-byte all-gather inside the header.
  for (int k = 0; k < w->ranks; ++k)
    if (k != w->rank && w->peer[k]) {
      cudaIpcCloseMemHandle(w->peer[k]);
      w->peer[k] = nullptr;
    }
  int ranks = 1, rank = 0;
  if (w->ranks > 1 && context_comm_shape(ctx, &ranks, &rank) &&
      swb_comm_allgather(ctx, w->local + 1024, w->local + 2048, 4, nullptr) == SWB_OK)
    cudaStreamSynchronize(nullptr);
  release(w);
  set_context_peer_window(ctx, nullptr);
}

}  // extern "C"
