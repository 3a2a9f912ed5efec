// Single-node data-parallel gradient exchange over NCCL (NVLink 5 / NVSwitch).
//
// Stands where the reference's ctypes binding of libnccl stands (gradtuity/dist/nccl.py:71-189)
// and the calls built on it (gradtuity/dist/comm.py:37-170): unique-id creation, communicator
// init / destroy, in-place fp32 all-reduce, broadcast, barrier.  Differences:
//   * collectives run on a dedicated non-blocking stream, ordered against the compute stream by
//     events, so an all-reduce of finished gradient buckets overlaps the rest of backward; the
//     reference brackets every call with cudaDeviceSynchronize on the NULL stream
//     (gradtuity/dist/comm.py:129-131);
//   * the 1/world_size scale is folded into the collective (ncclAvg) instead of a separate kernel
//     (gradtuity/dist/ddp.py:94-97);
//   * nothing on the host waits without a limit: communicator creation runs in a helper thread that the caller
//     joins against a deadline, and a host-side wait polls the communication stream and
//     ncclCommGetAsyncError against the same deadline (GRADTUITY_NCCL_TIMEOUT_S, default 120 s); when it runs
//     out, or NCCL reports an asynchronous error (a peer that died), the communicator is aborted with
//     ncclCommAbort, which also ends its kernels, and the call returns GT_ERR_TIMEOUT / GT_ERR_NCCL.  The
//     communicator stays a blocking one: a non-blocking communicator hands every collective's launch to a
//     background thread, which costs the overlap with backward the side stream exists for;
//   * NCCL is opened with dlopen (GRADTUITY_NCCL_LIBRARY, default libnccl.so.2) with local symbol
//     scope, so it never clashes with another NCCL copy in the process.
// No kernel of this library reads a peer GPU's memory; inter-GPU traffic is NCCL's.

#include <dlfcn.h>
#include <sched.h>
#include <stdlib.h>
#include <unistd.h>

#include <chrono>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <thread>

#include "gt_internal.h"

namespace {

typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0, ncclInProgress = 7 };
enum { ncclFloat32 = 7 };
enum { ncclSum = 0, ncclAvg = 4 };

struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(ncclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;      // optional (NCCL >= 2.4)
  int (*CommAbort)(ncclComm_t) = nullptr;                    // optional
};

NcclApi g_nccl;

int load_nccl(char* err, size_t errlen) {
  if (g_nccl.handle) return GT_OK;
  const char* name = getenv("GRADTUITY_NCCL_LIBRARY");
  if (!name || !name[0]) name = "libnccl.so.2";
  void* h = dlopen(name, RTLD_NOW | RTLD_LOCAL);
  if (!h) {
    snprintf(err, errlen, "dlopen(%s) failed: %s", name, dlerror());
    return GT_ERR_NCCL;
  }
#define GT_SYM(field, sym)                                                       \
  *(void**)(&g_nccl.field) = dlsym(h, sym);                                      \
  if (!g_nccl.field) { snprintf(err, errlen, "%s lacks %s", name, sym); dlclose(h); return GT_ERR_NCCL; }
  GT_SYM(GetUniqueId, "ncclGetUniqueId");
  GT_SYM(CommInitRank, "ncclCommInitRank");
  GT_SYM(CommDestroy, "ncclCommDestroy");
  GT_SYM(AllReduce, "ncclAllReduce");
  GT_SYM(Broadcast, "ncclBroadcast");
  GT_SYM(AllGather, "ncclAllGather");
  GT_SYM(GetErrorString, "ncclGetErrorString");
#undef GT_SYM
  *(void**)(&g_nccl.CommGetAsyncError) = dlsym(h, "ncclCommGetAsyncError");
  *(void**)(&g_nccl.CommAbort) = dlsym(h, "ncclCommAbort");
  g_nccl.handle = h;
  return GT_OK;
}

struct DistState {
  ncclComm_t comm = nullptr;
  cudaStream_t stream = nullptr;     // collectives
  cudaEvent_t ready = nullptr;       // compute -> comm: "the data is final"
  cudaEvent_t done = nullptr;        // comm -> compute: "the collective has finished"
  int rank = 0, world = 1;
  int pending = 0;                   // collectives enqueued since the last wait
  // optional per-step timeline (GRADTUITY_DIST_TIMELINE=1): timed events around every collective since the last wait
  bool timeline = false;
  static constexpr int TL_MAX = 64;
  int tl_n = 0;
  long long tl_count[TL_MAX];
  cudaEvent_t tl_ready[TL_MAX], tl_start[TL_MAX], tl_end[TL_MAX];   // compute stream; comm stream before / after
  cudaEvent_t tl_resume = nullptr;   // compute stream, right after it was made to wait for the collectives
  bool tl_closed = false;
};

DistState* g_dist[64] = {nullptr};

double host_timeout_seconds() {
  const char* v = getenv("GRADTUITY_NCCL_TIMEOUT_S");
  const double t = v ? atof(v) : 0.0;
  return t > 0.0 ? t : 120.0;
}

double seconds_since(std::chrono::steady_clock::time_point t0) {
  return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

void abort_comm(DistState* st) {
  if (st->comm && g_nccl.CommAbort) g_nccl.CommAbort(st->comm);
  st->comm = nullptr;
}

// Blocks the calling thread until the communication stream is idle, an asynchronous NCCL error shows up, or
// the deadline passes.  Yields for the first couple of milliseconds (short collectives), then sleeps.
int wait_for_stream(gt_ctx* ctx, DistState* st, const char* what) {
  const auto t0 = std::chrono::steady_clock::now();
  const double limit = host_timeout_seconds();
  for (long long it = 0;; ++it) {
    const cudaError_t q = cudaStreamQuery(st->stream);
    if (q == cudaSuccess) return GT_OK;
    if (q != cudaErrorNotReady) GT_CUDA_OK(ctx, q);
    if (st->comm && g_nccl.CommGetAsyncError && (it & 63) == 0) {
      int async_rc = ncclSuccess;
      const int r = g_nccl.CommGetAsyncError(st->comm, &async_rc);
      if (r != ncclSuccess || (async_rc != ncclSuccess && async_rc != ncclInProgress)) {
        const int bad = r != ncclSuccess ? r : async_rc;
        snprintf(ctx->last_error, sizeof(ctx->last_error), "%s: NCCL reported an asynchronous error (%s); communicator aborted", what,
                 g_nccl.GetErrorString(bad));
        abort_comm(st);
        return GT_ERR_NCCL;
      }
    }
    const double waited = seconds_since(t0);
    if (waited > limit) {
      snprintf(ctx->last_error, sizeof(ctx->last_error),
               "%s: collectives still running after %.1f s (GRADTUITY_NCCL_TIMEOUT_S); a peer rank is probably gone; communicator aborted",
               what, waited);
      abort_comm(st);
      return GT_ERR_TIMEOUT;
    }
    if (waited < 2e-3) sched_yield(); else usleep(100);
  }
}

DistState* state_of(gt_ctx* ctx) { return (ctx && ctx->device >= 0 && ctx->device < 64) ? g_dist[ctx->device] : nullptr; }

#define GT_NCCL_OK(ctx, expr)                                                                  \
  do {                                                                                         \
    int _r = (expr);                                                                           \
    if (_r != ncclSuccess) {                                                                   \
      snprintf((ctx)->last_error, sizeof((ctx)->last_error), "%s: %s", #expr,                  \
               g_nccl.GetErrorString ? g_nccl.GetErrorString(_r) : "nccl error");              \
      return GT_ERR_NCCL;                                                                      \
    }                                                                                          \
  } while (0)

}  // namespace

extern "C" int gt_dist_get_unique_id(gt_ctx* ctx, char* out128) {
  if (!ctx || !out128) return GT_ERR_INVALID_ARG;
  int rc = load_nccl(ctx->last_error, sizeof(ctx->last_error));
  if (rc != GT_OK) return rc;
  ncclUniqueId id;
  GT_NCCL_OK(ctx, g_nccl.GetUniqueId(&id));
  memcpy(out128, id.internal, 128);
  return GT_OK;
}

extern "C" int gt_dist_init(gt_ctx* ctx, int rank, int world, const char* uid128) {
  if (!ctx || !uid128 || world < 1 || rank < 0 || rank >= world) return GT_ERR_INVALID_ARG;
  if (ctx->device < 0 || ctx->device >= 64) return GT_ERR_UNSUPPORTED;
  if (g_dist[ctx->device]) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gt_dist_init: already initialised on device %d", ctx->device);
  int rc = load_nccl(ctx->last_error, sizeof(ctx->last_error));
  if (rc != GT_OK) return rc;
  GT_CUDA_OK(ctx, cudaSetDevice(ctx->device));
  DistState* st = new DistState();
  st->rank = rank; st->world = world;
  ncclUniqueId id;
  memcpy(id.internal, uid128, 128);
  // ncclCommInitRank blocks until every rank has called it.  It runs in a helper thread that is joined against
  // a deadline, so a rank that never arrives gives an error here instead of a process that sits forever.
  struct InitJob { std::mutex m; std::condition_variable cv; bool done = false; int rc = 0; ncclComm_t comm = nullptr; };
  auto job = std::make_shared<InitJob>();
  const int device = ctx->device;
  std::thread([job, device, world, id, rank]() {
    ncclComm_t c = nullptr;
    int r = cudaSetDevice(device) == cudaSuccess ? g_nccl.CommInitRank(&c, world, id, rank) : -1;
    std::lock_guard<std::mutex> lk(job->m);
    job->rc = r; job->comm = c; job->done = true;
    job->cv.notify_all();
  }).detach();
  {
    std::unique_lock<std::mutex> lk(job->m);
    const double limit = host_timeout_seconds();
    if (!job->cv.wait_for(lk, std::chrono::duration<double>(limit), [&] { return job->done; })) {
      snprintf(ctx->last_error, sizeof(ctx->last_error),
               "ncclCommInitRank(rank %d of %d) did not complete within %.1f s (GRADTUITY_NCCL_TIMEOUT_S): a rank never joined", rank, world, limit);
      delete st;
      return GT_ERR_TIMEOUT;
    }
    if (job->rc != ncclSuccess) {
      snprintf(ctx->last_error, sizeof(ctx->last_error), "ncclCommInitRank(rank %d of %d): %s", rank, world,
               job->rc > 0 ? g_nccl.GetErrorString(job->rc) : "cudaSetDevice failed in the helper thread");
      delete st;
      return GT_ERR_NCCL;
    }
    st->comm = job->comm;
  }
  GT_CUDA_OK(ctx, cudaStreamCreateWithFlags(&st->stream, cudaStreamNonBlocking));
  GT_CUDA_OK(ctx, cudaEventCreateWithFlags(&st->ready, cudaEventDisableTiming));
  GT_CUDA_OK(ctx, cudaEventCreateWithFlags(&st->done, cudaEventDisableTiming));
  const char* tl = getenv("GRADTUITY_DIST_TIMELINE");
  if (tl && tl[0] == '1') {
    st->timeline = true;
    for (int i = 0; i < DistState::TL_MAX; ++i) {
      GT_CUDA_OK(ctx, cudaEventCreate(&st->tl_ready[i]));
      GT_CUDA_OK(ctx, cudaEventCreate(&st->tl_start[i]));
      GT_CUDA_OK(ctx, cudaEventCreate(&st->tl_end[i]));
    }
    GT_CUDA_OK(ctx, cudaEventCreate(&st->tl_resume));
  }
  g_dist[ctx->device] = st;
  ctx->dist_active = 1;
  return GT_OK;
}

extern "C" int gt_dist_destroy(gt_ctx* ctx) {
  DistState* st = state_of(ctx);
  if (!st) return GT_OK;
  if (st->comm && wait_for_stream(ctx, st, "gt_dist_destroy") != GT_OK) cudaGetLastError();   // on failure the communicator is already aborted
  if (st->comm) g_nccl.CommDestroy(st->comm);
  cudaEventDestroy(st->ready);
  cudaEventDestroy(st->done);
  cudaStreamDestroy(st->stream);
  delete st;
  g_dist[ctx->device] = nullptr;
  ctx->dist_active = 0;
  return GT_OK;
}

// In-place all-reduce of `count` floats.  The collective is enqueued on the communication stream
// behind everything the compute stream has been given so far, and returns at once; the compute
// stream does not wait for it until gt_dist_wait.
extern "C" int gt_dist_allreduce(gt_ctx* ctx, float* ptr, int64_t count, int average) {
  DistState* st = state_of(ctx);
  if (!ctx || !ptr || count <= 0) return GT_ERR_INVALID_ARG;
  if (!st) GT_FAIL(ctx, GT_ERR_NOT_INIT, "gt_dist_allreduce: process group not initialised");
  if (!st->comm) GT_FAIL(ctx, GT_ERR_NCCL, "gt_dist_allreduce: the communicator was aborted after an error or a time-out");
  GT_CUDA_OK(ctx, cudaEventRecord(st->ready, ctx->stream));
  GT_CUDA_OK(ctx, cudaStreamWaitEvent(st->stream, st->ready, 0));
  int slot = -1;
  if (st->timeline) {
    if (st->tl_closed) { st->tl_n = 0; st->tl_closed = false; }       // first collective after a wait: a new window
    if (st->tl_n < DistState::TL_MAX) {
      slot = st->tl_n++;
      st->tl_count[slot] = count;
      GT_CUDA_OK(ctx, cudaEventRecord(st->tl_ready[slot], ctx->stream));
      GT_CUDA_OK(ctx, cudaEventRecord(st->tl_start[slot], st->stream));
    }
  }
  GT_NCCL_OK(ctx, g_nccl.AllReduce(ptr, ptr, (size_t)count, ncclFloat32, average ? ncclAvg : ncclSum, st->comm, st->stream));
  if (slot >= 0) GT_CUDA_OK(ctx, cudaEventRecord(st->tl_end[slot], st->stream));
  st->pending += 1;
  return GT_OK;
}

// dst (world x count floats) = the `count` floats at src of every rank, in rank order; enqueued like gt_dist_allreduce.
// Every rank must pass the same count.
extern "C" int gt_dist_allgather(gt_ctx* ctx, float* dst, const float* src, int64_t count) {
  DistState* st = state_of(ctx);
  if (!ctx || !dst || !src || count <= 0) return GT_ERR_INVALID_ARG;
  if (!st) GT_FAIL(ctx, GT_ERR_NOT_INIT, "gt_dist_allgather: process group not initialised");
  if (!st->comm) GT_FAIL(ctx, GT_ERR_NCCL, "gt_dist_allgather: the communicator was aborted after an error or a time-out");
  GT_CUDA_OK(ctx, cudaEventRecord(st->ready, ctx->stream));
  GT_CUDA_OK(ctx, cudaStreamWaitEvent(st->stream, st->ready, 0));
  int slot = -1;
  if (st->timeline) {
    if (st->tl_closed) { st->tl_n = 0; st->tl_closed = false; }
    if (st->tl_n < DistState::TL_MAX) {
      slot = st->tl_n++;
      st->tl_count[slot] = count * st->world;
      GT_CUDA_OK(ctx, cudaEventRecord(st->tl_ready[slot], ctx->stream));
      GT_CUDA_OK(ctx, cudaEventRecord(st->tl_start[slot], st->stream));
    }
  }
  GT_NCCL_OK(ctx, g_nccl.AllGather(src, dst, (size_t)count, ncclFloat32, st->comm, st->stream));
  if (slot >= 0) GT_CUDA_OK(ctx, cudaEventRecord(st->tl_end[slot], st->stream));
  st->pending += 1;
  return GT_OK;
}

extern "C" int gt_dist_broadcast(gt_ctx* ctx, float* ptr, int64_t count, int root) {
  DistState* st = state_of(ctx);
  if (!ctx || !ptr || count <= 0) return GT_ERR_INVALID_ARG;
  if (!st) GT_FAIL(ctx, GT_ERR_NOT_INIT, "gt_dist_broadcast: process group not initialised");
  if (root < 0 || root >= st->world) return GT_ERR_INVALID_ARG;
  if (!st->comm) GT_FAIL(ctx, GT_ERR_NCCL, "gt_dist_broadcast: the communicator was aborted after an error or a time-out");
  GT_CUDA_OK(ctx, cudaEventRecord(st->ready, ctx->stream));
  GT_CUDA_OK(ctx, cudaStreamWaitEvent(st->stream, st->ready, 0));
  GT_NCCL_OK(ctx, g_nccl.Broadcast(ptr, ptr, (size_t)count, ncclFloat32, root, st->comm, st->stream));
  st->pending += 1;
  return GT_OK;
}

// Makes the compute stream wait (on the device) for every collective enqueued so far.  With
// host_sync != 0 the calling thread also blocks until they have finished.
extern "C" int gt_dist_wait(gt_ctx* ctx, int host_sync) {
  DistState* st = state_of(ctx);
  if (!ctx) return GT_ERR_INVALID_ARG;
  if (!st) return GT_OK;
  if (st->pending) {
    GT_CUDA_OK(ctx, cudaEventRecord(st->done, st->stream));
    GT_CUDA_OK(ctx, cudaStreamWaitEvent(ctx->stream, st->done, 0));
    st->pending = 0;
    if (st->timeline && !st->tl_closed && st->tl_n > 0) {
      GT_CUDA_OK(ctx, cudaEventRecord(st->tl_resume, ctx->stream));
      st->tl_closed = true;
    }
  }
  if (host_sync) return wait_for_stream(ctx, st, "gt_dist_wait");
  return GT_OK;
}

// Timeline of the collectives between the last two waits (only with GRADTUITY_DIST_TIMELINE=1 at init; else *n = 0).
// Row i of `out` (4 floats): element count, then milliseconds relative to the first collective's enqueue point
// on the compute stream: when the compute stream reached collective i's enqueue point, when the communication
// stream started it, when it finished.  One more row at the end: (0, time the compute stream resumed after the
// wait, 0, 0).  Synchronises both streams.  Measurement aid; the reference has no counterpart.
extern "C" int gt_dist_timeline(gt_ctx* ctx, float* out, int max_rows, int* n) {
  DistState* st = state_of(ctx);
  if (!ctx || !out || !n || max_rows < 0) return GT_ERR_INVALID_ARG;
  *n = 0;
  if (!st || !st->timeline || !st->tl_closed || st->tl_n == 0) return GT_OK;
  GT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
  int rc = wait_for_stream(ctx, st, "gt_dist_timeline");
  if (rc != GT_OK) return rc;
  int rows = 0;
  for (int i = 0; i < st->tl_n && rows < max_rows; ++i, ++rows) {
    float a = 0, b = 0, c = 0;
    GT_CUDA_OK(ctx, cudaEventElapsedTime(&a, st->tl_ready[0], st->tl_ready[i]));
    GT_CUDA_OK(ctx, cudaEventElapsedTime(&b, st->tl_ready[0], st->tl_start[i]));
    GT_CUDA_OK(ctx, cudaEventElapsedTime(&c, st->tl_ready[0], st->tl_end[i]));
    out[4 * rows] = (float)st->tl_count[i]; out[4 * rows + 1] = a; out[4 * rows + 2] = b; out[4 * rows + 3] = c;
  }
  if (rows < max_rows) {
    float r = 0;
    GT_CUDA_OK(ctx, cudaEventElapsedTime(&r, st->tl_ready[0], st->tl_resume));
    out[4 * rows] = 0; out[4 * rows + 1] = r; out[4 * rows + 2] = 0; out[4 * rows + 3] = 0;
    ++rows;
  }
  *n = rows;
  return GT_OK;
}

extern "C" int gt_dist_info(gt_ctx* ctx, int* rank, int* world) {
  DistState* st = state_of(ctx);
  if (!ctx || !rank || !world) return GT_ERR_INVALID_ARG;
  *rank = st ? st->rank : 0;
  *world = st ? st->world : 1;
  return GT_OK;
}
