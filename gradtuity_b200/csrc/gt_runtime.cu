// Context, memory, events and error reporting of libgt_b200.so.
//
// Plays the part of the reference's ctypes bindings to libcudart
// (gradtuity/cuda_mem.py:30-153) and of its event timer (gradtuity/cuda_driver.py:472-511)
// for the GEMM path, with two differences: allocation is stream-ordered from a pooled
// allocator (the reference calls cudaMalloc/cudaFree once per tensor,
// gradtuity/tensor.py:122-126), and every call reports a status instead of ignoring it.

#include <mutex>
#include <unordered_map>
#include <vector>

#include <stdlib.h>

#include "gt_internal.h"

extern "C" const char* gt_strerror(int status) {
  switch (status) {
    case GT_OK: return "success";
    case GT_ERR_INVALID_ARG: return "invalid argument";
    case GT_ERR_CUDA: return "CUDA call failed";
    case GT_ERR_UNSUPPORTED: return "unsupported request";
    case GT_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case GT_ERR_NOMEM: return "out of memory";
    case GT_ERR_NCCL: return "NCCL call failed";
    case GT_ERR_TOO_LARGE: return "size exceeds the fixed maximum of this entry point";
    case GT_ERR_NOT_INIT: return "context not initialised";
    default: return "unknown status";
  }
}

extern "C" const char* gt_last_error(gt_ctx* ctx) { return ctx ? ctx->last_error : "null context"; }

namespace {
struct BlockCache {
  std::mutex lock;
  std::unordered_map<size_t, std::vector<void*>> free_by_size;
  std::unordered_map<void*, size_t> size_of;       // blocks handed out by gt_malloc, live or cached
  size_t cached_bytes = 0;
  size_t limit_bytes = (size_t)65536 << 20;
  bool enabled = true;
};

void block_cache_flush(gt_ctx* ctx, BlockCache* bc) {
  for (auto& kv : bc->free_by_size) {
    for (void* q : kv.second) { cudaFreeAsync(q, ctx->stream); bc->size_of.erase(q); }
    kv.second.clear();
  }
  bc->cached_bytes = 0;
}
}  // namespace

extern "C" int gt_init(int device, gt_ctx** out) {
  if (!out || device < 0) return GT_ERR_INVALID_ARG;
  *out = nullptr;
  gt_ctx* ctx = (gt_ctx*)calloc(1, sizeof(gt_ctx));
  if (!ctx) return GT_ERR_NOMEM;
  ctx->device = device;
  cudaError_t e = cudaSetDevice(device);
  if (e != cudaSuccess) { free(ctx); return GT_ERR_CUDA; }
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) { free(ctx); return GT_ERR_CUDA; }
  if (prop.major != 10) {
    // The kernels are sm_100a only; there is no fallback for other parts.
    free(ctx);
    return GT_ERR_UNSUPPORTED;
  }
  ctx->sm_count = prop.multiProcessorCount;
  if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) { free(ctx); return GT_ERR_CUDA; }
  if (cudaMalloc((void**)&ctx->d_status, 4096) != cudaSuccess) { free(ctx); return GT_ERR_CUDA; }
  cudaMemset(ctx->d_status, 0, 4096);
  ctx->tail_epoch = 0;
  if (cudaMalloc((void**)&ctx->d_sched, GT_SCHED_RING * sizeof(int)) != cudaSuccess) { cudaFree(ctx->d_status); free(ctx); return GT_ERR_CUDA; }
  cudaMemset(ctx->d_sched, 0, GT_SCHED_RING * sizeof(int));
  ctx->sched_seq = 0;
  {
    BlockCache* bc = new BlockCache();
    bc->enabled = getenv("GRADTUITY_NO_ALLOC_CACHE") == nullptr;
    const char* mb = getenv("GRADTUITY_ALLOC_CACHE_MB");
    if (mb && atoll(mb) > 0) bc->limit_bytes = (size_t)atoll(mb) << 20;
    ctx->block_cache = bc;
  }

  // Keep freed blocks in the pool instead of returning them to the driver at every sync.
  cudaMemPool_t pool;
  if (cudaDeviceGetDefaultMemPool(&pool, device) == cudaSuccess) {
    uint64_t keep = UINT64_MAX;
    cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
  }

  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
    cudaFree(ctx->d_status);
    free(ctx);
    return GT_ERR_CUDA;
  }
  ctx->encode_tiled = (gt_encode_tiled_fn)fn;
  const char* r = getenv("GRADTUITY_GEMM_TMA_ROUND");
  // Tensor maps of type TFLOAT32 make the TMA unit round fp32 to tf32 (nearest) on the way into
  // shared memory; with FLOAT32 maps the tensor core just drops the low 13 mantissa bits, which
  // biases every product towards zero (measured: 7.7e-4 relative error instead of 2.9e-4).
  ctx->tma_round = (r && r[0] == '0') ? 0 : 1;
  *out = ctx;
  return GT_OK;
}

extern "C" int gt_destroy(gt_ctx* ctx) {
  if (!ctx) return GT_ERR_INVALID_ARG;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->block_cache) {
    BlockCache* bc = (BlockCache*)ctx->block_cache;
    block_cache_flush(ctx, bc);
    delete bc;
    ctx->block_cache = nullptr;
  }
  gt_attn_release(ctx);
  if (ctx->scratch_event) cudaEventDestroy(ctx->scratch_event);
  if (ctx->side_stream) {
    cudaStreamSynchronize(ctx->side_stream);
    cudaStreamDestroy(ctx->side_stream);
    cudaEventDestroy(ctx->side_fork);
    cudaEventDestroy(ctx->side_done);
  }
  if (ctx->workspace) cudaFree(ctx->workspace);
  if (ctx->h2d_stream) {
    cudaStreamDestroy(ctx->h2d_stream);
    cudaStreamDestroy(ctx->d2h_stream);
    for (int i = 0; i < 8; ++i) cudaEventDestroy(ctx->host_ev[i]);
  }
  cudaFree(ctx->d_status);
  cudaFree(ctx->d_sched);
  cudaStreamDestroy(ctx->stream);
  free(ctx);
  return GT_OK;
}

extern "C" void* gt_ctx_stream(gt_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }
extern "C" int gt_sm_count(gt_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

extern "C" int gt_device_status(gt_ctx* ctx, int* status) {
  if (!ctx || !status) return GT_ERR_INVALID_ARG;
  gt_join_beside(ctx);
  GT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
  int h = 0;
  GT_CUDA_OK(ctx, cudaMemcpy(&h, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (h != 0) GT_CUDA_OK(ctx, cudaMemset(ctx->d_status, 0, sizeof(int)));
  *status = h;
  return GT_OK;
}

extern "C" int gt_launch_count(gt_ctx* ctx, int64_t* count) {
  if (!ctx || !count) return GT_ERR_INVALID_ARG;
  *count = ctx->launches;
  return GT_OK;
}

int gt_smem_opt_in(gt_ctx* ctx, const void* kernel, int bytes) {
  static std::mutex lock;
  static std::unordered_map<const void*, unsigned long long> done;       // kernel -> devices already served
  std::lock_guard<std::mutex> guard(lock);
  unsigned long long& mask = done[kernel];
  const unsigned long long bit = 1ull << (ctx->device & 63);
  if (mask & bit) return GT_OK;
  GT_CUDA_OK(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  mask |= bit;
  return GT_OK;
}

int gt_scratch_acquire(gt_ctx* ctx, cudaStream_t stream) {
  if (ctx->scratch_stream == stream) return GT_OK;
  if (!ctx->scratch_event) GT_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->scratch_event, cudaEventDisableTiming));
  if (ctx->scratch_stream) {
    // The previous user's stream is touched only if it is the context's own (always alive); a caller's stream had
    // the event recorded on it when its call returned (gt_scratch_release) and may be gone by now.
    if (ctx->scratch_stream == ctx->stream) GT_CUDA_OK(ctx, cudaEventRecord(ctx->scratch_event, ctx->stream));
    GT_CUDA_OK(ctx, cudaStreamWaitEvent(stream, ctx->scratch_event, 0));
  }
  ctx->scratch_stream = stream;
  return GT_OK;
}

int gt_scratch_release(gt_ctx* ctx, cudaStream_t stream) {
  if (ctx->scratch_stream != stream || stream == ctx->stream) return GT_OK;
  if (!ctx->scratch_event) GT_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->scratch_event, cudaEventDisableTiming));
  GT_CUDA_OK(ctx, cudaEventRecord(ctx->scratch_event, stream));
  return GT_OK;
}

int gt_workspace_reserve(gt_ctx* ctx, size_t nbytes, cudaStream_t stream) {
  const cudaStream_t previous = ctx->scratch_stream;
  int rc = gt_scratch_acquire(ctx, stream);
  if (rc != GT_OK) return rc;
  if (nbytes <= ctx->workspace_bytes) return GT_OK;
  // Growing is rare (first call at a new largest size); it orders itself against earlier users of the old block
  // on the host: the previous user's work (its event, if it was a caller's stream) and this stream's.
  if (previous && previous != stream) {
    if (previous == ctx->stream) GT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
    else GT_CUDA_OK(ctx, cudaEventSynchronize(ctx->scratch_event));
  }
  GT_CUDA_OK(ctx, cudaStreamSynchronize(stream));
  if (ctx->workspace) GT_CUDA_OK(ctx, cudaFree(ctx->workspace));
  ctx->workspace = nullptr;
  ctx->workspace_bytes = 0;
  size_t rounded = (nbytes + ((size_t)1 << 21) - 1) & ~(((size_t)1 << 21) - 1);
  GT_CUDA_OK(ctx, cudaMalloc(&ctx->workspace, rounded));
  ctx->workspace_bytes = rounded;
  return GT_OK;
}

// ---- memory ---------------------------------------------------------------------------

// gt_malloc / gt_free keep freed blocks in host-side free lists keyed by (rounded) size and hand them out again
// without any CUDA call.  Every block is used on the context's compute stream, so a block freed after kernel A was
// enqueued and handed to kernel B is ordered by the stream itself; this is the ordering the stream-ordered pool
// underneath gave before, minus two driver calls per tensor, and, above all, minus the stream operations between
// consecutive kernel launches that kept one kernel's set-up from overlapping its predecessor's tail.  A training
// step asks for the same sizes every time, so after the first step every request is a hit.  The cache is emptied
// (blocks go back to the CUDA pool) when it holds more than GRADTUITY_ALLOC_CACHE_MB (default 65536) or when the
// pool cannot serve a new size.  GRADTUITY_NO_ALLOC_CACHE=1 turns it off.

extern "C" int gt_malloc(gt_ctx* ctx, size_t nbytes, void** ptr) {
  if (!ctx || !ptr) return GT_ERR_INVALID_ARG;
  *ptr = nullptr;
  if (nbytes == 0) nbytes = 16;
  BlockCache* bc = (BlockCache*)ctx->block_cache;
  const size_t rounded = (nbytes + 511) & ~(size_t)511;
  if (bc && bc->enabled) {
    std::lock_guard<std::mutex> guard(bc->lock);
    auto it = bc->free_by_size.find(rounded);
    if (it != bc->free_by_size.end() && !it->second.empty()) {
      *ptr = it->second.back();
      it->second.pop_back();
      bc->cached_bytes -= rounded;
      return GT_OK;
    }
  }
  cudaError_t e = cudaMallocAsync(ptr, rounded, ctx->stream);
  if (e == cudaErrorMemoryAllocation && bc && bc->enabled) {
    // the pool is exhausted while we sit on cached blocks of other sizes: give them back and try once more
    cudaGetLastError();
    std::lock_guard<std::mutex> guard(bc->lock);
    block_cache_flush(ctx, bc);
    cudaStreamSynchronize(ctx->stream);
    e = cudaMallocAsync(ptr, rounded, ctx->stream);
  }
  if (e == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    GT_FAIL(ctx, GT_ERR_NOMEM, "cudaMallocAsync(%zu bytes): out of memory", nbytes);
  }
  GT_CUDA_OK(ctx, e);
  if (bc && bc->enabled) {
    std::lock_guard<std::mutex> guard(bc->lock);
    bc->size_of[*ptr] = rounded;
  }
  return GT_OK;
}

extern "C" int gt_free(gt_ctx* ctx, void* ptr) {
  if (!ctx) return GT_ERR_INVALID_ARG;
  if (!ptr) return GT_OK;
  BlockCache* bc = (BlockCache*)ctx->block_cache;
  if (ctx->side_pending) {
    // The side stream may still use this block: join first if the block overlaps one that the pending side work noted
    // (or if its size is unknown: the block did not come from the cache).
    size_t size = 0;
    if (bc && bc->enabled) {
      std::lock_guard<std::mutex> guard(bc->lock);
      auto it = bc->size_of.find(ptr);
      if (it != bc->size_of.end()) size = it->second;
    }
    if (size == 0 || gt_side_touches(ctx, ptr, size)) gt_join_beside(ctx);
  }
  if (bc && bc->enabled) {
    std::lock_guard<std::mutex> guard(bc->lock);
    auto it = bc->size_of.find(ptr);
    if (it != bc->size_of.end()) {
      bc->free_by_size[it->second].push_back(ptr);
      bc->cached_bytes += it->second;
      if (bc->cached_bytes > bc->limit_bytes) block_cache_flush(ctx, bc);
      return GT_OK;
    }
  }
  GT_CUDA_OK(ctx, cudaFreeAsync(ptr, ctx->stream));
  return GT_OK;
}

extern "C" int gt_memset(gt_ctx* ctx, void* ptr, int value, size_t nbytes) {
  if (!ctx || (!ptr && nbytes)) return GT_ERR_INVALID_ARG;
  GT_CUDA_OK(ctx, cudaMemsetAsync(ptr, value, nbytes, ctx->stream));
  return GT_OK;
}

extern "C" int gt_memcpy_h2d(gt_ctx* ctx, void* dst, const void* src, size_t nbytes) {
  if (!ctx || ((!dst || !src) && nbytes)) return GT_ERR_INVALID_ARG;
  GT_CUDA_OK(ctx, cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyHostToDevice, ctx->stream));
  GT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
  return GT_OK;
}

extern "C" int gt_memcpy_d2h(gt_ctx* ctx, void* dst, const void* src, size_t nbytes) {
  if (!ctx || ((!dst || !src) && nbytes)) return GT_ERR_INVALID_ARG;
  gt_join_beside(ctx);
  GT_CUDA_OK(ctx, cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, ctx->stream));
  GT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
  return GT_OK;
}

extern "C" int gt_memcpy_h2d_async(gt_ctx* ctx, void* dst, const void* src, size_t nbytes) {
  if (!ctx || ((!dst || !src) && nbytes)) return GT_ERR_INVALID_ARG;
  GT_CUDA_OK(ctx, cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyHostToDevice, ctx->stream));
  return GT_OK;
}

extern "C" int gt_memcpy_d2h_async(gt_ctx* ctx, void* dst, const void* src, size_t nbytes) {
  if (!ctx || ((!dst || !src) && nbytes)) return GT_ERR_INVALID_ARG;
  gt_join_beside(ctx);
  GT_CUDA_OK(ctx, cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, ctx->stream));
  return GT_OK;
}

extern "C" int gt_memcpy_d2d(gt_ctx* ctx, void* dst, const void* src, size_t nbytes) {
  if (!ctx || ((!dst || !src) && nbytes)) return GT_ERR_INVALID_ARG;
  GT_CUDA_OK(ctx, cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToDevice, ctx->stream));
  return GT_OK;
}

extern "C" int gt_sync(gt_ctx* ctx) {
  if (!ctx) return GT_ERR_INVALID_ARG;
  gt_join_beside(ctx);
  GT_CUDA_OK(ctx, cudaStreamSynchronize(ctx->stream));
  return GT_OK;
}

extern "C" int gt_host_alloc(gt_ctx* ctx, size_t nbytes, void** ptr) {
  if (!ctx || !ptr) return GT_ERR_INVALID_ARG;
  GT_CUDA_OK(ctx, cudaMallocHost(ptr, nbytes ? nbytes : 16));
  return GT_OK;
}

extern "C" int gt_host_free(gt_ctx* ctx, void* ptr) {
  if (!ctx) return GT_ERR_INVALID_ARG;
  if (ptr) GT_CUDA_OK(ctx, cudaFreeHost(ptr));
  return GT_OK;
}

// ---- events ---------------------------------------------------------------------------

extern "C" int gt_event_create(gt_ctx* ctx, void** ev) {
  if (!ctx || !ev) return GT_ERR_INVALID_ARG;
  cudaEvent_t e;
  GT_CUDA_OK(ctx, cudaEventCreate(&e));
  *ev = (void*)e;
  return GT_OK;
}

extern "C" int gt_event_destroy(gt_ctx* ctx, void* ev) {
  if (!ctx || !ev) return GT_ERR_INVALID_ARG;
  GT_CUDA_OK(ctx, cudaEventDestroy((cudaEvent_t)ev));
  return GT_OK;
}

extern "C" int gt_event_record(gt_ctx* ctx, void* ev) {
  if (!ctx || !ev) return GT_ERR_INVALID_ARG;
  GT_CUDA_OK(ctx, cudaEventRecord((cudaEvent_t)ev, ctx->stream));
  return GT_OK;
}

extern "C" int gt_event_elapsed_ms(gt_ctx* ctx, void* start, void* stop, float* ms) {
  if (!ctx || !start || !stop || !ms) return GT_ERR_INVALID_ARG;
  GT_CUDA_OK(ctx, cudaEventSynchronize((cudaEvent_t)stop));
  GT_CUDA_OK(ctx, cudaEventElapsedTime(ms, (cudaEvent_t)start, (cudaEvent_t)stop));
  return GT_OK;
}
