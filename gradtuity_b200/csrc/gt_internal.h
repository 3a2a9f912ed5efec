// Internal declarations shared by the translation units of libgt_b200.so.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "gt_b200.h"

typedef CUresult (*gt_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                       const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                       const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct gt_ctx {
  int device;
  int sm_count;
  cudaStream_t stream;        // compute stream (non-blocking)
  int* d_status;              // device status word written by bounded waits that ran out; the allocation is 4 KB:
                              // ints 16..271 are the "C tile zeroed" flags of the GEMM's last-wave split
  int tail_epoch;             // value those flags take in the next launch that uses them
  int* d_sched;               // ring of GT_SCHED_RING work-unit counters for dynamically scheduled launches (zero when idle)
  long long sched_seq;        // launches that took a counter so far
  int dist_active;            // a process group exists: collectives may hold SMs while GEMMs are launched
  void* block_cache;          // host-side free lists of gt_malloc blocks, by size (gt_runtime.cu)
  cudaStream_t h2d_stream, d2h_stream;   // copy streams of gt_gemm_host (created on first use)
  cudaEvent_t host_ev[8];                // its events
  gt_encode_tiled_fn encode_tiled;
  void* workspace;            // scratch for operand splitting (TF32X3) and split-K partials
  size_t workspace_bytes;
  cudaStream_t scratch_stream;   // stream of the last launch that used the workspace or the tail flags (null: none yet)
  cudaEvent_t scratch_event;     // orders a launch on another stream behind that one (created on first switch)
  cudaStream_t side_stream;      // second compute stream for small memory-bound kernels that run beside the GEMMs reading the same
  cudaEvent_t side_fork;         // input (gt_colsum_acc_beside): forks from `stream` at side_fork, joins again at side_done
  cudaEvent_t side_done;
  int side_pending;              // work was put on side_stream since the last gt_join_beside
  cudaStream_t side_saved;       // the compute stream while gt_beside_begin has `stream` point at side_stream (null otherwise)
  struct { const char* ptr; size_t nbytes; } side_blocks[16];   // memory the pending side work touches and that may be freed before the join
  int side_nblocks;              // entries in use; -1: too many to list, any gt_free joins
  void* attn_schedules;          // item tables of the attention kernels, by problem shape (gt_attn.cu)
  int64_t launches;
  int tma_round;              // 1: tensor maps use the TFLOAT32 data type (TMA rounds), 0: FLOAT32
  char last_error[256];
};

#define GT_SCHED_RING 1024     // launch n uses counter n % 1024 and zeroes counter (n + 512) % 1024 for a later launch

#define GT_CUDA_OK(ctx, expr)                                                              \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    if (_e != cudaSuccess) {                                                               \
      snprintf((ctx)->last_error, sizeof((ctx)->last_error), "%s: %s (%s:%d)", #expr,      \
               cudaGetErrorString(_e), __FILE__, __LINE__);                                \
      return GT_ERR_CUDA;                                                                  \
    }                                                                                      \
  } while (0)

#define GT_FAIL(ctx, code, ...)                                                            \
  do {                                                                                     \
    snprintf((ctx)->last_error, sizeof((ctx)->last_error), __VA_ARGS__);                   \
    return (code);                                                                         \
  } while (0)

// Opt a kernel in to `bytes` of dynamic shared memory, once per (kernel, device): the attribute belongs to the
// device's copy of the function, so a second context on another device of the same process needs its own call.
// Keyed by the kernel's address: kernels of one signature share a function-pointer TYPE, so a static flag inside
// a template or a generic lambda would be shared between them.
int gt_smem_opt_in(gt_ctx* ctx, const void* kernel, int bytes);

// Frees the attention kernels' item tables (gt_destroy).
void gt_attn_release(gt_ctx* ctx);

// Notes a block that pending side-stream work reads or writes and whose owner may free it before the join: gt_free of a
// block that overlaps a noted one joins first; gt_free of anything else does not have to.
void gt_side_note_block(gt_ctx* ctx, const void* ptr, size_t nbytes);
bool gt_side_touches(gt_ctx* ctx, const void* ptr, size_t nbytes);

// Makes ctx->stream wait for whatever was put on the side stream (gt_colsum_acc_beside); no-op when nothing was.
extern "C" int gt_join_beside(gt_ctx* ctx);
#define GT_SMEM_OPT_IN(ctx, kern, bytes)                                        \
  do {                                                                          \
    int _gt_rc = gt_smem_opt_in((ctx), (const void*)(kern), (int)(bytes));      \
    if (_gt_rc != GT_OK) return _gt_rc;                                         \
  } while (0)

// ---- programmatic dependent launch -------------------------------------------------------------------------
// A kernel launched with gt_launch_overlapped may have its CTAs placed on SMs while the previous kernel of the
// stream is still finishing (as that kernel's CTAs leave), run its set-up there (barrier initialisation, tensor
// memory allocation, index arithmetic) and must then call gt_wait_for_previous_kernel() before it touches global
// memory: the call returns once the previous kernel has completed and its writes are visible.  A kernel calls
// gt_let_next_kernel_start() early so that its successor may be placed this way; both calls are no-ops in a
// launch that has no such dependency.  Hides the launch latency and the prologue of ~300 short kernels per
// training step.  GRADTUITY_NO_PDL=1 launches everything in plain stream order.
#ifdef __CUDACC__
__device__ __forceinline__ void gt_let_next_kernel_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void gt_wait_for_previous_kernel() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

inline bool gt_pdl_enabled() {
  static const bool on = getenv("GRADTUITY_NO_PDL") == nullptr;
  return on;
}

template <class... KArgs, class... Args>
inline cudaError_t gt_launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = gt_pdl_enabled() ? 1 : 0;
  cfg.attrs = &attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// One GEMM problem, fully resolved (used by both kernels).
struct gt_gemm_args {
  int layout, epilogue, precision, accumulate, flags;
  int64_t M, N, K;
  const float* A; int64_t lda, sA0, sA1;
  const float* B; int64_t ldb, sB0, sB1;
  float* C; int64_t ldc, sC0, sC1;
  int64_t batch0, batch1;
  const float* bias;
  float* aux;
  float alpha;
  float* colsum = nullptr;   // GT_EPI_GELU_GRAD only: length N, receives += the column sums of the result
};

// The context's shared scratch (the workspace and the last-wave flags behind d_status) serves one launch at a
// time.  Launches on one stream are ordered by the stream; a launch on a DIFFERENT stream than the previous
// user is made to wait for everything enqueued so far on that stream.  Call before the launch that uses it.
int gt_scratch_acquire(gt_ctx* ctx, cudaStream_t stream);
// Call when an entry point that was given a caller's stream returns: records, on that stream, the point the next
// user of the scratch on another stream has to wait for.  The caller's stream is never touched again afterwards,
// so it may be destroyed once its work is done.
int gt_scratch_release(gt_ctx* ctx, cudaStream_t stream);
// gt_scratch_acquire + make the workspace at least nbytes large.
int gt_workspace_reserve(gt_ctx* ctx, size_t nbytes, cudaStream_t stream);
int gt_gemm_validate(gt_ctx* ctx, const gt_gemm_args& g);
int gt_gemm_fma_launch(gt_ctx* ctx, const gt_gemm_args& g, cudaStream_t stream);
int gt_gemm_umma_launch(gt_ctx* ctx, const gt_gemm_args& g, cudaStream_t stream);
bool gt_gemm_umma_eligible(const gt_gemm_args& g);

// GELU, tanh form (gradtuity/kernels_cuda/elemwise_kernels.py:104-137):
//     gelu(x) = 0.5 x (1 + tanh(u)),  u = sqrt(2/pi) (x + 0.044715 x^3).
// With tanh(u) = 1 - 2 r, r = 1 / (1 + e^(2u)), this is gelu(x) = x - x r = x s with s = 1 - r the logistic function of
// 2u, and d/dx gelu = s + x s r (2 u'), 2u' = 2 sqrt(2/pi) (1 + 3 * 0.044715 x^2).  The same function as the
// reference's two-branch form, in 7 (forward) and 12 (derivative) instructions with one ex2 and one rcp each: the
// GEMM epilogues that apply them are bound by the instructions they issue.  e^(2u) overflowing to +inf gives r = 0
// (gelu = x), underflowing to 0 gives r = 1 (gelu = 0); both products with r stay finite.
#ifdef __CUDACC__
__device__ __forceinline__ float gt_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }
__device__ __forceinline__ float gt_rcp(float x) { float y; asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

// r = 1 / (1 + e^(2u)); the constants fold 2 sqrt(2/pi) log2(e) into the cubic's coefficients
__device__ __forceinline__ float gt_gelu_r(float x, float x2) {
  const float w = x * fmaf(x2, 0.1029432395800235f, 2.302208198144325f);
  return gt_rcp(1.0f + gt_ex2(w));
}

__device__ __forceinline__ float gt_gelu_tanh_grad(float x) {
  const float x2 = x * x;
  const float r = gt_gelu_r(x, x2);
  const float s = 1.0f - r;
  const float du2 = fmaf(x2, 0.21406444881780076f, 1.5957691216057308f);
  return fmaf(x * s, r * du2, s);
}

__device__ __forceinline__ float gt_gelu_tanh(float x) {
  const float r = gt_gelu_r(x, x * x);
  return fmaf(-x, r, x);
}
#endif
