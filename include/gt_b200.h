/*
 * gt_b200.h — C ABI of libgt_b200.so, the B200 (sm_100a) GEMM subsystem for the
 * Gradtuity autograd engine.
 *
 * The library replaces, for the matmul family only, what the reference engine reaches
 * through `gradtuity/kernels.py` (the `kernel[grid](...)` dispatch proxy) and
 * `gradtuity/kernels_cuda/matmul_kernels.py` / `gradtuity/kernels_triton/matmul_kernels.py`
 * (the five GEMM kernels), plus the thin slices of `gradtuity/cuda_mem.py` and
 * `gradtuity/dist/nccl.py` the path needs.  It is loaded from Python with `ctypes.CDLL`
 * exactly as the reference loads libcudart / libcuda / libnccl.
 *
 * Conventions
 *  - every function returns an int status: 0 = GT_OK, negative = GT_ERR_* (never aborts);
 *  - all matrices are fp32, row-major; leading dimensions and batch strides are in ELEMENTS;
 *  - device pointers are plain `void*` / `float*`; the library never owns memory handed to it;
 *  - `stream` arguments are `cudaStream_t` passed as `void*`; NULL selects the context's
 *    own compute stream (see gt_ctx_stream);
 *  - one caller thread per context.
 */
#ifndef GT_B200_H
#define GT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct gt_ctx gt_ctx;

/* ---- status codes ------------------------------------------------------------------- */
#define GT_OK                 0
#define GT_ERR_INVALID_ARG   -1   /* null pointer, negative size, bad enum                  */
#define GT_ERR_CUDA          -2   /* a CUDA runtime/driver call failed (see gt_last_error)  */
#define GT_ERR_UNSUPPORTED   -3   /* valid request this build cannot serve                  */
#define GT_ERR_TIMEOUT       -4   /* a bounded device-side wait ran out (status word)       */
#define GT_ERR_NOMEM         -5
#define GT_ERR_NCCL          -6
#define GT_ERR_TOO_LARGE     -7   /* size beyond a documented fixed maximum                 */
#define GT_ERR_NOT_INIT      -8

/* ---- enums -------------------------------------------------------------------------- */
/* Operand layouts.  Logical op is always C[M,N] (+)= op(A)[M,K] * op(B)[K,N].
 *   NN: A stored (M,K), B stored (K,N)   — reference `matmul_kernel`, strides (K,1,N,1)
 *       (gradtuity/tensor.py:576-593)
 *   NT: A stored (M,K), B stored (N,K)   — reference `matmul_nt_acc_kernel`
 *       (gradtuity/kernels_triton/matmul_kernels.py:250-323) and the swapped-stride
 *       `matmul_kernel` call of `linear_tied` (gradtuity/tensor.py:1716-1732)
 *   TN: A stored (K,M), B stored (K,N)   — reference `matmul_tn_acc_kernel`
 *       (gradtuity/kernels_triton/matmul_kernels.py:327-400)                              */
#define GT_LAYOUT_NN 0
#define GT_LAYOUT_NT 1
#define GT_LAYOUT_TN 2

/* Epilogues.  v = alpha * acc (+ bias[n]);  aux (if non-NULL) receives v before the
 * activation;  then the activation / mask;  then C = v or C += v.
 *   NONE        reference matmul_kernel
 *   BIAS        reference matmul_bias_kernel        (kernels_triton/matmul_kernels.py:94-168)
 *   BIAS_RELU   reference matmul_bias_relu_kernel   (kernels_triton/matmul_kernels.py:172-246)
 *   BIAS_GELU   matmul_bias + gelu_kernel, tanh form (kernels_cuda/elemwise_kernels.py:104-125)
 *   CAUSAL      per batch slice, entries with n > m are written as GT_CAUSAL_MASK_VALUE
 *               (the NEG_INF of reference causal_mask_inplace, gradtuity/tensor.py:1316);
 *               tiles wholly above the diagonal skip the contraction.
 * Two kinds READ aux (same shape and leading dimension as C) instead of writing it:
 *   BIAS_ADD    C = alpha * acc + bias[n] + aux[m, n]: a Linear layer and the residual add that follows
 *               it in one launch (gpt2/model.py:64-71 adds the branch output to the stream afterwards)
 *   GELU_GRAD   C = alpha * acc * gelu'(aux[m, n]), aux = the stored pre-activation: dX of the second
 *               MLP layer and the GELU backward that follows it (gelu_backward_kernel,
 *               kernels_cuda/elemwise_kernels.py:127-137) in one launch; no bias.
 * Both need the tensor-core path with a 16-byte aligned C and aux (else GT_ERR_UNSUPPORTED).     */
#define GT_EPI_NONE       0
#define GT_EPI_BIAS       1
#define GT_EPI_BIAS_RELU  2
#define GT_EPI_BIAS_GELU  3
#define GT_EPI_CAUSAL     4
#define GT_EPI_BIAS_ADD   5
#define GT_EPI_GELU_GRAD  6
#define GT_CAUSAL_MASK_VALUE (-1.0e9f)

/* Multiply precision (accumulation is always fp32).
 *   TF32    one tcgen05.mma kind::tf32 per k-step; parity target: reference Triton path
 *   TF32X3  operands split hi+lo, three MMAs per k-step; parity target: reference CUDA-C
 *           path (scalar fp32 FMA) and the float64 oracle
 *   FP32    plain fp32 FMA on CUDA cores (the kernel that also serves operands TMA cannot
 *           describe: base not 16-byte aligned or leading dimension not a multiple of 4)   */
#define GT_PREC_TF32    0
#define GT_PREC_TF32X3  1
#define GT_PREC_FP32    2

/* ---- context / runtime (replaces the slices of gradtuity/cuda_mem.py:30-153 and
 *      gradtuity/cuda_driver.py:214-247,472-511 that the GEMM path uses) ---------------- */
int         gt_init(int device, gt_ctx** out);
int         gt_destroy(gt_ctx* ctx);
const char* gt_strerror(int status);
const char* gt_last_error(gt_ctx* ctx);            /* detail text of the last failing call */
void*       gt_ctx_stream(gt_ctx* ctx);            /* the context's compute stream         */
int         gt_sm_count(gt_ctx* ctx);
/* Synchronises the compute stream, then returns the device status word in *status
 * (0, or GT_ERR_TIMEOUT if a kernel's bounded wait ran out) and clears it.               */
int         gt_device_status(gt_ctx* ctx, int* status);

/* gt_malloc / gt_free: blocks come from the CUDA stream-ordered pool, ordered on the context's compute stream; freed
 * blocks are kept in host-side free lists by size and handed out again without a CUDA call (GRADTUITY_NO_ALLOC_CACHE=1
 * turns that off, GRADTUITY_ALLOC_CACHE_MB bounds it).  A block must only be used by work on the compute stream, or by
 * work ordered behind it.                                                                                            */
int gt_malloc(gt_ctx* ctx, size_t nbytes, void** ptr);
int gt_free(gt_ctx* ctx, void* ptr);
int gt_memset(gt_ctx* ctx, void* ptr, int value, size_t nbytes);
int gt_memcpy_h2d(gt_ctx* ctx, void* dst, const void* src, size_t nbytes);   /* blocking   */
int gt_memcpy_d2h(gt_ctx* ctx, void* dst, const void* src, size_t nbytes);   /* blocking   */
int gt_memcpy_d2d(gt_ctx* ctx, void* dst, const void* src, size_t nbytes);   /* async      */
int gt_sync(gt_ctx* ctx);
int gt_host_alloc(gt_ctx* ctx, size_t nbytes, void** ptr);  /* pinned host memory           */
int gt_host_free(gt_ctx* ctx, void* ptr);
int gt_memcpy_h2d_async(gt_ctx* ctx, void* dst, const void* src, size_t nbytes);
int gt_memcpy_d2h_async(gt_ctx* ctx, void* dst, const void* src, size_t nbytes);

/* cuEvent timing, as gradtuity/cuda_driver.py:472-511 (EventTimer). */
int gt_event_create(gt_ctx* ctx, void** ev);
int gt_event_destroy(gt_ctx* ctx, void* ev);
int gt_event_record(gt_ctx* ctx, void* ev);                 /* on the compute stream       */
int gt_event_elapsed_ms(gt_ctx* ctx, void* start, void* stop, float* ms); /* syncs on stop */

/* ---- the GEMM family ------------------------------------------------------------------
 * gt_gemm replaces the five reference kernels
 *   matmul_kernel / matmul_bias_kernel / matmul_bias_relu_kernel /
 *   matmul_nt_acc_kernel / matmul_tn_acc_kernel
 * (gradtuity/kernels_triton/matmul_kernels.py:18-400, gradtuity/kernels_cuda/matmul_kernels.py:21-236)
 * and their launch wrappers (gradtuity/kernels_cuda/matmul_kernels.py:254-341).
 *   accumulate = 0 : C  = epilogue(alpha * A*B)      (reference forward kernels)
 *   accumulate = 1 : C += epilogue(alpha * A*B)      (reference *_acc kernels)
 *   bias : length N, required for the BIAS* epilogues, else NULL
 *   aux  : optional (M,N) buffer, leading dimension ldc, that receives the pre-activation
 *   stream : NULL = the context's compute stream.  One context serves one stream at a time: the scratch the
 *            context owns (3xTF32 operand copies, split-K partials, last-wave flags) is handed from stream to
 *            stream in order (a launch on another stream than the previous user waits, on the device, for what
 *            that stream had been given); a caller's stream is not touched again after the call returns.
 * Kernel choice (tile 128 x 64 / 128 / 256 on one CTA, 256 x 256 on one CTA or on a CTA pair, K shares) follows
 * the problem's shape; GRADTUITY_GEMM_TRACE=1 prints it per launch, GRADTUITY_GEMM_PAIR=0|1,
 * GRADTUITY_GEMM_DETERMINISTIC=1, GRADTUITY_GEMM_NO_TAIL_SPLIT=1 and GRADTUITY_NO_PDL=1 override parts of it.
 */
int gt_gemm(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
            const float* A, int64_t lda, const float* B, int64_t ldb,
            float* C, int64_t ldc, const float* bias, float* aux,
            float alpha, int accumulate, int epilogue, int precision, void* stream);

/* Strided-batched form: batch0 x batch1 independent problems; slice (i1, i0) of operand X
 * starts at X + i0*strideX0 + i1*strideX1.  One launch replaces the per-slice Python loops of
 * Tensor.bmm (gradtuity/tensor.py:820-841 forward, :848-893 backward), and two batch strides
 * let the per-head Q/K/V slices of a (B,S,H,D) projection be read in place, which removes
 * transpose4d_12 / transpose4d_last2 (gradtuity/nn.py:534-539).                            */
int gt_gemm_batched(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                    const float* A, int64_t lda, int64_t strideA0, int64_t strideA1,
                    const float* B, int64_t ldb, int64_t strideB0, int64_t strideB1,
                    float* C, int64_t ldc, int64_t strideC0, int64_t strideC1,
                    int64_t batch0, int64_t batch1,
                    const float* bias, float* aux, float alpha, int accumulate,
                    int epilogue, int precision, void* stream);

/* gt_gemm_batched with structure hints (bit flags) for the attention products, where P and dS are
 * zero above the diagonal of every (T, T) slice:
 *   GT_GEMM_A_LOWER             A is stored (M, K), square, and A[m, k] == 0 for k > m: row tile tm
 *                               contracts only over k <= its last row        (O = P V, dQ = dS K)
 *   GT_GEMM_AT_LOWER            A is stored (K, M), square, and A[k, m] == 0 for k < m: row tile tm
 *                               contracts only over k >= its first row       (dV = P^T dO, dK = dS^T Q)
 *   GT_GEMM_CAUSAL_SKIP_MASKED  with GT_EPI_CAUSAL: 128-row tiles wholly above the diagonal are not
 *                               written at all (their contents are undefined); for consumers that
 *                               never read above the diagonal
 * The hints only remove work whose result is known to be zero / unused; results are unchanged.
 *   GT_GEMM_BIAS_PER_BATCH      (not a hint) bias holds batch0 * batch1 rows of N: batch entry
 *                               (i0, i1) uses row i0 + i1 * batch0 instead of one row shared by all.
 * Batch strides of 0 are allowed.  An operand with stride 0 is shared by the batch entries (the q, k
 * and v projections of one input are one launch with strideA0 = 0).  A C with stride 0 receives the
 * SUM over the batch entries: that needs accumulate = 1, no epilogue, and the tensor-core path.  */
#define GT_GEMM_A_LOWER             1
#define GT_GEMM_AT_LOWER            2
#define GT_GEMM_CAUSAL_SKIP_MASKED  4
#define GT_GEMM_BIAS_PER_BATCH      8
int gt_gemm_batched_ex(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                       const float* A, int64_t lda, int64_t strideA0, int64_t strideA1,
                       const float* B, int64_t ldb, int64_t strideB0, int64_t strideB1,
                       float* C, int64_t ldc, int64_t strideC0, int64_t strideC1,
                       int64_t batch0, int64_t batch1,
                       const float* bias, float* aux, float alpha, int accumulate,
                       int epilogue, int precision, int flags, void* stream);

/* gt_gemm with GT_EPI_GELU_GRAD that also produces the bias gradient of the layer whose pre-activation `pre` is:
 *   C = alpha * op(A) op(B) * gelu'(pre[m, n]),   colsum[n] += sum over m of C[m, n]
 * One launch stands where the reference runs the dX product, the GELU backward (gradtuity/tensor.py:954-984) and the
 * bias-gradient reduction of the first Linear layer (gradtuity/tensor.py:1781-1904) as separate passes: the sums are
 * taken from the output tiles while they are still in shared memory.  pre has C's shape and leading dimension; C and
 * pre must be 16-byte aligned with ldc a multiple of 4 and the problem must take the tensor-core path (else
 * GT_ERR_UNSUPPORTED).  The additions into colsum are atomic (run-to-run differences in its last bits);
 * GRADTUITY_GEMM_DETERMINISTIC=1 takes the sums with the ordered column-sum kernel after the product instead.
 * Runs on the context's compute stream.                                                                        */
int gt_gemm_gelu_grad_colsum(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                             const float* A, int64_t lda, const float* B, int64_t ldb,
                             float* C, int64_t ldc, const float* pre, float* colsum,
                             float alpha, int precision);

/* 3xTF32 GEMM for callers that must not cause a device allocation (no counterpart in the
 * reference, which allocates per tensor).  Same result as gt_gemm(..., GT_PREC_TF32X3) for a
 * single, non-batched problem without an aux output, but the hi/lo operand copies live in a
 * fixed 32 MiB array inside the library image rather than in a workspace that grows with
 * cudaMalloc.  Meant for callers that have given all device memory to their own pool, or that
 * cannot take the synchronisation an allocation may bring in the middle of a timed step.
 *   - limit: 2 * (rows(A) * cols4(A) + rows(B) * cols4(B)) <= 8 Mi floats, cols4 = columns
 *     rounded up to a multiple of 4 (for example M = N = K = 1024, or 2048 x 1024 x 512);
 *     larger problems return GT_ERR_TOO_LARGE and launch nothing;
 *   - any operand alignment and leading dimension is accepted (the split packs both operands);
 *   - the first call on each device looks up the array's device address (and, when the CUDA
 *     module is loaded lazily, may be the moment the driver places the 32 MiB array on that
 *     GPU): make that call before starting any stream capture and outside any timed region;
 *     every later call on the device touches no allocator at all;
 *   - all calls share the array: calls whose kernels may overlap on the GPU race on it.    */
#define GT_NOALLOC_SCRATCH_BYTES (32u << 20)
int gt_gemm_3xtf32_noalloc(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                           const float* A, int64_t lda, const float* B, int64_t ldb,
                           float* C, int64_t ldc, const float* bias, float alpha,
                           int accumulate, int epilogue, void* stream);

/* ---- fused causal attention (head dimension 64, sequence length a multiple of 128) ----------
 * The reference composes attention from transposes, two bmm calls, scale_inplace and
 * softmax_with_causal_mask (gradtuity/nn.py:511-554) and keeps the (B, H, T, T) scores in
 * memory; these entry points compute the same result without materialising them.
 * q, k, v, o (and dq, dk, dv, d_o) are (B, T, H * 64) row-major: the projection outputs, heads
 * side by side, read in place.  scale multiplies Q K^T before the softmax.  lse (B, H, T)
 * receives each row's log-sum-exp of the scaled, masked scores (needed by the backward).
 * p_out, when not NULL, also receives the probabilities P (B, H, T, T): rows are written up to
 * the end of their 128-wide diagonal block, exact zeros right of the diagonal inside it.
 * Returns GT_ERR_UNSUPPORTED for another head dimension or sequence length.                  */
int gt_attention_forward(gt_ctx* ctx, float* o, float* p_out, float* lse, const float* q,
                         const float* k, const float* v, int64_t B, int64_t T, int64_t H,
                         int64_t D, float scale, void* stream);
/* Backward of the above from q, k, v, o, lse and the upstream gradient d_o: two launches, one that
 * owns blocks of 128 queries (dQ, and delta (B, H, T) = rowsum(d_o * o), a scratch output the
 * second launch reads) and one that owns blocks of 128 keys (dK, dV).  P is recomputed from the
 * saved statistics; no (B, H, T, T) buffer is read or written.  acc_* = 1 adds to the gradient
 * buffer (dX += ..., the reference's accumulation contract, gradtuity/tensor.py:152-161), 0
 * overwrites it.                                                                             */
int gt_attention_backward(gt_ctx* ctx, float* dq, float* dk, float* dv, const float* d_o,
                          const float* q, const float* k, const float* v, const float* o,
                          const float* lse, float* delta, int64_t B, int64_t T, int64_t H,
                          int64_t D, float scale, int acc_dq, int acc_dk, int acc_dv,
                          void* stream);
/* The same; a non-null dbq / dbk / dbv (H * D floats each) also receives, added to its contents, the column sums over all
 * tokens of what this call computed for dQ / dK / dV: the bias gradients of the projections that produced q, k and v
 * (gradtuity/tensor.py:1673-1679 takes them with a separate pass over each gradient). */
int gt_attention_backward_bias(gt_ctx* ctx, float* dq, float* dk, float* dv, float* dbq, float* dbk, float* dbv,
                               const float* d_o, const float* q, const float* k, const float* v, const float* o,
                               const float* lse, float* delta, int64_t B, int64_t T, int64_t H, int64_t D, float scale,
                               int acc_dq, int acc_dk, int acc_dv, void* stream);

/* The GEMM on HOST buffers: hA, hB, hC, h_bias point to host memory (pinned, for the copies to
 * overlap); leading dimensions in elements.  B is uploaded once, A in `chunks` row blocks of C; the
 * upload of one block, the product of the previous one and the download of the one before that run
 * concurrently, so the call costs about max(upload, download) of PCIe time instead of their sum.
 * It returns when hC is complete.  Epilogues: NONE, BIAS, BIAS_RELU, BIAS_GELU.  The host-data
 * counterpart of `Tensor(list).matmul(...).to_list()` (gradtuity/tensor.py:192-220, 530-657).   */
int gt_gemm_host(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                 const float* hA, int64_t lda, const float* hB, int64_t ldb, float* hC, int64_t ldc,
                 const float* h_bias, float alpha, int epilogue, int precision, int chunks);

/* Which kernel a call with these arguments would run: 0 = tcgen05/TMA kernel, 1 = fp32 FMA
 * kernel.  No launch.                                                                       */
int gt_gemm_path(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                 const float* A, int64_t lda, const float* B, int64_t ldb,
                 const float* C, int64_t ldc, int precision, int* path);

/* Failure-detection self test (no counterpart in the reference): launches one CTA that waits, with
 * the library's bounded polling loop and a limit of `limit_cycles` SM cycles, on a barrier nothing
 * arrives on.  The wait gives up and records GT_ERR_TIMEOUT, which the next gt_device_status returns;
 * the context stays usable.                                                                   */
int gt_selftest_bounded_wait(gt_ctx* ctx, int64_t limit_cycles);

/* Number of kernels this library has launched on behalf of `ctx` since gt_init. */
int gt_launch_count(gt_ctx* ctx, int64_t* count);

/* ---- small kernels beside the GEMMs in the autograd closures -------------------------
 * fp32, element-wise or reductions, all on the context's compute stream.  They restate
 *   add_kernel / add_inplace_kernel / mul_kernel / mul_scalar_kernel / relu_kernel /
 *   relu_mask_mul_kernel / gelu_kernel / gelu_backward_kernel
 *     (gradtuity/kernels_cuda/elemwise_kernels.py:20-141),
 *   fill_kernel (gradtuity/kernels_cuda/optim_kernels.py), sum_all_kernel, sum_axis0_kernel,
 *   add_scalar_inplace_kernel, add_bias_kernel (gradtuity/kernels_cuda/reduce_kernels.py).
 * `accumulate` = 1 turns `out = f(...)` into `out += f(...)`, which is how the reference's
 * backward closures use them (accum_grad, gradtuity/tensor.py:158-161).                    */
int gt_fill(gt_ctx* ctx, float* out, float value, int64_t n);
int gt_add(gt_ctx* ctx, float* out, const float* a, const float* b, int64_t n, int accumulate);
int gt_mul(gt_ctx* ctx, float* out, const float* a, const float* b, int64_t n, int accumulate);
int gt_scale(gt_ctx* ctx, float* out, const float* a, float s, int64_t n, int accumulate);
int gt_relu(gt_ctx* ctx, float* out, const float* a, int64_t n);
int gt_relu_mask_mul(gt_ctx* ctx, float* out, const float* dy, const float* y, int64_t n, int accumulate);
int gt_gelu(gt_ctx* ctx, float* out, const float* a, int64_t n);
int gt_gelu_backward(gt_ctx* ctx, float* dx, const float* dy, const float* x, int64_t n, int accumulate);
int gt_add_scalar(gt_ctx* ctx, float* dst, const float* scalar, int64_t n);        /* dst[i] += *scalar */
int gt_add_bias(gt_ctx* ctx, float* out, const float* x, const float* bias, int64_t rows, int64_t cols);
int gt_sum_all(gt_ctx* ctx, float* out, const float* x, int64_t n, int accumulate); /* deterministic */
int gt_colsum_acc(gt_ctx* ctx, float* db, const float* dy, int64_t rows, int64_t cols, int64_t ld); /* db[c] += sum_r dy[r,c] */
/* The same sums put on a second stream of the context that forks from the compute stream at this call, so that they run
 * beside the kernels launched next (the dX and dW GEMMs of the same Linear layer, which read the same dy) instead of in
 * front of them.  gt_join_beside makes the compute stream wait for every such launch: call it before dy is freed or
 * rewritten and before db is read by anything but another gt_colsum_acc_beside.  gt_sync, gt_device_status and the
 * device-to-host copies join by themselves.  GRADTUITY_NO_SIDE_STREAM=1 turns the pair into gt_colsum_acc and a no-op. */
int gt_colsum_acc_beside(gt_ctx* ctx, float* db, const float* dy, int64_t rows, int64_t cols, int64_t ld);
/* `batch` matrices dy + i * dy_stride (floats) summed into db + i * db_stride in ONE launch on the side stream. */
int gt_colsum_acc_batched_beside(gt_ctx* ctx, float* db, int64_t db_stride, const float* dy, int64_t dy_stride,
                                 int64_t rows, int64_t cols, int64_t ld, int64_t batch);
int gt_join_beside(gt_ctx* ctx);
/* Everything the context launches between the two calls goes to the side stream, ordered behind what the compute stream
 * holds at the begin; gt_join_beside orders the compute stream behind it again.  Meant for memory-bound work whose
 * results the next kernels do not need (AdamW of the later layers beside the first layers of the next forward pass).
 * Allocate nothing in between.  What the side work touches must stay allocated until the join: the caller keeps it
 * alive, or notes it with gt_beside_touches, after which a gt_free of an overlapping block joins by itself (a gt_free of
 * any other block of this context's allocator does not). */
int gt_beside_begin(gt_ctx* ctx);
int gt_beside_end(gt_ctx* ctx);
int gt_beside_touches(gt_ctx* ctx, const void* ptr, size_t nbytes);
int gt_repack_rows(gt_ctx* ctx, float* dst, int64_t ld_dst, const float* src, int64_t ld_src, int64_t rows, int64_t cols); /* copy rows to another pitch */
/* conv2d as im2col + GEMM (gradtuity/tensor.py:1906-2167; im2col_kernel_2d / col2im_kernel of
 * kernels_cuda/conv_kernels.py).  x is (N, C, H, W); col is (N * H_out * W_out, C * kH * kW) with rows
 * ld_col floats apart, H_out = (H + 2 pad - kH) / stride + 1.  gt_col2im is the adjoint: dx (+)= ...   */
int gt_im2col(gt_ctx* ctx, float* col, int64_t ld_col, const float* x, int64_t N, int64_t C, int64_t H, int64_t W,
              int64_t kH, int64_t kW, int64_t stride, int64_t pad);
int gt_col2im(gt_ctx* ctx, float* dx, const float* dcol, int64_t ld_col, int64_t N, int64_t C, int64_t H, int64_t W,
              int64_t kH, int64_t kW, int64_t stride, int64_t pad, int accumulate);
/* maxpool2d_forward / backward (gradtuity/tensor.py:2169-2260).  idx holds, per output element, the offset
 * of the winning input inside its (H, W) plane, float-encoded; the backward adds dy there (dx must hold
 * the gradient accumulated so far, zeros for a fresh one).                                           */
int gt_maxpool2d(gt_ctx* ctx, float* out, float* idx, const float* x, int64_t N, int64_t C, int64_t H, int64_t W,
                 int64_t kH, int64_t kW, int64_t stride_h, int64_t stride_w);
int gt_maxpool2d_backward(gt_ctx* ctx, float* dx, const float* dy, const float* idx, int64_t planes, int64_t HW, int64_t HWo);

/* ---- the non-GEMM kernels of the GPT-2 training step -----------------------------------
 * fp32, memory-bound, on the context's compute stream.  Each restates the reference kernel named
 * beside it; differences are noted.
 *   gt_softmax(causal=0)          softmax_forward_kernel             kernels_cuda/softmax_kernels.py:22-58
 *   gt_softmax(causal=1)          softmax_with_causal_mask_forward   kernels_cuda/softmax_kernels.py:94-129
 *                                 (masked outputs exactly 0; masked inputs are never read)
 *                                 causal=2: as 1, but zeros are written only up to the end of the row's
 *                                 128-wide diagonal block (for GT_GEMM_A_LOWER / AT_LOWER consumers)
 *   gt_softmax_backward           softmax_backward_kernel            kernels_cuda/softmax_kernels.py:60-92
 *                                 (writes dx; `scale` folds the 1/sqrt(d) of attention; causal=1 reads
 *                                  only the kept columns and writes 0 elsewhere)
 *   gt_layernorm(_backward)       layernorm_fwd/bwd_kernel           kernels_cuda/layernorm_kernels.py
 *                                 (saves mean and rstd, recomputes x-hat; dgamma/dbeta by block partials)
 *   gt_embedding(_backward)       embedding_gather / scatter_add     kernels_cuda/gather_kernels.py
 *                                 (indices are floats; out-of-range indices set the status word)
 *   gt_cross_entropy(_backward)   cross_entropy_forward/backward     kernels_cuda/loss_kernels.py
 *                                 (keeps per-row log-sum-exp for the backward; deterministic mean)
 *   gt_adamw                      adamw_step_kernel                  kernels_cuda/optim_kernels.py:23-46
 *   gt_sumsq / gt_clip_scale / gt_scale_by_device_scalar            optim/utils.py:15-52 without host reads
 *   gt_transpose12                transpose4d_12_kernel              kernels_cuda/mask_kernels.py        */
int gt_softmax(gt_ctx* ctx, float* y, const float* x, int64_t rows, int64_t cols, int causal);
int gt_softmax_backward(gt_ctx* ctx, float* dx, const float* y, const float* dy, int64_t rows, int64_t cols,
                        int causal, float scale);
int gt_layernorm(gt_ctx* ctx, float* y, float* mean, float* rstd, const float* x, const float* gamma,
                 const float* beta, int64_t N, int64_t H, float eps);
int gt_layernorm_backward(gt_ctx* ctx, float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
                          const float* mean, const float* rstd, const float* gamma, int64_t N, int64_t H,
                          int dx_accumulate);
/* The same; with dx_colsum given, dx_colsum[j] += sum over rows of dx[row, j] as stored (after the accumulation).  When
 * dx is then the finished gradient of a residual stream, these are the bias gradient of the Linear layer that produced
 * the stream (gradtuity/tensor.py:1673-1679 computes it with a separate pass over the gradient). */
int gt_layernorm_backward_colsum(gt_ctx* ctx, float* dx, float* dgamma, float* dbeta, float* dx_colsum, const float* dy,
                                 const float* x, const float* mean, const float* rstd, const float* gamma, int64_t N, int64_t H,
                                 int dx_accumulate);
int gt_embedding(gt_ctx* ctx, float* out, const float* W, const float* idx, int64_t n, int64_t D, int64_t V);
int gt_embedding_backward(gt_ctx* ctx, float* dW, const float* dout, const float* idx, int64_t n, int64_t D, int64_t V);
/* The same with a factor: dW[idx[r], :] += alpha * dout[r, :] (the gathered rows of all ranks, alpha = 1 / world size). */
int gt_embedding_backward_scaled(gt_ctx* ctx, float* dW, const float* dout, const float* idx, int64_t n, int64_t D, int64_t V,
                                 float alpha);
/* Rows of C logits may be padded: ld_logits / ld_dlogits are the row pitches in elements (>= C).  The tied
 * LM head writes its 50257-wide logits at a 16-byte aligned pitch so that both kernels use vector loads
 * and the GEMMs that read dlogits take the TMA path. */
int gt_cross_entropy(gt_ctx* ctx, float* loss, float* row_loss, float* row_lse, const float* logits,
                     int64_t ld_logits, const float* targets, int64_t B, int64_t C, int mean);
/* gt_cross_entropy plus, in the same launch, dlogits = grad_scale * (softmax - onehot), written (not accumulated) at
 * pitch ld_dlogits: the loss kernel and the gradient kernel of the reference (cross_entropy_kernel and
 * cross_entropy_backward_kernel, gradtuity/tensor.py:1452-1525) share one pass over HBM.  For callers that know the
 * loss's upstream gradient when they compute the loss (grad_scale = upstream / B for mean, upstream for sum).       */
int gt_cross_entropy_fused(gt_ctx* ctx, float* loss, float* row_loss, float* row_lse, float* dlogits, int64_t ld_dlogits,
                           const float* logits, int64_t ld_logits, const float* targets, int64_t B, int64_t C, int mean,
                           float grad_scale);
int gt_cross_entropy_backward(gt_ctx* ctx, float* dlogits, int64_t ld_dlogits, const float* logits,
                              int64_t ld_logits, const float* targets, const float* row_lse,
                              const float* upstream, float scale, int64_t B, int64_t C, int accumulate);
int gt_adamw(gt_ctx* ctx, float* p, const float* g, float* m, float* v, int64_t n, float lr, float beta1,
             float beta2, float eps, float weight_decay, float bc1, float bc2, const float* grad_scale);
int gt_sumsq(gt_ctx* ctx, float* out, const float* x, int64_t n, int accumulate);
int gt_clip_scale(gt_ctx* ctx, float* scale_out, float* norm_out, const float* sumsq, float max_norm, float eps);
int gt_scale_by_device_scalar(gt_ctx* ctx, float* x, const float* s, int64_t n);
int gt_transpose12(gt_ctx* ctx, float* out, const float* in, int64_t B, int64_t d1, int64_t d2, int64_t D, int accumulate);
/* Multi-tensor forms: one launch for a whole parameter list.  `tensors` is a device array of
 * {float* p; const float* g; float* m; float* v; int64 n} (40 bytes each), `chunks` a device array of
 * {int32 tensor; int32 pad; int64 first_element} (16 bytes each) that assigns `chunk_elems` elements to
 * each block.  Same arithmetic as gt_adamw / gt_sumsq (gt_sumsq_multi: at most 4096 chunks).       */
int gt_adamw_multi(gt_ctx* ctx, const void* tensors, const void* chunks, int64_t n_chunks, int64_t chunk_elems,
                   float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
                   const float* grad_scale);
int gt_sumsq_multi(gt_ctx* ctx, float* out, const void* tensors, const void* chunks, int64_t n_chunks, int64_t chunk_elems);

/* ---- data-parallel gradient exchange (single node, NCCL over NVLink / NVSwitch) ----------
 * Replaces the reference's libnccl binding and the calls built on it:
 *   gt_dist_get_unique_id  nccl_get_unique_id        gradtuity/dist/nccl.py:71-79
 *   gt_dist_init           nccl_comm_init_rank       gradtuity/dist/nccl.py:92-112, dist/comm.py:97
 *   gt_dist_destroy        nccl_comm_destroy         gradtuity/dist/nccl.py:186-189
 *   gt_dist_allreduce      _nccl_all_reduce_inplace  gradtuity/dist/nccl.py:130-145, dist/comm.py:117-131
 *   gt_dist_broadcast      _nccl_broadcast_inplace   gradtuity/dist/nccl.py:163-178, dist/comm.py:134-147
 * Collectives are enqueued on a separate communication stream behind the work already given to
 * the compute stream and return at once; gt_dist_wait orders the compute stream behind them.
 * `average` != 0 divides by the world size inside the collective (ncclAvg).
 * Nothing on the host waits without a limit: gt_dist_init joins communicator creation, and gt_dist_wait with
 * host_sync != 0 polls the communication stream and ncclCommGetAsyncError, against GRADTUITY_NCCL_TIMEOUT_S
 * seconds (default 120); past it, or on an asynchronous NCCL error, the communicator is aborted and the call
 * returns GT_ERR_TIMEOUT / GT_ERR_NCCL (the reference waits 60 s for the id file, gradtuity/dist/comm.py:74-84,
 * and without limit in cudaDeviceSynchronize after that).
 * gt_dist_timeline (no counterpart in the reference; a measurement aid, active only when the process group was
 * created with GRADTUITY_DIST_TIMELINE=1): device times of the collectives between the last two waits, four
 * floats per row: element count, then ms from the first collective's enqueue point on the compute stream to
 * (this collective's enqueue point, its start on the communication stream, its end); a last row holds in its
 * second float when the compute stream resumed after the wait.                                 */
int gt_dist_get_unique_id(gt_ctx* ctx, char* out128);
int gt_dist_init(gt_ctx* ctx, int rank, int world, const char* uid128);
int gt_dist_destroy(gt_ctx* ctx);
int gt_dist_allreduce(gt_ctx* ctx, float* ptr, int64_t count, int average);
int gt_dist_broadcast(gt_ctx* ctx, float* ptr, int64_t count, int root);
/* dst (world x count floats) = the count floats at src of every rank, in rank order (ncclAllGather on the communication
 * stream, ordered like gt_dist_allreduce; every rank passes the same count).  Used for the rows of the embedding table that
 * a rank's batch touched, which are exchanged instead of a second all-reduce of the whole table's gradient. */
int gt_dist_allgather(gt_ctx* ctx, float* dst, const float* src, int64_t count);
int gt_dist_wait(gt_ctx* ctx, int host_sync);
int gt_dist_info(gt_ctx* ctx, int* rank, int* world);
int gt_dist_timeline(gt_ctx* ctx, float* out, int max_rows, int* n);

#ifdef __cplusplus
}
#endif
#endif /* GT_B200_H */
