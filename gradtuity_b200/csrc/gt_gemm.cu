// Entry points of the GEMM family: argument checking and the choice between the
// tcgen05/TMA kernel and the fp32 FMA kernel.
//
// gt_gemm / gt_gemm_batched stand where the reference's dispatch proxy
// (gradtuity/kernels.py:66-82, `kernel[grid](...)`) and the launch wrappers
// (gradtuity/kernels_cuda/matmul_kernels.py:254-341) stand.  Shape errors that the
// reference raises in Python before any launch (gradtuity/tensor.py:549-561) stay in
// Python; what is checked here is what only the native side can get wrong.

#include "gt_internal.h"

int gt_gemm_validate(gt_ctx* ctx, const gt_gemm_args& g) {
  if (g.layout < GT_LAYOUT_NN || g.layout > GT_LAYOUT_TN) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: layout %d is not NN/NT/TN", g.layout);
  if (g.epilogue < GT_EPI_NONE || g.epilogue > GT_EPI_GELU_GRAD) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: unknown epilogue %d", g.epilogue);
  if (g.precision < GT_PREC_TF32 || g.precision > GT_PREC_FP32) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: unknown precision %d", g.precision);
  if (g.M <= 0 || g.N <= 0 || g.K <= 0) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: M, N, K must be positive, got %lld %lld %lld", (long long)g.M, (long long)g.N, (long long)g.K);
  if (g.batch0 <= 0 || g.batch1 <= 0) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: batch counts must be positive");
  if (!g.A || !g.B || !g.C) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: null operand pointer");
  const bool needs_bias = (g.epilogue >= GT_EPI_BIAS && g.epilogue <= GT_EPI_BIAS_GELU) || g.epilogue == GT_EPI_BIAS_ADD;
  if ((g.epilogue == GT_EPI_BIAS_ADD || g.epilogue == GT_EPI_GELU_GRAD) && !g.aux) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: this epilogue reads aux, which is null");
  if (needs_bias && !g.bias) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: bias epilogue without a bias pointer");
  if (!needs_bias && g.bias) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: bias pointer given but the epilogue does not use it");
  if (g.accumulate != 0 && g.accumulate != 1) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: accumulate must be 0 or 1");
  const int64_t a_cols = g.layout == GT_LAYOUT_TN ? g.M : g.K;
  const int64_t b_cols = g.layout == GT_LAYOUT_NT ? g.K : g.N;
  if (g.lda < a_cols) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: lda %lld smaller than A's row length %lld", (long long)g.lda, (long long)a_cols);
  if (g.ldb < b_cols) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: ldb %lld smaller than B's row length %lld", (long long)g.ldb, (long long)b_cols);
  if (g.ldc < g.N) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: ldc %lld smaller than N %lld", (long long)g.ldc, (long long)g.N);
  if (g.M > 0x7fffffffLL || g.N > 0x7fffffffLL || g.K > 0x7fffffffLL) GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "gemm: dimensions beyond 2^31-1");
  return GT_OK;
}

namespace {

int run(gt_ctx* ctx, const gt_gemm_args& g, void* stream) {
  if (!ctx) return GT_ERR_INVALID_ARG;
  int rc = gt_gemm_validate(ctx, g);
  if (rc != GT_OK) return rc;
  cudaStream_t s = stream ? (cudaStream_t)stream : ctx->stream;
  if (gt_gemm_umma_eligible(g)) {
    rc = gt_gemm_umma_launch(ctx, g, s);
    const int rel = gt_scratch_release(ctx, s);      // a caller's stream that used the context's scratch: mark the hand-over point
    return rc != GT_OK ? rc : rel;
  }
  if (g.epilogue == GT_EPI_BIAS_ADD || g.epilogue == GT_EPI_GELU_GRAD)
    GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "gemm: the aux-reading epilogues need the tensor-core path (tf32 / 3xtf32, aligned B)");
  return gt_gemm_fma_launch(ctx, g, s);
}

}  // namespace

extern "C" int gt_gemm(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                       const float* A, int64_t lda, const float* B, int64_t ldb,
                       float* C, int64_t ldc, const float* bias, float* aux,
                       float alpha, int accumulate, int epilogue, int precision, void* stream) {
  gt_gemm_args g;
  g.layout = layout; g.epilogue = epilogue; g.precision = precision; g.accumulate = accumulate; g.flags = 0;
  g.M = M; g.N = N; g.K = K;
  g.A = A; g.lda = lda; g.sA0 = 0; g.sA1 = 0;
  g.B = B; g.ldb = ldb; g.sB0 = 0; g.sB1 = 0;
  g.C = C; g.ldc = ldc; g.sC0 = 0; g.sC1 = 0;
  g.batch0 = 1; g.batch1 = 1;
  g.bias = bias; g.aux = aux; g.alpha = alpha;
  return run(ctx, g, stream);
}

extern "C" int gt_gemm_batched(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                               const float* A, int64_t lda, int64_t strideA0, int64_t strideA1,
                               const float* B, int64_t ldb, int64_t strideB0, int64_t strideB1,
                               float* C, int64_t ldc, int64_t strideC0, int64_t strideC1,
                               int64_t batch0, int64_t batch1,
                               const float* bias, float* aux, float alpha, int accumulate,
                               int epilogue, int precision, void* stream) {
  return gt_gemm_batched_ex(ctx, layout, M, N, K, A, lda, strideA0, strideA1, B, ldb, strideB0, strideB1, C, ldc, strideC0,
                            strideC1, batch0, batch1, bias, aux, alpha, accumulate, epilogue, precision, 0, stream);
}

extern "C" int gt_gemm_batched_ex(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                                  const float* A, int64_t lda, int64_t strideA0, int64_t strideA1,
                                  const float* B, int64_t ldb, int64_t strideB0, int64_t strideB1,
                                  float* C, int64_t ldc, int64_t strideC0, int64_t strideC1,
                                  int64_t batch0, int64_t batch1,
                                  const float* bias, float* aux, float alpha, int accumulate,
                                  int epilogue, int precision, int flags, void* stream) {
  if (ctx) {
    if (flags & ~(GT_GEMM_A_LOWER | GT_GEMM_AT_LOWER | GT_GEMM_CAUSAL_SKIP_MASKED | GT_GEMM_BIAS_PER_BATCH)) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm_batched_ex: unknown flags 0x%x", flags);
    if ((flags & (GT_GEMM_A_LOWER | GT_GEMM_AT_LOWER)) && M != K) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm_batched_ex: triangular-A flags need a square A (M == K)");
    if ((flags & GT_GEMM_A_LOWER) && (flags & GT_GEMM_AT_LOWER)) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm_batched_ex: A_LOWER and AT_LOWER exclude each other");
    if ((flags & GT_GEMM_A_LOWER) && layout == GT_LAYOUT_TN) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm_batched_ex: A_LOWER describes an A stored (M, K)");
    if ((flags & GT_GEMM_AT_LOWER) && layout != GT_LAYOUT_TN) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm_batched_ex: AT_LOWER describes an A stored (K, M)");
    if ((flags & GT_GEMM_CAUSAL_SKIP_MASKED) && epilogue != GT_EPI_CAUSAL) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm_batched_ex: SKIP_MASKED needs the causal epilogue");
  }
  gt_gemm_args g;
  g.layout = layout; g.epilogue = epilogue; g.precision = precision; g.accumulate = accumulate; g.flags = flags;
  g.M = M; g.N = N; g.K = K;
  g.A = A; g.lda = lda; g.sA0 = strideA0; g.sA1 = strideA1;
  g.B = B; g.ldb = ldb; g.sB0 = strideB0; g.sB1 = strideB1;
  g.C = C; g.ldc = ldc; g.sC0 = strideC0; g.sC1 = strideC1;
  g.batch0 = batch0; g.batch1 = batch1;
  g.bias = bias; g.aux = aux; g.alpha = alpha;
  if (ctx && (strideA0 < 0 || strideA1 < 0 || strideB0 < 0 || strideB1 < 0 || strideC0 < 0 || strideC1 < 0))
    GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm_batched: negative batch stride");
  return run(ctx, g, stream);
}

// dX of the second Linear layer of a GELU MLP together with the bias gradient of the first:
//   C = alpha * op(A) op(B) * gelu'(pre),   colsum[n] += sum_m C[m, n]
// The sums are taken from the output tiles while they are staged in shared memory for their TMA store, so C is
// not read again from HBM by a column-sum kernel (gradtuity/tensor.py:954-984 runs GELU backward, and
// gradtuity/tensor.py:1781-1904 the bias sum, as separate passes over the (M, N) tensor).  The additions into
// colsum are atomic, in no fixed order; with GRADTUITY_GEMM_DETERMINISTIC=1 the sums come from the ordered
// column-sum kernel after the product instead.  Runs on the context's compute stream.
extern "C" int gt_gemm_gelu_grad_colsum(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                                        const float* A, int64_t lda, const float* B, int64_t ldb,
                                        float* C, int64_t ldc, const float* pre, float* colsum,
                                        float alpha, int precision) {
  if (!ctx) return GT_ERR_INVALID_ARG;
  if (!colsum) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm_gelu_grad_colsum: null column-sum pointer");
  static const bool ordered = getenv("GRADTUITY_GEMM_DETERMINISTIC") != nullptr;
  gt_gemm_args g;
  g.layout = layout; g.epilogue = GT_EPI_GELU_GRAD; g.precision = precision; g.accumulate = 0; g.flags = 0;
  g.M = M; g.N = N; g.K = K;
  g.A = A; g.lda = lda; g.sA0 = 0; g.sA1 = 0;
  g.B = B; g.ldb = ldb; g.sB0 = 0; g.sB1 = 0;
  g.C = C; g.ldc = ldc; g.sC0 = 0; g.sC1 = 0;
  g.batch0 = 1; g.batch1 = 1;
  g.bias = nullptr; g.aux = const_cast<float*>(pre); g.alpha = alpha;
  g.colsum = ordered ? nullptr : colsum;
  const int rc = run(ctx, g, nullptr);
  if (rc != GT_OK || !ordered) return rc;
  return gt_colsum_acc(ctx, colsum, C, M, N, ldc);
}

extern "C" int gt_gemm_path(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                            const float* A, int64_t lda, const float* B, int64_t ldb,
                            const float* C, int64_t ldc, int precision, int* path) {
  if (!ctx || !path) return GT_ERR_INVALID_ARG;
  gt_gemm_args g;
  memset(&g, 0, sizeof(g));
  g.layout = layout; g.precision = precision;
  g.M = M; g.N = N; g.K = K; g.A = A; g.lda = lda; g.B = B; g.ldb = ldb; g.C = (float*)C; g.ldc = ldc;
  g.batch0 = 1; g.batch1 = 1;
  *path = gt_gemm_umma_eligible(g) ? 0 : 1;
  return GT_OK;
}

// ---- GEMM on host buffers, copies overlapped with the product -----------------------------------
// C (host) = epilogue(alpha * op(A) op(B) (+ bias)) for A, B, C in HOST memory (pinned memory for the
// copies to overlap).  B goes to the device once; A is cut into row blocks of C, and the upload of
// block i + 1, the product of block i and the download of block i - 1 run at the same time on three
// streams (PCIe is full duplex), with two device buffers each for the A and C blocks.  The call
// returns when C is complete in host memory.  This is the form in which a caller with host data, such
// as the reference's `Tensor(list).matmul(...).to_list()` (gradtuity/tensor.py:192-220, 530-657), pays
// the least for the PCIe link: max(upload, download) instead of their sum.
extern "C" int gt_gemm_host(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                            const float* hA, int64_t lda, const float* hB, int64_t ldb, float* hC, int64_t ldc,
                            const float* h_bias, float alpha, int epilogue, int precision, int chunks) {
  if (!ctx || !hA || !hB || !hC || M <= 0 || N <= 0 || K <= 0 || chunks <= 0) return GT_ERR_INVALID_ARG;
  if (layout < GT_LAYOUT_NN || layout > GT_LAYOUT_TN) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm_host: layout %d is not NN/NT/TN", layout);
  if (epilogue < GT_EPI_NONE || epilogue > GT_EPI_BIAS_GELU) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm_host: epilogue %d is not none / bias / bias+ReLU / bias+GELU", epilogue);
  if ((epilogue != GT_EPI_NONE) != (h_bias != nullptr)) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm_host: bias pointer and epilogue do not agree");
  const int64_t a_rows = layout == GT_LAYOUT_TN ? K : M, a_cols = layout == GT_LAYOUT_TN ? M : K;
  const int64_t b_rows = layout == GT_LAYOUT_NT ? N : K, b_cols = layout == GT_LAYOUT_NT ? K : N;
  if (lda < a_cols || ldb < b_cols || ldc < N) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm_host: a leading dimension is smaller than its row length");
  (void)a_rows;
  if (!ctx->h2d_stream) {
    GT_CUDA_OK(ctx, cudaStreamCreateWithFlags(&ctx->h2d_stream, cudaStreamNonBlocking));
    GT_CUDA_OK(ctx, cudaStreamCreateWithFlags(&ctx->d2h_stream, cudaStreamNonBlocking));
    for (int i = 0; i < 8; ++i) GT_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->host_ev[i], cudaEventDisableTiming));
  }
  cudaStream_t cs = ctx->stream, up = ctx->h2d_stream, down = ctx->d2h_stream;
  cudaEvent_t ev_alloc = ctx->host_ev[0], ev_b = ctx->host_ev[1];
  cudaEvent_t ev_a[2] = {ctx->host_ev[2], ctx->host_ev[3]}, ev_g[2] = {ctx->host_ev[4], ctx->host_ev[5]},
              ev_d[2] = {ctx->host_ev[6], ctx->host_ev[7]};
  // row blocks of C: multiples of 128 rows (the kernels' tile height)
  int64_t rows_per = (M + chunks - 1) / chunks;
  rows_per = (rows_per + 127) / 128 * 128;
  const int nblk = (int)((M + rows_per - 1) / rows_per);
  // compact device copies; leading dimensions padded to a multiple of 4 floats so that TMA can describe them
  const int64_t ldb_d = (b_cols + 3) / 4 * 4, ldc_d = (N + 3) / 4 * 4;
  const int64_t lda_d = layout == GT_LAYOUT_TN ? rows_per : (K + 3) / 4 * 4;      // TN: a block is (K, rows_per)
  const size_t a_blk = (size_t)(layout == GT_LAYOUT_TN ? K * lda_d : rows_per * lda_d), c_blk = (size_t)(rows_per * ldc_d);
  float *dB = nullptr, *dA[2] = {nullptr, nullptr}, *dC[2] = {nullptr, nullptr}, *d_bias = nullptr;
  // Everything that can fail after the first allocation runs inside this lambda: a failure returns from the
  // lambda only, so the drain-and-free block below runs on every path.
  auto enqueue = [&]() -> int {
    GT_CUDA_OK(ctx, cudaMallocAsync((void**)&dB, (size_t)(b_rows * ldb_d) * sizeof(float), cs));
    for (int i = 0; i < 2; ++i) {
      GT_CUDA_OK(ctx, cudaMallocAsync((void**)&dA[i], a_blk * sizeof(float), cs));
      GT_CUDA_OK(ctx, cudaMallocAsync((void**)&dC[i], c_blk * sizeof(float), cs));
    }
    if (h_bias) GT_CUDA_OK(ctx, cudaMallocAsync((void**)&d_bias, (size_t)N * sizeof(float), cs));
    GT_CUDA_OK(ctx, cudaEventRecord(ev_alloc, cs));
    GT_CUDA_OK(ctx, cudaStreamWaitEvent(up, ev_alloc, 0));
    GT_CUDA_OK(ctx, cudaStreamWaitEvent(down, ev_alloc, 0));
    GT_CUDA_OK(ctx, cudaMemcpy2DAsync(dB, (size_t)ldb_d * 4, hB, (size_t)ldb * 4, (size_t)b_cols * 4, (size_t)b_rows, cudaMemcpyHostToDevice, up));
    if (h_bias) GT_CUDA_OK(ctx, cudaMemcpyAsync(d_bias, h_bias, (size_t)N * 4, cudaMemcpyHostToDevice, up));
    GT_CUDA_OK(ctx, cudaEventRecord(ev_b, up));
    for (int i = 0; i < nblk; ++i) {
      const int buf = i & 1;
      const int64_t m0 = (int64_t)i * rows_per, rows = (M - m0) < rows_per ? (M - m0) : rows_per;
      if (i >= 2) GT_CUDA_OK(ctx, cudaStreamWaitEvent(up, ev_g[buf], 0));             // the product that read this A buffer is done
      if (layout == GT_LAYOUT_TN)
        GT_CUDA_OK(ctx, cudaMemcpy2DAsync(dA[buf], (size_t)lda_d * 4, hA + m0, (size_t)lda * 4, (size_t)rows * 4, (size_t)K, cudaMemcpyHostToDevice, up));
      else
        GT_CUDA_OK(ctx, cudaMemcpy2DAsync(dA[buf], (size_t)lda_d * 4, hA + m0 * lda, (size_t)lda * 4, (size_t)K * 4, (size_t)rows, cudaMemcpyHostToDevice, up));
      GT_CUDA_OK(ctx, cudaEventRecord(ev_a[buf], up));
      GT_CUDA_OK(ctx, cudaStreamWaitEvent(cs, ev_a[buf], 0));
      if (i == 0) GT_CUDA_OK(ctx, cudaStreamWaitEvent(cs, ev_b, 0));
      if (i >= 2) GT_CUDA_OK(ctx, cudaStreamWaitEvent(cs, ev_d[buf], 0));             // this C buffer has been downloaded
      gt_gemm_args g;
      g.layout = layout; g.epilogue = epilogue; g.precision = precision; g.accumulate = 0; g.flags = 0;
      g.M = rows; g.N = N; g.K = K;
      g.A = dA[buf]; g.lda = lda_d; g.sA0 = 0; g.sA1 = 0;
      g.B = dB; g.ldb = ldb_d; g.sB0 = 0; g.sB1 = 0;
      g.C = dC[buf]; g.ldc = ldc_d; g.sC0 = 0; g.sC1 = 0;
      g.batch0 = 1; g.batch1 = 1; g.bias = d_bias; g.aux = nullptr; g.alpha = alpha;
      const int grc = run(ctx, g, cs);
      if (grc != GT_OK) return grc;
      GT_CUDA_OK(ctx, cudaEventRecord(ev_g[buf], cs));
      GT_CUDA_OK(ctx, cudaStreamWaitEvent(down, ev_g[buf], 0));
      GT_CUDA_OK(ctx, cudaMemcpy2DAsync(hC + m0 * ldc, (size_t)ldc * 4, dC[buf], (size_t)ldc_d * 4, (size_t)N * 4, (size_t)rows, cudaMemcpyDeviceToHost, down));
      GT_CUDA_OK(ctx, cudaEventRecord(ev_d[buf], down));
    }
    return GT_OK;
  };
  const int rc = enqueue();
  // everything in flight must finish before the buffers go back to the pool and the caller reads C
  cudaError_t e1 = cudaStreamSynchronize(up), e2 = cudaStreamSynchronize(cs), e3 = cudaStreamSynchronize(down);
  if (dB) cudaFreeAsync(dB, cs);
  for (int i = 0; i < 2; ++i) {
    if (dA[i]) cudaFreeAsync(dA[i], cs);
    if (dC[i]) cudaFreeAsync(dC[i], cs);
  }
  if (d_bias) cudaFreeAsync(d_bias, cs);
  if (rc != GT_OK) return rc;
  GT_CUDA_OK(ctx, e1); GT_CUDA_OK(ctx, e2); GT_CUDA_OK(ctx, e3);
  return GT_OK;
}
