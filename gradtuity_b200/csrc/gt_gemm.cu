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
  if (gt_gemm_umma_eligible(g)) return gt_gemm_umma_launch(ctx, g, s);
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
