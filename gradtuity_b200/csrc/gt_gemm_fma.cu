// fp32 FMA GEMM on CUDA cores.
//
// Serves GT_PREC_FP32 requests and every operand the TMA-fed tensor-core kernel cannot
// describe (base address not 16-byte aligned, leading dimension not a multiple of four
// elements).  It is the true-fp32 counterpart of the reference's CUDA-C kernels
// (gradtuity/kernels_cuda/matmul_kernels.py:21-236) but works on 64x64 tiles with a 4x4
// register block per thread instead of one thread per output, reads NN / NT / TN operands
// through element strides, and takes the whole batch in one launch.

#include "gt_internal.h"

namespace {

constexpr int TM = 64, TN = 64, TK = 16, THREADS = 256;

struct FmaParams {
  const float* A; const float* B; float* C; const float* bias; float* aux;
  long long sam, sak, sbk, sbn, ldc;
  long long sA0, sA1, sB0, sB1, sC0, sC1, bias_stride;
  int M, N, K;
  int batch0;
  int tiles_m, tiles_n;
  int epilogue, accumulate;
  float alpha;
};

__global__ void __launch_bounds__(THREADS) gt_gemm_fma_kernel(const FmaParams p) {
  __shared__ float As[TK][TM + 4];
  __shared__ float Bs[TK][TN + 4];

  long long tile = blockIdx.x;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int batch = (int)(tile / tiles_per_batch);
  const int t = (int)(tile % tiles_per_batch);
  const int tm = t / p.tiles_n, tn = t % p.tiles_n;
  const int i0 = batch % p.batch0, i1 = batch / p.batch0;
  const float* A = p.A + i0 * p.sA0 + i1 * p.sA1;
  const float* B = p.B + i0 * p.sB0 + i1 * p.sB1;
  const long long coff = i0 * p.sC0 + i1 * p.sC1;
  const int m0 = tm * TM, n0 = tn * TN;

  const int tid = threadIdx.x;
  const int tx = tid % 16, ty = tid / 16;   // 16 x 16 threads, each a 4 x 4 block
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

  // Causal epilogue: a tile wholly above the diagonal contributes only mask values.
  const bool skip = (p.epilogue == GT_EPI_CAUSAL) && (n0 > m0 + TM - 1);

  if (!skip) {
    for (int k0 = 0; k0 < p.K; k0 += TK) {
      // Each thread fetches 4 elements of the A tile and 4 of the B tile.  The fastest
      // thread index follows whichever operand dimension is contiguous in memory.
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        int e = tid + r * THREADS;          // 0 .. 1023
        int am, ak;
        if (p.sak == 1) { ak = e % TK; am = e / TK; } else { am = e % TM; ak = e / TM; }
        int gm = m0 + am, gk = k0 + ak;
        As[ak][am] = (gm < p.M && gk < p.K) ? A[gm * p.sam + gk * p.sak] : 0.0f;
        int bn, bk;
        if (p.sbn == 1) { bn = e % TN; bk = e / TN; } else { bk = e % TK; bn = e / TK; }
        int gn = n0 + bn; gk = k0 + bk;
        Bs[bk][bn] = (gn < p.N && gk < p.K) ? B[gk * p.sbk + gn * p.sbn] : 0.0f;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < TK; ++kk) {
        float a[4], b[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
        for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
      }
      __syncthreads();
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int gm = m0 + ty * 4 + i;
    if (gm >= p.M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int gn = n0 + tx * 4 + j;
      if (gn >= p.N) continue;
      float v = p.alpha * acc[i][j];
      if (p.epilogue >= GT_EPI_BIAS && p.epilogue <= GT_EPI_BIAS_GELU) v += p.bias[(long long)batch * p.bias_stride + gn];
      long long off = coff + (long long)gm * p.ldc + gn;
      if (p.aux) p.aux[off] = v;
      if (p.epilogue == GT_EPI_BIAS_RELU) v = fmaxf(v, 0.0f);
      else if (p.epilogue == GT_EPI_BIAS_GELU) v = gt_gelu_tanh(v);
      else if (p.epilogue == GT_EPI_CAUSAL && gn > gm) v = GT_CAUSAL_MASK_VALUE;
      if (p.accumulate) p.C[off] += v; else p.C[off] = v;
    }
  }
}

}  // namespace

int gt_gemm_fma_launch(gt_ctx* ctx, const gt_gemm_args& g, cudaStream_t stream) {
  FmaParams p;
  p.A = g.A; p.B = g.B; p.C = g.C; p.bias = g.bias; p.aux = g.aux;
  if (g.layout == GT_LAYOUT_TN) { p.sam = 1; p.sak = g.lda; } else { p.sam = g.lda; p.sak = 1; }
  if (g.layout == GT_LAYOUT_NT) { p.sbn = g.ldb; p.sbk = 1; } else { p.sbk = g.ldb; p.sbn = 1; }
  p.ldc = g.ldc;
  p.sA0 = g.sA0; p.sA1 = g.sA1; p.sB0 = g.sB0; p.sB1 = g.sB1; p.sC0 = g.sC0; p.sC1 = g.sC1;
  p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K;
  p.batch0 = (int)g.batch0;
  p.tiles_m = (int)((g.M + TM - 1) / TM);
  p.tiles_n = (int)((g.N + TN - 1) / TN);
  p.epilogue = g.epilogue; p.accumulate = g.accumulate; p.alpha = g.alpha;
  p.bias_stride = (g.flags & GT_GEMM_BIAS_PER_BATCH) ? g.N : 0;
  // batch entries that share one C would race on a plain read-modify-write
  if (g.batch0 * g.batch1 > 1 && ((g.batch0 > 1 && g.sC0 == 0) || (g.batch1 > 1 && g.sC1 == 0)))
    GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "gemm_batched: batch entries sharing one C are served by the tensor-core kernel only (tf32, aligned operands)");
  long long blocks = (long long)p.tiles_m * p.tiles_n * g.batch0 * g.batch1;
  if (blocks <= 0 || blocks > 0x7fffffffLL) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "fma gemm: %lld tiles out of range", blocks);
  gt_gemm_fma_kernel<<<(unsigned)blocks, THREADS, 0, stream>>>(p);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}
