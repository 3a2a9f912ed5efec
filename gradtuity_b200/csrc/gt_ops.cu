// The small element-wise and reduction kernels that sit beside the GEMMs in the autograd
// closures of Tensor.matmul / linear / linear_relu / bmm (gradtuity/tensor.py:530-657,
// 1561-1904): gradient seeding and accumulation, ReLU and its mask, the bias-gradient column
// sum, the scalar sum used as a test loss.  Plain CUDA, fp32, memory-bound; grids are sized
// in multiples of the SM count and walk the data with grid-stride loops of float4.
//
// fp32 specifications followed: gradtuity/kernels_cuda/elemwise_kernels.py:20-101 (add, mul,
// relu, relu_backward, relu_mask_mul), gradtuity/kernels_cuda/reduce_kernels.py (sum_all,
// sum_axis0, add_scalar_inplace, add_bias), gradtuity/kernels_cuda/optim_kernels.py (fill).

#include "gt_internal.h"

namespace {

constexpr int EW_THREADS = 256;

inline unsigned ew_blocks(gt_ctx* ctx, long long n_items) {
  long long b = (n_items + EW_THREADS - 1) / EW_THREADS;
  long long cap = (long long)ctx->sm_count * 8;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (unsigned)b;
}

enum { OP_ADD = 0, OP_MUL = 1, OP_RELU = 2, OP_RELU_MASK_MUL = 3, OP_SCALE = 4, OP_GELU = 5, OP_GELU_BWD = 6 };

template <int OP>
__device__ __forceinline__ float ew_apply(float a, float b, float s) {
  if (OP == OP_ADD) return a + b;
  if (OP == OP_MUL) return a * b;
  if (OP == OP_RELU) return fmaxf(a, 0.0f);
  if (OP == OP_RELU_MASK_MUL) return b > 0.0f ? a : 0.0f;        // a = dY, b = Y
  if (OP == OP_SCALE) return a * s;
  if (OP == OP_GELU) return gt_gelu_tanh(a);
  if (OP == OP_GELU_BWD) {                                        // a = dY, b = x
    float u = 0.7978845608028654f * (b + 0.044715f * b * b * b);
    float t = 1.0f - __fdividef(2.0f, 1.0f + __expf(2.0f * u));
    float du = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * b * b);
    return a * (0.5f * (1.0f + t) + 0.5f * b * (1.0f - t * t) * du);
  }
  return 0.0f;
}

// out = op(a, b) or out += op(a, b); b may be null for unary ops.
template <int OP, bool ACC>
__global__ void __launch_bounds__(EW_THREADS) ew_kernel(float* out, const float* a,
                                                        const float* b, float s, long long n, int vec) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (vec) {
    const long long n4 = n >> 2;
    const float4* a4 = reinterpret_cast<const float4*>(a);
    const float4* b4 = reinterpret_cast<const float4*>(b);
    float4* o4 = reinterpret_cast<float4*>(out);
    for (long long i = tid; i < n4; i += stride) {
      float4 x = a4[i];
      float4 y = b ? b4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      float4 r = make_float4(ew_apply<OP>(x.x, y.x, s), ew_apply<OP>(x.y, y.y, s), ew_apply<OP>(x.z, y.z, s), ew_apply<OP>(x.w, y.w, s));
      if (ACC) { float4 o = o4[i]; r.x += o.x; r.y += o.y; r.z += o.z; r.w += o.w; }
      o4[i] = r;
    }
    for (long long i = (n4 << 2) + tid; i < n; i += stride) {
      float r = ew_apply<OP>(a[i], b ? b[i] : 0.f, s);
      out[i] = ACC ? out[i] + r : r;
    }
  } else {
    for (long long i = tid; i < n; i += stride) {
      float r = ew_apply<OP>(a[i], b ? b[i] : 0.f, s);
      out[i] = ACC ? out[i] + r : r;
    }
  }
}

template <int OP>
int ew_launch(gt_ctx* ctx, float* out, const float* a, const float* b, float s, long long n, int accumulate) {
  if (!ctx || !out || !a || n < 0) return GT_ERR_INVALID_ARG;
  if (n == 0) return GT_OK;
  const int vec = (((uintptr_t)out | (uintptr_t)a | (uintptr_t)b) & 15) == 0;
  const unsigned blocks = ew_blocks(ctx, vec ? (n + 3) / 4 : n);
  if (accumulate) ew_kernel<OP, true><<<blocks, EW_THREADS, 0, ctx->stream>>>(out, a, b, s, n, vec);
  else ew_kernel<OP, false><<<blocks, EW_THREADS, 0, ctx->stream>>>(out, a, b, s, n, vec);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}

__global__ void __launch_bounds__(EW_THREADS) fill_kernel(float* __restrict__ out, float v, long long n) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) out[i] = v;
}

// dst[i] += *scalar (gradient of sum(): gradtuity/tensor.py:1380-1386)
__global__ void __launch_bounds__(EW_THREADS) add_scalar_kernel(float* __restrict__ dst, const float* __restrict__ scalar, long long n) {
  const float v = *scalar;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) dst[i] += v;
}

// out[r, c] = x[r, c] + bias[c]
__global__ void __launch_bounds__(EW_THREADS) add_bias_kernel(float* __restrict__ out, const float* __restrict__ x,
                                                              const float* __restrict__ bias, long long rows, int cols) {
  const long long n = rows * cols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = x[i] + bias[i % cols];
}

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = 0.0f;
  if (w == 0) {
    t = l < (blockDim.x >> 5) ? red[l] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  }
  __syncthreads();
  return t;   // valid in warp 0
}

// Two-pass deterministic sum: partial sums per block, then one block folds them.
__global__ void __launch_bounds__(EW_THREADS) sum_partial_kernel(const float* __restrict__ x, float* __restrict__ partial, long long n) {
  __shared__ float red[32];
  float v = 0.0f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) v += x[i];
  float t = block_sum(v, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = t;
}
__global__ void __launch_bounds__(EW_THREADS) sum_final_kernel(const float* __restrict__ partial, float* __restrict__ out, int n, int accumulate) {
  __shared__ float red[32];
  float v = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) v += partial[i];
  float t = block_sum(v, red);
  if (threadIdx.x == 0) *out = accumulate ? *out + t : t;
}

// db[c] += sum over rows of dY[r, c].  Block = 32 columns x 8 row lanes; grid.y splits the rows.
__global__ void __launch_bounds__(256) colsum_acc_kernel(float* __restrict__ db, const float* __restrict__ dy,
                                                         long long rows, int cols, long long ld, int rows_per_block) {
  __shared__ float red[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  long long r1 = r0 + rows_per_block; if (r1 > rows) r1 = rows;
  float v = 0.0f;
  if (c < cols) for (long long r = r0 + ry; r < r1; r += 8) v += dy[r * ld + c];
  red[ry][cx] = v;
  __syncthreads();
  if (ry == 0 && c < cols) {
    float t = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t += red[i][cx];
    atomicAdd(db + c, t);
  }
}

// The same for 16-byte aligned rows with cols % 4 == 0: a block covers 128 columns (one float4 per
// lane) x 8 row lanes, four rows in flight per thread.
__global__ void __launch_bounds__(256) colsum_acc_vec_kernel(float* __restrict__ db, const float* __restrict__ dy,
                                                             long long rows, int cols, long long ld, int rows_per_block,
                                                             long long db_stride, long long dy_stride) {
  __shared__ float4 red[8][32];
  gt_let_next_kernel_start();
  gt_wait_for_previous_kernel();
  db += blockIdx.z * db_stride;          // batch entry z: its own matrix and its own sums
  dy += blockIdx.z * dy_stride;
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
  const int c = (blockIdx.x * 32 + cx) * 4;
  const long long r0 = (long long)blockIdx.y * rows_per_block;
  long long r1 = r0 + rows_per_block; if (r1 > rows) r1 = rows;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  if (c < cols) {
    long long r = r0 + ry;
    for (; r + 24 < r1; r += 32) {
      const float4 a0 = *reinterpret_cast<const float4*>(dy + r * ld + c);
      const float4 a1 = *reinterpret_cast<const float4*>(dy + (r + 8) * ld + c);
      const float4 a2 = *reinterpret_cast<const float4*>(dy + (r + 16) * ld + c);
      const float4 a3 = *reinterpret_cast<const float4*>(dy + (r + 24) * ld + c);
      v.x += (a0.x + a1.x) + (a2.x + a3.x); v.y += (a0.y + a1.y) + (a2.y + a3.y);
      v.z += (a0.z + a1.z) + (a2.z + a3.z); v.w += (a0.w + a1.w) + (a2.w + a3.w);
    }
    for (; r < r1; r += 8) {
      const float4 a = *reinterpret_cast<const float4*>(dy + r * ld + c);
      v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
    }
  }
  red[ry][cx] = v;
  __syncthreads();
  if (ry == 0 && c < cols) {
    float4 t = red[0][cx];
#pragma unroll
    for (int i = 1; i < 8; ++i) { const float4 o = red[i][cx]; t.x += o.x; t.y += o.y; t.z += o.z; t.w += o.w; }
    atomicAdd(db + c, t.x); atomicAdd(db + c + 1, t.y); atomicAdd(db + c + 2, t.z); atomicAdd(db + c + 3, t.w);
  }
}

// dst[r, c] = src[r, c] for rows of `cols` floats at different pitches (used to give a matrix with an
// odd leading dimension a 16-byte aligned copy that TMA can read).
__global__ void __launch_bounds__(256) repack_rows_kernel(float* __restrict__ dst, long long ld_dst, const float* __restrict__ src,
                                                          long long ld_src, long long rows, int cols) {
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const float* s = src + r * ld_src;
    float* d = dst + r * ld_dst;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) d[c] = s[c];
  }
}

// im2col for conv2d: col[(n, ho, wo), (c, kh, kw)] = x[n, c, ho*s - p + kh, wo*s - p + kw], zero outside
// the image; rows of col are ld floats apart (gradtuity/kernels_cuda/conv_kernels.py im2col_kernel_2d,
// as launched from gradtuity/tensor.py:1955-1972).
__global__ void __launch_bounds__(256) im2col_kernel(float* __restrict__ col, const float* __restrict__ x, long long rows,
                                                     int C, int H, int W, int kH, int kW, int stride, int pad,
                                                     int H_out, int W_out, int ncols, long long ld) {
  const long long total = rows * ncols;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / ncols;
    const int cc = (int)(i - r * ncols);
    const int kw = cc % kW, kh = (cc / kW) % kH, c = cc / (kW * kH);
    const int wo = (int)(r % W_out), ho = (int)((r / W_out) % H_out);
    const long long n = r / ((long long)W_out * H_out);
    const int h = ho * stride - pad + kh, w = wo * stride - pad + kw;
    float v = 0.0f;
    if (h >= 0 && h < H && w >= 0 && w < W) v = x[((n * C + c) * H + h) * (long long)W + w];
    col[r * ld + cc] = v;
  }
}
// col2im, gather form (no atomics): dx[n, c, h, w] += sum over the (kh, kw) whose output position exists
// (gradtuity/tensor.py:2139-2158 launches the scatter form).
__global__ void __launch_bounds__(256) col2im_kernel(float* __restrict__ dx, const float* __restrict__ dcol, long long N,
                                                     int C, int H, int W, int kH, int kW, int stride, int pad,
                                                     int H_out, int W_out, long long ld, int accumulate) {
  const long long total = N * C * H * W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int w = (int)(i % W), h = (int)((i / W) % H), c = (int)((i / ((long long)W * H)) % C);
    const long long n = i / ((long long)W * H * C);
    float s = 0.0f;
    for (int kh = 0; kh < kH; ++kh) {
      const int hs = h + pad - kh;
      if (hs < 0 || hs % stride != 0) continue;
      const int ho = hs / stride;
      if (ho >= H_out) continue;
      for (int kw = 0; kw < kW; ++kw) {
        const int ws = w + pad - kw;
        if (ws < 0 || ws % stride != 0) continue;
        const int wo = ws / stride;
        if (wo >= W_out) continue;
        s += dcol[((n * H_out + ho) * W_out + wo) * ld + ((long long)c * kH + kh) * kW + kw];
      }
    }
    dx[i] = accumulate ? dx[i] + s : s;
  }
}

// Max pooling over (kH, kW) windows of an (N, C, H, W) tensor; idx receives the flat offset of the
// winning element inside its (H, W) plane, as a float (the engine has one dtype), for the backward
// (gradtuity/tensor.py:2169-2260: maxpool2d_forward_kernel / maxpool2d_backward_kernel).  The first
// maximum of a window wins.
__global__ void __launch_bounds__(256) maxpool2d_fwd_kernel(float* __restrict__ out, float* __restrict__ idx, const float* __restrict__ x,
                                                            long long planes, int H, int W, int kH, int kW, int sh, int sw,
                                                            int H_out, int W_out) {
  const long long total = planes * H_out * W_out;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int wo = (int)(i % W_out), ho = (int)((i / W_out) % H_out);
    const long long pl = i / ((long long)W_out * H_out);
    const float* xp = x + pl * H * W;
    float best = -INFINITY; int arg = 0;
    for (int kh = 0; kh < kH; ++kh)
      for (int kw = 0; kw < kW; ++kw) {
        const int off = (ho * sh + kh) * W + wo * sw + kw;
        const float v = xp[off];
        if (v > best) { best = v; arg = off; }
      }
    out[i] = best;
    idx[i] = (float)arg;
  }
}
// dx[plane, idx] += dy: windows may overlap (stride < kernel), so the scatter is atomic.
__global__ void __launch_bounds__(256) maxpool2d_bwd_kernel(float* __restrict__ dx, const float* __restrict__ dy, const float* __restrict__ idx,
                                                            long long planes, int HW, int HWo) {
  const long long total = planes * HWo;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long pl = i / HWo;
    atomicAdd(dx + pl * HW + (int)idx[i], dy[i]);
  }
}

}  // namespace

extern "C" int gt_maxpool2d(gt_ctx* ctx, float* out, float* idx, const float* x, int64_t N, int64_t C, int64_t H, int64_t W,
                            int64_t kH, int64_t kW, int64_t stride_h, int64_t stride_w) {
  if (!ctx || !out || !idx || !x || N <= 0 || C <= 0 || H <= 0 || W <= 0 || kH <= 0 || kW <= 0 || stride_h <= 0 || stride_w <= 0 ||
      kH > H || kW > W || H * W >= (1 << 24)) return GT_ERR_INVALID_ARG;
  const int64_t H_out = (H - kH) / stride_h + 1, W_out = (W - kW) / stride_w + 1;
  maxpool2d_fwd_kernel<<<ew_blocks(ctx, N * C * H_out * W_out), EW_THREADS, 0, ctx->stream>>>(out, idx, x, N * C, (int)H, (int)W, (int)kH, (int)kW,
                                                                                             (int)stride_h, (int)stride_w, (int)H_out, (int)W_out);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}

extern "C" int gt_maxpool2d_backward(gt_ctx* ctx, float* dx, const float* dy, const float* idx, int64_t planes, int64_t HW, int64_t HWo) {
  if (!ctx || !dx || !dy || !idx || planes <= 0 || HW <= 0 || HWo <= 0 || HW >= (1 << 24)) return GT_ERR_INVALID_ARG;
  maxpool2d_bwd_kernel<<<ew_blocks(ctx, planes * HWo), EW_THREADS, 0, ctx->stream>>>(dx, dy, idx, planes, (int)HW, (int)HWo);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}

extern "C" int gt_im2col(gt_ctx* ctx, float* col, int64_t ld_col, const float* x, int64_t N, int64_t C, int64_t H, int64_t W,
                         int64_t kH, int64_t kW, int64_t stride, int64_t pad) {
  if (!ctx || !col || !x || N <= 0 || C <= 0 || H <= 0 || W <= 0 || kH <= 0 || kW <= 0 || stride <= 0 || pad < 0) return GT_ERR_INVALID_ARG;
  const int64_t H_out = (H + 2 * pad - kH) / stride + 1, W_out = (W + 2 * pad - kW) / stride + 1;
  const int64_t ncols = C * kH * kW;
  if (H + 2 * pad < kH || W + 2 * pad < kW || ld_col < ncols || ncols > 0x7fffffff || H > 0x7fffffff || W > 0x7fffffff) return GT_ERR_INVALID_ARG;
  const long long rows = N * H_out * W_out;
  im2col_kernel<<<ew_blocks(ctx, rows * ncols), EW_THREADS, 0, ctx->stream>>>(col, x, rows, (int)C, (int)H, (int)W, (int)kH, (int)kW,
                                                                             (int)stride, (int)pad, (int)H_out, (int)W_out, (int)ncols, ld_col);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}

extern "C" int gt_col2im(gt_ctx* ctx, float* dx, const float* dcol, int64_t ld_col, int64_t N, int64_t C, int64_t H, int64_t W,
                         int64_t kH, int64_t kW, int64_t stride, int64_t pad, int accumulate) {
  if (!ctx || !dx || !dcol || N <= 0 || C <= 0 || H <= 0 || W <= 0 || kH <= 0 || kW <= 0 || stride <= 0 || pad < 0) return GT_ERR_INVALID_ARG;
  const int64_t H_out = (H + 2 * pad - kH) / stride + 1, W_out = (W + 2 * pad - kW) / stride + 1;
  if (H + 2 * pad < kH || W + 2 * pad < kW || ld_col < C * kH * kW || H > 0x7fffffff || W > 0x7fffffff || C > 0x7fffffff) return GT_ERR_INVALID_ARG;
  col2im_kernel<<<ew_blocks(ctx, N * C * H * W), EW_THREADS, 0, ctx->stream>>>(dx, dcol, N, (int)C, (int)H, (int)W, (int)kH, (int)kW,
                                                                               (int)stride, (int)pad, (int)H_out, (int)W_out, ld_col, accumulate);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}

extern "C" int gt_repack_rows(gt_ctx* ctx, float* dst, int64_t ld_dst, const float* src, int64_t ld_src, int64_t rows, int64_t cols) {
  if (!ctx || !dst || !src || rows <= 0 || cols <= 0 || cols > 0x7fffffff || ld_dst < cols || ld_src < cols) return GT_ERR_INVALID_ARG;
  long long blocks = rows < (long long)ctx->sm_count * 16 ? rows : (long long)ctx->sm_count * 16;
  repack_rows_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(dst, ld_dst, src, ld_src, rows, (int)cols);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}

extern "C" int gt_fill(gt_ctx* ctx, float* out, float value, int64_t n) {
  if (!ctx || !out || n < 0) return GT_ERR_INVALID_ARG;
  if (n == 0) return GT_OK;
  fill_kernel<<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>(out, value, n);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}
extern "C" int gt_add(gt_ctx* ctx, float* out, const float* a, const float* b, int64_t n, int accumulate) { return b ? ew_launch<OP_ADD>(ctx, out, a, b, 0.f, n, accumulate) : GT_ERR_INVALID_ARG; }
extern "C" int gt_mul(gt_ctx* ctx, float* out, const float* a, const float* b, int64_t n, int accumulate) { return b ? ew_launch<OP_MUL>(ctx, out, a, b, 0.f, n, accumulate) : GT_ERR_INVALID_ARG; }
extern "C" int gt_scale(gt_ctx* ctx, float* out, const float* a, float s, int64_t n, int accumulate) { return ew_launch<OP_SCALE>(ctx, out, a, nullptr, s, n, accumulate); }
extern "C" int gt_relu(gt_ctx* ctx, float* out, const float* a, int64_t n) { return ew_launch<OP_RELU>(ctx, out, a, nullptr, 0.f, n, 0); }
extern "C" int gt_relu_mask_mul(gt_ctx* ctx, float* out, const float* dy, const float* y, int64_t n, int accumulate) { return y ? ew_launch<OP_RELU_MASK_MUL>(ctx, out, dy, y, 0.f, n, accumulate) : GT_ERR_INVALID_ARG; }
extern "C" int gt_gelu(gt_ctx* ctx, float* out, const float* a, int64_t n) { return ew_launch<OP_GELU>(ctx, out, a, nullptr, 0.f, n, 0); }
extern "C" int gt_gelu_backward(gt_ctx* ctx, float* dx, const float* dy, const float* x, int64_t n, int accumulate) { return x ? ew_launch<OP_GELU_BWD>(ctx, dx, dy, x, 0.f, n, accumulate) : GT_ERR_INVALID_ARG; }

extern "C" int gt_add_scalar(gt_ctx* ctx, float* dst, const float* scalar, int64_t n) {
  if (!ctx || !dst || !scalar || n < 0) return GT_ERR_INVALID_ARG;
  if (n == 0) return GT_OK;
  add_scalar_kernel<<<ew_blocks(ctx, n), EW_THREADS, 0, ctx->stream>>>(dst, scalar, n);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}

extern "C" int gt_add_bias(gt_ctx* ctx, float* out, const float* x, const float* bias, int64_t rows, int64_t cols) {
  if (!ctx || !out || !x || !bias || rows <= 0 || cols <= 0 || cols > 0x7fffffff) return GT_ERR_INVALID_ARG;
  add_bias_kernel<<<ew_blocks(ctx, rows * cols), EW_THREADS, 0, ctx->stream>>>(out, x, bias, rows, (int)cols);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}

extern "C" int gt_sum_all(gt_ctx* ctx, float* out, const float* x, int64_t n, int accumulate) {
  if (!ctx || !out || !x || n <= 0) return GT_ERR_INVALID_ARG;
  const unsigned blocks = ew_blocks(ctx, n);
  int rc = gt_workspace_reserve(ctx, 4096 * sizeof(float), ctx->stream);
  if (rc != GT_OK) return rc;
  float* partial = (float*)ctx->workspace;
  sum_partial_kernel<<<blocks, EW_THREADS, 0, ctx->stream>>>(x, partial, n);
  sum_final_kernel<<<1, EW_THREADS, 0, ctx->stream>>>(partial, out, (int)blocks, accumulate);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 2;
  return GT_OK;
}

static int colsum_acc_on(gt_ctx* ctx, cudaStream_t stream, float* db, const float* dy, int64_t rows, int64_t cols, int64_t ld,
                         int64_t batch = 1, int64_t db_stride = 0, int64_t dy_stride = 0);

extern "C" int gt_colsum_acc(gt_ctx* ctx, float* db, const float* dy, int64_t rows, int64_t cols, int64_t ld) {
  if (!ctx) return GT_ERR_INVALID_ARG;
  return colsum_acc_on(ctx, ctx->stream, db, dy, rows, cols, ld);
}

// The column sums of a Linear layer's dY are memory-bound, read what the dX and dW GEMMs that follow read, and write
// only the bias gradient: put on a second stream that forks here, they run beside those GEMMs (whose persistent CTAs
// leave room for small blocks on every SM) instead of in front of them.  gt_join_beside makes the compute stream wait
// for them; call it before dY is freed or rewritten and before the bias gradient is read.
extern "C" int gt_colsum_acc_beside(gt_ctx* ctx, float* db, const float* dy, int64_t rows, int64_t cols, int64_t ld) {
  return gt_colsum_acc_batched_beside(ctx, db, 0, dy, 0, rows, cols, ld, 1);
}

// `batch` matrices dy + i * dy_stride (rows x cols each) summed into db + i * db_stride in one launch: the q, k, v
// gradients of an attention layer, which sit in one buffer, and their three adjacent bias gradients.
extern "C" int gt_colsum_acc_batched_beside(gt_ctx* ctx, float* db, int64_t db_stride, const float* dy, int64_t dy_stride, int64_t rows,
                                            int64_t cols, int64_t ld, int64_t batch) {
  if (!ctx || batch <= 0 || batch > 65535) return GT_ERR_INVALID_ARG;
  static const bool off = getenv("GRADTUITY_NO_SIDE_STREAM") != nullptr;
  if (off) return colsum_acc_on(ctx, ctx->stream, db, dy, rows, cols, ld, batch, db_stride, dy_stride);
  if (!ctx->side_stream) {
    GT_CUDA_OK(ctx, cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking));
    GT_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->side_fork, cudaEventDisableTiming));
    GT_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->side_done, cudaEventDisableTiming));
  }
  if (ctx->side_saved) return colsum_acc_on(ctx, ctx->stream, db, dy, rows, cols, ld, batch, db_stride, dy_stride);   // already on the side stream
  GT_CUDA_OK(ctx, cudaEventRecord(ctx->side_fork, ctx->stream));
  GT_CUDA_OK(ctx, cudaStreamWaitEvent(ctx->side_stream, ctx->side_fork, 0));
  const int rc = colsum_acc_on(ctx, ctx->side_stream, db, dy, rows, cols, ld, batch, db_stride, dy_stride);
  // recorded even when the launch failed: a join must never wait on an event that was not recorded after its fork
  GT_CUDA_OK(ctx, cudaEventRecord(ctx->side_done, ctx->side_stream));
  ctx->side_pending = 1;
  if (dy && rows > 0 && ld > 0) gt_side_note_block(ctx, dy, (size_t)(((batch - 1) * (dy_stride > 0 ? dy_stride : 0) + rows * ld) * 4));
  return rc;
}

// Everything this context launches between gt_beside_begin and gt_beside_end goes to the side stream, ordered behind what
// the compute stream holds at the begin; gt_join_beside (or gt_sync, gt_device_status, a device-to-host copy) orders the
// compute stream behind it again.  For memory-bound work whose results the next kernels do not need: the second half of
// an optimizer step beside the first layers of the next forward pass.  The caller keeps alive what that work touches
// until the join, or notes it with gt_beside_touches so that gt_free joins by itself.
extern "C" int gt_beside_begin(gt_ctx* ctx) {
  if (!ctx || ctx->side_saved) return GT_ERR_INVALID_ARG;
  static const bool off = getenv("GRADTUITY_NO_SIDE_STREAM") != nullptr;
  if (off) return GT_OK;
  if (!ctx->side_stream) {
    GT_CUDA_OK(ctx, cudaStreamCreateWithFlags(&ctx->side_stream, cudaStreamNonBlocking));
    GT_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->side_fork, cudaEventDisableTiming));
    GT_CUDA_OK(ctx, cudaEventCreateWithFlags(&ctx->side_done, cudaEventDisableTiming));
  }
  GT_CUDA_OK(ctx, cudaEventRecord(ctx->side_fork, ctx->stream));
  GT_CUDA_OK(ctx, cudaStreamWaitEvent(ctx->side_stream, ctx->side_fork, 0));
  ctx->side_saved = ctx->stream;
  ctx->stream = ctx->side_stream;
  return GT_OK;
}

extern "C" int gt_beside_end(gt_ctx* ctx) {
  if (!ctx) return GT_ERR_INVALID_ARG;
  if (!ctx->side_saved) return GT_OK;              // side stream switched off, or no matching begin
  ctx->stream = ctx->side_saved;
  ctx->side_saved = nullptr;
  GT_CUDA_OK(ctx, cudaEventRecord(ctx->side_done, ctx->side_stream));
  ctx->side_pending = 1;
  return GT_OK;
}

extern "C" int gt_beside_touches(gt_ctx* ctx, const void* ptr, size_t nbytes) {
  if (!ctx || !ptr) return GT_ERR_INVALID_ARG;
  gt_side_note_block(ctx, ptr, nbytes);
  return GT_OK;
}

void gt_side_note_block(gt_ctx* ctx, const void* ptr, size_t nbytes) {
  if (ctx->side_nblocks < 0) return;
  if (ctx->side_nblocks >= 16) { ctx->side_nblocks = -1; return; }
  ctx->side_blocks[ctx->side_nblocks].ptr = (const char*)ptr;
  ctx->side_blocks[ctx->side_nblocks].nbytes = nbytes;
  ++ctx->side_nblocks;
}

bool gt_side_touches(gt_ctx* ctx, const void* ptr, size_t nbytes) {
  if (ctx->side_nblocks < 0) return true;
  const char* a = (const char*)ptr;
  for (int i = 0; i < ctx->side_nblocks; ++i) {
    const char* b = ctx->side_blocks[i].ptr;
    if (a < b + ctx->side_blocks[i].nbytes && b < a + (nbytes ? nbytes : 1)) return true;
  }
  return false;
}

extern "C" int gt_join_beside(gt_ctx* ctx) {
  if (!ctx) return GT_ERR_INVALID_ARG;
  if (ctx->side_pending && !ctx->side_saved) {
    GT_CUDA_OK(ctx, cudaStreamWaitEvent(ctx->stream, ctx->side_done, 0));
    ctx->side_pending = 0;
    ctx->side_nblocks = 0;
  }
  return GT_OK;
}

static int colsum_acc_on(gt_ctx* ctx, cudaStream_t stream, float* db, const float* dy, int64_t rows, int64_t cols, int64_t ld,
                         int64_t batch, int64_t db_stride, int64_t dy_stride) {
  if (!ctx || !db || !dy || rows <= 0 || cols <= 0 || cols > 0x7fffffff || ld < cols) return GT_ERR_INVALID_ARG;
  if (batch > 1 && !((((uintptr_t)dy & 15) == 0) && cols % 4 == 0 && ld % 4 == 0 && dy_stride % 4 == 0)) {
    for (int64_t i = 0; i < batch; ++i) {                 // the scalar kernel takes one matrix at a time
      const int rc = colsum_acc_on(ctx, stream, db + i * db_stride, dy + i * dy_stride, rows, cols, ld, 1, 0, 0);
      if (rc != GT_OK) return rc;
    }
    return GT_OK;
  }
  if ((((uintptr_t)dy & 15) == 0) && cols % 4 == 0 && ld % 4 == 0) {
    const unsigned gxv = (unsigned)((cols + 127) / 128);
    long long want = ((long long)ctx->sm_count * 4 + gxv * batch - 1) / (gxv * batch);
    const long long most = (rows + 31) / 32;
    if (want > most) want = most;
    if (want < 1) want = 1;
    if (want > 65535) want = 65535;
    const int rpbv = (int)((rows + want - 1) / want);
    const unsigned gyv = (unsigned)((rows + rpbv - 1) / rpbv);
    GT_CUDA_OK(ctx, gt_launch_overlapped(colsum_acc_vec_kernel, dim3(gxv, gyv, (unsigned)batch), dim3(256), 0, stream, db, dy, rows, (int)cols, ld, rpbv,
                                         (long long)db_stride, (long long)dy_stride));
    ctx->launches += 1;
    return GT_OK;
  }
  const unsigned gx = (unsigned)((cols + 31) / 32);
  long long want_y = ((long long)ctx->sm_count * 4 + gx - 1) / gx;
  long long max_y = (rows + 63) / 64;
  if (want_y > max_y) want_y = max_y;
  if (want_y < 1) want_y = 1;
  if (want_y > 65535) want_y = 65535;
  const int rpb = (int)((rows + want_y - 1) / want_y);
  const unsigned gy = (unsigned)((rows + rpb - 1) / rpb);
  colsum_acc_kernel<<<dim3(gx, gy), 256, 0, stream>>>(db, dy, rows, (int)cols, ld, rpb);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}
