// The non-GEMM kernels a GPT-2 training step needs around the GEMMs: causal softmax and its
// backward, LayerNorm, embedding gather / scatter-add, cross-entropy, AdamW, gradient norm,
// the (B,S,H,D) <-> (B,H,S,D) transposes.  Plain CUDA, fp32, memory-bound: one row per block
// (or per warp), coalesced float4 access where the pitch allows, two-stage reductions instead
// of one atomic per element.
//
// fp32 specifications followed (the reference's CUDA-C twins):
//   gradtuity/kernels_cuda/softmax_kernels.py   softmax fwd/bwd, softmax_with_causal_mask
//   gradtuity/kernels_cuda/layernorm_kernels.py layernorm fwd/bwd
//   gradtuity/kernels_cuda/gather_kernels.py    embedding gather / scatter-add
//   gradtuity/kernels_cuda/loss_kernels.py      cross-entropy fwd/bwd
//   gradtuity/kernels_cuda/optim_kernels.py     adamw_step
//   gradtuity/kernels_cuda/mask_kernels.py      transpose4d_12

#include "gt_internal.h"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// Block-wide reductions; every thread gets the result.  red: 33 floats of shared memory.
__device__ __forceinline__ float block_sum_all(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = l < nw ? red[l] : 0.0f;
    t = warp_sum(t);
    if (l == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float block_max_all(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = l < nw ? red[l] : -INFINITY;
    t = warp_max(t);
    if (l == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

// causal == 1: everything beyond the diagonal is written as 0.  causal == 2: zeros are written only
// up to the end of the row's 128-wide diagonal block; what lies beyond is left untouched, for
// consumers that contract over k-blocks up to the diagonal only (GT_GEMM_A_LOWER / AT_LOWER).
__device__ __forceinline__ int zero_end(int causal, int r, int cols) {
  if (causal != 2) return cols;
  const int e = (r / 128 + 1) * 128;
  return e < cols ? e : cols;
}

// ---- softmax ------------------------------------------------------------------------------------
// y = softmax(x) over the last dimension.  causal: row r of each (cols x cols) block keeps columns
// j <= r % cols; the rest are written as exactly 0 and never read (they may hold anything, e.g.
// the mask value of the GEMM's causal epilogue).  In-place (y == x) is allowed.
__global__ void __launch_bounds__(256) softmax_fwd_kernel(const float* x, float* y, long long rows, int cols, int causal) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const float* xr = x + row * cols;
  float* yr = y + row * cols;
  const int limit = causal ? (int)(row % cols) + 1 : cols;
  float m = -INFINITY;
  for (int j = threadIdx.x; j < limit; j += blockDim.x) m = fmaxf(m, xr[j]);
  m = block_max_all(m, red);
  float s = 0.0f;
  for (int j = threadIdx.x; j < limit; j += blockDim.x) s += __expf(xr[j] - m);
  s = block_sum_all(s, red);
  const float inv = 1.0f / s;
  const int zend = zero_end(causal, (int)(row % cols), cols);
  for (int j = threadIdx.x; j < zend; j += blockDim.x) yr[j] = j < limit ? __expf(xr[j] - m) * inv : 0.0f;
}

// dx = scale * y * (dy - sum_j y_j dy_j), written (not accumulated), as the reference's
// softmax_backward_kernel does.  causal: only columns j <= r % cols are read; the rest of dx is 0.
__global__ void __launch_bounds__(256) softmax_bwd_kernel(float* dx, const float* y, const float* dy, long long rows, int cols,
                                                          int causal, float scale) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const float* yr = y + row * cols;
  const float* dyr = dy + row * cols;
  float* dxr = dx + row * cols;
  const int limit = causal ? (int)(row % cols) + 1 : cols;
  float dot = 0.0f;
  for (int j = threadIdx.x; j < limit; j += blockDim.x) dot += yr[j] * dyr[j];
  dot = block_sum_all(dot, red);
  const int zend = zero_end(causal, (int)(row % cols), cols);
  for (int j = threadIdx.x; j < zend; j += blockDim.x) dxr[j] = j < limit ? scale * yr[j] * (dyr[j] - dot) : 0.0f;
}

// Vectorised forms for rows of up to 4096 floats whose length is a multiple of 4: the row is read
// ONCE into registers (float4), reduced, and written once.  Under the causal mask the columns
// beyond the diagonal are not read at all.
constexpr int SM_VEC_ITERS = 4;          // 256 threads x 4 iterations x 4 floats = 4096 columns
__global__ void __launch_bounds__(256) softmax_fwd_vec_kernel(const float* x, float* y, int cols, int causal) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const float4* xr = reinterpret_cast<const float4*>(x + row * cols);
  float4* yr = reinterpret_cast<float4*>(y + row * cols);
  const int limit = causal ? (int)(row % cols) + 1 : cols;
  float4 v[SM_VEC_ITERS];
  float m = -INFINITY;
#pragma unroll
  for (int it = 0; it < SM_VEC_ITERS; ++it) {
    const int j = (it * 256 + threadIdx.x) * 4;
    if (j < limit) {
      float4 t = xr[j >> 2];
      if (j + 1 >= limit) t.y = -INFINITY;
      if (j + 2 >= limit) t.z = -INFINITY;
      if (j + 3 >= limit) t.w = -INFINITY;
      v[it] = t;
      m = fmaxf(m, fmaxf(fmaxf(t.x, t.y), fmaxf(t.z, t.w)));
    } else {
      v[it] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
  }
  m = block_max_all(m, red);
  float s = 0.0f;
#pragma unroll
  for (int it = 0; it < SM_VEC_ITERS; ++it) {
    v[it].x = __expf(v[it].x - m); v[it].y = __expf(v[it].y - m); v[it].z = __expf(v[it].z - m); v[it].w = __expf(v[it].w - m);
    s += (v[it].x + v[it].y) + (v[it].z + v[it].w);
  }
  s = block_sum_all(s, red);
  const float inv = 1.0f / s;
  const int zend = zero_end(causal, (int)(row % cols), cols);
#pragma unroll
  for (int it = 0; it < SM_VEC_ITERS; ++it) {
    const int j = (it * 256 + threadIdx.x) * 4;
    if (j < zend) yr[j >> 2] = make_float4(v[it].x * inv, v[it].y * inv, v[it].z * inv, v[it].w * inv);   // exp(-inf) = 0 beyond the limit
  }
}

__global__ void __launch_bounds__(256) softmax_bwd_vec_kernel(float* dx, const float* y, const float* dy, int cols, int causal, float scale) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const float4* yr = reinterpret_cast<const float4*>(y + row * cols);
  const float4* dyr = reinterpret_cast<const float4*>(dy + row * cols);
  float4* dxr = reinterpret_cast<float4*>(dx + row * cols);
  const int limit = causal ? (int)(row % cols) + 1 : cols;
  float4 yv[SM_VEC_ITERS], gv[SM_VEC_ITERS];
  float dot = 0.0f;
#pragma unroll
  for (int it = 0; it < SM_VEC_ITERS; ++it) {
    const int j = (it * 256 + threadIdx.x) * 4;
    if (j < limit) {
      float4 a = yr[j >> 2], g = dyr[j >> 2];
      // beyond the diagonal y is 0 by construction, but dy may hold anything there
      if (j + 1 >= limit) { a.y = 0.f; g.y = 0.f; }
      if (j + 2 >= limit) { a.z = 0.f; g.z = 0.f; }
      if (j + 3 >= limit) { a.w = 0.f; g.w = 0.f; }
      yv[it] = a; gv[it] = g;
      dot += (a.x * g.x + a.y * g.y) + (a.z * g.z + a.w * g.w);
    } else {
      yv[it] = make_float4(0.f, 0.f, 0.f, 0.f); gv[it] = yv[it];
    }
  }
  dot = block_sum_all(dot, red);
  const int zend = zero_end(causal, (int)(row % cols), cols);
#pragma unroll
  for (int it = 0; it < SM_VEC_ITERS; ++it) {
    const int j = (it * 256 + threadIdx.x) * 4;
    if (j < zend)
      dxr[j >> 2] = make_float4(scale * yv[it].x * (gv[it].x - dot), scale * yv[it].y * (gv[it].y - dot),
                                scale * yv[it].z * (gv[it].z - dot), scale * yv[it].w * (gv[it].w - dot));
  }
}

// Warp-per-row forms for rows of 128 * NV floats (NV <= 16): a warp keeps its row in registers
// (NV float4 per lane), reduces with shuffles only, eight rows per block.  The block-per-row kernels
// above spend most of their time on block scheduling and barriers when a row is only 4 KB.
template <int NV>
__global__ void __launch_bounds__(256) softmax_fwd_warp_kernel(const float* x, float* y, long long rows, int causal) {
  constexpr int cols = 128 * NV;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float4* xr = reinterpret_cast<const float4*>(x + row * cols);
  float4* yr = reinterpret_cast<float4*>(y + row * cols);
  const int r = (int)(row % cols);
  const int limit = causal ? r + 1 : cols;
  const int zend = zero_end(causal, r, cols);
  float4 v[NV];
  float m = -INFINITY;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int j = (i * 32 + lane) * 4;
    if (j < limit) {
      float4 t = xr[i * 32 + lane];
      if (j + 1 >= limit) t.y = -INFINITY;
      if (j + 2 >= limit) t.z = -INFINITY;
      if (j + 3 >= limit) t.w = -INFINITY;
      v[i] = t;
      m = fmaxf(m, fmaxf(fmaxf(t.x, t.y), fmaxf(t.z, t.w)));
    } else {
      v[i] = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    }
  }
  m = warp_max(m);
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    v[i].x = __expf(v[i].x - m); v[i].y = __expf(v[i].y - m); v[i].z = __expf(v[i].z - m); v[i].w = __expf(v[i].w - m);
    s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
  }
  s = warp_sum(s);
  const float inv = 1.0f / s;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int j = (i * 32 + lane) * 4;
    if (j < zend) yr[i * 32 + lane] = make_float4(v[i].x * inv, v[i].y * inv, v[i].z * inv, v[i].w * inv);
  }
}

template <int NV>
__global__ void __launch_bounds__(256) softmax_bwd_warp_kernel(float* dx, const float* y, const float* dy, long long rows, int causal, float scale) {
  constexpr int cols = 128 * NV;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float4* yr = reinterpret_cast<const float4*>(y + row * cols);
  const float4* gr = reinterpret_cast<const float4*>(dy + row * cols);
  float4* dxr = reinterpret_cast<float4*>(dx + row * cols);
  const int r = (int)(row % cols);
  const int limit = causal ? r + 1 : cols;
  const int zend = zero_end(causal, r, cols);
  float4 yv[NV], gv[NV];
  float dot = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int j = (i * 32 + lane) * 4;
    if (j < limit) {
      float4 a = yr[i * 32 + lane], g = gr[i * 32 + lane];
      if (j + 1 >= limit) { a.y = 0.f; g.y = 0.f; }
      if (j + 2 >= limit) { a.z = 0.f; g.z = 0.f; }
      if (j + 3 >= limit) { a.w = 0.f; g.w = 0.f; }
      yv[i] = a; gv[i] = g;
      dot += (a.x * g.x + a.y * g.y) + (a.z * g.z + a.w * g.w);
    } else {
      yv[i] = make_float4(0.f, 0.f, 0.f, 0.f); gv[i] = yv[i];
    }
  }
  dot = warp_sum(dot);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int j = (i * 32 + lane) * 4;
    if (j < zend)
      dxr[i * 32 + lane] = make_float4(scale * yv[i].x * (gv[i].x - dot), scale * yv[i].y * (gv[i].y - dot),
                                       scale * yv[i].z * (gv[i].z - dot), scale * yv[i].w * (gv[i].w - dot));
  }
}

// ---- LayerNorm ----------------------------------------------------------------------------------
// y = (x - mean) * rstd * gamma + beta per row; mean and rstd are saved (two floats per row)
// and x-hat is recomputed in the backward instead of being stored.
__global__ void __launch_bounds__(256) layernorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                            const float* __restrict__ beta, float* __restrict__ y,
                                                            float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                            int H, float eps) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const float* xr = x + row * H;
  float s = 0.0f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) s += xr[j];
  const float mean = block_sum_all(s, red) / (float)H;
  float q = 0.0f;
  for (int j = threadIdx.x; j < H; j += blockDim.x) { const float d = xr[j] - mean; q += d * d; }
  const float var = block_sum_all(q, red) / (float)H;
  const float rstd = rsqrtf(var + eps);
  if (threadIdx.x == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }
  float* yr = y + row * H;
  for (int j = threadIdx.x; j < H; j += blockDim.x) yr[j] = (xr[j] - mean) * rstd * gamma[j] + beta[j];
}

// Warp-per-row form for H = 128 * KV (KV <= 8) and 16-byte aligned rows: the row is read once into
// registers as float4, mean and variance come from two warp reductions, no block-wide barrier.
template <int KV>
__global__ void __launch_bounds__(256) layernorm_fwd_warp_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                                                 const float* __restrict__ beta, float* __restrict__ y,
                                                                 float* __restrict__ mean_out, float* __restrict__ rstd_out,
                                                                 long long N, float eps) {
  constexpr int H = 128 * KV;
  gt_let_next_kernel_start();
  gt_wait_for_previous_kernel();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long warps_total = (long long)gridDim.x * 8;
  for (long long row = (long long)blockIdx.x * 8 + warp; row < N; row += warps_total) {
    const float4* xr = reinterpret_cast<const float4*>(x + row * H);
    float4 v[KV];
    float s = 0.0f;
#pragma unroll
    for (int c = 0; c < KV; ++c) { v[c] = xr[c * 32 + lane]; s += (v[c].x + v[c].y) + (v[c].z + v[c].w); }
    const float mean = warp_sum(s) / (float)H;
    float q = 0.0f;
#pragma unroll
    for (int c = 0; c < KV; ++c) {
      v[c].x -= mean; v[c].y -= mean; v[c].z -= mean; v[c].w -= mean;
      q += (v[c].x * v[c].x + v[c].y * v[c].y) + (v[c].z * v[c].z + v[c].w * v[c].w);
    }
    const float rstd = rsqrtf(warp_sum(q) / (float)H + eps);
    if (lane == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }
    float4* yr = reinterpret_cast<float4*>(y + row * H);
#pragma unroll
    for (int c = 0; c < KV; ++c) {
      const float4 g = reinterpret_cast<const float4*>(gamma)[c * 32 + lane], b = reinterpret_cast<const float4*>(beta)[c * 32 + lane];
      yr[c * 32 + lane] = make_float4(v[c].x * rstd * g.x + b.x, v[c].y * rstd * g.y + b.y, v[c].z * rstd * g.z + b.z, v[c].w * rstd * g.w + b.w);
    }
  }
}

// dx += rstd/H * (H*dxhat - sum(dxhat) - xhat*sum(dxhat*xhat)), dxhat = dy*gamma;
// dgamma += sum_rows dy*xhat, dbeta += sum_rows dy.  Each block walks `rows_per_block` rows and
// keeps its column partials in registers, so there is one atomic per column per block instead
// of one per element (the reference: gradtuity/kernels_cuda/layernorm_kernels.py:76-81).
constexpr int LN_MAX_COLS_PER_THREAD = 16;    // H <= 4096 with 256 threads
__global__ void __launch_bounds__(256) layernorm_bwd_kernel(float* __restrict__ dx, float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                            const float* __restrict__ dy, const float* __restrict__ x,
                                                            const float* __restrict__ mean, const float* __restrict__ rstd,
                                                            const float* __restrict__ gamma, long long N, int H, int rows_per_block,
                                                            int dx_accumulate) {
  __shared__ float red[33];
  float pg[LN_MAX_COLS_PER_THREAD], pb[LN_MAX_COLS_PER_THREAD];
#pragma unroll
  for (int c = 0; c < LN_MAX_COLS_PER_THREAD; ++c) { pg[c] = 0.0f; pb[c] = 0.0f; }
  const long long r0 = (long long)blockIdx.x * rows_per_block;
  long long r1 = r0 + rows_per_block; if (r1 > N) r1 = N;
  for (long long row = r0; row < r1; ++row) {
    const float mu = mean[row], rs = rstd[row];
    const float* xr = x + row * H;
    const float* dyr = dy + row * H;
    float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
    for (int c = 0; c < LN_MAX_COLS_PER_THREAD; ++c) {
      const int j = threadIdx.x + c * 256;
      if (j < H) {
        const float g = dyr[j];
        const float xh = (xr[j] - mu) * rs;
        const float dxh = g * gamma[j];
        s1 += dxh; s2 += dxh * xh;
        pg[c] += g * xh; pb[c] += g;
      }
    }
    s1 = block_sum_all(s1, red);
    s2 = block_sum_all(s2, red);
    const float invH = 1.0f / (float)H;
    if (dx) {
      float* dxr = dx + row * H;
#pragma unroll
      for (int c = 0; c < LN_MAX_COLS_PER_THREAD; ++c) {
        const int j = threadIdx.x + c * 256;
        if (j < H) {
          const float xh = (xr[j] - mu) * rs;
          const float dxh = dyr[j] * gamma[j];
          const float v = rs * invH * ((float)H * dxh - s1 - xh * s2);
          dxr[j] = dx_accumulate ? dxr[j] + v : v;
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < LN_MAX_COLS_PER_THREAD; ++c) {
    const int j = threadIdx.x + c * 256;
    if (j < H) {
      if (dgamma) atomicAdd(dgamma + j, pg[c]);
      if (dbeta) atomicAdd(dbeta + j, pb[c]);
    }
  }
}

// Warp-per-row form for H = 128 * KV (KV <= 8), float4 access: no block-wide barrier per row; the
// per-column partials of dgamma / dbeta stay in registers across the rows a warp visits and are
// combined through shared memory once per block.
template <int KV>
__global__ void __launch_bounds__(256) layernorm_bwd_warp_kernel(float* __restrict__ dx, float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                                 const float* __restrict__ dy, const float* __restrict__ x,
                                                                 const float* __restrict__ mean, const float* __restrict__ rstd,
                                                                 const float* __restrict__ gamma, long long N, int dx_accumulate,
                                                                 float* __restrict__ dx_colsum) {
  constexpr int H = 128 * KV;
  __shared__ float sg[H], sb[H], sd[H];
  gt_let_next_kernel_start();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int j = threadIdx.x; j < H; j += 256) { sg[j] = 0.0f; sb[j] = 0.0f; sd[j] = 0.0f; }
  __syncthreads();
  gt_wait_for_previous_kernel();
  // pd: column sums of the dx values as stored (after the accumulation): when dx is the finished gradient of the
  // residual stream, they are the bias gradient of the Linear layer that produced the stream, and the separate
  // pass over dx that would compute them is saved.
  float4 gam[KV], pg[KV], pb[KV], pd[KV];
#pragma unroll
  for (int c = 0; c < KV; ++c) {
    gam[c] = reinterpret_cast<const float4*>(gamma)[c * 32 + lane];
    pg[c] = make_float4(0.f, 0.f, 0.f, 0.f); pb[c] = pg[c]; pd[c] = pg[c];
  }
  const long long warps_total = (long long)gridDim.x * 8;
  for (long long row = (long long)blockIdx.x * 8 + warp; row < N; row += warps_total) {
    const float mu = mean[row], rs = rstd[row];
    const float4* xr = reinterpret_cast<const float4*>(x + row * H);
    const float4* gr = reinterpret_cast<const float4*>(dy + row * H);
    float4 xh[KV], dxh[KV], old[KV];
    float s1 = 0.0f, s2 = 0.0f;
    // what dx holds (when the result is added to it) is asked for together with x and dy, not after the row's sums are
    // known: one memory latency per row instead of two
    const bool add_old = dx != nullptr && dx_accumulate != 0;
#pragma unroll
    for (int c = 0; c < KV; ++c)
      old[c] = add_old ? reinterpret_cast<const float4*>(dx + row * H)[c * 32 + lane] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int c = 0; c < KV; ++c) {
      const float4 xv = xr[c * 32 + lane], g = gr[c * 32 + lane];
      xh[c] = make_float4((xv.x - mu) * rs, (xv.y - mu) * rs, (xv.z - mu) * rs, (xv.w - mu) * rs);
      dxh[c] = make_float4(g.x * gam[c].x, g.y * gam[c].y, g.z * gam[c].z, g.w * gam[c].w);
      s1 += (dxh[c].x + dxh[c].y) + (dxh[c].z + dxh[c].w);
      s2 += (dxh[c].x * xh[c].x + dxh[c].y * xh[c].y) + (dxh[c].z * xh[c].z + dxh[c].w * xh[c].w);
      pg[c].x += g.x * xh[c].x; pg[c].y += g.y * xh[c].y; pg[c].z += g.z * xh[c].z; pg[c].w += g.w * xh[c].w;
      pb[c].x += g.x; pb[c].y += g.y; pb[c].z += g.z; pb[c].w += g.w;
    }
    s1 = warp_sum(s1); s2 = warp_sum(s2);
    if (dx) {
      float4* dxr = reinterpret_cast<float4*>(dx + row * H);
      const float k = rs / (float)H;
#pragma unroll
      for (int c = 0; c < KV; ++c) {
        float4 v = make_float4(k * ((float)H * dxh[c].x - s1 - xh[c].x * s2), k * ((float)H * dxh[c].y - s1 - xh[c].y * s2),
                               k * ((float)H * dxh[c].z - s1 - xh[c].z * s2), k * ((float)H * dxh[c].w - s1 - xh[c].w * s2));
        if (add_old) { v.x += old[c].x; v.y += old[c].y; v.z += old[c].z; v.w += old[c].w; }
        dxr[c * 32 + lane] = v;
        pd[c].x += v.x; pd[c].y += v.y; pd[c].z += v.z; pd[c].w += v.w;
      }
    }
  }
#pragma unroll
  for (int c = 0; c < KV; ++c) {
    const int j = (c * 32 + lane) * 4;
    atomicAdd(&sg[j], pg[c].x); atomicAdd(&sg[j + 1], pg[c].y); atomicAdd(&sg[j + 2], pg[c].z); atomicAdd(&sg[j + 3], pg[c].w);
    atomicAdd(&sb[j], pb[c].x); atomicAdd(&sb[j + 1], pb[c].y); atomicAdd(&sb[j + 2], pb[c].z); atomicAdd(&sb[j + 3], pb[c].w);
    if (dx_colsum) { atomicAdd(&sd[j], pd[c].x); atomicAdd(&sd[j + 1], pd[c].y); atomicAdd(&sd[j + 2], pd[c].z); atomicAdd(&sd[j + 3], pd[c].w); }
  }
  __syncthreads();
  for (int j = threadIdx.x; j < H; j += 256) {
    if (dgamma) atomicAdd(dgamma + j, sg[j]);
    if (dbeta) atomicAdd(dbeta + j, sb[j]);
    if (dx_colsum) atomicAdd(dx_colsum + j, sd[j]);
  }
}

// ---- embedding ----------------------------------------------------------------------------------
// out[n, :] = W[idx[n], :]; indices are stored as floats (the engine has one dtype).  An index
// outside [0, V) raises the status word and is clamped, instead of the reference's host-side loop
// over a device-to-host copy (gradtuity/tensor.py:694-703).
__global__ void __launch_bounds__(256) embedding_gather_kernel(float* __restrict__ out, const float* __restrict__ W,
                                                               const float* __restrict__ idx, long long n, int D, int V, int* status) {
  const long long row = blockIdx.x;
  int t = (int)idx[row];
  if (t < 0 || t >= V) { if (threadIdx.x == 0) atomicExch(status, GT_ERR_INVALID_ARG); t = t < 0 ? 0 : V - 1; }
  const float* w = W + (long long)t * D;
  float* o = out + row * D;
  for (int j = threadIdx.x; j < D; j += blockDim.x) o[j] = w[j];
}
__global__ void __launch_bounds__(256) embedding_scatter_add_kernel(float* __restrict__ dW, const float* __restrict__ dout,
                                                                    const float* __restrict__ idx, long long n, int D, int V, float alpha) {
  const long long row = blockIdx.x;
  int t = (int)idx[row];
  if (t < 0 || t >= V) return;
  float* w = dW + (long long)t * D;
  const float* g = dout + row * D;
  for (int j = threadIdx.x; j < D; j += blockDim.x) atomicAdd(w + j, alpha * g[j]);
}

// ---- cross-entropy ------------------------------------------------------------------------------
// Per row: lse = log sum exp(logits), loss_row = lse - logits[target].  One pass over the row
// (online max / sum).  The per-row losses and lse values are kept; the mean is taken by a
// deterministic reduction, and the backward reuses lse.
// One block per row.  VEC: the row starts on a 16-byte boundary (pitch a multiple of 4 floats), so the
// body is read as float4 with a scalar tail; the running (max, sum) pair is rescaled once per vector.
template <bool VEC>
__global__ void __launch_bounds__(512) cross_entropy_fwd_kernel(const float* __restrict__ logits, long long ld,
                                                                const float* __restrict__ targets,
                                                                float* __restrict__ row_loss, float* __restrict__ row_lse,
                                                                int C, int* status) {
  __shared__ float red[33];
  const long long row = blockIdx.x;
  const float* xr = logits + row * ld;
  float m = -INFINITY, s = 0.0f;
  if (VEC) {
    const float4* x4 = reinterpret_cast<const float4*>(xr);
    const int n4 = C >> 2;
#pragma unroll 4
    for (int j = threadIdx.x; j < n4; j += blockDim.x) {
      const float4 v = x4[j];
      const float vm = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
      if (vm > m) { s *= __expf(m - vm); m = vm; }
      s += (__expf(v.x - m) + __expf(v.y - m)) + (__expf(v.z - m) + __expf(v.w - m));
    }
    const int j = (n4 << 2) + threadIdx.x;
    if (j < C) {
      const float v = xr[j];
      if (v > m) { s = s * __expf(m - v) + 1.0f; m = v; } else { s += __expf(v - m); }
    }
  } else {
    for (int j = threadIdx.x; j < C; j += blockDim.x) {
      const float v = xr[j];
      if (v > m) { s = s * __expf(m - v) + 1.0f; m = v; } else { s += __expf(v - m); }
    }
  }
  const float gm = block_max_all(m, red);
  s = (m == -INFINITY) ? 0.0f : s * __expf(m - gm);
  s = block_sum_all(s, red);
  if (threadIdx.x == 0) {
    int t = (int)targets[row];
    if (t < 0 || t >= C) { atomicExch(status, GT_ERR_INVALID_ARG); t = t < 0 ? 0 : C - 1; }
    const float lse = gm + logf(s);
    row_lse[row] = lse;
    row_loss[row] = lse - xr[t];
  }
}
// Loss and gradient in one launch: pass 1 as cross_entropy_fwd_kernel, then, the row still being in L2 (the launch
// asks for enough shared memory that only two 512-thread blocks share an SM: about 300 rows of 200 KB in flight, read
// and written, against 126 MB of L2), pass 2 writes dlogits = scale * (softmax - onehot).  Saves the second pass over
// HBM (1.65 GB for GPT-2's logits) and a launch; valid when the loss's upstream gradient is known at forward time.
constexpr int CE_FUSED_SMEM = 100 * 1024;
template <bool VEC>
__global__ void __launch_bounds__(512) cross_entropy_fused_kernel(float* __restrict__ dlogits, long long ld_d,
                                                                  const float* __restrict__ logits, long long ld_x,
                                                                  const float* __restrict__ targets, float* __restrict__ row_loss,
                                                                  float* __restrict__ row_lse, float scale, int C, int* status) {
  __shared__ float red[33];
  __shared__ float s_lse;
  __shared__ int s_t;
  const long long row = blockIdx.x;
  const float* xr = logits + row * ld_x;
  float* dr = dlogits + row * ld_d;
  float m = -INFINITY, s = 0.0f;
  if (VEC) {
    const float4* x4 = reinterpret_cast<const float4*>(xr);
    const int n4 = C >> 2;
#pragma unroll 4
    for (int j = threadIdx.x; j < n4; j += blockDim.x) {
      const float4 v = x4[j];
      const float vm = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
      if (vm > m) { s *= __expf(m - vm); m = vm; }
      s += (__expf(v.x - m) + __expf(v.y - m)) + (__expf(v.z - m) + __expf(v.w - m));
    }
    const int j = (n4 << 2) + threadIdx.x;
    if (j < C) {
      const float v = xr[j];
      if (v > m) { s = s * __expf(m - v) + 1.0f; m = v; } else { s += __expf(v - m); }
    }
  } else {
    for (int j = threadIdx.x; j < C; j += blockDim.x) {
      const float v = xr[j];
      if (v > m) { s = s * __expf(m - v) + 1.0f; m = v; } else { s += __expf(v - m); }
    }
  }
  const float gm = block_max_all(m, red);
  s = (m == -INFINITY) ? 0.0f : s * __expf(m - gm);
  s = block_sum_all(s, red);
  if (threadIdx.x == 0) {
    int t = (int)targets[row];
    if (t < 0 || t >= C) { atomicExch(status, GT_ERR_INVALID_ARG); t = t < 0 ? 0 : C - 1; }
    const float lse = gm + logf(s);
    row_lse[row] = lse;
    row_loss[row] = lse - xr[t];
    s_lse = lse;
    s_t = t;
  }
  __syncthreads();
  const float lse = s_lse;
  const int t = s_t;
  int j0 = 0;
  if (VEC) {
    const float4* x4 = reinterpret_cast<const float4*>(xr);
    float4* d4 = reinterpret_cast<float4*>(dr);
    const int n4 = C >> 2;
#pragma unroll 4
    for (int j = threadIdx.x; j < n4; j += blockDim.x) {
      const float4 x = x4[j];
      float4 v;
      v.x = scale * __expf(x.x - lse); v.y = scale * __expf(x.y - lse); v.z = scale * __expf(x.z - lse); v.w = scale * __expf(x.w - lse);
      if ((t >> 2) == j) {
        const int k = t & 3;
        if (k == 0) v.x -= scale; else if (k == 1) v.y -= scale; else if (k == 2) v.z -= scale; else v.w -= scale;
      }
      d4[j] = v;
    }
    j0 = n4 << 2;
  }
  for (int j = j0 + threadIdx.x; j < C; j += blockDim.x) dr[j] = scale * (__expf(xr[j] - lse) - (j == t ? 1.0f : 0.0f));
}
// The same with the row held in shared memory, for rows of up to 56 000 classes that start on 16-byte boundaries
// (GPT-2's 50257 at a pitch of 50272): one persistent block per SM takes rows in turn; the bulk-copy engine brings a
// row in as a few chunks (an mbarrier each, so the first pass starts on chunk 0 while the last is still in flight),
// the second pass overwrites it in place with the gradient, and the engine writes it out chunk by chunk; a chunk of
// the next row is requested as soon as the store of the same chunk has been read out of shared memory, which is
// while the following chunk's gradient is being computed.  Every byte of the logits crosses HBM once in each
// direction, whatever the L2 holds.
constexpr int CE_ROW_CHUNKS = 8;          // chunks a short row is cut into (the launcher picks the number)
constexpr int CE_ROW_MAX_CHUNKS = 14;     // barriers provided
constexpr int CE_ROW_THREADS = 1024;
constexpr int CE_ROW_MAX_CLASSES = 56000;

__device__ __forceinline__ void ce_bar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void ce_bar_expect(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ce_bar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded: after about a second the block gives up, raises the status word and every thread leaves its loops.
__device__ __forceinline__ bool ce_bar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
  if (ce_bar_test(bar, parity)) return true;
  const long long t0 = clock64();
  while (true) {
    if (ce_bar_test(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > 2000000000LL) { *abort_flag = 1; atomicExch(status, GT_ERR_TIMEOUT); return false; }
  }
}

constexpr float CE_LOG2E = 1.4426950408889634f;
__device__ __forceinline__ float ce_ex2(float x) { float y; asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x)); return y; }

__global__ void __launch_bounds__(CE_ROW_THREADS, 1)
cross_entropy_row_in_smem_kernel(float* __restrict__ dlogits, long long ld_d, const float* __restrict__ logits, long long ld_x,
                                 const float* __restrict__ targets, float* __restrict__ row_loss, float* __restrict__ row_lse,
                                 float scale, int C, long long rows, int nchunks, int* status) {
  extern __shared__ __align__(128) uint8_t ce_smem[];
  __shared__ float red_m[32], red_s[32];                     // one (maximum, sum) pair per warp
  __shared__ __align__(8) unsigned long long bars[CE_ROW_MAX_CHUNKS];
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  float4* const row4 = reinterpret_cast<float4*>(ce_smem);
  const uint32_t row_addr = (uint32_t)__cvta_generic_to_shared(ce_smem);
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(bars);
  const int n4 = (C + 3) >> 2;                               // 16-byte units of a row (the pitch covers the last one)
  const int q4 = (n4 + nchunks - 1) / nchunks;               // units per chunk (none is empty: the caller admits C >= 4096 only)
  const int tid = threadIdx.x;
  if (tid == 0) {
    for (int c = 0; c < CE_ROW_MAX_CHUNKS; ++c) ce_bar_init(bar0 + 8 * c, 1);
    abort_word = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  auto request = [&](long long row, int c) {                 // chunk c of `row` -> shared memory
    const int u0 = c * q4, u1 = min(u0 + q4, n4);
    const uint32_t bytes = (uint32_t)(u1 - u0) * 16u;
    ce_bar_expect(bar0 + 8 * c, bytes);
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(row_addr + (uint32_t)u0 * 16u), "l"(logits + row * ld_x + (long long)u0 * 4), "r"(bytes), "r"(bar0 + 8 * c) : "memory");
  };
  long long row = blockIdx.x;
  if (tid == 0 && row < rows)
    for (int c = 0; c < nchunks; ++c) request(row, c);
  bool ok = true;
  uint32_t failed_parity = 0;
  for (int it = 0; ok && row < rows; row += gridDim.x, ++it) {
    const uint32_t parity = (uint32_t)(it & 1);
    const float t_early = targets[row];                        // asked for now by every thread, needed after the reduction
    // ---- pass 1: running maximum and sum, chunk by chunk as they arrive
    float m = -INFINITY, sum = 0.0f, m2 = 0.0f;                // m2 = -m log2(e), set with the first maximum
    for (int c = 0; c < nchunks; ++c) {
      if (!ce_bar_wait(bar0 + 8 * c, parity, abort_flag, status)) { ok = false; break; }     // leaves the chunk loop only
      const int u1 = min((c + 1) * q4, n4);
      for (int u = c * q4 + tid; u < u1; u += CE_ROW_THREADS) {
        float4 v = row4[u];
        if (4 * u + 3 >= C) {                                // the last unit of the row: columns beyond C do not exist
          if (4 * u + 1 >= C) v.y = -INFINITY;
          if (4 * u + 2 >= C) v.z = -INFINITY;
          v.w = -INFINITY;
        }
        const float vm = fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w));
        if (vm > m) { sum *= __expf(m - vm); m = vm; m2 = -vm * CE_LOG2E; }
        // e^(x - m) as 2^(x log2(e) - m log2(e)): one multiply-add and one ex2 per logit
        sum += (ce_ex2(fmaf(v.x, CE_LOG2E, m2)) + ce_ex2(fmaf(v.y, CE_LOG2E, m2))) + (ce_ex2(fmaf(v.z, CE_LOG2E, m2)) + ce_ex2(fmaf(v.w, CE_LOG2E, m2)));
      }
    }
    // One block-wide step between the passes: each warp reduces its (maximum, sum) pairs, the 32 warp results go through
    // shared memory, and every warp reduces those again for itself, so that all threads hold the log-sum-exp after a
    // single barrier (which is also the vote on `ok`: all threads leave together, or none).
    {
      const float wm = warp_max(m);
      sum = warp_sum(m == -INFINITY ? 0.0f : sum * __expf(m - wm));
      if ((tid & 31) == 0) { red_m[tid >> 5] = wm; red_s[tid >> 5] = sum; }
    }
    if (!__syncthreads_and(ok)) { ok = false; failed_parity = parity; break; }
    m = red_m[tid & 31];
    const float gm = warp_max(m);
    sum = warp_sum(m == -INFINITY ? 0.0f : red_s[tid & 31] * __expf(m - gm));
    const float lse = gm + logf(sum);
    const float k2 = log2f(scale) - lse * CE_LOG2E;
    int t = (int)t_early;
    if (t < 0 || t >= C) {
      if (tid == 0) atomicExch(status, GT_ERR_INVALID_ARG);
      t = t < 0 ? 0 : C - 1;
    }
    // ---- pass 2: the gradient over the row, in place; each chunk leaves as soon as the whole block has written it
    const long long next = row + gridDim.x;
    for (int c = 0; c < nchunks; ++c) {
      const int u0 = c * q4, u1 = min(u0 + q4, n4);
      for (int u = u0 + tid; u < u1; u += CE_ROW_THREADS) {
        const float4 x = row4[u];
        float4 g;
        // scale e^(x - lse) as 2^(x log2(e) + k), k = log2(scale) - lse log2(e): one multiply-add and one ex2 per logit
        g.x = ce_ex2(fmaf(x.x, CE_LOG2E, k2)); g.y = ce_ex2(fmaf(x.y, CE_LOG2E, k2)); g.z = ce_ex2(fmaf(x.z, CE_LOG2E, k2)); g.w = ce_ex2(fmaf(x.w, CE_LOG2E, k2));
        if ((t >> 2) == u) {                                 // the one thread that holds the target's logit also writes the loss
          const int k = t & 3;
          row_lse[row] = lse;
          row_loss[row] = lse - (k == 0 ? x.x : k == 1 ? x.y : k == 2 ? x.z : x.w);
          if (k == 0) g.x -= scale; else if (k == 1) g.y -= scale; else if (k == 2) g.z -= scale; else g.w -= scale;
        }
        if (4 * u + 3 >= C) {
          if (4 * u + 1 >= C) g.y = 0.0f;
          if (4 * u + 2 >= C) g.z = 0.0f;
          g.w = 0.0f;
        }
        row4[u] = g;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncthreads();
      if (tid == 0) {
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                     ::"l"(dlogits + row * ld_d + (long long)u0 * 4), "r"(row_addr + (uint32_t)u0 * 16u), "r"((uint32_t)(u1 - u0) * 16u) : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        // chunk c - 1 of the next row may come in once the store of chunk c - 1 has been read out of shared memory: it was
        // issued a chunk ago, so the wait is short, and the next row's first chunks are on their way while this row's
        // last ones are still being computed
        if (c >= 1 && next < rows) {
          asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          request(next, c - 1);
        }
      }
    }
    if (tid == 0 && next < rows) {
      asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
      request(next, nchunks - 1);
    }
  }
  if (tid == 0) {
    if (!ok) {     // giving up: let the copies of the row that was being waited for land (bounded) before shared memory is released
      const long long t0 = clock64();
      for (int c = 0; c < nchunks; ++c)
        while (!ce_bar_test(bar0 + 8 * c, failed_parity) && clock64() - t0 < 2000000000LL) {}
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
}

// dlogits (+)= scale * (softmax - onehot)
template <bool VEC>
__global__ void __launch_bounds__(512) cross_entropy_bwd_kernel(float* __restrict__ dlogits, long long ld_d,
                                                                const float* __restrict__ logits, long long ld_x,
                                                                const float* __restrict__ targets, const float* __restrict__ row_lse,
                                                                const float* __restrict__ upstream, float scale, int C, int accumulate) {
  const long long row = blockIdx.x;
  const float* xr = logits + row * ld_x;
  float* dr = dlogits + row * ld_d;
  const float lse = row_lse[row];
  const int t = (int)targets[row];
  const float sc = scale * (upstream ? *upstream : 1.0f);
  int j0 = 0;
  if (VEC) {
    const float4* x4 = reinterpret_cast<const float4*>(xr);
    float4* d4 = reinterpret_cast<float4*>(dr);
    const int n4 = C >> 2;
#pragma unroll 4
    for (int j = threadIdx.x; j < n4; j += blockDim.x) {
      const float4 x = x4[j];
      float4 v;
      v.x = sc * __expf(x.x - lse); v.y = sc * __expf(x.y - lse); v.z = sc * __expf(x.z - lse); v.w = sc * __expf(x.w - lse);
      if ((t >> 2) == j) {
        const int k = t & 3;
        if (k == 0) v.x -= sc; else if (k == 1) v.y -= sc; else if (k == 2) v.z -= sc; else v.w -= sc;
      }
      if (accumulate) { const float4 o = d4[j]; v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w; }
      d4[j] = v;
    }
    j0 = n4 << 2;
  }
  for (int j = j0 + threadIdx.x; j < C; j += blockDim.x) {
    const float v = sc * (__expf(xr[j] - lse) - (j == t ? 1.0f : 0.0f));
    dr[j] = accumulate ? dr[j] + v : v;
  }
}

// ---- optimizer ----------------------------------------------------------------------------------
// AdamW exactly as gradtuity/kernels_cuda/optim_kernels.py:23-46; grad_scale (read from device
// memory when given) folds the gradient-clipping factor into the update.
__global__ void __launch_bounds__(256) adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                                    float* __restrict__ v, long long n, float lr, float beta1, float beta2, float eps,
                                                    float wd, float bc1, float bc2, const float* __restrict__ grad_scale) {
  const float gs = grad_scale ? *grad_scale : 1.0f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    float pi = p[i];
    const float gi = g[i] * gs;
    const float mi = beta1 * m[i] + (1.0f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.0f - beta2) * gi * gi;
    const float upd = (mi * bc1) / (sqrtf(vi * bc2) + eps);
    pi = pi - lr * upd - lr * wd * pi;
    m[i] = mi; v[i] = vi; p[i] = pi;
  }
}

// out[0] (+)= sum x^2, deterministic two-stage.
__global__ void __launch_bounds__(256) sumsq_partial_kernel(const float* __restrict__ x, float* __restrict__ partial, long long n) {
  __shared__ float red[33];
  float s = 0.0f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) { const float v = x[i]; s += v * v; }
  s = block_sum_all(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void __launch_bounds__(256) sum_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, int n, int accumulate) {
  __shared__ float red[33];
  float s = 0.0f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = block_sum_all(s, red);
  if (threadIdx.x == 0) *out = accumulate ? *out + s : s;
}
// scale_out[0] = total_norm > max_norm ? max_norm / (total_norm + eps) : 1; norm_out[0] = total_norm
// (gradtuity/optim/utils.py:38-51, kept on the device so the step needs no host round trip).
__global__ void clip_scale_kernel(const float* __restrict__ sumsq, float max_norm, float eps, float* __restrict__ scale_out, float* __restrict__ norm_out) {
  const float nrm = sqrtf(*sumsq);
  *norm_out = nrm;
  *scale_out = nrm > max_norm ? max_norm / (nrm + eps) : 1.0f;
}
__global__ void __launch_bounds__(256) scale_by_device_scalar_kernel(float* __restrict__ x, const float* __restrict__ s, long long n) {
  const float v = *s;
  if (v == 1.0f) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) x[i] *= v;
}

// ---- multi-tensor forms -------------------------------------------------------------------------
// One launch over a list of tensors instead of one launch per parameter (the reference launches
// adamw_step once per tensor, gradtuity/optim/__init__.py:134-159, and clip_grad_norm_ runs a
// multiply, a sum and a host read per tensor, gradtuity/optim/utils.py:38-45).  The list is a
// device table of {p, g, m, v, n}; a second table maps each block to (tensor, first element).
struct MtTensor { float* p; const float* g; float* m; float* v; long long n; };
struct MtChunk { int tensor; int pad; long long start; };

__global__ void __launch_bounds__(256) adamw_multi_kernel(const MtTensor* __restrict__ tensors, const MtChunk* __restrict__ chunks,
                                                          long long chunk_elems, float lr, float beta1, float beta2, float eps,
                                                          float wd, float bc1, float bc2, const float* __restrict__ grad_scale) {
  const MtChunk c = chunks[blockIdx.x];
  const MtTensor t = tensors[c.tensor];
  const float gs = grad_scale ? *grad_scale : 1.0f;
  long long end = c.start + chunk_elems; if (end > t.n) end = t.n;
  long long begin = c.start;
  if (((((uintptr_t)t.p | (uintptr_t)t.g | (uintptr_t)t.m | (uintptr_t)t.v) & 15) == 0) && (c.start & 3) == 0) {
    // 16-byte aligned tensors: the body of the chunk as float4 (seven 16-byte accesses per four elements)
    const long long n4 = (end - c.start) >> 2;
    float4* p4 = reinterpret_cast<float4*>(t.p + c.start);
    const float4* g4 = reinterpret_cast<const float4*>(t.g + c.start);
    float4* m4 = reinterpret_cast<float4*>(t.m + c.start);
    float4* v4 = reinterpret_cast<float4*>(t.v + c.start);
    for (long long i = threadIdx.x; i < n4; i += blockDim.x) {
      float4 pv = p4[i], mv = m4[i], vv = v4[i];
      const float4 gv = g4[i];
      float* pp = reinterpret_cast<float*>(&pv); float* mm = reinterpret_cast<float*>(&mv); float* vq = reinterpret_cast<float*>(&vv);
      const float* gg = reinterpret_cast<const float*>(&gv);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gi = gg[k] * gs;
        const float mi = beta1 * mm[k] + (1.0f - beta1) * gi;
        const float vi = beta2 * vq[k] + (1.0f - beta2) * gi * gi;
        const float upd = (mi * bc1) / (sqrtf(vi * bc2) + eps);
        pp[k] = pp[k] - lr * upd - lr * wd * pp[k];
        mm[k] = mi; vq[k] = vi;
      }
      p4[i] = pv; m4[i] = mv; v4[i] = vv;
    }
    begin = c.start + (n4 << 2);
  }
  for (long long i = begin + threadIdx.x; i < end; i += blockDim.x) {
    float pi = t.p[i];
    const float gi = t.g[i] * gs;
    const float mi = beta1 * t.m[i] + (1.0f - beta1) * gi;
    const float vi = beta2 * t.v[i] + (1.0f - beta2) * gi * gi;
    const float upd = (mi * bc1) / (sqrtf(vi * bc2) + eps);
    pi = pi - lr * upd - lr * wd * pi;
    t.m[i] = mi; t.v[i] = vi; t.p[i] = pi;
  }
}

__global__ void __launch_bounds__(256) sumsq_multi_kernel(const MtTensor* __restrict__ tensors, const MtChunk* __restrict__ chunks,
                                                          long long chunk_elems, float* __restrict__ partial) {
  __shared__ float red[33];
  const MtChunk c = chunks[blockIdx.x];
  const MtTensor t = tensors[c.tensor];
  long long end = c.start + chunk_elems; if (end > t.n) end = t.n;
  float s = 0.0f;
  for (long long i = c.start + threadIdx.x; i < end; i += blockDim.x) { const float v = t.g[i]; s += v * v; }
  s = block_sum_all(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

// ---- (B, d1, d2, D) -> (B, d2, d1, D) ------------------------------------------------------------
__global__ void __launch_bounds__(256) transpose12_kernel(float* __restrict__ out, const float* __restrict__ in, int d1, int d2, int D, int accumulate) {
  // one block per (b, i1, i2) row of D elements
  const long long r = blockIdx.x;
  const int i2 = (int)(r % d2);
  const long long t = r / d2;
  const int i1 = (int)(t % d1);
  const long long b = t / d1;
  const float* src = in + r * D;
  float* dst = out + ((b * d2 + i2) * d1 + i1) * (long long)D;
  for (int j = threadIdx.x; j < D; j += blockDim.x) dst[j] = accumulate ? dst[j] + src[j] : src[j];
}

inline unsigned blocks_for(gt_ctx* ctx, long long n) {
  long long b = (n + 255) / 256, cap = (long long)ctx->sm_count * 8;
  if (b > cap) b = cap;
  return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace

#define GT_LAUNCH_CHECK(ctx, n_launches)          \
  GT_CUDA_OK(ctx, cudaGetLastError());            \
  (ctx)->launches += (n_launches);                \
  return GT_OK

extern "C" int gt_softmax(gt_ctx* ctx, float* y, const float* x, int64_t rows, int64_t cols, int causal) {
  if (!ctx || !y || !x || rows <= 0 || cols <= 0 || cols > 0x7fffffff || rows > 0x7fffffff) return GT_ERR_INVALID_ARG;
  const bool al16 = ((((uintptr_t)x | (uintptr_t)y) & 15) == 0);
  if (al16 && cols % 128 == 0 && cols <= 2048) {
    const unsigned nb = (unsigned)((rows + 7) / 8);
#define GT_SM_CASE(NV_) case NV_: softmax_fwd_warp_kernel<NV_><<<nb, 256, 0, ctx->stream>>>(x, y, rows, causal); break
    switch ((int)(cols / 128)) {
      GT_SM_CASE(1); GT_SM_CASE(2); GT_SM_CASE(3); GT_SM_CASE(4); GT_SM_CASE(5); GT_SM_CASE(6); GT_SM_CASE(7); GT_SM_CASE(8);
      GT_SM_CASE(9); GT_SM_CASE(10); GT_SM_CASE(11); GT_SM_CASE(12); GT_SM_CASE(13); GT_SM_CASE(14); GT_SM_CASE(15); GT_SM_CASE(16);
    }
#undef GT_SM_CASE
    GT_LAUNCH_CHECK(ctx, 1);
  }
  const bool vec = (cols % 4 == 0) && cols <= 256 * 4 * SM_VEC_ITERS && al16;
  if (vec) softmax_fwd_vec_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(x, y, (int)cols, causal);
  else softmax_fwd_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(x, y, rows, (int)cols, causal);
  GT_LAUNCH_CHECK(ctx, 1);
}

extern "C" int gt_softmax_backward(gt_ctx* ctx, float* dx, const float* y, const float* dy, int64_t rows, int64_t cols,
                                   int causal, float scale) {
  if (!ctx || !dx || !y || !dy || rows <= 0 || cols <= 0 || cols > 0x7fffffff || rows > 0x7fffffff) return GT_ERR_INVALID_ARG;
  const bool al16 = ((((uintptr_t)dx | (uintptr_t)y | (uintptr_t)dy) & 15) == 0);
  if (al16 && cols % 128 == 0 && cols <= 2048) {
    const unsigned nb = (unsigned)((rows + 7) / 8);
#define GT_SM_CASE(NV_) case NV_: softmax_bwd_warp_kernel<NV_><<<nb, 256, 0, ctx->stream>>>(dx, y, dy, rows, causal, scale); break
    switch ((int)(cols / 128)) {
      GT_SM_CASE(1); GT_SM_CASE(2); GT_SM_CASE(3); GT_SM_CASE(4); GT_SM_CASE(5); GT_SM_CASE(6); GT_SM_CASE(7); GT_SM_CASE(8);
      GT_SM_CASE(9); GT_SM_CASE(10); GT_SM_CASE(11); GT_SM_CASE(12); GT_SM_CASE(13); GT_SM_CASE(14); GT_SM_CASE(15); GT_SM_CASE(16);
    }
#undef GT_SM_CASE
    GT_LAUNCH_CHECK(ctx, 1);
  }
  const bool vec = (cols % 4 == 0) && cols <= 256 * 4 * SM_VEC_ITERS && al16;
  if (vec) softmax_bwd_vec_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(dx, y, dy, (int)cols, causal, scale);
  else softmax_bwd_kernel<<<(unsigned)rows, 256, 0, ctx->stream>>>(dx, y, dy, rows, (int)cols, causal, scale);
  GT_LAUNCH_CHECK(ctx, 1);
}

extern "C" int gt_layernorm(gt_ctx* ctx, float* y, float* mean, float* rstd, const float* x, const float* gamma,
                            const float* beta, int64_t N, int64_t H, float eps) {
  if (!ctx || !y || !mean || !rstd || !x || !gamma || !beta || N <= 0 || H <= 0 || N > 0x7fffffff || H > 0x7fffffff) return GT_ERR_INVALID_ARG;
  const bool al = ((((uintptr_t)x | (uintptr_t)y | (uintptr_t)gamma | (uintptr_t)beta) & 15) == 0);
  if (al && H % 128 == 0 && H / 128 <= 8) {
    long long wb = (N + 7) / 8, cap = (long long)ctx->sm_count * 8;
    const unsigned nb = (unsigned)(wb < cap ? wb : cap);
#define GT_LNF_CASE(KV_) case KV_: GT_CUDA_OK(ctx, gt_launch_overlapped(layernorm_fwd_warp_kernel<KV_>, dim3(nb), dim3(256), 0, ctx->stream, x, gamma, beta, y, mean, rstd, N, eps)); break
    switch ((int)(H / 128)) { GT_LNF_CASE(1); GT_LNF_CASE(2); GT_LNF_CASE(3); GT_LNF_CASE(4); GT_LNF_CASE(5); GT_LNF_CASE(6); GT_LNF_CASE(7); GT_LNF_CASE(8); }
#undef GT_LNF_CASE
    GT_LAUNCH_CHECK(ctx, 1);
  }
  layernorm_fwd_kernel<<<(unsigned)N, 256, 0, ctx->stream>>>(x, gamma, beta, y, mean, rstd, (int)H, eps);
  GT_LAUNCH_CHECK(ctx, 1);
}

extern "C" int gt_layernorm_backward(gt_ctx* ctx, float* dx, float* dgamma, float* dbeta, const float* dy, const float* x,
                                     const float* mean, const float* rstd, const float* gamma, int64_t N, int64_t H,
                                     int dx_accumulate) {
  return gt_layernorm_backward_colsum(ctx, dx, dgamma, dbeta, nullptr, dy, x, mean, rstd, gamma, N, H, dx_accumulate);
}

// The same, and dx_colsum[j] += sum over rows of dx[row, j] as stored (after the accumulation) when dx_colsum is given.
extern "C" int gt_layernorm_backward_colsum(gt_ctx* ctx, float* dx, float* dgamma, float* dbeta, float* dx_colsum, const float* dy,
                                            const float* x, const float* mean, const float* rstd, const float* gamma, int64_t N, int64_t H,
                                            int dx_accumulate) {
  if (!ctx || !dy || !x || !mean || !rstd || !gamma || N <= 0 || H <= 0 || N > 0x7fffffff || (dx_colsum && !dx)) return GT_ERR_INVALID_ARG;
  if (H > 256 * LN_MAX_COLS_PER_THREAD) GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "layernorm backward supports H <= %d, got %lld", 256 * LN_MAX_COLS_PER_THREAD, (long long)H);
  const bool al = ((((uintptr_t)dx | (uintptr_t)dy | (uintptr_t)x | (uintptr_t)gamma) & 15) == 0);
  if (al && H % 128 == 0 && H / 128 <= 8) {
    // One resident round of blocks (the kernel's registers allow one or two blocks per SM): every block
    // pays the prologue and the dgamma / dbeta atomics once, and each warp walks several rows.
    long long wb = (N + 7) / 8;
    unsigned nb = 0;
#define GT_LN_CASE(KV_) case KV_: { \
      static int per_sm = 0; \
      if (per_sm == 0) { \
        int v = 0; \
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, layernorm_bwd_warp_kernel<KV_>, 256, 0) != cudaSuccess || v < 1) v = 1; \
        per_sm = v; \
      } \
      const long long cap = (long long)ctx->sm_count * per_sm; \
      nb = (unsigned)(wb < cap ? wb : cap); \
      GT_CUDA_OK(ctx, gt_launch_overlapped(layernorm_bwd_warp_kernel<KV_>, dim3(nb), dim3(256), 0, ctx->stream, dx, dgamma, dbeta, dy, x, mean, rstd, gamma, N, dx_accumulate, dx_colsum)); } break
    switch ((int)(H / 128)) { GT_LN_CASE(1); GT_LN_CASE(2); GT_LN_CASE(3); GT_LN_CASE(4); GT_LN_CASE(5); GT_LN_CASE(6); GT_LN_CASE(7); GT_LN_CASE(8); }
#undef GT_LN_CASE
    GT_LAUNCH_CHECK(ctx, 1);
  }
  long long blocks = (long long)ctx->sm_count * 4;
  if (blocks > N) blocks = N;
  const int rpb = (int)((N + blocks - 1) / blocks);
  blocks = (N + rpb - 1) / rpb;
  layernorm_bwd_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(dx, dgamma, dbeta, dy, x, mean, rstd, gamma, N, (int)H, rpb, dx_accumulate);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  if (dx_colsum) return gt_colsum_acc(ctx, dx_colsum, dx, N, H, H);      // this form of the kernel does not carry the sums
  return GT_OK;
}

extern "C" int gt_embedding(gt_ctx* ctx, float* out, const float* W, const float* idx, int64_t n, int64_t D, int64_t V) {
  if (!ctx || !out || !W || !idx || n <= 0 || D <= 0 || V <= 0 || n > 0x7fffffff || D > 0x7fffffff || V > 0x7fffffff) return GT_ERR_INVALID_ARG;
  embedding_gather_kernel<<<(unsigned)n, 256, 0, ctx->stream>>>(out, W, idx, n, (int)D, (int)V, ctx->d_status);
  GT_LAUNCH_CHECK(ctx, 1);
}

extern "C" int gt_embedding_backward(gt_ctx* ctx, float* dW, const float* dout, const float* idx, int64_t n, int64_t D, int64_t V) {
  return gt_embedding_backward_scaled(ctx, dW, dout, idx, n, D, V, 1.0f);
}

// dW[idx[r], :] += alpha * dout[r, :]: the rows of several ranks, gathered, are added with alpha = 1 / world size.
extern "C" int gt_embedding_backward_scaled(gt_ctx* ctx, float* dW, const float* dout, const float* idx, int64_t n, int64_t D, int64_t V,
                                            float alpha) {
  if (!ctx || !dW || !dout || !idx || n <= 0 || D <= 0 || V <= 0 || n > 0x7fffffff || D > 0x7fffffff || V > 0x7fffffff) return GT_ERR_INVALID_ARG;
  embedding_scatter_add_kernel<<<(unsigned)n, 256, 0, ctx->stream>>>(dW, dout, idx, n, (int)D, (int)V, alpha);
  GT_LAUNCH_CHECK(ctx, 1);
}

extern "C" int gt_cross_entropy(gt_ctx* ctx, float* loss, float* row_loss, float* row_lse, const float* logits,
                                int64_t ld_logits, const float* targets, int64_t B, int64_t C, int mean) {
  if (!ctx || !loss || !row_loss || !row_lse || !logits || !targets || B <= 0 || C <= 0 || B > 0x7fffffff || C > 0x7fffffff ||
      ld_logits < C) return GT_ERR_INVALID_ARG;
  if ((((uintptr_t)logits & 15) == 0) && ld_logits % 4 == 0)
    cross_entropy_fwd_kernel<true><<<(unsigned)B, 512, 0, ctx->stream>>>(logits, ld_logits, targets, row_loss, row_lse, (int)C, ctx->d_status);
  else
    cross_entropy_fwd_kernel<false><<<(unsigned)B, 512, 0, ctx->stream>>>(logits, ld_logits, targets, row_loss, row_lse, (int)C, ctx->d_status);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  int rc = gt_sum_all(ctx, loss, row_loss, B, 0);
  if (rc != GT_OK) return rc;
  if (mean) return gt_scale(ctx, loss, loss, 1.0f / (float)B, 1, 0);
  return GT_OK;
}

// gt_cross_entropy and, in the same launch, dlogits = grad_scale * (softmax - onehot): grad_scale = upstream / B for a
// mean loss whose upstream gradient is known (1 when the loss is what backward() starts from), upstream for a sum.
extern "C" int gt_cross_entropy_fused(gt_ctx* ctx, float* loss, float* row_loss, float* row_lse, float* dlogits, int64_t ld_dlogits,
                                      const float* logits, int64_t ld_logits, const float* targets, int64_t B, int64_t C, int mean,
                                      float grad_scale) {
  if (!ctx || !loss || !row_loss || !row_lse || !dlogits || !logits || !targets || B <= 0 || C <= 0 || B > 0x7fffffff ||
      C > 0x7fffffff || ld_logits < C || ld_dlogits < C) return GT_ERR_INVALID_ARG;
  const bool vec = (((uintptr_t)logits & 15) == 0) && ld_logits % 4 == 0 && (((uintptr_t)dlogits & 15) == 0) && ld_dlogits % 4 == 0;
  static const bool row_in_smem = getenv("GRADTUITY_CE_NO_ROW_IN_SMEM") == nullptr;
  if (vec && row_in_smem && C >= 4096 && C <= CE_ROW_MAX_CLASSES && grad_scale > 0.0f) {     // the kernel folds log2(grad_scale) into an exponent
    const int bytes = (int)((C + 3) / 4 * 16);
    GT_SMEM_OPT_IN(ctx, cross_entropy_row_in_smem_kernel, CE_ROW_MAX_CLASSES * 4);      // once, for the widest row admitted
    // Chunks per row: eight for rows of up to 20 480 classes, chunks of about 40 KB beyond.  Measured at 50257 classes
    // (201 KB), 4 / 5 / 6 / 7 / 8 / 10 / 13 chunks: 0.576 / 0.531 / 0.560 / 0.558 / 0.602 / 0.724 / 0.658 ms: large
    // copies move faster, and the block's passes over a chunk should fill their last step (GRADTUITY_CE_CHUNKS overrides).
    static const int ce_chunks_env = getenv("GRADTUITY_CE_CHUNKS") ? atoi(getenv("GRADTUITY_CE_CHUNKS")) : 0;
    const long long units = (C + 3) / 4;
    const int ce_chunks_rule = units >= 5120 ? (int)((units + 1280) / 2560) : CE_ROW_CHUNKS;
    const int ce_chunks_want = ce_chunks_env > 0 ? ce_chunks_env : ce_chunks_rule;
    const int ce_chunks = ce_chunks_want < 2 ? 2 : ce_chunks_want > CE_ROW_MAX_CHUNKS ? CE_ROW_MAX_CHUNKS : ce_chunks_want;
    const unsigned grid = (unsigned)(B < ctx->sm_count ? B : ctx->sm_count);
    cross_entropy_row_in_smem_kernel<<<grid, CE_ROW_THREADS, bytes, ctx->stream>>>(dlogits, ld_dlogits, logits, ld_logits, targets, row_loss, row_lse,
                                                                                  grad_scale, (int)C, (long long)B, ce_chunks, ctx->d_status);
  } else if (vec) {
    GT_SMEM_OPT_IN(ctx, cross_entropy_fused_kernel<true>, CE_FUSED_SMEM);
    cross_entropy_fused_kernel<true><<<(unsigned)B, 512, CE_FUSED_SMEM, ctx->stream>>>(dlogits, ld_dlogits, logits, ld_logits, targets, row_loss,
                                                                                      row_lse, grad_scale, (int)C, ctx->d_status);
  } else {
    GT_SMEM_OPT_IN(ctx, cross_entropy_fused_kernel<false>, CE_FUSED_SMEM);
    cross_entropy_fused_kernel<false><<<(unsigned)B, 512, CE_FUSED_SMEM, ctx->stream>>>(dlogits, ld_dlogits, logits, ld_logits, targets, row_loss,
                                                                                       row_lse, grad_scale, (int)C, ctx->d_status);
  }
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  int rc = gt_sum_all(ctx, loss, row_loss, B, 0);
  if (rc != GT_OK) return rc;
  if (mean) return gt_scale(ctx, loss, loss, 1.0f / (float)B, 1, 0);
  return GT_OK;
}

extern "C" int gt_cross_entropy_backward(gt_ctx* ctx, float* dlogits, int64_t ld_dlogits, const float* logits,
                                         int64_t ld_logits, const float* targets, const float* row_lse,
                                         const float* upstream, float scale, int64_t B, int64_t C, int accumulate) {
  if (!ctx || !dlogits || !logits || !targets || !row_lse || B <= 0 || C <= 0 || B > 0x7fffffff || C > 0x7fffffff ||
      ld_logits < C || ld_dlogits < C) return GT_ERR_INVALID_ARG;
  if ((((uintptr_t)logits & 15) == 0) && ld_logits % 4 == 0 && (((uintptr_t)dlogits & 15) == 0) && ld_dlogits % 4 == 0)
    cross_entropy_bwd_kernel<true><<<(unsigned)B, 512, 0, ctx->stream>>>(dlogits, ld_dlogits, logits, ld_logits, targets, row_lse, upstream, scale, (int)C, accumulate);
  else
    cross_entropy_bwd_kernel<false><<<(unsigned)B, 512, 0, ctx->stream>>>(dlogits, ld_dlogits, logits, ld_logits, targets, row_lse, upstream, scale, (int)C, accumulate);
  GT_LAUNCH_CHECK(ctx, 1);
}

extern "C" int gt_adamw(gt_ctx* ctx, float* p, const float* g, float* m, float* v, int64_t n, float lr, float beta1,
                        float beta2, float eps, float weight_decay, float bc1, float bc2, const float* grad_scale) {
  if (!ctx || !p || !g || !m || !v || n <= 0) return GT_ERR_INVALID_ARG;
  adamw_kernel<<<blocks_for(ctx, n), 256, 0, ctx->stream>>>(p, g, m, v, n, lr, beta1, beta2, eps, weight_decay, bc1, bc2, grad_scale);
  GT_LAUNCH_CHECK(ctx, 1);
}

extern "C" int gt_sumsq(gt_ctx* ctx, float* out, const float* x, int64_t n, int accumulate) {
  if (!ctx || !out || !x || n <= 0) return GT_ERR_INVALID_ARG;
  int rc = gt_workspace_reserve(ctx, 8192 * sizeof(float), ctx->stream);
  if (rc != GT_OK) return rc;
  float* partial = (float*)ctx->workspace + 4096;
  const unsigned blocks = blocks_for(ctx, n);
  sumsq_partial_kernel<<<blocks, 256, 0, ctx->stream>>>(x, partial, n);
  sum_partials_kernel<<<1, 256, 0, ctx->stream>>>(partial, out, (int)blocks, accumulate);
  GT_LAUNCH_CHECK(ctx, 2);
}

extern "C" int gt_clip_scale(gt_ctx* ctx, float* scale_out, float* norm_out, const float* sumsq, float max_norm, float eps) {
  if (!ctx || !scale_out || !norm_out || !sumsq) return GT_ERR_INVALID_ARG;
  clip_scale_kernel<<<1, 1, 0, ctx->stream>>>(sumsq, max_norm, eps, scale_out, norm_out);
  GT_LAUNCH_CHECK(ctx, 1);
}

extern "C" int gt_scale_by_device_scalar(gt_ctx* ctx, float* x, const float* s, int64_t n) {
  if (!ctx || !x || !s || n <= 0) return GT_ERR_INVALID_ARG;
  scale_by_device_scalar_kernel<<<blocks_for(ctx, n), 256, 0, ctx->stream>>>(x, s, n);
  GT_LAUNCH_CHECK(ctx, 1);
}

extern "C" int gt_transpose12(gt_ctx* ctx, float* out, const float* in, int64_t B, int64_t d1, int64_t d2, int64_t D, int accumulate) {
  if (!ctx || !out || !in || B <= 0 || d1 <= 0 || d2 <= 0 || D <= 0) return GT_ERR_INVALID_ARG;
  const long long rows = B * d1 * d2;
  if (rows > 0x7fffffffLL || D > 0x7fffffff) return GT_ERR_INVALID_ARG;
  transpose12_kernel<<<(unsigned)rows, D >= 256 ? 256 : (D >= 128 ? 128 : 64), 0, ctx->stream>>>(out, in, (int)d1, (int)d2, (int)D, accumulate);
  GT_LAUNCH_CHECK(ctx, 1);
}

extern "C" int gt_adamw_multi(gt_ctx* ctx, const void* tensors, const void* chunks, int64_t n_chunks, int64_t chunk_elems,
                              float lr, float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
                              const float* grad_scale) {
  if (!ctx || !tensors || !chunks || n_chunks <= 0 || n_chunks > 0x7fffffff || chunk_elems <= 0) return GT_ERR_INVALID_ARG;
  adamw_multi_kernel<<<(unsigned)n_chunks, 256, 0, ctx->stream>>>((const MtTensor*)tensors, (const MtChunk*)chunks, chunk_elems, lr, beta1,
                                                                  beta2, eps, weight_decay, bc1, bc2, grad_scale);
  GT_LAUNCH_CHECK(ctx, 1);
}

// out[0] = sum over all listed gradients of g^2 (deterministic: per-chunk partials, then one block).
extern "C" int gt_sumsq_multi(gt_ctx* ctx, float* out, const void* tensors, const void* chunks, int64_t n_chunks, int64_t chunk_elems) {
  if (!ctx || !out || !tensors || !chunks || n_chunks <= 0 || chunk_elems <= 0) return GT_ERR_INVALID_ARG;
  if (n_chunks > 4096) GT_FAIL(ctx, GT_ERR_TOO_LARGE, "gt_sumsq_multi: at most 4096 chunks, got %lld", (long long)n_chunks);
  int rc = gt_workspace_reserve(ctx, 8192 * sizeof(float), ctx->stream);
  if (rc != GT_OK) return rc;
  float* partial = (float*)ctx->workspace + 4096;
  sumsq_multi_kernel<<<(unsigned)n_chunks, 256, 0, ctx->stream>>>((const MtTensor*)tensors, (const MtChunk*)chunks, chunk_elems, partial);
  sum_partials_kernel<<<1, 256, 0, ctx->stream>>>(partial, out, (int)n_chunks, 0);
  GT_LAUNCH_CHECK(ctx, 2);
}
