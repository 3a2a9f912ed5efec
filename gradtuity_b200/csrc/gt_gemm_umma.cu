// TF32 / 3xTF32 GEMM for sm_100a: TMA-fed shared-memory tiles, tcgen05.mma accumulating in
// tensor memory, fused epilogue.
//
// One persistent CTA (320 threads) per SM walks a list of 128 x BN output tiles (BN = 64, 128, 256;
// gt_gemm_umma256_kernel holds 256 x 256 tiles for large, long-K problems; gt_gemm_pair_kernel holds a
// 256 x 256 tile on a PAIR of CTAs, tcgen05 cta_group::2, for problems with K up to 4096).  Inside a CTA:
//   warp 0     producer   one lane issues cp.async.bulk.tensor (TMA) loads of A and B k-blocks
//                         (32 fp32 = one 128-byte swizzle row per k-block) into a ring of stages
//   warp 1     MMA        one lane issues tcgen05.mma.kind::tf32 (K = 8 per instruction) into
//                         one of two tensor-memory accumulators; tcgen05.commit hands stages
//                         back to the producer and finished accumulators to the epilogue
//   warps 2-9  epilogue   two warps per tensor-memory lane quarter share a tile's 32-column chunks:
//                         tcgen05.ld the accumulator (lane = row), apply alpha / bias / ReLU / GELU /
//                         causal mask / residual add / gelu', write the 32 x 32 block into a swizzled
//                         staging tile and hand it to TMA (store, or reduce-add for C += ...)
// so the epilogue of tile i overlaps the main loop of tile i+1.  With an A that TMA cannot describe,
// warps 6-9 copy it with cp.async instead and warps 2-5 are the epilogue.
//
// Work units: normally one tile each.  Few tiles and a long K: every tile is cut into K shares
// (split-K).  A last wave that is at most half full: only its tiles are cut.  Shares add into C with
// the TMA reduce-add (or, on request, go through a workspace and an ordered second kernel).
//
// NN / NT / TN are read straight from the row-major buffers: an operand whose contraction
// index is contiguous in memory is "K-major" (one TMA box of 32 x rows), the other kind is
// "MN-major" (32-wide chunks of 4 KB in the 32-byte-chunk swizzle that fp32 MN-major operands
// require, loaded as one five-dimensional box when the extent allows, else chunk by chunk); the
// instruction descriptor's major bits tell the tensor core which is which.  No transpose is
// materialised.  Batch strides may be 0 (operand shared by the batch entries, or a C that receives
// their sum).
//
// 3xTF32: the operands are split beforehand into hi = x & 0xffffe000 and lo = x - hi (both
// exact); each k-step issues lo*hi, hi*lo, hi*hi into the same accumulator.
//
// Every wait in the kernel is bounded: when a limit runs out the waiting thread raises the
// CTA's abort flag and the context's status word (GT_ERR_TIMEOUT), all roles leave their
// loops, copies in flight are waited for (bounded), tensor memory is freed, the CTA returns.
//
// Replaces: gradtuity/kernels_triton/matmul_kernels.py:18-400 (five kernels, 32x32x32 tiles,
// tl.dot) and gradtuity/kernels_cuda/matmul_kernels.py:21-236.

#include <stdio.h>
#include <stdlib.h>

#include "gt_internal.h"
#include "gt_umma_common.cuh"

namespace {

constexpr int BK = 32;                       // fp32 elements per k-block = 128 bytes
constexpr int UMMA_K = 8;                    // tf32 elements per tcgen05.mma
constexpr int NUM_THREADS = 320;            // producer warp, MMA warp, 8 epilogue warps (two per tensor-memory lane quarter)
constexpr int NUM_THREADS_AGEN = 320;       // producer, MMA, 4 epilogue warps, 4 warps that copy an unaligned A with cp.async
constexpr int EPI_WARP_BYTES = 4096;                 // per epilogue warp: one 32 x 32 fp32 staging tile (TMA store / coalesced fallback)
constexpr int EPI_SCRATCH_BYTES = 8 * EPI_WARP_BYTES;
constexpr int MAX_STAGES = 8;
constexpr int X3_CHUNK_KB = 8;                // 3xTF32: k-blocks accumulated in tensor memory before an fp32 register add
constexpr int SMEM_BUDGET = 232448 - 1024 - 512 - EPI_SCRATCH_BYTES;   // 227 KB minus alignment slack, barriers, epilogue staging

struct UmmaParams {
  const float* A; long long lda, sA0, sA1;     // used only when A is copied with cp.async
  float* C; const float* bias; float* aux;
  float* colsum;                         // GT_EPI_GELU_GRAD: column sums of the result are added here (null: not wanted)
  long long bias_stride;                 // elements between the bias rows of consecutive batch entries (0: one shared bias)
  long long ldc, sC0, sC1;
  int M, N, K;
  int batch0;
  int tiles_m, tiles_n, num_tiles;       // num_tiles counts work units: output tiles x ksplit
  int ksplit, kb_per;                    // split-K: units per tile, k-blocks per unit
  long long ks_stride;                   // split-K: element offset between the partial-sum planes of C
  int group_m;
  int epilogue, accumulate, vec_ok;
  int flags;                             // GT_GEMM_* flags of gt_gemm_batched_ex
  int c_tma;                             // C is written by TMA store / reduce-add through shared memory
  int a_onebox, b_onebox;                // MN-major operand described as (32, K, MN/32, b0, b1): one TMA box per stage
  int tail_first, tail_split, tail_kb_per;   // last partial wave: tiles from tail_first on are cut into tail_split K shares
  int tail_zero, tail_epoch;             // C is not accumulated into: CTA i zeroes the i-th last-wave tile first and
  int* tail_flags;                       // publishes tail_flags[i] = tail_epoch; the shares wait for it before they add
  float alpha;
  int* status;
  // Dynamic tile scheduling: after its first unit (its block index) a CTA takes `gridDim.x + atomicAdd(sched, 1)`,
  // so a CTA that starts late (its SM was busy with another kernel, e.g. a collective) takes less work instead of
  // making the launch wait for its fixed share.  Null: static round-robin.  sched_reset: the counter of a later
  // launch, zeroed by this one.
  int* sched;
  int* sched_reset;
};

// Shared-memory ring through which the producer thread, which draws the work units, hands them to the MMA thread
// and the epilogue (and cp.async) warps of its CTA.
constexpr int SCHED_SLOTS = 4;
constexpr int SCHED_CONSUMERS = 9;            // the MMA thread + eight warps (epilogue, or epilogue + cp.async)
struct SchedRing {
  uint32_t full, empty;                       // SCHED_SLOTS mbarriers each
  volatile int* units;                        // SCHED_SLOTS ints
  bool dynamic;
};

// Producer side: publish `unit` (-1: no more work).  False when the CTA is aborting.
__device__ __forceinline__ bool sched_publish(const SchedRing& r, int unit, int& slot, uint32_t& ph, volatile int* abort_flag, int* status) {
  if (!r.dynamic) return true;
  if (!mbar_wait(r.empty + 8 * slot, ph ^ 1u, abort_flag, status)) return false;
  r.units[slot] = unit;
  mbar_arrive(r.full + 8 * slot);
  if (++slot == SCHED_SLOTS) { slot = 0; ph ^= 1u; }
  return true;
}

// Consumer side, called by every thread of a consuming warp (or by the lone MMA thread with whole_warp = false):
// the next unit of this CTA, -1 when there is none, -2 when the CTA is aborting.  `k` counts the units taken.
__device__ __forceinline__ int sched_take(const SchedRing& r, int num_units, int& k, int& slot, uint32_t& ph, bool whole_warp,
                                          volatile int* abort_flag, int* status) {
  if (!r.dynamic) {
    const long long u = (long long)blockIdx.x + (long long)k * gridDim.x;
    ++k;
    return u < num_units ? (int)u : -1;
  }
  if (!mbar_wait(r.full + 8 * slot, ph, abort_flag, status)) return -2;
  const int unit = r.units[slot];
  if (whole_warp) {
    __syncwarp();                              // every lane has read the slot
    if ((threadIdx.x & 31) == 0) mbar_arrive(r.empty + 8 * slot);
  } else {
    mbar_arrive(r.empty + 8 * slot);
  }
  if (++slot == SCHED_SLOTS) { slot = 0; ph ^= 1u; }
  ++k;
  return unit;
}

template <int BN, bool X3>
struct Cfg {
  static constexpr int A_BYTES = BM * BK * 4;                 // 16 KB
  static constexpr int B_BYTES = BN * BK * 4;
  static constexpr int STAGE_BYTES = (A_BYTES + B_BYTES) * (X3 ? 2 : 1);
  static constexpr int STAGES_RAW = SMEM_BUDGET / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > MAX_STAGES ? MAX_STAGES : STAGES_RAW;
  static constexpr int TMEM_COLS = (2 * BN) < 32 ? 32 : (2 * BN);   // 128 / 256 / 512: powers of two
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 512 + EPI_SCRATCH_BYTES;
};

// Tile list order: groups of `group_m` row-tiles sweep all column-tiles before the next
// group starts, so CTAs that run together share A and B panels in L2.
__device__ __forceinline__ void tile_coords(const UmmaParams& p, int unit, int& batch, int& tm, int& tn, int& ks) {
  int tile;
  if (p.tail_split > 1) {
    // Work units of the last, partial wave: each of its tiles is contracted by tail_split CTAs (ks = share),
    // all other tiles by one CTA over the whole K (ks = -1).
    if (unit < p.tail_first) { tile = unit; ks = -1; }
    else { const int u = unit - p.tail_first; tile = p.tail_first + u / p.tail_split; ks = u % p.tail_split; }
  } else {
    ks = unit % p.ksplit;
    tile = unit / p.ksplit;
  }
  const int per_batch = p.tiles_m * p.tiles_n;
  batch = tile / per_batch;
  const int t = tile - batch * per_batch;
  const int group_size = p.group_m * p.tiles_n;
  const int g = t / group_size;
  const int first_m = g * p.group_m;
  const int rows = min(p.tiles_m - first_m, p.group_m);
  const int r = t - g * group_size;
  tm = first_m + r % rows;
  tn = r / rows;
}

// k-blocks a work unit contracts over: its split-K share, narrowed when the caller has declared
// A triangular (attention: P and dS are zero above the diagonal, so the products that read them
// as A need only the k-blocks up to the tile's last row, and those that read them transposed
// only the k-blocks from the tile's first row on).
__device__ __forceinline__ void k_range(const UmmaParams& p, int tm, int ks, int num_kb, int& lo, int& hi) {
  if (p.tail_split > 1) {
    lo = ks < 0 ? 0 : ks * p.tail_kb_per;
    hi = ks < 0 ? num_kb : min(num_kb, lo + p.tail_kb_per);
  } else {
    lo = ks * p.kb_per;
    hi = min(num_kb, lo + p.kb_per);
  }
  if (p.flags & GT_GEMM_A_LOWER) hi = min(hi, ((tm + 1) * BM + BK - 1) / BK);
  if (p.flags & GT_GEMM_AT_LOWER) lo = max(lo, (tm * BM) / BK);
}

template <int BN>
__device__ __forceinline__ bool tile_is_masked(const UmmaParams& p, int tm, int tn) {
  return p.epilogue == GT_EPI_CAUSAL && (tn * BN > tm * BM + BM - 1);
}

// Fused epilogue for 32 consecutive columns of one output row: v holds the accumulator.
// cpre: the 32 values of C this chunk accumulates into, loaded ahead of time (or null).
__device__ __forceinline__ void epilogue_chunk(const UmmaParams& p, const float* bias, const float* v, int row, int nb, long long row_off,
                                               const float4* cpre = nullptr) {
  const bool full_chunk = (nb + 32 <= p.N);
  float* cptr = p.C + row_off + nb;
  const bool has_bias = p.epilogue >= GT_EPI_BIAS && p.epilogue <= GT_EPI_BIAS_GELU;
  if (full_chunk && p.vec_ok) {
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      float4 x = make_float4(p.alpha * v[j], p.alpha * v[j + 1], p.alpha * v[j + 2], p.alpha * v[j + 3]);
      if (has_bias) {
        const float4 b = *reinterpret_cast<const float4*>(bias + nb + j);
        x.x += b.x; x.y += b.y; x.z += b.z; x.w += b.w;
      }
      if (p.aux) *reinterpret_cast<float4*>(p.aux + row_off + nb + j) = x;
      if (p.epilogue == GT_EPI_BIAS_RELU) {
        x.x = fmaxf(x.x, 0.0f); x.y = fmaxf(x.y, 0.0f); x.z = fmaxf(x.z, 0.0f); x.w = fmaxf(x.w, 0.0f);
      } else if (p.epilogue == GT_EPI_BIAS_GELU) {
        x.x = gt_gelu_tanh(x.x); x.y = gt_gelu_tanh(x.y); x.z = gt_gelu_tanh(x.z); x.w = gt_gelu_tanh(x.w);
      } else if (p.epilogue == GT_EPI_CAUSAL) {
        const int col = nb + j;
        if (col > row) x.x = GT_CAUSAL_MASK_VALUE;
        if (col + 1 > row) x.y = GT_CAUSAL_MASK_VALUE;
        if (col + 2 > row) x.z = GT_CAUSAL_MASK_VALUE;
        if (col + 3 > row) x.w = GT_CAUSAL_MASK_VALUE;
      }
      float4* dst = reinterpret_cast<float4*>(cptr + j);
      if (p.accumulate) {
        const float4 o = cpre ? cpre[j >> 2] : *dst;
        x.x += o.x; x.y += o.y; x.z += o.z; x.w += o.w;
      }
      *dst = x;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int col = nb + j;
      if (col < p.N) {
        float x = p.alpha * v[j];
        if (has_bias) x += bias[col];
        if (p.aux) p.aux[row_off + col] = x;
        if (p.epilogue == GT_EPI_BIAS_RELU) x = fmaxf(x, 0.0f);
        else if (p.epilogue == GT_EPI_BIAS_GELU) x = gt_gelu_tanh(x);
        else if (p.epilogue == GT_EPI_CAUSAL && col > row) x = GT_CAUSAL_MASK_VALUE;
        if (p.accumulate) x += cptr[j];
        cptr[j] = x;
      }
    }
  }
}

// Loads the 32 floats of C that chunk `nb` of this thread's row will accumulate into.  Issued one
// chunk ahead (the first one before the accumulator is even ready), so the read latency of
// `C += ...` hides behind the main loop and the previous chunk instead of stalling every chunk.
__device__ __forceinline__ bool prefetch_c(const UmmaParams& p, bool enabled, int nb, long long row_off, float4* out) {
  if (!enabled || nb + 32 > p.N) return false;
  const float4* src = reinterpret_cast<const float4*>(p.C + row_off + nb);
#pragma unroll
  for (int j = 0; j < 8; ++j) out[j] = src[j];
  return true;
}

// Column sums of the 32 x 32 block a warp has just written into its staging tile (128-byte-swizzle order), added into
// colsum[nb ... nb + 31]: lane c reads column c of every row (one 128-byte row per instruction: no bank conflict) and
// the warp issues one 128-byte reduction.  Rows at or beyond M hold zeros (their operand rows are the TMA fill value).
// This is the bias gradient of the layer whose dX the product is, taken while the tile is still on the SM.
__device__ __forceinline__ void staged_tile_colsum(float* colsum, const uint8_t* tile, int lane, int nb, int n_end) {
  float s = 0.0f;
  const int g = lane >> 2, w = (lane & 3) << 2;
#pragma unroll
  for (int r = 0; r < 32; ++r) s += *reinterpret_cast<const float*>(tile + r * 128 + ((g ^ (r & 7)) << 4) + w);
  if (nb + lane < n_end) atomicAdd(colsum + nb + lane, s);
}

// Epilogue of one 32 x 32 block through shared memory and a TMA store.  Each lane owns one row:
// it applies the fused epilogue in registers, writes its 128-byte row into the staging tile in the
// 128-byte-swizzle order, and lane 0 hands the tile to the TMA unit, which writes whole rows,
// clips at M and N, and for `C += ...` performs the addition in L2 (no read of C by the SM).
// Each epilogue warp has one staging tile (a second tile per warp, or requesting the next chunk's
// accumulator columns early, measured no faster: the warps are bound by the instructions they issue,
// not by these latencies).  With an aux output the pre-activation is stored directly from registers.
// This is the general form: bias, aux and the output may end inside the chunk.
__device__ __forceinline__ void epilogue_chunk_tma_any(const UmmaParams& p, const float* bias, const CUtensorMap* map_c, const float* v, int lane,
                                                       int row0, int nb, int i0, int i1, long long row_off, bool row_ok,
                                                       uint8_t* tile, uint32_t tile_u32, int epi, bool add, bool aux_out, bool aux_staged) {
  const int row = row0 + lane;
  const bool has_bias = (epi >= GT_EPI_BIAS && epi <= GT_EPI_BIAS_GELU) || epi == GT_EPI_BIAS_ADD;
  const bool aux_in = epi == GT_EPI_BIAS_ADD || epi == GT_EPI_GELU_GRAD;       // aux is read, not written
  if (lane == 0) tma_store_wait_read<0>();          // the previous store of this warp has finished reading the tile
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 32; j += 4) {
    float4 x = make_float4(p.alpha * v[j], p.alpha * v[j + 1], p.alpha * v[j + 2], p.alpha * v[j + 3]);
    if (has_bias) {
      const int col = nb + j;                       // bias may end inside this chunk
      if (col + 3 < p.N) {
        const float4 b = *reinterpret_cast<const float4*>(bias + col);
        x.x += b.x; x.y += b.y; x.z += b.z; x.w += b.w;
      } else {
        if (col < p.N) x.x += bias[col];
        if (col + 1 < p.N) x.y += bias[col + 1];
        if (col + 2 < p.N) x.z += bias[col + 2];
      }
    }
    if (aux_in) {
      float a4[4] = {0.f, 0.f, 0.f, 0.f};
      if (aux_staged) {                             // a TMA load has put the block of aux into the tile (zeros outside the tensor)
        const float4 a = *reinterpret_cast<const float4*>(tile + lane * 128 + ((((j >> 2) ^ (lane & 7))) << 4));
        a4[0] = a.x; a4[1] = a.y; a4[2] = a.z; a4[3] = a.w;
      } else if (row_ok) {
#pragma unroll
        for (int t = 0; t < 4; ++t) if (nb + j + t < p.N) a4[t] = p.aux[row_off + nb + j + t];
      }
      if (epi == GT_EPI_BIAS_ADD) { x.x += a4[0]; x.y += a4[1]; x.z += a4[2]; x.w += a4[3]; }
      else { x.x *= gt_gelu_tanh_grad(a4[0]); x.y *= gt_gelu_tanh_grad(a4[1]); x.z *= gt_gelu_tanh_grad(a4[2]); x.w *= gt_gelu_tanh_grad(a4[3]); }
    } else if (aux_out && row_ok && nb + j + 3 < p.N) *reinterpret_cast<float4*>(p.aux + row_off + nb + j) = x;
    else if (aux_out && row_ok) {
      float* a = p.aux + row_off + nb + j;
      if (nb + j < p.N) a[0] = x.x;
      if (nb + j + 1 < p.N) a[1] = x.y;
      if (nb + j + 2 < p.N) a[2] = x.z;
    }
    if (epi == GT_EPI_BIAS_RELU) {
      x.x = fmaxf(x.x, 0.0f); x.y = fmaxf(x.y, 0.0f); x.z = fmaxf(x.z, 0.0f); x.w = fmaxf(x.w, 0.0f);
    } else if (epi == GT_EPI_BIAS_GELU) {
      x.x = gt_gelu_tanh(x.x); x.y = gt_gelu_tanh(x.y); x.z = gt_gelu_tanh(x.z); x.w = gt_gelu_tanh(x.w);
    } else if (epi == GT_EPI_CAUSAL) {
      const int col = nb + j;
      if (col > row) x.x = GT_CAUSAL_MASK_VALUE;
      if (col + 1 > row) x.y = GT_CAUSAL_MASK_VALUE;
      if (col + 2 > row) x.z = GT_CAUSAL_MASK_VALUE;
      if (col + 3 > row) x.w = GT_CAUSAL_MASK_VALUE;
    }
    *reinterpret_cast<float4*>(tile + lane * 128 + ((((j >> 2) ^ (lane & 7))) << 4)) = x;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  if (lane == 0) tma_store_4d(map_c, tile_u32, nb, row0, i0, i1, add);
  if (epi == GT_EPI_GELU_GRAD && p.colsum) staged_tile_colsum(p.colsum, tile, lane, nb, p.N);
}

// The same for a chunk that lies wholly inside N, with the epilogue kind fixed at compile time: no
// per-element branches, a third of the instructions of the general form.  The epilogue warps are
// instruction-bound on short-K problems (the score products, the 768-deep Linear layers), so this
// is what their throughput depends on.
template <int EPI, bool AUX, bool UNIT_ALPHA>
__device__ __forceinline__ void epilogue_chunk_tma_fast(const UmmaParams& p, const float* bias, const CUtensorMap* map_c, const float* v, int lane,
                                                        int row0, int nb, int i0, int i1, long long row_off, bool row_ok,
                                                        uint8_t* tile, uint32_t tile_u32, bool add, bool aux_staged) {
  constexpr bool HAS_BIAS = (EPI >= GT_EPI_BIAS && EPI <= GT_EPI_BIAS_GELU) || EPI == GT_EPI_BIAS_ADD;
  constexpr bool AUX_IN = EPI == GT_EPI_BIAS_ADD || EPI == GT_EPI_GELU_GRAD;     // aux is read, not written
  const int row = row0 + lane;
  const float alpha = p.alpha;
  const float4* bias4 = reinterpret_cast<const float4*>(bias + nb);
  float4* aux4 = reinterpret_cast<float4*>(p.aux + row_off + nb);
  uint8_t* my_row = tile + lane * 128;
  const int sw = lane & 7;
  if (lane == 0) tma_store_wait_read<0>();
  __syncwarp();
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float4 x = UNIT_ALPHA ? make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3])
                          : make_float4(alpha * v[4 * j], alpha * v[4 * j + 1], alpha * v[4 * j + 2], alpha * v[4 * j + 3]);
    if (HAS_BIAS) {
      const float4 b = bias4[j];
      x.x += b.x; x.y += b.y; x.z += b.z; x.w += b.w;
    }
    if (AUX_IN) {
      // aux_staged: a TMA load has put this block of aux into the tile, in the layout the result is written back in
      const float4 a = aux_staged ? *reinterpret_cast<const float4*>(my_row + ((j ^ sw) << 4))
                                  : (row_ok ? aux4[j] : make_float4(0.f, 0.f, 0.f, 0.f));
      if (EPI == GT_EPI_BIAS_ADD) { x.x += a.x; x.y += a.y; x.z += a.z; x.w += a.w; }
      else { x.x *= gt_gelu_tanh_grad(a.x); x.y *= gt_gelu_tanh_grad(a.y); x.z *= gt_gelu_tanh_grad(a.z); x.w *= gt_gelu_tanh_grad(a.w); }
    } else if (AUX) { if (row_ok) aux4[j] = x; }
    if (EPI == GT_EPI_BIAS_RELU) {
      x.x = fmaxf(x.x, 0.0f); x.y = fmaxf(x.y, 0.0f); x.z = fmaxf(x.z, 0.0f); x.w = fmaxf(x.w, 0.0f);
    } else if (EPI == GT_EPI_BIAS_GELU) {
      x.x = gt_gelu_tanh(x.x); x.y = gt_gelu_tanh(x.y); x.z = gt_gelu_tanh(x.z); x.w = gt_gelu_tanh(x.w);
    } else if (EPI == GT_EPI_CAUSAL) {
      const int col = nb + 4 * j;
      if (col > row) x.x = GT_CAUSAL_MASK_VALUE;
      if (col + 1 > row) x.y = GT_CAUSAL_MASK_VALUE;
      if (col + 2 > row) x.z = GT_CAUSAL_MASK_VALUE;
      if (col + 3 > row) x.w = GT_CAUSAL_MASK_VALUE;
    }
    *reinterpret_cast<float4*>(my_row + ((j ^ sw) << 4)) = x;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  if (lane == 0) tma_store_4d(map_c, tile_u32, nb, row0, i0, i1, add);
  if (EPI == GT_EPI_GELU_GRAD && p.colsum) staged_tile_colsum(p.colsum, tile, lane, nb, p.N);
}

__device__ __forceinline__ void epilogue_chunk_tma(const UmmaParams& p, const float* bias, const CUtensorMap* map_c, const float* v, int lane,
                                                   int row0, int nb, int i0, int i1, long long row_off, bool row_ok,
                                                   uint8_t* tile, uint32_t tile_u32, int epi, bool add, bool aux_staged = false) {
  // aux is an OUTPUT (pre-activation) only for the kinds that produce one, and never for a K share that merely adds
  const bool aux_out = p.aux != nullptr && epi == p.epilogue && epi != GT_EPI_BIAS_ADD && epi != GT_EPI_GELU_GRAD;
  // alpha == 1 (every Linear layer): the multiply is left out of the per-element work (warp-uniform choice)
#define GT_EPI_FAST(E, X)                                                                                                       \
  do {                                                                                                                          \
    if (p.alpha == 1.0f) epilogue_chunk_tma_fast<E, X, true>(p, bias, map_c, v, lane, row0, nb, i0, i1, row_off, row_ok, tile, tile_u32, add, aux_staged);  \
    else epilogue_chunk_tma_fast<E, X, false>(p, bias, map_c, v, lane, row0, nb, i0, i1, row_off, row_ok, tile, tile_u32, add, aux_staged); \
  } while (0)
  if (nb + 32 <= p.N) {                              // warp-uniform
    switch (epi) {
      case GT_EPI_NONE:
        if (!aux_out) { GT_EPI_FAST(GT_EPI_NONE, false); return; }
        break;
      case GT_EPI_BIAS:
        if (aux_out) GT_EPI_FAST(GT_EPI_BIAS, true); else GT_EPI_FAST(GT_EPI_BIAS, false);
        return;
      case GT_EPI_BIAS_RELU:
        if (aux_out) GT_EPI_FAST(GT_EPI_BIAS_RELU, true); else GT_EPI_FAST(GT_EPI_BIAS_RELU, false);
        return;
      case GT_EPI_BIAS_GELU:
        if (aux_out) GT_EPI_FAST(GT_EPI_BIAS_GELU, true); else GT_EPI_FAST(GT_EPI_BIAS_GELU, false);
        return;
      case GT_EPI_BIAS_ADD: GT_EPI_FAST(GT_EPI_BIAS_ADD, false); return;
      case GT_EPI_GELU_GRAD: GT_EPI_FAST(GT_EPI_GELU_GRAD, false); return;
      case GT_EPI_CAUSAL:
        if (!aux_out) {
          // a 32 x 32 block whose last column is not right of its first row holds no masked element
          if (nb + 31 > row0) GT_EPI_FAST(GT_EPI_CAUSAL, false); else GT_EPI_FAST(GT_EPI_NONE, false);
          return;
        }
        break;
      default: break;
    }
  }
#undef GT_EPI_FAST
  epilogue_chunk_tma_any(p, bias, map_c, v, lane, row0, nb, i0, i1, row_off, row_ok, tile, tile_u32, epi, add, aux_out, aux_staged);
}

// Same epilogue for outputs whose rows are not 16-byte aligned (odd leading dimension, e.g. the
// 50257-wide logits): the warp's 32 x 32 accumulator block goes through a shared-memory tile so
// that each store instruction writes 32 consecutive floats of ONE row, whatever its alignment.
__device__ __forceinline__ void epilogue_chunk_coalesced(const UmmaParams& p, const float* bias, const float* v, float* tile, int lane,
                                                         int row0, int nb, long long batch_off) {
#pragma unroll
  for (int j = 0; j < 32; ++j) tile[lane * 32 + (j ^ lane)] = v[j];      // XOR keeps both phases free of bank conflicts
  __syncwarp();
  const int col = nb + lane;
  const bool col_ok = col < p.N;
  const bool has_bias = p.epilogue >= GT_EPI_BIAS && p.epilogue <= GT_EPI_BIAS_GELU;
  const float b = (has_bias && col_ok) ? bias[col] : 0.0f;
  const int rows = min(32, p.M - row0);
  for (int r = 0; r < rows; ++r) {
    if (col_ok) {
      const int row = row0 + r;
      const long long off = batch_off + (long long)row * p.ldc + col;
      float x = p.alpha * tile[r * 32 + (lane ^ r)] + b;
      if (p.aux) p.aux[off] = x;
      if (p.epilogue == GT_EPI_BIAS_RELU) x = fmaxf(x, 0.0f);
      else if (p.epilogue == GT_EPI_BIAS_GELU) x = gt_gelu_tanh(x);
      else if (p.epilogue == GT_EPI_CAUSAL && col > row) x = GT_CAUSAL_MASK_VALUE;
      if (p.accumulate) x += p.C[off];
      p.C[off] = x;
    }
  }
  __syncwarp();
}

template <int BN, bool A_MN, bool B_MN, bool X3, bool A_GEN>
__global__ void __launch_bounds__(A_GEN ? NUM_THREADS_AGEN : NUM_THREADS, 1)
gt_gemm_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_a_lo, const __grid_constant__ CUtensorMap map_b_lo,
                    const __grid_constant__ CUtensorMap map_c, const UmmaParams p) {
  using C = Cfg<BN, X3>;
  constexpr int STAGES = C::STAGES;
  // Epilogue warp sets: two sets of four warps share a tile's 32-column chunks alternately; with
  // the cp.async warps present there is room for one set only.
  constexpr int EPI_SETS = A_GEN ? 1 : 2;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  uint8_t* epi_scratch = smem_aligned + STAGES * C::STAGE_BYTES;   // 1024-byte aligned: the stages are multiples of 1 KB
  uint8_t* ctrl = epi_scratch + EPI_SCRATCH_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);              // full[S], empty[S], tfull[2], tempty[2], drain
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 8 * (2 * MAX_STAGES + 5));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * MAX_STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * MAX_STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;
  const uint32_t bar_drain = bar_tempty + 16;
  SchedRing ring;
  ring.full = smem_u32(ctrl + 192);
  ring.empty = ring.full + 8 * SCHED_SLOTS;
  ring.units = reinterpret_cast<volatile int*>(ctrl + 192 + 16 * SCHED_SLOTS);
  ring.dynamic = p.sched != nullptr;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SCHED_SLOTS; ++s) { mbar_init(ring.full + 8 * s, 1); mbar_init(ring.empty + 8 * s, SCHED_CONSUMERS); }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, A_GEN ? 1 + 128 : 1);   // TMA issuer (+ one arrival per cp.async thread)
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 128 * EPI_SETS);
    }
    mbar_init(bar_drain, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  gt_let_next_kernel_start();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  gt_wait_for_previous_kernel();         // everything above ran beside the previous kernel's tail; global memory from here on
  if (p.sched_reset && threadIdx.x == 0 && blockIdx.x == 0) *p.sched_reset = 0;

  const int num_kb = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      long long issued = 0;
      bool ok = true;
      int sslot = 0; uint32_t sph = 0;
      long long next_unit = blockIdx.x;                 // the first unit is the CTA's own index, later ones are drawn
      while (ok) {
        const int tile = next_unit < p.num_tiles ? (int)next_unit : -1;
        if (!sched_publish(ring, tile, sslot, sph, abort_flag, p.status)) { ok = false; break; }
        if (tile < 0) break;
        // drawn now, needed only after this unit's loads have been issued: the atomic's latency hides behind them
        next_unit = ring.dynamic ? (long long)gridDim.x + atomicAdd(p.sched, 1) : next_unit + gridDim.x;
        int batch, tm, tn, ks;
        tile_coords(p, tile, batch, tm, tn, ks);
        int kb_lo, kb_hi;
        k_range(p, tm, ks, num_kb, kb_lo, kb_hi);
        if (tile_is_masked<BN>(p, tm, tn)) continue;
        const int i0 = batch % p.batch0, i1 = batch / p.batch0;
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status)) { ok = false; break; }
          const uint32_t full = bar_full + 8 * s;
          mbar_expect_tx(full, A_GEN ? C::B_BYTES : C::STAGE_BYTES);
          const uint32_t sa = smem_base + s * C::STAGE_BYTES;
          const uint32_t sb = sa + C::A_BYTES * (X3 ? 2 : 1);
          const int k0 = kb * BK;
          if (A_GEN) {
            // A arrives through the cp.async warps
          } else if (A_MN) {
            if (p.a_onebox) {
              tma_load_5d(sa, &map_a, full, 0, k0, m0 >> 5, i0, i1);
              if (X3) tma_load_5d(sa + C::A_BYTES, &map_a_lo, full, 0, k0, m0 >> 5, i0, i1);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 32; ++j) {
                tma_load_4d(sa + j * 4096, &map_a, full, m0 + 32 * j, k0, i0, i1);
                if (X3) tma_load_4d(sa + C::A_BYTES + j * 4096, &map_a_lo, full, m0 + 32 * j, k0, i0, i1);
              }
            }
          } else {
            tma_load_4d(sa, &map_a, full, k0, m0, i0, i1);
            if (X3) tma_load_4d(sa + C::A_BYTES, &map_a_lo, full, k0, m0, i0, i1);
          }
          if (B_MN) {
            if (p.b_onebox) {
              tma_load_5d(sb, &map_b, full, 0, k0, n0 >> 5, i0, i1);
              if (X3) tma_load_5d(sb + C::B_BYTES, &map_b_lo, full, 0, k0, n0 >> 5, i0, i1);
            } else {
#pragma unroll
              for (int j = 0; j < BN / 32; ++j) {
                tma_load_4d(sb + j * 4096, &map_b, full, n0 + 32 * j, k0, i0, i1);
                if (X3) tma_load_4d(sb + C::B_BYTES + j * 4096, &map_b_lo, full, n0 + 32 * j, k0, i0, i1);
              }
            }
          } else {
            tma_load_4d(sb, &map_b, full, k0, n0, i0, i1);
            if (X3) tma_load_4d(sb + C::B_BYTES, &map_b_lo, full, k0, n0, i0, i1);
          }
          ++issued;
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok) {
        // Aborting: let the loads already issued land before shared memory is released.
        long long first = issued > STAGES ? issued - STAGES : 0;
        for (long long i = first; i < issued; ++i) {
          const int st = (int)(i % STAGES);
          const uint32_t par = (uint32_t)((i / STAGES) & 1);
          const long long t0 = clock64();
          while (!mbar_try_wait(bar_full + 8 * st, par) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BN, A_MN, B_MN);
      int s = 0; uint32_t ph = 0;
      int acc = 0; uint32_t aph = 0;
      bool ok = true;
      bool any_issued = false;
      int sk = 0, sslot = 0; uint32_t sph = 0;
      while (ok) {
        const int tile = sched_take(ring, p.num_tiles, sk, sslot, sph, false, abort_flag, p.status);
        if (tile < 0) { ok = tile == -1; break; }
        int batch, tm, tn, ks;
        tile_coords(p, tile, batch, tm, tn, ks);
        int kb_lo, kb_hi;
        k_range(p, tm, ks, num_kb, kb_lo, kb_hi);
        if (tile_is_masked<BN>(p, tm, tn)) continue;
        // tf32: one accumulator per tile.  3xTF32: a fresh accumulator every X3_CHUNK_KB k-blocks,
        // because the tensor core truncates on every accumulate and the bias grows with the
        // length of the chain (measured 2.4e-6 relative per 1024 of K).
        const int chunk_kb = X3 ? X3_CHUNK_KB : (kb_hi - kb_lo);
        for (int kb0 = kb_lo; ok && kb0 < kb_hi; kb0 += chunk_kb) {
          if (!mbar_wait(bar_tempty + 8 * acc, aph ^ 1u, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
          const int kb1 = min(kb0 + chunk_kb, kb_hi);
          for (int kb = kb0; kb < kb1; ++kb) {
            if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status)) { ok = false; break; }
            if (A_GEN) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // cp.async wrote A through the generic proxy
            tc_fence_after();
            const uint32_t sa = smem_base + s * C::STAGE_BYTES;
            const uint32_t sb = sa + C::A_BYTES * (X3 ? 2 : 1);
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              // K-major: the 8 k-values of this step are 32 bytes further along each 128-byte row.
              // MN-major: they are the next 8 rows (1024 bytes) of every 32-wide column of atoms.
              const uint32_t a_off = A_MN ? kk * 1024 : kk * 32;
              const uint32_t b_off = B_MN ? kk * 1024 : kk * 32;
              const uint32_t a_lbo = A_MN ? 4096 : 16, b_lbo = B_MN ? 4096 : 16;
              const uint32_t a_sbo = A_MN ? 512 : 1024, b_sbo = B_MN ? 512 : 1024;
              const uint32_t a_sw = A_MN ? 1 : 2, b_sw = B_MN ? 1 : 2;
              const uint64_t ad = make_smem_desc(sa + a_off, a_lbo, a_sbo, a_sw);
              const uint64_t bd = make_smem_desc(sb + b_off, b_lbo, b_sbo, b_sw);
              const uint32_t keep = (kb != kb0 || kk != 0) ? 1u : 0u;   // 0: overwrite the accumulator
              if (X3) {
                const uint64_t ad_lo = make_smem_desc(sa + C::A_BYTES + a_off, a_lbo, a_sbo, a_sw);
                const uint64_t bd_lo = make_smem_desc(sb + C::B_BYTES + b_off, b_lbo, b_sbo, b_sw);
                tc_mma_tf32(d_tmem, ad_lo, bd, idesc, keep);
                tc_mma_tf32(d_tmem, ad, bd_lo, idesc, 1u);
                tc_mma_tf32(d_tmem, ad, bd, idesc, 1u);
              } else {
                tc_mma_tf32(d_tmem, ad, bd, idesc, keep);
              }
            }
            any_issued = true;
            tc_commit(bar_empty + 8 * s);          // stage reusable once these MMAs have read it
            if (++s == STAGES) { s = 0; ph ^= 1u; }
          }
          if (!ok) break;
          tc_commit(bar_tfull + 8 * acc);          // accumulator (chunk) complete
          if (++acc == 2) { acc = 0; aph ^= 1u; }
        }
      }
      if (!ok && any_issued) {
        // Aborting: wait (bounded) until the tensor core has retired what was issued.
        tc_commit(bar_drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(bar_drain, 0) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
      }
    }
  } else if (A_GEN && warp >= 6) {
    // ------------------------------ cp.async copy of A ------------------------------
    // A's leading dimension (or base) is not 16-byte aligned, so TMA cannot describe it.  These
    // 128 threads write the same swizzled tile TMA would have written, 4 bytes at a time, a warp
    // per 128-byte run; each thread's copies arrive on the stage's full barrier when they land.
    const int t = threadIdx.x - 192;
    int s = 0; uint32_t ph = 0;
    bool ok = true;
    int sk = 0, sslot = 0; uint32_t sph = 0;
    while (ok) {
      const int tile = sched_take(ring, p.num_tiles, sk, sslot, sph, true, abort_flag, p.status);
      if (tile < 0) break;
      int batch, tm, tn, ks;
      tile_coords(p, tile, batch, tm, tn, ks);
      int kb_lo, kb_hi;
      k_range(p, tm, ks, num_kb, kb_lo, kb_hi);
      if (tile_is_masked<BN>(p, tm, tn)) continue;
      const int i0 = batch % p.batch0, i1 = batch / p.batch0;
      const float* Ab = p.A + (long long)i0 * p.sA0 + (long long)i1 * p.sA1;
      const int m0 = tm * BM;
      for (int kb = kb_lo; kb < kb_hi; ++kb) {
        if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status)) { ok = false; break; }
        const uint32_t sa = smem_base + s * C::STAGE_BYTES;
        const int k0 = kb * BK;
        if (A_MN) {
          // stored (K, M): thread t owns column m0 + t of every k-row; a warp covers 32 consecutive m
          const int m = t;
          const bool m_ok = (m0 + m) < p.M;
          const uint32_t base = sa + (uint32_t)(m >> 5) * 4096u + (uint32_t)(m & 7) * 4u;
          const int c32 = (m & 31) >> 3;
#pragma unroll 8
          for (int kr = 0; kr < BK; ++kr) {
            const bool okk = m_ok && (k0 + kr) < p.K;
            const float* src = okk ? Ab + (long long)(k0 + kr) * p.lda + (m0 + m) : Ab;
            const uint32_t dst = base + (uint32_t)kr * 128u + (uint32_t)((c32 ^ (kr & 3)) << 5);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(okk ? 4 : 0) : "memory");
          }
        } else {
          // stored (M, K): a warp covers the 32 k-values of one row; thread t takes rows (t/32) + 4 i
          const int k = t & 31;
          const bool k_ok = (k0 + k) < p.K;
#pragma unroll 8
          for (int i = 0; i < BM / 4; ++i) {
            const int r = i * 4 + (t >> 5);
            const bool okk = k_ok && (m0 + r) < p.M;
            const float* src = okk ? Ab + (long long)(m0 + r) * p.lda + (k0 + k) : Ab;
            const uint32_t dst = sa + (uint32_t)r * 128u + (uint32_t)((((k >> 2) ^ (r & 7)) << 4) + (k & 3) * 4);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(okk ? 4 : 0) : "memory");
          }
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar_full + 8 * s) : "memory");
        if (++s == STAGES) { s = 0; ph ^= 1u; }
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else {
    // ------------------------------ epilogue ------------------------------
    const int q = warp & 3;                       // tensor-memory lane quarter this warp may read
    const int eset = (warp - 2) >> 2;             // which of the EPI_SETS warp sets this warp belongs to
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    uint8_t* epi_bytes = epi_scratch + (warp - 2) * EPI_WARP_BYTES;
    float* epi_tile = reinterpret_cast<float*>(epi_bytes);
    const uint32_t epi_u32 = smem_u32(epi_bytes);
    constexpr int MY_CHUNKS = (BN / 32 + EPI_SETS - 1) / EPI_SETS;     // chunks c = eset, eset + EPI_SETS, ...
    int acc = 0; uint32_t aph = 0;
    bool ok = true;
    // Last-wave split without C += ...: the shares of a last-wave tile ADD into C, so C must be zero under
    // that tile.  CTA i zeroes the i-th such tile now, a whole wave before any share can reach its epilogue:
    // one warp stores a zero-filled staging tile over it with TMA, waits for the stores to complete and
    // publishes the launch's epoch in the tile's flag.
    if (p.tail_split > 1 && p.tail_zero && warp == 2) {
      const int n_tail = (p.num_tiles - p.tail_first) / p.tail_split;
      if ((int)blockIdx.x < n_tail) {
        int batch, tm, tn, ks;
        tile_coords(p, p.tail_first + (int)blockIdx.x * p.tail_split, batch, tm, tn, ks);
#pragma unroll
        for (int g = 0; g < 8; ++g) *reinterpret_cast<float4*>(epi_bytes + lane * 128 + (g << 4)) = make_float4(0.f, 0.f, 0.f, 0.f);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          const int i0 = batch % p.batch0, i1 = batch / p.batch0;
          for (int r = 0; r < BM / 32; ++r)
            for (int c = 0; c < BN / 32; ++c)
              if (tn * BN + c * 32 < p.N && tm * BM + r * 32 < p.M)
                tma_store_4d(&map_c, epi_u32, tn * BN + c * 32, tm * BM + r * 32, i0, i1, false);
          tma_store_wait_all();
          asm volatile("fence.proxy.async;" ::: "memory");
          __threadfence();
          atomicExch(p.tail_flags + blockIdx.x, p.tail_epoch);
        }
        __syncwarp();
      }
    }
    int sk = 0, sslot = 0; uint32_t sph = 0;
    while (ok) {
      const int tile = sched_take(ring, p.num_tiles, sk, sslot, sph, true, abort_flag, p.status);
      if (tile < 0) break;
      int batch, tm, tn, ks;
      tile_coords(p, tile, batch, tm, tn, ks);
      int kb_lo, kb_hi;
      k_range(p, tm, ks, num_kb, kb_lo, kb_hi);
      const bool masked = tile_is_masked<BN>(p, tm, tn);
      if (masked && (p.flags & GT_GEMM_CAUSAL_SKIP_MASKED)) continue;     // the reader never looks above the diagonal
      const int i0 = batch % p.batch0, i1 = batch / p.batch0;
      const int row0 = tm * BM + q * 32;
      const int row = row0 + lane;
      const int n0 = tn * BN;
      const long long batch_off = (long long)i0 * p.sC0 + (long long)i1 * p.sC1 + (long long)ks * p.ks_stride;
      const long long row_off = batch_off + (long long)row * p.ldc;
      const bool row_ok = row < p.M;
      const float* unit_bias = p.bias ? p.bias + (long long)batch * p.bias_stride : nullptr;   // one bias row per batch entry when asked
      // a K share of a last-wave tile adds its partial sum into C; the bias goes in with share 0
      const bool tail_unit = p.tail_split > 1 && ks >= 0;
      const bool unit_add = p.accumulate != 0 || tail_unit;
      // bias and residual belong to one share; the gelu' factor multiplies the whole sum, so every share applies it
      const int unit_epi = (tail_unit && ks > 0 && p.epilogue != GT_EPI_GELU_GRAD) ? (int)GT_EPI_NONE : p.epilogue;
      if (tail_unit && p.tail_zero) {
        // the tile must have been zeroed before this share adds into it (bounded wait; normally already true)
        if (lane == 0) {
          const volatile int* flag = p.tail_flags + (tile - p.tail_first) / p.tail_split;
          const long long t0 = clock64();
          while (*flag != p.tail_epoch) {
            if (*abort_flag) break;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) { *abort_flag = 1; atomicExch(p.status, GT_ERR_TIMEOUT); break; }
          }
          __threadfence();
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        __syncwarp();
        if (*abort_flag) { ok = false; break; }
      }
      if constexpr (X3) {
        // The accumulator arrives in K-chunks; they are summed here in fp32 registers
        // (round-to-nearest adds) before the fused epilogue runs once.
        float sum[MY_CHUNKS * 32];
#pragma unroll
        for (int j = 0; j < MY_CHUNKS * 32; ++j) sum[j] = 0.0f;
        if (!masked) {
          const int nchunks = (kb_hi - kb_lo + X3_CHUNK_KB - 1) / X3_CHUNK_KB;
          for (int ch = 0; ch < nchunks; ++ch) {
            if (!mbar_wait(bar_tfull + 8 * acc, aph, abort_flag, p.status)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int lc = 0; lc < MY_CHUNKS; ++lc) {
              const int c = lc * EPI_SETS + eset;
              if (c < BN / 32 && n0 + c * 32 < p.N) {
                float v[32];
                tc_ld32(lane_base + (uint32_t)(acc * BN + c * 32), v);
                tc_wait_ld();
#pragma unroll
                for (int j = 0; j < 32; ++j) sum[lc * 32 + j] += v[j];
              }
            }
            tc_fence_before();
            mbar_arrive(bar_tempty + 8 * acc);
            if (++acc == 2) { acc = 0; aph ^= 1u; }
          }
          if (!ok) break;
        }
#pragma unroll
        for (int lc = 0; lc < MY_CHUNKS; ++lc) {
          const int c = lc * EPI_SETS + eset;
          const int nb = n0 + c * 32;
          if (c < BN / 32 && nb < p.N) {
            if (p.c_tma) epilogue_chunk_tma(p, unit_bias, &map_c, &sum[lc * 32], lane, row0, nb, i0, i1, row_off, row_ok, epi_bytes, epi_u32, p.epilogue, p.accumulate != 0);
            else if (p.vec_ok) { if (row_ok) epilogue_chunk(p, unit_bias, &sum[lc * 32], row, nb, row_off); }
            else epilogue_chunk_coalesced(p, unit_bias, &sum[lc * 32], epi_tile, lane, row0, nb, batch_off);
          }
        }
      } else {
        if (!masked) {
          if (!mbar_wait(bar_tfull + 8 * acc, aph, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
        }
#pragma unroll 1
        for (int c = eset; c < BN / 32; c += EPI_SETS) {
          const int nb = n0 + c * 32;
          if (nb >= p.N) break;
          float v[32];
          if (!masked) {
            tc_ld32(lane_base + (uint32_t)(acc * BN + c * 32), v);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.0f;
          }
          if (p.c_tma) epilogue_chunk_tma(p, unit_bias, &map_c, v, lane, row0, nb, i0, i1, row_off, row_ok, epi_bytes, epi_u32, unit_epi, unit_add);
          else if (p.vec_ok) { if (row_ok) epilogue_chunk(p, unit_bias, v, row, nb, row_off); }
          else epilogue_chunk_coalesced(p, unit_bias, v, epi_tile, lane, row0, nb, batch_off);
        }
        if (!masked) {
          tc_fence_before();
          mbar_arrive(bar_tempty + 8 * acc);        // every epilogue thread hands the accumulator back
          if (++acc == 2) { acc = 0; aph ^= 1u; }
        }
      }
    }
    if (p.c_tma && lane == 0) tma_store_wait_all();   // staging tiles must outlive the stores that read them
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLS) : "memory");
  }
}

// ---- 256 x 256 tiles ------------------------------------------------------------------------------
// For large tf32 problems.  A 128 x 256 tile needs 48 KB of operands per k-block, i.e. 96 bytes per
// cycle per SM at full tensor rate, and an SM takes in only about 64-69 bytes per cycle from L2
// (measured).  A 256 x 256 tile held by ONE CTA needs 64 KB per k-block for twice the flops = 64
// bytes per cycle: two M=128 MMAs per k-step share the B tile and write two accumulators that
// together fill tensor memory (2 x 256 columns).  Warps: 0 TMA producer, 1 MMA issuer, 2-5
// epilogue of rows 0-127, 6-9 epilogue of rows 128-255.  Three 64 KB stages.  Tensor memory is
// not double-buffered here, so a tile's epilogue does not overlap the next main loop (3 % at K = 8192);
// the host picks this kernel only for long K and at least one full wave of tiles.
constexpr int T256_STAGE_BYTES = 65536;
constexpr int T256_STAGES = 3;
constexpr int T256_THREADS = 320;
constexpr int T256_SMEM_BYTES = T256_STAGES * T256_STAGE_BYTES + 1024 + 512 + EPI_SCRATCH_BYTES;   // 8 warps x one 4 KB staging tile

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(T256_THREADS, 1)
gt_gemm_umma256_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       const __grid_constant__ CUtensorMap map_c, const UmmaParams p) {
  constexpr int STAGES = T256_STAGES;
  constexpr int TM = 256, TN = 256;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  uint8_t* epi_scratch = smem_aligned + STAGES * T256_STAGE_BYTES;
  uint8_t* ctrl = epi_scratch + EPI_SCRATCH_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 8 * (2 * MAX_STAGES + 5));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * MAX_STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * MAX_STAGES;     // [half]
  const uint32_t bar_tempty = bar_tfull + 16;                // [half]
  const uint32_t bar_drain = bar_tempty + 16;
  SchedRing ring;
  ring.full = smem_u32(ctrl + 192);
  ring.empty = ring.full + 8 * SCHED_SLOTS;
  ring.units = reinterpret_cast<volatile int*>(ctrl + 192 + 16 * SCHED_SLOTS);
  ring.dynamic = p.sched != nullptr;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SCHED_SLOTS; ++s) { mbar_init(ring.full + 8 * s, 1); mbar_init(ring.empty + 8 * s, SCHED_CONSUMERS); }
    for (int s = 0; s < STAGES; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int h = 0; h < 2; ++h) { mbar_init(bar_tfull + 8 * h, 1); mbar_init(bar_tempty + 8 * h, 128); }
    mbar_init(bar_drain, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  gt_let_next_kernel_start();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  gt_wait_for_previous_kernel();
  if (p.sched_reset && threadIdx.x == 0 && blockIdx.x == 0) *p.sched_reset = 0;
  const int num_kb = (p.K + BK - 1) / BK;
  constexpr uint32_t A_BYTES = TM * BK * 4;      // 32 KB

  if (warp == 0) {
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      long long issued = 0;
      bool ok = true;
      int sslot = 0; uint32_t sph = 0;
      long long next_unit = blockIdx.x;
      while (ok) {
        const int tile = next_unit < p.num_tiles ? (int)next_unit : -1;
        if (!sched_publish(ring, tile, sslot, sph, abort_flag, p.status)) { ok = false; break; }
        if (tile < 0) break;
        next_unit = ring.dynamic ? (long long)gridDim.x + atomicAdd(p.sched, 1) : next_unit + gridDim.x;
        int batch, tm, tn, ks;
        tile_coords(p, tile, batch, tm, tn, ks);
        const int i0 = batch % p.batch0, i1 = batch / p.batch0;
        const int m0 = tm * TM, n0 = tn * TN;
        const int kb_lo = ks * p.kb_per, kb_hi = min(num_kb, kb_lo + p.kb_per);      // this unit's share of K (all of it without split-K)
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status)) { ok = false; break; }
          const uint32_t full = bar_full + 8 * s;
          mbar_expect_tx(full, T256_STAGE_BYTES);
          const uint32_t sa = smem_base + s * T256_STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
          const int k0 = kb * BK;
          if (A_MN) {
            if (p.a_onebox) tma_load_5d(sa, &map_a, full, 0, k0, m0 >> 5, i0, i1);
            else {
#pragma unroll
              for (int j = 0; j < TM / 32; ++j) tma_load_4d(sa + j * 4096, &map_a, full, m0 + 32 * j, k0, i0, i1);
            }
          } else {
            tma_load_4d(sa, &map_a, full, k0, m0, i0, i1);                  // one 32 x 256 box
          }
          if (B_MN) {
            if (p.b_onebox) tma_load_5d(sb, &map_b, full, 0, k0, n0 >> 5, i0, i1);
            else {
#pragma unroll
              for (int j = 0; j < TN / 32; ++j) tma_load_4d(sb + j * 4096, &map_b, full, n0 + 32 * j, k0, i0, i1);
            }
          } else {
            tma_load_4d(sb, &map_b, full, k0, n0, i0, i1);
          }
          ++issued;
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok) {
        long long first = issued > STAGES ? issued - STAGES : 0;
        for (long long i = first; i < issued; ++i) {
          const long long t0 = clock64();
          while (!mbar_try_wait(bar_full + 8 * (int)(i % STAGES), (uint32_t)((i / STAGES) & 1)) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(TN, A_MN, B_MN);
      int s = 0; uint32_t ph = 0, tph = 0;
      bool ok = true, any_issued = false;
      int sk = 0, sslot = 0; uint32_t sph = 0;
      while (ok) {
        const int tile = sched_take(ring, p.num_tiles, sk, sslot, sph, false, abort_flag, p.status);
        if (tile < 0) { ok = tile == -1; break; }
        // both accumulators must have been drained by the previous tile's epilogue
        if (!mbar_wait(bar_tempty, tph ^ 1u, abort_flag, p.status)) { ok = false; break; }
        if (!mbar_wait(bar_tempty + 8, tph ^ 1u, abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        const int ks = tile % p.ksplit;
        const int kb_lo = ks * p.kb_per, kb_hi = min(num_kb, kb_lo + p.kb_per);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + s * T256_STAGE_BYTES;
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint32_t a_off = A_MN ? kk * 1024 : kk * 32;
            const uint32_t b_off = B_MN ? kk * 1024 : kk * 32;
            const uint64_t bd = make_smem_desc(sb + b_off, B_MN ? 4096 : 16, B_MN ? 512 : 1024, B_MN ? 1 : 2);
            const uint32_t keep = (kb != kb_lo || kk != 0) ? 1u : 0u;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              // rows 128 h .. 128 h + 127 of the A tile: 16 KB further (K-major) or four 4 KB column blocks further (MN-major)
              const uint64_t ad = make_smem_desc(sa + h * 16384 + a_off, A_MN ? 4096 : 16, A_MN ? 512 : 1024, A_MN ? 1 : 2);
              tc_mma_tf32(tmem_base + (uint32_t)(h * TN), ad, bd, idesc, keep);
            }
          }
          any_issued = true;
          tc_commit(bar_empty + 8 * s);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        tc_commit(bar_tfull);
        tc_commit(bar_tfull + 8);
        tph ^= 1u;
      }
      if (!ok && any_issued) {
        tc_commit(bar_drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(bar_drain, 0) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
      }
    }
  } else {
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(half * TN);
    uint8_t* epi_bytes = epi_scratch + (warp - 2) * 4096;
    const uint32_t epi_u32 = smem_u32(epi_bytes);
    uint32_t tph = 0;
    int sk = 0, sslot = 0; uint32_t sph = 0;
    while (true) {
      const int tile = sched_take(ring, p.num_tiles, sk, sslot, sph, true, abort_flag, p.status);
      if (tile < 0) break;
      int batch, tm, tn, ks;
      tile_coords(p, tile, batch, tm, tn, ks);
      const int i0 = batch % p.batch0, i1 = batch / p.batch0;
      const int row0 = tm * TM + half * 128 + q * 32;
      const int row = row0 + lane;
      const int n0 = tn * TN;
      const long long batch_off = (long long)i0 * p.sC0 + (long long)i1 * p.sC1;
      const long long row_off = batch_off + (long long)row * p.ldc;
      const bool row_ok = row < p.M;
      const float* unit_bias = p.bias ? p.bias + (long long)batch * p.bias_stride : nullptr;
      if (!mbar_wait(bar_tfull + 8 * half, tph, abort_flag, p.status)) break;
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < TN / 32; ++c) {
        const int nb = n0 + c * 32;
        if (nb >= p.N) break;
        float v[32];
        tc_ld32(lane_base + (uint32_t)(c * 32), v);
        tc_wait_ld();
        if (p.c_tma) {
          // with split-K every share adds its partial sum into C; bias / residual go in with share 0
          epilogue_chunk_tma(p, unit_bias, &map_c, v, lane, row0, nb, i0, i1, row_off, row_ok, epi_bytes, epi_u32,
                             (p.ksplit > 1 && ks > 0) ? (int)GT_EPI_NONE : p.epilogue, p.accumulate != 0 || p.ksplit > 1);
        } else if (row_ok) {
          epilogue_chunk(p, unit_bias, v, row, nb, row_off);     // host guarantees aligned rows for this kernel
        }
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * half);
      tph ^= 1u;
    }
    if (p.c_tma && lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---- 256 x 256 tiles held by a CTA PAIR (tcgen05 cta_group::2) -------------------------------------
// Two CTAs of a cluster, on two SMs, share one 256 x 256 output tile.  Each CTA loads its own half of both
// operands into its own shared memory (rows m0 + 128 r of A, columns n0 + 128 r of B for the CTA of rank r:
// 16 KB + 16 KB per k-block, straight from this GPU's memory, no multicast) and holds the accumulator of its
// own 128 rows (128 tensor-memory lanes x 256 columns).  One thread of the leader CTA (rank 0) issues
// tcgen05.mma.cta_group::2 for both: the tensor cores of the two SMs read A from their own CTA and B from both.
// Per SM that is 32 KB of operands per k-block for a 128 x 256 x 32 product: the 64 bytes per cycle the
// SM's L2 path sustains, where a single CTA's 128 x 256 tile needs 96.  Against the one-CTA 256 x 256 kernel
// above the stage is half as large (six stages instead of three) and the accumulator only half of tensor
// memory, so it is double-buffered and a tile's epilogue overlaps the next main loop, which is what the
// short-K (768) GEMMs of the GPT-2 step need.
//   barriers (all in shared memory, "leader's" = the copy in the CTA of rank 0):
//     full[s]   leader's only: one arrive.expect_tx by the leader's producer for the bytes of BOTH CTAs; all four
//               TMA loads of a k-block (two per CTA) complete on it
//     empty[s]  one per CTA: the leader's MMA thread commits to its own and to the peer's
//     tfull[a]  one per CTA, same; tempty[a] leader's only: one arrival per epilogue warp of either CTA
// Every wait is bounded as elsewhere; the CTAs leave together through a cluster barrier, so neither frees
// shared or tensor memory the other may still touch.
constexpr int PAIR_STAGE_BYTES = 32768;
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_THREADS = 320;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 512 + EPI_SCRATCH_BYTES;
static_assert(PAIR_SMEM_BYTES <= 232448, "CTA-pair kernel exceeds the 227 KB of shared memory a CTA may use");

template <bool A_MN, bool B_MN>
__global__ void __launch_bounds__(PAIR_THREADS, 1)
gt_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_aux, const UmmaParams p) {
  constexpr int STAGES = PAIR_STAGES;
  constexpr int TM = 256, TN = 256, HALF = 128;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_aligned = smem_raw + (smem_base - smem_u32(smem_raw));
  uint8_t* epi_scratch = smem_aligned + STAGES * PAIR_STAGE_BYTES;
  uint8_t* ctrl = epi_scratch + EPI_SCRATCH_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 8 * (2 * MAX_STAGES + 5));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * MAX_STAGES;
  const uint32_t bar_tfull = bar_empty + 8 * MAX_STAGES;
  const uint32_t bar_tempty = bar_tfull + 16;
  const uint32_t bar_drain = bar_tempty + 16;
  const uint32_t bar_aux = smem_u32(ctrl + 384);           // one per epilogue warp: its block of aux has landed in its staging tile
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                 // 0: leader
  const bool cta_wait = (p.flags & (1 << 30)) != 0;        // tuning aid: CTA-scope waits where no generic-proxy data crosses CTAs
  auto wait_x = [&](uint32_t bar, uint32_t parity) -> bool {
    return cta_wait ? mbar_wait(bar, parity, abort_flag, p.status) : mbar_wait_cluster(bar, parity, abort_flag, p.status);
  };
  const int first_unit = (int)cluster_id_x(), unit_step = (int)nclusters_x();

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, 16); }   // 8 epilogue warps x 2 CTAs
    mbar_init(bar_drain, 1);
    for (int w = 0; w < 8; ++w) mbar_init(bar_aux + 8 * w, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {      // the same warp in both CTAs, with the same destination slot
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  gt_let_next_kernel_start();
  tc_fence_before();
  __syncwarp();
  cluster_sync_all();                    // both CTAs' barriers exist before either signals the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  gt_wait_for_previous_kernel();
  const int num_kb = (p.K + BK - 1) / BK;
  const uint32_t leader_full = map_to_cta(bar_full, 0);
  const uint32_t leader_tempty = map_to_cta(bar_tempty, 0);

  if (warp == 0) {
    // ------------------------------ producer (one per CTA) ------------------------------
    if (lane == 0) {
      int s = 0; uint32_t ph = 0;
      long long issued = 0;
      bool ok = true;
      for (int unit = first_unit; ok && unit < p.num_tiles; unit += unit_step) {
        int batch, tm, tn, ks;
        tile_coords(p, unit, batch, tm, tn, ks);
        const int i0 = batch % p.batch0, i1 = batch / p.batch0;
        const int m0 = tm * TM + (int)rank * HALF, n0 = tn * TN + (int)rank * HALF;     // this CTA's halves
        int kb_lo, kb_hi;
        k_range(p, tm, ks, num_kb, kb_lo, kb_hi);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!wait_x(bar_empty + 8 * s, ph ^ 1u)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(bar_full + 8 * s, 2 * PAIR_STAGE_BYTES);
          const uint32_t full = leader_full + 8 * s;
          const uint32_t sa = smem_base + s * PAIR_STAGE_BYTES;
          const uint32_t sb = sa + HALF * BK * 4;
          const int k0 = kb * BK;
          if (A_MN) {
            if (p.a_onebox) tma_load_5d_pair(sa, &map_a, full, 0, k0, m0 >> 5, i0, i1);
            else {
#pragma unroll
              for (int j = 0; j < HALF / 32; ++j) tma_load_4d_pair(sa + j * 4096, &map_a, full, m0 + 32 * j, k0, i0, i1);
            }
          } else {
            tma_load_4d_pair(sa, &map_a, full, k0, m0, i0, i1);                 // one 32 x 128 box
          }
          if (B_MN) {
            if (p.b_onebox) tma_load_5d_pair(sb, &map_b, full, 0, k0, n0 >> 5, i0, i1);
            else {
#pragma unroll
              for (int j = 0; j < HALF / 32; ++j) tma_load_4d_pair(sb + j * 4096, &map_b, full, n0 + 32 * j, k0, i0, i1);
            }
          } else {
            tma_load_4d_pair(sb, &map_b, full, k0, n0, i0, i1);
          }
          ++issued;
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      if (!ok && rank == 0) {
        // Aborting: the loads already issued (by either CTA) complete on these barriers; give them time to land.
        long long first = issued > STAGES ? issued - STAGES : 0;
        for (long long i = first; i < issued; ++i) {
          const long long t0 = clock64();
          while (!mbar_try_wait(bar_full + 8 * (int)(i % STAGES), (uint32_t)((i / STAGES) & 1)) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) ------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = make_idesc_pair(TN, A_MN, B_MN);
      const uint32_t peer_empty = map_to_cta(bar_empty, 1), peer_tfull = map_to_cta(bar_tfull, 1);
      const uint32_t own_empty = map_to_cta(bar_empty, 0), own_tfull = map_to_cta(bar_tfull, 0);
      int s = 0; uint32_t ph = 0;
      int acc = 0; uint32_t aph = 0;
      bool ok = true, any_issued = false;
      for (int unit = first_unit; ok && unit < p.num_tiles; unit += unit_step) {
        int batch, tm, tn, ks;
        tile_coords(p, unit, batch, tm, tn, ks);
        int kb_lo, kb_hi;
        k_range(p, tm, ks, num_kb, kb_lo, kb_hi);
        if (!mbar_wait_cluster(bar_tempty + 8 * acc, aph ^ 1u, abort_flag, p.status)) { ok = false; break; }   // both CTAs drained it
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * TN);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!wait_x(bar_full + 8 * s, ph)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_base + s * PAIR_STAGE_BYTES;
          const uint32_t sb = sa + HALF * BK * 4;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint32_t a_off = A_MN ? kk * 1024 : kk * 32;
            const uint32_t b_off = B_MN ? kk * 1024 : kk * 32;
            const uint64_t ad = make_smem_desc(sa + a_off, A_MN ? 4096 : 16, A_MN ? 512 : 1024, A_MN ? 1 : 2);
            const uint64_t bd = make_smem_desc(sb + b_off, B_MN ? 4096 : 16, B_MN ? 512 : 1024, B_MN ? 1 : 2);
            tc_mma_tf32_pair(d_tmem, ad, bd, idesc, (kb != kb_lo || kk != 0) ? 1u : 0u);
          }
          any_issued = true;
          tc_commit_pair(own_empty + 8 * s);          // both CTAs may refill the stage once these MMAs have read it
          tc_commit_pair(peer_empty + 8 * s);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (!ok) break;
        tc_commit_pair(own_tfull + 8 * acc);          // both halves of the accumulator are complete
        tc_commit_pair(peer_tfull + 8 * acc);
        if (++acc == 2) { acc = 0; aph ^= 1u; }
      }
      if (!ok && any_issued) {
        tc_commit_pair(map_to_cta(bar_drain, 0));
        const long long t0 = clock64();
        while (!mbar_try_wait(bar_drain, 0) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
      }
    }
  } else {
    // ------------------------------ epilogue (eight warps per CTA, its own 128 rows) ------------------------------
    const int q = warp & 3;
    const int eset = (warp - 2) >> 2;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    uint8_t* epi_bytes = epi_scratch + (warp - 2) * EPI_WARP_BYTES;
    const uint32_t epi_u32 = smem_u32(epi_bytes);
    int acc = 0; uint32_t aph = 0;
    const uint32_t my_aux_bar = bar_aux + 8 * (uint32_t)(warp - 2);
    uint32_t aux_ph = 0;
    // Last-wave split (see gt_gemm_umma_kernel): the K shares of a last-wave tile ADD into C, so unless the call is
    // C += ..., pair i zeroes the i-th such tile first, each CTA its own 128 rows, and publishes flag 2 i + rank.
    if (p.tail_split > 1 && p.tail_zero && warp == 2) {
      const int n_tail = (p.num_tiles - p.tail_first) / p.tail_split;
      if (first_unit < n_tail) {
        int batch, tm, tn, ks;
        tile_coords(p, p.tail_first + first_unit * p.tail_split, batch, tm, tn, ks);
#pragma unroll
        for (int g = 0; g < 8; ++g) *reinterpret_cast<float4*>(epi_bytes + lane * 128 + (g << 4)) = make_float4(0.f, 0.f, 0.f, 0.f);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          const int i0 = batch % p.batch0, i1 = batch / p.batch0;
          const int r_base = tm * TM + (int)rank * HALF;
          for (int r = 0; r < HALF / 32; ++r)
            for (int c = 0; c < TN / 32; ++c)
              if (tn * TN + c * 32 < p.N && r_base + r * 32 < p.M)
                tma_store_4d(&map_c, epi_u32, tn * TN + c * 32, r_base + r * 32, i0, i1, false);
          tma_store_wait_all();
          asm volatile("fence.proxy.async;" ::: "memory");
          __threadfence();
          atomicExch(p.tail_flags + 2 * first_unit + (int)rank, p.tail_epoch);
        }
        __syncwarp();
      }
    }
    for (int unit = first_unit; unit < p.num_tiles; unit += unit_step) {
      int batch, tm, tn, ks;
      tile_coords(p, unit, batch, tm, tn, ks);
      const int i0 = batch % p.batch0, i1 = batch / p.batch0;
      const int row0 = tm * TM + (int)rank * HALF + q * 32;
      const int row = row0 + lane;
      const int n0 = tn * TN;
      const long long batch_off = (long long)i0 * p.sC0 + (long long)i1 * p.sC1;
      const long long row_off = batch_off + (long long)row * p.ldc;
      const bool row_ok = row < p.M;
      const float* unit_bias = p.bias ? p.bias + (long long)batch * p.bias_stride : nullptr;
      // a K share (split-K, or the split of a last-wave tile) adds its partial sum into C; bias / residual go in with share 0
      const bool tail_unit = p.tail_split > 1 && ks >= 0;
      const bool share = p.ksplit > 1 || tail_unit;
      // the gelu' factor multiplies the whole sum, so every share applies it
      const int unit_epi = (share && ks > 0 && p.epilogue != GT_EPI_GELU_GRAD) ? (int)GT_EPI_NONE : p.epilogue;
      const bool unit_add = p.accumulate != 0 || share;
      if (tail_unit && p.tail_zero) {
        // this CTA's half of the tile must have been zeroed before the share adds into it (bounded wait; normally long true)
        bool gave_up = false;
        if (lane == 0) {
          const volatile int* flag = p.tail_flags + 2 * ((unit - p.tail_first) / p.tail_split) + (int)rank;
          const long long t0 = clock64();
          while (*flag != p.tail_epoch) {
            if (*abort_flag) { gave_up = true; break; }
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) { *abort_flag = 1; atomicExch(p.status, GT_ERR_TIMEOUT); gave_up = true; break; }
          }
          __threadfence();
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        gave_up = __shfl_sync(0xffffffffu, gave_up ? 1 : 0, 0) != 0;
        if (gave_up) break;
      }
      if (!wait_x(bar_tfull + 8 * acc, aph)) break;
      tc_fence_after();
      // The epilogues that READ aux (residual, stored pre-activation): a TMA load brings the warp's 32 x 32 block of aux
      // into its staging tile while the accumulator columns come out of tensor memory; the lanes then read aux from the
      // tile and write the result over it.  (Read with one global load per lane and row piece, 32 lines per
      // instruction, these warps stalled on the loads four times as long as they issued.)
      const bool aux_staged = unit_epi == GT_EPI_BIAS_ADD || unit_epi == GT_EPI_GELU_GRAD;
      bool lost = false;
      if (row0 < p.M) {                       // warp-uniform: a 32-row block wholly below M has nothing to write
#pragma unroll 1
        for (int c = eset; c < TN / 32; c += 2) {
          const int nb = n0 + c * 32;
          if (nb >= p.N) break;
          if (aux_staged) {
            __syncwarp();                     // every lane is done with the tile's previous contents
            if (lane == 0) {
              tma_store_wait_read<0>();       // and so is the store that was reading them
              mbar_expect_tx(my_aux_bar, EPI_WARP_BYTES);
              tma_load_4d(epi_u32, &map_aux, my_aux_bar, nb, row0, i0, i1);
            }
          }
          float v[32];
          tc_ld32(lane_base + (uint32_t)(acc * TN + c * 32), v);
          tc_wait_ld();
          if (aux_staged) {
            if (!mbar_wait(my_aux_bar, aux_ph, abort_flag, p.status)) { lost = true; break; }
            aux_ph ^= 1u;
          }
          epilogue_chunk_tma(p, unit_bias, &map_c, v, lane, row0, nb, i0, i1, row_off, row_ok, epi_bytes, epi_u32, unit_epi, unit_add, aux_staged);
        }
      }
      if (__any_sync(0xffffffffu, lost)) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_tempty + 8 * acc);      // this warp is done with the accumulator
      if (++acc == 2) { acc = 0; aph ^= 1u; }
    }
    if (lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncwarp();                          // the cluster barrier is a warp-wide instruction: lanes that skipped a role loop rejoin here
  cluster_sync_all();                    // nobody leaves while the peer may still signal or read this CTA
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---- operand splitting for 3xTF32 ---------------------------------------------------------
// hi keeps the 19 bits a tf32 operand carries (sign, exponent, 10 mantissa bits), lo = x - hi
// is exact in fp32.  Rows of `cols` elements with pitch `ld` are packed at pitch `cols_pad`.
__global__ void gt_split_tf32_kernel(const float* __restrict__ x, float* __restrict__ hi, float* __restrict__ lo,
                                     long long rows, int cols, long long ld, int cols_pad,
                                     int batch0, long long s0, long long s1, long long slice_out) {
  const long long per_slice = rows * cols_pad;
  const int b = blockIdx.y;
  const float* src = x + (long long)(b % batch0) * s0 + (long long)(b / batch0) * s1;
  float* h = hi + (long long)b * slice_out;
  float* l = lo + (long long)b * slice_out;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < per_slice; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / cols_pad;
    const int c = (int)(i - r * cols_pad);
    float v = c < cols ? src[r * ld + c] : 0.0f;
    const float vh = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
    h[i] = vh;
    l[i] = v - vh;
  }
}

// ---- split-K reduction --------------------------------------------------------------------------
// C (+)= epilogue(alpha * sum_s partial[s] (+ bias)), partial planes packed (batch, M, N).  The sum
// runs in plane order, so the result does not depend on which CTA finished first.
__global__ void __launch_bounds__(256) gt_splitk_reduce_kernel(const float* __restrict__ ws, int ksplit, long long plane,
                                                               float* C, const float* __restrict__ bias, float* aux,
                                                               int M, int N, int batch0, long long ldc, long long sC0, long long sC1,
                                                               float alpha, int epilogue, int accumulate, long long total, int vec) {
  const bool has_bias = epilogue >= GT_EPI_BIAS && epilogue <= GT_EPI_BIAS_GELU;
  if (vec) {
    // N, ldc and the batch strides are multiples of 4 and every base is 16-byte aligned: four columns at a time
    const long long total4 = total >> 2;
    for (long long i4 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i4 < total4; i4 += (long long)gridDim.x * blockDim.x) {
      const long long i = i4 << 2;
      const int n = (int)(i % N);
      const long long t = i / N;
      const int m = (int)(t % M);
      const int b = (int)(t / M);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s2 = 0; s2 < ksplit; ++s2) {
        const float4 w = *reinterpret_cast<const float4*>(ws + (long long)s2 * plane + i);
        acc.x += w.x; acc.y += w.y; acc.z += w.z; acc.w += w.w;
      }
      float4 x = make_float4(alpha * acc.x, alpha * acc.y, alpha * acc.z, alpha * acc.w);
      if (has_bias) { const float4 bb = *reinterpret_cast<const float4*>(bias + n); x.x += bb.x; x.y += bb.y; x.z += bb.z; x.w += bb.w; }
      const long long off = (long long)(b % batch0) * sC0 + (long long)(b / batch0) * sC1 + (long long)m * ldc + n;
      if (aux) *reinterpret_cast<float4*>(aux + off) = x;
      if (epilogue == GT_EPI_BIAS_RELU) { x.x = fmaxf(x.x, 0.f); x.y = fmaxf(x.y, 0.f); x.z = fmaxf(x.z, 0.f); x.w = fmaxf(x.w, 0.f); }
      else if (epilogue == GT_EPI_BIAS_GELU) { x.x = gt_gelu_tanh(x.x); x.y = gt_gelu_tanh(x.y); x.z = gt_gelu_tanh(x.z); x.w = gt_gelu_tanh(x.w); }
      float4* dst = reinterpret_cast<float4*>(C + off);
      if (accumulate) { const float4 o = *dst; x.x += o.x; x.y += o.y; x.z += o.z; x.w += o.w; }
      *dst = x;
    }
    return;
  }
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int n = (int)(i % N);
    const long long t = i / N;
    const int m = (int)(t % M);
    const int b = (int)(t / M);
    float acc = 0.0f;
    for (int s2 = 0; s2 < ksplit; ++s2) acc += ws[(long long)s2 * plane + i];
    float x = alpha * acc;
    if (has_bias) x += bias[n];
    const long long off = (long long)(b % batch0) * sC0 + (long long)(b / batch0) * sC1 + (long long)m * ldc + n;
    if (aux) aux[off] = x;
    if (epilogue == GT_EPI_BIAS_RELU) x = fmaxf(x, 0.0f);
    else if (epilogue == GT_EPI_BIAS_GELU) x = gt_gelu_tanh(x);
    C[off] = accumulate ? C[off] + x : x;
  }
}

// ---- host side ------------------------------------------------------------------------------

template <int BN, bool A_MN, bool B_MN, bool X3, bool A_GEN>
int launch_cfg(gt_ctx* ctx, const CUtensorMap maps[5], const UmmaParams& p, int grid, cudaStream_t stream) {
  using C = Cfg<BN, X3>;
  auto kern = gt_gemm_umma_kernel<BN, A_MN, B_MN, X3, A_GEN>;
  GT_SMEM_OPT_IN(ctx, kern, C::SMEM_BYTES);
  GT_CUDA_OK(ctx, gt_launch_overlapped(kern, dim3(grid), dim3(A_GEN ? NUM_THREADS_AGEN : NUM_THREADS), C::SMEM_BYTES, stream,
                                       maps[0], maps[1], maps[2], maps[3], maps[4], p));
  ctx->launches += 1;
  return GT_OK;
}

template <int BN, bool X3, bool A_GEN>
int launch_layout(gt_ctx* ctx, int layout, const CUtensorMap maps[5], const UmmaParams& p, int grid, cudaStream_t stream) {
  switch (layout) {
    case GT_LAYOUT_NN: return launch_cfg<BN, false, true, X3, A_GEN>(ctx, maps, p, grid, stream);
    case GT_LAYOUT_NT: return launch_cfg<BN, false, false, X3, A_GEN>(ctx, maps, p, grid, stream);
    case GT_LAYOUT_TN: return launch_cfg<BN, true, true, X3, A_GEN>(ctx, maps, p, grid, stream);
  }
  return GT_ERR_INVALID_ARG;
}

// ---- CTA-pair kernel: launch as clusters of two ---------------------------------------------------
template <class Kern>
void pair_launch_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int clusters, cudaStream_t stream) {
  memset(cfg, 0, sizeof(*cfg));
  cfg->gridDim = dim3(2u * (unsigned)clusters, 1, 1);
  cfg->blockDim = dim3(PAIR_THREADS, 1, 1);
  cfg->dynamicSmemBytes = PAIR_SMEM_BYTES;
  cfg->stream = stream;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = gt_pdl_enabled() ? 1 : 0;
  cfg->attrs = attr;
  cfg->numAttrs = 2;
}

template <class Kern>
int pair_launch(gt_ctx* ctx, Kern kern, int clusters, cudaStream_t stream, const CUtensorMap* maps, const UmmaParams& p) {
  GT_SMEM_OPT_IN(ctx, kern, PAIR_SMEM_BYTES);
  cudaLaunchConfig_t cfg; cudaLaunchAttribute attr[2];
  pair_launch_config<Kern>(&cfg, attr, clusters, stream);
  GT_CUDA_OK(ctx, cudaLaunchKernelEx(&cfg, kern, maps[0], maps[1], maps[4], maps[5], p));
  ctx->launches += 1;
  return GT_OK;
}

// How many two-CTA clusters of the pair kernel the device can hold at once (each CTA takes a whole SM, and a
// cluster needs two free SMs of one GPC, so this can be less than half the SM count).  Asked once per device
// and layout; 0 when the query fails, which turns the pair kernel off.
template <class Kern>
int pair_clusters_query(gt_ctx* ctx, Kern kern) {
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES) != cudaSuccess) { cudaGetLastError(); return 0; }
  cudaLaunchConfig_t cfg; cudaLaunchAttribute attr[2];
  pair_launch_config<Kern>(&cfg, attr, ctx->sm_count / 2, ctx->stream);
  cfg.numAttrs = 1;                      // the occupancy question concerns the cluster shape only
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
  return n;
}

int pair_max_clusters(gt_ctx* ctx, int layout) {
  static int cached[64][3];
  static bool known[64][3];
  if (ctx->device < 0 || ctx->device >= 64 || layout < 0 || layout > 2) return 0;
  if (!known[ctx->device][layout]) {
    int n = 0;
    if (layout == GT_LAYOUT_NN) n = pair_clusters_query(ctx, gt_gemm_pair_kernel<false, true>);
    else if (layout == GT_LAYOUT_NT) n = pair_clusters_query(ctx, gt_gemm_pair_kernel<false, false>);
    else n = pair_clusters_query(ctx, gt_gemm_pair_kernel<true, true>);
    cached[ctx->device][layout] = n;
    known[ctx->device][layout] = true;
  }
  return cached[ctx->device][layout];
}

// When the pair kernel is taken without being forced.  Measured against the one-CTA kernels (tf32, NN / NT):
// (8192, 3072, 768) +7 %, with bias + GELU +8 %, (8192, 2304, 768) +7 %, (8192, 768, 3072) +17 %, (8192, 768, 768) +3 %,
// 4096^3 +2 %; but 2048^3 -26 % (64 tiles leave ten of the 74 pairs idle) and 8192^3 -5 % (a long main loop gains
// nothing from the overlapped epilogue and pays the pair's extra signalling hops).  So: at least one full wave of
// 256 x 256 tiles, and K up to 4096.
bool pair_rule(const gt_gemm_args& g, long long tiles256, int clusters, int sms) {
  (void)sms;
  if (g.M < 256 || g.N < 256 || g.K < 256) return false;
  return tiles256 >= clusters && g.K <= 4096;
}

int pick_bn(const gt_gemm_args& g, int sms, bool x3, bool a_gen) {
  if (g.N <= 64) return 64;
  if (g.N <= 128) return 128;
  // An unaligned A is copied 4 bytes at a time; the widest tile gives those copies the most
  // tensor-core time to hide behind.
  if (a_gen && g.N >= 256) return 256;
  const long long batches = g.batch0 * g.batch1;
  const long long tm = (g.M + BM - 1) / BM;
  // Few output tiles and a long K: take the widest tile, split-K fills the remaining SMs.  Not for a short K
  // (<= 2048) whose 64-wide tiles already occupy half the SMs: there the memset and the reduce-adds of the split
  // cost more than the narrow tile's extra operand traffic (1024^3: 16.5 -> 14.4 us, with bias + GELU 24.7 -> 15.3 us).
  const bool narrow_fills = g.K <= 2048 && tm * ((g.N + 63) / 64) * batches * 2 >= sms;
  if (!x3 && g.epilogue < GT_EPI_CAUSAL && g.K >= 32 * BK && tm * ((g.N + 255) / 256) * batches * 2 <= sms && !narrow_fills) return 256;
  // Cost in "column units per SM": waves x tile width x a per-width efficiency penalty.
  double best = 1e30; int best_bn = 256;
  const int cands[3] = {256, 128, 64};
  const double pen[3] = {1.0, 1.4, 2.0};       // measured on GPT-2 shapes: wider tiles win unless they cost a whole extra wave
  for (int i = 0; i < 3; ++i) {
    if (x3 && cands[i] == 256) continue;            // 3xTF32 at 256 leaves only two stages
    const long long tiles = tm * ((g.N + cands[i] - 1) / cands[i]) * batches;
    const long long waves = (tiles + sms - 1) / sms;
    const double cost = (double)waves * cands[i] * pen[i];
    if (cost < best) { best = cost; best_bn = cands[i]; }
  }
  return best_bn;
}

}  // namespace

bool gt_gemm_umma_eligible(const gt_gemm_args& g) {
  if (g.precision == GT_PREC_FP32) return false;
  if (g.M > 0x7fffffffLL || g.N > 0x7fffffffLL || g.K > 0x7fffffffLL) return false;
  if (g.batch0 * g.batch1 > 0x7fffffffLL) return false;
  // 3xTF32 reads packed, aligned hi/lo copies of both operands, so any alignment will do.
  if (g.precision == GT_PREC_TF32X3) return g.batch0 * g.batch1 <= 65535;
  // tf32: B must be describable by TMA; an unaligned A is copied by the cp.async warps instead.
  return tma_ok(g.B, g.ldb, g.sB0, g.sB1, g.batch0, g.batch1);
}

// fixed_scratch: when non-null, the 3xTF32 operand split goes there (capacity
// fixed_scratch_floats) instead of into the context's growable workspace.
static int umma_launch_impl(gt_ctx* ctx, const gt_gemm_args& g, cudaStream_t stream,
                            float* fixed_scratch, size_t fixed_scratch_floats, bool allow_pair = true) {
  const bool x3 = g.precision == GT_PREC_TF32X3;
  const bool a_mn = g.layout == GT_LAYOUT_TN;
  const bool b_mn = g.layout != GT_LAYOUT_NT;
  const bool a_gen = !x3 && !tma_ok(g.A, g.lda, g.sA0, g.sA1, g.batch0, g.batch1);
  const long long nbatch = g.batch0 * g.batch1;
  // Large tf32 problems (long K, at least one full wave of 256 x 256 tiles) take the big-tile kernel.
  const long long tiles256 = ((g.M + 255) / 256) * ((g.N + 255) / 256) * nbatch;
  static const bool t256_off = getenv("GRADTUITY_GEMM_NO_T256") != nullptr;
  static const long long t256_min_k = getenv("GRADTUITY_GEMM_T256_MIN_K") ? atoll(getenv("GRADTUITY_GEMM_T256_MIN_K")) : 2048;
  static const int t256_min_tiles = getenv("GRADTUITY_GEMM_T256_MIN_TILES") ? atoi(getenv("GRADTUITY_GEMM_T256_MIN_TILES")) : 0;   // tuning aid
  // Measured: with K >= 2048 the big tiles win once they keep 60 % of the SMs busy ((8192, 768, 3072): 96
  // tiles, +5 %; 2048^3: 64 tiles, half the speed); with a shorter K their epilogue, which does not overlap
  // the next main loop, only pays off on outputs of many waves without a second (aux) output (the
  // 8192 x 50272 x 768 logits: +5 %).
  const bool big_enough = t256_min_tiles > 0 ? (g.K >= t256_min_k && tiles256 >= t256_min_tiles)
                                             : ((g.K >= t256_min_k && tiles256 * 5 >= (long long)ctx->sm_count * 3) ||
                                                (g.K >= 512 && tiles256 >= (long long)ctx->sm_count * 8 && !g.aux));
  const int hints = g.flags & (GT_GEMM_A_LOWER | GT_GEMM_AT_LOWER | GT_GEMM_CAUSAL_SKIP_MASKED);
  bool use256 = !t256_off && hints == 0 && !x3 && !a_gen && g.epilogue != GT_EPI_CAUSAL && big_enough &&
                      tma_ok(g.C, g.ldc, g.sC0, g.sC1, g.batch0, g.batch1) && (!g.aux || ((uintptr_t)g.aux & 15) == 0) &&
                      (!g.bias || ((uintptr_t)g.bias & 15) == 0);
  // CTA pairs (256 x 256 tile over two SMs).  GRADTUITY_GEMM_PAIR: 0 = never, 1 = whenever the kernel can serve
  // the problem, unset = the rule below.
  static const int pair_mode = getenv("GRADTUITY_GEMM_PAIR") ? atoi(getenv("GRADTUITY_GEMM_PAIR")) : 2;
  const int pair_clusters = (allow_pair && pair_mode != 0) ? pair_max_clusters(ctx, g.layout) : 0;
  const bool pair_can = pair_clusters > 0 && hints == 0 && !x3 && !a_gen && g.epilogue != GT_EPI_CAUSAL &&
                        getenv("GRADTUITY_GEMM_NO_TMA_STORE") == nullptr &&
                        tma_ok(g.C, g.ldc, g.sC0, g.sC1, g.batch0, g.batch1) && (!g.aux || ((uintptr_t)g.aux & 15) == 0) &&
                        (!g.bias || ((uintptr_t)g.bias & 15) == 0);
  const bool pair = pair_can && (pair_mode == 1 || pair_rule(g, tiles256, pair_clusters, ctx->sm_count));
  if (pair) use256 = true;
  const int workers = pair ? pair_clusters : ctx->sm_count;      // tiles that are worked on at the same time
  static const int force_bn = getenv("GRADTUITY_GEMM_FORCE_BN") ? atoi(getenv("GRADTUITY_GEMM_FORCE_BN")) : 0;   // tuning aid
  int bn = use256 ? 256 : pick_bn(g, ctx->sm_count, x3, a_gen);
  if (!use256 && (force_bn == 64 || force_bn == 128 || (force_bn == 256 && !x3)) && g.N > force_bn / 2) bn = force_bn;
  const int tile_m = use256 ? 256 : BM;

  OperandView va, vb;
  if (a_mn) va = {g.A, g.K, g.M, g.lda, g.sA0, g.sA1}; else va = {g.A, g.M, g.K, g.lda, g.sA0, g.sA1};
  if (b_mn) vb = {g.B, g.K, g.N, g.ldb, g.sB0, g.sB1}; else vb = {g.B, g.N, g.K, g.ldb, g.sB0, g.sB1};

  CUtensorMap maps[6];           // A (hi, lo), B (hi, lo), C, aux
  long long b0 = g.batch0, b1 = g.batch1;
  OperandView va_lo = va, vb_lo = vb;
  if (x3) {
    // Packed hi/lo copies of both operands in the context's scratch block.
    const int a_pad = (int)((va.cols + 3) & ~3LL), b_pad = (int)((vb.cols + 3) & ~3LL);
    const long long a_slice = va.rows * a_pad, b_slice = vb.rows * b_pad;
    const size_t need = (size_t)(2 * (a_slice + b_slice) * nbatch) * sizeof(float);
    float* a_hi;
    if (fixed_scratch) {
      if (need > fixed_scratch_floats * sizeof(float))
        GT_FAIL(ctx, GT_ERR_TOO_LARGE, "operand split needs %zu bytes of scratch, the fixed scratch holds %zu", need,
                fixed_scratch_floats * sizeof(float));
      a_hi = fixed_scratch;
    } else {
      int rc = gt_workspace_reserve(ctx, need, stream);
      if (rc != GT_OK) return rc;
      a_hi = (float*)ctx->workspace;
    }
    float* a_lo = a_hi + a_slice * nbatch;
    float* b_hi = a_lo + a_slice * nbatch;
    float* b_lo = b_hi + b_slice * nbatch;
    const int threads = 256;
    auto blocks_for = [&](long long n) { long long b = (n + threads - 1) / threads; return (unsigned)(b > 4096 ? 4096 : (b < 1 ? 1 : b)); };
    if (nbatch > 65535) GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "3xTF32 batched GEMM supports at most 65535 slices, got %lld", nbatch);
    gt_split_tf32_kernel<<<dim3(blocks_for(a_slice), (unsigned)nbatch), threads, 0, stream>>>(
        va.ptr, a_hi, a_lo, va.rows, (int)va.cols, va.ld, a_pad, (int)g.batch0, va.s0, va.s1, a_slice);
    gt_split_tf32_kernel<<<dim3(blocks_for(b_slice), (unsigned)nbatch), threads, 0, stream>>>(
        vb.ptr, b_hi, b_lo, vb.rows, (int)vb.cols, vb.ld, b_pad, (int)g.batch0, vb.s0, vb.s1, b_slice);
    GT_CUDA_OK(ctx, cudaGetLastError());
    ctx->launches += 2;
    va = {a_hi, va.rows, va.cols, a_pad, a_slice, a_slice * g.batch0};
    va_lo = va; va_lo.ptr = a_lo;
    vb = {b_hi, vb.rows, vb.cols, b_pad, b_slice, b_slice * g.batch0};
    vb_lo = vb; vb_lo.ptr = b_lo;
  }

  // rows of one TMA box: a whole tile side, or the half one CTA of a pair loads
  const int a_side = pair ? 128 : tile_m, b_side = pair ? 128 : bn;
  const int a_box_c = 32, a_box_r = a_mn ? 32 : a_side;
  const int b_box_c = 32, b_box_r = b_mn ? 32 : b_side;
  int rc;
  static const bool onebox_off = getenv("GRADTUITY_GEMM_NO_ONEBOX") != nullptr;
  // one-box form for MN-major operands whose MN extent is a multiple of 32 (else a box would run past a row's end)
  bool a_one = !onebox_off && a_mn && !a_gen && (va.cols % 32 == 0);
  bool b_one = !onebox_off && b_mn && (vb.cols % 32 == 0);
  if (a_one) a_one = encode_map_mn5(ctx, &maps[0], va, a_side / 32, b0, b1) && (!x3 || encode_map_mn5(ctx, &maps[2], va_lo, a_side / 32, b0, b1));
  if (b_one) b_one = encode_map_mn5(ctx, &maps[1], vb, b_side / 32, b0, b1) && (!x3 || encode_map_mn5(ctx, &maps[3], vb_lo, b_side / 32, b0, b1));
  if (!b_one && (rc = encode_map(ctx, &maps[1], vb, b_box_c, b_box_r, b0, b1, b_mn)) != GT_OK) return rc;
  if (a_gen) maps[0] = maps[1];               // unused by the kernel in this mode
  else if (!a_one && (rc = encode_map(ctx, &maps[0], va, a_box_c, a_box_r, b0, b1, a_mn)) != GT_OK) return rc;
  if (x3) {
    if (!a_one && (rc = encode_map(ctx, &maps[2], va_lo, a_box_c, a_box_r, b0, b1, a_mn)) != GT_OK) return rc;
    if (!b_one && (rc = encode_map(ctx, &maps[3], vb_lo, b_box_c, b_box_r, b0, b1, b_mn)) != GT_OK) return rc;
  } else {
    maps[2] = maps[0];
    maps[3] = maps[1];
  }

  UmmaParams p;
  p.A = g.A; p.lda = g.lda; p.sA0 = g.sA0; p.sA1 = g.sA1;
  p.C = g.C; p.bias = g.bias; p.aux = g.aux; p.colsum = g.colsum;
  p.bias_stride = (g.flags & GT_GEMM_BIAS_PER_BATCH) ? g.N : 0;
  p.ldc = g.ldc; p.sC0 = g.sC0; p.sC1 = g.sC1;
  p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K;
  p.batch0 = (int)g.batch0;
  p.tiles_m = (int)((g.M + tile_m - 1) / tile_m);
  p.tiles_n = (int)((g.N + bn - 1) / bn);
  const long long tiles = (long long)p.tiles_m * p.tiles_n * nbatch;
  if (tiles > 0x7fffffffLL) GT_FAIL(ctx, GT_ERR_INVALID_ARG, "gemm: %lld tiles out of range", tiles);
  p.group_m = use256 ? 8 : 16;
  // Split-K: when the output has far fewer tiles than the GPU has SMs and K is long (the dW
  // GEMMs: 768 x 768 output, K = 8192 -> 18 tiles), several CTAs share a tile's K range.  Two ways
  // to combine the partial sums:
  //  * direct: every CTA adds its partial into C with the TMA reduce-add of the epilogue (C is
  //    zeroed first unless the call is C += ...).  No workspace, no second kernel; the order of
  //    the fp32 additions, and so the last bits of C, can differ from run to run.
  //  * ordered: partials go to the workspace and a second kernel adds them in a fixed order.
  //    Taken with GRADTUITY_GEMM_DETERMINISTIC=1, with a bias / activation epilogue, or when C
  //    cannot be described to TMA.
  const int num_kb = (int)((g.K + BK - 1) / BK);
  int ksplit = 1;
  if (!x3 && g.epilogue < GT_EPI_CAUSAL && hints == 0 && tiles * 2 <= workers && num_kb >= 32) {
    ksplit = (int)(workers / tiles);
    if (ksplit > num_kb / 8) ksplit = num_kb / 8;
    if (ksplit > 32) ksplit = 32;
    if (ksplit < 1) ksplit = 1;
  }
  // Big tiles that do not fill the SMs (96 tiles of 256 x 256 for the (8192, 768, K) products): the tiles are cut
  // along K so that about two waves of shares exist; the shares add into C with the TMA reduce-add (C zeroed
  // first unless the call is C += ...), bias / residual with share 0.
  static const bool deterministic256 = getenv("GRADTUITY_GEMM_DETERMINISTIC") != nullptr;
  bool split256 = false;
  if (use256 && !deterministic256 && tiles < workers && nbatch == 1 && g.ldc == g.N &&
      (g.epilogue == GT_EPI_NONE || g.epilogue == GT_EPI_BIAS || g.epilogue == GT_EPI_BIAS_ADD) &&
      (g.epilogue == GT_EPI_BIAS_ADD || !g.aux) && getenv("GRADTUITY_GEMM_NO_TMA_STORE") == nullptr) {
    int want = (int)((2LL * workers) / tiles);
    if (want > num_kb / 16) want = num_kb / 16;
    if (want > 8) want = 8;
    if (want >= 2) { ksplit = want; split256 = true; }
  }
  p.kb_per = (num_kb + ksplit - 1) / ksplit;
  ksplit = (num_kb + p.kb_per - 1) / p.kb_per;
  p.ksplit = ksplit;
  p.ks_stride = 0;
  p.num_tiles = (int)(tiles * ksplit);
  p.epilogue = g.epilogue; p.accumulate = g.accumulate;
  p.alpha = g.alpha;
  p.flags = g.flags;
  if (pair && getenv("GRADTUITY_GEMM_PAIR_CTA_WAIT") != nullptr) p.flags |= (1 << 30);
  p.a_onebox = a_one ? 1 : 0;
  p.b_onebox = b_one ? 1 : 0;
  p.tail_first = 0; p.tail_split = 1; p.tail_kb_per = num_kb;
  p.tail_zero = 0; p.tail_epoch = 0; p.tail_flags = nullptr;
  p.status = ctx->d_status;
  p.sched = nullptr; p.sched_reset = nullptr;
  bool vec = (((uintptr_t)g.C & 15) == 0) && (g.ldc % 4 == 0) && (g.sC0 % 4 == 0) && (g.sC1 % 4 == 0);
  if (g.aux) vec = vec && (((uintptr_t)g.aux & 15) == 0);
  if (g.bias) vec = vec && (((uintptr_t)g.bias & 15) == 0);
  p.vec_ok = vec ? 1 : 0;
  const long long plane = nbatch * g.M * g.N;
  float* ws = nullptr;
  static const bool deterministic = getenv("GRADTUITY_GEMM_DETERMINISTIC") != nullptr;
  static const bool c_tma_off = getenv("GRADTUITY_GEMM_NO_TMA_STORE") != nullptr;
  const bool c_dense = g.ldc == g.N && (g.batch0 == 1 || g.sC0 == g.M * g.N) && (g.batch1 == 1 || g.sC1 == g.M * g.N * g.batch0);
  const bool splitk_direct = split256 || (ksplit > 1 && !deterministic && !c_tma_off && g.epilogue == GT_EPI_NONE && !g.aux &&
                                          tma_ok(g.C, g.ldc, g.sC0, g.sC1, g.batch0, g.batch1) && (g.accumulate || c_dense));
  // Batch entries that share one C (batch stride 0, "C += sum over the batch") rely on the atomic TMA
  // reduce-add of the epilogue; a per-batch bias is applied by the tensor-core kernel's epilogue only.
  const bool c_shared = nbatch > 1 && ((g.batch0 > 1 && g.sC0 == 0) || (g.batch1 > 1 && g.sC1 == 0));
  if (c_shared && (!g.accumulate || c_tma_off || !tma_ok(g.C, g.ldc, g.sC0, g.sC1, g.batch0, g.batch1) || (ksplit > 1 && !splitk_direct) ||
                   g.epilogue != GT_EPI_NONE || g.aux))
    GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "gemm_batched: batch entries sharing one C need accumulate = 1, no epilogue and a 16-byte aligned C");
  if ((g.flags & GT_GEMM_BIAS_PER_BATCH) && ksplit > 1 && !splitk_direct)
    GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "gemm_batched: a per-batch bias is not available on this split-K path");
  // the pair kernel writes C through TMA only: an ordered (workspace) split-K goes to the one-CTA kernels
  if (pair && ksplit > 1 && !splitk_direct) return umma_launch_impl(ctx, g, stream, fixed_scratch, fixed_scratch_floats, false);
  if (splitk_direct) {
    if (!g.accumulate) GT_CUDA_OK(ctx, cudaMemsetAsync(g.C, 0, (size_t)plane * sizeof(float), stream));
    p.accumulate = 1;
  } else if (ksplit > 1) {
    int rc2 = gt_workspace_reserve(ctx, (size_t)(8192 + plane * ksplit) * sizeof(float), stream);
    if (rc2 != GT_OK) return rc2;
    ws = (float*)ctx->workspace + 8192;           // the first 8192 floats belong to the reductions
    p.C = ws; p.bias = nullptr; p.aux = nullptr;
    p.ldc = g.N; p.sC0 = g.M * g.N; p.sC1 = g.M * g.N * g.batch0;
    p.ks_stride = plane;
    p.epilogue = GT_EPI_NONE; p.accumulate = 0; p.alpha = 1.0f;
    p.vec_ok = (g.N % 4 == 0) ? 1 : 0;
  }
  // C through TMA (store, or reduce-add for C += ...) when its rows can be described; split-K partials
  // and unaligned outputs keep the direct / coalesced stores.
  p.c_tma = (!c_tma_off && (ksplit == 1 || splitk_direct) && tma_ok(g.C, g.ldc, g.sC0, g.sC1, g.batch0, g.batch1) &&
             (!g.aux || ((uintptr_t)g.aux & 15) == 0) && (!g.bias || ((uintptr_t)g.bias & 15) == 0)) ? 1 : 0;   // the TMA epilogue uses float4 on aux and bias
  if (!p.c_tma && (g.epilogue == GT_EPI_BIAS_ADD || g.epilogue == GT_EPI_GELU_GRAD))
    GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "gemm: the aux-reading epilogues need a C that TMA can describe (16-byte aligned, ldc a multiple of 4)");
  // the column sums are taken from the staged output tiles: every element of the result must pass through one exactly once
  if (g.colsum && (g.epilogue != GT_EPI_GELU_GRAD || nbatch != 1 || ksplit != 1 || g.accumulate))
    GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "gemm: column sums come with the gelu' epilogue of a single, non-accumulating product only");
  if (p.c_tma) {
    OperandView vc = {g.C, g.M, g.N, g.ldc, g.sC0, g.sC1};
    if ((rc = encode_map(ctx, &maps[4], vc, 32, 32, b0, b1, false, /*plain_f32=*/true)) != GT_OK) return rc;
  } else {
    maps[4] = maps[1];
  }
  // the CTA-pair kernel loads the aux its epilogue READS (residual, pre-activation) by TMA, block by block like C
  if (pair && p.c_tma && (g.epilogue == GT_EPI_BIAS_ADD || g.epilogue == GT_EPI_GELU_GRAD)) {
    OperandView vx = {g.aux, g.M, g.N, g.ldc, g.sC0, g.sC1};
    if ((rc = encode_map(ctx, &maps[5], vx, 32, 32, b0, b1, false, /*plain_f32=*/true)) != GT_OK) return rc;
  } else {
    maps[5] = maps[4];
  }
  // Last partial wave.  A persistent CTA per SM walks the tiles round-robin, so T tiles on P SMs take
  // ceil(T / P) rounds even when the last round has few tiles (the 768-wide projections of GPT-2: 192
  // tiles on 148 SMs = a second round that is 30 % full).  When that round is at most half full its tiles
  // are cut along K into `s` shares taken by different CTAs, which add their partial sums into C with the
  // epilogue's TMA reduce-add (unless the call is C += ..., the kernel zeroes C under those tiles at its
  // start and the shares wait for that; see the epilogue warps).
  static const bool tail_off = getenv("GRADTUITY_GEMM_NO_TAIL_SPLIT") != nullptr;
  // Epilogues that survive a cut along K: none, bias and residual add (applied by share 0 only) and the gelu' factor (a
  // product with the whole sum: every share applies it); an aux OUTPUT (stored pre-activation) does not.
  const bool tail_epi_ok = g.epilogue == GT_EPI_NONE || g.epilogue == GT_EPI_BIAS || g.epilogue == GT_EPI_BIAS_ADD ||
                           g.epilogue == GT_EPI_GELU_GRAD;
  const bool aux_is_input = g.epilogue == GT_EPI_BIAS_ADD || g.epilogue == GT_EPI_GELU_GRAD;
  if (!tail_off && !deterministic && (!use256 || pair) && !x3 && !a_gen && ksplit == 1 && p.c_tma && nbatch == 1 && hints == 0 &&
      (!g.aux || aux_is_input) && tail_epi_ok && num_kb >= 16 && tiles > workers) {
    const int P = workers;                       // a pair counts once and uses two flags per tile
    const int tail = (int)(tiles % P);
    if (tail > 0 && tail * 2 <= P && tail * (pair ? 2 : 1) <= 240) {
      int sp = P / tail;
      if (sp > num_kb / 4) sp = num_kb / 4;
      if (sp > 8) sp = 8;
      if (sp >= 2) {
        const int kb_per = (num_kb + sp - 1) / sp;
        sp = (num_kb + kb_per - 1) / kb_per;
        p.tail_first = (int)(tiles - tail);
        p.tail_split = sp;
        p.tail_kb_per = kb_per;
        p.num_tiles = p.tail_first + tail * sp;
        p.tail_zero = g.accumulate ? 0 : 1;
        p.tail_epoch = ++ctx->tail_epoch;
        p.tail_flags = ctx->d_status + 16;
        // the flags are shared by every launch of this context: one on another stream waits for the previous user
        if ((rc = gt_scratch_acquire(ctx, stream)) != GT_OK) return rc;
      }
    }
  }
  const int grid = (int)(p.num_tiles < ctx->sm_count ? p.num_tiles : ctx->sm_count);
  // Optional dynamic scheduling (GRADTUITY_GEMM_DYNAMIC_SCHED=1): with more units than CTAs, the CTAs draw their later
  // units from a counter instead of taking every grid-th one, so a CTA whose SM is still held by another kernel
  // when the launch starts (an all-reduce on the communication stream) takes less work instead of making the launch
  // wait for its fixed share.  Measured on the data-parallel GPT-2 step (2 GPUs): 21.0 ms against 20.9 ms with the
  // fixed assignment, and alone on a GPU 0-6 % slower per GEMM (the atomics; the last-wave split no longer meets the
  // wave it planned for), so the fixed assignment stays the default.
  static const bool dynamic_sched = getenv("GRADTUITY_GEMM_DYNAMIC_SCHED") != nullptr && atoi(getenv("GRADTUITY_GEMM_DYNAMIC_SCHED")) != 0;
  if (dynamic_sched && !pair && p.num_tiles > grid && ctx->d_sched) {
    if ((rc = gt_scratch_acquire(ctx, stream)) != GT_OK) return rc;      // the counter ring serves one stream at a time
    const int slot = (int)(ctx->sched_seq++ % GT_SCHED_RING);
    p.sched = ctx->d_sched + slot;
    p.sched_reset = ctx->d_sched + (slot + GT_SCHED_RING / 2) % GT_SCHED_RING;
  }
  static const bool trace = getenv("GRADTUITY_GEMM_TRACE") != nullptr;     // one line per launch on stderr
  if (trace)
    fprintf(stderr, "gt_gemm: layout %d M %lld N %lld K %lld batch %lld epi %d acc %d | tile %dx%d x3 %d a_gen %d ksplit %d direct %d tail_split %d (from tile %d) units %d grid %d c_tma %d onebox %d%d\n",
            g.layout, (long long)g.M, (long long)g.N, (long long)g.K, nbatch, g.epilogue, g.accumulate, tile_m, bn, (int)x3, (int)a_gen,
            ksplit, (int)splitk_direct, p.tail_split, p.tail_first, p.num_tiles, grid, p.c_tma, p.a_onebox, p.b_onebox);

  if (pair) {
    const int clusters = p.num_tiles < pair_clusters ? p.num_tiles : pair_clusters;
    if (trace) fprintf(stderr, "gt_gemm:   CTA pairs: %d clusters of 2 (at most %d fit)\n", clusters, pair_clusters);
    switch (g.layout) {
      case GT_LAYOUT_NN: return pair_launch(ctx, gt_gemm_pair_kernel<false, true>, clusters, stream, maps, p);
      case GT_LAYOUT_NT: return pair_launch(ctx, gt_gemm_pair_kernel<false, false>, clusters, stream, maps, p);
      default: return pair_launch(ctx, gt_gemm_pair_kernel<true, true>, clusters, stream, maps, p);
    }
  }
  if (use256) {
    auto launch256 = [&](auto kern, int idx) -> int {      // generic lambda: one instantiation (and one static) per kernel
      (void)idx;
      GT_SMEM_OPT_IN(ctx, kern, T256_SMEM_BYTES);
      GT_CUDA_OK(ctx, gt_launch_overlapped(kern, dim3(grid), dim3(T256_THREADS), T256_SMEM_BYTES, stream, maps[0], maps[1], maps[4], p));
      ctx->launches += 1;
      return GT_OK;
    };
    switch (g.layout) {
      case GT_LAYOUT_NN: return launch256(gt_gemm_umma256_kernel<false, true>, 0);
      case GT_LAYOUT_NT: return launch256(gt_gemm_umma256_kernel<false, false>, 1);
      default: return launch256(gt_gemm_umma256_kernel<true, true>, 2);
    }
  }
#define GT_DISPATCH(BN_)                                                                         \
  rc = x3 ? launch_layout<BN_, true, false>(ctx, g.layout, maps, p, grid, stream)               \
          : (a_gen ? launch_layout<BN_, false, true>(ctx, g.layout, maps, p, grid, stream)      \
                   : launch_layout<BN_, false, false>(ctx, g.layout, maps, p, grid, stream))
  if (bn == 256 && !x3)
    rc = a_gen ? launch_layout<256, false, true>(ctx, g.layout, maps, p, grid, stream)
               : launch_layout<256, false, false>(ctx, g.layout, maps, p, grid, stream);
  else if (bn == 128) { GT_DISPATCH(128); }
  else { GT_DISPATCH(64); }
#undef GT_DISPATCH
  if (rc != GT_OK || ksplit == 1 || splitk_direct) return rc;
  const int rvec = (vec && g.N % 4 == 0) ? 1 : 0;      // `vec`: C, aux and bias 16-byte aligned with strides that are multiples of 4
  long long blocks = ((rvec ? plane / 4 : plane) + 255) / 256;
  if (blocks > (long long)ctx->sm_count * 8) blocks = (long long)ctx->sm_count * 8;
  gt_splitk_reduce_kernel<<<(unsigned)blocks, 256, 0, stream>>>(ws, ksplit, plane, g.C, g.bias, g.aux, (int)g.M, (int)g.N,
                                                                (int)g.batch0, g.ldc, g.sC0, g.sC1, g.alpha, g.epilogue,
                                                                g.accumulate, plane, rvec);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}

int gt_gemm_umma_launch(gt_ctx* ctx, const gt_gemm_args& g, cudaStream_t stream) {
  return umma_launch_impl(ctx, g, stream, nullptr, 0);
}

// ---- 3xTF32 GEMM that allocates nothing ---------------------------------------------------------
//
// Some callers must not trigger a device allocation while they run: a serving loop that has
// handed all free device memory to its own pool, so that a cudaMalloc from inside a library
// fails or evicts; a step that is timed to the microsecond and cannot absorb the device-wide
// synchronisation cudaMalloc / cudaFree may imply; code that runs while another component
// holds the allocator lock.  gt_gemm in 3xTF32 mode does allocate, the first time it meets
// a new largest problem: the hi/lo copies of A and B live in a workspace that grows on demand.
// This entry point runs the same kernels with those copies in a fixed array inside the
// library's own image instead, so no cudaMalloc, cudaFree, cudaMallocAsync or allocating library
// routine is reached, and problems that do not fit are refused rather than served slowly.
//
// The array is a file-scope __device__ object: every GPU that loads the library keeps
// GT_NOALLOC_SCRATCH_BYTES of it until the process exits.  In host code its name is only a
// handle; the device address is looked up with cudaGetSymbolAddress once per device, with
// that device current, on the first call made for that device (the caller's current device is
// restored).  That first call should therefore come before any stream capture begins and outside
// any timed region: with lazy module loading it can be the moment the array is placed on the GPU,
// so "allocates nothing" is a property of every call after the first one on a device.  All calls share the array and it keeps
// the previous call's contents: the split kernels overwrite every element the GEMM reads
// (padding columns included), so nothing needs clearing, but two calls whose kernels overlap
// on the GPU (different streams without an ordering between them) race on it.
constexpr size_t GT_NOALLOC_SCRATCH_FLOATS = (size_t)8 << 20;            // 32 MiB
static __device__ __align__(256) float gt_noalloc_scratch[GT_NOALLOC_SCRATCH_FLOATS];
static float* g_noalloc_scratch_ptr[64] = {nullptr};

extern "C" int gt_gemm_3xtf32_noalloc(gt_ctx* ctx, int layout, int64_t M, int64_t N, int64_t K,
                                      const float* A, int64_t lda, const float* B, int64_t ldb,
                                      float* C, int64_t ldc, const float* bias, float alpha,
                                      int accumulate, int epilogue, void* stream) {
  if (!ctx) return GT_ERR_INVALID_ARG;
  gt_gemm_args g;
  g.layout = layout; g.epilogue = epilogue; g.precision = GT_PREC_TF32X3; g.accumulate = accumulate; g.flags = 0;
  g.M = M; g.N = N; g.K = K;
  g.A = A; g.lda = lda; g.sA0 = 0; g.sA1 = 0;
  g.B = B; g.ldb = ldb; g.sB0 = 0; g.sB1 = 0;
  g.C = C; g.ldc = ldc; g.sC0 = 0; g.sC1 = 0;
  g.batch0 = 1; g.batch1 = 1;
  g.bias = bias; g.aux = nullptr; g.alpha = alpha;
  int rc = gt_gemm_validate(ctx, g);
  if (rc != GT_OK) return rc;
  if (ctx->device < 0 || ctx->device >= 64) GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "device index %d out of range", ctx->device);
  // Refuse oversize problems before touching the device.
  const int64_t a_rows = layout == GT_LAYOUT_TN ? K : M, a_cols = layout == GT_LAYOUT_TN ? M : K;
  const int64_t b_rows = layout == GT_LAYOUT_NT ? N : K, b_cols = layout == GT_LAYOUT_NT ? K : N;
  const double need = 2.0 * ((double)a_rows * (double)((a_cols + 3) & ~3LL) + (double)b_rows * (double)((b_cols + 3) & ~3LL));
  if (need > (double)GT_NOALLOC_SCRATCH_FLOATS)
    GT_FAIL(ctx, GT_ERR_TOO_LARGE,
            "gt_gemm_3xtf32_noalloc: A and B need %.0f floats of split scratch, the built-in array holds %zu (32 MiB); use gt_gemm",
            need, GT_NOALLOC_SCRATCH_FLOATS);
  if (!g_noalloc_scratch_ptr[ctx->device]) {
    // One-time set-up for this device: the symbol's address is per device and is looked up with that device
    // current; the caller's current device is put back afterwards.  (With CUDA's lazy module loading this
    // look-up may also be the moment the driver places the array on the GPU.)
    int previous = -1;
    GT_CUDA_OK(ctx, cudaGetDevice(&previous));
    if (previous != ctx->device) GT_CUDA_OK(ctx, cudaSetDevice(ctx->device));
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&p, gt_noalloc_scratch);
    if (previous != ctx->device) cudaSetDevice(previous);
    GT_CUDA_OK(ctx, e);
    if (!p) GT_FAIL(ctx, GT_ERR_CUDA, "gt_gemm_3xtf32_noalloc: the scratch array has no device address on device %d", ctx->device);
    g_noalloc_scratch_ptr[ctx->device] = p;
  }
  cudaStream_t s = stream ? (cudaStream_t)stream : ctx->stream;
  rc = umma_launch_impl(ctx, g, s, g_noalloc_scratch_ptr[ctx->device], GT_NOALLOC_SCRATCH_FLOATS);
  const int rel = gt_scratch_release(ctx, s);
  return rc != GT_OK ? rc : rel;
}

// ---- bounded-wait self test ---------------------------------------------------------------------
// One CTA waits on an mbarrier that nothing will ever arrive on, with the same polling loop the GEMM
// kernels use but a caller-chosen cycle limit.  The wait must give up, record GT_ERR_TIMEOUT in the
// status word and return, leaving the context usable: the host-visible half of "no wait in this
// library can hang the GPU".
__global__ void gt_selftest_wait_kernel(int* status, long long limit_cycles) {
  __shared__ __align__(8) uint64_t bar;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    const long long t0 = clock64();
    bool done = false;
    while (!done) {
      if (mbar_try_wait(b, 0)) done = true;
      else if (clock64() - t0 > limit_cycles) { atomicExch(status, GT_ERR_TIMEOUT); done = true; }
    }
  }
}

extern "C" int gt_selftest_bounded_wait(gt_ctx* ctx, int64_t limit_cycles) {
  if (!ctx || limit_cycles <= 0 || limit_cycles > 4000000000LL) return GT_ERR_INVALID_ARG;
  gt_selftest_wait_kernel<<<1, 32, 0, ctx->stream>>>(ctx->d_status, limit_cycles);
  GT_CUDA_OK(ctx, cudaGetLastError());
  ctx->launches += 1;
  return GT_OK;
}
