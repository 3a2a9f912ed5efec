// Fused causal attention for sm_100a, head dimension 64, tf32 multiply / fp32 accumulate.
//
// The reference builds attention from separate launches (gradtuity/nn.py:511-554: three
// transposes, bmm, scale_inplace, softmax_with_causal_mask, bmm) and keeps S, P, dP and dS, each
// (B, H, T, T), in memory.  The kernels here compute the same quantities tile by tile:
//
//   gt_attn_fwd_online_kernel  O = softmax(scale * Q K^T + causal mask) V in one pass over the key tiles, row
//                              statistics (log-sum-exp) saved: the form the training step uses.
//   gt_attn_fwd_kernel         the same in two passes, with P written out on request.
//   gt_attn_bwd_dq_kernel      per 128-query block: recomputes P from Q, K and the saved statistics,
//                              dP = dO V^T, dS = scale * P (dP - delta), dQ = dS K; also writes
//                              delta = rowsum(dO * O).
//   gt_attn_bwd_dkv_kernel     per 128-key block: the transposed products S^T = K Q^T, dP^T = V dO^T,
//                              dV = P^T dO, dK = dS^T Q.
//
// Common structure: a persistent CTA per SM takes (batch, head, block) items from a table built on the host
// (heaviest first, each to the CTA with the least work so far); warp 0 issues TMA loads into a ring of 32 KB
// slots, lane 0 of warp 1 issues tcgen05.mma, warps 2-17 (lane = row of the 128-row tile, four warps per
// tensor-memory lane quarter, one per 32-column chunk of a tile) do the softmax arithmetic.  In the three
// training kernels that arithmetic stays in tensor memory: P (or dS, P^T, dS^T) is written over the accumulator
// it was computed from, rounded to tf32, and the next product reads it from there as its A operand; the products
// are issued in an order that lets the tensor core's in-order execution stand in for "buffer free" barriers (see
// each kernel).  Q, K, V, dO are read in place from the (B, T, H * 64) projection outputs; TMA rounds them to tf32.
//
// Every wait is bounded (see mbar_wait): on a time-out the CTA raises the context's status word,
// all roles leave their loops and tensor memory is released.

#include <stdlib.h>

#include <array>
#include <map>
#include <mutex>
#include <queue>
#include <vector>

#include "gt_internal.h"
#include "gt_umma_common.cuh"

namespace {

constexpr int AT_D = 64;                        // head dimension
constexpr int AT_TILE = 128;                    // queries per item, keys per tile
constexpr int AT_THREADS = 576;                 // producer warp, MMA warp, 16 softmax warps (four per tensor-memory lane quarter)
// 576 threads = 18 warps, which the register file allots as 20: 96 registers per thread is the most a launch accepts
// (112 is refused: "too many resources requested"), hence the few spilled values in the softmax loops.
constexpr int AT_SOFTMAX_WARPS = 16;
constexpr int AT_SLOT_BYTES = 32768;            // one 128 x 64 fp32 operand tile
constexpr int AT_SLOTS = 4;
constexpr int AT_P_BYTES = 65536;               // 128 x 128 fp32 tile of P / dS (four 128-byte-swizzle atoms of 32 columns)
constexpr int AT_SMEM_BYTES = AT_SLOT_BYTES /*Q*/ + AT_SLOTS * AT_SLOT_BYTES + AT_P_BYTES + 1024 + 512;
constexpr float AT_LOG2E = 1.4426950408889634f;
constexpr float AT_LN2 = 0.6931471805599453f;

struct AttnParams {
  int S, H, B;
  int nblk;                 // S / 128
  int num_items;            // B * H * nblk
  float scale_log2;         // scale * log2(e)
  float scale;
  int write_p;
  int online;               // forward: single pass with a running maximum (no P output)
  float* lse;               // (B, H, S) log-sum-exp of the scaled scores, natural log
  float* delta;             // (B, H, S) rowsum(dO * O) (backward)
  const float* o; const float* d_o;   // (B, S, H * 64), read directly by the dQ kernel for delta
  int* status;
  float* dbq; float* dbk; float* dbv;   // backward, optional: (H * 64) vectors that receive the column sums of dQ, dK, dV (the projections' bias gradients)
  const int* sched;         // [gridDim.x][sched_stride] item numbers of every CTA in the order it takes them, -1 after the last
  int sched_stride;
};

// The k-th item of this CTA, or -1.
__device__ __forceinline__ int sched_item(const AttnParams& p, int k) { return __ldg(p.sched + (long long)blockIdx.x * p.sched_stride + k); }

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Round to tf32 (nearest, ties away from zero: what cvt.rna.tf32.f32 gives) with two integer instructions; the
// conversion instruction shares the 16-lane unit with ex2, which these kernels already keep busy.
__device__ __forceinline__ float to_tf32(float x) { return __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xffffe000u); }

// Item order: the query blocks with the most key tiles first, so the tail of the persistent loop is light.
__device__ __forceinline__ void item_coords(const AttnParams& p, int item, int& i, int& h, int& b) {
  const int bh = p.B * p.H;
  i = p.nblk - 1 - item / bh;
  const int r = item % bh;
  h = r % p.H;
  b = r / p.H;
}

// The products below are issued by ONE thread that shares its scheduler with four busy softmax warps, so every
// instruction in front of a tcgen05.mma delays it: the descriptors of a k-step are the first k-step's plus a
// compile-time constant (the start-address field counts 16-byte units and never carries out of its 14 bits here).

// S = A(128 x 64, K-major) * B(128 x 64, K-major)^T into 128 columns of tensor memory: 8 k-steps.
__device__ __forceinline__ void mma_qk(uint32_t d_tmem, uint32_t sa, uint32_t sb) {
  constexpr uint32_t idesc = make_idesc(128, false, false);
  const uint64_t da = make_smem_desc(sa, 16, 1024, 2), db = make_smem_desc(sb, 16, 1024, 2);
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint64_t off = (uint64_t)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
    tc_mma_tf32(d_tmem, da + off, db + off, idesc, kk ? 1u : 0u);
  }
}
// D(128 x 64) (+)= A(128 x 128, K-major: four atoms of 32 columns) * B(128 x 64 stored (k, n), n contiguous:
// MN-major, two 32-wide chunks 16 KB apart): 16 k-steps.
__device__ __forceinline__ void mma_pv(uint32_t d_tmem, uint32_t sa, uint32_t sb, bool keep) {
  constexpr uint32_t idesc = make_idesc(64, false, true);
  const uint64_t da = make_smem_desc(sa, 16, 1024, 2), db = make_smem_desc(sb, 16384, 512, 1);
#pragma unroll
  for (int kk = 0; kk < 16; ++kk) {
    const uint64_t a_off = (uint64_t)(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
    tc_mma_tf32(d_tmem, da + a_off, db + (uint64_t)(kk * 64), idesc, (keep || kk) ? 1u : 0u);
  }
}

// D(128 x 64) (+)= A(128 x 128 in tensor memory, columns a_tmem .. a_tmem + 127) * B(128 x 64, MN-major as in mma_pv).
__device__ __forceinline__ void mma_pv_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t sb, bool keep) {
  constexpr uint32_t idesc = make_idesc(64, false, true);
  const uint64_t db = make_smem_desc(sb, 16384, 512, 1);
#pragma unroll
  for (int kk = 0; kk < 16; ++kk)
    tc_mma_tf32_ts(d_tmem, a_tmem + (uint32_t)kk * 8u, db + (uint64_t)(kk * 64), idesc, (keep || kk) ? 1u : 0u);
}

// Position in a ring of `n` shared-memory slots: the slot, the parity of the round, the number of steps so far.
// (Kept as three counters: slot = count % n and parity = (count / n) & 1 would be a 64-bit division per access, on a
// thread whose every instruction delays the next tcgen05.mma or TMA load.)
struct RingPos {
  int slot, n;
  uint32_t phase;
  long long count;
  __device__ __forceinline__ explicit RingPos(int n_) : slot(0), n(n_), phase(0), count(0) {}
  __device__ __forceinline__ RingPos& operator++() {
    ++count;
    if (++slot == n) { slot = 0; phase ^= 1u; }
    return *this;
  }
};

// v[0..31] are 32 columns of this lane's row; returns in lane l the sum of column l over the warp's 32 rows (a butterfly
// of 31 shuffles: each stage keeps half of the columns and adds the partner's half).  v is used up.
__device__ __forceinline__ float warp_column_sums(float* v, int lane) {
#pragma unroll
  for (int s = 16; s >= 1; s >>= 1) {
    const bool upper = (lane & s) != 0;
#pragma unroll
    for (int i = 0; i < s; ++i) {
      const float send = upper ? v[i] : v[i + s];
      const float keep = upper ? v[i + s] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
    }
  }
  return v[0];
}

// One 128 x 64 operand tile (two boxes of 32 columns) into L2.
__device__ __forceinline__ void prefetch_tile(const CUtensorMap* map, int row0, int h, int b) {
  tma_prefetch_l2_4d(map, 0, row0, h, b);
  tma_prefetch_l2_4d(map, 32, row0, h, b);
}

struct AttnSmem {
  uint32_t q, ring, ptile;                // shared-memory addresses (u32)
  uint8_t* ptile_ptr;
  uint32_t bar_q_full, bar_q_empty, bar_kv_full, bar_kv_empty, bar_s_full, bar_s_empty, bar_p_full, bar_p_empty, bar_o_full, bar_o_empty;
  uint32_t bar_group, bar_drain;          // rendezvous of the eight softmax warps; completion of MMAs in flight on an abort
  uint32_t* tmem_slot;
  volatile int* abort_flag;
  float* stats;                           // [4][128][2]: per column-chunk partial (max, sum) of each row
};

__device__ __forceinline__ AttnSmem carve(uint8_t* smem_raw) {
  AttnSmem s;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  s.q = base;
  s.ring = base + AT_SLOT_BYTES;
  s.ptile = s.ring + AT_SLOTS * AT_SLOT_BYTES;
  s.ptile_ptr = aligned + AT_SLOT_BYTES + AT_SLOTS * AT_SLOT_BYTES;
  uint8_t* ctrl = s.ptile_ptr + AT_P_BYTES;
  const uint32_t bars = smem_u32(ctrl);
  s.bar_q_full = bars;            s.bar_q_empty = bars + 8;
  s.bar_kv_full = bars + 16;      s.bar_kv_empty = bars + 16 + 8 * AT_SLOTS;
  s.bar_s_full = bars + 16 + 16 * AT_SLOTS;   s.bar_s_empty = s.bar_s_full + 16;
  s.bar_p_full = s.bar_s_empty + 16;          s.bar_p_empty = s.bar_p_full + 8;
  s.bar_o_full = s.bar_p_empty + 8;           s.bar_o_empty = s.bar_o_full + 8;
  s.bar_group = s.bar_o_empty + 8;            s.bar_drain = s.bar_group + 8;
  s.tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 192);
  s.abort_flag = reinterpret_cast<volatile int*>(ctrl + 196);
  // the statistics exchange reuses the first 4 KB of the P tile between the two passes (the tile is idle then)
  s.stats = reinterpret_cast<float*>(s.ptile_ptr);
  return s;
}

// ---- forward ---------------------------------------------------------------------------------
// Two passes over the key tiles of a query block.  Pass 1 computes S tile by tile and keeps only each
// row's running maximum and sum; pass 2 computes S again (K = 64: the products are cheap, the K
// tiles come from L2), turns it into the final probabilities exp(s - max) / sum, writes them to
// shared memory (and, on request, from there to P with a TMA store), and accumulates O += P V in
// tensor memory, so O never needs rescaling.
__global__ void __launch_bounds__(AT_THREADS, 1)
gt_attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_p,
                   const __grid_constant__ CUtensorMap map_o, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const AttnSmem sm = carve(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(sm.bar_q_full, 1); mbar_init(sm.bar_q_empty, 1);
    for (int i = 0; i < AT_SLOTS; ++i) { mbar_init(sm.bar_kv_full + 8 * i, 1); mbar_init(sm.bar_kv_empty + 8 * i, 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(sm.bar_s_full + 8 * i, 1); mbar_init(sm.bar_s_empty + 8 * i, AT_SOFTMAX_WARPS); }
    mbar_init(sm.bar_p_full, AT_SOFTMAX_WARPS); mbar_init(sm.bar_p_empty, 1);
    mbar_init(sm.bar_o_full, 1); mbar_init(sm.bar_o_empty, 8);
    mbar_init(sm.bar_group, AT_SOFTMAX_WARPS); mbar_init(sm.bar_drain, 1);
    *sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(sm.tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  gt_let_next_kernel_start();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *sm.tmem_slot;
  gt_wait_for_previous_kernel();         // set-up above overlaps the previous kernel's tail; global memory from here on
  const uint32_t tmem_o = tmem_base + 256u;
  constexpr int nslots = AT_SLOTS;

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      long long ring_it = 0; int q_it = 0;
      bool ok = true;
      auto load_slot = [&](const CUtensorMap* map, bool is_v, int row0, int h, int b) -> bool {
        const int slot = (int)(ring_it % nslots);
        const uint32_t par = (uint32_t)((ring_it / nslots) & 1);
        if (!mbar_wait(sm.bar_kv_empty + 8 * slot, par ^ 1u, sm.abort_flag, p.status)) return false;
        const uint32_t dst = sm.ring + slot * AT_SLOT_BYTES, full = sm.bar_kv_full + 8 * slot;
        mbar_expect_tx(full, AT_SLOT_BYTES);
        if (is_v) {
          tma_load_5d(dst, map, full, 0, row0, 0, h, b);
        } else {
          tma_load_4d(dst, map, full, 0, row0, h, b);
          tma_load_4d(dst + 16384, map, full, 32, row0, h, b);
        }
        ++ring_it;
        return true;
      };
      for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_) {
        int i, h, b;
        item_coords(p, item, i, h, b);
        if (!mbar_wait(sm.bar_q_empty, (uint32_t)(q_it & 1) ^ 1u, sm.abort_flag, p.status)) { ok = false; break; }
        mbar_expect_tx(sm.bar_q_full, AT_SLOT_BYTES);
        tma_load_4d(sm.q, &map_q, sm.bar_q_full, 0, i * AT_TILE, h, b);
        tma_load_4d(sm.q + 16384, &map_q, sm.bar_q_full, 32, i * AT_TILE, h, b);
        ++q_it;
        if (const int next = sched_item(p, k_ + 1); next >= 0) {     // the next item's Q towards L2
          int i2, h2, b2;
          item_coords(p, next, i2, h2, b2);
          prefetch_tile(&map_q, i2 * AT_TILE, h2, b2);
        }
        for (int j = 0; ok && j <= i; ++j) ok = load_slot(&map_k, false, j * AT_TILE, h, b);           // pass 1
        // pass 2, in the order the MMA lane consumes them: K0, K1, V0, K2, V1, ..., Ki, V(i-1), Vi
        if (ok) ok = load_slot(&map_k, false, 0, h, b);
        for (int j = 0; ok && j <= i; ++j) {
          if (j + 1 <= i) ok = load_slot(&map_k, false, (j + 1) * AT_TILE, h, b);
          if (ok) ok = load_slot(&map_v, true, j * AT_TILE, h, b);
        }
      }
      if (!ok) {     // aborting: let the loads already issued land before shared memory is released
        const long long first = ring_it > nslots ? ring_it - nslots : 0;
        for (long long r = first; r < ring_it; ++r) {
          const long long t0 = clock64();
          while (!mbar_try_wait(sm.bar_kv_full + 8 * (int)(r % nslots), (uint32_t)((r / nslots) & 1)) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      long long ring_it = 0; int q_it = 0, s_it = 0, p_it = 0, o_it = 0;
      bool ok = true;
      auto issue_s = [&]() -> bool {            // next ring slot holds a K tile
        const int slot = (int)(ring_it % nslots);
        const int sb = s_it & 1;
        if (!mbar_wait(sm.bar_kv_full + 8 * slot, (uint32_t)((ring_it / nslots) & 1), sm.abort_flag, p.status)) return false;
        if (!mbar_wait(sm.bar_s_empty + 8 * sb, (uint32_t)((s_it >> 1) & 1) ^ 1u, sm.abort_flag, p.status)) return false;
        tc_fence_after();
        mma_qk(tmem_base + (uint32_t)(sb * 128), sm.q, sm.ring + slot * AT_SLOT_BYTES);
        tc_commit(sm.bar_kv_empty + 8 * slot);
        tc_commit(sm.bar_s_full + 8 * sb);
        ++ring_it; ++s_it;
        return true;
      };
      for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_) {
        int i, h, b;
        item_coords(p, item, i, h, b);
        if (!mbar_wait(sm.bar_q_full, (uint32_t)(q_it & 1), sm.abort_flag, p.status)) { ok = false; break; }
        ++q_it;
        for (int j = 0; ok && j <= i; ++j) ok = issue_s();          // pass 1
        if (ok) ok = issue_s();                                     // pass 2: S_0
        for (int j = 0; ok && j <= i; ++j) {
          if (j + 1 <= i) { ok = issue_s(); if (!ok) break; }
          if (j == i) tc_commit(sm.bar_q_empty);                    // every product with this Q has been issued
          const int slot = (int)(ring_it % nslots);
          if (!mbar_wait(sm.bar_kv_full + 8 * slot, (uint32_t)((ring_it / nslots) & 1), sm.abort_flag, p.status)) { ok = false; break; }
          if (!mbar_wait(sm.bar_p_full, (uint32_t)(p_it & 1), sm.abort_flag, p.status)) { ok = false; break; }
          if (j == 0 && !mbar_wait(sm.bar_o_empty, (uint32_t)(o_it & 1) ^ 1u, sm.abort_flag, p.status)) { ok = false; break; }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          tc_fence_after();
          mma_pv(tmem_o, sm.ptile, sm.ring + slot * AT_SLOT_BYTES, j != 0);
          tc_commit(sm.bar_kv_empty + 8 * slot);
          tc_commit(sm.bar_p_empty);
          if (j == i) { tc_commit(sm.bar_o_full); ++o_it; }
          ++ring_it; ++p_it;
        }
      }
      if (!ok) {                    // aborting: wait (bounded) for the products in flight before tensor memory is released
        tc_commit(sm.bar_drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(sm.bar_drain, 0) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
      }
    }
  } else {
    // ------------------------------ softmax warps ------------------------------
    const int q = warp & 3;                    // tensor-memory lane quarter this warp may read
    const int eset = (warp - 2) >> 2;          // the 32-column chunk of every tile this warp owns (0..3)
    const int r_local = q * 32 + lane;         // row inside the 128-row tile
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    uint8_t* const my_row = sm.ptile_ptr + eset * 16384 + r_local * 128;     // this thread's 128 bytes of the P tile
    const uint32_t my_sub = sm.ptile + (uint32_t)(eset * 16384 + q * 4096);  // this warp's 32 x 32 part of it
    const int sw = r_local & 7;
    int s_it = 0, p_it = 0, o_it = 0, g_it = 0;
    bool ok = true;
    // Rendezvous of the softmax warps on an mbarrier, so that it is bounded like every other wait.
    auto group_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.bar_group);
      const bool r = mbar_wait(sm.bar_group, (uint32_t)(g_it & 1), sm.abort_flag, p.status);
      ++g_it;
      return r;
    };
    for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_) {
      int i, h, b;
      item_coords(p, item, i, h, b);
      const int row = i * AT_TILE + r_local;   // query index
      // ---- pass 1: running maximum and sum over this warp's column chunk of every key tile
      float m = -INFINITY, l = 0.0f;
      for (int j = 0; j <= i; ++j) {
        const int sb = s_it & 1;
        if (!mbar_wait(sm.bar_s_full + 8 * sb, (uint32_t)((s_it >> 1) & 1), sm.abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        const int col0 = j * AT_TILE + eset * 32;
        if (j < i || col0 <= i * AT_TILE + q * 32 + 31) {        // else: wholly right of the diagonal for this warp's rows
          float v[32];
          tc_ld32(lane_base + (uint32_t)(sb * 128 + eset * 32), v);
          tc_wait_ld();
          float mx = -INFINITY;
          if (j < i) {
#pragma unroll
            for (int t = 0; t < 32; ++t) mx = fmaxf(mx, v[t]);
          } else {
            const int nvalid = row - col0 + 1;                   // columns <= row
#pragma unroll
            for (int t = 0; t < 32; ++t) { if (t >= nvalid) v[t] = -INFINITY; mx = fmaxf(mx, v[t]); }
          }
          if (mx > -INFINITY) {
            const float m_new = fmaxf(m, mx * p.scale_log2);
            float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
            for (int t = 0; t < 32; t += 2) {
              a0 += ex2(fmaf(v[t], p.scale_log2, -m_new));
              a1 += ex2(fmaf(v[t + 1], p.scale_log2, -m_new));
            }
            l = l * ex2(m - m_new) + (a0 + a1);
            m = m_new;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.bar_s_empty + 8 * sb);
        ++s_it;
      }
      if (!ok) break;
      // ---- combine the four column chunks of every row (the P tile is idle: its last reader, the
      // previous item's final PV product and this warp's own stores from it, is waited for first)
      if (!mbar_wait(sm.bar_p_empty, (uint32_t)(p_it & 1) ^ 1u, sm.abort_flag, p.status)) { ok = false; break; }
      if (lane == 0) tma_store_wait_read<0>();
      if (!group_sync()) { ok = false; break; }
      sm.stats[(eset * 128 + r_local) * 2] = m;
      sm.stats[(eset * 128 + r_local) * 2 + 1] = l;
      if (!group_sync()) { ok = false; break; }
      float M = -INFINITY;
#pragma unroll
      for (int e = 0; e < 4; ++e) M = fmaxf(M, sm.stats[(e * 128 + r_local) * 2]);
      float L = 0.0f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float me = sm.stats[(e * 128 + r_local) * 2];
        if (me > -INFINITY) L += sm.stats[(e * 128 + r_local) * 2 + 1] * ex2(me - M);
      }
      const float ML = M + log2f(L);           // p = 2^(s * scale * log2 e - ML)
      if (p.lse && eset == 0) p.lse[((long long)b * p.H + h) * p.S + row] = ML * AT_LN2;
      if (!group_sync()) { ok = false; break; }   // the statistics have been read: the tile may be overwritten
      // ---- pass 2: probabilities -> shared memory (-> P), O += P V
      for (int j = 0; j <= i; ++j) {
        const int sb = s_it & 1;
        if (!mbar_wait(sm.bar_s_full + 8 * sb, (uint32_t)((s_it >> 1) & 1), sm.abort_flag, p.status)) { ok = false; break; }
        if (j > 0) {
          if (!mbar_wait(sm.bar_p_empty, (uint32_t)(p_it & 1) ^ 1u, sm.abort_flag, p.status)) { ok = false; break; }
          if (lane == 0) tma_store_wait_read<0>();
          __syncwarp();
        }
        tc_fence_after();
        const int col0 = j * AT_TILE + eset * 32;
        float v[32];
        const bool dead = (j == i) && (eset > q);        // chunk wholly right of the diagonal for this warp's rows
        if (!dead) {
          tc_ld32(lane_base + (uint32_t)(sb * 128 + eset * 32), v);
          tc_wait_ld();
        }
        if (dead) {
#pragma unroll
          for (int g = 0; g < 8; ++g) *reinterpret_cast<float4*>(my_row + ((g ^ sw) << 4)) = make_float4(0.f, 0.f, 0.f, 0.f);
        } else if (j < i) {
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            float4 x;
            x.x = to_tf32(ex2(fmaf(v[4 * g], p.scale_log2, -ML)));
            x.y = to_tf32(ex2(fmaf(v[4 * g + 1], p.scale_log2, -ML)));
            x.z = to_tf32(ex2(fmaf(v[4 * g + 2], p.scale_log2, -ML)));
            x.w = to_tf32(ex2(fmaf(v[4 * g + 3], p.scale_log2, -ML)));
            *reinterpret_cast<float4*>(my_row + ((g ^ sw) << 4)) = x;
          }
        } else {
          const int nvalid = row - col0 + 1;
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            float4 x;
            x.x = (4 * g < nvalid) ? to_tf32(ex2(fmaf(v[4 * g], p.scale_log2, -ML))) : 0.0f;
            x.y = (4 * g + 1 < nvalid) ? to_tf32(ex2(fmaf(v[4 * g + 1], p.scale_log2, -ML))) : 0.0f;
            x.z = (4 * g + 2 < nvalid) ? to_tf32(ex2(fmaf(v[4 * g + 2], p.scale_log2, -ML))) : 0.0f;
            x.w = (4 * g + 3 < nvalid) ? to_tf32(ex2(fmaf(v[4 * g + 3], p.scale_log2, -ML))) : 0.0f;
            *reinterpret_cast<float4*>(my_row + ((g ^ sw) << 4)) = x;
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (p.write_p) tma_store_4d(&map_p, my_sub, col0, i * AT_TILE + q * 32, h, b, false);
          mbar_arrive(sm.bar_p_full);
          mbar_arrive(sm.bar_s_empty + 8 * sb);
        }
        ++s_it; ++p_it;
      }
      if (!ok) break;
      // ---- O: 64 columns = chunks 0 and 1; their owners pass them through their part of the P tile
      if (!mbar_wait(sm.bar_o_full, (uint32_t)(o_it & 1), sm.abort_flag, p.status)) { ok = false; break; }
      ++o_it;
      tc_fence_after();
      if (eset < 2) {
        float v[32];
        tc_ld32(lane_base + 256u + (uint32_t)(eset * 32), v);
        tc_wait_ld();
        tc_fence_before();
        // the final PV product has completed (o_full), so the tensor core no longer reads the tile;
        // this warp's own P store from its part is waited for here
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
#pragma unroll
        for (int g = 0; g < 8; ++g)
          *reinterpret_cast<float4*>(my_row + ((g ^ sw) << 4)) = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          tma_store_4d(&map_o, my_sub, eset * 32, i * AT_TILE + q * 32, h, b, false);
          mbar_arrive(sm.bar_o_empty);
        }
      }
    }
    if (lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---- forward, single pass (no P output) ----------------------------------------------------------------
// The kernel the training step uses.  Tensor memory: S in two buffers (columns 0 and 128) and FOUR 64-column O
// accumulators (256 ... 511), one per 32-key chunk of a tile.  The softmax warp that owns rows r and key chunk e of
// every tile keeps its own running reference maximum and row sum for that chunk, turns S into P = 2^(s - reference)
// in place, and the P V product adds chunk e's part (four of its sixteen k-steps) into accumulator e: no warp ever
// needs another warp's maximum while the tiles stream by.  When a tile's maximum exceeds the reference by more than 8
// (log2 units) the warp rescales its own accumulator once; otherwise the stale reference stays (p <= 2^8).  At the
// end of the item the four (reference, sum) pairs of a row meet in shared memory and the output is the weighted sum
// of the four accumulators.  The MMA thread issues S(j+1), P(j) V(j) per tile and relies on the tensor core's issue
// order: S(j+1) overwrites the buffer whose P(j-1) the earlier P V product read.
constexpr uint32_t FW_S = 0, FW_O = 256;
constexpr int ATF_SLOTS = 5;
constexpr int ATF_STATS_BYTES = 4096;          // [4 chunks][128 rows][reference, sum]
constexpr int ATF_SMEM_BYTES = AT_SLOT_BYTES + ATF_SLOTS * AT_SLOT_BYTES + ATF_STATS_BYTES + 1024 + 512;

struct FwdSmem {
  uint32_t q, ring;
  uint8_t* ring_ptr;
  float* stats;
  uint32_t bar_q_full, bar_q_empty, bar_kv_full, bar_kv_empty, bar_s_full, bar_p_full, bar_pv_done, bar_o_full, bar_o_empty, bar_group, bar_drain;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
};

__device__ __forceinline__ FwdSmem carve_fwd(uint8_t* smem_raw) {
  FwdSmem s;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  s.q = base;
  s.ring = base + AT_SLOT_BYTES;
  s.ring_ptr = aligned + AT_SLOT_BYTES;
  s.stats = reinterpret_cast<float*>(s.ring_ptr + ATF_SLOTS * AT_SLOT_BYTES);
  uint8_t* ctrl = s.ring_ptr + ATF_SLOTS * AT_SLOT_BYTES + ATF_STATS_BYTES;
  const uint32_t bars = smem_u32(ctrl);
  s.bar_q_full = bars;           s.bar_q_empty = bars + 8;
  s.bar_kv_full = bars + 16;     s.bar_kv_empty = bars + 64;       // up to six slots each
  s.bar_s_full = bars + 112;     /* two */  s.bar_p_full = bars + 128;   /* two */
  s.bar_pv_done = bars + 144;    s.bar_o_full = bars + 152;        s.bar_o_empty = bars + 160;
  s.bar_group = bars + 168;      s.bar_drain = bars + 176;
  s.tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 256);
  s.abort_flag = reinterpret_cast<volatile int*>(ctrl + 260);
  return s;
}

// O_e(128 x 64) (+)= P(128 x 128 in tensor memory)[:, 32 e .. 32 e + 31] * V[32 e .. 32 e + 31, :] for the four chunks e.
__device__ __forceinline__ void mma_pv_chunks(uint32_t o_tmem, uint32_t p_tmem, uint32_t sb, bool keep) {
  constexpr uint32_t idesc = make_idesc(64, false, true);
  const uint64_t db = make_smem_desc(sb, 16384, 512, 1);
#pragma unroll
  for (int kk = 0; kk < 16; ++kk)
    tc_mma_tf32_ts(o_tmem + (uint32_t)(kk >> 2) * 64u, p_tmem + (uint32_t)kk * 8u, db + (uint64_t)(kk * 64), idesc, (keep || (kk & 3)) ? 1u : 0u);
}

__global__ void __launch_bounds__(AT_THREADS, 1)
gt_attn_fwd_online_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const FwdSmem sm = carve_fwd(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(sm.bar_q_full, 1); mbar_init(sm.bar_q_empty, 1);
    for (int i = 0; i < ATF_SLOTS; ++i) { mbar_init(sm.bar_kv_full + 8 * i, 1); mbar_init(sm.bar_kv_empty + 8 * i, 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(sm.bar_s_full + 8 * i, 1); mbar_init(sm.bar_p_full + 8 * i, AT_SOFTMAX_WARPS); }
    mbar_init(sm.bar_pv_done, 1);
    mbar_init(sm.bar_o_full, 1); mbar_init(sm.bar_o_empty, AT_SOFTMAX_WARPS);
    mbar_init(sm.bar_group, AT_SOFTMAX_WARPS); mbar_init(sm.bar_drain, 1);
    *sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(sm.tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  gt_let_next_kernel_start();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *sm.tmem_slot;
  gt_wait_for_previous_kernel();         // set-up above overlaps the previous kernel's tail; global memory from here on

  if (warp == 0) {
    // ------------------------------ producer ------------------------------
    if (lane == 0) {
      RingPos ring_it(ATF_SLOTS); int q_it = 0;
      bool ok = true;
      auto load_slot = [&](const CUtensorMap* map, bool is_v, int row0, int h, int b) -> bool {
        const int slot = ring_it.slot;
        const uint32_t par = ring_it.phase;
        if (!mbar_wait(sm.bar_kv_empty + 8 * slot, par ^ 1u, sm.abort_flag, p.status)) return false;
        const uint32_t dst = sm.ring + slot * AT_SLOT_BYTES, full = sm.bar_kv_full + 8 * slot;
        mbar_expect_tx(full, AT_SLOT_BYTES);
        if (is_v) {
          tma_load_5d(dst, map, full, 0, row0, 0, h, b);
        } else {
          tma_load_4d(dst, map, full, 0, row0, h, b);
          tma_load_4d(dst + 16384, map, full, 32, row0, h, b);
        }
        ++ring_it;
        return true;
      };
      for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_) {
        int i, h, b;
        item_coords(p, item, i, h, b);
        // ring order: K0; then per tile K(j+1), V(j).  K0 needs only a free slot and goes out before the wait for Q's tile.
        ok = load_slot(&map_k, false, 0, h, b);
        if (!ok || !mbar_wait(sm.bar_q_empty, (uint32_t)(q_it & 1) ^ 1u, sm.abort_flag, p.status)) { ok = false; break; }
        mbar_expect_tx(sm.bar_q_full, AT_SLOT_BYTES);
        tma_load_4d(sm.q, &map_q, sm.bar_q_full, 0, i * AT_TILE, h, b);
        tma_load_4d(sm.q + 16384, &map_q, sm.bar_q_full, 32, i * AT_TILE, h, b);
        ++q_it;
        if (const int next = sched_item(p, k_ + 1); next >= 0) {     // the next item's Q towards L2
          int i2, h2, b2;
          item_coords(p, next, i2, h2, b2);
          prefetch_tile(&map_q, i2 * AT_TILE, h2, b2);
        }
        for (int j = 0; ok && j <= i; ++j) {
          if (j + 1 <= i) ok = load_slot(&map_k, false, (j + 1) * AT_TILE, h, b);
          if (ok) ok = load_slot(&map_v, true, j * AT_TILE, h, b);
        }
      }
      if (!ok) {     // aborting: let the loads already issued land before shared memory is released
        const long long first = ring_it.count > ATF_SLOTS ? ring_it.count - ATF_SLOTS : 0;
        for (long long r = first; r < ring_it.count; ++r) {
          const long long t0 = clock64();
          while (!mbar_try_wait(sm.bar_kv_full + 8 * (int)(r % ATF_SLOTS), (uint32_t)((r / ATF_SLOTS) & 1)) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      RingPos ring_it(ATF_SLOTS); int q_it = 0, s_it = 0 /* S products issued */, tt = 0 /* P V products issued */, o_it = 0;
      bool ok = true;
      auto issue_s = [&]() -> bool {            // next ring slot holds a K tile; S goes to buffer s_it & 1
        const int slot = ring_it.slot;
        if (!mbar_wait(sm.bar_kv_full + 8 * slot, ring_it.phase, sm.abort_flag, p.status)) return false;
        tc_fence_after();
        mma_qk(tmem_base + FW_S + (uint32_t)((s_it & 1) * 128), sm.q, sm.ring + slot * AT_SLOT_BYTES);
        tc_commit(sm.bar_s_full + 8 * (s_it & 1));            // also tells the first softmax warp that the K slot is free (see there)
        ++ring_it; ++s_it;
        return true;
      };
      for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_) {
        int i, h, b;
        item_coords(p, item, i, h, b);
        if (!mbar_wait(sm.bar_q_full, (uint32_t)(q_it & 1), sm.abort_flag, p.status)) { ok = false; break; }
        ++q_it;
        ok = issue_s();
        for (int j = 0; ok && j <= i; ++j) {
          if (j + 1 <= i) { ok = issue_s(); if (!ok) break; }
          if (j == i) tc_commit(sm.bar_q_empty);                    // every product with this Q has been issued
          const int slot = ring_it.slot;
          if (!mbar_wait(sm.bar_kv_full + 8 * slot, ring_it.phase, sm.abort_flag, p.status)) { ok = false; break; }
          if (!mbar_wait(sm.bar_p_full + 8 * (tt & 1), (uint32_t)((tt >> 1) & 1), sm.abort_flag, p.status)) { ok = false; break; }
          if (j == 0 && !mbar_wait(sm.bar_o_empty, (uint32_t)(o_it & 1) ^ 1u, sm.abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          mma_pv_chunks(tmem_base + FW_O, tmem_base + FW_S + (uint32_t)((tt & 1) * 128), sm.ring + slot * AT_SLOT_BYTES, j != 0);
          tc_commit(sm.bar_pv_done);                                // the V slot is handed back by the first softmax warp
          if (j == i) { tc_commit(sm.bar_o_full); ++o_it; }
          ++ring_it; ++tt;
        }
      }
      if (!ok) {                    // aborting: wait (bounded) for the products in flight before tensor memory is released
        tc_commit(sm.bar_drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(sm.bar_drain, 0) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
      }
    }
  } else {
    // ------------------------------ softmax warps ------------------------------
    const int q = warp & 3;                    // tensor-memory lane quarter this warp may read
    const int eset = (warp - 2) >> 2;          // the 32-key chunk of every tile this warp owns (0..3)
    const int r_local = q * 32 + lane;         // row inside the 128-row tile
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    const uint32_t my_o = lane_base + FW_O + (uint32_t)(eset * 64);      // this warp's accumulator
    const int sw = r_local & 7;
    int tt = 0, o_it = 0, g_it = 0;
    int base_mod = 0;                          // ring slot of the item's first load (2 loads per tile: K0; then K(j+1), V(j))
    bool ok = true;
    auto group_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.bar_group);
      const bool r = mbar_wait(sm.bar_group, (uint32_t)(g_it & 1), sm.abort_flag, p.status);
      ++g_it;
      return r;
    };
    for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_) {
      int i, h, b;
      item_coords(p, item, i, h, b);
      const int row = i * AT_TILE + r_local;
      float m_ref = -INFINITY, l = 0.0f;       // of this thread's chunk of the row
      for (int j = 0; j <= i; ++j) {
        const int sb = tt & 1;
        if (!mbar_wait(sm.bar_s_full + 8 * sb, (uint32_t)((tt >> 1) & 1), sm.abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        if (warp == 2 && lane == 0) {
          // Ring slots go back to the producer from here, not from the MMA thread (whose every instruction delays the
          // next product): S(j) complete means K(j) has been read, and, the tensor core executing in issue order
          // S(j), P(j-1) V(j-1), S(j+1), ..., that the product with V(j-2) has completed too.
          mbar_arrive(sm.bar_kv_empty + 8 * ((base_mod + (j == 0 ? 0 : 2 * j - 1)) % ATF_SLOTS));
          if (j >= 2) mbar_arrive(sm.bar_kv_empty + 8 * ((base_mod + 2 * j - 2) % ATF_SLOTS));
        }
        const int col0 = j * AT_TILE + eset * 32;
        const bool dead = (j == i) && (eset > q);              // chunk wholly right of the diagonal for this warp's rows
        const int nvalid = (j < i) ? 32 : row - col0 + 1;      // keys <= query
        const uint32_t s_col = lane_base + FW_S + (uint32_t)(sb * 128 + eset * 32);
        float v[32];
        float mx = -INFINITY;
        if (!dead) {
          tc_ld32(s_col, v);
          tc_wait_ld();
          if (j < i) {                     // warp-uniform: no masked element left of the diagonal
#pragma unroll
            for (int t = 0; t < 32; ++t) { v[t] *= p.scale_log2; mx = fmaxf(mx, v[t]); }
          } else {
#pragma unroll
            for (int t = 0; t < 32; ++t) { v[t] = (t < nvalid) ? v[t] * p.scale_log2 : -INFINITY; mx = fmaxf(mx, v[t]); }
          }
        }
        float f = 1.0f;
        if (mx > m_ref + 8.0f) { f = ex2(m_ref - mx); m_ref = mx; }
        l *= f;
        if (j > 0 && __any_sync(0xffffffffu, f != 1.0f)) {
          // rescale this warp's accumulator: the previous P V product must have completed (no later one has been issued)
          if (!mbar_wait(sm.bar_pv_done, (uint32_t)(tt & 1) ^ 1u, sm.abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int part = 0; part < 4; ++part) {
            float o[16];
            tc_ld16(my_o + (uint32_t)(part * 16), o);
            tc_wait_ld();
#pragma unroll
            for (int t = 0; t < 16; ++t) o[t] *= f;
            tc_st16(my_o + (uint32_t)(part * 16), o);
            tc_wait_st();
          }
        }
        float acc = 0.0f;
        if (dead || m_ref == -INFINITY) {                      // nothing of this row's chunk is visible (yet)
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = 0.0f;
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) { v[t] = to_tf32(ex2(v[t] - m_ref)); acc += v[t]; }
        }
        l += acc;
        tc_st32(s_col, v);                                     // P over S, in place
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.bar_p_full + 8 * sb);
        ++tt;
      }
      if (!ok) break;
      // ---- the row's four (reference, sum) pairs meet; weights of the four accumulators
      sm.stats[(eset * 128 + r_local) * 2] = m_ref;
      sm.stats[(eset * 128 + r_local) * 2 + 1] = l;
      if (!group_sync()) { ok = false; break; }
      float M = -INFINITY;
#pragma unroll
      for (int e = 0; e < 4; ++e) M = fmaxf(M, sm.stats[(e * 128 + r_local) * 2]);
      float L = 0.0f, w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float me = sm.stats[(e * 128 + r_local) * 2];
        w[e] = (me > -INFINITY) ? ex2(me - M) : 0.0f;
        L += sm.stats[(e * 128 + r_local) * 2 + 1] * w[e];
      }
      const float inv = 1.0f / L;
      if (p.lse && eset == 0) p.lse[((long long)b * p.H + h) * p.S + row] = (M + log2f(L)) * AT_LN2;
      if (!mbar_wait(sm.bar_o_full, (uint32_t)(o_it & 1), sm.abort_flag, p.status)) { ok = false; break; }
      ++o_it;
      tc_fence_after();
      if (warp == 2 && lane == 0 && i >= 1) mbar_arrive(sm.bar_kv_empty + 8 * ((base_mod + 2 * i) % ATF_SLOTS));     // V(i-1); V(i) stages the output
      // this thread's 16 output columns: the weighted sum over the four accumulators
      float out[16];
#pragma unroll
      for (int t = 0; t < 16; ++t) out[t] = 0.0f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float o[16];
        tc_ld16(lane_base + FW_O + (uint32_t)(e * 64 + eset * 16), o);
        tc_wait_ld();
        const float we = w[e] * inv;
#pragma unroll
        for (int t = 0; t < 16; ++t) out[t] = fmaf(we, o[t], out[t]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.bar_o_empty);
      // O leaves through the ring slot of the item's last load (V of the last tile), whose reader has completed
      const int slot_out = (base_mod + 2 * i + 1) % ATF_SLOTS;
      base_mod = (base_mod + 2 * (i + 1)) % ATF_SLOTS;
      {
        uint8_t* const my_row = sm.ring_ptr + slot_out * AT_SLOT_BYTES + (eset >> 1) * 16384 + r_local * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g)
          *reinterpret_cast<float4*>(my_row + ((((eset & 1) * 4 + g) ^ sw) << 4)) = make_float4(out[4 * g], out[4 * g + 1], out[4 * g + 2], out[4 * g + 3]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      if (!group_sync()) { ok = false; break; }                  // both warps of every 32 x 32 box have written it (and the statistics have been read)
      if ((eset & 1) == 0 && lane == 0) {
        const uint32_t my_sub = sm.ring + (uint32_t)(slot_out * AT_SLOT_BYTES + (eset >> 1) * 16384 + q * 4096);
        tma_store_4d(&map_o, my_sub, (eset >> 1) * 32, i * AT_TILE + q * 32, h, b, false);
        tma_store_wait_read<0>();
      }
      if (!group_sync()) { ok = false; break; }                  // every store has read its box: the slot goes back to the producer
      if (warp == 2 && lane == 0) mbar_arrive(sm.bar_kv_empty + 8 * slot_out);
    }
    if (lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// ---- backward ----------------------------------------------------------------------------------
// Both backward kernels hold two operand tiles for the whole item (Q and dO of the query block, or
// K and V of the key block) and stream the other side's tiles through a ring of five 32 KB slots; S, dP
// (or their transposes), P and dS live in tensor memory only.  The B operand of the second products
// (K, dO or Q, stored (rows, 64) with the head dimension contiguous) is MN-major: it is loaded a second
// time with the five-dimensional map that lays it out in 32-wide chunks (a K-major descriptor cannot read
// that layout).  The item's last ring slot(s) stage the outputs for TMA stores.
constexpr int ATB_CTRL_BYTES = 1536;           // barriers, the tensor-memory address, the abort flag, 2 x 128 floats of statistics

struct BwdSmem {
  int nslots;
  uint32_t fix0, fix1, ring, tile;
  uint8_t* tile_ptr;
  uint32_t bar_fix_full, bar_fix_empty, bar_ring_full, bar_ring_empty, bar_sdp_full, bar_sdp_empty;
  uint32_t bar_out_full, bar_out_empty, bar_group, bar_drain;
  uint32_t bar_s_full, bar_dp_full, bar_pa_full, bar_pb_full;      // dK / dV kernel (s_full, pa_full, pb_full: two barriers each)
  uint32_t bar_ds_full, bar_delta_full, bar_delta_empty;           // dQ kernel (two barriers each)
  uint32_t* tmem_slot;
  volatile int* abort_flag;
  float* stats;
};

// Layout: two fixed operand tiles | `nslots` ring slots | a tile of `tile_bytes` (P^T / dS^T, or the output staging) | control.
__device__ __forceinline__ BwdSmem carve_bwd(uint8_t* smem_raw, int nslots, int tile_bytes) {
  BwdSmem s;
  s.nslots = nslots;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* aligned = smem_raw + (base - smem_u32(smem_raw));
  s.fix0 = base;
  s.fix1 = base + AT_SLOT_BYTES;
  s.ring = base + 2 * AT_SLOT_BYTES;
  s.tile = s.ring + nslots * AT_SLOT_BYTES;
  s.tile_ptr = aligned + (2 + nslots) * AT_SLOT_BYTES;
  uint8_t* ctrl = s.tile_ptr + tile_bytes;
  const uint32_t bars = smem_u32(ctrl);
  s.bar_fix_full = bars;        s.bar_fix_empty = bars + 8;
  s.bar_ring_full = bars + 16;  s.bar_ring_empty = bars + 16 + 8 * nslots;       // up to six slots below offset 128
  s.bar_sdp_full = bars + 128;  s.bar_sdp_empty = bars + 136;
  s.bar_out_full = bars + 176;  s.bar_out_empty = bars + 184;
  s.bar_group = bars + 192;     s.bar_drain = bars + 200;
  s.bar_s_full = bars + 208;    /* two */  s.bar_dp_full = bars + 224;
  s.bar_pa_full = bars + 232;   /* two */  s.bar_pb_full = bars + 248;   /* two */
  s.bar_ds_full = bars + 264;   /* two */  s.bar_delta_full = bars + 280;   /* two */  s.bar_delta_empty = bars + 296;   /* two */
  s.tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 384);
  s.abort_flag = reinterpret_cast<volatile int*>(ctrl + 388);
  s.stats = reinterpret_cast<float*>(ctrl + 512);
  return s;
}

__device__ __forceinline__ void bwd_setup(const BwdSmem& sm, int warp, int out_arrivals) {
  if (threadIdx.x == 0) {
    mbar_init(sm.bar_fix_full, 1); mbar_init(sm.bar_fix_empty, 1);
    for (int i = 0; i < sm.nslots; ++i) { mbar_init(sm.bar_ring_full + 8 * i, 1); mbar_init(sm.bar_ring_empty + 8 * i, 1); }
    mbar_init(sm.bar_sdp_full, 1); mbar_init(sm.bar_sdp_empty, AT_SOFTMAX_WARPS);
    mbar_init(sm.bar_out_full, 1); mbar_init(sm.bar_out_empty, out_arrivals);
    mbar_init(sm.bar_group, AT_SOFTMAX_WARPS); mbar_init(sm.bar_drain, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(sm.bar_s_full + 8 * i, 1);
      mbar_init(sm.bar_pa_full + 8 * i, AT_SOFTMAX_WARPS); mbar_init(sm.bar_pb_full + 8 * i, AT_SOFTMAX_WARPS);
      mbar_init(sm.bar_ds_full + 8 * i, AT_SOFTMAX_WARPS);
      mbar_init(sm.bar_delta_full + 8 * i, 2); mbar_init(sm.bar_delta_empty + 8 * i, AT_SOFTMAX_WARPS);
    }
    mbar_init(sm.bar_dp_full, 1);
    *sm.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(sm.tmem_slot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  gt_let_next_kernel_start();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  gt_wait_for_previous_kernel();         // set-up above overlaps the previous kernel's tail; global memory from here on
}

// One ring load: a K-major tile (two boxes of 32 columns) or an MN-major tile (one five-dimensional box).
__device__ __forceinline__ bool bwd_ring_load(const BwdSmem& sm, const AttnParams& p, RingPos& ring_it, const CUtensorMap* map,
                                              bool mn, int row0, int h, int b) {
  const int slot = ring_it.slot;
  const uint32_t par = ring_it.phase;
  if (!mbar_wait(sm.bar_ring_empty + 8 * slot, par ^ 1u, sm.abort_flag, p.status)) return false;
  const uint32_t dst = sm.ring + slot * AT_SLOT_BYTES, full = sm.bar_ring_full + 8 * slot;
  mbar_expect_tx(full, AT_SLOT_BYTES);
  if (mn) {
    tma_load_5d(dst, map, full, 0, row0, 0, h, b);
  } else {
    tma_load_4d(dst, map, full, 0, row0, h, b);
    tma_load_4d(dst + 16384, map, full, 32, row0, h, b);
  }
  ++ring_it;
  return true;
}
__device__ __forceinline__ void bwd_ring_drain(const BwdSmem& sm, const RingPos& ring_it) {
  const long long first = ring_it.count > sm.nslots ? ring_it.count - sm.nslots : 0;
  for (long long r = first; r < ring_it.count; ++r) {
    const long long t0 = clock64();
    while (!mbar_try_wait(sm.bar_ring_full + 8 * (int)(r % sm.nslots), (uint32_t)((r / sm.nslots) & 1)) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
  }
}
__device__ __forceinline__ bool bwd_ring_wait(const BwdSmem& sm, const AttnParams& p, const RingPos& ring_it) {
  return mbar_wait(sm.bar_ring_full + 8 * ring_it.slot, ring_it.phase, sm.abort_flag, p.status);
}

// Item order of the key-block owner: key block 0 sees every query block, so it goes first.
__device__ __forceinline__ void item_coords_kv(const AttnParams& p, int item, int& j, int& h, int& b) {
  const int bh = p.B * p.H;
  j = item / bh;
  const int r = item % bh;
  h = r % p.H;
  b = r / p.H;
}

// dQ for one block of 128 queries; also delta = rowsum(dO * O).
//
// Tensor memory: S (columns 0-127), dP in two buffers (128, 256), dQ (384-447).  The softmax warps turn dP into dS in
// place and the dQ product reads it from there; per key tile j the MMA thread issues
//     S(j+1)   dP(j+1) -> the other buffer   dQ += dS(j) K(j)
// so that the softmax arithmetic of tile j+1 runs beside the dQ product of tile j.  dP(j+1) overwrites the buffer whose
// dS(j-1) the earlier dQ product read (the tensor core executes one thread's products in issue order); S is single
// and waits for the softmax warps to have loaded it.
// Two extra warps run one item ahead and compute delta for the block's 128 queries (two rows per thread), handing it
// over through shared memory, so the softmax warps do not wait for global memory at the start of an item.
constexpr uint32_t DQ_S = 0, DQ_DP = 128, DQ_ACC = 384;
constexpr int ATQ_THREADS = AT_THREADS + 64;
constexpr int ATQ_SLOTS = 5;
constexpr int ATQ_SMEM_BYTES = 2 * AT_SLOT_BYTES + ATQ_SLOTS * AT_SLOT_BYTES + 1024 + ATB_CTRL_BYTES;

__global__ void __launch_bounds__(ATQ_THREADS, 1)
gt_attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                      const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const __grid_constant__ CUtensorMap map_kmn, const __grid_constant__ CUtensorMap map_dq,
                      const AttnParams p, const int accumulate) {
  extern __shared__ uint8_t smem_raw[];
  const BwdSmem sm = carve_bwd(smem_raw, ATQ_SLOTS, 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t bar_delta_full = sm.bar_delta_full, bar_delta_empty = sm.bar_delta_empty;   // "delta ready" (two delta warps), "delta read" (softmax warps)
  bwd_setup(sm, warp, 8);
  const uint32_t tmem_base = *sm.tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      RingPos ring_it(sm.nslots); int f_it = 0;
      bool ok = true;
      for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_) {
        int i, h, b;
        item_coords(p, item, i, h, b);
        // the first ring tiles need only free slots, which the end of the previous item leaves: they go out before the
        // wait for the fixed tiles, which are busy until that item's last S / dP product has completed
        ok = bwd_ring_load(sm, p, ring_it, &map_k, false, 0, h, b) && bwd_ring_load(sm, p, ring_it, &map_v, false, 0, h, b);
        if (!ok || !mbar_wait(sm.bar_fix_empty, (uint32_t)(f_it & 1) ^ 1u, sm.abort_flag, p.status)) { ok = false; break; }
        mbar_expect_tx(sm.bar_fix_full, 2 * AT_SLOT_BYTES);
        tma_load_4d(sm.fix0, &map_q, sm.bar_fix_full, 0, i * AT_TILE, h, b);
        tma_load_4d(sm.fix0 + 16384, &map_q, sm.bar_fix_full, 32, i * AT_TILE, h, b);
        tma_load_4d(sm.fix1, &map_do, sm.bar_fix_full, 0, i * AT_TILE, h, b);
        tma_load_4d(sm.fix1 + 16384, &map_do, sm.bar_fix_full, 32, i * AT_TILE, h, b);
        ++f_it;
        if (const int next = sched_item(p, k_ + 1); next >= 0) {     // the next item's Q and dO: nobody has read them yet, so start them towards L2 now
          int i2, h2, b2;
          item_coords(p, next, i2, h2, b2);
          prefetch_tile(&map_q, i2 * AT_TILE, h2, b2);
          prefetch_tile(&map_do, i2 * AT_TILE, h2, b2);
        }
        // in the order the MMA thread consumes them: K(0), V(0); then per tile K(j+1), V(j+1), K(j) MN-major
        for (int j = 0; ok && j <= i; ++j) {
          if (j + 1 <= i)
            ok = bwd_ring_load(sm, p, ring_it, &map_k, false, (j + 1) * AT_TILE, h, b) &&
                 bwd_ring_load(sm, p, ring_it, &map_v, false, (j + 1) * AT_TILE, h, b);
          if (ok) ok = bwd_ring_load(sm, p, ring_it, &map_kmn, true, j * AT_TILE, h, b);
        }
      }
      if (!ok) bwd_ring_drain(sm, ring_it);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      RingPos ring_it(sm.nslots); int f_it = 0, s_it = 0 /* S / dP pairs issued */, tt = 0 /* dQ products issued */, o_it = 0;
      bool ok = true;
      auto issue_sdp = [&]() -> bool {        // S = Q K^T and dP = dO V^T of the next key tile
        if (!bwd_ring_wait(sm, p, ring_it)) return false;
        // S is single: the softmax warps must have loaded the previous tile's
        if (!mbar_wait(sm.bar_sdp_empty, (uint32_t)(s_it & 1) ^ 1u, sm.abort_flag, p.status)) return false;
        tc_fence_after();
        int slot = ring_it.slot;
        mma_qk(tmem_base + DQ_S, sm.fix0, sm.ring + slot * AT_SLOT_BYTES);
        ++ring_it;
        if (!bwd_ring_wait(sm, p, ring_it)) return false;
        tc_fence_after();
        slot = ring_it.slot;
        mma_qk(tmem_base + DQ_DP + (uint32_t)((s_it & 1) * 128), sm.fix1, sm.ring + slot * AT_SLOT_BYTES);
        ++ring_it;
        tc_commit(sm.bar_sdp_full);                           // the ring slots are handed back by the first softmax warp (see there)
        ++s_it;
        return true;
      };
      for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_) {
        int i, h, b;
        item_coords(p, item, i, h, b);
        if (!mbar_wait(sm.bar_fix_full, (uint32_t)(f_it & 1), sm.abort_flag, p.status)) { ok = false; break; }
        ++f_it;
        ok = issue_sdp();
        for (int j = 0; ok && j <= i; ++j) {
          if (j + 1 <= i) { ok = issue_sdp(); if (!ok) break; }
          if (j == i) tc_commit(sm.bar_fix_empty);          // the item's last product with Q and dO has been issued
          if (!bwd_ring_wait(sm, p, ring_it)) { ok = false; break; }
          if (!mbar_wait(sm.bar_ds_full + 8 * (tt & 1), (uint32_t)((tt >> 1) & 1), sm.abort_flag, p.status)) { ok = false; break; }
          if (j == 0 && !mbar_wait(sm.bar_out_empty, (uint32_t)(o_it & 1) ^ 1u, sm.abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          const int slot = ring_it.slot;
          mma_pv_ts(tmem_base + DQ_ACC, tmem_base + DQ_DP + (uint32_t)((tt & 1) * 128), sm.ring + slot * AT_SLOT_BYTES, j != 0);     // dQ (+)= dS K
          if (j == i) { tc_commit(sm.bar_out_full); ++o_it; }
          ++ring_it; ++tt;
        }
      }
      if (!ok) {
        tc_commit(sm.bar_drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(sm.bar_drain, 0) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
      }
    }
  } else if (warp >= 2 + AT_SOFTMAX_WARPS) {
    // ------------------------------ delta warps: rows t and t + 64 of every item, one item ahead ------------------------------
    const int t = threadIdx.x - (2 + AT_SOFTMAX_WARPS) * 32;       // 0 .. 63
    const long long E = (long long)p.H * AT_D;
    int n_it = 0;
    bool ok = true;
    for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_, ++n_it) {
      int i, h, b;
      item_coords(p, item, i, h, b);
      const int par = n_it & 1;
      if (!mbar_wait(bar_delta_empty + 8 * par, (uint32_t)((n_it >> 1) & 1) ^ 1u, sm.abort_flag, p.status)) { ok = false; break; }
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = t + half * 64;
        const long long off = ((long long)b * p.S + i * AT_TILE + r) * E + (long long)h * AT_D;
        const float4* o4 = reinterpret_cast<const float4*>(p.o + off);
        const float4* g4 = reinterpret_cast<const float4*>(p.d_o + off);
        float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
        for (int c = 0; c < 16; c += 2) {
          const float4 a = o4[c], g = g4[c], a2 = o4[c + 1], g2 = g4[c + 1];
          s0 += (a.x * g.x + a.y * g.y) + (a.z * g.z + a.w * g.w);
          s1 += (a2.x * g2.x + a2.y * g2.y) + (a2.z * g2.z + a2.w * g2.w);
        }
        sm.stats[par * 128 + r] = s0 + s1;
        p.delta[((long long)b * p.H + h) * p.S + i * AT_TILE + r] = s0 + s1;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_delta_full + 8 * par);
    }
  } else {
    const int q = warp & 3, eset = (warp - 2) >> 2;
    const int r_local = q * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    const int sw = r_local & 7;
    int tt = 0, o_it = 0, g_it = 0, n_it = 0;
    int base_mod = 0;                          // ring slot of the item's first load (3 loads per tile: K0, V0; then K(j+1), V(j+1), K(j) MN-major)
    bool ok = true;
    for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_, ++n_it) {
      int i, h, b;
      item_coords(p, item, i, h, b);
      const int row = i * AT_TILE + r_local;
      const float lse2 = p.lse[((long long)b * p.H + h) * p.S + row] * AT_LOG2E;
      const int par = n_it & 1;
      if (!mbar_wait(bar_delta_full + 8 * par, (uint32_t)((n_it >> 1) & 1), sm.abort_flag, p.status)) { ok = false; break; }
      const float delta = sm.stats[par * 128 + r_local];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_delta_empty + 8 * par);
      for (int j = 0; j <= i; ++j) {
        if (!mbar_wait(sm.bar_sdp_full, (uint32_t)(tt & 1), sm.abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        if (warp == 2 && lane == 0) {
          // Ring slots go back to the producer from here, not from the MMA thread: S(j) and dP(j) complete means K(j)
          // and V(j) have been read and, the tensor core executing in issue order ... dQ(j-2), S(j), dP(j), dQ(j-1) ...,
          // that the dQ product with the MN-major K(j-2) has completed too.
          mbar_arrive(sm.bar_ring_empty + 8 * ((base_mod + (j == 0 ? 0 : 3 * j - 1)) % sm.nslots));
          mbar_arrive(sm.bar_ring_empty + 8 * ((base_mod + (j == 0 ? 1 : 3 * j)) % sm.nslots));
          if (j >= 2) mbar_arrive(sm.bar_ring_empty + 8 * ((base_mod + 3 * (j - 2) + 4) % sm.nslots));
        }
        const int col0 = j * AT_TILE + eset * 32;
        const int nvalid = (j < i) ? 32 : row - col0 + 1;        // keys <= query
        const bool dead = (j == i) && (eset > q);                 // chunk wholly right of the diagonal for this warp's rows
        const uint32_t dp_col = DQ_DP + (uint32_t)((tt & 1) * 128 + eset * 32);
        float pr[32], v[32];
        if (!dead) {
          tc_ld32(lane_base + DQ_S + (uint32_t)(eset * 32), v);
          tc_wait_ld();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.bar_sdp_empty);             // S is in registers: the next tile's may be issued
        if (!dead) {
          if (j < i) {                       // warp-uniform: a tile left of the diagonal has no masked element
#pragma unroll
            for (int t = 0; t < 32; ++t) pr[t] = ex2(fmaf(v[t], p.scale_log2, -lse2));
          } else {
#pragma unroll
            for (int t = 0; t < 32; ++t) pr[t] = (t < nvalid) ? ex2(fmaf(v[t], p.scale_log2, -lse2)) : 0.0f;
          }
          tc_ld32(lane_base + dp_col, v);
          tc_wait_ld();
          // dS without its factor `scale`: dQ = scale * sum_j (P (dP - delta)) K takes it once, at the output
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = to_tf32(pr[t] * (v[t] - delta));
        } else {
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = 0.0f;
        }
        tc_st32(lane_base + dp_col, v);                           // dS over dP, in place
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.bar_ds_full + 8 * (tt & 1));
        ++tt;
      }
      if (!ok) break;
      if (!mbar_wait(sm.bar_out_full, (uint32_t)(o_it & 1), sm.abort_flag, p.status)) { ok = false; break; }
      ++o_it;
      tc_fence_after();
      // dQ (64 columns: chunks 0 and 1) leaves through the ring slot of the item's last load (K of the last tile,
      // MN-major), whose reader, the last dQ product, has completed; the slot goes back to the producer below.
      if (warp == 2 && lane == 0 && i >= 1) mbar_arrive(sm.bar_ring_empty + 8 * ((base_mod + 3 * (i - 1) + 4) % sm.nslots));   // MN-major K(i-1); K(i) stages the output
      const int slot_out = (base_mod + 3 * i + 2) % sm.nslots;
      base_mod = (base_mod + 3 * (i + 1)) % sm.nslots;
      if (eset < 2) {
        float v[32];
        tc_ld32(lane_base + DQ_ACC + (uint32_t)(eset * 32), v);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.bar_out_empty);
        const uint32_t stage_off = (uint32_t)(slot_out * AT_SLOT_BYTES + eset * 16384);
        uint8_t* const my_row = sm.tile_ptr - sm.nslots * AT_SLOT_BYTES + stage_off + r_local * 128;
        const uint32_t my_sub = sm.ring + stage_off + (uint32_t)(q * 4096);
#pragma unroll
        for (int g = 0; g < 8; ++g)
          *reinterpret_cast<float4*>(my_row + ((g ^ sw) << 4)) =
              make_float4(p.scale * v[4 * g], p.scale * v[4 * g + 1], p.scale * v[4 * g + 2], p.scale * v[4 * g + 3]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) tma_store_4d(&map_dq, my_sub, eset * 32, i * AT_TILE + q * 32, h, b, accumulate != 0);
        if (p.dbq) atomicAdd(p.dbq + h * AT_D + eset * 32 + lane, p.scale * warp_column_sums(v, lane));    // bias gradient of the q projection
        if (lane == 0) tma_store_wait_read<0>();
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(sm.bar_group);
      if (!mbar_wait(sm.bar_group, (uint32_t)(g_it & 1), sm.abort_flag, p.status)) { ok = false; break; }
      ++g_it;
      if (warp == 2 && lane == 0) mbar_arrive(sm.bar_ring_empty + 8 * slot_out);
    }
    if (lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

// dK and dV for one block of 128 keys: everything transposed, so that a thread owns a key.
//
// Tensor memory: S^T in two buffers (columns 0 and 128), dP^T (256), dV (384), dK (448).  The softmax warps turn S^T
// into P^T and dP^T into dS^T IN PLACE, and the dV / dK products read them from there as their A operand, so neither
// passes through shared memory and the ring gets the room.  The MMA thread issues, per query tile i,
//     S^T(i+1)   dV += P^T(i) dO(i)   dK += dS^T(i) Q(i)   dP^T(i+1)
// and relies on the tensor core executing one thread's products in issue order: S^T(i+1) may overwrite the buffer
// whose P^T(i-1) the earlier dV product read, and dP^T(i+1) may overwrite dS^T(i) behind the dK product, with no
// "empty" barrier in between.  While dV(i) and dK(i) run, the softmax warps already work on S^T(i+1).
constexpr uint32_t KV_ST = 0, KV_DPT = 256, KV_DV = 384, KV_DK = 448;
constexpr int ATK_SLOTS = 5;
constexpr int ATK_SMEM_BYTES = 2 * AT_SLOT_BYTES + ATK_SLOTS * AT_SLOT_BYTES + 1024 + ATB_CTRL_BYTES;

__global__ void __launch_bounds__(AT_THREADS, 1)
gt_attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                       const __grid_constant__ CUtensorMap map_qmn, const __grid_constant__ CUtensorMap map_domn,
                       const __grid_constant__ CUtensorMap map_dk, const __grid_constant__ CUtensorMap map_dv,
                       const AttnParams p, const int acc_dk, const int acc_dv) {
  extern __shared__ uint8_t smem_raw[];
  const BwdSmem sm = carve_bwd(smem_raw, ATK_SLOTS, 0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  bwd_setup(sm, warp, AT_SOFTMAX_WARPS);
  const uint32_t tmem_base = *sm.tmem_slot;
  const int nblk = p.nblk;

  if (warp == 0) {
    if (lane == 0) {
      RingPos ring_it(sm.nslots); int f_it = 0;
      bool ok = true;
      for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_) {
        int j, h, b;
        item_coords_kv(p, item, j, h, b);
        // Ring tiles in the order the MMA thread consumes them: Q(j), dO(j); then per tile Q(i+1), dO(i) MN-major, Q(i)
        // MN-major, dO(i+1).  The first two need only free slots and go out before the wait for the fixed tiles.
        ok = bwd_ring_load(sm, p, ring_it, &map_q, false, j * AT_TILE, h, b) && bwd_ring_load(sm, p, ring_it, &map_do, false, j * AT_TILE, h, b);
        if (!ok || !mbar_wait(sm.bar_fix_empty, (uint32_t)(f_it & 1) ^ 1u, sm.abort_flag, p.status)) { ok = false; break; }
        mbar_expect_tx(sm.bar_fix_full, 2 * AT_SLOT_BYTES);
        tma_load_4d(sm.fix0, &map_k, sm.bar_fix_full, 0, j * AT_TILE, h, b);
        tma_load_4d(sm.fix0 + 16384, &map_k, sm.bar_fix_full, 32, j * AT_TILE, h, b);
        tma_load_4d(sm.fix1, &map_v, sm.bar_fix_full, 0, j * AT_TILE, h, b);
        tma_load_4d(sm.fix1 + 16384, &map_v, sm.bar_fix_full, 32, j * AT_TILE, h, b);
        ++f_it;
        if (const int next = sched_item(p, k_ + 1); next >= 0) {     // the next item's K and V: nobody has read them yet, so start them towards L2 now
          int j2, h2, b2;
          item_coords_kv(p, next, j2, h2, b2);
          prefetch_tile(&map_k, j2 * AT_TILE, h2, b2);
          prefetch_tile(&map_v, j2 * AT_TILE, h2, b2);
        }
        for (int i = j; ok && i < nblk; ++i) {
          if (i + 1 < nblk) ok = bwd_ring_load(sm, p, ring_it, &map_q, false, (i + 1) * AT_TILE, h, b);
          if (ok) ok = bwd_ring_load(sm, p, ring_it, &map_domn, true, i * AT_TILE, h, b) &&
                       bwd_ring_load(sm, p, ring_it, &map_qmn, true, i * AT_TILE, h, b);
          if (ok && i + 1 < nblk) ok = bwd_ring_load(sm, p, ring_it, &map_do, false, (i + 1) * AT_TILE, h, b);
        }
      }
      if (!ok) bwd_ring_drain(sm, ring_it);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      RingPos ring_it(sm.nslots); int f_it = 0, tt = 0 /* tiles issued so far: S^T buffer and barrier parities */, o_it = 0;
      int s_tt = 0;                         // S^T products issued so far
      bool ok = true;
      auto issue_st = [&]() -> bool {       // S^T = K Q^T of the next query tile into buffer s_tt & 1
        if (!bwd_ring_wait(sm, p, ring_it)) return false;
        tc_fence_after();
        const int slot = ring_it.slot;
        mma_qk(tmem_base + KV_ST + (uint32_t)((s_tt & 1) * 128), sm.fix0, sm.ring + slot * AT_SLOT_BYTES);
        tc_commit(sm.bar_s_full + 8 * (s_tt & 1));          // the ring slots are handed back by the first softmax warp (see there)
        ++ring_it; ++s_tt;
        return true;
      };
      auto issue_dpt = [&]() -> bool {      // dP^T = V dO^T of the same tile
        if (!bwd_ring_wait(sm, p, ring_it)) return false;
        tc_fence_after();
        const int slot = ring_it.slot;
        mma_qk(tmem_base + KV_DPT, sm.fix1, sm.ring + slot * AT_SLOT_BYTES);
        tc_commit(sm.bar_dp_full);
        ++ring_it;
        return true;
      };
      for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_) {
        int j, h, b;
        item_coords_kv(p, item, j, h, b);
        if (!mbar_wait(sm.bar_fix_full, (uint32_t)(f_it & 1), sm.abort_flag, p.status)) { ok = false; break; }
        ++f_it;
        ok = issue_st() && issue_dpt();
        if (ok && j == nblk - 1) tc_commit(sm.bar_fix_empty);           // a one-tile item: K and V have been read
        for (int i = j; ok && i < nblk; ++i) {
          if (i + 1 < nblk) { ok = issue_st(); if (!ok) break; }
          // dV (+)= P^T dO
          if (!bwd_ring_wait(sm, p, ring_it)) { ok = false; break; }
          if (!mbar_wait(sm.bar_pa_full + 8 * (tt & 1), (uint32_t)((tt >> 1) & 1), sm.abort_flag, p.status)) { ok = false; break; }
          if (i == j && !mbar_wait(sm.bar_out_empty, (uint32_t)(o_it & 1) ^ 1u, sm.abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          int slot = ring_it.slot;
          mma_pv_ts(tmem_base + KV_DV, tmem_base + KV_ST + (uint32_t)((tt & 1) * 128), sm.ring + slot * AT_SLOT_BYTES, i != j);
          ++ring_it;
          // dK (+)= dS^T Q
          if (!bwd_ring_wait(sm, p, ring_it)) { ok = false; break; }
          if (!mbar_wait(sm.bar_pb_full + 8 * (tt & 1), (uint32_t)((tt >> 1) & 1), sm.abort_flag, p.status)) { ok = false; break; }
          tc_fence_after();
          slot = ring_it.slot;
          mma_pv_ts(tmem_base + KV_DK, tmem_base + KV_DPT, sm.ring + slot * AT_SLOT_BYTES, i != j);
          ++ring_it; ++tt;
          if (i == nblk - 1) { tc_commit(sm.bar_out_full); ++o_it; }
          if (i + 1 < nblk) {
            ok = issue_dpt();                                          // behind dK(i) in the pipe: dS^T(i) has been read
            if (ok && i + 1 == nblk - 1) tc_commit(sm.bar_fix_empty);  // the item's last product with K and V has been issued
          }
        }
      }
      if (!ok) {
        tc_commit(sm.bar_drain);
        const long long t0 = clock64();
        while (!mbar_try_wait(sm.bar_drain, 0) && clock64() - t0 < WAIT_LIMIT_CYCLES) {}
      }
    }
  } else {
    const int q = warp & 3, eset = (warp - 2) >> 2;
    const int r_local = q * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
    const int sw = r_local & 7;
    int tt = 0, o_it = 0, g_it = 0;
    int base_mod = 0;                          // ring slot of the item's first load (4 loads per tile: Q(j), dO(j); then Q(i+1), dO(i) and Q(i) MN-major, dO(i+1))
    bool ok = true;
    for (int k_ = 0, item; ok && (item = sched_item(p, k_)) >= 0; ++k_) {
      int j, h, b;
      item_coords_kv(p, item, j, h, b);
      const float* lse_bh = p.lse + ((long long)b * p.H + h) * p.S;
      const float* delta_bh = p.delta + ((long long)b * p.H + h) * p.S;
      for (int i = j; i < nblk; ++i) {
        const uint32_t st_col = KV_ST + (uint32_t)((tt & 1) * 128 + eset * 32);
        const int q0 = i * AT_TILE + eset * 32;                   // query of this chunk's first column
        const int first_valid = (i > j) ? 0 : r_local - eset * 32;   // columns (queries) >= this thread's key
        const float4* l4 = reinterpret_cast<const float4*>(lse_bh + q0);
        const float4* d4 = reinterpret_cast<const float4*>(delta_bh + q0);
        const bool dead = (i == j) && (eset < q);                 // queries of this chunk all precede this warp's keys
        float pr[32], v[32];
        // ---- S^T -> P^T, in place
        if (!mbar_wait(sm.bar_s_full + 8 * (tt & 1), (uint32_t)((tt >> 1) & 1), sm.abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        const int t_in = i - j;                  // tile number inside the item
        // Ring slots go back to the producer from here, not from the MMA thread: S^T(i) complete means Q(i) has been read
        if (warp == 2 && lane == 0) mbar_arrive(sm.bar_ring_empty + 8 * ((base_mod + (t_in == 0 ? 0 : 4 * t_in - 2)) % sm.nslots));
        if (dead) {
#pragma unroll
          for (int t = 0; t < 32; ++t) pr[t] = 0.0f;
        } else {
          tc_ld32(lane_base + st_col, v);
          tc_wait_ld();
          if (i > j) {                       // warp-uniform: every query of the block may see every key of ours
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const float4 l = l4[g];
              pr[4 * g] = ex2(fmaf(v[4 * g], p.scale_log2, -l.x * AT_LOG2E));
              pr[4 * g + 1] = ex2(fmaf(v[4 * g + 1], p.scale_log2, -l.y * AT_LOG2E));
              pr[4 * g + 2] = ex2(fmaf(v[4 * g + 2], p.scale_log2, -l.z * AT_LOG2E));
              pr[4 * g + 3] = ex2(fmaf(v[4 * g + 3], p.scale_log2, -l.w * AT_LOG2E));
            }
          } else {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
              const float4 l = l4[g];
              pr[4 * g] = (4 * g >= first_valid) ? ex2(fmaf(v[4 * g], p.scale_log2, -l.x * AT_LOG2E)) : 0.0f;
              pr[4 * g + 1] = (4 * g + 1 >= first_valid) ? ex2(fmaf(v[4 * g + 1], p.scale_log2, -l.y * AT_LOG2E)) : 0.0f;
              pr[4 * g + 2] = (4 * g + 2 >= first_valid) ? ex2(fmaf(v[4 * g + 2], p.scale_log2, -l.z * AT_LOG2E)) : 0.0f;
              pr[4 * g + 3] = (4 * g + 3 >= first_valid) ? ex2(fmaf(v[4 * g + 3], p.scale_log2, -l.w * AT_LOG2E)) : 0.0f;
            }
          }
        }
#pragma unroll
        for (int t = 0; t < 32; ++t) v[t] = to_tf32(pr[t]);
        tc_st32(lane_base + st_col, v);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.bar_pa_full + 8 * (tt & 1));
        // ---- dP^T -> dS^T, in place (without the factor `scale`: dK takes it once, at the output)
        if (!mbar_wait(sm.bar_dp_full, (uint32_t)(tt & 1), sm.abort_flag, p.status)) { ok = false; break; }
        tc_fence_after();
        if (warp == 2 && lane == 0) {
          // dP^T(i) complete: dO(i) has been read and, in issue order ... dV(i-1), dK(i-1), dP^T(i) ..., so have the
          // MN-major dO(i-1) and Q(i-1)
          mbar_arrive(sm.bar_ring_empty + 8 * ((base_mod + (t_in == 0 ? 1 : 4 * t_in + 1)) % sm.nslots));
          if (t_in >= 1) {
            mbar_arrive(sm.bar_ring_empty + 8 * ((base_mod + 4 * (t_in - 1) + 3) % sm.nslots));
            mbar_arrive(sm.bar_ring_empty + 8 * ((base_mod + 4 * (t_in - 1) + 4) % sm.nslots));
          }
        }
        if (dead) {
#pragma unroll
          for (int t = 0; t < 32; ++t) v[t] = 0.0f;
        } else {
          tc_ld32(lane_base + KV_DPT + (uint32_t)(eset * 32), v);
          tc_wait_ld();
#pragma unroll
          for (int g = 0; g < 8; ++g) {
            const float4 d = d4[g];
            v[4 * g] = to_tf32(pr[4 * g] * (v[4 * g] - d.x));
            v[4 * g + 1] = to_tf32(pr[4 * g + 1] * (v[4 * g + 1] - d.y));
            v[4 * g + 2] = to_tf32(pr[4 * g + 2] * (v[4 * g + 2] - d.z));
            v[4 * g + 3] = to_tf32(pr[4 * g + 3] * (v[4 * g + 3] - d.w));
          }
        }
        tc_st32(lane_base + KV_DPT + (uint32_t)(eset * 32), v);
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.bar_pb_full + 8 * (tt & 1));
        ++tt;
      }
      if (!ok) break;
      if (!mbar_wait(sm.bar_out_full, (uint32_t)(o_it & 1), sm.abort_flag, p.status)) { ok = false; break; }
      ++o_it;
      tc_fence_after();
      {
        // chunks 0, 1: dV columns 0-31, 32-63; chunks 2, 3: dK columns 0-31, 32-63.  They leave through the ring slots
        // of the item's last two loads (dO and Q of the last tile, MN-major), whose readers, the last dV and dK
        // products, have completed: the MMA thread left those two slots unreleased, and they are handed back to the
        // producer below, once the TMA stores have read them.
        float v[32];
        tc_ld32(lane_base + (eset < 2 ? KV_DV : KV_DK) + (uint32_t)((eset & 1) * 32), v);
        tc_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.bar_out_empty);
        const int n_tiles = nblk - j;
        const int slot_dv = (base_mod + 4 * n_tiles - 2) % sm.nslots, slot_dk = (base_mod + 4 * n_tiles - 1) % sm.nslots;
        base_mod = (base_mod + 4 * n_tiles) % sm.nslots;
        const uint32_t stage_off = (uint32_t)((eset < 2 ? slot_dv : slot_dk) * AT_SLOT_BYTES + (eset & 1) * 16384);
        uint8_t* const my_row = sm.tile_ptr - sm.nslots * AT_SLOT_BYTES + stage_off + r_local * 128;    // the ring ends where the tile would start
        const uint32_t my_sub = sm.ring + stage_off + (uint32_t)(q * 4096);
        const float out_scale = eset < 2 ? 1.0f : p.scale;       // dK carries the factor its dS^T tiles left out
#pragma unroll
        for (int g = 0; g < 8; ++g)
          *reinterpret_cast<float4*>(my_row + ((g ^ sw) << 4)) =
              make_float4(out_scale * v[4 * g], out_scale * v[4 * g + 1], out_scale * v[4 * g + 2], out_scale * v[4 * g + 3]);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) {
          if (eset < 2) tma_store_4d(&map_dv, my_sub, eset * 32, j * AT_TILE + q * 32, h, b, acc_dv != 0);
          else tma_store_4d(&map_dk, my_sub, (eset - 2) * 32, j * AT_TILE + q * 32, h, b, acc_dk != 0);
        }
        if (float* const dbias = eset < 2 ? p.dbv : p.dbk)        // bias gradients of the v and k projections
          atomicAdd(dbias + h * AT_D + (eset & 1) * 32 + lane, out_scale * warp_column_sums(v, lane));
        if (lane == 0) tma_store_wait_read<0>();
        // every warp's store has read its part: the two slots go back to the producer
        __syncwarp();
        if (lane == 0) mbar_arrive(sm.bar_group);
        if (!mbar_wait(sm.bar_group, (uint32_t)(g_it & 1), sm.abort_flag, p.status)) { ok = false; break; }
        ++g_it;
        if (warp == 2 && lane == 0) { mbar_arrive(sm.bar_ring_empty + 8 * slot_dv); mbar_arrive(sm.bar_ring_empty + 8 * slot_dk); }
      }
    }
    if (lane == 0) tma_store_wait_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
}

int check_attn_args(gt_ctx* ctx, const void* q, const void* k, const void* v, int64_t B, int64_t S, int64_t H, int64_t D) {
  if (!ctx || !q || !k || !v || B <= 0 || S <= 0 || H <= 0) return GT_ERR_INVALID_ARG;
  if (D != AT_D) GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "fused attention supports head dimension 64, got %lld", (long long)D);
  if (S % AT_TILE != 0) GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "fused attention needs a sequence length that is a multiple of 128, got %lld", (long long)S);
  if (B * H * (S / AT_TILE) > 0x7fffffffLL || S > (1 << 24)) return GT_ERR_INVALID_ARG;
  if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) != 0) GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "fused attention needs 16-byte aligned q, k, v");
  return GT_OK;
}

// Which items each CTA takes, and in which order.  An item costs its number of 128 x 128 tiles plus a fixed part
// (operand reload, output, statistics); the items, heaviest first, go one by one to the CTA with the least work so
// far.  For 8 x 12 heads of 1024 tokens on 148 SMs the busiest CTA gets 24 tiles instead of the 27 of a round robin.
// One table per (B, H, blocks, grid) and context, built on first use and kept until the context is destroyed.
struct AttnSchedules {
  std::mutex lock;
  std::map<std::array<long long, 4>, std::pair<int*, int>> tables;     // -> (device table, stride)
};

int attn_schedule(gt_ctx* ctx, long long B, long long H, int nblk, int grid, const int** table, int* stride) {
  if (!ctx->attn_schedules) ctx->attn_schedules = new AttnSchedules();
  AttnSchedules* sc = (AttnSchedules*)ctx->attn_schedules;
  std::lock_guard<std::mutex> guard(sc->lock);
  const std::array<long long, 4> key = {B, H, (long long)nblk, (long long)grid};
  auto it = sc->tables.find(key);
  if (it == sc->tables.end()) {
    const long long bh = B * H, items = bh * nblk;
    constexpr double fixed_cost = 1.5;
    std::vector<std::vector<int>> lists((size_t)grid);
    std::priority_queue<std::pair<double, int>, std::vector<std::pair<double, int>>, std::greater<std::pair<double, int>>> least;
    for (int c = 0; c < grid; ++c) least.push({0.0, c});
    for (long long item = 0; item < items; ++item) {       // item numbers are already in order of decreasing cost
      const double cost = (double)(nblk - item / bh) + fixed_cost;
      const auto top = least.top();
      least.pop();
      lists[(size_t)top.second].push_back((int)item);
      least.push({top.first + cost, top.second});
    }
    size_t longest = 0;
    for (const auto& l : lists) longest = l.size() > longest ? l.size() : longest;
    const int st = (int)((longest + 1 + 3) / 4 * 4);
    std::vector<int> host((size_t)grid * st, -1);
    for (int c = 0; c < grid; ++c)
      for (size_t k = 0; k < lists[(size_t)c].size(); ++k) host[(size_t)c * st + k] = lists[(size_t)c][k];
    int* dev = nullptr;
    GT_CUDA_OK(ctx, cudaMalloc(&dev, host.size() * sizeof(int)));
    GT_CUDA_OK(ctx, cudaMemcpy(dev, host.data(), host.size() * sizeof(int), cudaMemcpyHostToDevice));
    it = sc->tables.emplace(key, std::make_pair(dev, st)).first;
  }
  *table = it->second.first;
  *stride = it->second.second;
  return GT_OK;
}

}  // namespace

void gt_attn_release(gt_ctx* ctx) {
  if (!ctx->attn_schedules) return;
  AttnSchedules* sc = (AttnSchedules*)ctx->attn_schedules;
  for (auto& kv : sc->tables) cudaFree(kv.second.first);
  delete sc;
  ctx->attn_schedules = nullptr;
}

extern "C" int gt_attention_forward(gt_ctx* ctx, float* o, float* p_out, float* lse, const float* q, const float* k,
                                    const float* v, int64_t B, int64_t S, int64_t H, int64_t D, float scale, void* stream_) {
  int rc = check_attn_args(ctx, q, k, v, B, S, H, D);
  if (rc != GT_OK) return rc;
  if (!o || ((uintptr_t)o & 15) || (p_out && ((uintptr_t)p_out & 15))) return GT_ERR_INVALID_ARG;
  cudaStream_t stream = stream_ ? (cudaStream_t)stream_ : ctx->stream;
  const long long E = H * D;
  CUtensorMap mq, mk, mv, mp, mo;
  const OperandView vq = {q, S, D, E, D, S * E}, vk = {k, S, D, E, D, S * E}, vv = {v, S, D, E, D, S * E};
  if ((rc = encode_map(ctx, &mq, vq, 32, AT_TILE, H, B, false)) != GT_OK) return rc;
  if ((rc = encode_map(ctx, &mk, vk, 32, AT_TILE, H, B, false)) != GT_OK) return rc;
  if (!encode_map_mn5(ctx, &mv, vv, 2, H, B, false, AT_TILE)) GT_FAIL(ctx, GT_ERR_CUDA, "fused attention: the tensor map of V was refused");
  const OperandView vo = {o, S, D, E, D, S * E};
  if ((rc = encode_map(ctx, &mo, vo, 32, 32, H, B, false, /*plain_f32=*/true)) != GT_OK) return rc;
  if (p_out) {
    const OperandView vp = {p_out, S, S, S, S * S, H * S * S};
    if ((rc = encode_map(ctx, &mp, vp, 32, 32, H, B, false, true)) != GT_OK) return rc;
  } else {
    mp = mo;
  }
  AttnParams p;
  p.S = (int)S; p.H = (int)H; p.B = (int)B;
  p.nblk = (int)(S / AT_TILE);
  p.num_items = (int)(B * H * p.nblk);
  p.scale = scale; p.scale_log2 = scale * AT_LOG2E;
  p.write_p = p_out ? 1 : 0;
  static const bool two_pass = getenv("GRADTUITY_ATTENTION_TWO_PASS") != nullptr;   // tuning aid: the two-pass forward also without P
  p.online = (!p_out && !two_pass) ? 1 : 0;
  p.lse = lse; p.delta = nullptr; p.o = nullptr; p.d_o = nullptr;
  p.dbq = p.dbk = p.dbv = nullptr;
  p.status = ctx->d_status;
  const int grid = p.num_items < ctx->sm_count ? p.num_items : ctx->sm_count;
  if ((rc = attn_schedule(ctx, B, H, p.nblk, grid, &p.sched, &p.sched_stride)) != GT_OK) return rc;
  if (p.online) {
    GT_SMEM_OPT_IN(ctx, gt_attn_fwd_online_kernel, ATF_SMEM_BYTES);
    GT_CUDA_OK(ctx, gt_launch_overlapped(gt_attn_fwd_online_kernel, dim3(grid), dim3(AT_THREADS), ATF_SMEM_BYTES, stream, mq, mk, mv, mo, p));
    ctx->launches += 1;
    return GT_OK;
  }
  GT_SMEM_OPT_IN(ctx, gt_attn_fwd_kernel, AT_SMEM_BYTES);
  GT_CUDA_OK(ctx, gt_launch_overlapped(gt_attn_fwd_kernel, dim3(grid), dim3(AT_THREADS), AT_SMEM_BYTES, stream, mq, mk, mv, mp, mo, p));
  ctx->launches += 1;
  return GT_OK;
}

extern "C" int gt_attention_backward(gt_ctx* ctx, float* dq, float* dk, float* dv, const float* d_o, const float* q,
                                     const float* k, const float* v, const float* o, const float* lse, float* delta,
                                     int64_t B, int64_t S, int64_t H, int64_t D, float scale, int acc_dq, int acc_dk,
                                     int acc_dv, void* stream_) {
  return gt_attention_backward_bias(ctx, dq, dk, dv, nullptr, nullptr, nullptr, d_o, q, k, v, o, lse, delta, B, S, H, D, scale, acc_dq, acc_dk,
                                    acc_dv, stream_);
}

// The same; a non-null dbq / dbk / dbv (H * 64 floats) also receives the column sums over all tokens of what this call
// computed for dQ / dK / dV (added to its contents): the bias gradients of the projections that produced q, k, v.
extern "C" int gt_attention_backward_bias(gt_ctx* ctx, float* dq, float* dk, float* dv, float* dbq, float* dbk, float* dbv, const float* d_o,
                                          const float* q, const float* k, const float* v, const float* o, const float* lse, float* delta,
                                          int64_t B, int64_t S, int64_t H, int64_t D, float scale, int acc_dq, int acc_dk, int acc_dv,
                                          void* stream_) {
  int rc = check_attn_args(ctx, q, k, v, B, S, H, D);
  if (rc != GT_OK) return rc;
  if (!dq || !dk || !dv || !d_o || !o || !lse || !delta) return GT_ERR_INVALID_ARG;
  if ((((uintptr_t)dq | (uintptr_t)dk | (uintptr_t)dv | (uintptr_t)d_o | (uintptr_t)o | (uintptr_t)lse | (uintptr_t)delta) & 15) != 0)
    GT_FAIL(ctx, GT_ERR_UNSUPPORTED, "fused attention backward needs 16-byte aligned buffers");
  cudaStream_t stream = stream_ ? (cudaStream_t)stream_ : ctx->stream;
  const long long E = H * D;
  auto view = [&](const float* ptr) { return OperandView{ptr, S, D, E, D, S * E}; };
  CUtensorMap mq, mk, mv, mdo, mkmn, mqmn, mdomn, mdq, mdk, mdv;
  if ((rc = encode_map(ctx, &mq, view(q), 32, AT_TILE, H, B, false)) != GT_OK) return rc;
  if ((rc = encode_map(ctx, &mk, view(k), 32, AT_TILE, H, B, false)) != GT_OK) return rc;
  if ((rc = encode_map(ctx, &mv, view(v), 32, AT_TILE, H, B, false)) != GT_OK) return rc;
  if ((rc = encode_map(ctx, &mdo, view(d_o), 32, AT_TILE, H, B, false)) != GT_OK) return rc;
  if (!encode_map_mn5(ctx, &mkmn, view(k), 2, H, B, false, AT_TILE) || !encode_map_mn5(ctx, &mqmn, view(q), 2, H, B, false, AT_TILE) ||
      !encode_map_mn5(ctx, &mdomn, view(d_o), 2, H, B, false, AT_TILE))
    GT_FAIL(ctx, GT_ERR_CUDA, "fused attention backward: a tensor map was refused");
  if ((rc = encode_map(ctx, &mdq, view(dq), 32, 32, H, B, false, true)) != GT_OK) return rc;
  if ((rc = encode_map(ctx, &mdk, view(dk), 32, 32, H, B, false, true)) != GT_OK) return rc;
  if ((rc = encode_map(ctx, &mdv, view(dv), 32, 32, H, B, false, true)) != GT_OK) return rc;
  AttnParams p;
  p.S = (int)S; p.H = (int)H; p.B = (int)B;
  p.nblk = (int)(S / AT_TILE);
  p.num_items = (int)(B * H * p.nblk);
  p.scale = scale; p.scale_log2 = scale * AT_LOG2E;
  p.write_p = 0; p.online = 0;
  p.lse = const_cast<float*>(lse); p.delta = delta; p.o = o; p.d_o = d_o;
  p.dbq = dbq; p.dbk = dbk; p.dbv = dbv;
  p.status = ctx->d_status;
  GT_SMEM_OPT_IN(ctx, gt_attn_bwd_dq_kernel, ATQ_SMEM_BYTES);
  GT_SMEM_OPT_IN(ctx, gt_attn_bwd_dkv_kernel, ATK_SMEM_BYTES);
  const int grid = p.num_items < ctx->sm_count ? p.num_items : ctx->sm_count;
  if ((rc = attn_schedule(ctx, B, H, p.nblk, grid, &p.sched, &p.sched_stride)) != GT_OK) return rc;
  GT_CUDA_OK(ctx, gt_launch_overlapped(gt_attn_bwd_dq_kernel, dim3(grid), dim3(ATQ_THREADS), ATQ_SMEM_BYTES, stream, mq, mdo, mk, mv, mkmn, mdq, p, acc_dq));
  GT_CUDA_OK(ctx, gt_launch_overlapped(gt_attn_bwd_dkv_kernel, dim3(grid), dim3(AT_THREADS), ATK_SMEM_BYTES, stream, mk, mv, mq, mdo, mqmn, mdomn, mdk, mdv,
                                       p, acc_dk, acc_dv));
  ctx->launches += 2;
  return GT_OK;
}
