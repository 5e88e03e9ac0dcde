// SDPA backward for sm_100a (bf16, head size 128), mask from token positions.
//
// Given dO, the forward's O and log-sum-exp, computes
//   dQ (B,H,T,D) bf16, and accumulates dK, dV into fp32 cache-shaped buffers (B,G,C,D).
// Two launches of one kernel template, so that every output tile has exactly one
// owner CTA (no atomics, deterministic):
//   MODE_DQ : CTA = 128 query rows (positions x heads of a KV group), streams KV slots
//             S = Q K^T, dP = dO V^T  ->  dS = P (dP − δ) scale  ->  dQ += dS K
//   MODE_DKV: CTA = 128 KV slots, streams query rows
//             S^T = K Q^T, dP^T = V dO^T -> P^T, dS^T -> dV += P^T dO, dK += dS^T Q
// Both are the same pipeline. A fixed "row" tile has two K-major operands (R1, R2) in shared
// memory. The streamed "column" operands (C1, C2) arrive by TMA in units of 64 columns through a
// 4-stage ring. For every unit, X = R1 C1^T and Y = R2 C2^T (128 x 64, fp32) are formed in one of
// two TMEM buffers; the 256 compute threads (TMEM lane = row) turn them into bf16 P and dS, which
// they write back into the same TMEM columns; the accumulating MMAs then take P / dS as their
// A operand straight from TMEM and the column operands, from the same shared memory, as
// MN-major B operands (acc1 += P C2, acc2 += dS C1). P and dS never touch shared memory, whose
// bandwidth is what bounds this kernel. MMAs of one thread execute in issue order, so the X/Y
// MMAs of unit u+2, which overwrite the buffer of unit u, are issued after the accumulating
// MMAs of unit u. δ = rowsum(dO ⊙ O) comes from a small kernel.
//
// Replaces the blocked fp32 PyTorch backward of the reference
// (keys_values/attention/sdpa_op.py:31-251) and the library SDPA backward it otherwise uses.
#include <cuda.h>
#include <limits.h>
#include <stdlib.h>

#include "common.cuh"
#include "kvb200.h"

namespace kvb {

constexpr int BW_TILE_BYTES = 128 * 128 * 2;   // row operand: two 64-feature chunks of [128 rows x 128 B]
constexpr int BW_UNIT_BYTES = 64 * 128 * 2;    // column operand of one unit: two chunks of [64 rows x 128 B]
constexpr int BW_STAGES = 4;                   // ring of column units (C1 | C2 per stage)
constexpr int BW_THREADS = 352;                // TMA warp + MMA warp (even units) + 8 compute warps + MMA warp (odd units)
enum { MODE_DQ = 0, MODE_DKV = 1 };

struct BwSmem {
  static constexpr int R1 = 0;
  static constexpr int R2 = R1 + BW_TILE_BYTES;
  static constexpr int C = R2 + BW_TILE_BYTES;                    // per stage: C1 | C2
  static constexpr int STATS = C + BW_STAGES * 2 * BW_UNIT_BYTES; // tp[128] | nlse[2][128] | ndls[2][128]
  static constexpr int FLAGS = STATS + 512 + 1024 + 1024;         // one byte per column tile: bit 0 active, bit 1 masked
  static constexpr int NFLAGS = 4096;
  static constexpr int BAR = FLAGS + NFLAGS;
  static constexpr int TOTAL = BAR + 256 + 1024;
};

struct BwParams {
  const int32_t* token_pos;
  const int32_t* tile_min;
  const int32_t* tile_max;
  const float* lse;     // (B,H,T) natural log
  const float* delta;   // (B,H,T)
  __nv_bfloat16* dq;    // (B,H,T,D)
  float* dk;            // (B,G,C,D) accumulated
  float* dv;
  int B, H, G, T, L, nT, nQT, gs, npos;
  // Query rows are packed head-major: a 128-row tile of the dQ launch holds npos = 128 / gs (rounded down) positions
  // x gs heads (rows_used of 128 rows), a 64-column unit of the dK/dV launch holds hnpos positions x u_heads
  // heads (cols_used of 64 columns); a column tile of the dK/dV launch is two units and spans npos_col positions.
  int rows_used, hnpos, cols_used, npos_col, nCT;
  // Unit h of a column tile holds u_heads heads x hnpos positions, from head h·u_dh and position h·u_dp of the tile:
  // half of the heads over all positions of the tile when the group size is an even power of two (u_dh = gs / 2,
  // u_dp = 0), all heads over half of the positions otherwise (u_dh = 0, u_dp = hnpos).
  int u_heads, u_dh, u_dp;
  long long tp_sb, tp_sg, dk_sb, dk_sg;
  float scale, scale_log2;
  int input_pos;
  // Sliding window (0: none): a slot is visible to a query at position q iff q - window < token <= q.
  // Soft-capping (cap_pre = 0: none): s' = cap·tanh(scale·s / cap) with cap_pre = scale / cap, cap_l2 = cap·log2(e);
  // then P = exp2(cap_l2·t − lse·log2(e)) and dS = P (dP − δ) scale (1 − t²) with t = tanh(cap_pre·s).
  int window;
  float cap_pre, cap_l2;
  int* status;
  long long* trace;     // optional timeline of CTA 0: per role trace_cap (tag, clock) pairs
  int trace_cap;
};

// Timeline event of one role (1 MMA issuer, 2 first compute warp) of CTA 0.
#define BW_TRACE(role, tag)                                               \
  do {                                                                    \
    if (p.trace && blockIdx.x == 0 && tr_n < p.trace_cap) {               \
      p.trace[((role) * p.trace_cap + tr_n) * 2] = (long long)(tag);      \
      p.trace[((role) * p.trace_cap + tr_n) * 2 + 1] = clock64();         \
      ++tr_n;                                                             \
    }                                                                     \
  } while (0)

__device__ __forceinline__ float bw_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// hardware tanh, as in the forward kernels (P must be recomputed from the same capped scores)
__device__ __forceinline__ float bw_tanh(float z) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(z));
  return t;
}

// delta[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]
// With dOt the kernel also leaves a head-major copy dOt[b,h,t,:] of dO (which it reads anyway): the TMA boxes of the
// two launches then read runs of consecutive positions of one head, as they do for Q.
template <int HD>
__global__ void att_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O,
                                 float* __restrict__ delta, __nv_bfloat16* __restrict__ dOt, int B, int T, int H) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (row >= (long long)B * T * H) return;
  const int lane = threadIdx.x & 31;
  constexpr int PER = HD / 32;  // features per lane: 4 (one 8-byte access) or 2 (one 4-byte access)
  uint2 a = make_uint2(0, 0), o = make_uint2(0, 0);
  if (PER == 4) {
    a = *reinterpret_cast<const uint2*>(dO + row * HD + lane * 4);
    o = *reinterpret_cast<const uint2*>(O + row * HD + lane * 4);
  } else {
    a.x = *reinterpret_cast<const uint32_t*>(dO + row * HD + lane * 2);
    o.x = *reinterpret_cast<const uint32_t*>(O + row * HD + lane * 2);
  }
  const __nv_bfloat162* ap = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* op = reinterpret_cast<const __nv_bfloat162*>(&o);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < PER / 2; ++i) {
    const float2 x = __bfloat1622float2(ap[i]), y = __bfloat1622float2(op[i]);
    s += x.x * y.x + x.y * y.y;
  }
  s = warp_sum(s);
  const int h = (int)(row % H);
  const long long bt = row / H;
  const int t = (int)(bt % T);
  const int b = (int)(bt / T);
  const long long hrow = ((long long)b * H + h) * T + t;
  if (dOt) {
    if (PER == 4) *reinterpret_cast<uint2*>(dOt + hrow * HD + lane * 4) = a;
    else *reinterpret_cast<uint32_t*>(dOt + hrow * HD + lane * 2) = a.x;
  }
  if (lane == 0) delta[hrow] = s;
}

// tmR1/tmR2: row operands (boxes of 128 rows); tmC1/tmC2: column operands (boxes of 64 rows).
//   MODE_DQ : R1 = Q, R2 = dO, C1 = K, C2 = V      MODE_DKV: R1 = K, R2 = V, C1 = Q, C2 = dO
// GEN: sliding window and / or soft-capping are in use (separate instantiations, so that the plain kernels keep their
// register allocation)
// HD: head size, 128 or 64 (row operands and units of one 64-feature chunk, half as many K steps for X / Y,
// accumulators of 64 columns)
template <int MODE, bool GEN, int HD>
__global__ void __launch_bounds__(BW_THREADS, 1)
sdpa_bwd_kernel(const __grid_constant__ CUtensorMap tmR1, const __grid_constant__ CUtensorMap tmR2,
                const __grid_constant__ CUtensorMap tmC1, const __grid_constant__ CUtensorMap tmC2, const BwParams p) {
  using S = BwSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::BAR);
  uint64_t* r_full = bars + 0;
  uint64_t* c_full = bars + 1;     // [4]
  uint64_t* c_empty = bars + 5;    // [4]
  uint64_t* xy_full = bars + 9;    // [2]
  uint64_t* pds_full = bars + 11;  // [2]
  uint64_t* acc_full = bars + 13;
  uint64_t* grp_bar = bars + 14;
  uint64_t* rows_ready = bars + 15;  // accumulators zeroed (and, MODE_DQ, the row operands moved to TMEM)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stat_nlse = reinterpret_cast<float*>(smem + S::STATS + 512);  // MODE_DKV: [2][128] −lse·log2(e) of the query tile
  float* stat_ndls = reinterpret_cast<float*>(smem + S::STATS + 1536); // MODE_DKV: [2][128] −delta·scale of the query tile

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_row_tiles = MODE == MODE_DQ ? p.nQT : p.nT;
  const int qtile_pos = MODE == MODE_DQ ? p.npos : p.npos_col;  // positions per query tile of this launch
  const int rt = blockIdx.x % n_row_tiles;                 // row tile: query tile (DQ) or KV tile (DKV)
  const int g = (blockIdx.x / n_row_tiles) % p.G;
  const int b = blockIdx.x / (n_row_tiles * p.G);
  const int32_t* tmin = p.tile_min + ((long long)b * p.G + g) * p.nT;
  const int32_t* tmax = p.tile_max + ((long long)b * p.G + g) * p.nT;
  const int n_col_tiles = MODE == MODE_DQ ? p.nT : p.nCT;

  // (kv tile t, query tile qt) is active iff some slot of t is visible to some query of qt
  auto qpos_min_of = [&](int qt) { return p.input_pos + qt * qtile_pos; };
  auto qpos_max_of = [&](int qt) { return p.input_pos + min((qt + 1) * qtile_pos, p.T) - 1; };
  // with a window, a tile is also inactive when its newest token has left the window of the first query, and
  // masked when its oldest token has left the window of the last query
  const int win = GEN ? p.window : 0;
  auto active_g = [&](int ct) -> bool {
    const int kt = MODE == MODE_DQ ? ct : rt, qt = MODE == MODE_DQ ? rt : ct;
    return tmin[kt] <= qpos_max_of(qt) && (win <= 0 || tmax[kt] > qpos_min_of(qt) - win);
  };
  auto masked_g = [&](int ct) -> bool {
    const int kt = MODE == MODE_DQ ? ct : rt, qt = MODE == MODE_DQ ? rt : ct;
    return tmax[kt] > qpos_min_of(qt) || (win > 0 && tmin[kt] <= qpos_max_of(qt) - win);
  };
  // the flags of the column tiles are kept in shared memory so that no role reads global memory
  // inside its tile loop
  uint8_t* tflags = smem + S::FLAGS;
  for (int ct = threadIdx.x; ct < n_col_tiles && ct < S::NFLAGS; ct += BW_THREADS)
    tflags[ct] = (uint8_t)((active_g(ct) ? 1 : 0) | (masked_g(ct) ? 2 : 0));
  auto active = [&](int ct) -> bool { return ct < S::NFLAGS ? (tflags[ct] & 1) != 0 : active_g(ct); };
  auto masked = [&](int ct) -> bool { return ct < S::NFLAGS ? (tflags[ct] & 2) != 0 : masked_g(ct); };
  auto next_active = [&](int ct) -> int {
    while (ct < n_col_tiles && !active(ct)) ++ct;
    return ct;
  };

  // Rows that no TMA box ever writes (group sizes that do not divide the tile: 128 − rows_used rows of the row
  // operands in the dQ launch, 64 − cols_used rows of every streamed unit in the dK/dV launch) are zeroed once: they
  // enter MMAs as operand rows, and 0 · anything finite is 0 while stale shared memory could hold NaN patterns.
  if (MODE == MODE_DQ && p.rows_used < 128) {
    const int n16 = (128 - p.rows_used) * 8;  // 16-byte pieces per 64-feature chunk
    constexpr int NCH = HD / 64;
    for (int i = threadIdx.x; i < 2 * NCH * n16; i += BW_THREADS) {
      uint8_t* chunk = smem + ((i / n16) / NCH == 0 ? S::R1 : S::R2) + ((i / n16) % NCH) * (BW_TILE_BYTES / 2);
      *reinterpret_cast<uint4*>(chunk + p.rows_used * 128 + (i % n16) * 16) = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async_smem();
  }
  if (MODE == MODE_DKV && p.cols_used < 64) {
    const int n16 = (64 - p.cols_used) * 8;
    constexpr int NCH = HD / 64;
    for (int i = threadIdx.x; i < BW_STAGES * 2 * NCH * n16; i += BW_THREADS) {
      const int idx = i / n16;  // (stage, operand C1 | C2, 64-feature chunk)
      uint8_t* chunk = smem + S::C + (idx / NCH) * BW_UNIT_BYTES + (idx % NCH) * (BW_UNIT_BYTES / 2);
      *reinterpret_cast<uint4*>(chunk + p.cols_used * 128 + (i % n16) * 16) = make_uint4(0, 0, 0, 0);
    }
    fence_proxy_async_smem();
  }
  if (threadIdx.x == 0) {
    mbar_init(r_full, 1);
    for (int s = 0; s < BW_STAGES; ++s) {
      mbar_init(&c_full[s], 1);
      mbar_init(&c_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&xy_full[s], 1);
      mbar_init(&pds_full[s], 8);
    }
    mbar_init(acc_full, 2);  // one commit per MMA issuer
    mbar_init(grp_bar, 256);
    mbar_init(rows_ready, 8);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // X buffers: columns [0,64) and [64,128); Y buffers: [128,192) and [192,256); accumulators after
  // MODE_DQ has one accumulator only; the free 128 columns hold its row operands Q and dO as bf16
  // pairs (64 columns each), so that the X / Y MMAs take A from TMEM and read only the streamed
  // columns from shared memory.
  const uint32_t tmem_X = tmem_base, tmem_Y = tmem_base + 128, tmem_A1 = tmem_base + 256;
  const uint32_t tmem_A2 = tmem_base + (MODE == MODE_DQ ? 256 : 384);
  const uint32_t tmem_R1 = tmem_base + 384, tmem_R2 = tmem_base + 448;  // MODE_DQ only

  int n_active = 0;
  for (int ct = 0; ct < n_col_tiles; ++ct) n_active += active(ct) ? 1 : 0;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && n_active > 0) {
      tma_prefetch_desc(&tmR1);
      tma_prefetch_desc(&tmR2);
      tma_prefetch_desc(&tmC1);
      tma_prefetch_desc(&tmC2);
      mbar_expect_tx(r_full, MODE == MODE_DQ ? (uint32_t)(4 * p.rows_used * HD) : (uint32_t)(2 * 128 * HD * 2));
      {
        const int c1 = MODE == MODE_DQ ? rt * p.npos : rt * 128;
        const int c2 = MODE == MODE_DQ ? g * p.gs : g;
        tma_load_4d(smem + S::R1, &tmR1, r_full, 0, c1, c2, b);
        if (HD == 128) tma_load_4d(smem + S::R1 + BW_TILE_BYTES / 2, &tmR1, r_full, 64, c1, c2, b);
        tma_load_4d(smem + S::R2, &tmR2, r_full, 0, c1, c2, b);
        if (HD == 128) tma_load_4d(smem + S::R2 + BW_TILE_BYTES / 2, &tmR2, r_full, 64, c1, c2, b);
      }
      uint32_t u = 0;
      bool ok = true;
      for (int ct = 0; ct < n_col_tiles && ok; ++ct) {
        if (!active(ct)) continue;
        for (int h = 0; h < 2; ++h, ++u) {
          const int st = u % BW_STAGES;
          if (!mbar_wait_bounded(&c_empty[st], ((u / BW_STAGES) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) { ok = false; break; }
          uint8_t* c1 = smem + S::C + st * 2 * BW_UNIT_BYTES;
          uint8_t* c2 = c1 + BW_UNIT_BYTES;
          int x1, x2;  // coordinates 1 and 2 of the 64-row box
          if (MODE == MODE_DQ) {
            x1 = ct * 128 + h * 64;
            x2 = g;
          } else {  // unit h of query tile ct
            x1 = ct * p.npos_col + h * p.u_dp;
            x2 = g * p.gs + h * p.u_dh;
          }
          mbar_expect_tx(&c_full[st], MODE == MODE_DQ ? (uint32_t)(2 * 64 * HD * 2) : (uint32_t)(4 * p.cols_used * HD));
          tma_load_4d(c1, &tmC1, &c_full[st], 0, x1, x2, b);
          if (HD == 128) tma_load_4d(c1 + BW_UNIT_BYTES / 2, &tmC1, &c_full[st], 64, x1, x2, b);
          tma_load_4d(c2, &tmC2, &c_full[st], 0, x1, x2, b);
          if (HD == 128) tma_load_4d(c2 + BW_UNIT_BYTES / 2, &tmC2, &c_full[st], 64, x1, x2, b);
        }
      }
      if (!ok) {  // let copies in flight land before the CTA's shared memory is released
        long long c0 = clock64();
        while (clock64() - c0 < 2000000LL) {
        }
      }
    }
  } else if (warp == 1 || warp == 10) {
    // ------------------------------------------------------------ MMA issuers
    // Two threads issue: warp 1 the even units, warp 10 the odd ones. A unit's MMAs (its X / Y pair
    // and, two units later in the same thread, the accumulating MMAs that read P / dS from the same
    // TMEM buffer) stay in one thread, so their order is the issue order; the accumulators are
    // shared by both threads, which is why they are zeroed up front and every MMA accumulates.
    // While one thread sits in its barrier waits (≈ 250 cycles each, even when satisfied) the other
    // one keeps the tensor pipe fed.
    if (lane == 0 && n_active > 0) {
      const uint32_t par = warp == 1 ? 0u : 1u;
      constexpr uint32_t idesc_xy = make_idesc_bf16(128, 64, 0, 0);     // both operands K-major
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, HD, 0, 1);    // A from TMEM, B MN-major
      const uint32_t r1 = smem_u32(smem + S::R1), r2 = smem_u32(smem + S::R2);
      const uint32_t cbase = smem_u32(smem + S::C);
      const uint32_t n_units = 2u * (uint32_t)n_active;
      bool ok = mbar_wait_bounded(r_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL);
      if (ok) {
        ok = mbar_wait_bounded(rows_ready, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL);
        tc_fence_after();
      }
      int tr_n = par == 0 ? 0 : (1 << 30);  // only the first issuer records
      auto wait_c = [&](uint32_t u) -> bool {
        return mbar_wait_bounded(&c_full[u % BW_STAGES], (u / BW_STAGES) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL);
      };
      auto issue_xy = [&](uint32_t u) -> bool {  // after wait_c(u)
        const uint32_t st = u % BW_STAGES, hb = u & 1;
        tc_fence_after();
        const uint32_t c1 = cbase + st * 2 * BW_UNIT_BYTES, c2 = c1 + BW_UNIT_BYTES;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t a_off = (uint32_t)((kk >> 2) * (BW_TILE_BYTES / 2) + (kk & 3) * 32);
          const uint32_t b_off = (uint32_t)((kk >> 2) * (BW_UNIT_BYTES / 2) + (kk & 3) * 32);
          if (MODE == MODE_DQ)
            umma_f16_ts(tmem_X + 64 * hb, tmem_R1 + 8 * kk, make_smem_desc_sw128(c1 + b_off, 16, 1024), idesc_xy, kk != 0);
          else
            umma_f16_ss(tmem_X + 64 * hb, make_smem_desc_sw128(r1 + a_off, 16, 1024), make_smem_desc_sw128(c1 + b_off, 16, 1024),
                        idesc_xy, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t a_off = (uint32_t)((kk >> 2) * (BW_TILE_BYTES / 2) + (kk & 3) * 32);
          const uint32_t b_off = (uint32_t)((kk >> 2) * (BW_UNIT_BYTES / 2) + (kk & 3) * 32);
          if (MODE == MODE_DQ)
            umma_f16_ts(tmem_Y + 64 * hb, tmem_R2 + 8 * kk, make_smem_desc_sw128(c2 + b_off, 16, 1024), idesc_xy, kk != 0);
          else
            umma_f16_ss(tmem_Y + 64 * hb, make_smem_desc_sw128(r2 + a_off, 16, 1024), make_smem_desc_sw128(c2 + b_off, 16, 1024),
                        idesc_xy, kk != 0);
        }
        umma_commit(&xy_full[hb]);
        return true;
      };
      auto issue_acc = [&](uint32_t u) -> bool {
        const uint32_t st = u % BW_STAGES, hb = u & 1;
        if (!mbar_wait_bounded(&pds_full[hb], (u >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL)) return false;
        BW_TRACE(1, 1200000 + u);
        tc_fence_after();
        const uint32_t c1 = cbase + st * 2 * BW_UNIT_BYTES, c2 = c1 + BW_UNIT_BYTES;
        // A: 16 columns of the unit per step = 8 TMEM columns; the two compute warps of a lane
        // quarter keep their 32 columns in separate 32-column halves of the buffer.
        // B: MN-major, 16 rows of the unit per step (2048 B); the 64-feature chunks are LBO apart.
        // All steps of one accumulator are issued back to back: changing the accumulator between
        // MMAs costs far more than the MMA itself.
        if (MODE == MODE_DKV) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t a_col = (uint32_t)(32 * (kk >> 1) + 8 * (kk & 1));
            const uint32_t b_off = (uint32_t)(kk * 16 * 128);
            umma_f16_ts(tmem_A1, tmem_X + 64 * hb + a_col, make_smem_desc_sw128(c2 + b_off, BW_UNIT_BYTES / 2, 1024), idesc_acc, 1);
          }
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          const uint32_t a_col = (uint32_t)(32 * (kk >> 1) + 8 * (kk & 1));
          const uint32_t b_off = (uint32_t)(kk * 16 * 128);
          umma_f16_ts(tmem_A2, tmem_Y + 64 * hb + a_col, make_smem_desc_sw128(c1 + b_off, BW_UNIT_BYTES / 2, 1024), idesc_acc, 1);
        }
        umma_commit(&c_empty[st]);
        return true;
      };
      if (ok && par < n_units) {
        ok = wait_c(par);
        if (ok) ok = issue_xy(par);
      }
      for (uint32_t u = par; u < n_units && ok; u += 2) {
        // the columns of unit u + 2 are awaited while the compute warps still work on unit u, so
        // that only the wait for P / dS lies between them and the next MMAs
        BW_TRACE(1, 1000000 + u);
        if (u + 2 < n_units) ok = wait_c(u + 2);
        BW_TRACE(1, 1100000 + u);
        if (ok) ok = issue_acc(u);
        BW_TRACE(1, 1300000 + u);
        if (ok && u + 2 < n_units) ok = issue_xy(u + 2);
        BW_TRACE(1, 1400000 + u);
      }
      if (ok) umma_commit(acc_full);
    }
  } else if (warp >= 2) {
    // ----------------------------------------------- compute + epilogue warps
    // 8 warps: two per TMEM lane quarter; thread (row, hh) owns columns [32·hh, +32) of its row in
    // every 64-column unit, and columns [64·hh, +64) of the accumulators in the epilogue
    const int quarter = warp & 3;
    const int hh = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int tid = threadIdx.x - 64;  // 0..255
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    bool ok = n_active > 0;
    uint32_t s = 0, grp_phase = 0;
    int tr_n = (warp == 2 && lane == 0) ? 0 : (1 << 30);  // only the first compute warp records
    auto group_sync = [&]() -> bool {
      mbar_arrive(grp_bar);
      const bool done = mbar_wait_bounded(grp_bar, grp_phase, abort_flag, p.status, STATUS_TIMEOUT_MISC);
      grp_phase ^= 1;
      return done;
    };
    // per-row constants
    float row_nlse = -INFINITY, row_ndls = 0.f;
    int row_pos = 0, row_tp = INT_MAX;
    bool row_valid;
    int hq = 0, tq = 0;
    if (MODE == MODE_DQ) {
      hq = row / p.npos;
      tq = rt * p.npos + row % p.npos;
      row_valid = row < p.rows_used && tq < p.T;
      if (!row_valid) hq = 0;
      row_pos = p.input_pos + tq;
      if (row_valid) {
        const long long idx = ((long long)b * p.H + g * p.gs + hq) * p.T + tq;
        row_nlse = -p.lse[idx] * 1.4426950408889634f;
        row_ndls = -p.delta[idx] * p.scale;
      }
    } else {
      const int j = rt * 128 + row;
      row_valid = j < p.L;
      if (row_valid) row_tp = p.token_pos ? p.token_pos[b * p.tp_sb + g * p.tp_sg + j] : j;
    }
    // MODE_DKV: statistics of query tile ct, column cc <-> (head cc / npos, position cc % npos);
    // threads 0..127 fetch −lse·log2(e), threads 128..255 fetch −delta·scale
    auto fetch_stat = [&](int ct) -> float {
      const int cc = tid & 127;                       // column of the tile: unit cc / 64, column cu of the unit
      const int cu = cc & 63;
      const int c_hq = (cc >> 6) * p.u_dh + cu / p.hnpos, c_tq = ct * p.npos_col + (cc >> 6) * p.u_dp + cu % p.hnpos;
      // columns beyond the unit's heads (padding) and positions beyond the chunk: P = exp2(x − inf) = 0, dS = 0
      if (ct >= n_col_tiles || cu >= p.cols_used || c_tq >= p.T) return tid < 128 ? -INFINITY : 0.f;
      const long long idx = ((long long)b * p.H + g * p.gs + c_hq) * p.T + c_tq;
      return tid < 128 ? -p.lse[idx] * 1.4426950408889634f : -p.delta[idx] * p.scale;
    };
    auto store_stat = [&](int buf, float v) {
      if (tid < 128) stat_nlse[buf * 128 + tid] = v;
      else stat_ndls[buf * 128 + (tid - 128)] = v;
    };
    if (ok) {
      // zero this thread's 64 columns of the accumulator(s): both MMA issuers only ever accumulate
      uint32_t z[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) z[i] = 0;
#pragma unroll
      for (int c = 0; c < HD / 2; c += 16) {
        if (MODE == MODE_DKV) tmem_st_32x32b_x16(tmem_A1 + lane_base + (uint32_t)((HD / 2) * hh + c), z);
        tmem_st_32x32b_x16(tmem_A2 + lane_base + (uint32_t)((HD / 2) * hh + c), z);
      }
      if (MODE == MODE_DQ) ok = mbar_wait_bounded(r_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL);
      // MODE_DQ row operands: shared memory -> registers -> TMEM. This thread moves features
      // [64·hh, +64) of its row: one 128-byte swizzled row of chunk hh = 32 columns of bf16 pairs.
      if (MODE == MODE_DQ && ok && (HD == 128 || hh == 0)) {
#pragma unroll
        for (int op = 0; op < 2; ++op) {
          const uint8_t* src = smem + (op == 0 ? S::R1 : S::R2) + hh * (BW_TILE_BYTES / 2);
          uint32_t w[32];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint4 q4 = *reinterpret_cast<const uint4*>(src + sw128_offset(row, u));
            w[4 * u] = q4.x; w[4 * u + 1] = q4.y; w[4 * u + 2] = q4.z; w[4 * u + 3] = q4.w;
          }
          const uint32_t dst = (op == 0 ? tmem_R1 : tmem_R2) + lane_base + (uint32_t)(32 * hh);
          tmem_st_32x32b_x16(dst, w);
          tmem_st_32x32b_x16(dst + 16, w + 16);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0 && ok) mbar_arrive(rows_ready);
    }
    int ct = next_active(0);
    if (MODE == MODE_DKV && ok) {
      store_stat(0, fetch_stat(ct));
      ok = group_sync();
    }
    const float2 c2 = make_float2(p.scale_log2, p.scale_log2);
    const float2 sc2 = make_float2(p.scale, p.scale);
    const int32_t* tpp = p.token_pos ? p.token_pos + b * p.tp_sb + g * p.tp_sg : nullptr;
    while (ct < n_col_tiles && ok) {
      const bool msk = masked(ct);
      const int ct_next = next_active(ct + 1);
      float stat_next = 0.f;
      if (MODE == MODE_DKV) stat_next = fetch_stat(ct_next);  // in flight while this tile is processed
      const int sbuf = s & 1;
      const int cpos0 = p.input_pos + ct * p.npos_col;  // MODE_DKV: first position of the query tile
      for (int h = 0; h < 2 && ok; ++h) {
        const int cc0 = 64 * h + 32 * hh;  // first column of this thread within the 128-column tile
        // MODE_DQ: lane holds the token position of column cc0 + lane (asked for before the wait)
        int v_tp = INT_MAX;
        if (MODE == MODE_DQ && msk) {
          const int jj = ct * 128 + cc0 + lane;
          if (jj < p.L) v_tp = tpp ? tpp[jj] : jj;
        }
        BW_TRACE(2, 2000000 + 2 * s + h);
        if (!mbar_wait_bounded(&xy_full[h], s & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) { ok = false; break; }
        BW_TRACE(2, 2100000 + 2 * s + h);
        tc_fence_after();
        const uint32_t xaddr = tmem_X + lane_base + (uint32_t)(64 * h + 32 * hh);
        const uint32_t yaddr = tmem_Y + lane_base + (uint32_t)(64 * h + 32 * hh);
        uint32_t xr[32], yr[32];
        tmem_ld_32x32b_x32(xaddr, xr);
        tmem_ld_32x32b_x32(yaddr, yr);
        tmem_ld_wait();
        BW_TRACE(2, 2200000 + 2 * s + h);
        // bit e of `hide`: column cc0 + e is not visible to this thread's row
        uint32_t hide = 0;
        bool win_done = false;
        if constexpr (GEN) {
         if (msk && win > 0) {
          // visible iff 0 <= position of the query − token < window
          win_done = true;
          if (MODE == MODE_DQ) {
            uint32_t nm = __ballot_sync(0xffffffffu, v_tp > qpos_min_of(rt) || v_tp <= qpos_max_of(rt) - win);
            while (nm) {
              const int e = __ffs(nm) - 1;
              nm &= nm - 1;
              const int d = row_pos - __shfl_sync(0xffffffffu, v_tp, e);
              hide |= (uint32_t)((uint32_t)d >= (uint32_t)win) << e;
            }
          } else {
            const int upos0 = cpos0 + h * p.u_dp;
            int pp_ = (32 * hh) % p.hnpos;
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int d = upos0 + pp_ - row_tp;
              hide |= (uint32_t)((uint32_t)d >= (uint32_t)win) << e;
              pp_ = pp_ + 1 == p.hnpos ? 0 : pp_ + 1;
            }
          }
         }
        }
        if (msk && !win_done) {
          if (MODE == MODE_DQ) {
            // only columns beyond the first query of the CTA need the per-row comparison
            // (positions broadcast by shuffle)
            uint32_t nm = __ballot_sync(0xffffffffu, v_tp > qpos_min_of(rt));
            while (nm) {
              const int e = __ffs(nm) - 1;
              nm &= nm - 1;
              hide |= (uint32_t)(__shfl_sync(0xffffffffu, v_tp, e) > row_pos) << e;
            }
          } else if (__any_sync(0xffffffffu, row_tp > cpos0)) {
            // column cu of unit h holds position cpos0 + h·hnpos + cu % hnpos (head-major columns)
            const int upos0 = cpos0 + h * p.u_dp;
            if ((p.hnpos & (p.hnpos - 1)) == 0) {
#pragma unroll
              for (int e = 0; e < 32; ++e) hide |= (uint32_t)(row_tp > upos0 + ((32 * hh + e) & (p.hnpos - 1))) << e;
            } else {
              int pp_ = (32 * hh) % p.hnpos;
#pragma unroll
              for (int e = 0; e < 32; ++e) {
                hide |= (uint32_t)(row_tp > upos0 + pp_) << e;
                pp_ = pp_ + 1 == p.hnpos ? 0 : pp_ + 1;
              }
            }
          }
        }
        uint32_t pk[16], dk_[16];
        if (GEN && p.cap_pre != 0.f) {
          // capped scores: the raw score goes through tanh, and dS takes the factor 1 − tanh² of the cap
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float2 nl, nd;
            if (MODE == MODE_DQ) {
              nl = make_float2(row_nlse, row_nlse);
              nd = make_float2(row_ndls, row_ndls);
            } else {
              nl = *reinterpret_cast<const float2*>(stat_nlse + sbuf * 128 + cc0 + e);
              nd = *reinterpret_cast<const float2*>(stat_ndls + sbuf * 128 + cc0 + e);
            }
            const float2 th = make_float2(bw_tanh(__uint_as_float(xr[e]) * p.cap_pre), bw_tanh(__uint_as_float(xr[e + 1]) * p.cap_pre));
            const float2 xx = ffma2(th, make_float2(p.cap_l2, p.cap_l2), nl);
            float2 pp = make_float2(bw_exp2(xx.x), bw_exp2(xx.y));
            if (hide & (1u << e)) pp.x = 0.f;
            if (hide & (1u << (e + 1))) pp.y = 0.f;
            float2 tt = ffma2(make_float2(__uint_as_float(yr[e]), __uint_as_float(yr[e + 1])), sc2, nd);
            tt = fmul2(tt, make_float2(fmaf(-th.x, th.x, 1.f), fmaf(-th.y, th.y, 1.f)));
            const float2 ds = fmul2(pp, tt);
            pk[e >> 1] = pack_bf16x2(pp.x, pp.y);
            dk_[e >> 1] = pack_bf16x2(ds.x, ds.y);
          }
        } else
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float2 nl, nd;
          if (MODE == MODE_DQ) {
            nl = make_float2(row_nlse, row_nlse);
            nd = make_float2(row_ndls, row_ndls);
          } else {
            nl = *reinterpret_cast<const float2*>(stat_nlse + sbuf * 128 + cc0 + e);
            nd = *reinterpret_cast<const float2*>(stat_ndls + sbuf * 128 + cc0 + e);
          }
          const float2 xx = ffma2(make_float2(__uint_as_float(xr[e]), __uint_as_float(xr[e + 1])), c2, nl);
          float2 pp = make_float2(bw_exp2(xx.x), bw_exp2(xx.y));
          if (hide & (1u << e)) pp.x = 0.f;
          if (hide & (1u << (e + 1))) pp.y = 0.f;
          const float2 tt = ffma2(make_float2(__uint_as_float(yr[e]), __uint_as_float(yr[e + 1])), sc2, nd);
          const float2 ds = fmul2(pp, tt);
          pk[e >> 1] = pack_bf16x2(pp.x, pp.y);
          dk_[e >> 1] = pack_bf16x2(ds.x, ds.y);
        }
        BW_TRACE(2, 2300000 + 2 * s + h);
        // P and dS go back into the first 16 columns of the 32 that this thread has just read
        if (MODE == MODE_DKV) tmem_st_32x32b_x16(xaddr, pk);
        tmem_st_32x32b_x16(yaddr, dk_);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pds_full[h]);
        BW_TRACE(2, 2400000 + 2 * s + h);
      }
      if (!ok) break;
      if (MODE == MODE_DKV) {
        // the other buffer was last read during the previous tile, before that tile's barrier
        store_stat(sbuf ^ 1, stat_next);
        if (!group_sync()) { ok = false; break; }
      }
      ++s;
      ct = ct_next;
    }
    // ---- epilogue
    if (ok) ok = mbar_wait_bounded(acc_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL);
    if (ok) {
      tc_fence_after();
      if (MODE == MODE_DQ) {
        __nv_bfloat16* dst = p.dq + (((long long)b * p.H + g * p.gs + hq) * p.T + tq) * HD;
#pragma unroll 1
        for (int c0 = (HD / 2) * hh; c0 < (HD / 2) * (hh + 1); c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_A2 + lane_base + (uint32_t)c0, r);
          tmem_ld_wait();
          if (row_valid) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[8 * u + 0]), __uint_as_float(r[8 * u + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[8 * u + 2]), __uint_as_float(r[8 * u + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[8 * u + 4]), __uint_as_float(r[8 * u + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[8 * u + 6]), __uint_as_float(r[8 * u + 7]));
              *reinterpret_cast<uint4*>(dst + c0 + 8 * u) = o;
            }
          }
        }
      } else {
        const long long off = b * p.dk_sb + g * p.dk_sg + (long long)(rt * 128 + row) * HD;
#pragma unroll 1
        for (int c0 = (HD / 2) * hh; c0 < (HD / 2) * (hh + 1); c0 += 32) {
          uint32_t r1v[32], r2v[32];
          tmem_ld_32x32b_x32(tmem_A1 + lane_base + (uint32_t)c0, r1v);
          tmem_ld_32x32b_x32(tmem_A2 + lane_base + (uint32_t)c0, r2v);
          tmem_ld_wait();
          if (row_valid) {
            // accumulate with vector reductions: no load -> add -> store chain in the epilogue. Every
            // address is touched by this CTA only, so the result does not depend on any order.
            float* dvp = p.dv + off + c0;
            float* dkp = p.dk + off + c0;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dvp + 4 * u), "f"(__uint_as_float(r1v[4 * u])),
                           "f"(__uint_as_float(r1v[4 * u + 1])), "f"(__uint_as_float(r1v[4 * u + 2])),
                           "f"(__uint_as_float(r1v[4 * u + 3]))
                           : "memory");
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dkp + 4 * u), "f"(__uint_as_float(r2v[4 * u])),
                           "f"(__uint_as_float(r2v[4 * u + 1])), "f"(__uint_as_float(r2v[4 * u + 2])),
                           "f"(__uint_as_float(r2v[4 * u + 3]))
                           : "memory");
            }
          }
        }
      }
    } else if (n_active == 0 && MODE == MODE_DQ && row_valid) {
      __nv_bfloat16* dst = p.dq + (((long long)b * p.H + g * p.gs + hq) * p.T + tq) * HD;
      for (int c = (HD / 2) * hh; c < (HD / 2) * (hh + 1); c += 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int bw_make_tmap_4d(CUtensorMap* tm, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1,
                           uint64_t s2, uint64_t s3, uint32_t b0, uint32_t b1, uint32_t b2) {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* pp = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &pp, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return KVB_ERR_DRIVER;
    fn = reinterpret_cast<EncodeTiledFn>(pp);
  }
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1 * 2, s2 * 2, s3 * 2};
  cuuint32_t box[4] = {b0, b1, b2, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? KVB_OK : KVB_ERR_TMAP;
}

// the two launches of one backward call for one (GEN, head size) instantiation: dQ on the side stream, dK / dV on the caller's
template <bool GEN, int HD>
static void bw_launch(const CUtensorMap& tmQ, const CUtensorMap& tmdO, const CUtensorMap& tmKh, const CUtensorMap& tmVh,
                      const BwParams& pq, const CUtensorMap& tmK, const CUtensorMap& tmV, const CUtensorMap& tmQh,
                      const CUtensorMap& tmdOh, const BwParams& p, cudaStream_t side, cudaStream_t s) {
  static kvb::PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(sdpa_bwd_kernel<MODE_DQ, GEN, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwSmem::TOTAL);
    cudaFuncSetAttribute(sdpa_bwd_kernel<MODE_DKV, GEN, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwSmem::TOTAL);
  }
  sdpa_bwd_kernel<MODE_DQ, GEN, HD><<<p.B * p.G * p.nQT, BW_THREADS, BwSmem::TOTAL, side>>>(tmQ, tmdO, tmKh, tmVh, pq);
  sdpa_bwd_kernel<MODE_DKV, GEN, HD><<<p.B * p.G * p.nT, BW_THREADS, BwSmem::TOTAL, s>>>(tmK, tmV, tmQh, tmdOh, p);
}

}  // namespace kvb

extern "C" int kvb_att_tile_minmax(const int32_t* token_pos, int32_t* tmin, int32_t* tmax, int B, int G, int L, long long tp_sb,
                                   long long tp_sg, int tile, void* stream);

// Optional timeline trace (diagnostics): `buf` holds 3 roles x `cap` events x 2 int64 (tag, SM clock),
// filled by CTA 0 of the dQ launch (mode 0) or the dK/dV launch (mode 1) of every later kvb_sdpa_bwd
// call of this process; buf = NULL switches tracing off. Tags: 1e6+ MMA issuer, 2e6+ compute warp;
// the digits below 1e5 count 64-column units.
static long long* g_bw_trace = nullptr;
static int g_bw_trace_cap = 0, g_bw_trace_mode = 0;
extern "C" int kvb_sdpa_bwd_set_trace(void* buf, int cap, int mode) {
  g_bw_trace = reinterpret_cast<long long*>(buf);
  g_bw_trace_cap = buf ? cap : 0;
  g_bw_trace_mode = mode;
  return KVB_OK;
}

static long long bw_round4(long long n) { return (n + 3) / 4 * 4; }
// scratch: tile_min | tile_max (B*G*nT int32 each) | delta (B*H*T fp32) | head-major copy of dO (B*H*T*128 bf16)
extern "C" long long kvb_sdpa_bwd_scratch_bytes(int B, int H, int G, int q_len, int kv_len) {
  const long long nT = (kv_len + 127) / 128;
  return (bw_round4(2LL * B * G * nT) + bw_round4((long long)B * H * q_len)) * 4 + (long long)B * H * q_len * 128 * 2;
}

// head_size: 128 or 64; q_sb, q_sh: batch and head strides of q in elements (0, 0: contiguous (B,H,T,D)); window: sliding
// window in tokens (0: none); softcap: logit soft-capping threshold (0: none), as in the forward.
extern "C" int kvb_sdpa_bwd_ex(const void* q, const void* k, const void* v, const int32_t* token_pos, const void* out,
                               const void* dout, const float* lse, void* dq, float* dk, float* dv, void* scratch, int B, int H,
                               int G, int q_len, int kv_len, int head_size, long long q_sb, long long q_sh, long long k_sb,
                               long long k_sg, long long tp_sb, long long tp_sg, long long dk_sb, long long dk_sg, float scale,
                               int input_pos, int window, float softcap, int* status, void* stream);

extern "C" int kvb_sdpa_bwd(const void* q, const void* k, const void* v, const int32_t* token_pos, const void* out,
                            const void* dout, const float* lse, void* dq, float* dk, float* dv, void* scratch, int B, int H,
                            int G, int q_len, int kv_len, long long k_sb, long long k_sg, long long tp_sb, long long tp_sg,
                            long long dk_sb, long long dk_sg, float scale, int input_pos, int* status, void* stream) {
  return kvb_sdpa_bwd_ex(q, k, v, token_pos, out, dout, lse, dq, dk, dv, scratch, B, H, G, q_len, kv_len, 128, 0, 0, k_sb, k_sg,
                         tp_sb, tp_sg, dk_sb, dk_sg, scale, input_pos, 0, 0.f, status, stream);
}

extern "C" int kvb_sdpa_bwd_ex(const void* q, const void* k, const void* v, const int32_t* token_pos, const void* out,
                               const void* dout, const float* lse, void* dq, float* dk, float* dv, void* scratch, int B, int H,
                               int G, int q_len, int kv_len, int head_size, long long q_sb, long long q_sh, long long k_sb,
                               long long k_sg, long long tp_sb, long long tp_sg, long long dk_sb, long long dk_sg, float scale,
                               int input_pos, int window, float softcap, int* status, void* stream) {
  using namespace kvb;
  if (B <= 0 || H <= 0 || G <= 0 || q_len <= 0 || kv_len <= 0 || H % G) return KVB_ERR_ARG;
  if (window < 0 || softcap < 0.f || (softcap > 0.f && scale <= 0.f)) return KVB_ERR_ARG;
  if (head_size != 128 && head_size != 64) return KVB_ERR_UNSUPPORTED;
  if (q_sh == 0) q_sh = (long long)q_len * head_size;
  if (q_sb == 0) q_sb = (long long)H * q_sh;
  if ((q_sb % 8) || (q_sh % 8) || q_sh < (long long)q_len * head_size) return KVB_ERR_ALIGN;
  const int gs = H / G;
  if (gs > 64) return KVB_ERR_UNSUPPORTED;  // a 64-column unit of the dK/dV launch holds all heads of a group
  if ((k_sb % 8) || (k_sg % 8) || (dk_sb % 4) || (dk_sg % 4)) return KVB_ERR_ALIGN;
  cudaStream_t s = (cudaStream_t)stream;
  BwParams p;
  p.B = B; p.H = H; p.G = G; p.T = q_len; p.L = kv_len;
  p.gs = gs; p.npos = 128 / gs; p.rows_used = p.npos * gs;
  if (gs >= 2 && (gs & (gs - 1)) == 0) {  // half of the heads x all positions of the tile per unit
    p.u_heads = gs / 2; p.u_dh = gs / 2; p.u_dp = 0;
    p.hnpos = 128 / gs; p.npos_col = p.hnpos;
  } else {                                 // all heads x half of the positions of the tile per unit
    p.u_heads = gs; p.u_dh = 0;
    p.hnpos = 64 / gs; p.u_dp = p.hnpos; p.npos_col = 2 * p.hnpos;
  }
  p.cols_used = p.hnpos * p.u_heads;
  p.nCT = (q_len + p.npos_col - 1) / p.npos_col;
  p.nT = (kv_len + 127) / 128;
  p.nQT = (q_len + p.npos - 1) / p.npos;
  p.token_pos = token_pos; p.tp_sb = tp_sb; p.tp_sg = tp_sg;
  p.dk_sb = dk_sb; p.dk_sg = dk_sg;
  int32_t* sc = reinterpret_cast<int32_t*>(scratch);
  int32_t* tmin = sc;
  int32_t* tmax = sc + (long long)B * G * p.nT;
  float* delta = reinterpret_cast<float*>(sc + bw_round4(2LL * B * G * p.nT));
  static const int dout_headmajor = [] {
    const char* e = getenv("KVB200_BWD_DOUT_T");  // "0": read dO in place (diagnostics)
    return (e && e[0] == '0') ? 0 : 1;
  }();
  __nv_bfloat16* dOt = dout_headmajor ? reinterpret_cast<__nv_bfloat16*>(delta + bw_round4((long long)B * H * q_len)) : nullptr;
  p.tile_min = tmin; p.tile_max = tmax; p.lse = lse; p.delta = delta;
  p.dq = (__nv_bfloat16*)dq; p.dk = dk; p.dv = dv;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.input_pos = input_pos; p.status = status;
  p.window = window;
  p.cap_pre = softcap > 0.f ? scale / softcap : 0.f;
  p.cap_l2 = softcap * 1.4426950408889634f;

  // row operands: boxes of npos positions x gs heads (dQ launch) or 128 slots (dK/dV launch); streamed units: boxes of
  // 64 slots (dQ launch) or hnpos positions x gs heads (dK/dV launch)
  CUtensorMap tmQ, tmdO, tmK, tmV, tmQh, tmdOh, tmKh, tmVh;
  int rc;
  const uint64_t qT = (uint64_t)q_len, HT = (uint64_t)H * q_len, hd = (uint64_t)head_size;
  // Q (B,H,T,D): dims (D,T,H,B)
  if ((rc = bw_make_tmap_4d(&tmQ, q, hd, q_len, H, B, hd, (uint64_t)q_sh, (uint64_t)q_sb, 64, p.npos, gs))) return rc;
  if ((rc = bw_make_tmap_4d(&tmQh, q, hd, q_len, H, B, hd, (uint64_t)q_sh, (uint64_t)q_sb, 64, p.hnpos, p.u_heads))) return rc;
  // dO (B,T,H,D) viewed with dims (D,T,H,B): T stride H*D, H stride D
  if (dOt) {  // the head-major copy that the delta kernel leaves: same strides as Q
    if ((rc = bw_make_tmap_4d(&tmdO, dOt, hd, q_len, H, B, hd, qT * hd, HT * hd, 64, p.npos, gs))) return rc;
    if ((rc = bw_make_tmap_4d(&tmdOh, dOt, hd, q_len, H, B, hd, qT * hd, HT * hd, 64, p.hnpos, p.u_heads))) return rc;
  } else {
    if ((rc = bw_make_tmap_4d(&tmdO, dout, hd, q_len, H, B, (uint64_t)H * hd, hd, HT * hd, 64, p.npos, gs))) return rc;
    if ((rc = bw_make_tmap_4d(&tmdOh, dout, hd, q_len, H, B, (uint64_t)H * hd, hd, HT * hd, 64, p.hnpos, p.u_heads))) return rc;
  }
  if ((rc = bw_make_tmap_4d(&tmK, k, hd, kv_len, G, B, hd, k_sg, k_sb, 64, 128, 1))) return rc;
  if ((rc = bw_make_tmap_4d(&tmV, v, hd, kv_len, G, B, hd, k_sg, k_sb, 64, 128, 1))) return rc;
  if ((rc = bw_make_tmap_4d(&tmKh, k, hd, kv_len, G, B, hd, k_sg, k_sb, 64, 64, 1))) return rc;
  if ((rc = bw_make_tmap_4d(&tmVh, v, hd, kv_len, G, B, hd, k_sg, k_sb, 64, 64, 1))) return rc;

  if ((rc = kvb_att_tile_minmax(token_pos, tmin, tmax, B, G, kv_len, tp_sb, tp_sg, 128, stream))) return rc;
  const long long rows = (long long)B * q_len * H;
  if (head_size == 128)
    att_delta_kernel<128><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, delta, dOt, B, q_len, H);
  else
    att_delta_kernel<64><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)out, delta, dOt, B, q_len, H);
  // The two launches are independent (dQ | dK, dV). They run on two streams, forked from and joined
  // back into the caller's stream, so that the tail of one grid (256 CTAs of the dQ launch fill
  // 148 SMs 1.73 times) is filled with CTAs of the other.
  static cudaStream_t side[64] = {nullptr};
  static cudaEvent_t ev_fork[64] = {nullptr}, ev_join[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return KVB_ERR_CUDA;
  if (!side[dev]) {
    if (cudaStreamCreateWithFlags(&side[dev], cudaStreamNonBlocking) != cudaSuccess) return KVB_ERR_CUDA;
    if (cudaEventCreateWithFlags(&ev_fork[dev], cudaEventDisableTiming) != cudaSuccess) return KVB_ERR_CUDA;
    if (cudaEventCreateWithFlags(&ev_join[dev], cudaEventDisableTiming) != cudaSuccess) return KVB_ERR_CUDA;
  }
  cudaEventRecord(ev_fork[dev], s);
  cudaStreamWaitEvent(side[dev], ev_fork[dev], 0);
  BwParams pq = p;
  pq.trace = g_bw_trace_mode == 0 ? g_bw_trace : nullptr; pq.trace_cap = g_bw_trace_cap;
  p.trace = g_bw_trace_mode == 1 ? g_bw_trace : nullptr; p.trace_cap = g_bw_trace_cap;
  // the launch with few long CTAs goes first: the short CTAs of the other one fill its second wave
  const bool gen = window > 0 || softcap > 0.f;
  if (head_size == 128) {
    if (gen) bw_launch<true, 128>(tmQ, tmdO, tmKh, tmVh, pq, tmK, tmV, tmQh, tmdOh, p, side[dev], s);
    else bw_launch<false, 128>(tmQ, tmdO, tmKh, tmVh, pq, tmK, tmV, tmQh, tmdOh, p, side[dev], s);
  } else {
    if (gen) bw_launch<true, 64>(tmQ, tmdO, tmKh, tmVh, pq, tmK, tmV, tmQh, tmdOh, p, side[dev], s);
    else bw_launch<false, 64>(tmQ, tmdO, tmKh, tmVh, pq, tmK, tmV, tmQh, tmdOh, p, side[dev], s);
  }
  cudaEventRecord(ev_join[dev], side[dev]);
  cudaStreamWaitEvent(s, ev_join[dev], 0);
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}
