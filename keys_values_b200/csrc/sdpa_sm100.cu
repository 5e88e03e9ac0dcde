// SDPA forward for sm_100a that also returns the per-KV-slot summed attention
// weights (the H2O score input), with the causal mask taken from token positions.
//
//   out[b, t, h, :]   = softmax_j(scale · q[b,h,t]·k[b,g,j] | token_pos[b,g,j] <= input_pos + t) · v[b,g,:]
//   lse[b, h, t]      = natural-log normaliser of that softmax
//   weights[b, g, j]  = (1 / (H/G)) · sum over t and over the H/G heads of group g of the softmax weight of slot j
//
// Design (bf16, head size 128):
//   * CTA tile = 128 query rows = (128 / gs) consecutive positions x gs heads of one KV
//     group (gs = H/G), so every K/V tile is loaded once per group, not once per head.
//   * S = Q K^T (M=128, N=64) and O += P V (M=128, N=128) run on tcgen05.mma. Q is moved once
//     from shared memory into TMEM and is the A operand of every QK MMA from there, so that
//     those MMAs read only K from shared memory (operand traffic from shared memory, 128 B per
//     clock, is what bounds tcgen05 at these tile sizes). S has one TMEM buffer: the softmax
//     warps pull a tile into registers and hand the buffer back at once, so the next QK runs
//     during their arithmetic. O stays in TMEM. K tiles of 64 slots arrive by TMA into a
//     4-stage ring, V tiles into a 2-stage ring (128B swizzle; no multicast). V is consumed as
//     an MN-major B operand.
//   * A CTA uses 112.5 KB of shared memory and 256 TMEM columns, so two CTAs share an SM:
//     while one waits on its MMA -> softmax -> MMA chain the other one issues.
//   * Two sweeps over the KV tiles: sweep 1 computes the exact row log-sum-exp (online
//     max / sum), sweep 2 recomputes S, forms the already-normalised P = exp2(S·c − lse),
//     accumulates O without any rescaling and takes the column sums of P. The column
//     sums of a tile are complete once its P tile is written, so they are stored as
//     deterministic per-(query tile) partials and reduced by a second small kernel:
//     no atomics, hence run-to-run identical eviction decisions.
//   * KV tiles whose smallest token position lies beyond the last query of the CTA are
//     skipped by every role; tiles that contain no position beyond the first query of
//     the CTA take the mask-free path. In a masked tile only the columns whose token lies
//     beyond the first query need a per-row comparison; their positions travel by warp
//     shuffle and end up as a 64-bit mask per row, without shared memory or block barriers.
//   * warp 0 = TMA producer, warp 1 = MMA issuer / TMEM owner, then the softmax + epilogue warps.
//     Two instantiations: 4 softmax warps (a thread owns a query row = its TMEM lane and all 64
//     columns of a tile; used for plain causal attention) and 8 softmax warps (two per TMEM lane
//     quarter, 32 columns per thread; used over an evicting cache, where most tiles need masks).
//
// Replaces FlashInfer prefill + Triton score-sum + K/V reordering + query padding of the
// reference (keys_values/attention/flashinfer_wrapper.py:51-273, :367-510,
// csrc/kernels/sdpa_prefill.cu, attention/sdpa_wrapper.py:66-432).
#include <cuda.h>
#include <limits.h>

#include "common.cuh"
#include "kvb200.h"

namespace kvb {

int make_tmap_2d_bf16(CUtensorMap* tm, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);

constexpr int ATT_BM = 128;   // query rows per CTA
constexpr int ATT_BN = 64;    // KV slots per tile
constexpr int ATT_D = 128;    // head size
// TMA warp + MMA warp + SW softmax warps; two CTAs per SM. SW = 4: a thread owns one query row and all
// 64 columns of a tile (best when few tiles need masks: prefill, plain causal attention); SW = 8: two
// warps per TMEM lane quarter, 32 columns per thread (best when most tiles hold tokens of the current
// chunk, as in training over an evicting cache, where building the masks dominates the chain).
constexpr int att_threads(int sw) { return 64 + 32 * sw; }
constexpr int ATT_Q_BYTES = ATT_BM * ATT_D * 2;    // 32 KB: two 64-feature chunks of [128 rows x 128 B]
constexpr int ATT_KV_BYTES = ATT_BN * ATT_D * 2;   // 16 KB: two 64-feature chunks of [64 rows x 128 B]
constexpr int ATT_P_BYTES = ATT_BM * ATT_BN * 2;   // 16 KB: one 64-column chunk of [128 rows x 128 B]
constexpr int ATT_TMEM_COLS = 256;                 // Q as bf16 pairs (64 columns) | S (64) | O (128)
constexpr int ATT_KSTAGES = 4;

// Shared memory of one CTA: 112.5 KB, so that two CTAs fit into the 228 KB of an SM (each
// CTA also costs 1 KB of system reserve). The dynamic shared memory window must be 1024-byte
// aligned for the 128B-swizzled tiles; the kernel checks this and reports instead of running.
struct AttSmem {
  static constexpr int K = 0;                              // ring of ATT_KSTAGES K tiles
  static constexpr int Q = K + 2 * ATT_KV_BYTES;           // Q lands in K stages 2, 3 and moves on to TMEM
  static constexpr int V = K + ATT_KSTAGES * ATT_KV_BYTES; // ring of 2 V tiles
  static constexpr int P = V + 2 * ATT_KV_BYTES;
  static constexpr int TF = P + ATT_P_BYTES;   // 2 bits per KV tile (active, masked) for the first 1024 tiles
  static constexpr int BAR = TF + 256;
  static constexpr int TOTAL = BAR + 256;
};
static_assert(ATT_Q_BYTES == 2 * ATT_KV_BYTES, "Q must fit into two K stages");

struct AttParams {
  const int32_t* token_pos;  // (B,G,L) with strides tp_sb, tp_sg, or nullptr (slot j holds token j)
  const int32_t* tile_min;   // (B,G,nT)
  const int32_t* tile_max;   // (B,G,nT)
  __nv_bfloat16* out;        // (B,T,H,D)
  float* lse;                // (B,H,T)
  float* wpart;              // (B,G,4*nQT,L) or nullptr
  int B, H, G, T, L, nT, nQT, gs, npos;
  long long tp_sb, tp_sg;
  float scale_log2;          // scale * log2(e)
  int input_pos;
  int* status;
  long long* trace;          // optional timeline of CTA 0: per role trace_cap (tag, clock) pairs
  int trace_cap;
};

// Timeline event of one role (0 producer, 1 MMA issuer, 2 first softmax warp) of CTA 0.
#define ATT_TRACE(role, tag)                                              \
  do {                                                                    \
    if (p.trace && blockIdx.x == 0 && tr_n < p.trace_cap) {               \
      p.trace[((role) * p.trace_cap + tr_n) * 2] = (long long)(tag);      \
      p.trace[((role) * p.trace_cap + tr_n) * 2 + 1] = clock64();         \
      ++tr_n;                                                             \
    }                                                                     \
  } while (0)

__global__ void att_tile_minmax_kernel(const int32_t* __restrict__ tp, int32_t* __restrict__ tmin, int32_t* __restrict__ tmax, int G,
                                       int L, int nT, long long tp_sb, long long tp_sg) {
  // one block per tile; blockDim.x = tile size (64 or 128)
  const int tile = blockDim.x;
  const int t = blockIdx.x % nT;
  const int bg = blockIdx.x / nT;
  const int b = bg / G, g = bg % G;
  const int j = t * tile + threadIdx.x;
  int lo = INT_MAX, hi = INT_MIN;
  if (j < L) {
    const int v = tp ? tp[b * tp_sb + g * tp_sg + j] : j;
    lo = hi = v;
  }
  for (int o = 16; o > 0; o >>= 1) {
    lo = min(lo, __shfl_xor_sync(0xffffffffu, lo, o));
    hi = max(hi, __shfl_xor_sync(0xffffffffu, hi, o));
  }
  __shared__ int slo[4], shi[4];
  if ((threadIdx.x & 31) == 0) {
    slo[threadIdx.x >> 5] = lo;
    shi[threadIdx.x >> 5] = hi;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < tile / 32; ++w) {
      lo = min(lo, slo[w]);
      hi = max(hi, shi[w]);
    }
    if ((t + 1) * tile > L) hi = INT_MAX;  // ragged last tile always takes the masked path
    tmin[blockIdx.x] = lo;
    tmax[blockIdx.x] = hi;
  }
}

// weights[b,g,j] = inv_gs * sum_qt wpart[b,g,qt,j]
__global__ void att_reduce_weights_kernel(const float* __restrict__ wpart, float* __restrict__ weights, int nQT, int L, float inv_gs) {
  const long long bg = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= L) return;
  const float* p = wpart + bg * nQT * (long long)L + j;
  float s = 0.f;
  for (int q = 0; q < nQT; ++q) s += p[(long long)q * L];
  weights[bg * L + j] = s * inv_gs;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int SW>
__global__ void __launch_bounds__(att_threads(SW), 2)
sdpa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // swizzled tiles need a 1024-byte aligned window: report, do not run
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, STATUS_TIMEOUT_MISC);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttSmem::BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;    // [4]
  uint64_t* k_empty = bars + 5;   // [4]
  uint64_t* v_full = bars + 9;    // [2]
  uint64_t* v_empty = bars + 11;  // [2]
  uint64_t* s_full = bars + 13;
  uint64_t* s_empty = bars + 14;
  uint64_t* p_full = bars + 15;
  uint64_t* p_empty = bars + 16;
  uint64_t* o_full = bars + 17;
  uint64_t* q_ready = bars + 18;  // Q has been moved from shared memory to TMEM
  uint64_t* grp_bar = bars + 19;  // barrier among the 256 softmax threads (bounded, unlike bar.sync)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // block -> (query tile, group, batch); query tiles fastest so that co-resident CTAs share K/V in L2
  const int qt = blockIdx.x % p.nQT;
  const int g = (blockIdx.x / p.nQT) % p.G;
  const int b = blockIdx.x / (p.nQT * p.G);
  const int t0 = qt * p.npos;
  const int qpos_min = p.input_pos + t0;
  const int qpos_max = p.input_pos + min(t0 + p.npos, p.T) - 1;
  const int32_t* tmin = p.tile_min + ((long long)b * p.G + g) * p.nT;
  const int32_t* tmax = p.tile_max + ((long long)b * p.G + g) * p.nT;

  // (active, masked) bits of the KV tiles for this query tile, so that no role reads global
  // memory inside its tile loop
  uint32_t* tflags = reinterpret_cast<uint32_t*>(smem + AttSmem::TF);
  constexpr int TF_TILES = 1024;
  for (int w = threadIdx.x; w < TF_TILES / 16; w += att_threads(SW)) {
    uint32_t bits = 0;
#pragma unroll 4
    for (int i = 0; i < 16; ++i) {
      const int t = w * 16 + i;
      if (t < p.nT) bits |= ((uint32_t)(tmin[t] <= qpos_max) | ((uint32_t)(tmax[t] > qpos_min) << 1)) << (2 * i);
    }
    tflags[w] = bits;
  }
  // bit 0: active, bit 1: masked. Shared memory is slow to reach while the tensor core streams its
  // operands from it, so each role keeps the word of 16 tiles in a register.
  auto tile_bits = [&](int t, uint32_t& fw, int& fwi) -> uint32_t {
    if (t >= TF_TILES) return (uint32_t)(tmin[t] <= qpos_max) | ((uint32_t)(tmax[t] > qpos_min) << 1);
    if ((t >> 4) != fwi) {
      fwi = t >> 4;
      fw = tflags[fwi];
    }
    return (fw >> ((t & 15) * 2)) & 3u;
  };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < ATT_KSTAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, SW);
    mbar_init(p_full, SW);
    mbar_init(p_empty, 1);
    mbar_init(o_full, 1);
    mbar_init(q_ready, SW);
    mbar_init(grp_bar, 32 * SW);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, ATT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Q stays in TMEM as the A operand of S = Q K^T, so that each QK MMA reads only K from shared
  // memory. S has one buffer: the softmax warps pull a tile into registers and hand the buffer
  // back at once, so that the next QK runs during their arithmetic.
  const uint32_t tmem_Q = tmem_base;           // columns [0,64): 128 features as bf16 pairs
  const uint32_t tmem_S = tmem_base + 64;      // columns [64,128)
  const uint32_t tmem_O = tmem_base + 128;     // columns [128,256)

  int n_active = 0;
  for (int w = 0; w < TF_TILES / 16; ++w) n_active += __popc(tflags[w] & 0x55555555u);
  for (int t = TF_TILES; t < p.nT; ++t) n_active += (tmin[t] <= qpos_max);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && n_active > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, ATT_Q_BYTES);
      tma_load_4d(smem + AttSmem::Q, &tmQ, q_full, 0, t0, g * p.gs, b);
      tma_load_4d(smem + AttSmem::Q + ATT_Q_BYTES / 2, &tmQ, q_full, 64, t0, g * p.gs, b);
      uint32_t i = 0, j = 0;
      bool ok = true;
      int tr_n = 0;
      uint32_t fw = 0;
      int fwi = -1;
      for (int sweep = 0; sweep < 2 && ok; ++sweep) {
        for (int t = 0; t < p.nT && ok; ++t) {
          if (!(tile_bits(t, fw, fwi) & 1u)) continue;
          const int ks = i % ATT_KSTAGES;
          // stages 2 and 3 first hold Q
          if (i == 2 && !mbar_wait_bounded(q_ready, 0, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) { ok = false; break; }
          if (!mbar_wait_bounded(&k_empty[ks], ((i / ATT_KSTAGES) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) { ok = false; break; }
          ATT_TRACE(0, 100000 + sweep * 50000 + t);
          uint8_t* kd = smem + AttSmem::K + ks * ATT_KV_BYTES;
          mbar_expect_tx(&k_full[ks], ATT_KV_BYTES);
          tma_load_4d(kd, &tmK, &k_full[ks], 0, t * ATT_BN, g, b);
          tma_load_4d(kd + ATT_KV_BYTES / 2, &tmK, &k_full[ks], 64, t * ATT_BN, g, b);
          ++i;
          if (sweep == 1) {
            const int vs = j & 1;
            if (!mbar_wait_bounded(&v_empty[vs], ((j >> 1) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) { ok = false; break; }
            uint8_t* vd = smem + AttSmem::V + vs * ATT_KV_BYTES;
            mbar_expect_tx(&v_full[vs], ATT_KV_BYTES);
            tma_load_4d(vd, &tmV, &v_full[vs], 0, t * ATT_BN, g, b);
            tma_load_4d(vd + ATT_KV_BYTES / 2, &tmV, &v_full[vs], 64, t * ATT_BN, g, b);
            ++j;
          }
        }
      }
      if (!ok) {  // let copies in flight land before the CTA's shared memory is released
        long long c0 = clock64();
        while (clock64() - c0 < 2000000LL) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_active > 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(ATT_BM, ATT_BN, 0, 0);  // Q, K both K-major
      constexpr uint32_t idesc_pv = make_idesc_bf16(ATT_BM, ATT_D, 0, 1);   // P K-major, V MN-major
      const uint32_t p_addr = smem_u32(smem + AttSmem::P);
      bool ok = mbar_wait_bounded(q_ready, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL);
      tc_fence_after();
      uint32_t i = 0, j = 0;
      int tr_n = 0;
      auto issue_qk = [&]() -> bool {
        const int ks = i % ATT_KSTAGES;
        ATT_TRACE(1, 1000000 + i);
        if (!mbar_wait_bounded(&k_full[ks], (i / ATT_KSTAGES) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL)) return false;
        ATT_TRACE(1, 1100000 + i);
        if (!mbar_wait_bounded(s_empty, (i & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY)) return false;
        ATT_TRACE(1, 1200000 + i);
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + AttSmem::K + ks * ATT_KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // 16 features per step: 8 TMEM columns of Q; chunk kk/4 of K, 32 bytes per step inside the swizzled row
          const uint32_t k_off = (uint32_t)((kk >> 2) * (ATT_KV_BYTES / 2) + (kk & 3) * 32);
          umma_f16_ts(tmem_S, tmem_Q + 8 * kk, make_smem_desc_sw128(k_addr + k_off, 16, 1024), idesc_qk, kk != 0);
        }
        umma_commit(&k_empty[ks]);
        umma_commit(s_full);
        ATT_TRACE(1, 1300000 + i);
        ++i;
        return true;
      };
      auto issue_pv = [&]() -> bool {
        const int vs = j & 1;
        ATT_TRACE(1, 2000000 + j);
        // V first: it does not depend on the softmax, so only the wait for P is on the critical path
        if (!mbar_wait_bounded(&v_full[vs], (j >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL)) return false;
        ATT_TRACE(1, 2100000 + j);
        if (!mbar_wait_bounded(p_full, j & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL)) return false;
        ATT_TRACE(1, 2200000 + j);
        tc_fence_after();
        const uint32_t v_addr = smem_u32(smem + AttSmem::V + vs * ATT_KV_BYTES);
#pragma unroll
        for (int kk = 0; kk < ATT_BN / 16; ++kk) {
          // A = P: K-major, 16 kv columns (32 B) per step inside the single 64-column chunk
          const uint32_t a_off = (uint32_t)(kk * 32);
          // B = V: MN-major; 16 kv rows per step (2048 B); the two 64-wide d chunks are LBO apart
          const uint32_t b_off = (uint32_t)(kk * 16 * 128);
          umma_f16_ss(tmem_O, make_smem_desc_sw128(p_addr + a_off, 16, 1024),
                      make_smem_desc_sw128(v_addr + b_off, ATT_KV_BYTES / 2, 1024), idesc_pv, (j | kk) != 0);
        }
        umma_commit(&v_empty[vs]);
        umma_commit(p_empty);
        ATT_TRACE(1, 2300000 + j);
        ++j;
        return true;
      };
      // sweep 1: S only
      uint32_t fw = 0;
      int fwi = -1;
      for (int t = 0; t < p.nT && ok; ++t) {
        if (!(tile_bits(t, fw, fwi) & 1u)) continue;
        ok = issue_qk();
      }
      // sweep 2: QK of the next tile is issued before PV of the current one
      bool pending = false;
      for (int t = 0; t < p.nT && ok; ++t) {
        if (!(tile_bits(t, fw, fwi) & 1u)) continue;
        ok = issue_qk();
        if (ok && pending) ok = issue_pv();
        pending = true;
      }
      if (ok && pending) ok = issue_pv();
      if (ok) umma_commit(o_full);
    }
  } else {
    // ------------------------------------------------- softmax + epilogue warps
    // 8 warps: two per TMEM lane quarter. A thread owns one query row (its TMEM lane) and 32 of the
    // 64 columns of every KV tile (hh = which half), so the serial chain of a tile (barrier wait,
    // TMEM load, exp2, P store, column sums) is half as long per warp and four warps per SM
    // sub-partition (two CTAs) fill each other's latencies.
    const int quarter = warp & 3;
    const int hh = SW == 8 ? (warp - 2) >> 2 : 0;
    constexpr int NC = SW == 8 ? ATT_BN / 2 : ATT_BN;  // columns per thread
    constexpr int NW = NC / 32;                       // 32-column words per thread
    const int row = quarter * 32 + lane;          // TMEM lane = query row of the tile
    const int hq = row / p.npos;                  // head within the group
    const int pl = row % p.npos;                  // position within the tile
    const int tq = t0 + pl;
    const bool row_valid = tq < p.T;
    const int my_pos = p.input_pos + tq;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float c = p.scale_log2;
    const float2 c2 = make_float2(c, c);
    bool ok = n_active > 0;
    uint32_t i = 0, j = 0;
    float m = -1e30f, l = 0.f;
    int tr_n = (warp == 2 && lane == 0) ? 0 : (1 << 30);  // only the first softmax warp records
    uint32_t fw = 0;
    int fwi = -1;
    // Token positions of a tile: lane holds columns lane and lane + 32 (INT_MAX beyond the cache).
    // The positions of the next tile are fetched one tile ahead.
    const int32_t* tpp = p.token_pos ? p.token_pos + b * p.tp_sb + g * p.tp_sg : nullptr;
    // lane holds columns NC·hh + 32·w + lane (w < NW) of the tile
    auto fetch_tp = [&](int t, int (&v)[NW]) {
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        const int j0 = t * ATT_BN + NC * hh + 32 * w + lane;
        v[w] = j0 < p.L ? (tpp ? tpp[j0] : j0) : INT_MAX;
      }
    };
    int pf[NW], pf_t = -1;
#pragma unroll
    for (int w = 0; w < NW; ++w) pf[w] = INT_MAX;
    // Mask bits of this thread's row for a masked tile (bit e of word w: column 32·w + e of the thread's
    // columns is hidden). Only columns whose token lies beyond the first query of the CTA need the
    // per-row comparison; their positions are broadcast by shuffle, so no shared memory is involved.
    auto row_mask = [&](const int (&v)[NW], uint32_t (&mk)[NW]) {
#pragma unroll
      for (int w = 0; w < NW; ++w) {
        uint32_t n0 = __ballot_sync(0xffffffffu, v[w] > qpos_min);
        mk[w] = 0;
        while (n0) {
          const int e = __ffs(n0) - 1;
          n0 &= n0 - 1;
          mk[w] |= (uint32_t)(__shfl_sync(0xffffffffu, v[w], e) > my_pos) << e;
        }
      }
    };
    uint32_t grp_phase = 0;
    auto group_sync = [&]() -> bool {  // all 256 softmax threads; false if it ran into the wait limit
      mbar_arrive(grp_bar);
      const bool done = mbar_wait_bounded(grp_bar, grp_phase, abort_flag, p.status, STATUS_TIMEOUT_MISC);
      grp_phase ^= 1;
      return done;
    };
    // column-sum partials: slot (4·qt + warp quarter) of wpart (B,G,4·nQT,L). A warp sums the 32
    // rows x 32 columns that it wrote itself, so the column sums need no barrier among the warps.
    float* wbase = p.wpart ? p.wpart + ((((long long)b * p.G + g) * (4 * p.nQT) + 4 * qt + quarter) * p.L) : nullptr;
    if (n_active == 0 && wbase) {
      for (int jj = NC * hh + lane; jj < p.L; jj += 32)
        if ((jj % ATT_BN) / NC == hh) wbase[jj] = 0.f;
    }
    const uint32_t NEG_INF_BITS = 0xff800000u;

    // ---- Q: shared memory -> registers -> TMEM (row = lane; feature pair f/2 = column)
    if (ok) ok = mbar_wait_bounded(q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL);
    if (ok) {
#pragma unroll
      for (int ch = (SW == 8 ? hh : 0); ch < (SW == 8 ? hh + 1 : 2); ++ch) {  // feature chunk(s) that this warp moves
        const uint8_t* src = smem + AttSmem::Q + ch * (ATT_Q_BYTES / 2);
        uint32_t w[32];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const uint4 q4 = *reinterpret_cast<const uint4*>(src + sw128_offset(row, u));
          w[4 * u] = q4.x; w[4 * u + 1] = q4.y; w[4 * u + 2] = q4.z; w[4 * u + 3] = q4.w;
        }
        tmem_st_32x32b_x16(tmem_Q + lane_base + (uint32_t)(32 * ch), w);
        tmem_st_32x32b_x16(tmem_Q + lane_base + (uint32_t)(32 * ch + 16), w + 16);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_ready);
    }

    // ---- sweep 1: exact row max and sum over this thread's 32 columns of every tile
    for (int t = 0; t < p.nT && ok; ++t) {
      const uint32_t tb = tile_bits(t, fw, fwi);
      if (!(tb & 1u)) continue;
      const bool masked = (tb & 2u) != 0;
      int v0[NW];
#pragma unroll
      for (int w = 0; w < NW; ++w) v0[w] = pf[w];
      if (masked && pf_t != t) fetch_tp(t, v0);
      if (t + 1 < p.nT) {
        fetch_tp(t + 1, pf);
        pf_t = t + 1;
      }
      ATT_TRACE(2, 3000000 + i);
      if (!mbar_wait_bounded(s_full, i & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      ATT_TRACE(2, 3100000 + i);
      tc_fence_after();
      uint32_t r[NC];
#pragma unroll
      for (int w = 0; w < NW; ++w) tmem_ld_32x32b_x32(tmem_S + lane_base + (uint32_t)(NC * hh + 32 * w), r + 32 * w);
      tmem_ld_wait();
      ATT_TRACE(2, 3200000 + i);
      // the tile is in registers: hand the S buffer back before the arithmetic
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty);
      ++i;
      if (masked) {
        uint32_t mk[NW];
        row_mask(v0, mk);
#pragma unroll
        for (int e = 0; e < NC; ++e)
          if (mk[e >> 5] & (1u << (e & 31))) r[e] = NEG_INF_BITS;
      }
      // max of the raw scores (the scale is positive): four independent chains of 3-input max
      float a0 = -INFINITY, a1 = -INFINITY, a2 = -INFINITY, a3 = -INFINITY;
#pragma unroll
      for (int e = 0; e < NC; e += 8) {
        a0 = fmax3(a0, __uint_as_float(r[e]), __uint_as_float(r[e + 1]));
        a1 = fmax3(a1, __uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
        a2 = fmax3(a2, __uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
        a3 = fmax3(a3, __uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
      }
      const float m_new = fmaxf(m, fmax3(a0, a1, fmaxf(a2, a3)) * c);
      const float2 neg_m2 = make_float2(-m_new, -m_new);
      float2 s0 = make_float2(0.f, 0.f), s1 = s0, s2 = s0, s3 = s0;
#pragma unroll
      for (int e = 0; e < NC; e += 8) {
        float2 x0 = ffma2(make_float2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), c2, neg_m2);
        float2 x1 = ffma2(make_float2(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3])), c2, neg_m2);
        float2 x2 = ffma2(make_float2(__uint_as_float(r[e + 4]), __uint_as_float(r[e + 5])), c2, neg_m2);
        float2 x3 = ffma2(make_float2(__uint_as_float(r[e + 6]), __uint_as_float(r[e + 7])), c2, neg_m2);
        s0 = fadd2(s0, make_float2(fast_exp2(x0.x), fast_exp2(x0.y)));
        s1 = fadd2(s1, make_float2(fast_exp2(x1.x), fast_exp2(x1.y)));
        s2 = fadd2(s2, make_float2(fast_exp2(x2.x), fast_exp2(x2.y)));
        s3 = fadd2(s3, make_float2(fast_exp2(x3.x), fast_exp2(x3.y)));
      }
      s0 = fadd2(fadd2(s0, s1), fadd2(s2, s3));
      l = l * fast_exp2(m - m_new) + (s0.x + s0.y);
      m = m_new;
      ATT_TRACE(2, 3300000 + i);
    }
    if (SW == 8) {
      // merge (m, l) of the two column halves of a row through the P area, which is idle in sweep 1
      float2* ml_x = reinterpret_cast<float2*>(smem + AttSmem::P);
      ml_x[hh * ATT_BM + row] = make_float2(m, l);
      if (ok && !group_sync()) ok = false;
      if (ok) {
        const float2 o = ml_x[(hh ^ 1) * ATT_BM + row];
        const float mm = fmaxf(m, o.x);
        l = l * fast_exp2(m - mm) + o.y * fast_exp2(o.x - mm);
        m = mm;
        if (!group_sync()) ok = false;  // everyone has read the exchange area before P tiles land in it
      }
    }
    const float lse2 = l > 0.f ? m + log2f(l) : INFINITY;
    // rows beyond the end of the query get P = 0 (their Q rows are zero-filled, so S = 0)
    const float nl = row_valid ? -lse2 : -INFINITY;
    const float2 neg_lse2 = make_float2(nl, nl);

    // ---- sweep 2: P = exp2(S·c − lse), O += P V, column sums of P
    uint8_t* Ps = smem + AttSmem::P;
    for (int t = 0; t < p.nT && ok; ++t) {
      float* wdst = wbase ? wbase + (long long)t * ATT_BN + NC * hh : nullptr;
      const uint32_t tb = tile_bits(t, fw, fwi);
      if (!(tb & 1u)) {
        if (wdst) {
#pragma unroll
          for (int w = 0; w < NW; ++w)
            if (t * ATT_BN + NC * hh + 32 * w + lane < p.L) wdst[32 * w + lane] = 0.f;
        }
        continue;
      }
      const bool masked = (tb & 2u) != 0;
      int v0[NW];
#pragma unroll
      for (int w = 0; w < NW; ++w) v0[w] = pf[w];
      if (masked && pf_t != t) fetch_tp(t, v0);
      if (t + 1 < p.nT) {
        fetch_tp(t + 1, pf);
        pf_t = t + 1;
      }
      ATT_TRACE(2, 4000000 + i);
      if (!mbar_wait_bounded(s_full, i & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) { ok = false; break; }
      ATT_TRACE(2, 4100000 + i);
      tc_fence_after();
      uint32_t r[NC];
#pragma unroll
      for (int w = 0; w < NW; ++w) tmem_ld_32x32b_x32(tmem_S + lane_base + (uint32_t)(NC * hh + 32 * w), r + 32 * w);
      tmem_ld_wait();
      ATT_TRACE(2, 4200000 + i);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty);
      ++i;
      if (masked) {
        uint32_t mk[NW];
        row_mask(v0, mk);
#pragma unroll
        for (int e = 0; e < NC; ++e)
          if (mk[e >> 5] & (1u << (e & 31))) r[e] = NEG_INF_BITS;
      }
      uint32_t pk[NC / 2];
#pragma unroll
      for (int e = 0; e < NC; e += 2) {
        const float2 x = ffma2(make_float2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), c2, neg_lse2);
        pk[e >> 1] = pack_bf16x2(fast_exp2(x.x), fast_exp2(x.y));
      }
      // the PV MMA of the previous tile must have finished reading P
      ATT_TRACE(2, 4300000 + i);
      if (!mbar_wait_bounded(p_empty, (j & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_MISC)) { ok = false; break; }
      ATT_TRACE(2, 4400000 + i);
#pragma unroll
      for (int u = 0; u < NC / 8; ++u) {
        uint4 val = make_uint4(pk[4 * u], pk[4 * u + 1], pk[4 * u + 2], pk[4 * u + 3]);
        *reinterpret_cast<uint4*>(Ps + sw128_offset(row, (NC / 8) * hh + u)) = val;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      ATT_TRACE(2, 4500000 + i);
      ++j;
      // column sums over this warp's 32 rows x NC columns of the P tile (as rounded to bf16):
      // lane -> (column pair lane % (NC/2), part of the rows lane / (NC/2))
      if (wdst) {
        constexpr int NP = NC / 2;       // column pairs of this warp
        constexpr int RPL = 32 / (32 / NP);  // rows per lane
        float2 ca = make_float2(0.f, 0.f), cb = ca;
        const int cp = lane % NP, rh = lane / NP;
        const uint32_t coff = (uint32_t)((cp & 3) * 4);
        const int cu = (NC / 8) * hh + (cp >> 2);
#pragma unroll
        for (int rr = 0; rr < RPL; rr += 2) {
          const int r0 = quarter * 32 + rh * RPL + rr;
          const uint32_t w0 = *reinterpret_cast<const uint32_t*>(Ps + sw128_offset(r0, cu) + coff);
          const uint32_t w1 = *reinterpret_cast<const uint32_t*>(Ps + sw128_offset(r0 + 1, cu) + coff);
          ca = fadd2(ca, make_float2(__uint_as_float(w0 << 16), __uint_as_float(w0 & 0xffff0000u)));
          cb = fadd2(cb, make_float2(__uint_as_float(w1 << 16), __uint_as_float(w1 & 0xffff0000u)));
        }
        ca = fadd2(ca, cb);
        if (NP < 32) {
          ca.x += __shfl_xor_sync(0xffffffffu, ca.x, 16);
          ca.y += __shfl_xor_sync(0xffffffffu, ca.y, 16);
        }
        if (rh == 0) {
          if (t * ATT_BN + NC * hh + 2 * cp < p.L) wdst[2 * cp] = ca.x;
          if (t * ATT_BN + NC * hh + 2 * cp + 1 < p.L) wdst[2 * cp + 1] = ca.y;
        }
        __syncwarp();  // all lanes have read the warp's rows before the next tile overwrites them
      }
      ATT_TRACE(2, 4600000 + i);
    }

    // ---- epilogue: O (already normalised) -> bf16 -> out; lse
    if (ok) ok = mbar_wait_bounded(o_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL);
    if (ok || n_active == 0) {
      tc_fence_after();
      __nv_bfloat16* dst = p.out + (((long long)b * p.T + tq) * p.H + (g * p.gs + hq)) * ATT_D;
#pragma unroll 1
      for (int c0 = (ATT_D / (SW / 4)) * hh; c0 < (ATT_D / (SW / 4)) * (hh + 1); c0 += 32) {
        uint32_t r[32];
        if (n_active > 0) {
          tmem_ld_32x32b_x32(tmem_O + lane_base + (uint32_t)c0, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = 0;
        }
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
      if (hh == 0 && row_valid && p.lse) p.lse[((long long)b * p.H + (g * p.gs + hq)) * p.T + tq] = lse2 * 0.6931471805599453f;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, ATT_TMEM_COLS);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int make_tmap_4d_bf16(CUtensorMap* tm, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1,
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

}  // namespace kvb

// Per-tile min/max of the token positions for tiles of `tile` slots (64 or 128): (B,G,nT) each.
extern "C" int kvb_att_tile_minmax(const int32_t* token_pos, int32_t* tmin, int32_t* tmax, int B, int G, int L, long long tp_sb,
                                   long long tp_sg, int tile, void* stream) {
  if (tile != 64 && tile != 128) return KVB_ERR_ARG;
  const int nT = (L + tile - 1) / tile;
  kvb::att_tile_minmax_kernel<<<B * G * nT, tile, 0, (cudaStream_t)stream>>>(token_pos, tmin, tmax, G, L, nT, tp_sb, tp_sg);
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

// Optional timeline trace of the forward kernel (diagnostics): `buf` holds 3 roles x `cap` events
// x 2 int64 (tag, SM clock) and is filled by CTA 0 of every later kvb_sdpa_fwd launch of this
// process; buf = NULL switches tracing off. Tags: 1e5 producer, 1e6+ QK issue, 2e6+ PV issue,
// 3e6+ / 4e6+ softmax of sweep 1 / 2; the digits below 1e5 count tiles.
static long long* g_att_trace = nullptr;
static int g_att_trace_cap = 0;
extern "C" int kvb_sdpa_fwd_set_trace(void* buf, int cap) {
  g_att_trace = reinterpret_cast<long long*>(buf);
  g_att_trace_cap = buf ? cap : 0;
  return KVB_OK;
}

// Scratch layout (int32 words), provided by the caller:
//   tile_min (B*G*nT) | tile_max (B*G*nT) | wpart (B*G*4*nQT*L floats, only if weights != NULL)
extern "C" long long kvb_sdpa_fwd_scratch_bytes(int B, int H, int G, int q_len, int kv_len, int want_weights) {
  if (G <= 0 || H % G) return -1;
  const int gs = H / G;
  const long long nT = (kv_len + kvb::ATT_BN - 1) / kvb::ATT_BN;
  const long long npos = 128 / gs;
  const long long nQT = (q_len + npos - 1) / npos;
  long long words = 2LL * B * G * nT;
  if (want_weights) words += 4LL * B * G * nQT * kv_len;
  return words * 4;
}

extern "C" int kvb_sdpa_fwd(const void* q, const void* k, const void* v, const int32_t* token_pos, void* out, float* lse,
                            float* weights, void* scratch, int B, int H, int G, int q_len, int kv_len, long long k_sb,
                            long long k_sg, long long tp_sb, long long tp_sg, float scale, int input_pos, int* status,
                            void* stream) {
  using namespace kvb;
  if (B <= 0 || H <= 0 || G <= 0 || q_len <= 0 || kv_len <= 0 || H % G) return KVB_ERR_ARG;
  const int gs = H / G;
  if (gs > 128 || (gs & (gs - 1))) return KVB_ERR_UNSUPPORTED;
  if ((k_sb % 8) || (k_sg % 8)) return KVB_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return KVB_ERR_ALIGN;
  cudaStream_t s = (cudaStream_t)stream;
  AttParams p;
  p.B = B; p.H = H; p.G = G; p.T = q_len; p.L = kv_len;
  p.gs = gs; p.npos = 128 / gs;
  p.nT = (kv_len + ATT_BN - 1) / ATT_BN;
  p.nQT = (q_len + p.npos - 1) / p.npos;
  p.token_pos = token_pos; p.tp_sb = tp_sb; p.tp_sg = tp_sg;
  int32_t* sc = reinterpret_cast<int32_t*>(scratch);
  int32_t* tmin = sc;
  int32_t* tmax = sc + (long long)B * G * p.nT;
  p.tile_min = tmin; p.tile_max = tmax;
  p.wpart = weights ? reinterpret_cast<float*>(sc + 2LL * B * G * p.nT) : nullptr;
  p.out = (__nv_bfloat16*)out; p.lse = lse;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.input_pos = input_pos; p.status = status;
  p.trace = g_att_trace; p.trace_cap = g_att_trace_cap;

  CUtensorMap tmQ, tmK, tmV;
  int rc;
  // Q (B,H,T,D): dims (D, T, H, B); box = 64 x npos x gs
  if ((rc = make_tmap_4d_bf16(&tmQ, q, ATT_D, q_len, H, B, ATT_D, (uint64_t)q_len * ATT_D, (uint64_t)H * q_len * ATT_D, 64,
                              p.npos, gs)))
    return rc;
  // K, V (B,G,L,D) with strides: dims (D, L, G, B); box = 64 x ATT_BN x 1
  if ((rc = make_tmap_4d_bf16(&tmK, k, ATT_D, kv_len, G, B, ATT_D, k_sg, k_sb, 64, ATT_BN, 1))) return rc;
  if ((rc = make_tmap_4d_bf16(&tmV, v, ATT_D, kv_len, G, B, ATT_D, k_sg, k_sb, 64, ATT_BN, 1))) return rc;

  att_tile_minmax_kernel<<<B * G * p.nT, ATT_BN, 0, s>>>(token_pos, tmin, tmax, G, kv_len, p.nT, tp_sb, tp_sg);
  static kvb::PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(sdpa_fwd_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttSmem::TOTAL);
    cudaFuncSetAttribute(sdpa_fwd_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttSmem::TOTAL);
  }
  // explicit token positions = an evicting cache: most tiles hold tokens of the current chunk and need
  // masks, which the 8-warp variant builds faster; plain causal attention runs best with 4 softmax warps
  if (token_pos) sdpa_fwd_kernel<8><<<B * G * p.nQT, att_threads(8), AttSmem::TOTAL, s>>>(tmQ, tmK, tmV, p);
  else sdpa_fwd_kernel<4><<<B * G * p.nQT, att_threads(4), AttSmem::TOTAL, s>>>(tmQ, tmK, tmV, p);
  if (weights) {
    dim3 grid((kv_len + 255) / 256, B * G);
    att_reduce_weights_kernel<<<grid, 256, 0, s>>>(p.wpart, weights, 4 * p.nQT, kv_len, 1.f / gs);
  }
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}
