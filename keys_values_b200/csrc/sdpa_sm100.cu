// SDPA forward for sm_100a with summed attention weights: one flash sweep for the output and the row
// normalisers, and a column-owner kernel for the per-slot weight sums.
//
//   out[b, t, h, :]   = softmax_j(scale · q[b,h,t]·k[b,g,j] | token_pos[b,g,j] <= input_pos + t) · v[b,g,:]
//                       (optionally: only tokens newer than input_pos + t − window; scores soft-capped by cap·tanh(·/cap))
//   lse[b, h, t]      = natural-log normaliser of that softmax
//   weights[b, g, j]  = (1 / (H/G)) · sum over t and over the H/G heads of group g of the softmax weight of slot j
//
// Kernel A (flash_fwd_kernel), one CTA per SM, per (batch, KV group, pair of query tiles):
//   * A query tile is 128 rows = npos consecutive positions x gs = H/G heads of one KV group, position
//     major (row = position · gs + head), so a K/V tile is read once per group. npos = 128 / gs (any
//     gs <= 128; rows beyond npos · gs are zero and ignored).
//   * S = Q K^T (M = 128, N = 128, both operands in shared memory) and O += P V run on tcgen05.mma with
//     accumulators in TMEM: S0 | S1 | O0 | O1, 128 columns each, all 512 columns of the SM.
//     Online softmax in one sweep over the KV tiles: the softmax warps read S from TMEM, write the
//     unnormalised P = exp2(S·c − m) back into the columns of S as packed bf16, and P is the A operand
//     of the PV MMA straight from TMEM, so neither S nor P touches shared memory. The running
//     maximum m of a row is only raised when it grows by more than 8 (a factor 256), in which case the
//     warp rescales its rows of O in TMEM; after the first tiles that is rare.
//   * Two query tiles per CTA, one softmax warpgroup each: while one warpgroup works on its S tile the
//     tensor core runs PV and the next QK of the other.
//   * K and V tiles of 128 slots arrive by TMA (128B swizzle, no multicast) in one ring of four 32 KB
//     stages in the order K0 V0 K1 V1 ...; V is consumed as an MN-major B operand.
//   * Masks come from token positions. A tile that holds no token beyond the first query of the CTA is
//     mask free. Slots whose token lies beyond the last query of the CTA are hidden from all of its rows:
//     they are masked by the tensor core itself, through one more K = 16 step of S whose A operand is a
//     column of ones and whose B operand holds 0 or -inf per slot (written by the producer warp from a
//     padded copy of the positions). Over an evicting cache that covers nearly all hidden slots; the few
//     slots in between are patched column by column in TMEM, and a tile with many of them (the diagonal
//     of plain causal attention) is compared element by element. Tiles that no query can see are skipped.
//
// Kernel B (colsum_kernel), per (batch, KV group, KV tile of 128 slots): S^T = K Q^T per query tile
//   on tcgen05 (M = 128 slots, N = 128 query rows), four S^T buffers in TMEM. A thread owns one slot
//   and adds exp2(S·c − lse_row) over the 128 query rows of every tile from registers: no shared
//   memory, no atomics, no partial buffers, a fixed order (run-to-run identical eviction decisions).
//   Position-major query rows turn the causal mask of a slot into one threshold on the column index.
//
// Variants: head size 64 and 128 are template parameters of these kernels (HD), sliding window and logit soft-capping a
// separate instantiation (GEN); head size 256 has its own flash kernel further down (flash256_fwd_kernel) and shares the
// column-sum and merge kernels. Launches with few query tiles are split over the KV axis (fp32 partials, merged in a
// fixed order by flash_merge_kernel).
//
// Replaces FlashInfer prefill + Triton score-sum + K/V reordering + query padding of the reference
// (keys_values/attention/flashinfer_wrapper.py:51-273, :367-510, csrc/kernels/sdpa_prefill.cu,
// attention/sdpa_wrapper.py:66-432).
#include <cuda.h>
#include <limits.h>

#include <stdlib.h>

#include "common.cuh"
#include "kvb200.h"

namespace kvb {

constexpr int F2_T = 128;                        // rows of a query tile, slots of a KV tile, head size
constexpr int F2_TILE_BYTES = F2_T * F2_T * 2;   // 32 KB: two 64-feature chunks of [128 rows x 128 B]
constexpr int F2_CHUNK_BYTES = F2_TILE_BYTES / 2;
constexpr int F2_STAGES = 4;
constexpr int F2_THREADS = 64 + 256;             // TMA warp, MMA warp, two softmax warpgroups
constexpr int F2_MAX_FLAG_TILES = 4096;           // tiles whose flags live in shared memory (one byte each)
constexpr float F2_RESCALE_STEP = 8.0f;          // log2 units
constexpr int F2_PATCH_MAX_COLS = 6;             // masked tiles with at most this many candidate columns are patched in TMEM
// Bias operand tiles of the extra K = 16 step of S: 128 rows x 16 bf16, K-major without swizzle. A core
// matrix is 8 rows x 16 bytes, stored contiguously (128 B); groups of 8 rows follow one another (stride byte
// offset 128 B), the second core matrix along K lies 2 KB further (leading byte offset).
constexpr int F2_BIAS_TILE_BYTES = 128 * 16 * 2;
constexpr uint32_t F2_BIAS_LBO = 2048, F2_BIAS_SBO = 128;
__device__ __forceinline__ uint32_t f2_bias_offset(int row) { return (uint32_t)((row >> 3) * F2_BIAS_SBO + (row & 7) * 16); }
// descriptor of such a tile: no swizzle (layout type 0), version 1
__device__ __forceinline__ uint64_t f2_bias_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)((F2_BIAS_LBO >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((F2_BIAS_SBO >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

struct F2Smem {
  static constexpr int Q = 0;                                   // two query tiles
  static constexpr int KV = Q + 2 * F2_TILE_BYTES;              // ring of K / V tiles
  static constexpr int TF = KV + F2_STAGES * F2_TILE_BYTES;     // one byte per KV tile: bit 0 active, bit 1 masked
  static constexpr int QX = TF + F2_MAX_FLAG_TILES;             // [128 x 16] bf16, column 0 = 1: A operand of the bias step
  static constexpr int KX = QX + F2_BIAS_TILE_BYTES;            // per ring stage: [128 x 16] bf16, column 0 = 0 or -inf
  static constexpr int BAR = KX + F2_STAGES * F2_BIAS_TILE_BYTES;
  static constexpr int TOTAL = BAR + 256;
};
static_assert(F2Smem::TOTAL <= 232448, "shared memory of the flash kernel exceeds the limit of a CTA");

struct F2Params {
  const int32_t* pos;        // (B,G,nT*128) padded token positions (INT_MAX beyond the cache)
  const int32_t* tile_min;   // (B,G,nT)
  const int32_t* tile_max;   // (B,G,nT)
  __nv_bfloat16* out;        // (B,T,H,D)
  float* lse;                // (B,H,T) natural log, or nullptr
  float* lse2;               // (B,G,nQT,128) log2 normaliser per packed query row, +inf for rows without a query
  float* weights;            // (B,G,L) or nullptr
  int B, H, G, T, L, nT, nQT, gs, npos, rows_used;
  float scale_log2;          // scale * log2(e)
  float inv_gs;
  int input_pos;
  int* status;
  long long* trace;          // optional phase profile of CTA 0: 4 roles x 8 cycle counters
  // split over the KV axis (few query tiles): grid.y = n_split CTAs per query-tile pair, each over tiles_per_split KV
  // tiles; they write normalised fp32 partial outputs and their log2 normalisers, a merge kernel combines them
  int n_split, tiles_per_split;
  float* part_o;             // (n_split, B, H, T, D)
  float* part_lse2;          // (n_split, B, H, T), -inf for a split that saw no visible slot
  // Sliding window (0: none): a slot is visible to a query at position q iff q - window < token <= q.
  // Logit soft-capping (cap_pre = 0: none): the score scale·s becomes cap·tanh(scale·s / cap); the kernels rewrite the
  // raw score s as cap_post·tanh(cap_pre·s) with cap_pre = scale / cap, cap_post = cap / scale and go on as without.
  int window;
  float cap_pre, cap_post;
};

// Hardware tanh (one special-function operation, relative error about 5e-4: below the rounding of bf16 scores). The
// exponentials already bound the softmax warps, so a tanh built from ex2 and rcp would cost twice as much again.
__device__ __forceinline__ float f2_tanh(float z) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(z));
  return t;
}
// the capped raw score; −inf (a slot hidden by the bias step of the MMA) stays −inf
__device__ __forceinline__ float f2_softcap(float s, float pre, float post) {
  return s == -INFINITY ? s : post * f2_tanh(pre * s);
}

// Optional phase profile of CTA 0 (diagnostics): each role adds the cycles spent since its previous mark to one of
// eight counters and writes them once at the end, so that the measurement costs a clock read per mark.
// Roles: 0 MMA issuer, 1 / 2 first warp of softmax warpgroup 0 / 1, 3 producer.
__device__ __forceinline__ uint32_t f2_clock() {
  uint32_t c;
  asm volatile("mov.u32 %0, %%clock;" : "=r"(c));
  return c;
}
#define F2_TRACE_DECL(active) uint32_t tr_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; const bool tr_on = p.trace != nullptr && blockIdx.x == 0 && (active); uint32_t tr_last = tr_on ? f2_clock() : 0u
#define F2_MARK(k)                                \
  do {                                            \
    if (tr_on) {                                  \
      const uint32_t now_ = f2_clock();           \
      tr_acc[k] += now_ - tr_last;                \
      tr_last = now_;                             \
    }                                             \
  } while (0)
#define F2_TRACE_STORE(role)                                                         \
  do {                                                                               \
    if (tr_on)                                                                       \
      for (int k_ = 0; k_ < 8; ++k_) p.trace[(role) * 8 + k_] = (long long)tr_acc[k_]; \
  } while (0)

// Per-tile min / max of the token positions for tiles of blockDim.x (64 or 128) slots (used by the backward kernels).
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

// tile_min / tile_max of the token positions per tile of 128 slots and a padded copy of the positions.
__global__ void f2_prepare_kernel(const int32_t* __restrict__ tp, int32_t* __restrict__ tmin, int32_t* __restrict__ tmax,
                                  int32_t* __restrict__ pos, int G, int L, int nT, long long tp_sb, long long tp_sg) {
  const int t = blockIdx.x % nT;
  const int bg = blockIdx.x / nT;
  const int b = bg / G, g = bg % G;
  const int j = t * F2_T + threadIdx.x;
  int lo = INT_MAX, hi = INT_MIN, v = INT_MAX;
  if (j < L) {
    v = tp ? tp[b * tp_sb + g * tp_sg + j] : j;
    lo = hi = v;
  }
  pos[(long long)blockIdx.x * F2_T + threadIdx.x] = v;
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
    for (int w = 1; w < 4; ++w) {
      lo = min(lo, slo[w]);
      hi = max(hi, shi[w]);
    }
    if ((t + 1) * F2_T > L) hi = INT_MAX;  // ragged last tile always takes the masked path
    tmin[blockIdx.x] = lo;
    tmax[blockIdx.x] = hi;
  }
}

__device__ __forceinline__ float f2_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// exp2 of two values on the FMA pipe instead of the special-function unit (16 results per clock and SM,
// which is what bounds a softmax at head size 128): round to the nearest integer n with the 1.5·2^23
// trick, a cubic for 2^f on f = x − n in [−0.5, 0.5] (relative error 7.5e-5, far below the bf16 rounding of
// P), and n added into the exponent field. Inputs below −126 (masked scores arrive as −inf) give ~1e-38.
__device__ __forceinline__ float2 f2_exp2_poly2(float2 x) {
  x.x = fmaxf(x.x, -126.f);
  x.y = fmaxf(x.y, -126.f);
  const float2 magic = make_float2(12582912.f, 12582912.f);
  const float2 t = fadd2(x, magic);
  const float2 n = fadd2(t, make_float2(-12582912.f, -12582912.f));
  const float2 f = ffma2(n, make_float2(-1.f, -1.f), x);
  float2 q = ffma2(make_float2(0.0551716194f, 0.0551716194f), f, make_float2(0.242611118f, 0.242611118f));
  q = ffma2(q, f, make_float2(0.693260995f, 0.693260995f));
  q = ffma2(q, f, make_float2(0.999928074f, 0.999928074f));
  float2 r;
  r.x = __int_as_float(__float_as_int(q.x) + (__float_as_int(t.x) << 23));
  r.y = __int_as_float(__float_as_int(q.y) + (__float_as_int(t.y) << 23));
  return r;
}
// of every 8 pairs of scores, the pairs listed here take the FMA-pipe exponential
// (none in the flash kernel: once the softmax warps were off the critical path, the tensor-core side bounded it
// and the extra FMA-pipe instructions cost more than the shorter exponential phase gained)
__device__ __forceinline__ constexpr bool f2_pair_on_fma(int pair) { return false && pair < 0; }
// the column-sum kernel is bound by the exponentials alone: 3 of 8 pairs go to the FMA pipe
__device__ __forceinline__ constexpr bool cs_pair_on_fma(int pair) { return (pair & 7) == 0 || (pair & 7) == 3 || (pair & 7) == 6; }

// Rows of a query tile that TMA does not write (npos · gs < 128) are cleared once, so that their
// scores are finite zeros.
__device__ __forceinline__ void f2_zero_unused_rows(uint8_t* tile, int rows_used, int tid, int nthreads, int nch) {
  const int n16 = (F2_T - rows_used) * 8 * nch;  // 16-byte units: rows x 8 units x chunks of 64 features
  for (int u = tid; u < n16; u += nthreads) {
    const int chunk = u / ((F2_T - rows_used) * 8);
    const int rem = u % ((F2_T - rows_used) * 8);
    const int row = rows_used + rem / 8;
    *reinterpret_cast<uint4*>(tile + chunk * F2_CHUNK_BYTES + sw128_offset(row, rem % 8)) = make_uint4(0, 0, 0, 0);
  }
}

// GEN: sliding window and / or soft-capping are in use (a separate instantiation, so that the plain kernel keeps its
// register allocation)
// HD: head size, 128 or 64 (one 64-feature chunk per tile, half as many K steps for S, O of 64 columns)
template <bool GEN, int HD>
__global__ void __launch_bounds__(F2_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const F2Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {  // swizzled tiles need a 1024-byte aligned window: report, do not run
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, STATUS_TIMEOUT_MISC);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + F2Smem::BAR);
  uint64_t* q_full = bars + 0;     // [2]
  uint64_t* kv_full = bars + 2;    // [4]
  uint64_t* kv_empty = bars + 6;   // [4]
  uint64_t* s_full = bars + 10;    // [2]
  uint64_t* p_full = bars + 12;    // [2]
  uint64_t* o_full = bars + 14;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* tflags = smem + F2Smem::TF;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nPair = (p.nQT + 1) / 2;
  const int pair = blockIdx.x % nPair;
  const int g = (blockIdx.x / nPair) % p.G;
  const int b = blockIdx.x / (nPair * p.G);
  const int t0 = 2 * pair * p.npos;  // first position of the pair
  const int qpos_min = p.input_pos + t0;
  const int qpos_max = p.input_pos + min(t0 + 2 * p.npos, p.T) - 1;
  const long long bg = (long long)b * p.G + g;
  const int32_t* tmin = p.tile_min + bg * p.nT;
  const int32_t* tmax = p.tile_max + bg * p.nT;

  // the KV tiles of this CTA: all of them, or the range of its split (tiles outside count as inactive)
  const int split = p.n_split > 1 ? (int)blockIdx.y : 0;
  const int t_lo = p.n_split > 1 ? split * p.tiles_per_split : 0;
  const int t_hi = p.n_split > 1 ? min(p.nT, t_lo + p.tiles_per_split) : p.nT;
  // With a window, tokens at or below lo_all are hidden from every row of the CTA, those at or below lo_some from some row.
  const int f_window = GEN ? p.window : 0;
  const int lo_all = f_window > 0 ? qpos_min - f_window : INT_MIN;
  const int lo_some = f_window > 0 ? qpos_max - f_window : INT_MIN;
  const bool soft = GEN && p.cap_pre != 0.f;
  constexpr bool general = GEN;  // masked tiles are then always treated element by element
  auto calc_bits = [&](int t) -> uint32_t {
    if (t < t_lo || t >= t_hi) return 0u;
    const int lo = tmin[t], hi = tmax[t];
    const uint32_t act = (lo <= qpos_max) && (hi > lo_all);
    const uint32_t msk = (hi > qpos_min) || (lo <= lo_some) || soft;  // soft-capping rewrites every tile
    return act | (msk << 1);
  };
  for (int t = threadIdx.x; t < min(p.nT, F2_MAX_FLAG_TILES); t += F2_THREADS) tflags[t] = (uint8_t)calc_bits(t);
  auto tile_bits = [&](int t) -> uint32_t { return t >= F2_MAX_FLAG_TILES ? calc_bits(t) : (uint32_t)tflags[t]; };
  if (p.rows_used < F2_T) {
    f2_zero_unused_rows(smem + F2Smem::Q, p.rows_used, threadIdx.x, F2_THREADS, HD / 64);
    f2_zero_unused_rows(smem + F2Smem::Q + F2_TILE_BYTES, p.rows_used, threadIdx.x, F2_THREADS, HD / 64);
    fence_proxy_async_smem();
  }
  // bias operands: zero everywhere, then ones in column 0 of the A tile (the producer fills column 0 of the B tiles)
  for (int u = threadIdx.x; u < (1 + F2_STAGES) * F2_BIAS_TILE_BYTES / 16; u += F2_THREADS)
    *reinterpret_cast<uint4*>(smem + F2Smem::QX + 16 * u) = make_uint4(0, 0, 0, 0);
  __syncthreads();
  if (threadIdx.x < F2_T) *reinterpret_cast<uint16_t*>(smem + F2Smem::QX + f2_bias_offset(threadIdx.x)) = 0x3F80;  // bf16 1.0
  fence_proxy_async_smem();
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
    }
    for (int s = 0; s < F2_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    mbar_init(o_full, 1);
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
  // columns: S0 [0,128) | S1 [128,256) | O0 [256,384) | O1 [384,512); P aliases the first 64 columns of its S
  int n_active = 0;
  for (int t = 0; t < p.nT; ++t) n_active += (int)(tile_bits(t) & 1u);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    // Lane 0 issues the copies; all lanes write the bias column of a masked K tile (4 slots per lane).
    if (n_active > 0) {
      if (lane == 0) {
        tma_prefetch_desc(&tmQ);
        tma_prefetch_desc(&tmK);
        tma_prefetch_desc(&tmV);
        const uint32_t q_bytes = (uint32_t)p.rows_used * (uint32_t)HD * 2u;
        for (int w = 0; w < 2; ++w) {
          uint8_t* qd = smem + F2Smem::Q + w * F2_TILE_BYTES;
          mbar_expect_tx(&q_full[w], q_bytes);
          tma_load_4d(qd, &tmQ, &q_full[w], 0, g * p.gs, t0 + w * p.npos, b);
          if (HD == 128) tma_load_4d(qd + F2_CHUNK_BYTES, &tmQ, &q_full[w], 64, g * p.gs, t0 + w * p.npos, b);
        }
      }
      const int32_t* pos_row = p.pos + bg * p.nT * F2_T;
      uint32_t seq = 0;
      bool ok = true;
      F2_TRACE_DECL(lane == 0);
      int4 pv_next = make_int4(0, 0, 0, 0);
      {
        int tf = 0;
        while (tf < p.nT && !(tile_bits(tf) & 1u)) ++tf;
        if (tf < p.nT && (tile_bits(tf) & 2u)) pv_next = __ldg(reinterpret_cast<const int4*>(pos_row + (long long)tf * F2_T) + lane);
      }
      for (int t = 0; t < p.nT && ok; ++t) {
        const uint32_t tb = tile_bits(t);
        if (!(tb & 1u)) continue;
        for (int kv = 0; kv < 2 && ok; ++kv) {
          const int st = seq % F2_STAGES;
          int4 pv = pv_next;
          if (kv == 0) {
            // positions of the next active tile travel while this one is handled
            int tn = t + 1;
            while (tn < p.nT && !(tile_bits(tn) & 1u)) ++tn;
            if (tn < p.nT && (tile_bits(tn) & 2u)) pv_next = __ldg(reinterpret_cast<const int4*>(pos_row + (long long)tn * F2_T) + lane);
          }
          F2_MARK(2);
          ok = mbar_wait_bounded(&kv_empty[st], ((seq / F2_STAGES) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY);
          F2_MARK(kv);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          if (kv == 0 && (tb & 2u)) {
            uint8_t* kx = smem + F2Smem::KX + st * F2_BIAS_TILE_BYTES;
            *reinterpret_cast<uint16_t*>(kx + f2_bias_offset(4 * lane + 0)) = (pv.x > qpos_max || pv.x <= lo_all) ? 0xFF80 : 0;  // bf16 -inf
            *reinterpret_cast<uint16_t*>(kx + f2_bias_offset(4 * lane + 1)) = (pv.y > qpos_max || pv.y <= lo_all) ? 0xFF80 : 0;
            *reinterpret_cast<uint16_t*>(kx + f2_bias_offset(4 * lane + 2)) = (pv.z > qpos_max || pv.z <= lo_all) ? 0xFF80 : 0;
            *reinterpret_cast<uint16_t*>(kx + f2_bias_offset(4 * lane + 3)) = (pv.w > qpos_max || pv.w <= lo_all) ? 0xFF80 : 0;
            fence_proxy_async_smem();
            __syncwarp();
          }
          if (lane == 0) {
            uint8_t* d = smem + F2Smem::KV + st * F2_TILE_BYTES;
            const CUtensorMap* tm = kv == 0 ? &tmK : &tmV;
            mbar_expect_tx(&kv_full[st], F2_T * HD * 2);
            tma_load_4d(d, tm, &kv_full[st], 0, t * F2_T, g, b);
            if (HD == 128) tma_load_4d(d + F2_CHUNK_BYTES, tm, &kv_full[st], 64, t * F2_T, g, b);
          }
          ++seq;
        }
      }
      F2_TRACE_STORE(3);
      if (!ok && lane == 0) {  // let copies in flight land before the CTA's shared memory is released
        long long c0 = clock64();
        while (clock64() - c0 < 2000000LL) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0 && n_active > 0) {
      constexpr uint32_t idesc_qk = make_idesc_bf16(F2_T, F2_T, 0, 0);  // Q, K both K-major
      constexpr uint32_t idesc_pv = make_idesc_bf16(F2_T, HD, 0, 1);    // P K-major (TMEM), V MN-major
      bool ok = true;
      F2_TRACE_DECL(true);
      for (int w = 0; w < 2 && ok; ++w) ok = mbar_wait_bounded(&q_full[w], 0, abort_flag, p.status, STATUS_TIMEOUT_FULL);
      tc_fence_after();
      // stages are used in the order K0 V0 K1 V1 ...: tile i reads K from sequence number 2i and V from 2i + 1
      auto stage_addr = [&](uint32_t s) { return smem_u32(smem + F2Smem::KV + (s % F2_STAGES) * F2_TILE_BYTES); };
      auto wait_stage = [&](uint32_t s) {
        return mbar_wait_bounded(&kv_full[s % F2_STAGES], (s / F2_STAGES) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL);
      };
      auto issue_qk = [&](int w, uint32_t kseq, bool masked) {
        const uint32_t q_addr = smem_u32(smem + F2Smem::Q + w * F2_TILE_BYTES);
        const uint32_t k_addr = stage_addr(kseq);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          // 16 features per step: chunk kk/4, 32 bytes per step inside the swizzled 128-byte row
          const uint32_t off = (uint32_t)((kk >> 2) * F2_CHUNK_BYTES + (kk & 3) * 32);
          umma_f16_ss(tmem_base + (uint32_t)(w * F2_T), make_smem_desc_sw128(q_addr + off, 16, 1024),
                      make_smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, kk != 0);
        }
        if (masked)  // S += 1 · bias^T: -inf for the slots that no row of this CTA may see
          umma_f16_ss(tmem_base + (uint32_t)(w * F2_T), f2_bias_desc(smem_u32(smem + F2Smem::QX)),
                      f2_bias_desc(smem_u32(smem + F2Smem::KX + (kseq % F2_STAGES) * F2_BIAS_TILE_BYTES)), idesc_qk, 1);
        umma_commit(&s_full[w]);
      };
      // the issuer walks the active tiles in step with the producer
      int t_next = 0;
      auto next_active_masked = [&]() -> bool {
        while (t_next < p.nT && !(tile_bits(t_next) & 1u)) ++t_next;
        const bool m = t_next < p.nT && (tile_bits(t_next) & 2u);
        ++t_next;
        return m;
      };
      auto issue_pv = [&](int w, uint32_t vseq, bool first) {
        const uint32_t v_addr = stage_addr(vseq);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A = P from TMEM: 16 slots = 8 columns of packed bf16 pairs per step.
          // B = V: MN-major; 16 slot rows per step (2048 B); the two 64-wide feature chunks are LBO apart.
          umma_f16_ts(tmem_base + (uint32_t)(2 * F2_T + w * F2_T), tmem_base + (uint32_t)(w * F2_T + 8 * kk),
                      make_smem_desc_sw128(v_addr + (uint32_t)(kk * 16 * 128), F2_CHUNK_BYTES, 1024), idesc_pv,
                      (first && kk == 0) ? 0u : 1u);
        }
      };
      // prologue: S0 and S1 of the first tile
      if (ok) ok = wait_stage(0);
      if (ok) {
        tc_fence_after();
        const bool m0 = next_active_masked();
        issue_qk(0, 0, m0);
        issue_qk(1, 0, m0);
        umma_commit(&kv_empty[0]);
      }
      for (int i = 0; i < n_active && ok; ++i) {
        const uint32_t vseq = 2u * i + 1, knext = 2u * i + 2;
        const bool more = i + 1 < n_active;
        F2_MARK(6);
        if (!(ok = wait_stage(vseq))) break;
        F2_MARK(4);
        if (more && !(ok = wait_stage(knext))) break;
        F2_MARK(5);
        const bool m_next = more ? next_active_masked() : false;
        for (int w = 0; w < 2 && ok; ++w) {
          F2_MARK(6);
          if (!(ok = mbar_wait_bounded(&p_full[w], i & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL))) break;
          F2_MARK(2 * w);
          tc_fence_after();
          issue_pv(w, vseq, i == 0);
          if (w == 1) umma_commit(&kv_empty[vseq % F2_STAGES]);
          if (more) {
            issue_qk(w, knext, m_next);
            if (w == 1) umma_commit(&kv_empty[knext % F2_STAGES]);
          }
          F2_MARK(2 * w + 1);
        }
      }
      if (ok) umma_commit(o_full);
      F2_TRACE_STORE(0);
    }
  } else {
    // ------------------------------------------------- softmax + epilogue warps
    const int wg = (warp - 2) >> 2;               // which query tile of the pair
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;          // TMEM lane = packed query row
    const int pl = row / p.gs, hq = row % p.gs;   // position within the tile, head within the group
    const int qt = 2 * pair + wg;
    const int tq = qt * p.npos + pl;
    const bool row_valid = row < p.rows_used && tq < p.T;
    const int my_pos = p.input_pos + tq;
    const int my_lo = f_window > 0 ? my_pos - f_window : INT_MIN;  // tokens at or below are outside this row's window
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tmem_S = tmem_base + (uint32_t)(wg * F2_T) + lane_base;
    const uint32_t tmem_O = tmem_base + (uint32_t)(2 * F2_T + wg * F2_T) + lane_base;
    const float c = p.scale_log2;
    const float2 c2 = make_float2(c, c);
    const int32_t* pos_row = p.pos + bg * p.nT * F2_T;
    // smallest and largest position among the 32 rows of this warp (rows beyond the query included)
    int wpos_min = my_pos, wpos_max = my_pos;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      wpos_min = min(wpos_min, __shfl_xor_sync(0xffffffffu, wpos_min, o));
      wpos_max = max(wpos_max, __shfl_xor_sync(0xffffffffu, wpos_max, o));
    }
    // Positions of the slots of the next masked tile (lane holds slots 4·lane .. 4·lane+3): requested one
    // tile ahead, because they come from L2 and are needed the moment the tile's scores are complete.
    int4 pf_v = make_int4(0, 0, 0, 0);
    int pf_t = -1;
    auto request_positions = [&](int t) {
      pf_v = __ldg(reinterpret_cast<const int4*>(pos_row + (long long)t * F2_T) + lane);
      pf_t = t;
    };
    auto next_active = [&](int t) {
      int tn = t + 1;
      while (tn < p.nT && !(tile_bits(tn) & 1u)) ++tn;
      return tn;
    };
    bool ok = n_active > 0;
    float m_used = -1e30f, l = 0.f;
    int i = 0;
    F2_TRACE_DECL((warp == 2 || warp == 6) && lane == 0);  // the first warp of each warpgroup records
    {
      const int tf = next_active(-1);
      if (ok && tf < p.nT && (tile_bits(tf) & 2u)) request_positions(tf);
    }
    for (int t = 0; t < p.nT && ok; ++t) {
      const uint32_t tb = tile_bits(t);
      if (!(tb & 1u)) continue;
      // Masks. Slots beyond the last query of the CTA arrive as -inf from the MMA. What is left are slots
      // whose token lies between the first row of this warp and the last query of the CTA: few over an
      // evicting cache, and then patched column by column in TMEM before the tile is read (a column
      // address may be a run-time value, a register index may not); many on the diagonal of plain causal
      // attention, and then the tile is compared element by element and written back.
      uint32_t m_all[4] = {0, 0, 0, 0}, m_some[4] = {0, 0, 0, 0};
      int mpos[4] = {0, 0, 0, 0};
      int n_cand = 0;
      if (tb & 2u) {
        if (pf_t != t) request_positions(t);
        mpos[0] = pf_v.x; mpos[1] = pf_v.y; mpos[2] = pf_v.z; mpos[3] = pf_v.w;
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const uint32_t cand = __ballot_sync(0xffffffffu, mpos[cc] > wpos_min && mpos[cc] <= qpos_max);
          m_all[cc] = __ballot_sync(0xffffffffu, mpos[cc] > wpos_max && mpos[cc] <= qpos_max);
          m_some[cc] = cand & ~m_all[cc];
          n_cand += __popc(cand);
        }
        if (general) n_cand = F2_T;  // window edges and capped scores: every element of the tile is looked at
      }
      {
        const int tn = next_active(t);
        if (tn < p.nT && (tile_bits(tn) & 2u)) request_positions(tn);
      }
      F2_MARK(6);
      if (!mbar_wait_bounded(&s_full[wg], i & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      F2_MARK(0);
      tc_fence_after();
      float a8[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) a8[u] = -INFINITY;
      bool have_max = false;  // GEN: the element pass below also takes the maximum of the row
      if (n_cand > F2_PATCH_MAX_COLS) {
        // element by element: the masked tile goes back to TMEM, the two passes below read it from there
        const int4* pp = reinterpret_cast<const int4*>(pos_row + (long long)t * F2_T);
#pragma unroll 1
        for (int c0 = 0; c0 < F2_T; c0 += 32) {
          uint32_t x[32];
          tmem_ld_32x32b_x32(tmem_S + (uint32_t)c0, x);
          tmem_ld_wait();
          if (soft) {
#pragma unroll
            for (int e = 0; e < 32; ++e) x[e] = __float_as_uint(f2_softcap(__uint_as_float(x[e]), p.cap_pre, p.cap_post));
          }
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const int4 v = __ldg(pp + ((c0 + e) >> 2));
            if (v.x > my_pos || v.x <= my_lo) x[e] = 0xff800000u;
            if (v.y > my_pos || v.y <= my_lo) x[e + 1] = 0xff800000u;
            if (v.z > my_pos || v.z <= my_lo) x[e + 2] = 0xff800000u;
            if (v.w > my_pos || v.w <= my_lo) x[e + 3] = 0xff800000u;
          }
          if (GEN) {
#pragma unroll
            for (int e = 0; e < 32; e += 16) {
#pragma unroll
              for (int u = 0; u < 8; ++u) a8[u] = fmax3(a8[u], __uint_as_float(x[e + 2 * u]), __uint_as_float(x[e + 2 * u + 1]));
            }
          }
          tmem_st_32x32b_x16(tmem_S + (uint32_t)c0, x);
          tmem_st_32x32b_x16(tmem_S + (uint32_t)(c0 + 16), x + 16);
        }
        tmem_st_wait();
        have_max = GEN;
      } else if (n_cand > 0) {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t bits = m_all[cc];  // hidden from every row of this warp: no need to look at the scores
          while (bits) {
            const int src = __ffs(bits) - 1;
            bits &= bits - 1;
            tmem_st_32x32b_x1(tmem_S + (uint32_t)(4 * src + cc), 0xff800000u);
          }
          bits = m_some[cc];          // hidden from some rows
          while (bits) {
            const int src = __ffs(bits) - 1;
            bits &= bits - 1;
            const int pe = __shfl_sync(0xffffffffu, mpos[cc], src);
            const uint32_t col = tmem_S + (uint32_t)(4 * src + cc);
            uint32_t a = tmem_ld_32x32b_x1(col);
            tmem_ld_wait();
            if (pe > my_pos) a = 0xff800000u;
            tmem_st_32x32b_x1(col, a);
          }
        }
        tmem_st_wait();
      }
      F2_MARK(1);
      // pass 1: maximum of the row; the scores stay in TMEM, 32 of them are in registers at a time
      if (!have_max) {
        uint32_t x[2][32];
        tmem_ld_32x32b_x32(tmem_S, x[0]);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          tmem_ld_wait();
          if (w < 3) tmem_ld_32x32b_x32(tmem_S + (uint32_t)(32 * (w + 1)), x[(w + 1) & 1]);
#pragma unroll
          for (int e = 0; e < 32; e += 16) {
#pragma unroll
            for (int u = 0; u < 8; ++u)
              a8[u] = fmax3(a8[u], __uint_as_float(x[w & 1][e + 2 * u]), __uint_as_float(x[w & 1][e + 2 * u + 1]));
          }
        }
      }
      F2_MARK(2);
      const float m_tile = fmax3(fmax3(a8[0], a8[1], a8[2]), fmax3(a8[3], a8[4], a8[5]), fmaxf(a8[6], a8[7])) * c;  // -inf: all hidden
      // raise the reference maximum of the row only when it grows by more than the step
      const bool raise = m_tile > m_used + F2_RESCALE_STEP;
      const float m_new = raise ? m_tile : m_used;
      if (i > 0 && __any_sync(0xffffffffu, raise)) {
        // the PV MMA of the previous tile finished before this tile's S was signalled: O may be rescaled
        const float f = raise ? f2_exp2(m_used - m_new) : 1.f;
        l *= f;
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tmem_O + (uint32_t)c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
          tmem_st_32x32b_x16(tmem_O + (uint32_t)c0, o);
          tmem_st_32x32b_x16(tmem_O + (uint32_t)(c0 + 16), o + 16);
        }
      }
      m_used = m_new;
      F2_MARK(3);
      // pass 2: P = exp2(S·c − m) as packed bf16 into the first 64 columns of S. Chunk u of the scores
      // (columns 32u ..) is in registers before P of chunk u (columns 16u ..) overwrites older columns.
      const float2 neg_m2 = make_float2(-m_used, -m_used);
      float2 s0 = make_float2(0.f, 0.f), s1 = s0;
      {
        uint32_t x[2][32];
        tmem_ld_32x32b_x32(tmem_S, x[0]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          tmem_ld_wait();
          if (u < 3) tmem_ld_32x32b_x32(tmem_S + (uint32_t)(32 * (u + 1)), x[(u + 1) & 1]);
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const float2 x0 = ffma2(make_float2(__uint_as_float(x[u & 1][e]), __uint_as_float(x[u & 1][e + 1])), c2, neg_m2);
            const float2 x1 = ffma2(make_float2(__uint_as_float(x[u & 1][e + 2]), __uint_as_float(x[u & 1][e + 3])), c2, neg_m2);
            const float2 y0 = f2_pair_on_fma(e >> 1) ? f2_exp2_poly2(x0) : make_float2(f2_exp2(x0.x), f2_exp2(x0.y));
            const float2 y1 = f2_pair_on_fma((e >> 1) + 1) ? f2_exp2_poly2(x1) : make_float2(f2_exp2(x1.x), f2_exp2(x1.y));
            s0 = fadd2(s0, y0);
            s1 = fadd2(s1, y1);
            pk[e >> 1] = pack_bf16x2(y0.x, y0.y);
            pk[(e >> 1) + 1] = pack_bf16x2(y1.x, y1.y);
          }
          // the load of chunk u + 1 (columns 32(u+1) ..) must have left TMEM before P of chunk u lands on
          // columns 16u .. 16u+15 only if those overlap, which they never do (16u + 16 <= 32(u + 1))
          tmem_st_32x32b_x16(tmem_S + (uint32_t)(16 * u), pk);
        }
      }
      s0 = fadd2(s0, s1);
      l += s0.x + s0.y;
      F2_MARK(4);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[wg]);
      F2_MARK(5);
      ++i;
    }

    F2_TRACE_STORE(1 + wg);
    // ---- epilogue: O / l -> bf16 -> out; normalisers
    if (ok) ok = mbar_wait_bounded(o_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL);
    if (ok || n_active == 0) {
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const float lse2 = l > 0.f ? m_used + log2f(l) : INFINITY;
      if (p.n_split > 1) {
        // partial result of this split: normalised fp32 rows and their log2 normaliser
        const long long prow = (((long long)split * p.B + b) * p.H + (g * p.gs + (row_valid ? hq : 0))) * p.T + (row_valid ? tq : 0);
        float* pdst = p.part_o + prow * HD;
#pragma unroll 1
        for (int c0 = 0; c0 < HD; c0 += 32) {
          uint32_t o[32];
          if (n_active > 0) {
            tmem_ld_32x32b_x32(tmem_O + (uint32_t)c0, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = 0;
          }
          if (row_valid) {
#pragma unroll
            for (int u = 0; u < 8; ++u)
              *reinterpret_cast<float4*>(pdst + c0 + 4 * u) =
                  make_float4(__uint_as_float(o[4 * u]) * inv_l, __uint_as_float(o[4 * u + 1]) * inv_l,
                              __uint_as_float(o[4 * u + 2]) * inv_l, __uint_as_float(o[4 * u + 3]) * inv_l);
          }
        }
        if (row_valid) p.part_lse2[prow] = l > 0.f ? lse2 : -INFINITY;
      } else {
      // tcgen05.ld is warp-collective: rows without a query take part in the loads and skip the stores
      __nv_bfloat16* dst = p.out + (((long long)b * p.T + (row_valid ? tq : 0)) * p.H + (g * p.gs + (row_valid ? hq : 0))) * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t o[32];
        if (n_active > 0) {
          tmem_ld_32x32b_x32(tmem_O + (uint32_t)c0, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = 0;
        }
        if (row_valid) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[8 * u + 0]) * inv_l, __uint_as_float(o[8 * u + 1]) * inv_l);
            v.y = pack_bf16x2(__uint_as_float(o[8 * u + 2]) * inv_l, __uint_as_float(o[8 * u + 3]) * inv_l);
            v.z = pack_bf16x2(__uint_as_float(o[8 * u + 4]) * inv_l, __uint_as_float(o[8 * u + 5]) * inv_l);
            v.w = pack_bf16x2(__uint_as_float(o[8 * u + 6]) * inv_l, __uint_as_float(o[8 * u + 7]) * inv_l);
            *reinterpret_cast<uint4*>(dst + c0 + 8 * u) = v;
          }
        }
      }
      if (row_valid && p.lse) p.lse[((long long)b * p.H + (g * p.gs + hq)) * p.T + tq] = lse2 * 0.6931471805599453f;
      if (p.lse2 && qt < p.nQT) p.lse2[(bg * p.nQT + qt) * F2_T + row] = row_valid ? lse2 : INFINITY;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Combines the partial results of the splits of a query row: out = Σ_s w_s O_s / Σ_s w_s with w_s = 2^(lse2_s − max),
// in a fixed order of the splits. One warp per packed query row (the rows of the lse2 layout, padding rows included,
// which get +inf there as in the unsplit kernel); lane l holds features 4l .. 4l+3.
template <int HD>
__global__ void __launch_bounds__(256) flash_merge_kernel(const F2Params p) {
  const long long wrow = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);  // index into (B, G, nQT, 128)
  const int lane = threadIdx.x & 31;
  if (wrow >= (long long)p.B * p.G * p.nQT * F2_T) return;
  const int row = (int)(wrow % F2_T);
  const int qt = (int)((wrow / F2_T) % p.nQT);
  const long long bg = wrow / ((long long)F2_T * p.nQT);
  const int g = (int)(bg % p.G), b = (int)(bg / p.G);
  const int pl = row / p.gs, hq = row % p.gs;
  const int tq = qt * p.npos + pl;
  const bool row_valid = row < p.rows_used && tq < p.T;
  if (!row_valid) {
    if (lane == 0 && p.lse2) p.lse2[wrow] = INFINITY;
    return;
  }
  const int h = g * p.gs + hq;
  const long long stride = (long long)p.B * p.H * p.T;  // rows per split
  const long long prow = ((long long)b * p.H + h) * p.T + tq;
  float mx = -INFINITY;
  for (int sidx = 0; sidx < p.n_split; ++sidx) mx = fmaxf(mx, p.part_lse2[sidx * stride + prow]);
  constexpr int PER = HD / 32;  // features per lane: lane l holds features PER·l .. PER·l + PER − 1
  float acc[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) acc[e] = 0.f;
  float total = 0.f;
  if (mx > -INFINITY) {
    for (int sidx = 0; sidx < p.n_split; ++sidx) {
      const float w = exp2f(p.part_lse2[sidx * stride + prow] - mx);
      if (w > 0.f) {
        const float2* src = reinterpret_cast<const float2*>(p.part_o + (sidx * stride + prow) * HD + PER * lane);
#pragma unroll
        for (int e = 0; e < PER / 2; ++e) {
          const float2 o = src[e];
          acc[2 * e] += w * o.x;
          acc[2 * e + 1] += w * o.y;
        }
        total += w;
      }
    }
  }
  const float inv = total > 0.f ? 1.f / total : 0.f;
  uint32_t* dst = reinterpret_cast<uint32_t*>(p.out + (((long long)b * p.T + tq) * p.H + h) * HD + PER * lane);
#pragma unroll
  for (int e = 0; e < PER / 2; ++e) dst[e] = pack_bf16x2(acc[2 * e] * inv, acc[2 * e + 1] * inv);
  if (lane == 0) {
    const float lse2 = total > 0.f ? mx + log2f(total) : INFINITY;
    if (p.lse) p.lse[prow] = lse2 * 0.6931471805599453f;
    if (p.lse2) p.lse2[wrow] = lse2;
  }
}

// ------------------------------------------------------------------ head size 256
// The flash sweep for head size 256 (Gemma-2 2b / 9b, Gemma-3 shapes). A query tile of 128 rows x 256 features and one
// K and one V tile of 128 slots x 256 features are 64 KB each, and O is 256 TMEM columns, so a CTA has ONE query tile:
//   shared memory: Q | K stage | V stage (64 KB each, four 64-feature chunks of [128 rows x 128 B]);
//   TMEM: S0 [0,128) | S1 [128,256) | O [256,512). S is double buffered over the KV tiles of the same query tile: the
//   QK MMAs of tile i + 1 (16 K-steps) run while the softmax warpgroup works on tile i; P aliases the first 64 columns
//   of its S buffer and is the A operand of the PV MMAs (N = 256) from TMEM.
// MMA order: QK(0), then per tile i: QK(i + 1), PV(i). O may still be accumulating PV(i - 1) when S(i) is complete, so a
// softmax warp that has to rescale O first waits for that PV (the barrier that also frees the V stage).
// Masks are taken element by element in every tile that needs one (no bias step); soft-capping rewrites every tile.
constexpr int F3_HD = 256;
constexpr int F3_TILE_BYTES = F2_T * F3_HD * 2;
constexpr int F3_THREADS = 64 + 128;  // TMA warp, MMA warp, one softmax warpgroup
struct F3Smem {
  static constexpr int Q = 0;
  static constexpr int K = Q + F3_TILE_BYTES;
  static constexpr int V = K + F3_TILE_BYTES;
  static constexpr int TF = V + F3_TILE_BYTES;
  static constexpr int BAR = TF + F2_MAX_FLAG_TILES;
  static constexpr int TOTAL = BAR + 256;
};
static_assert(F3Smem::TOTAL <= 232448, "shared memory of the head-size-256 flash kernel exceeds the limit of a CTA");

__global__ void __launch_bounds__(F3_THREADS, 1)
flash256_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const F2Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, STATUS_TIMEOUT_MISC);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + F3Smem::BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;
  uint64_t* v_full = bars + 2;
  uint64_t* k_empty = bars + 3;
  uint64_t* v_empty = bars + 4;   // PV of a tile is complete: the V stage is free and O is quiet
  uint64_t* s_full = bars + 5;    // [2]
  uint64_t* p_full = bars + 7;    // [2]
  uint64_t* o_full = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  uint8_t* tflags = smem + F3Smem::TF;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x % p.nQT;
  const int g = (blockIdx.x / p.nQT) % p.G;
  const int b = blockIdx.x / (p.nQT * p.G);
  const int t0 = qt * p.npos;
  const int qpos_min = p.input_pos + t0;
  const int qpos_max = p.input_pos + min(t0 + p.npos, p.T) - 1;
  const long long bg = (long long)b * p.G + g;
  const int32_t* tmin = p.tile_min + bg * p.nT;
  const int32_t* tmax = p.tile_max + bg * p.nT;
  const int split = p.n_split > 1 ? (int)blockIdx.y : 0;
  const int t_lo = p.n_split > 1 ? split * p.tiles_per_split : 0;
  const int t_hi = p.n_split > 1 ? min(p.nT, t_lo + p.tiles_per_split) : p.nT;
  const int lo_all = p.window > 0 ? qpos_min - p.window : INT_MIN;   // tokens at or below: outside every row's window
  const int lo_some = p.window > 0 ? qpos_max - p.window : INT_MIN;  // ... outside some row's window
  const bool soft = p.cap_pre != 0.f;
  auto calc_bits = [&](int t) -> uint32_t {
    if (t < t_lo || t >= t_hi) return 0u;
    const int lo = tmin[t], hi = tmax[t];
    const uint32_t act = (lo <= qpos_max) && (hi > lo_all);
    const uint32_t msk = (hi > qpos_min) || (lo <= lo_some) || soft;
    return act | (msk << 1);
  };
  for (int t = threadIdx.x; t < min(p.nT, F2_MAX_FLAG_TILES); t += F3_THREADS) tflags[t] = (uint8_t)calc_bits(t);
  auto tile_bits = [&](int t) -> uint32_t { return t >= F2_MAX_FLAG_TILES ? calc_bits(t) : (uint32_t)tflags[t]; };
  if (p.rows_used < F2_T) {
    f2_zero_unused_rows(smem + F3Smem::Q, p.rows_used, threadIdx.x, F3_THREADS, F3_HD / 64);
    fence_proxy_async_smem();
  }
  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(k_empty, 1);
    mbar_init(v_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
    }
    mbar_init(o_full, 1);
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
  int n_active = 0;
  for (int t = 0; t < p.nT; ++t) n_active += (int)(tile_bits(t) & 1u);

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && n_active > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, (uint32_t)p.rows_used * F3_HD * 2u);
      for (int c = 0; c < 4; ++c) tma_load_4d(smem + F3Smem::Q + c * F2_CHUNK_BYTES, &tmQ, q_full, 64 * c, g * p.gs, t0, b);
      bool ok = true;
      int i = 0;
      for (int t = 0; t < p.nT && ok; ++t) {
        if (!(tile_bits(t) & 1u)) continue;
        if (!(ok = mbar_wait_bounded(k_empty, (i & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY))) break;
        mbar_expect_tx(k_full, F3_TILE_BYTES);
        for (int c = 0; c < 4; ++c) tma_load_4d(smem + F3Smem::K + c * F2_CHUNK_BYTES, &tmK, k_full, 64 * c, t * F2_T, g, b);
        if (!(ok = mbar_wait_bounded(v_empty, (i & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY))) break;
        mbar_expect_tx(v_full, F3_TILE_BYTES);
        for (int c = 0; c < 4; ++c) tma_load_4d(smem + F3Smem::V + c * F2_CHUNK_BYTES, &tmV, v_full, 64 * c, t * F2_T, g, b);
        ++i;
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
      constexpr uint32_t idesc_qk = make_idesc_bf16(F2_T, F2_T, 0, 0);    // Q, K both K-major
      constexpr uint32_t idesc_pv = make_idesc_bf16(F2_T, F3_HD, 0, 1);   // P K-major (TMEM), V MN-major, N = 256
      const uint32_t q_addr = smem_u32(smem + F3Smem::Q), k_addr = smem_u32(smem + F3Smem::K), v_addr = smem_u32(smem + F3Smem::V);
      auto issue_qk = [&](int buf) {
#pragma unroll
        for (int kk = 0; kk < F3_HD / 16; ++kk) {
          const uint32_t off = (uint32_t)((kk >> 2) * F2_CHUNK_BYTES + (kk & 3) * 32);
          umma_f16_ss(tmem_base + (uint32_t)(buf * F2_T), make_smem_desc_sw128(q_addr + off, 16, 1024),
                      make_smem_desc_sw128(k_addr + off, 16, 1024), idesc_qk, kk != 0);
        }
        umma_commit(k_empty);
        umma_commit(&s_full[buf]);
      };
      bool ok = mbar_wait_bounded(q_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL);
      if (ok) ok = mbar_wait_bounded(k_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int i = 0; i < n_active && ok; ++i) {
        if (i + 1 < n_active) {
          if (!(ok = mbar_wait_bounded(k_full, (i + 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL))) break;
          tc_fence_after();
          issue_qk((i + 1) & 1);  // its buffer held P of tile i - 1, whose PV MMAs were issued before
        }
        if (!(ok = mbar_wait_bounded(v_full, i & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL))) break;
        if (!(ok = mbar_wait_bounded(&p_full[i & 1], (i >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL))) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          // A = P from TMEM: 16 slots = 8 columns of packed bf16 pairs per step; B = V, MN-major: 16 slot rows per step
          // (2048 B), the four 64-wide feature chunks LBO apart
          umma_f16_ts(tmem_base + 256u, tmem_base + (uint32_t)((i & 1) * F2_T + 8 * kk),
                      make_smem_desc_sw128(v_addr + (uint32_t)(kk * 16 * 128), F2_CHUNK_BYTES, 1024), idesc_pv,
                      (i == 0 && kk == 0) ? 0u : 1u);
        }
        umma_commit(v_empty);
      }
      if (ok) umma_commit(o_full);
    }
  } else {
    // ------------------------------------------------- softmax + epilogue warps (one warpgroup)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int pl = row / p.gs, hq = row % p.gs;
    const int tq = t0 + pl;
    const bool row_valid = row < p.rows_used && tq < p.T;
    const int my_pos = p.input_pos + tq;
    const int my_lo = p.window > 0 ? my_pos - p.window : INT_MIN;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tmem_O = tmem_base + 256u + lane_base;
    const float c = p.scale_log2;
    const float2 c2 = make_float2(c, c);
    const int32_t* pos_row = p.pos + bg * p.nT * F2_T;
    bool ok = n_active > 0;
    float m_used = -1e30f, l = 0.f;
    int i = 0;
    for (int t = 0; t < p.nT && ok; ++t) {
      const uint32_t tb = tile_bits(t);
      if (!(tb & 1u)) continue;
      const uint32_t tmem_S = tmem_base + (uint32_t)((i & 1) * F2_T) + lane_base;
      if (!mbar_wait_bounded(&s_full[i & 1], (i >> 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      float a8[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) a8[u] = -INFINITY;
      if (tb & 2u) {
        // element by element: capped scores, causal and window masks; the row maximum in the same pass
        const int4* pp = reinterpret_cast<const int4*>(pos_row + (long long)t * F2_T);
#pragma unroll 1
        for (int c0 = 0; c0 < F2_T; c0 += 32) {
          uint32_t x[32];
          tmem_ld_32x32b_x32(tmem_S + (uint32_t)c0, x);
          tmem_ld_wait();
          if (soft) {
#pragma unroll
            for (int e = 0; e < 32; ++e) x[e] = __float_as_uint(f2_softcap(__uint_as_float(x[e]), p.cap_pre, p.cap_post));
          }
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const int4 v = __ldg(pp + ((c0 + e) >> 2));
            if (v.x > my_pos || v.x <= my_lo) x[e] = 0xff800000u;
            if (v.y > my_pos || v.y <= my_lo) x[e + 1] = 0xff800000u;
            if (v.z > my_pos || v.z <= my_lo) x[e + 2] = 0xff800000u;
            if (v.w > my_pos || v.w <= my_lo) x[e + 3] = 0xff800000u;
          }
#pragma unroll
          for (int e = 0; e < 32; e += 16) {
#pragma unroll
            for (int u = 0; u < 8; ++u) a8[u] = fmax3(a8[u], __uint_as_float(x[e + 2 * u]), __uint_as_float(x[e + 2 * u + 1]));
          }
          tmem_st_32x32b_x16(tmem_S + (uint32_t)c0, x);
          tmem_st_32x32b_x16(tmem_S + (uint32_t)(c0 + 16), x + 16);
        }
        tmem_st_wait();
      } else {
        uint32_t x[2][32];
        tmem_ld_32x32b_x32(tmem_S, x[0]);
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          tmem_ld_wait();
          if (w < 3) tmem_ld_32x32b_x32(tmem_S + (uint32_t)(32 * (w + 1)), x[(w + 1) & 1]);
#pragma unroll
          for (int e = 0; e < 32; e += 16) {
#pragma unroll
            for (int u = 0; u < 8; ++u)
              a8[u] = fmax3(a8[u], __uint_as_float(x[w & 1][e + 2 * u]), __uint_as_float(x[w & 1][e + 2 * u + 1]));
          }
        }
      }
      const float m_tile = fmax3(fmax3(a8[0], a8[1], a8[2]), fmax3(a8[3], a8[4], a8[5]), fmaxf(a8[6], a8[7])) * c;
      const bool raise = m_tile > m_used + F2_RESCALE_STEP;
      const float m_new = raise ? m_tile : m_used;
      if (i > 0 && __any_sync(0xffffffffu, raise)) {
        // O may still be accumulating the PV MMAs of the previous tile: wait for them, then rescale the rows
        if (!mbar_wait_bounded(v_empty, (i - 1) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const float f = raise ? f2_exp2(m_used - m_new) : 1.f;
        l *= f;
#pragma unroll 1
        for (int c0 = 0; c0 < F3_HD; c0 += 32) {
          uint32_t o[32];
          tmem_ld_32x32b_x32(tmem_O + (uint32_t)c0, o);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
          tmem_st_32x32b_x16(tmem_O + (uint32_t)c0, o);
          tmem_st_32x32b_x16(tmem_O + (uint32_t)(c0 + 16), o + 16);
        }
      }
      m_used = m_new;
      const float2 neg_m2 = make_float2(-m_used, -m_used);
      float2 s0 = make_float2(0.f, 0.f), s1 = s0;
      {
        uint32_t x[2][32];
        tmem_ld_32x32b_x32(tmem_S, x[0]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          tmem_ld_wait();
          if (u < 3) tmem_ld_32x32b_x32(tmem_S + (uint32_t)(32 * (u + 1)), x[(u + 1) & 1]);
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const float2 x0 = ffma2(make_float2(__uint_as_float(x[u & 1][e]), __uint_as_float(x[u & 1][e + 1])), c2, neg_m2);
            const float2 x1 = ffma2(make_float2(__uint_as_float(x[u & 1][e + 2]), __uint_as_float(x[u & 1][e + 3])), c2, neg_m2);
            const float2 y0 = make_float2(f2_exp2(x0.x), f2_exp2(x0.y));
            const float2 y1 = make_float2(f2_exp2(x1.x), f2_exp2(x1.y));
            s0 = fadd2(s0, y0);
            s1 = fadd2(s1, y1);
            pk[e >> 1] = pack_bf16x2(y0.x, y0.y);
            pk[(e >> 1) + 1] = pack_bf16x2(y1.x, y1.y);
          }
          tmem_st_32x32b_x16(tmem_S + (uint32_t)(16 * u), pk);
        }
      }
      s0 = fadd2(s0, s1);
      l += s0.x + s0.y;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[i & 1]);
      ++i;
    }
    // ---- epilogue
    if (ok) ok = mbar_wait_bounded(o_full, 0, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL);
    if (ok || n_active == 0) {
      tc_fence_after();
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const float lse2 = l > 0.f ? m_used + log2f(l) : INFINITY;
      const int h = g * p.gs + (row_valid ? hq : 0);
      const int tqv = row_valid ? tq : 0;
      if (p.n_split > 1) {
        const long long prow = (((long long)split * p.B + b) * p.H + h) * p.T + tqv;
        float* pdst = p.part_o + prow * F3_HD;
#pragma unroll 1
        for (int c0 = 0; c0 < F3_HD; c0 += 32) {
          uint32_t o[32];
          if (n_active > 0) {
            tmem_ld_32x32b_x32(tmem_O + (uint32_t)c0, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = 0;
          }
          if (row_valid) {
#pragma unroll
            for (int u = 0; u < 8; ++u)
              *reinterpret_cast<float4*>(pdst + c0 + 4 * u) =
                  make_float4(__uint_as_float(o[4 * u]) * inv_l, __uint_as_float(o[4 * u + 1]) * inv_l,
                              __uint_as_float(o[4 * u + 2]) * inv_l, __uint_as_float(o[4 * u + 3]) * inv_l);
          }
        }
        if (row_valid) p.part_lse2[prow] = l > 0.f ? lse2 : -INFINITY;
      } else {
        __nv_bfloat16* dst = p.out + (((long long)b * p.T + tqv) * p.H + h) * F3_HD;
#pragma unroll 1
        for (int c0 = 0; c0 < F3_HD; c0 += 32) {
          uint32_t o[32];
          if (n_active > 0) {
            tmem_ld_32x32b_x32(tmem_O + (uint32_t)c0, o);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) o[e] = 0;
          }
          if (row_valid) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(o[8 * u + 0]) * inv_l, __uint_as_float(o[8 * u + 1]) * inv_l);
              v.y = pack_bf16x2(__uint_as_float(o[8 * u + 2]) * inv_l, __uint_as_float(o[8 * u + 3]) * inv_l);
              v.z = pack_bf16x2(__uint_as_float(o[8 * u + 4]) * inv_l, __uint_as_float(o[8 * u + 5]) * inv_l);
              v.w = pack_bf16x2(__uint_as_float(o[8 * u + 6]) * inv_l, __uint_as_float(o[8 * u + 7]) * inv_l);
              *reinterpret_cast<uint4*>(dst + c0 + 8 * u) = v;
            }
          }
        }
        if (row_valid && p.lse) p.lse[((long long)b * p.H + h) * p.T + tq] = lse2 * 0.6931471805599453f;
        if (p.lse2) p.lse2[(bg * p.nQT + qt) * F2_T + row] = row_valid ? lse2 : INFINITY;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// ------------------------------------------------------------------ column sums
constexpr int CS_SBUF = 4;
// K tile | ring of query tiles (four, or two of the 64 KB tiles of head size 256) | barriers | exchange
template <int HD>
struct CsSmemT {
  static constexpr int TILE = F2_T * (HD < 128 ? 128 : HD) * 2;  // head size 64 keeps the 32 KB slots of 128
  static constexpr int QSTAGES = HD == 256 ? 2 : 4;
  static constexpr int K = 0;
  static constexpr int Q = K + TILE;
  static constexpr int BAR = Q + QSTAGES * TILE;
  static constexpr int XCH = BAR + 256;   // 128 floats: sums of the second warpgroup
  static constexpr int TOTAL = XCH + 512;
};
static_assert(CsSmemT<256>::TOTAL <= 232448, "shared memory of the column-sum kernel exceeds the limit of a CTA");

template <bool GEN, int HD>
__global__ void __launch_bounds__(F2_THREADS, 1)
colsum_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const F2Params p) {
  using CsSmem = CsSmemT<HD>;
  constexpr int CS_QSTAGES = CsSmem::QSTAGES;
  constexpr int CS_TILE = CsSmem::TILE;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0 && p.status) atomicCAS(p.status, 0, STATUS_TIMEOUT_MISC);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + CsSmem::BAR);
  uint64_t* k_full = bars + 0;
  uint64_t* q_full = bars + 1;     // [4]
  uint64_t* q_empty = bars + 5;    // [4]
  uint64_t* s_full = bars + 9;     // [4]
  uint64_t* s_empty = bars + 13;   // [4]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x % p.nT;          // KV tile
  const int g = (blockIdx.x / p.nT) % p.G;
  const int b = blockIdx.x / (p.nT * p.G);
  const long long bg = (long long)b * p.G + g;
  const int tile_lo = p.tile_min[bg * p.nT + t];
  const int tile_hi = p.tile_max[bg * p.nT + t];
  // query tiles that can see at least one slot of this tile: those whose last position reaches tile_lo
  // (positions grow with the tile index, so they form a suffix qt_first .. nQT-1)
  int qt_first = 0;
  {
    const long long need = (long long)tile_lo - p.input_pos;  // first position index that sees the oldest slot
    if (need > 0) qt_first = (int)min((long long)p.nQT, need / p.npos);
    if (tile_lo == INT_MAX) qt_first = p.nQT;
  }
  int qt_end = p.nQT;  // with a window, query tiles whose first position lies beyond the newest slot's window see nothing
  const int c_window = GEN ? p.window : 0;
  if (c_window > 0 && tile_hi != INT_MAX) {
    const long long last = (long long)tile_hi + c_window - 1 - p.input_pos;  // last position index that sees the newest slot
    qt_end = last < 0 ? 0 : (int)min((long long)p.nQT, last / p.npos + 1);
  }
  const int n_q = max(qt_end - qt_first, 0);
  const bool soft = GEN && p.cap_pre != 0.f;

  if (p.rows_used < F2_T) {
    for (int s = 0; s < CS_QSTAGES; ++s)
      f2_zero_unused_rows(smem + CsSmem::Q + s * CS_TILE, p.rows_used, threadIdx.x, F2_THREADS, HD / 64);
    fence_proxy_async_smem();
  }
  if (threadIdx.x == 0) {
    mbar_init(k_full, 1);
    for (int s = 0; s < CS_QSTAGES; ++s) {
      mbar_init(&q_full[s], 1);
      mbar_init(&q_empty[s], 1);
    }
    for (int s = 0; s < CS_SBUF; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 4);
    }
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

  if (warp == 0) {
    if (lane == 0 && n_q > 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      mbar_expect_tx(k_full, F2_T * HD * 2);
#pragma unroll
      for (int cch = 0; cch < HD / 64; ++cch)
        tma_load_4d(smem + CsSmem::K + cch * F2_CHUNK_BYTES, &tmK, k_full, 64 * cch, t * F2_T, g, b);
      const uint32_t q_bytes = (uint32_t)p.rows_used * (uint32_t)HD * 2u;
      bool ok = true;
      for (int i = 0; i < n_q && ok; ++i) {
        const int st = i % CS_QSTAGES;
        if (!mbar_wait_bounded(&q_empty[st], ((i / CS_QSTAGES) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_EMPTY)) {
          ok = false;
          break;
        }
        uint8_t* qd = smem + CsSmem::Q + st * CS_TILE;
        mbar_expect_tx(&q_full[st], q_bytes);
#pragma unroll
        for (int cch = 0; cch < HD / 64; ++cch)
          tma_load_4d(qd + cch * F2_CHUNK_BYTES, &tmQ, &q_full[st], 64 * cch, g * p.gs, (qt_first + i) * p.npos, b);
      }
      if (!ok) {
        long long c0 = clock64();
        while (clock64() - c0 < 2000000LL) {
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_q > 0) {
      constexpr uint32_t idesc = make_idesc_bf16(F2_T, F2_T, 0, 0);  // K (slots = M) and Q (rows = N), both K-major
      bool ok = mbar_wait_bounded(k_full, 0, abort_flag, p.status, STATUS_TIMEOUT_FULL);
      const uint32_t k_addr = smem_u32(smem + CsSmem::K);
      for (int i = 0; i < n_q && ok; ++i) {
        const int st = i % CS_QSTAGES, sb = i % CS_SBUF;
        if (!(ok = mbar_wait_bounded(&q_full[st], (i / CS_QSTAGES) & 1, abort_flag, p.status, STATUS_TIMEOUT_FULL))) break;
        if (!(ok = mbar_wait_bounded(&s_empty[sb], ((i / CS_SBUF) & 1) ^ 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_EMPTY))) break;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(smem + CsSmem::Q + st * CS_TILE);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (uint32_t)((kk >> 2) * F2_CHUNK_BYTES + (kk & 3) * 32);
          umma_f16_ss(tmem_base + (uint32_t)(sb * F2_T), make_smem_desc_sw128(k_addr + off, 16, 1024),
                      make_smem_desc_sw128(q_addr + off, 16, 1024), idesc, kk != 0);
        }
        umma_commit(&q_empty[st]);
        umma_commit(&s_full[sb]);
      }
    }
  } else {
    const int wg = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int slot_in_tile = quarter * 32 + lane;   // TMEM lane = slot of the tile
    const int j = t * F2_T + slot_in_tile;
    const int pj = p.pos[(bg * p.nT + t) * F2_T + slot_in_tile];
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const float c = p.scale_log2;
    const float2 c2 = make_float2(c, c);
    float2 acc0 = make_float2(0.f, 0.f), acc1 = acc0;
    bool ok = true;
    auto lse_row = [&](int i) { return p.lse2 + (bg * p.nQT + (qt_first + i)) * F2_T; };
    auto prefetch_lse = [&](int i) {  // 512 bytes = four lines, one per 8 lanes is enough: lanes 0..3 ask
      if (i < n_q && lane < 4) asm volatile("prefetch.global.L1 [%0];" ::"l"(lse_row(i) + 32 * lane));
    };
    prefetch_lse(wg);
    for (int i = wg; i < n_q && ok; i += 2) {
      const int qt = qt_first + i;
      const int sb = i % CS_SBUF;
      prefetch_lse(i + 2);
      // row e of the query tile sits at position qt·npos + e / gs: the slot is visible from column thr on
      const long long first_vis = ((long long)pj - p.input_pos - (long long)qt * p.npos) * p.gs;
      const int thr = first_vis <= 0 ? 0 : (first_vis >= F2_T ? F2_T : (int)first_vis);
      // with a window the slot is visible up to (not including) column thr_hi
      const long long end_vis = first_vis + (long long)c_window * p.gs;
      const int thr_hi = c_window <= 0 ? F2_T : (end_vis <= 0 ? 0 : (end_vis >= F2_T ? F2_T : (int)end_vis));
      const bool masked = __any_sync(0xffffffffu, thr > 0 || thr_hi < F2_T);
      const float4* lp = reinterpret_cast<const float4*>(lse_row(i));
      if (!mbar_wait_bounded(&s_full[sb], (i / CS_SBUF) & 1, abort_flag, p.status, STATUS_TIMEOUT_TMEM_FULL)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // 32 columns at a time: the next chunk of scores and of normalisers travels while this one is summed
      const uint32_t tS = tmem_base + (uint32_t)(sb * F2_T) + lane_base;
      uint32_t x[2][32];
      float4 ls[2][8];
      tmem_ld_32x32b_x32(tS, x[0]);
#pragma unroll
      for (int k = 0; k < 8; ++k) ls[0][k] = __ldg(lp + k);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        tmem_ld_wait();
        if (u < 3) {
          tmem_ld_32x32b_x32(tS + (uint32_t)(32 * (u + 1)), x[(u + 1) & 1]);
#pragma unroll
          for (int k = 0; k < 8; ++k) ls[(u + 1) & 1][k] = __ldg(lp + 8 * (u + 1) + k);
        } else {
          // the whole tile has left TMEM: hand the buffer back before the last chunk is summed
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&s_empty[sb]);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int e = 32 * u + 4 * k;
          const float4 lv = ls[u & 1][k];
          float2 r0 = make_float2(__uint_as_float(x[u & 1][4 * k]), __uint_as_float(x[u & 1][4 * k + 1]));
          float2 r1 = make_float2(__uint_as_float(x[u & 1][4 * k + 2]), __uint_as_float(x[u & 1][4 * k + 3]));
          if (soft) {
            r0 = make_float2(f2_softcap(r0.x, p.cap_pre, p.cap_post), f2_softcap(r0.y, p.cap_pre, p.cap_post));
            r1 = make_float2(f2_softcap(r1.x, p.cap_pre, p.cap_post), f2_softcap(r1.y, p.cap_pre, p.cap_post));
          }
          const float2 x0 = ffma2(r0, c2, make_float2(-lv.x, -lv.y));
          const float2 x1 = ffma2(r1, c2, make_float2(-lv.z, -lv.w));
          float2 y0 = cs_pair_on_fma(2 * k) ? f2_exp2_poly2(x0) : make_float2(f2_exp2(x0.x), f2_exp2(x0.y));
          float2 y1 = cs_pair_on_fma(2 * k + 1) ? f2_exp2_poly2(x1) : make_float2(f2_exp2(x1.x), f2_exp2(x1.y));
          if (masked) {
            if (e < thr || e >= thr_hi) y0.x = 0.f;
            if (e + 1 < thr || e + 1 >= thr_hi) y0.y = 0.f;
            if (e + 2 < thr || e + 2 >= thr_hi) y1.x = 0.f;
            if (e + 3 < thr || e + 3 >= thr_hi) y1.y = 0.f;
          }
          acc0 = fadd2(acc0, y0);
          acc1 = fadd2(acc1, y1);
        }
      }
    }
    // the two warpgroups hold the even and the odd query tiles of the same slots: add them in a fixed order
    float* xch = reinterpret_cast<float*>(smem + CsSmem::XCH);
    const float mine = (acc0.x + acc0.y) + (acc1.x + acc1.y);
    if (wg == 1) xch[slot_in_tile] = mine;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (wg == 0 && j < p.L && p.weights) p.weights[bg * p.L + j] = ok ? (mine + xch[slot_in_tile]) * p.inv_gs : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

typedef CUresult (*F2EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                    const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// 4-d bf16 map: dims d0 (contiguous), d1..d3 with element strides s1..s3; box b0 x b1 x b2 x 1
static int f2_make_tmap(CUtensorMap* tm, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t d3, uint64_t s1,
                        uint64_t s2, uint64_t s3, uint32_t b0, uint32_t b1, uint32_t b2) {
  static F2EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* pp = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &pp, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
      return KVB_ERR_DRIVER;
    fn = reinterpret_cast<F2EncodeTiledFn>(pp);
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

static inline long long f2_round4(long long x) { return (x + 3) / 4 * 4; }

// the launches of one forward call for one (GEN, head size) instantiation
template <bool GEN, int HD>
static int f2_launch(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const F2Params& p, cudaStream_t s) {
  static kvb::PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(flash_fwd_kernel<GEN, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, F2Smem::TOTAL);
    cudaFuncSetAttribute(colsum_kernel<GEN, HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, CsSmemT<HD>::TOTAL);
  }
  const int nPair = (p.nQT + 1) / 2;
  flash_fwd_kernel<GEN, HD><<<dim3(p.B * p.G * nPair, p.n_split), F2_THREADS, F2Smem::TOTAL, s>>>(tmQ, tmK, tmV, p);
  if (p.n_split > 1) {
    const long long rows = (long long)p.B * p.G * p.nQT * F2_T;
    flash_merge_kernel<HD><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(p);
  }
  if (p.weights) colsum_kernel<GEN, HD><<<p.B * p.G * p.nT, F2_THREADS, CsSmemT<HD>::TOTAL, s>>>(tmQ, tmK, p);
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

// the launches of one forward call for head size 256
static int f3_launch(const CUtensorMap& tmQ, const CUtensorMap& tmK, const CUtensorMap& tmV, const F2Params& p, bool gen,
                     cudaStream_t s) {
  static kvb::PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(flash256_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F3Smem::TOTAL);
    cudaFuncSetAttribute(colsum_kernel<false, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, CsSmemT<256>::TOTAL);
    cudaFuncSetAttribute(colsum_kernel<true, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, CsSmemT<256>::TOTAL);
  }
  flash256_fwd_kernel<<<dim3(p.B * p.G * p.nQT, p.n_split), F3_THREADS, F3Smem::TOTAL, s>>>(tmQ, tmK, tmV, p);
  if (p.n_split > 1) {
    const long long rows = (long long)p.B * p.G * p.nQT * F2_T;
    flash_merge_kernel<256><<<(unsigned)((rows + 7) / 8), 256, 0, s>>>(p);
  }
  if (p.weights) {
    if (gen) colsum_kernel<true, 256><<<p.B * p.G * p.nT, F2_THREADS, CsSmemT<256>::TOTAL, s>>>(tmQ, tmK, p);
    else colsum_kernel<false, 256><<<p.B * p.G * p.nT, F2_THREADS, CsSmemT<256>::TOTAL, s>>>(tmQ, tmK, p);
  }
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
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

// Optional phase profile of the flash kernel (diagnostics): `buf` holds 4 roles x 8 int64 cycle counters, written by
// CTA 0 of every later kvb_sdpa_fwd launch of this process; NULL switches it off. Counters: issuer 0 wait P of tile 0,
// 1 issue PV + next QK of tile 0, 2 / 3 the same for tile 1, 4 wait V, 5 wait K, 6 rest; softmax 0 wait S, 1 masks,
// 2 S into registers, 3 maximum and rescale, 4 exponentials, 5 hand-over of P, 6 rest; producer 0 wait for a free K
// stage, 1 for a free V stage, 2 rest.
static long long* g_f2_trace = nullptr;
extern "C" int kvb_sdpa_fwd_set_trace(void* buf) {
  g_f2_trace = reinterpret_cast<long long*>(buf);
  return KVB_OK;
}

// Scratch layout (int32 words, 16-byte aligned parts), provided by the caller:
//   tile_min (B*G*nT) | tile_max (B*G*nT) | positions (B*G*nT*128) | lse2 (B*G*nQT*128 floats)
// Number of CTAs along the KV axis per query-tile pair: 1 unless the launch would leave most SMs idle (few queries:
// short chunks at batch 1) while the cache is long enough to give every split at least 8 tiles.
static int f2_num_splits(long long ctas, long long nT) {
  static const int enabled = [] {
    const char* e = getenv("KVB200_F2_SPLIT");  // "0" switches the split off (diagnostics)
    return (e && e[0] == '0') ? 0 : 1;
  }();
  if (!enabled || ctas <= 0 || ctas * 2 > 148 || nT < 16) return 1;
  long long n = 148 / ctas;
  if (n > nT / 8) n = nT / 8;
  if (n > 8) n = 8;
  return n < 2 ? 1 : (int)n;
}

//   ... | split partials: part_lse2 (n_split*B*H*T floats) | part_o (n_split*B*H*T*128 floats), present when the
//   launch is split over the KV axis (f2_num_splits)
extern "C" long long kvb_sdpa_fwd_scratch_bytes(int B, int H, int G, int q_len, int kv_len) {
  if (G <= 0 || H % G || H / G > 128) return -1;
  const int gs = H / G;
  const long long nT = (kv_len + kvb::F2_T - 1) / kvb::F2_T;
  const long long npos = 128 / gs;
  const long long nQT = (q_len + npos - 1) / npos;
  const long long bgt = kvb::f2_round4((long long)B * G * nT);
  long long words = 2 * bgt + (long long)B * G * nT * 128 + (long long)B * G * nQT * 128;
  const int n_split = f2_num_splits((long long)B * G * ((nQT + 1) / 2), nT);
  // partial outputs sized for the largest head size (256); the number of splits of a launch never exceeds this one's
  if (n_split > 1) words += kvb::f2_round4((long long)n_split * B * H * q_len) + (long long)n_split * B * H * q_len * 256;
  return words * 4;
}

// q (B,H,T,128) contiguous bf16; k, v (B,G,L,128) bf16 with batch / group strides k_sb, k_sg (elements);
// token_pos (B,G,L) int32 with strides, or NULL (slot j holds token j); out (B,T,H,128) bf16;
// lse (B,H,T) fp32 or NULL; weights (B,G,L) fp32 or NULL.
// head_size: 128 or 64 (the last axis of q, k, v, out); q_sb, q_sh: batch and head strides of q in elements (0, 0:
// contiguous (B,H,T,D); rows of one head are always head_size apart), so that a slice of positions of a longer
// (B,H,T',D) tensor is read in place; window: sliding window in tokens (0: none); softcap: logit soft-capping
// threshold (0: none).
extern "C" int kvb_sdpa_fwd_ex(const void* q, const void* k, const void* v, const int32_t* token_pos, void* out, float* lse,
                                float* weights, void* scratch, int B, int H, int G, int q_len, int kv_len, int head_size,
                                long long q_sb, long long q_sh, long long k_sb, long long k_sg, long long tp_sb, long long tp_sg,
                                float scale, int input_pos, int window, float softcap, int* status, void* stream);

extern "C" int kvb_sdpa_fwd(const void* q, const void* k, const void* v, const int32_t* token_pos, void* out, float* lse,
                             float* weights, void* scratch, int B, int H, int G, int q_len, int kv_len, long long k_sb,
                             long long k_sg, long long tp_sb, long long tp_sg, float scale, int input_pos, int* status,
                             void* stream) {
  return kvb_sdpa_fwd_ex(q, k, v, token_pos, out, lse, weights, scratch, B, H, G, q_len, kv_len, 128, 0, 0, k_sb, k_sg, tp_sb,
                         tp_sg, scale, input_pos, 0, 0.f, status, stream);
}

extern "C" int kvb_sdpa_fwd_ex(const void* q, const void* k, const void* v, const int32_t* token_pos, void* out, float* lse,
                                float* weights, void* scratch, int B, int H, int G, int q_len, int kv_len, int head_size,
                                long long q_sb, long long q_sh, long long k_sb, long long k_sg, long long tp_sb, long long tp_sg,
                                float scale, int input_pos, int window, float softcap, int* status, void* stream) {
  using namespace kvb;
  if (window < 0 || softcap < 0.f || (softcap > 0.f && scale <= 0.f)) return KVB_ERR_ARG;
  if (head_size != 128 && head_size != 64 && head_size != 256) return KVB_ERR_UNSUPPORTED;
  if (q_sh == 0) q_sh = (long long)q_len * head_size;
  if (q_sb == 0) q_sb = (long long)H * q_sh;
  if ((q_sb % 8) || (q_sh % 8) || q_sh < (long long)q_len * head_size) return KVB_ERR_ALIGN;
  if (B <= 0 || H <= 0 || G <= 0 || q_len <= 0 || kv_len <= 0 || H % G) return KVB_ERR_ARG;
  const int gs = H / G;
  if (gs > 128) return KVB_ERR_UNSUPPORTED;
  if ((k_sb % 8) || (k_sg % 8)) return KVB_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(scratch)) & 15)
    return KVB_ERR_ALIGN;
  cudaStream_t s = (cudaStream_t)stream;
  F2Params p;
  p.B = B; p.H = H; p.G = G; p.T = q_len; p.L = kv_len;
  p.gs = gs; p.npos = 128 / gs; p.rows_used = p.npos * gs;
  p.nT = (kv_len + F2_T - 1) / F2_T;
  p.nQT = (q_len + p.npos - 1) / p.npos;
  const long long bgt = f2_round4((long long)B * G * p.nT);
  int32_t* sc = reinterpret_cast<int32_t*>(scratch);
  int32_t* tmin = sc;
  int32_t* tmax = sc + bgt;
  int32_t* pos = sc + 2 * bgt;
  float* lse2 = reinterpret_cast<float*>(pos + (long long)B * G * p.nT * 128);
  p.tile_min = tmin; p.tile_max = tmax; p.pos = pos; p.lse2 = lse2;
  p.out = (__nv_bfloat16*)out; p.lse = lse; p.weights = weights;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.inv_gs = 1.f / gs;
  p.input_pos = input_pos; p.status = status;
  p.trace = g_f2_trace;
  p.window = window;
  p.cap_pre = softcap > 0.f ? scale / softcap : 0.f;
  p.cap_post = softcap > 0.f ? softcap / scale : 0.f;

  CUtensorMap tmQ, tmK, tmV;
  int rc;
  // Q (B,H,T,D) read position-major: dims (D, H, T, B) with strides (T·D, D, H·T·D); box = 64 x gs x npos
  const uint64_t hd = (uint64_t)head_size;
  if ((rc = f2_make_tmap(&tmQ, q, hd, H, q_len, B, (uint64_t)q_sh, hd, (uint64_t)q_sb, 64, gs, p.npos))) return rc;
  // K, V (B,G,L,D) with strides: dims (D, L, G, B); box = 64 x 128 x 1
  if ((rc = f2_make_tmap(&tmK, k, hd, kv_len, G, B, hd, k_sg, k_sb, 64, F2_T, 1))) return rc;
  if ((rc = f2_make_tmap(&tmV, v, hd, kv_len, G, B, hd, k_sg, k_sb, 64, F2_T, 1))) return rc;

  f2_prepare_kernel<<<B * G * p.nT, F2_T, 0, s>>>(token_pos, tmin, tmax, pos, G, kv_len, p.nT, tp_sb, tp_sg);
  const int nPair = head_size == 256 ? p.nQT : (p.nQT + 1) / 2;  // head size 256: one query tile per CTA
  p.n_split = f2_num_splits((long long)B * G * nPair, p.nT);
  p.tiles_per_split = (p.nT + p.n_split - 1) / p.n_split;
  p.part_lse2 = lse2 + (long long)B * G * p.nQT * 128;
  p.part_o = p.part_lse2 + f2_round4((long long)p.n_split * B * H * q_len);
  const bool gen = window > 0 || softcap > 0.f;
  if (head_size == 256) return f3_launch(tmQ, tmK, tmV, p, gen, s);
  if (head_size == 128) return gen ? f2_launch<true, 128>(tmQ, tmK, tmV, p, s) : f2_launch<false, 128>(tmQ, tmK, tmV, p, s);
  return gen ? f2_launch<true, 64>(tmQ, tmK, tmV, p, s) : f2_launch<false, 64>(tmQ, tmK, tmV, p, s);
}
