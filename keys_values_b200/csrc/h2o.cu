// H2O policy update on the device: scores += weights, optional age normalisation,
// and selection of the k lowest-scoring evictable slots, ascending — all in one
// kernel, one CTA per (batch row, KV head), so the next cache write can consume
// the result without the host ever seeing it.
//
// Selection = 4-pass radix select on the order-preserving integer image of the
// fp32 scores (exact k-th value), an index-ordered compaction (ties are resolved
// towards lower slot indices, so results are run-to-run identical), then a
// bitonic sort of the k survivors.
//
// Replaces the ATen add + topk/argsort of keys_values/kvcache/attn_weights.py:637-783
// and h2o.py:146-199.
#include "common.cuh"
#include "kvb200.h"

namespace kvb {

constexpr int H2O_THREADS = 1024;
constexpr int H2O_MAX_K = 4096;
constexpr int H2O_SMALL_K = 32;  // up to here the slots are found by repeated block-wide minima

__device__ __forceinline__ uint32_t ordered_key(float f) {
  uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(H2O_THREADS, 1)
h2o_update_kernel(float* __restrict__ scores, const float* __restrict__ weights, const int32_t* __restrict__ token_pos,
                  int32_t* __restrict__ out_idx, int G, int C, int n_evict, int k_select, int kpad, int normalize, int input_pos,
                  int prefill_length, long long sc_sb, long long sc_sg, long long tp_sb, long long tp_sg,
                  const int* __restrict__ pos_ptr) {
  extern __shared__ uint32_t smem_u[];
  uint32_t* keys = smem_u;                       // [n_evict] selection keys
  uint32_t* sort_key = keys + n_evict;           // [kpad]
  int32_t* sort_idx = (int32_t*)(sort_key + kpad);  // [kpad]
  __shared__ uint32_t hist[256];
  __shared__ uint32_t scan_less[H2O_THREADS / 32], scan_eq[H2O_THREADS / 32];
  __shared__ uint32_t sh_prefix, sh_remaining, sh_nless;

  const int b = blockIdx.x / G, g = blockIdx.x % G;
  float* sc = scores + b * sc_sb + g * sc_sg;
  const float* w = weights ? weights + ((long long)b * G + g) * C : nullptr;  // null: select only
  const int32_t* tp = token_pos ? token_pos + b * tp_sb + g * tp_sg : nullptr;
  const int tid = threadIdx.x;
  if (pos_ptr) input_pos = *pos_ptr + 1;  // device-resident position of the token just written; scores are aged to the next one

  // 1) accumulate and build selection keys. Only B·G CTAs run, so the pass is bound by the latency of
  //    its loads: with 16-byte accesses all of a row's scores and weights are requested in one or two
  //    rounds (4 x 4 slots per thread and round).
  auto key_of = [&](float s, int j, int t) {
    float sel = s;
    if (normalize) {
      if (t < prefill_length - 1) t = prefill_length - 1;
      sel = __fdiv_rn(s, (float)(input_pos - t));
    }
    keys[j] = ordered_key(sel);
  };
  const bool vec = (C & 3) == 0 && ((reinterpret_cast<uintptr_t>(sc) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(tp)) & 15) == 0;
  if (vec) {
    constexpr int UB = 4;
    const int nv = C >> 2;
    for (int q0 = tid; q0 < nv; q0 += UB * H2O_THREADS) {
      float4 sv[UB], wv[UB];
      int4 tv[UB];
#pragma unroll
      for (int u = 0; u < UB; ++u) {
        const int q = q0 + u * H2O_THREADS;
        sv[u] = wv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        tv[u] = make_int4(0, 0, 0, 0);
        if (q < nv) {
          sv[u] = reinterpret_cast<const float4*>(sc)[q];
          if (w) wv[u] = reinterpret_cast<const float4*>(w)[q];
          if (normalize && 4 * q < n_evict) tv[u] = reinterpret_cast<const int4*>(tp)[q];
        }
      }
#pragma unroll
      for (int u = 0; u < UB; ++u) {
        const int q = q0 + u * H2O_THREADS;
        if (q >= nv) break;
        const float4 s4 = make_float4(sv[u].x + wv[u].x, sv[u].y + wv[u].y, sv[u].z + wv[u].z, sv[u].w + wv[u].w);
        if (w) reinterpret_cast<float4*>(sc)[q] = s4;
        const int j = 4 * q;
        if (j < n_evict) key_of(s4.x, j, tv[u].x);
        if (j + 1 < n_evict) key_of(s4.y, j + 1, tv[u].y);
        if (j + 2 < n_evict) key_of(s4.z, j + 2, tv[u].z);
        if (j + 3 < n_evict) key_of(s4.w, j + 3, tv[u].w);
      }
    }
  } else {
    for (int j = tid; j < C; j += H2O_THREADS) {
      const float s = sc[j] + (w ? w[j] : 0.f);
      if (w) sc[j] = s;
      if (j < n_evict) key_of(s, j, normalize ? tp[j] : 0);
    }
  }
  if (tid == 0) {
    sh_prefix = 0;
    sh_remaining = (uint32_t)k_select;
    sh_nless = 0;
  }
  __syncthreads();

  // 2a) few slots (the selection after a single-token step): k block-wide minima of (key, index),
  //     each removed before the next; the same order as the general path (ascending key, ties by index)
  if (k_select <= H2O_SMALL_K) {
    __shared__ unsigned long long wmin[H2O_THREADS / 32];
    __shared__ unsigned long long chosen;
    int32_t* out = out_idx + ((long long)b * G + g) * k_select;
    // every thread keeps the minimum of its own slots (j = tid, tid + 1024, ...); after a slot has
    // been taken only its owner scans again
    auto scan = [&]() {
      unsigned long long best = ~0ull;
      for (int j = tid; j < n_evict; j += H2O_THREADS) {
        const unsigned long long cand = ((unsigned long long)keys[j] << 32) | (unsigned)j;
        best = cand < best ? cand : best;
      }
      return best;
    };
    unsigned long long mine = scan();
    for (int it = 0; it < k_select; ++it) {
      unsigned long long best = mine;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
        best = other < best ? other : best;
      }
      if ((tid & 31) == 0) wmin[tid >> 5] = best;
      __syncthreads();
      if (tid < 32) {
        unsigned long long v = wmin[tid];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
          v = other < v ? other : v;
        }
        if (tid == 0) {
          chosen = v;
          const int idx = (int)(v & 0xffffffffu);
          out[it] = idx;
          keys[idx] = 0xFFFFFFFFu;  // scores are finite, so no live key has this value: the slot is out of the race
        }
      }
      __syncthreads();
      if ((int)(chosen & 0xffffffffu) % H2O_THREADS == tid) mine = scan();
    }
    return;
  }
  // 2) radix select: find the k-th smallest key exactly
  uint32_t mask = 0;
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    for (int i = tid; i < 256; i += H2O_THREADS) hist[i] = 0;
    __syncthreads();
    const uint32_t prefix = sh_prefix;
    for (int j = tid; j < n_evict; j += H2O_THREADS) {
      const uint32_t kx = keys[j];
      if ((kx & mask) == prefix) atomicAdd(&hist[(kx >> shift) & 0xFF], 1u);
    }
    __syncthreads();
    if (tid == 0) {
      uint32_t rem = sh_remaining, acc = 0;
      int bin = 0;
      for (; bin < 256; ++bin) {
        if (acc + hist[bin] >= rem) break;
        acc += hist[bin];
      }
      if (bin > 255) bin = 255;
      sh_nless += acc;
      sh_remaining = rem - acc;
      sh_prefix = prefix | ((uint32_t)bin << shift);
    }
    mask |= 0xFFu << shift;
    __syncthreads();
  }
  const uint32_t kth = sh_prefix;
  const uint32_t n_less = sh_nless;
  const uint32_t n_eq_take = (uint32_t)k_select - n_less;

  // 3) index-ordered compaction of {key < kth} and the first n_eq_take of {key == kth}
  const int per = (n_evict + H2O_THREADS - 1) / H2O_THREADS;
  const int j0 = tid * per, j1 = min(j0 + per, n_evict);
  uint32_t c_less = 0, c_eq = 0;
  for (int j = j0; j < j1; ++j) {
    const uint32_t kx = keys[j];
    c_less += kx < kth;
    c_eq += kx == kth;
  }
  // block exclusive scan of (c_less, c_eq)
  uint32_t i_less = c_less, i_eq = c_eq;
  const int lane = tid & 31, warp = tid >> 5;
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t a = __shfl_up_sync(0xffffffffu, i_less, o), e = __shfl_up_sync(0xffffffffu, i_eq, o);
    if (lane >= o) {
      i_less += a;
      i_eq += e;
    }
  }
  if (lane == 31) {
    scan_less[warp] = i_less;
    scan_eq[warp] = i_eq;
  }
  __syncthreads();
  if (warp == 0) {
    uint32_t a = scan_less[lane], e = scan_eq[lane];
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t a2 = __shfl_up_sync(0xffffffffu, a, o), e2 = __shfl_up_sync(0xffffffffu, e, o);
      if (lane >= o) {
        a += a2;
        e += e2;
      }
    }
    scan_less[lane] = a;
    scan_eq[lane] = e;
  }
  __syncthreads();
  uint32_t off_less = i_less - c_less + (warp ? scan_less[warp - 1] : 0);
  uint32_t off_eq = i_eq - c_eq + (warp ? scan_eq[warp - 1] : 0);
  for (int j = tid; j < kpad; j += H2O_THREADS) {
    sort_key[j] = 0xFFFFFFFFu;
    sort_idx[j] = 0x7FFFFFFF;
  }
  __syncthreads();
  for (int j = j0; j < j1; ++j) {
    const uint32_t kx = keys[j];
    if (kx < kth) {
      sort_key[off_less] = kx;
      sort_idx[off_less] = j;
      ++off_less;
    } else if (kx == kth) {
      if (off_eq < n_eq_take) {
        sort_key[n_less + off_eq] = kx;
        sort_idx[n_less + off_eq] = j;
      }
      ++off_eq;
    }
  }
  __syncthreads();

  // 4) bitonic sort of (key, idx) ascending
  for (int size = 2; size <= kpad; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int t = tid; t < kpad / 2; t += H2O_THREADS) {
        const int lo = 2 * t - (t & (stride - 1));
        const int hi = lo + stride;
        const bool up = (lo & size) == 0;
        const uint32_t ka = sort_key[lo], kb = sort_key[hi];
        const int32_t ia = sort_idx[lo], ib = sort_idx[hi];
        const bool gt = ka > kb || (ka == kb && ia > ib);
        if (gt == up) {
          sort_key[lo] = kb;
          sort_key[hi] = ka;
          sort_idx[lo] = ib;
          sort_idx[hi] = ia;
        }
      }
      __syncthreads();
    }
  }
  int32_t* out = out_idx + ((long long)b * G + g) * k_select;
  for (int j = tid; j < k_select; j += H2O_THREADS) out[j] = sort_idx[j];
}

}  // namespace kvb

extern "C" int kvb_h2o_update(float* scores, const float* weights, const int32_t* token_pos, int32_t* out_idx, int B, int G,
                              int C, int n_evictable, int k_select, int normalize, int input_pos, int prefill_length,
                              long long sc_sb, long long sc_sg, long long tp_sb, long long tp_sg, void* stream) {
  using namespace kvb;
  if (B <= 0 || G <= 0 || C <= 0 || n_evictable <= 0 || n_evictable > C || k_select <= 0 || k_select > n_evictable)
    return KVB_ERR_ARG;
  if (k_select > H2O_MAX_K) return KVB_ERR_UNSUPPORTED;
  if (normalize && !token_pos) return KVB_ERR_ARG;
  int kpad = 2;
  while (kpad < k_select) kpad <<= 1;
  const size_t smem = (size_t)n_evictable * 4 + (size_t)kpad * 8;
  if (smem > 200 * 1024) return KVB_ERR_TOO_LARGE;
  static kvb::PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(h2o_update_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  }
  h2o_update_kernel<<<B * G, H2O_THREADS, smem, (cudaStream_t)stream>>>(scores, weights, token_pos, out_idx, G, C, n_evictable,
                                                                       k_select, kpad, normalize, input_pos, prefill_length,
                                                                       sc_sb, sc_sg, tp_sb, tp_sg, kvb_position_source());
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}
