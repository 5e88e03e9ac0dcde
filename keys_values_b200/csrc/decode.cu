// GQA decode attention (one new query token per sequence) over a bf16, int8 or int4
// KV cache, with de-quantization fused into the tile load and the per-slot summed
// attention weights (H2O score input) as a second output.
//
//   split-KV: grid (B·G, n_splits, head blocks); every CTA scores 256 slots for (up to 8 of) the
//   H/G heads of its KV group, keeps the raw scores in a (B,H,L) scratch, accumulates its
//   partial (max, sum, O); a merge kernel combines the partials; a third kernel turns the raw
//   scores into weights[b,g,j] = (1/(H/G)) Σ_h exp(s_hj − lse_h). A warp reads four cache rows
//   at a time as whole 16-byte units (8 lanes per row), several loads in flight per lane: the
//   kernel is bound by the HBM read of the cache.
//
// The quantized storage is read directly: x = (q − zp)·scale is folded into the dot
// products (q·k = scale·(Σ q_i·code_i − zp·Σ q_i)), so no full-precision copy of the cache
// is ever materialised for decoding. The row of the token that is being decoded is
// taken in full precision from `k_new/v_new` (it has not been through quantization
// from the point of view of this step).
//
// Replaces csrc/kernels/sdpa_decode.cu of the reference (FlashInfer single-decode in a
// host loop over the batch, and its CUDA-core kernels with atomics) plus the per-token
// de/re-quantization of whole layers in keys_values/kvcache/quant_buffers.py:473-503.
#include <float.h>

#include "common.cuh"
#include "kvb200.h"

namespace kvb {

constexpr int DEC_D = 128;
constexpr int DEC_SPLIT = 256;    // slots per CTA
constexpr int DEC_THREADS = 128;  // 4 warps
constexpr int DEC_MAX_GS = 16;
constexpr int DEC_BATCH = 4;     // groups of four slots whose loads are issued together
constexpr int DEC_HB = 8;         // heads of a group handled by one CTA (more heads: more CTAs along z)

struct DecParams {
  const __nv_bfloat16* q;       // (B,H,D)
  const void* kq;               // (Bmax,G,C,Dq) codes or bf16
  const void* vq;
  const float *ks, *vs;         // (Bmax,G,C)
  const int32_t *kz, *vz;
  const __nv_bfloat16 *k_new, *v_new;  // (B,G,D) or nullptr
  const int32_t* new_slot;      // (B,G) or nullptr
  __nv_bfloat16* out;           // (B,H*D)
  float* weights;               // (B,G,L) or nullptr
  float* logits;                // (B,H,L)
  float* part_m;                // (B,H,nS)
  float* part_l;                // (B,H,nS)
  float* part_o;                // (B,H,nS,D)
  float* lse;                   // (B,H)
  int B, H, G, L, C, gs, nS;
  float scale;
};

// Feature that element k (0..15) of a lane's row fragment holds; fl = lane & 7.
//   bf16 : two 16-byte units, fl and fl + 8        -> features 8 fl + k, 64 + 8 fl + (k − 8)
//   int8 : one 16-byte unit                        -> features 16 fl + k
//   int4 : 8 bytes, byte i = (feature i, feature i + 64) as (high, low) nibble
//                                                  -> features 8 fl + k, 64 + 8 fl + (k − 8)
template <int BITS>
__device__ __forceinline__ int dec_feature(int fl, int k) {
  if (BITS == 8) return 16 * fl + k;
  return k < 8 ? 8 * fl + k : 64 + 8 * fl + (k - 8);
}

// Byte `idx` of w as a float without the conversion unit: the byte becomes the low mantissa bits
// of 2^23 (one PRMT), and 2^23 is subtracted (one FADD).
__device__ __forceinline__ float dec_u8_to_f32(uint32_t w, int idx) {
  return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440u | (uint32_t)idx)) - 8388608.f;
}

// Raw 16 elements of row `row` for feature lane fl (32 bytes of bf16, 16 of int8, 8 of int4).
template <int BITS>
__device__ __forceinline__ void dec_load_raw(const void* base, long long row, int fl, uint4& a, uint4& c) {
  if (BITS == 16) {
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + row * DEC_D);
    a = __ldg(p + fl);
    c = __ldg(p + fl + 8);
  } else if (BITS == 8) {
    a = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(base) + row * DEC_D) + fl);
  } else {
    const uint2 v = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(base) + row * (DEC_D / 2)) + fl);
    a.x = v.x;
    a.y = v.y;
  }
}

// ... as floats (codes are not de-quantized here).
template <int BITS>
__device__ __forceinline__ void dec_convert(const uint4& a, const uint4& c, float* x) {
  if (BITS == 16) {
    const __nv_bfloat162* ha = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* hc = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(ha[j]), g = __bfloat1622float2(hc[j]);
      x[2 * j] = f.x; x[2 * j + 1] = f.y;
      x[8 + 2 * j] = g.x; x[8 + 2 * j + 1] = g.y;
    }
  } else if (BITS == 8) {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 16; ++j) x[j] = dec_u8_to_f32(w[j >> 2], j & 3);
  } else {
    const uint32_t w[2] = {a.x, a.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t byte = (w[j >> 2] >> (8 * (j & 3))) & 0xFFu;
      x[j] = __uint_as_float(0x4B000000u | (byte >> 4)) - 8388608.f;
      x[8 + j] = __uint_as_float(0x4B000000u | (byte & 0xFu)) - 8388608.f;
    }
  }
}

// One CTA = (batch, KV group, split of DEC_SPLIT slots, block of GS heads). A warp handles four
// slots at a time: 8 lanes per slot, 16 features per lane, so that a row is read as whole
// 16-byte units, coalesced, several loads in flight per lane. Scores are reduced over the 8
// lanes by shuffles; p·V accumulates in registers (GS x 16 per lane) and is reduced once.
template <int BITS, int GS>
__global__ void __launch_bounds__(DEC_THREADS)
decode_partial_kernel(const DecParams p) {
  __shared__ float sc[GS][DEC_SPLIT];           // scores, later p · v_scale
  __shared__ float red[DEC_THREADS / 32][GS];   // per-warp reductions
  __shared__ float stat[2][GS];                 // block max, Σ p · v_scale · v_zero_point
  __shared__ float ored[DEC_THREADS / 32][GS][DEC_D];
  const int bg = blockIdx.x, split = blockIdx.y, h0 = blockIdx.z * GS;
  const int b = bg / p.G, g = bg % p.G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int fl = lane & 7, sub = lane >> 3;
  const int j0 = split * DEC_SPLIT, j1 = min(j0 + DEC_SPLIT, p.L);
  const int n = j1 - j0;
  const long long row0 = ((long long)b * p.G + g) * p.C;
  const int ns = p.new_slot ? p.new_slot[b * p.G + g] : -1;
  const long long head0 = (long long)b * p.H + g * p.gs + h0;  // first head of this CTA

  // query fragment of this lane and Σ_i q_i per head (for the zero-point term)
  float qf[GS][16], qsum[GS];
#pragma unroll
  for (int h = 0; h < GS; ++h) {
    const __nv_bfloat16* qr = p.q + (head0 + h) * DEC_D;
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      qf[h][k] = __bfloat162float(qr[dec_feature<BITS>(fl, k)]);
      s += qf[h][k];
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    qsum[h] = s;
  }

  // ---- pass A: raw scores
  float lmax[GS];
#pragma unroll
  for (int h = 0; h < GS; ++h) lmax[h] = -FLT_MAX;
  // DEC_BATCH groups of four slots per iteration: all their loads are issued before the first
  // conversion, so that 8 x 16 bytes (bf16) are in flight per lane
  for (int jb0 = warp * 4; jb0 < n; jb0 += DEC_BATCH * (DEC_THREADS / 8)) {  // warp-uniform trip count (shuffles inside)
    uint4 ra[DEC_BATCH], rc[DEC_BATCH];
    float ksc[DEC_BATCH], kz[DEC_BATCH];
#pragma unroll
    for (int q = 0; q < DEC_BATCH; ++q) {
      const int jj = min(jb0 + q * (DEC_THREADS / 8) + sub, n - 1);  // rows beyond the split re-read its last row
      dec_load_raw<BITS>(p.kq, row0 + j0 + jj, fl, ra[q], rc[q]);
      ksc[q] = 1.f;
      kz[q] = 0.f;
      if (BITS != 16) {
        ksc[q] = __ldg(p.ks + row0 + j0 + jj);
        kz[q] = (float)__ldg(p.kz + row0 + j0 + jj);
      }
    }
#pragma unroll
    for (int q = 0; q < DEC_BATCH; ++q) {
      const int jj = jb0 + q * (DEC_THREADS / 8) + sub;
      const bool valid = jj < n;
      const int j = j0 + jj;
      float x[16];
      dec_convert<BITS>(ra[q], rc[q], x);
      float kscale = ksc[q], kzp = kz[q];
      if (valid && j == ns) {  // the token being decoded: exact values instead of the cache row
        const __nv_bfloat16* kr = p.k_new + ((long long)b * p.G + g) * DEC_D;
#pragma unroll
        for (int k = 0; k < 16; ++k) x[k] = __bfloat162float(kr[dec_feature<BITS>(fl, k)]);
        kscale = 1.f;
        kzp = 0.f;
      }
#pragma unroll
      for (int h = 0; h < GS; ++h) {
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < 16; ++k) acc = fmaf(qf[h][k], x[k], acc);
        acc += __shfl_xor_sync(0xffffffffu, acc, 1);
        acc += __shfl_xor_sync(0xffffffffu, acc, 2);
        acc += __shfl_xor_sync(0xffffffffu, acc, 4);
        const float sv = p.scale * kscale * (acc - kzp * qsum[h]);
        if (valid) lmax[h] = fmaxf(lmax[h], sv);
        if (fl == 0 && valid) {
          sc[h][jj] = sv;
          p.logits[(head0 + h) * p.L + j] = sv;
        }
      }
    }
  }
#pragma unroll
  for (int h = 0; h < GS; ++h) {
    const float m = warp_max(lmax[h]);
    if (lane == 0) red[warp][h] = m;
  }
  __syncthreads();
  if (tid < GS) {
    float m = -FLT_MAX;
    for (int w = 0; w < DEC_THREADS / 32; ++w) m = fmaxf(m, red[w][tid]);
    stat[0][tid] = m;
  }
  __syncthreads();
  // ---- p = exp(s − m) with the V scale folded in; block sums of p and of p · v_scale · v_zp
  float lsum[GS], zsum[GS];
#pragma unroll
  for (int h = 0; h < GS; ++h) lsum[h] = zsum[h] = 0.f;
  for (int jj = tid; jj < n; jj += DEC_THREADS) {
    const int j = j0 + jj;
    float vscale = 1.f, vzp = 0.f;
    if (BITS != 16 && j != ns) {
      vscale = __ldg(p.vs + row0 + j);
      vzp = (float)__ldg(p.vz + row0 + j);
    }
#pragma unroll
    for (int h = 0; h < GS; ++h) {
      const float pr = __expf(sc[h][jj] - stat[0][h]);
      lsum[h] += pr;
      zsum[h] += pr * vscale * vzp;
      sc[h][jj] = pr * vscale;
    }
  }
  __syncthreads();  // red is reused
#pragma unroll
  for (int h = 0; h < GS; ++h) {
    const float s1 = warp_sum(lsum[h]), s2 = warp_sum(zsum[h]);
    if (lane == 0) {
      red[warp][h] = s1;
      ored[warp][h][0] = s2;
    }
  }
  __syncthreads();
  if (tid < GS) {
    float s1 = 0.f, s2 = 0.f;
    for (int w = 0; w < DEC_THREADS / 32; ++w) {
      s1 += red[w][tid];
      s2 += ored[w][tid][0];
    }
    const long long idx = (head0 + tid) * p.nS + split;
    p.part_m[idx] = stat[0][tid];
    p.part_l[idx] = s1;
    stat[1][tid] = s2;
  }
  __syncthreads();
  // ---- pass B: O += (p · v_scale) · code ; the zero-point term is subtracted once at the end
  float acc[GS][16];
#pragma unroll
  for (int h = 0; h < GS; ++h)
#pragma unroll
    for (int k = 0; k < 16; ++k) acc[h][k] = 0.f;
  for (int jb0 = warp * 4; jb0 < n; jb0 += DEC_BATCH * (DEC_THREADS / 8)) {
    uint4 ra[DEC_BATCH], rc[DEC_BATCH];
#pragma unroll
    for (int q = 0; q < DEC_BATCH; ++q) {
      const int jj = min(jb0 + q * (DEC_THREADS / 8) + sub, n - 1);
      dec_load_raw<BITS>(p.vq, row0 + j0 + jj, fl, ra[q], rc[q]);
    }
#pragma unroll
    for (int q = 0; q < DEC_BATCH; ++q) {
      const int jj = jb0 + q * (DEC_THREADS / 8) + sub;
      const bool valid = jj < n;
      float x[16];
      dec_convert<BITS>(ra[q], rc[q], x);
      if (valid && j0 + jj == ns) {
        const __nv_bfloat16* vr = p.v_new + ((long long)b * p.G + g) * DEC_D;
#pragma unroll
        for (int k = 0; k < 16; ++k) x[k] = __bfloat162float(vr[dec_feature<BITS>(fl, k)]);
      }
#pragma unroll
      for (int h = 0; h < GS; ++h) {
        const float ps = valid ? sc[h][jj] : 0.f;
#pragma unroll
        for (int k = 0; k < 16; ++k) acc[h][k] = fmaf(ps, x[k], acc[h][k]);
      }
    }
  }
  // reduce over the four slot lanes of the warp, then over the warps
#pragma unroll
  for (int h = 0; h < GS; ++h)
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      float v = acc[h][k];
      v += __shfl_xor_sync(0xffffffffu, v, 8);
      v += __shfl_xor_sync(0xffffffffu, v, 16);
      if (sub == 0) ored[warp][h][dec_feature<BITS>(fl, k)] = v;
    }
  __syncthreads();
  for (int i = tid; i < GS * DEC_D; i += DEC_THREADS) {
    const int h = i / DEC_D, d = i % DEC_D;
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_THREADS / 32; ++w) s += ored[w][h][d];
    p.part_o[((head0 + h) * p.nS + split) * DEC_D + d] = s - stat[1][h];
  }
}

__global__ void decode_merge_kernel(const DecParams p) {
  const int bh = blockIdx.x, d = threadIdx.x;  // 128 threads
  const float* pm = p.part_m + (long long)bh * p.nS;
  const float* pl = p.part_l + (long long)bh * p.nS;
  float M = -FLT_MAX;
  for (int s = 0; s < p.nS; ++s) M = fmaxf(M, pm[s]);
  float Lsum = 0.f, o = 0.f;
  for (int s = 0; s < p.nS; ++s) {
    const float w = __expf(pm[s] - M);
    Lsum += pl[s] * w;
    o += p.part_o[((long long)bh * p.nS + s) * DEC_D + d] * w;
  }
  p.out[(long long)bh * DEC_D + d] = __float2bfloat16_rn(o / Lsum);
  if (d == 0) p.lse[bh] = M + logf(Lsum);
}

__global__ void decode_weights_kernel(const DecParams p) {
  const int bg = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= p.L) return;
  const int b = bg / p.G, g = bg % p.G;
  float s = 0.f;
  for (int h = 0; h < p.gs; ++h) {
    const long long bh = (long long)b * p.H + g * p.gs + h;
    s += __expf(p.logits[bh * p.L + j] - p.lse[bh]);
  }
  p.weights[(long long)bg * p.L + j] = s / p.gs;
}

}  // namespace kvb

extern "C" long long kvb_decode_scratch_bytes(int B, int H, int L) {
  const long long nS = (L + kvb::DEC_SPLIT - 1) / kvb::DEC_SPLIT;
  return ((long long)B * H * L + 2LL * B * H * nS + (long long)B * H * nS * kvb::DEC_D + (long long)B * H) * 4;
}

extern "C" int kvb_decode_attn(const void* q, const void* kq, const void* vq, const float* ks, const int32_t* kz, const float* vs,
                               const int32_t* vz, const void* k_new, const void* v_new, const int32_t* new_slot, void* out,
                               float* weights, void* scratch, int B, int H, int G, int L, int C, int bits, float scale,
                               void* stream) {
  using namespace kvb;
  if (B <= 0 || H <= 0 || G <= 0 || L <= 0 || C < L || H % G) return KVB_ERR_ARG;
  const int gs = H / G;
  if (gs > DEC_MAX_GS) return KVB_ERR_UNSUPPORTED;
  if (bits != 16 && bits != 8 && bits != 4) return KVB_ERR_ARG;
  if (bits != 16 && (!ks || !kz || !vs || !vz)) return KVB_ERR_ARG;
  DecParams p;
  p.q = (const __nv_bfloat16*)q; p.kq = kq; p.vq = vq; p.ks = ks; p.kz = kz; p.vs = vs; p.vz = vz;
  p.k_new = (const __nv_bfloat16*)k_new; p.v_new = (const __nv_bfloat16*)v_new; p.new_slot = k_new ? new_slot : nullptr;
  p.out = (__nv_bfloat16*)out; p.weights = weights;
  p.B = B; p.H = H; p.G = G; p.L = L; p.C = C; p.gs = gs; p.scale = scale;
  p.nS = (L + DEC_SPLIT - 1) / DEC_SPLIT;
  float* sc = reinterpret_cast<float*>(scratch);
  p.logits = sc; sc += (long long)B * H * L;
  p.part_m = sc; sc += (long long)B * H * p.nS;
  p.part_l = sc; sc += (long long)B * H * p.nS;
  p.part_o = sc; sc += (long long)B * H * p.nS * DEC_D;
  p.lse = sc;
  cudaStream_t s = (cudaStream_t)stream;
  // heads of a group per CTA: the group size up to DEC_HB; larger groups use more CTAs along z
  const int hb = gs < DEC_HB ? gs : DEC_HB;
  if (gs % hb) return KVB_ERR_UNSUPPORTED;
  dim3 grid(B * G, p.nS, gs / hb);
#define KVB_DEC_LAUNCH(BITS_)                                                            \
  switch (hb) {                                                                          \
    case 1: decode_partial_kernel<BITS_, 1><<<grid, DEC_THREADS, 0, s>>>(p); break;      \
    case 2: decode_partial_kernel<BITS_, 2><<<grid, DEC_THREADS, 0, s>>>(p); break;      \
    case 4: decode_partial_kernel<BITS_, 4><<<grid, DEC_THREADS, 0, s>>>(p); break;      \
    case 8: decode_partial_kernel<BITS_, 8><<<grid, DEC_THREADS, 0, s>>>(p); break;      \
    default: return KVB_ERR_UNSUPPORTED;                                                 \
  }
  if (bits == 16) { KVB_DEC_LAUNCH(16) }
  else if (bits == 8) { KVB_DEC_LAUNCH(8) }
  else { KVB_DEC_LAUNCH(4) }
#undef KVB_DEC_LAUNCH
  decode_merge_kernel<<<B * H, DEC_D, 0, s>>>(p);
  if (weights) {
    dim3 g2((L + 255) / 256, B * G);
    decode_weights_kernel<<<g2, 256, 0, s>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

// ------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// Some callers cannot hand this library a scratch buffer because they cannot create one
// at the point of the call: code running while the CUDA caching allocator is frozen,
// latency-critical serving loops that pre-plan every byte of device memory at start-up and
// forbid cudaMalloc afterwards, or host runtimes in other languages that only link the C
// symbols and have no tensor allocator at all. For them the workspace of the decode kernels
// (raw scores, per-split partial results, log-sum-exp) lives in a fixed array inside this
// library's device image. Every GPU that loads the library holds these
// KVB_DECODE_STATIC_SCRATCH_BYTES until the process exits.
//
// Host code must never hand the array's name to a kernel: in host code the name is only a
// stand-in for the symbol, not a device address. The device address is looked up with
// cudaGetSymbolAddress, once per device, with that device current, and cached here.
// ------------------------------------------------------------------------------------
#define KVB_DECODE_STATIC_SCRATCH_BYTES (8u << 20)
#define KVB_DECODE_STATIC_MAX_DEVICES 64

static __device__ __align__(256) unsigned char kvb_decode_static_scratch[KVB_DECODE_STATIC_SCRATCH_BYTES];
static void* kvb_decode_static_scratch_addr[KVB_DECODE_STATIC_MAX_DEVICES] = {nullptr};

extern "C" long long kvb_decode_attn_noalloc_max_bytes(void) { return (long long)KVB_DECODE_STATIC_SCRATCH_BYTES; }

extern "C" int kvb_decode_attn_noalloc(const void* q, const void* kq, const void* vq, const float* ks, const int32_t* kz,
                                       const float* vs, const int32_t* vz, const void* k_new, const void* v_new,
                                       const int32_t* new_slot, void* out, float* weights, int B, int H, int G, int L, int C,
                                       int bits, float scale, void* stream) {
  if (B <= 0 || H <= 0 || L <= 0) return KVB_ERR_ARG;
  // workspace needed by this problem size; refuse what does not fit the fixed array
  const long long need = kvb_decode_scratch_bytes(B, H, L);
  if (need > (long long)KVB_DECODE_STATIC_SCRATCH_BYTES) return KVB_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= KVB_DECODE_STATIC_MAX_DEVICES) return KVB_ERR_CUDA;
  if (kvb_decode_static_scratch_addr[dev] == nullptr) {
    // first call on this device: resolve the device address of the array (no allocation)
    void* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, kvb_decode_static_scratch) != cudaSuccess || ptr == nullptr) return KVB_ERR_CUDA;
    kvb_decode_static_scratch_addr[dev] = ptr;
  }
  // Every word of the workspace that the kernels read (scores, partial max/sum/output,
  // log-sum-exp) is written earlier in the same call, so nothing has to be cleared.
  return kvb_decode_attn(q, kq, vq, ks, kz, vs, vz, k_new, v_new, new_slot, out, weights, kvb_decode_static_scratch_addr[dev], B, H,
                         G, L, C, bits, scale, stream);
}
