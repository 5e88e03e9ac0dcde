// GQA decode attention (one new query token per sequence) over a bf16, int8 or int4
// KV cache, with de-quantization fused into the tile load and the per-slot summed
// attention weights (H2O score input) as a second output.
//
//   split-KV: grid (B·G, n_splits); every CTA scores SPLIT slots for all H/G heads of
//   its KV group, keeps the raw scores in a (B,H,L) scratch, accumulates its partial
//   (max, sum, O); a merge kernel combines the partials; a third kernel turns the raw
//   scores into weights[b,g,j] = (1/(H/G)) Σ_h exp(s_hj − lse_h).
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
constexpr int DEC_SPLIT = 1024;
constexpr int DEC_THREADS = 256;
constexpr int DEC_MAX_GS = 16;

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

template <int BITS>
__device__ __forceinline__ void load_row_f32(const void* base, long long row, float* x) {
  // x[128] <- codes (or bf16 values) of one row
  if (BITS == 16) {
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + row * DEC_D);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      uint4 v = p[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(h[j]);
        x[i * 8 + 2 * j] = f.x;
        x[i * 8 + 2 * j + 1] = f.y;
      }
    }
  } else if (BITS == 8) {
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(base) + row * DEC_D);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint4 v = p[i];
      const uint8_t* c = reinterpret_cast<const uint8_t*>(&v);
#pragma unroll
      for (int j = 0; j < 16; ++j) x[i * 16 + j] = (float)c[j];
    }
  } else {
    const uint4* p = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(base) + row * (DEC_D / 2));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 v = p[i];
      const uint8_t* c = reinterpret_cast<const uint8_t*>(&v);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        x[i * 16 + j] = (float)(c[j] >> 4);
        x[64 + i * 16 + j] = (float)(c[j] & 0xF);
      }
    }
  }
}

template <int BITS>
__global__ void __launch_bounds__(DEC_THREADS)
decode_partial_kernel(const DecParams p) {
  extern __shared__ float sm[];
  float* q_s = sm;                                  // [gs][128]
  float* qsum = q_s + p.gs * DEC_D;                 // [gs]
  float* sc = qsum + DEC_MAX_GS;                    // [gs][SPLIT] scores, later p·scale
  float* pz = sc + p.gs * DEC_SPLIT;                // [gs][SPLIT] p·scale·zp
  float* red = pz + p.gs * DEC_SPLIT;               // [8 warps][gs] reductions / [8][gs][128] at the end
  const int bg = blockIdx.x, split = blockIdx.y;
  const int b = bg / p.G, g = bg % p.G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int j0 = split * DEC_SPLIT, j1 = min(j0 + DEC_SPLIT, p.L);
  const int n = j1 - j0;
  const long long row0 = ((long long)b * p.G + g) * p.C;
  const int gs = p.gs;
  const int ns = p.new_slot ? p.new_slot[b * p.G + g] : -1;

  for (int i = tid; i < gs * DEC_D; i += DEC_THREADS) q_s[i] = __bfloat162float(p.q[((long long)b * p.H + g * gs) * DEC_D + i]);
  __syncthreads();
  if (tid < gs) {
    float s = 0.f;
    for (int i = 0; i < DEC_D; ++i) s += q_s[tid * DEC_D + i];
    qsum[tid] = s;
  }
  __syncthreads();

  // ---- pass A: raw scores, one slot per thread
  float lmax[DEC_MAX_GS];
#pragma unroll
  for (int h = 0; h < DEC_MAX_GS; ++h) lmax[h] = -FLT_MAX;
  for (int jj = tid; jj < n; jj += DEC_THREADS) {
    const int j = j0 + jj;
    float x[DEC_D];
    float kscale = 1.f, kzp = 0.f;
    if (j == ns) {
      const __nv_bfloat16* kr = p.k_new + ((long long)b * p.G + g) * DEC_D;
      for (int i = 0; i < DEC_D; ++i) x[i] = __bfloat162float(kr[i]);
    } else {
      load_row_f32<BITS>(p.kq, row0 + j, x);
      if (BITS != 16) {
        kscale = p.ks[row0 + j];
        kzp = (float)p.kz[row0 + j];
      }
    }
    for (int h = 0; h < gs; ++h) {
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < DEC_D; ++i) acc = fmaf(q_s[h * DEC_D + i], x[i], acc);
      const float s = p.scale * kscale * (acc - kzp * qsum[h]);
      sc[h * DEC_SPLIT + jj] = s;
      p.logits[((long long)b * p.H + g * gs + h) * p.L + j] = s;
      lmax[h] = fmaxf(lmax[h], s);
    }
  }
  // block max per head
  for (int h = 0; h < gs; ++h) {
    float m = warp_max(lmax[h]);
    if (lane == 0) red[warp * DEC_MAX_GS + h] = m;
  }
  __syncthreads();
  float cmax[DEC_MAX_GS];
  for (int h = 0; h < gs; ++h) {
    float m = -FLT_MAX;
    for (int w = 0; w < DEC_THREADS / 32; ++w) m = fmaxf(m, red[w * DEC_MAX_GS + h]);
    cmax[h] = m;
  }
  __syncthreads();
  // ---- p = exp(s − m); fold the V scale / zero point; block sum per head
  float lsum[DEC_MAX_GS];
  for (int h = 0; h < gs; ++h) lsum[h] = 0.f;
  for (int jj = tid; jj < n; jj += DEC_THREADS) {
    const int j = j0 + jj;
    float vscale = 1.f, vzp = 0.f;
    if (BITS != 16 && j != ns) {
      vscale = p.vs[row0 + j];
      vzp = (float)p.vz[row0 + j];
    }
    for (int h = 0; h < gs; ++h) {
      const float pr = __expf(sc[h * DEC_SPLIT + jj] - cmax[h]);
      lsum[h] += pr;
      sc[h * DEC_SPLIT + jj] = pr * vscale;
      pz[h * DEC_SPLIT + jj] = pr * vscale * vzp;
    }
  }
  for (int h = 0; h < gs; ++h) {
    float s = warp_sum(lsum[h]);
    if (lane == 0) red[warp * DEC_MAX_GS + h] = s;
  }
  __syncthreads();
  if (tid < gs) {
    float s = 0.f;
    for (int w = 0; w < DEC_THREADS / 32; ++w) s += red[w * DEC_MAX_GS + tid];
    const long long idx = ((long long)b * p.H + g * gs + tid) * p.nS + split;
    p.part_m[idx] = cmax[tid];
    p.part_l[idx] = s;
  }
  __syncthreads();
  // ---- pass B: O += p · v ; lane owns 4 features, warps stride over slots
  float acc[DEC_MAX_GS][4];
#pragma unroll
  for (int h = 0; h < DEC_MAX_GS; ++h) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
  for (int jj = warp; jj < n; jj += DEC_THREADS / 32) {
    const int j = j0 + jj;
    float v[4];
    if (j == ns) {
      const __nv_bfloat16* vr = p.v_new + ((long long)b * p.G + g) * DEC_D + lane * 4;
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = __bfloat162float(vr[i]);
    } else if (BITS == 16) {
      const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(p.vq) + (row0 + j) * DEC_D + lane * 4);
      const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
      float2 a = __bfloat1622float2(hh[0]), c = __bfloat1622float2(hh[1]);
      v[0] = a.x; v[1] = a.y; v[2] = c.x; v[3] = c.y;
    } else if (BITS == 8) {
      const uint32_t raw = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(p.vq) + (row0 + j) * DEC_D + lane * 4);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = (float)((raw >> (8 * i)) & 0xFF);
    } else {
      // features lane*4 .. lane*4+3: high nibbles of bytes [lane*4, +4) if lane < 16, else low nibbles of bytes [(lane-16)*4, +4)
      const int bo = (lane & 15) * 4;
      const uint32_t raw = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(p.vq) + (row0 + j) * (DEC_D / 2) + bo);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t byte = (raw >> (8 * i)) & 0xFF;
        v[i] = (float)(lane < 16 ? (byte >> 4) : (byte & 0xF));
      }
    }
#pragma unroll
    for (int h = 0; h < DEC_MAX_GS; ++h) {
      if (h < gs) {
        const float ps = sc[h * DEC_SPLIT + jj], pzv = pz[h * DEC_SPLIT + jj];
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[h][i] += ps * v[i] - pzv;
      }
    }
  }
  __syncthreads();
  // cross-warp reduction through shared memory (re-using the score area)
  float* ored = sc;  // [8][gs][128]
#pragma unroll
  for (int h = 0; h < DEC_MAX_GS; ++h) {
    if (h < gs) {
#pragma unroll
      for (int i = 0; i < 4; ++i) ored[(warp * gs + h) * DEC_D + lane * 4 + i] = acc[h][i];
    }
  }
  __syncthreads();
  for (int i = tid; i < gs * DEC_D; i += DEC_THREADS) {
    float s = 0.f;
    for (int w = 0; w < DEC_THREADS / 32; ++w) s += ored[w * gs * DEC_D + i];
    const int h = i / DEC_D, d = i % DEC_D;
    p.part_o[(((long long)b * p.H + g * gs + h) * p.nS + split) * DEC_D + d] = s;
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
  const size_t smem = (size_t)(gs * DEC_D + DEC_MAX_GS + 2 * gs * DEC_SPLIT + (DEC_THREADS / 32) * DEC_MAX_GS) * 4;
  dim3 grid(B * G, p.nS);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(decode_partial_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    cudaFuncSetAttribute(decode_partial_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    cudaFuncSetAttribute(decode_partial_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    attr_set = true;
  }
  if (smem > 160 * 1024) return KVB_ERR_TOO_LARGE;
  if (bits == 16) decode_partial_kernel<16><<<grid, DEC_THREADS, smem, s>>>(p);
  else if (bits == 8) decode_partial_kernel<8><<<grid, DEC_THREADS, smem, s>>>(p);
  else decode_partial_kernel<4><<<grid, DEC_THREADS, smem, s>>>(p);
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
