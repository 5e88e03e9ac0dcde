// Memory-bound fused ops: RMSNorm, QKV split + per-head QK-RMSNorm + RoPE + layout
// change, SwiGLU; forward and backward. One warp per row, fp32 math, 16-byte
// accesses where the layout allows.
//
// Replaces the reference's Triton kernels (keys_values/fused/fused_rmsnorm.py:28-209,
// fused_rope.py:30-169, fused_swiglu.py:28-73) and the split/transposes/norms of
// keys_values/model.py:690-779.
#include "common.cuh"
#include "kvb200.h"

namespace kvb {

#define KVB_DISPATCH_DTYPE(dtype, ...)                      \
  switch (dtype) {                                          \
    case 0: { using T = float; __VA_ARGS__; break; }        \
    case 1: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case 2: { using T = __half; __VA_ARGS__; break; }       \
    default: return KVB_ERR_ARG;                            \
  }

constexpr int EW_WARPS = 8;

// ------------------------------------------------------------------- RMSNorm
template <typename T>
__global__ void rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, float* __restrict__ rstd,
                                   long long rows, int dim, float eps, int unit) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * EW_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * dim;
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) {
    float v = to_f32(xr[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / dim + eps);
  if (lane == 0 && rstd) rstd[row] = r;
  T* yr = y + row * dim;
  for (int i = lane; i < dim; i += 32) {
    float v = to_f32(xr[i]) * r;
    if (w) {
      float ww = to_f32(w[i]);
      v *= unit ? 1.f + ww : ww;
    }
    yr[i] = from_f32<T>(v);
  }
}

template <typename T>
__global__ void rmsnorm_bwd_kernel(const T* __restrict__ gy, const T* __restrict__ x, const T* __restrict__ w,
                                   const float* __restrict__ rstd, T* __restrict__ dx, float* __restrict__ dw_partial,
                                   long long rows, int dim, int unit) {
  extern __shared__ float dw_s[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (dw_partial) {
    for (int i = threadIdx.x; i < dim; i += blockDim.x) dw_s[i] = 0.f;
    __syncthreads();
  }
  for (long long row = (long long)blockIdx.x * EW_WARPS + warp; row < rows; row += (long long)gridDim.x * EW_WARPS) {
    const T* xr = x + row * dim;
    const T* gr = gy + row * dim;
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = lane; i < dim; i += 32) {
      float ww = w ? to_f32(w[i]) : 1.f;
      if (w && unit) ww += 1.f;
      dot += to_f32(gr[i]) * ww * to_f32(xr[i]) * r;
    }
    dot = warp_sum(dot) / dim;
    T* dr = dx + row * dim;
    for (int i = lane; i < dim; i += 32) {
      float ww = w ? to_f32(w[i]) : 1.f;
      if (w && unit) ww += 1.f;
      const float xh = to_f32(xr[i]) * r;
      const float g = to_f32(gr[i]);
      dr[i] = from_f32<T>(r * (g * ww - xh * dot));
      if (dw_partial) atomicAdd(&dw_s[i], g * xh);
    }
  }
  if (dw_partial) {
    __syncthreads();
    for (int i = threadIdx.x; i < dim; i += blockDim.x) dw_partial[(long long)blockIdx.x * dim + i] = dw_s[i];
  }
}

// ---- bf16 fast path: one warp per row, the whole row in registers (dim a multiple of 256, at most
// 8192), 16-byte accesses, optional fused residual add in the forward pass (s = x + res is written
// out, rounded to bf16, and normalised) and optional fused add of the gradient that reaches s by its
// other consumer in the backward pass.

template <int NC>
__global__ void __launch_bounds__(EW_WARPS * 32)
rmsnorm_fwd_bf16_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                        const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ sum_out,
                        float* __restrict__ rstd, long long rows, float eps, int unit) {
  constexpr int dim = NC * 256;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * EW_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const long long base = row * dim + lane * 8;
  uint4 v[NC];
#pragma unroll
  for (int c = 0; c < NC; ++c) v[c] = *reinterpret_cast<const uint4*>(x + base + c * 256);
  if (res) {
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const uint4 rv = *reinterpret_cast<const uint4*>(res + base + c * 256);
      __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&v[c]);
      const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 fa = __bfloat1622float2(a[j]), fb = __bfloat1622float2(b[j]);
        a[j] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
      }
      *reinterpret_cast<uint4*>(sum_out + base + c * 256) = v[c];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&v[c]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(a[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / dim + eps);
  if (lane == 0 && rstd) rstd[row] = r;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    uint4 wv = make_uint4(0, 0, 0, 0);
    if (w) wv = *reinterpret_cast<const uint4*>(w + lane * 8 + c * 256);
    __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&v[c]);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(a[j]);
      f.x *= r;
      f.y *= r;
      if (w) {
        float2 ww = __bfloat1622float2(b[j]);
        if (unit) { ww.x += 1.f; ww.y += 1.f; }
        f.x *= ww.x;
        f.y *= ww.y;
      }
      a[j] = __floats2bfloat162_rn(f.x, f.y);
    }
    *reinterpret_cast<uint4*>(y + base + c * 256) = v[c];
  }
}

// dx = r (g ⊙ w − x^ · mean(g ⊙ w ⊙ x^)) (+ gadd); no weight gradient (frozen norm weights)
template <int NC>
__global__ void __launch_bounds__(EW_WARPS * 32)
rmsnorm_bwd_bf16_kernel(const __nv_bfloat16* __restrict__ gy, const __nv_bfloat16* __restrict__ x,
                        const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd,
                        const __nv_bfloat16* __restrict__ gadd, __nv_bfloat16* __restrict__ dx, long long rows, int unit) {
  constexpr int dim = NC * 256;
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * EW_WARPS + (threadIdx.x >> 5);
  if (row >= rows) return;
  const long long base = row * dim + lane * 8;
  const float r = rstd[row];
  float gw[NC][8], xh[NC][8];
  float dot = 0.f;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    const uint4 gv = *reinterpret_cast<const uint4*>(gy + base + c * 256);
    const uint4 xv = *reinterpret_cast<const uint4*>(x + base + c * 256);
    uint4 wv = make_uint4(0, 0, 0, 0);
    if (w) wv = *reinterpret_cast<const uint4*>(w + lane * 8 + c * 256);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&xv);
    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 g = __bfloat1622float2(g2[j]), xx = __bfloat1622float2(x2[j]);
      float2 ww = make_float2(1.f, 1.f);
      if (w) {
        ww = __bfloat1622float2(w2[j]);
        if (unit) { ww.x += 1.f; ww.y += 1.f; }
      }
      gw[c][2 * j] = g.x * ww.x;
      gw[c][2 * j + 1] = g.y * ww.y;
      xh[c][2 * j] = xx.x * r;
      xh[c][2 * j + 1] = xx.y * r;
      dot += gw[c][2 * j] * xh[c][2 * j] + gw[c][2 * j + 1] * xh[c][2 * j + 1];
    }
  }
  dot = warp_sum(dot) / dim;
#pragma unroll
  for (int c = 0; c < NC; ++c) {
    uint4 av = make_uint4(0, 0, 0, 0);
    if (gadd) av = *reinterpret_cast<const uint4*>(gadd + base + c * 256);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float d0 = r * (gw[c][2 * j] - xh[c][2 * j] * dot), d1 = r * (gw[c][2 * j + 1] - xh[c][2 * j + 1] * dot);
      if (gadd) {
        const float2 a = __bfloat1622float2(a2[j]);
        d0 += a.x;
        d1 += a.y;
      }
      o2[j] = __floats2bfloat162_rn(d0, d1);
    }
    *reinterpret_cast<uint4*>(dx + base + c * 256) = ov;
  }
}

// Few rows (single-token decode steps: rows = batch size): one CTA per row, so that a row is spread
// over 8 warps and the loads of x, the residual and the weight are all in flight before the one
// block-wide reduction; the warp-per-row kernel above serialises three memory round trips on a
// handful of warps. dim is a multiple of 256 and at most 256 · 8 · RMS_ROW_UNITS.
constexpr int RMS_ROW_THREADS = 256;
constexpr int RMS_ROW_UNITS = 3;
__global__ void __launch_bounds__(RMS_ROW_THREADS)
rmsnorm_fwd_fewrows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                           const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ sum_out,
                           float* __restrict__ rstd, int dim, float eps, int unit) {
  __shared__ float red[RMS_ROW_THREADS / 32];
  const long long base = (long long)blockIdx.x * dim;
  const int units = dim / 8, tid = threadIdx.x;
  uint4 v[RMS_ROW_UNITS], rv[RMS_ROW_UNITS], wv[RMS_ROW_UNITS];
#pragma unroll
  for (int c = 0; c < RMS_ROW_UNITS; ++c) {
    const int u = tid + c * RMS_ROW_THREADS;
    v[c] = rv[c] = wv[c] = make_uint4(0, 0, 0, 0);
    if (u < units) {
      v[c] = *reinterpret_cast<const uint4*>(x + base + u * 8);
      if (res) rv[c] = *reinterpret_cast<const uint4*>(res + base + u * 8);
      if (w) wv[c] = *reinterpret_cast<const uint4*>(w + u * 8);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < RMS_ROW_UNITS; ++c) {
    __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&v[c]);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&rv[c]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(a[j]);
      if (res) {
        const float2 fb = __bfloat1622float2(b[j]);
        a[j] = __floats2bfloat162_rn(f.x + fb.x, f.y + fb.y);  // the sum as the next layer will read it
        f = __bfloat1622float2(a[j]);
      }
      ss += f.x * f.x + f.y * f.y;
    }
    const int u = tid + c * RMS_ROW_THREADS;
    if (res && u < units) *reinterpret_cast<uint4*>(sum_out + base + u * 8) = v[c];
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < RMS_ROW_THREADS / 32; ++i) tot += red[i];
  const float r = rsqrtf(tot / dim + eps);
  if (tid == 0 && rstd) rstd[blockIdx.x] = r;
#pragma unroll
  for (int c = 0; c < RMS_ROW_UNITS; ++c) {
    const int u = tid + c * RMS_ROW_THREADS;
    if (u >= units) continue;
    __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&v[c]);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&wv[c]);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 f = __bfloat1622float2(a[j]);
      f.x *= r;
      f.y *= r;
      if (w) {
        float2 ww = __bfloat1622float2(b[j]);
        if (unit) { ww.x += 1.f; ww.y += 1.f; }
        f.x *= ww.x;
        f.y *= ww.y;
      }
      a[j] = __floats2bfloat162_rn(f.x, f.y);
    }
    *reinterpret_cast<uint4*>(y + base + u * 8) = v[c];
  }
}

#define KVB_RMS_DISPATCH(NCV, ...)                                  \
  switch (NCV) {                                                    \
    case 4: { constexpr int NC = 4; __VA_ARGS__; break; }           \
    case 8: { constexpr int NC = 8; __VA_ARGS__; break; }           \
    case 10: { constexpr int NC = 10; __VA_ARGS__; break; }         \
    case 12: { constexpr int NC = 12; __VA_ARGS__; break; }         \
    case 14: { constexpr int NC = 14; __VA_ARGS__; break; }         \
    case 16: { constexpr int NC = 16; __VA_ARGS__; break; }         \
    case 20: { constexpr int NC = 20; __VA_ARGS__; break; }         \
    default: return KVB_ERR_UNSUPPORTED;                            \
  }
#define KVB_RMS_DISPATCH_BWD(NCV, ...)                              \
  switch (NCV) {                                                    \
    case 4: { constexpr int NC = 4; __VA_ARGS__; break; }           \
    case 8: { constexpr int NC = 8; __VA_ARGS__; break; }           \
    case 10: { constexpr int NC = 10; __VA_ARGS__; break; }         \
    case 12: { constexpr int NC = 12; __VA_ARGS__; break; }         \
    default: return KVB_ERR_UNSUPPORTED;                            \
  }
static bool rms_fast_dim(int dim) {
  if (dim % 256) return false;
  const int nc = dim / 256;
  return nc == 4 || nc == 8 || nc == 10 || nc == 12 || nc == 14 || nc == 16 || nc == 20;
}

// ------------------------------------------------- QKV split + QK-norm + RoPE
// Row id = ((b * T + t) * (H + 2G) + head); heads [0,H) are queries, [H,H+G) keys,
// [H+G,H+2G) values.
template <typename T>
__global__ void qknorm_rope_fwd_kernel(const T* __restrict__ qkv, const float* __restrict__ cosT, const float* __restrict__ sinT,
                                       const T* __restrict__ qw, const T* __restrict__ kw, T* __restrict__ q, T* __restrict__ k,
                                       T* __restrict__ v, float* __restrict__ rstd, int B, int Tn, int H, int G, int D, float eps,
                                       int rope_n, int unit) {
  extern __shared__ float sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* xs = sm + warp * D;
  const int NH = H + 2 * G;
  const long long row = (long long)blockIdx.x * EW_WARPS + warp;
  if (row >= (long long)B * Tn * NH) return;
  const int head = (int)(row % NH);
  const long long bt = row / NH;
  const int t = (int)(bt % Tn);
  const int b = (int)(bt / Tn);
  const T* src = qkv + row * D;
  T* dst;
  if (head < H) dst = q + (((long long)b * H + head) * Tn + t) * D;
  else if (head < H + G) dst = k + (((long long)b * G + (head - H)) * Tn + t) * D;
  else {
    dst = v + (((long long)b * G + (head - H - G)) * Tn + t) * D;
    for (int i = lane; i < D; i += 32) dst[i] = src[i];
    return;
  }
  const T* w = head < H ? qw : kw;
  float ss = 0.f;
  for (int i = lane; i < D; i += 32) {
    float x = to_f32(src[i]);
    xs[i] = x;
    ss += x * x;
  }
  float r = 1.f;
  if (w) {
    ss = warp_sum(ss);
    r = rsqrtf(ss / D + eps);
    if (lane == 0) rstd[bt * (H + G) + head] = r;
  }
  __syncwarp();
  if (w) {
    for (int i = lane; i < D; i += 32) {
      float ww = to_f32(w[i]);
      xs[i] = xs[i] * r * (unit ? 1.f + ww : ww);
    }
    __syncwarp();
  }
  const int half = rope_n >> 1;
  for (int i = lane; i < D; i += 32) {
    float y = xs[i];
    if (i < rope_n) {
      const float c = cosT[(long long)t * rope_n + i], s = sinT[(long long)t * rope_n + i];
      const float rot = i < half ? -xs[i + half] : xs[i - half];
      y = y * c + rot * s;
    }
    dst[i] = from_f32<T>(y);
  }
}

template <typename T>
__global__ void qknorm_rope_bwd_kernel(const T* __restrict__ gq, const T* __restrict__ gk, const T* __restrict__ gv,
                                       const T* __restrict__ qkv, const float* __restrict__ cosT, const float* __restrict__ sinT,
                                       const T* __restrict__ qw, const T* __restrict__ kw, const float* __restrict__ rstd,
                                       T* __restrict__ dqkv, float* __restrict__ dw_partial, int B, int Tn, int H, int G, int D,
                                       int rope_n, int unit) {
  extern __shared__ float sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* gs = sm + warp * D;             // per-warp staging of the incoming gradient
  float* dw_s = sm + EW_WARPS * D;       // [2][D] partial weight gradients (q, k)
  if (dw_partial) {
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) dw_s[i] = 0.f;
    __syncthreads();
  }
  const int NH = H + 2 * G;
  const long long total = (long long)B * Tn * NH;
  for (long long row = (long long)blockIdx.x * EW_WARPS + warp; row < total; row += (long long)gridDim.x * EW_WARPS) {
    const int head = (int)(row % NH);
    const long long bt = row / NH;
    const int t = (int)(bt % Tn);
    const int b = (int)(bt / Tn);
    T* dst = dqkv + row * D;
    if (head >= H + G) {
      const T* g = gv + (((long long)b * G + (head - H - G)) * Tn + t) * D;
      for (int i = lane; i < D; i += 32) dst[i] = g[i];
      continue;
    }
    const T* g = head < H ? gq + (((long long)b * H + head) * Tn + t) * D : gk + (((long long)b * G + (head - H)) * Tn + t) * D;
    const T* w = head < H ? qw : kw;
    for (int i = lane; i < D; i += 32) gs[i] = to_f32(g[i]);
    __syncwarp();
    const int half = rope_n >> 1;
    float gr[8];  // D <= 256 -> at most 8 elements per lane
    int cnt = 0;
    for (int i = lane; i < D; i += 32, ++cnt) {
      float gi = gs[i];
      if (i < rope_n) {
        const float c = cosT[(long long)t * rope_n + i];
        if (i < half) gi = gi * c + gs[i + half] * sinT[(long long)t * rope_n + i + half];
        else gi = gi * c - gs[i - half] * sinT[(long long)t * rope_n + i - half];
      }
      gr[cnt] = gi;
    }
    if (!w) {
      cnt = 0;
      for (int i = lane; i < D; i += 32, ++cnt) dst[i] = from_f32<T>(gr[cnt]);
      __syncwarp();
      continue;
    }
    const T* src = qkv + row * D;
    const float r = rstd[bt * (H + G) + head];
    float dot = 0.f;
    cnt = 0;
    for (int i = lane; i < D; i += 32, ++cnt) {
      float ww = to_f32(w[i]);
      if (unit) ww += 1.f;
      dot += gr[cnt] * ww * to_f32(src[i]) * r;
    }
    dot = warp_sum(dot) / D;
    cnt = 0;
    for (int i = lane; i < D; i += 32, ++cnt) {
      float ww = to_f32(w[i]);
      if (unit) ww += 1.f;
      const float xh = to_f32(src[i]) * r;
      dst[i] = from_f32<T>(r * (gr[cnt] * ww - xh * dot));
      if (dw_partial) atomicAdd(&dw_s[(head < H ? 0 : D) + i], gr[cnt] * xh);
    }
    __syncwarp();
  }
  if (dw_partial) {
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) dw_partial[(long long)blockIdx.x * 2 * D + i] = dw_s[i];
  }
}

// ---- fast paths: bf16, head size 128, RoPE over the whole head. One warp per token: a lane
// holds 4 consecutive features of a head (8-byte loads and stores), the rotation partner
// (feature ± 64) lives in lane ± 16 and is fetched by shuffle, cos / sin of the token are loaded
// once and reused for all heads, weight gradients accumulate in registers.
__device__ __forceinline__ void bf16x4_to_f32(const uint2 v, float* x) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
  const float2 a = __bfloat1622float2(h[0]), c = __bfloat1622float2(h[1]);
  x[0] = a.x; x[1] = a.y; x[2] = c.x; x[3] = c.y;
}
__device__ __forceinline__ uint2 f32_to_bf16x4(const float* x) {
  uint2 v;
  __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), c = __floats2bfloat162_rn(x[2], x[3]);
  v.x = *reinterpret_cast<uint32_t*>(&a);
  v.y = *reinterpret_cast<uint32_t*>(&c);
  return v;
}

__global__ void __launch_bounds__(EW_WARPS * 32)
qknorm_rope_fwd128_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ cosT, const float* __restrict__ sinT,
                          const __nv_bfloat16* __restrict__ qw, const __nv_bfloat16* __restrict__ kw,
                          __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k, __nv_bfloat16* __restrict__ v,
                          float* __restrict__ rstd, int B, int Tn, int H, int G, float eps, int unit) {
  constexpr int D = 128;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long tok = (long long)blockIdx.x * EW_WARPS + warp;
  if (tok >= (long long)B * Tn) return;
  const int t = (int)(tok % Tn), b = (int)(tok / Tn);
  const int NH = H + 2 * G;
  const float4 c4 = *reinterpret_cast<const float4*>(cosT + (long long)t * D + 4 * lane);
  const float4 s4 = *reinterpret_cast<const float4*>(sinT + (long long)t * D + 4 * lane);
  const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
  float wq[4] = {1.f, 1.f, 1.f, 1.f}, wk[4] = {1.f, 1.f, 1.f, 1.f};
  if (qw) {
    bf16x4_to_f32(*reinterpret_cast<const uint2*>(qw + 4 * lane), wq);
    bf16x4_to_f32(*reinterpret_cast<const uint2*>(kw + 4 * lane), wk);
    if (unit) {
#pragma unroll
      for (int i = 0; i < 4; ++i) { wq[i] += 1.f; wk[i] += 1.f; }
    }
  }
  const __nv_bfloat16* src = qkv + tok * NH * D + 4 * lane;
  const float sgn = lane < 16 ? -1.f : 1.f;
#pragma unroll 4
  for (int head = 0; head < H + G; ++head) {
    float x[4];
    bf16x4_to_f32(*reinterpret_cast<const uint2*>(src + (long long)head * D), x);
    const float* w = head < H ? wq : wk;
    if (qw) {
      float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
      ss = warp_sum(ss);
      const float r = rsqrtf(ss / D + eps);
      if (lane == 0) rstd[tok * (H + G) + head] = r;
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = x[i] * r * w[i];
    }
    float y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float partner = __shfl_xor_sync(0xffffffffu, x[i], 16);
      y[i] = x[i] * cs[i] + sgn * partner * sn[i];
    }
    __nv_bfloat16* dst = head < H ? q + (((long long)b * H + head) * Tn + t) * D : k + (((long long)b * G + (head - H)) * Tn + t) * D;
    *reinterpret_cast<uint2*>(dst + 4 * lane) = f32_to_bf16x4(y);
  }
#pragma unroll 4
  for (int head = 0; head < G; ++head)
    *reinterpret_cast<uint2*>(v + (((long long)b * G + head) * Tn + t) * D + 4 * lane) =
        *reinterpret_cast<const uint2*>(src + (long long)(H + G + head) * D);
}

__global__ void __launch_bounds__(EW_WARPS * 32)
qknorm_rope_bwd128_kernel(const __nv_bfloat16* __restrict__ gq, const __nv_bfloat16* __restrict__ gk,
                          const __nv_bfloat16* __restrict__ gv, const __nv_bfloat16* __restrict__ qkv,
                          const float* __restrict__ cosT, const float* __restrict__ sinT, const __nv_bfloat16* __restrict__ qw,
                          const __nv_bfloat16* __restrict__ kw, const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dqkv,
                          float* __restrict__ dw_partial, int B, int Tn, int H, int G, int unit) {
  constexpr int D = 128;
  __shared__ float dw_s[EW_WARPS][2][D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int NH = H + 2 * G;
  float wq[4] = {1.f, 1.f, 1.f, 1.f}, wk[4] = {1.f, 1.f, 1.f, 1.f};
  if (qw) {
    bf16x4_to_f32(*reinterpret_cast<const uint2*>(qw + 4 * lane), wq);
    bf16x4_to_f32(*reinterpret_cast<const uint2*>(kw + 4 * lane), wk);
    if (unit) {
#pragma unroll
      for (int i = 0; i < 4; ++i) { wq[i] += 1.f; wk[i] += 1.f; }
    }
  }
  float dwq[4] = {0.f, 0.f, 0.f, 0.f}, dwk[4] = {0.f, 0.f, 0.f, 0.f};
  // the partner of feature i contributes g·sin taken at ITS index: + for i < 64, − otherwise
  const float sgn = lane < 16 ? 1.f : -1.f;
  for (long long tok = (long long)blockIdx.x * EW_WARPS + warp; tok < (long long)B * Tn; tok += (long long)gridDim.x * EW_WARPS) {
    const int t = (int)(tok % Tn), b = (int)(tok / Tn);
    const float4 c4 = *reinterpret_cast<const float4*>(cosT + (long long)t * D + 4 * lane);
    const float4 s4 = *reinterpret_cast<const float4*>(sinT + (long long)t * D + 4 * lane);
    const float cs[4] = {c4.x, c4.y, c4.z, c4.w}, sn[4] = {s4.x, s4.y, s4.z, s4.w};
    const __nv_bfloat16* src = qkv + tok * NH * D + 4 * lane;
    __nv_bfloat16* dst = dqkv + tok * NH * D + 4 * lane;
#pragma unroll 2
    for (int head = 0; head < H + G; ++head) {
      const __nv_bfloat16* g = head < H ? gq + (((long long)b * H + head) * Tn + t) * D : gk + (((long long)b * G + (head - H)) * Tn + t) * D;
      float gi[4], gr[4];
      bf16x4_to_f32(*reinterpret_cast<const uint2*>(g + 4 * lane), gi);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float partner = __shfl_xor_sync(0xffffffffu, gi[i] * sn[i], 16);
        gr[i] = gi[i] * cs[i] + sgn * partner;
      }
      if (!qw) {
        *reinterpret_cast<uint2*>(dst + (long long)head * D) = f32_to_bf16x4(gr);
        continue;
      }
      float x[4];
      bf16x4_to_f32(*reinterpret_cast<const uint2*>(src + (long long)head * D), x);
      const float r = rstd[tok * (H + G) + head];
      const float* w = head < H ? wq : wk;
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) dot += gr[i] * w[i] * x[i] * r;
      dot = warp_sum(dot) * (1.f / D);
      float o[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float xh = x[i] * r;
        o[i] = r * (gr[i] * w[i] - xh * dot);
        if (head < H) dwq[i] += gr[i] * xh;
        else dwk[i] += gr[i] * xh;
      }
      *reinterpret_cast<uint2*>(dst + (long long)head * D) = f32_to_bf16x4(o);
    }
#pragma unroll 4
    for (int head = 0; head < G; ++head)
      *reinterpret_cast<uint2*>(dst + (long long)(H + G + head) * D) =
          *reinterpret_cast<const uint2*>(gv + (((long long)b * G + head) * Tn + t) * D + 4 * lane);
  }
  if (dw_partial) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      dw_s[warp][0][4 * lane + i] = dwq[i];
      dw_s[warp][1][4 * lane + i] = dwk[i];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < EW_WARPS; ++w) sum += dw_s[w][i / D][i % D];
      dw_partial[(long long)blockIdx.x * 2 * D + i] = sum;
    }
  }
}

// -------------------------------------------------------------------- SwiGLU
template <typename T>
__global__ void swiglu_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ y, long long n) {
  constexpr int V = 16 / sizeof(T);
  const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (i0 + V <= n) {
    uint4 av = *reinterpret_cast<const uint4*>(a + i0), bv = *reinterpret_cast<const uint4*>(b + i0), yv;
    const T* ap = reinterpret_cast<const T*>(&av);
    const T* bp = reinterpret_cast<const T*>(&bv);
    T* yp = reinterpret_cast<T*>(&yv);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float x = to_f32(ap[j]);
      yp[j] = from_f32<T>(x / (1.f + __expf(-x)) * to_f32(bp[j]));
    }
    *reinterpret_cast<uint4*>(y + i0) = yv;
  } else {
    for (long long i = i0; i < n; ++i) {
      const float x = to_f32(a[i]);
      y[i] = from_f32<T>(x / (1.f + __expf(-x)) * to_f32(b[i]));
    }
  }
}

template <typename T>
__global__ void swiglu_bwd_kernel(const T* __restrict__ gy, const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ da,
                                  T* __restrict__ db, long long n) {
  constexpr int V = 16 / sizeof(T);
  const long long i0 = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (i0 + V <= n) {
    uint4 gvv = *reinterpret_cast<const uint4*>(gy + i0), av = *reinterpret_cast<const uint4*>(a + i0),
          bv = *reinterpret_cast<const uint4*>(b + i0), dav, dbv;
    const T* gp = reinterpret_cast<const T*>(&gvv);
    const T* ap = reinterpret_cast<const T*>(&av);
    const T* bp = reinterpret_cast<const T*>(&bv);
    T* dap = reinterpret_cast<T*>(&dav);
    T* dbp = reinterpret_cast<T*>(&dbv);
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const float x = to_f32(ap[j]), g = to_f32(gp[j]), bb = to_f32(bp[j]);
      const float sg = 1.f / (1.f + __expf(-x));
      dap[j] = from_f32<T>(g * bb * sg * (1.f + x * (1.f - sg)));
      dbp[j] = from_f32<T>(g * x * sg);
    }
    *reinterpret_cast<uint4*>(da + i0) = dav;
    *reinterpret_cast<uint4*>(db + i0) = dbv;
  } else {
    for (long long i = i0; i < n; ++i) {
      const float x = to_f32(a[i]), g = to_f32(gy[i]), bb = to_f32(b[i]);
      const float sg = 1.f / (1.f + __expf(-x));
      da[i] = from_f32<T>(g * bb * sg * (1.f + x * (1.f - sg)));
      db[i] = from_f32<T>(g * x * sg);
    }
  }
}

static inline int check_launch() { return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH; }

}  // namespace kvb

using namespace kvb;

// y = rmsnorm(x + res) · w and sum_out = x + res (res and sum_out may be NULL together). bf16 only,
// dim in {1024, 2048, 2560, 3072, 3584, 4096, 5120}; other cases: KVB_ERR_UNSUPPORTED.
extern "C" int kvb_add_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out, float* rstd,
                                   long long rows, int dim, float eps, int add_unit_offset, void* stream) {
  if (rows <= 0 || dim <= 0 || ((res == nullptr) != (sum_out == nullptr))) return KVB_ERR_ARG;
  if (!rms_fast_dim(dim)) return KVB_ERR_UNSUPPORTED;
  if (rows <= 64 && dim <= 256 * 8 * RMS_ROW_UNITS) {
    rmsnorm_fwd_fewrows_kernel<<<(unsigned)rows, RMS_ROW_THREADS, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, (__nv_bfloat16*)sum_out, rstd,
        dim, eps, add_unit_offset);
    return check_launch();
  }
  const unsigned grid = (unsigned)((rows + EW_WARPS - 1) / EW_WARPS);
  KVB_RMS_DISPATCH(dim / 256, (rmsnorm_fwd_bf16_kernel<NC><<<grid, EW_WARPS * 32, 0, (cudaStream_t)stream>>>(
                                  (const __nv_bfloat16*)x, (const __nv_bfloat16*)res, (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
                                  (__nv_bfloat16*)sum_out, rstd, rows, eps, add_unit_offset)));
  return check_launch();
}

// dx = rmsnorm_backward(gy; x, w, rstd) + gadd (gadd may be NULL); bf16, dim in {1024, 2048, 2560, 3072}.
extern "C" int kvb_rmsnorm_bwd_add(const void* gy, const void* x, const void* w, const float* rstd, const void* gadd, void* dx,
                                   long long rows, int dim, int add_unit_offset, void* stream) {
  if (rows <= 0 || dim <= 0) return KVB_ERR_ARG;
  if (!rms_fast_dim(dim) || dim > 3072) return KVB_ERR_UNSUPPORTED;  // the row lives in registers as fp32
  const unsigned grid = (unsigned)((rows + EW_WARPS - 1) / EW_WARPS);
  KVB_RMS_DISPATCH_BWD(dim / 256, (rmsnorm_bwd_bf16_kernel<NC><<<grid, EW_WARPS * 32, 0, (cudaStream_t)stream>>>(
                                  (const __nv_bfloat16*)gy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,
                                  (const __nv_bfloat16*)gadd, (__nv_bfloat16*)dx, rows, add_unit_offset)));
  return check_launch();
}

extern "C" int kvb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int dim, float eps,
                               int add_unit_offset, int dtype, void* stream) {
  if (rows <= 0 || dim <= 0) return KVB_ERR_ARG;
  if (dtype == 1 && rms_fast_dim(dim)) return kvb_add_rmsnorm_fwd(x, nullptr, w, y, nullptr, rstd, rows, dim, eps, add_unit_offset, stream);
  const unsigned grid = (unsigned)((rows + EW_WARPS - 1) / EW_WARPS);
  KVB_DISPATCH_DTYPE(dtype, (rmsnorm_fwd_kernel<T><<<grid, EW_WARPS * 32, 0, (cudaStream_t)stream>>>(
                                (const T*)x, (const T*)w, (T*)y, rstd, rows, dim, eps, add_unit_offset)));
  return check_launch();
}

extern "C" int kvb_rmsnorm_bwd(const void* gy, const void* x, const void* w, const float* rstd, void* dx, float* dw_partial,
                               long long rows, int dim, int add_unit_offset, int dtype, int n_partial, void* stream) {
  if (rows <= 0 || dim <= 0 || n_partial <= 0) return KVB_ERR_ARG;
  if (dtype == 1 && !dw_partial && rms_fast_dim(dim) && dim <= 3072) return kvb_rmsnorm_bwd_add(gy, x, w, rstd, nullptr, dx, rows, dim, add_unit_offset, stream);
  const size_t smem = dw_partial ? (size_t)dim * 4 : 0;
  if (smem > 48 * 1024) return KVB_ERR_TOO_LARGE;
  KVB_DISPATCH_DTYPE(dtype, (rmsnorm_bwd_kernel<T><<<n_partial, EW_WARPS * 32, smem, (cudaStream_t)stream>>>(
                                (const T*)gy, (const T*)x, (const T*)w, rstd, (T*)dx, dw_partial, rows, dim, add_unit_offset)));
  return check_launch();
}

extern "C" int kvb_qknorm_rope_fwd(const void* qkv, const float* cos, const float* sin, const void* qw, const void* kw, void* q,
                                   void* k, void* v, float* rstd, int B, int T_, int H, int G, int D, float eps,
                                   int rope_n_elem, int add_unit_offset, int dtype, void* stream) {
  if (D > 256 || D <= 0 || rope_n_elem > D || (rope_n_elem & 1)) return KVB_ERR_UNSUPPORTED;
  if (dtype == 1 && D == 128 && rope_n_elem == 128 && ((qw == nullptr) == (kw == nullptr))) {
    const unsigned g128 = (unsigned)(((long long)B * T_ + EW_WARPS - 1) / EW_WARPS);
    qknorm_rope_fwd128_kernel<<<g128, EW_WARPS * 32, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)qkv, cos, sin, (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, (__nv_bfloat16*)q,
        (__nv_bfloat16*)k, (__nv_bfloat16*)v, rstd, B, T_, H, G, eps, add_unit_offset);
    return check_launch();
  }
  const long long rows = (long long)B * T_ * (H + 2 * G);
  const unsigned grid = (unsigned)((rows + EW_WARPS - 1) / EW_WARPS);
  const size_t smem = (size_t)EW_WARPS * D * 4;
  KVB_DISPATCH_DTYPE(dtype, (qknorm_rope_fwd_kernel<T><<<grid, EW_WARPS * 32, smem, (cudaStream_t)stream>>>(
                                (const T*)qkv, cos, sin, (const T*)qw, (const T*)kw, (T*)q, (T*)k, (T*)v, rstd, B, T_, H, G, D,
                                eps, rope_n_elem, add_unit_offset)));
  return check_launch();
}

extern "C" int kvb_qknorm_rope_bwd(const void* gq, const void* gk, const void* gv, const void* qkv, const float* cos,
                                   const float* sin, const void* qw, const void* kw, const float* rstd, void* dqkv,
                                   float* dw_partial, int B, int T_, int H, int G, int D, int rope_n_elem, int add_unit_offset,
                                   int dtype, int n_partial, void* stream) {
  if (D > 256 || D <= 0 || rope_n_elem > D || (rope_n_elem & 1) || n_partial <= 0) return KVB_ERR_UNSUPPORTED;
  if (dtype == 1 && D == 128 && rope_n_elem == 128 && ((qw == nullptr) == (kw == nullptr))) {
    qknorm_rope_bwd128_kernel<<<n_partial, EW_WARPS * 32, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)gq, (const __nv_bfloat16*)gk, (const __nv_bfloat16*)gv, (const __nv_bfloat16*)qkv, cos, sin,
        (const __nv_bfloat16*)qw, (const __nv_bfloat16*)kw, rstd, (__nv_bfloat16*)dqkv, dw_partial, B, T_, H, G, add_unit_offset);
    return check_launch();
  }
  const size_t smem = (size_t)(EW_WARPS + 2) * D * 4;
  KVB_DISPATCH_DTYPE(dtype, (qknorm_rope_bwd_kernel<T><<<n_partial, EW_WARPS * 32, smem, (cudaStream_t)stream>>>(
                                (const T*)gq, (const T*)gk, (const T*)gv, (const T*)qkv, cos, sin, (const T*)qw, (const T*)kw,
                                rstd, (T*)dqkv, dw_partial, B, T_, H, G, D, rope_n_elem, add_unit_offset)));
  return check_launch();
}

extern "C" int kvb_swiglu_fwd(const void* a, const void* b, void* y, long long n, int dtype, void* stream) {
  if (n <= 0) return KVB_ERR_ARG;
  KVB_DISPATCH_DTYPE(dtype, {
    constexpr int V = 16 / sizeof(T);
    const unsigned grid = (unsigned)((n + 256LL * V - 1) / (256LL * V));
    swiglu_fwd_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>((const T*)a, (const T*)b, (T*)y, n);
  });
  return check_launch();
}

extern "C" int kvb_swiglu_bwd(const void* gy, const void* a, const void* b, void* da, void* db, long long n, int dtype,
                              void* stream) {
  if (n <= 0) return KVB_ERR_ARG;
  KVB_DISPATCH_DTYPE(dtype, {
    constexpr int V = 16 / sizeof(T);
    const unsigned grid = (unsigned)((n + 256LL * V - 1) / (256LL * V));
    swiglu_bwd_kernel<T><<<grid, 256, 0, (cudaStream_t)stream>>>((const T*)gy, (const T*)a, (const T*)b, (T*)da, (T*)db, n);
  });
  return check_launch();
}
