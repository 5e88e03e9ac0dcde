// KV-cache storage kernels: asymmetric affine int8/int4 row quantization,
// de-quantization of (strided) slot ranges, and the fused cache write
// (scatter new K/V rows into their slots + token_pos update + quantize-on-write).
//
// Quantization math per row of D values (keys_values/kvcache/quantize/pytorch.py:100-154):
//   scale = max((max - min) / (2^bits - 1), eps);  zp = -round(min / scale)  (int32)
//   q = clamp(round(x / scale) + zp, 0, 2^bits - 1);  x^ = (q - zp) * scale
//   4 bit: byte j = (q[j] << 4) | q[j + D/2].
// Replaces buffers.py:498-523 (scatter), attn_weights.py:214-317 (token_pos update)
// and the ATen chains of quantize/pytorch.py:312-455.
#include <float.h>

#include "common.cuh"
#include "kvb200.h"

namespace kvb {

constexpr int Q_WARPS = 8;
constexpr float QUANT_EPS = 1.1920928955078125e-07f;  // float32 machine epsilon

// Quantizes one row held in shared memory (fp32) by one warp.
__device__ __forceinline__ void quantize_row_warp(const float* xs, int D, int bits, uint8_t* qdst, float* sdst, int32_t* zdst,
                                                  int lane) {
  float mn = FLT_MAX, mx = -FLT_MAX;
  for (int i = lane; i < D; i += 32) {
    mn = fminf(mn, xs[i]);
    mx = fmaxf(mx, xs[i]);
  }
  mn = warp_min(mn);
  mx = warp_max(mx);
  const float qmax = (float)((1 << bits) - 1);
  const float scale = fmaxf(__fdiv_rn(mx - mn, qmax), QUANT_EPS);
  const float zpf = 0.f - rintf(__fdiv_rn(mn, scale));
  if (lane == 0) {
    *sdst = scale;
    *zdst = (int32_t)zpf;
  }
  if (bits == 8) {
    for (int i = lane; i < D; i += 32) {
      float qv = fminf(fmaxf(rintf(__fdiv_rn(xs[i], scale)) + zpf, 0.f), qmax);
      qdst[i] = (uint8_t)qv;
    }
  } else {
    const int half = D >> 1;
    for (int i = lane; i < half; i += 32) {
      float hi = fminf(fmaxf(rintf(__fdiv_rn(xs[i], scale)) + zpf, 0.f), qmax);
      float lo = fminf(fmaxf(rintf(__fdiv_rn(xs[i + half], scale)) + zpf, 0.f), qmax);
      qdst[i] = (uint8_t)(((uint32_t)hi << 4) | (uint32_t)lo);
    }
  }
}

// ---- fast paths: bf16 rows of 128 values. A lane holds features 4·lane .. 4·lane + 3 (one
// 8-byte load), the row statistics are warp reductions, the codes leave as one 32-bit store.
__device__ __forceinline__ void q128_load(const __nv_bfloat16* row, int lane, float* x, uint2& raw) {
  raw = *reinterpret_cast<const uint2*>(row + 4 * lane);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
  const float2 a = __bfloat1622float2(h[0]), c = __bfloat1622float2(h[1]);
  x[0] = a.x; x[1] = a.y; x[2] = c.x; x[3] = c.y;
}

// Same arithmetic as quantize_row_warp, for a row held as 4 values per lane.
__device__ __forceinline__ void quantize_row128(const float* x, int bits, uint8_t* qdst, float* sdst, int32_t* zdst, int lane) {
  float mn = fminf(fminf(x[0], x[1]), fminf(x[2], x[3])), mx = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
  mn = warp_min(mn);
  mx = warp_max(mx);
  const float qmax = (float)((1 << bits) - 1);
  const float scale = fmaxf(__fdiv_rn(mx - mn, qmax), QUANT_EPS);
  const float zpf = 0.f - rintf(__fdiv_rn(mn, scale));
  if (lane == 0) {
    *sdst = scale;
    *zdst = (int32_t)zpf;
  }
  uint32_t c[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) c[i] = (uint32_t)fminf(fmaxf(rintf(__fdiv_rn(x[i], scale)) + zpf, 0.f), qmax);
  if (bits == 8) {
    *reinterpret_cast<uint32_t*>(qdst + 4 * lane) = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
  } else {
    // byte j = (code[j] << 4) | code[j + 64]: the low nibbles come from lane + 16
    uint32_t packed = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
    const uint32_t low = __shfl_down_sync(0xffffffffu, packed, 16);
    if (lane < 16) *reinterpret_cast<uint32_t*>(qdst + 4 * lane) = (packed << 4) | low;
  }
}

constexpr int Q128_ROWS = 8;

__global__ void __launch_bounds__(Q_WARPS * 32)
quantize_rows128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale,
                        int32_t* __restrict__ zp, long long rows, int bits) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int Dq = bits == 8 ? 128 : 64;
  // Q128_ROWS rows per warp, all loads issued before the arithmetic (64 bytes in flight per lane)
  const long long r0 = ((long long)blockIdx.x * Q_WARPS + warp) * Q128_ROWS;
  if (r0 >= rows) return;
  float a[Q128_ROWS][4];
  uint2 raw;
#pragma unroll
  for (int r = 0; r < Q128_ROWS; ++r)
    if (r0 + r < rows) q128_load(x + (r0 + r) * 128, lane, a[r], raw);
#pragma unroll
  for (int r = 0; r < Q128_ROWS; ++r)
    if (r0 + r < rows) quantize_row128(a[r], bits, q + (r0 + r) * Dq, scale + r0 + r, zp + r0 + r, lane);
}

__global__ void __launch_bounds__(Q_WARPS * 32)
dequantize_rows128_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scale, const int32_t* __restrict__ zp,
                          __nv_bfloat16* __restrict__ out, int B, int G, int n, long long q_sb, long long q_sg, long long q_sn,
                          long long m_sb, long long m_sg, long long o_sb, long long o_sg, long long o_sn, int bits) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * Q_WARPS + (threadIdx.x >> 5);
  if (row >= (long long)B * G * n) return;
  const int i = (int)(row % n);
  const int g = (int)((row / n) % G);
  const int b = (int)(row / ((long long)n * G));
  const uint8_t* qr = q + b * q_sb + g * q_sg + i * q_sn;
  const float s = scale[b * m_sb + g * m_sg + i];
  const float z = (float)zp[b * m_sb + g * m_sg + i];
  uint32_t c[4];
  if (bits == 8) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(qr + 4 * lane);
#pragma unroll
    for (int k = 0; k < 4; ++k) c[k] = (w >> (8 * k)) & 0xFFu;
  } else {
    // features 4·lane ..: high nibbles of bytes 4·lane .. for lane < 16, low nibbles of bytes 4·(lane − 16) .. otherwise
    const uint32_t w = *reinterpret_cast<const uint32_t*>(qr + 4 * (lane & 15));
    const int sh = lane < 16 ? 4 : 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) c[k] = (w >> (8 * k + sh)) & 0xFu;
  }
  __nv_bfloat162 lo = __floats2bfloat162_rn(((float)c[0] - z) * s, ((float)c[1] - z) * s);
  __nv_bfloat162 hi = __floats2bfloat162_rn(((float)c[2] - z) * s, ((float)c[3] - z) * s);
  uint2 o;
  o.x = *reinterpret_cast<uint32_t*>(&lo);
  o.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(out + b * o_sb + g * o_sg + i * o_sn + 4 * lane) = o;
}

// One warp per new row (b, g, i): scatter K and V into their slot, token position, quantize-on-write.
__global__ void __launch_bounds__(Q_WARPS * 32)
cache_write128_kernel(__nv_bfloat16* __restrict__ k_buf, __nv_bfloat16* __restrict__ v_buf, int32_t* __restrict__ token_pos,
                      const int32_t* __restrict__ slots, const __nv_bfloat16* __restrict__ key,
                      const __nv_bfloat16* __restrict__ value, uint8_t* __restrict__ qk, float* __restrict__ sk,
                      int32_t* __restrict__ zk, uint8_t* __restrict__ qv, float* __restrict__ sv, int32_t* __restrict__ zv, int B,
                      int G, int n, int C, long long slot_sb, long long slot_sg, long long kv_sb, long long kv_sg, int input_pos,
                      const int* __restrict__ pos_ptr, int bits, int* status) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long row = (long long)blockIdx.x * Q_WARPS + warp;
  if (row >= (long long)B * G * n) return;
  if (pos_ptr) input_pos = *pos_ptr;  // position kept on the device (captured decode step)
  const int i = (int)(row % n);
  const int g = (int)((row / n) % G);
  const int b = (int)(row / ((long long)n * G));
  const int slot = slots[b * slot_sb + g * slot_sg + i];
  if (slot < 0 || slot >= C) {  // never write out of bounds: record and skip
    if (lane == 0 && status) atomicCAS(status, 0, STATUS_BAD_INDEX);
    return;
  }
  const long long dst_row = ((long long)b * G + g) * C + slot;
  const int Dq = bits == 8 ? 128 : 64;
  float kx[4], vx[4];
  uint2 kraw, vraw;
  const long long src = b * kv_sb + g * kv_sg + (long long)i * 128;  // key / value (B,G,n,128) with batch and group strides
  q128_load(key + src, lane, kx, kraw);
  q128_load(value + src, lane, vx, vraw);
  if (lane == 0) token_pos[dst_row] = input_pos + i;
  if (k_buf) *reinterpret_cast<uint2*>(k_buf + dst_row * 128 + 4 * lane) = kraw;
  if (v_buf) *reinterpret_cast<uint2*>(v_buf + dst_row * 128 + 4 * lane) = vraw;
  if (qk) quantize_row128(kx, bits, qk + dst_row * Dq, sk + dst_row, zk + dst_row, lane);
  if (qv) quantize_row128(vx, bits, qv + dst_row * Dq, sv + dst_row, zv + dst_row, lane);
}

// ---- gradient replay: one kernel per direction instead of a dozen gathers / scatters / casts.
// Forward of a replay step: save what the slots held (K, V rows and token positions), then write
// the chunk's rows. bf16, rows of 128 values, one warp per new row (b, g, i).
__global__ void __launch_bounds__(Q_WARPS * 32)
replay_write128_kernel(__nv_bfloat16* __restrict__ k_buf, __nv_bfloat16* __restrict__ v_buf, int32_t* __restrict__ token_pos,
                       const int32_t* __restrict__ slots, const __nv_bfloat16* __restrict__ key,
                       const __nv_bfloat16* __restrict__ value, __nv_bfloat16* __restrict__ old_k, __nv_bfloat16* __restrict__ old_v,
                       int32_t* __restrict__ old_tp, int B, int G, int n, int C, long long slot_sb, long long slot_sg,
                       long long kv_sb, long long kv_sg, long long kv_sn, int input_pos, int* status) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long row = (long long)blockIdx.x * Q_WARPS + warp;
  if (row >= (long long)B * G * n) return;
  const int i = (int)(row % n);
  const int g = (int)((row / n) % G);
  const int b = (int)(row / ((long long)n * G));
  const int slot = slots[b * slot_sb + g * slot_sg + i];
  if (slot < 0 || slot >= C) {  // never touch memory out of bounds: record and skip
    if (lane == 0 && status) atomicCAS(status, 0, STATUS_BAD_INDEX);
    return;
  }
  const long long dst_row = ((long long)b * G + g) * C + slot;
  const long long src = b * kv_sb + g * kv_sg + i * kv_sn + 4 * lane;
  const uint2 kn = *reinterpret_cast<const uint2*>(key + src), vn = *reinterpret_cast<const uint2*>(value + src);
  uint2* kd = reinterpret_cast<uint2*>(k_buf + dst_row * 128 + 4 * lane);
  uint2* vd = reinterpret_cast<uint2*>(v_buf + dst_row * 128 + 4 * lane);
  *reinterpret_cast<uint2*>(old_k + row * 128 + 4 * lane) = *kd;
  *reinterpret_cast<uint2*>(old_v + row * 128 + 4 * lane) = *vd;
  *kd = kn;
  *vd = vn;
  if (lane == 0) {
    old_tp[row] = token_pos[dst_row];
    token_pos[dst_row] = input_pos + i;
  }
}

// Backward of a replay step: the gradients of the chunk's K, V rows are what has accumulated in
// their slots (taken out as bf16, the slots are cleared), and the slots get their old content back.
__global__ void __launch_bounds__(Q_WARPS * 32)
replay_undo128_kernel(__nv_bfloat16* __restrict__ k_buf, __nv_bfloat16* __restrict__ v_buf, int32_t* __restrict__ token_pos,
                      float* __restrict__ dk_buf, float* __restrict__ dv_buf, const int32_t* __restrict__ slots,
                      const __nv_bfloat16* __restrict__ old_k, const __nv_bfloat16* __restrict__ old_v,
                      const int32_t* __restrict__ old_tp, __nv_bfloat16* __restrict__ dk_new, __nv_bfloat16* __restrict__ dv_new,
                      int B, int G, int n, int C, long long slot_sb, long long slot_sg, int* status) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long row = (long long)blockIdx.x * Q_WARPS + warp;
  if (row >= (long long)B * G * n) return;
  const int i = (int)(row % n);
  const int g = (int)((row / n) % G);
  const int b = (int)(row / ((long long)n * G));
  const int slot = slots[b * slot_sb + g * slot_sg + i];
  if (slot < 0 || slot >= C) {
    if (lane == 0 && status) atomicCAS(status, 0, STATUS_BAD_INDEX);
    return;
  }
  const long long dst_row = ((long long)b * G + g) * C + slot;
  float4* dkp = reinterpret_cast<float4*>(dk_buf + dst_row * 128 + 4 * lane);
  float4* dvp = reinterpret_cast<float4*>(dv_buf + dst_row * 128 + 4 * lane);
  const float4 a = *dkp, c = *dvp;
  __nv_bfloat162 a0 = __floats2bfloat162_rn(a.x, a.y), a1 = __floats2bfloat162_rn(a.z, a.w);
  __nv_bfloat162 c0 = __floats2bfloat162_rn(c.x, c.y), c1 = __floats2bfloat162_rn(c.z, c.w);
  uint2 ao, co;
  ao.x = *reinterpret_cast<uint32_t*>(&a0); ao.y = *reinterpret_cast<uint32_t*>(&a1);
  co.x = *reinterpret_cast<uint32_t*>(&c0); co.y = *reinterpret_cast<uint32_t*>(&c1);
  *reinterpret_cast<uint2*>(dk_new + row * 128 + 4 * lane) = ao;
  *reinterpret_cast<uint2*>(dv_new + row * 128 + 4 * lane) = co;
  *dkp = make_float4(0.f, 0.f, 0.f, 0.f);
  *dvp = make_float4(0.f, 0.f, 0.f, 0.f);
  *reinterpret_cast<uint2*>(k_buf + dst_row * 128 + 4 * lane) = *reinterpret_cast<const uint2*>(old_k + row * 128 + 4 * lane);
  *reinterpret_cast<uint2*>(v_buf + dst_row * 128 + 4 * lane) = *reinterpret_cast<const uint2*>(old_v + row * 128 + 4 * lane);
  if (lane == 0) token_pos[dst_row] = old_tp[row];
}

template <typename T>
__global__ void quantize_rows_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scale,
                                     int32_t* __restrict__ zp, long long rows, int D, int bits) {
  extern __shared__ float sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* xs = sm + warp * D;
  const long long row = (long long)blockIdx.x * Q_WARPS + warp;
  if (row >= rows) return;
  const T* xr = x + row * D;
  for (int i = lane; i < D; i += 32) xs[i] = to_f32(xr[i]);
  __syncwarp();
  const int Dq = bits == 8 ? D : D / 2;
  quantize_row_warp(xs, D, bits, q + row * Dq, scale + row, zp + row, lane);
}

template <typename T>
__global__ void dequantize_rows_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scale,
                                       const int32_t* __restrict__ zp, T* __restrict__ out, int B, int G, int n, int D,
                                       long long q_sb, long long q_sg, long long q_sn, long long m_sb, long long m_sg,
                                       long long o_sb, long long o_sg, long long o_sn, int bits) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * Q_WARPS + (threadIdx.x >> 5);
  if (row >= (long long)B * G * n) return;
  const int i = (int)(row % n);
  const int g = (int)((row / n) % G);
  const int b = (int)(row / ((long long)n * G));
  const uint8_t* qr = q + b * q_sb + g * q_sg + i * q_sn;
  const float s = scale[b * m_sb + g * m_sg + i];
  const float z = (float)zp[b * m_sb + g * m_sg + i];
  T* o = out + b * o_sb + g * o_sg + i * o_sn;
  if (bits == 8) {
    for (int j = lane; j < D; j += 32) o[j] = from_f32<T>(((float)qr[j] - z) * s);
  } else {
    const int half = D >> 1;
    for (int j = lane; j < half; j += 32) {
      const uint32_t byte = qr[j];
      o[j] = from_f32<T>(((float)(byte >> 4) - z) * s);
      o[j + half] = from_f32<T>(((float)(byte & 0xF) - z) * s);
    }
  }
}

// One warp per new row (b, g, i).
template <typename T>
__global__ void cache_write_kernel(T* __restrict__ k_buf, T* __restrict__ v_buf, int32_t* __restrict__ token_pos,
                                   const int32_t* __restrict__ slots, const T* __restrict__ key, const T* __restrict__ value,
                                   uint8_t* __restrict__ qk, float* __restrict__ sk, int32_t* __restrict__ zk,
                                   uint8_t* __restrict__ qv, float* __restrict__ sv, int32_t* __restrict__ zv, int B, int G, int n,
                                   int D, int C, long long slot_sb, long long slot_sg, long long kv_sb, long long kv_sg, int input_pos,
                                   const int* __restrict__ pos_ptr, int bits, int* status) {
  extern __shared__ float sm[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* xs = sm + warp * D;
  const long long row = (long long)blockIdx.x * Q_WARPS + warp;
  if (row >= (long long)B * G * n) return;
  if (pos_ptr) input_pos = *pos_ptr;
  const int i = (int)(row % n);
  const int g = (int)((row / n) % G);
  const int b = (int)(row / ((long long)n * G));
  const int slot = slots[b * slot_sb + g * slot_sg + i];
  if (slot < 0 || slot >= C) {  // never write out of bounds: record and skip
    if (lane == 0 && status) atomicCAS(status, 0, STATUS_BAD_INDEX);
    return;
  }
  const long long bg = (long long)b * G + g;
  const long long dst_row = bg * C + slot;
  const T* kr = key + b * kv_sb + g * kv_sg + (long long)i * D;
  const T* vr = value + b * kv_sb + g * kv_sg + (long long)i * D;
  if (lane == 0) token_pos[dst_row] = input_pos + i;
  const int Dq = bits == 8 ? D : D / 2;
  // keys
  for (int j = lane; j < D; j += 32) {
    T val = kr[j];
    if (k_buf) k_buf[dst_row * D + j] = val;
    xs[j] = to_f32(val);
  }
  __syncwarp();
  if (qk) quantize_row_warp(xs, D, bits, qk + dst_row * Dq, sk + dst_row, zk + dst_row, lane);
  __syncwarp();
  // values
  for (int j = lane; j < D; j += 32) {
    T val = vr[j];
    if (v_buf) v_buf[dst_row * D + j] = val;
    xs[j] = to_f32(val);
  }
  __syncwarp();
  if (qv) quantize_row_warp(xs, D, bits, qv + dst_row * Dq, sv + dst_row, zv + dst_row, lane);
}

}  // namespace kvb

using namespace kvb;

#define KVB_DISPATCH_DTYPE(dtype, ...)                      \
  switch (dtype) {                                          \
    case 0: { using T = float; __VA_ARGS__; break; }        \
    case 1: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
    case 2: { using T = __half; __VA_ARGS__; break; }       \
    default: return KVB_ERR_ARG;                            \
  }

extern "C" int kvb_quantize_rows(const void* x, uint8_t* q, float* scale, int32_t* zp, long long rows, int D, int bits,
                                 int dtype, void* stream) {
  if (rows <= 0 || D <= 0 || (bits != 4 && bits != 8) || (bits == 4 && (D & 1))) return KVB_ERR_ARG;
  if (dtype == 1 && D == 128 && !(reinterpret_cast<uintptr_t>(x) & 7) && !(reinterpret_cast<uintptr_t>(q) & 3)) {
    const unsigned g128 = (unsigned)((rows + Q128_ROWS * Q_WARPS - 1) / (Q128_ROWS * Q_WARPS));
    quantize_rows128_kernel<<<g128, Q_WARPS * 32, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, q, scale, zp, rows, bits);
    return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
  }
  if ((size_t)Q_WARPS * D * 4 > 48 * 1024) return KVB_ERR_TOO_LARGE;
  const unsigned grid = (unsigned)((rows + Q_WARPS - 1) / Q_WARPS);
  KVB_DISPATCH_DTYPE(dtype, (quantize_rows_kernel<T><<<grid, Q_WARPS * 32, (size_t)Q_WARPS * D * 4, (cudaStream_t)stream>>>(
                                (const T*)x, q, scale, zp, rows, D, bits)));
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

extern "C" int kvb_dequantize_rows(const uint8_t* q, const float* scale, const int32_t* zp, void* out, int B, int G, int n, int D,
                                   long long q_sb, long long q_sg, long long q_sn, long long m_sb, long long m_sg,
                                   long long o_sb, long long o_sg, long long o_sn, int bits, int dtype, void* stream) {
  if (B <= 0 || G <= 0 || n <= 0 || D <= 0 || (bits != 4 && bits != 8)) return KVB_ERR_ARG;
  const long long rows = (long long)B * G * n;
  const unsigned grid = (unsigned)((rows + Q_WARPS - 1) / Q_WARPS);
  if (dtype == 1 && D == 128 && !(reinterpret_cast<uintptr_t>(q) & 3) && !(reinterpret_cast<uintptr_t>(out) & 7) &&
      !((q_sb | q_sg | q_sn) & 3) && !((o_sb | o_sg | o_sn) & 3)) {
    dequantize_rows128_kernel<<<grid, Q_WARPS * 32, 0, (cudaStream_t)stream>>>(q, scale, zp, (__nv_bfloat16*)out, B, G, n, q_sb, q_sg,
                                                                              q_sn, m_sb, m_sg, o_sb, o_sg, o_sn, bits);
    return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
  }
  KVB_DISPATCH_DTYPE(dtype, (dequantize_rows_kernel<T><<<grid, Q_WARPS * 32, 0, (cudaStream_t)stream>>>(
                                q, scale, zp, (T*)out, B, G, n, D, q_sb, q_sg, q_sn, m_sb, m_sg, o_sb, o_sg, o_sn, bits)));
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

// While a position source is set, cache writes and the H2O update take the position of the step's
// first token from that device word instead of their host argument, so that a captured CUDA graph
// of a decode step can be replayed for later positions. The pointer must stay valid until cleared.
static const int* g_position_source = nullptr;
extern "C" void kvb_set_position_source(const int* device_word) { g_position_source = device_word; }
extern "C" const int* kvb_position_source() { return g_position_source; }

extern "C" int kvb_cache_write(void* k_buf, void* v_buf, int32_t* token_pos, const int32_t* slots, const void* key,
                               const void* value, uint8_t* qk, float* sk, int32_t* zk, uint8_t* qv, float* sv, int32_t* zv, int B,
                               int G, int n, int D, int C, long long slot_sb, long long slot_sg, int input_pos, int bits,
                               int dtype, int* status, void* stream) {
  return kvb_cache_write_strided(k_buf, v_buf, token_pos, slots, key, value, qk, sk, zk, qv, sv, zv, B, G, n, D, C, slot_sb, slot_sg,
                                 (long long)G * n * D, (long long)n * D, input_pos, bits, dtype, status, stream);
}

// key / value (B,G,n,D) with batch and group strides kv_sb, kv_sg in elements (rows D apart): a slice of positions of a
// longer (B,G,T,D) tensor is written without a copy.
extern "C" int kvb_cache_write_strided(void* k_buf, void* v_buf, int32_t* token_pos, const int32_t* slots, const void* key,
                                       const void* value, uint8_t* qk, float* sk, int32_t* zk, uint8_t* qv, float* sv, int32_t* zv,
                                       int B, int G, int n, int D, int C, long long slot_sb, long long slot_sg, long long kv_sb,
                                       long long kv_sg, int input_pos, int bits, int dtype, int* status, void* stream) {
  if (B <= 0 || G <= 0 || n <= 0 || D <= 0 || C <= 0) return KVB_ERR_ARG;
  if (qk && bits != 4 && bits != 8) return KVB_ERR_ARG;
  if ((size_t)Q_WARPS * D * 4 > 48 * 1024) return KVB_ERR_TOO_LARGE;
  const long long rows = (long long)B * G * n;
  const unsigned grid = (unsigned)((rows + Q_WARPS - 1) / Q_WARPS);
  auto al = [](const void* p, uintptr_t m) { return (reinterpret_cast<uintptr_t>(p) & m) == 0; };
  if (dtype == 1 && D == 128 && al(key, 7) && al(value, 7) && al(k_buf, 7) && al(v_buf, 7) && al(qk, 3) && al(qv, 3) &&
      kv_sb % 4 == 0 && kv_sg % 4 == 0) {
    cache_write128_kernel<<<grid, Q_WARPS * 32, 0, (cudaStream_t)stream>>>(
        (__nv_bfloat16*)k_buf, (__nv_bfloat16*)v_buf, token_pos, slots, (const __nv_bfloat16*)key, (const __nv_bfloat16*)value, qk,
        sk, zk, qv, sv, zv, B, G, n, C, slot_sb, slot_sg, kv_sb, kv_sg, input_pos, g_position_source, bits ? bits : 8, status);
    return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
  }
  KVB_DISPATCH_DTYPE(dtype, (cache_write_kernel<T><<<grid, Q_WARPS * 32, (size_t)Q_WARPS * D * 4, (cudaStream_t)stream>>>(
                                (T*)k_buf, (T*)v_buf, token_pos, slots, (const T*)key, (const T*)value, qk, sk, zk, qv, sv, zv, B,
                                G, n, D, C, slot_sb, slot_sg, kv_sb, kv_sg, input_pos, g_position_source, bits ? bits : 8, status)));
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

// Replay step forward / backward for bf16 caches with head size 128 (see the kernels). key / value
// may be strided views (strides in elements; the last axis has unit stride); old_* and d*_new are
// contiguous (B,G,n,128) / (B,G,n). Slots of one (b, g) must be distinct.
extern "C" int kvb_replay_write(void* k_buf, void* v_buf, int32_t* token_pos, const int32_t* slots, const void* key,
                                const void* value, void* old_k, void* old_v, int32_t* old_tp, int B, int G, int n, int D, int C,
                                long long slot_sb, long long slot_sg, long long kv_sb, long long kv_sg, long long kv_sn,
                                int input_pos, int* status, void* stream) {
  if (B <= 0 || G <= 0 || n <= 0 || C <= 0) return KVB_ERR_ARG;
  if (D != 128 || ((kv_sb | kv_sg | kv_sn) & 3)) return KVB_ERR_UNSUPPORTED;
  const long long rows = (long long)B * G * n;
  const unsigned grid = (unsigned)((rows + Q_WARPS - 1) / Q_WARPS);
  replay_write128_kernel<<<grid, Q_WARPS * 32, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)k_buf, (__nv_bfloat16*)v_buf, token_pos, slots, (const __nv_bfloat16*)key, (const __nv_bfloat16*)value,
      (__nv_bfloat16*)old_k, (__nv_bfloat16*)old_v, old_tp, B, G, n, C, slot_sb, slot_sg, kv_sb, kv_sg, kv_sn, input_pos, status);
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

extern "C" int kvb_replay_undo(void* k_buf, void* v_buf, int32_t* token_pos, float* dk_buf, float* dv_buf, const int32_t* slots,
                               const void* old_k, const void* old_v, const int32_t* old_tp, void* dk_new, void* dv_new, int B,
                               int G, int n, int D, int C, long long slot_sb, long long slot_sg, int* status, void* stream) {
  if (B <= 0 || G <= 0 || n <= 0 || C <= 0) return KVB_ERR_ARG;
  if (D != 128) return KVB_ERR_UNSUPPORTED;
  const long long rows = (long long)B * G * n;
  const unsigned grid = (unsigned)((rows + Q_WARPS - 1) / Q_WARPS);
  replay_undo128_kernel<<<grid, Q_WARPS * 32, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)k_buf, (__nv_bfloat16*)v_buf, token_pos, dk_buf, dv_buf, slots, (const __nv_bfloat16*)old_k,
      (const __nv_bfloat16*)old_v, old_tp, (__nv_bfloat16*)dk_new, (__nv_bfloat16*)dv_new, B, G, n, C, slot_sb, slot_sg, status);
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}
