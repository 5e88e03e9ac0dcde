// Token cross-entropy over a chunk of logits, forward and backward.
//
//   loss[r] = logsumexp(logits[r, :]) − logits[r, target[r]]      (0 where target[r] == ignore_index)
//   dlogits[r, v] = g[r] · (exp(logits[r, v] − lse[r]) − [v == target[r]])
//
// One CTA per row: 16-byte loads of the row in its storage dtype (bf16 or fp32; no fp32 copy of
// the logits is made), online max / sum per thread, one block reduction. The backward writes the
// gradient in the dtype of the logits. Used on the ≤ 2 GiB pieces of logits that the loss of a
// chunk is evaluated in.
//
// Replaces the fp32 upcast + library cross_entropy of keys_values/head_model.py:94-114 and the
// chunked loss of keys_values/long_context.py:226-300.
#include <float.h>

#include "common.cuh"
#include "kvb200.h"

namespace kvb {

constexpr int CE_THREADS = 256;

template <typename T>
__device__ __forceinline__ float ce_load(const T* p, long long i);
template <>
__device__ __forceinline__ float ce_load<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float ce_load<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }

// (max, sum of exp(x − max)) of one row, reduced over the block
template <typename T>
__device__ __forceinline__ void ce_row_stats(const T* row, int V, float& m_out, float& l_out) {
  constexpr int VEC = 16 / sizeof(T);
  float m = -FLT_MAX, l = 0.f;
  const int nvec = ((reinterpret_cast<uintptr_t>(row) & 15) == 0) ? V / VEC : 0;
  for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + (long long)i * VEC);
    const T* e = reinterpret_cast<const T*>(&raw);
    float x[VEC], mx = -FLT_MAX;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      x[j] = ce_load<T>(e, j);
      mx = fmaxf(mx, x[j]);
    }
    const float mn = fmaxf(m, mx);
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < VEC; ++j) s += __expf(x[j] - mn);
    l = l * __expf(m - mn) + s;
    m = mn;
  }
  for (int i = nvec * VEC + threadIdx.x; i < V; i += CE_THREADS) {
    const float x = ce_load<T>(row, i);
    const float mn = fmaxf(m, x);
    l = l * __expf(m - mn) + __expf(x - mn);
    m = mn;
  }
  // block reduction of (m, l)
  __shared__ float sm_m[CE_THREADS / 32], sm_l[CE_THREADS / 32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), l2 = __shfl_xor_sync(0xffffffffu, l, o);
    const float mn = fmaxf(m, m2);
    l = l * __expf(m - mn) + l2 * __expf(m2 - mn);
    m = mn;
  }
  if (lane == 0) {
    sm_m[warp] = m;
    sm_l[warp] = l;
  }
  __syncthreads();
  m = sm_m[0];
  l = sm_l[0];
  for (int w = 1; w < CE_THREADS / 32; ++w) {
    const float mn = fmaxf(m, sm_m[w]);
    l = l * __expf(m - mn) + sm_l[w] * __expf(sm_m[w] - mn);
    m = mn;
  }
  m_out = m;
  l_out = l;
}

template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_kernel(const T* __restrict__ logits, const long long* __restrict__ targets, float* __restrict__ loss, float* __restrict__ lse,
              int V, long long ld, long long ignore_index) {
  const long long r = blockIdx.x;
  const T* row = logits + r * ld;
  float m, l;
  ce_row_stats<T>(row, V, m, l);
  if (threadIdx.x == 0) {
    const float z = m + logf(l);
    lse[r] = z;
    const long long t = targets[r];
    loss[r] = (t == ignore_index || t < 0 || t >= V) ? 0.f : z - ce_load<T>(row, t);
  }
}

template <typename T>
__global__ void __launch_bounds__(CE_THREADS)
ce_bwd_kernel(const T* __restrict__ logits, const long long* __restrict__ targets, const float* __restrict__ lse,
              const float* __restrict__ grad, T* __restrict__ dlogits, int V, long long ld, long long ignore_index) {
  const long long r = blockIdx.x;
  const T* row = logits + r * ld;
  T* drow = dlogits + r * ld;
  const long long t = targets[r];
  const bool live = !(t == ignore_index || t < 0 || t >= V);
  const float g = live ? grad[r] : 0.f;
  const float z = lse[r];
  for (int i = threadIdx.x; i < V; i += CE_THREADS) {
    float d = g * __expf(ce_load<T>(row, i) - z);
    if (i == t) d -= g;
    if (sizeof(T) == 4) reinterpret_cast<float*>(drow)[i] = d;
    else reinterpret_cast<__nv_bfloat16*>(drow)[i] = __float2bfloat16_rn(d);
  }
}

}  // namespace kvb

// logits (rows, V) with row stride ld (elements), dtype 0 = fp32, 1 = bf16; targets int64 (rows);
// loss, lse fp32 (rows).
extern "C" int kvb_ce_loss_fwd(const void* logits, const long long* targets, float* loss, float* lse, long long rows, int V,
                               long long ld, long long ignore_index, int dtype, void* stream) {
  using namespace kvb;
  if (rows <= 0 || V <= 0 || ld < V) return KVB_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == 0) ce_fwd_kernel<float><<<(unsigned)rows, CE_THREADS, 0, s>>>((const float*)logits, targets, loss, lse, V, ld, ignore_index);
  else if (dtype == 1)
    ce_fwd_kernel<__nv_bfloat16><<<(unsigned)rows, CE_THREADS, 0, s>>>((const __nv_bfloat16*)logits, targets, loss, lse, V, ld, ignore_index);
  else return KVB_ERR_ARG;
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

// grad (rows) fp32: gradient of the objective w.r.t. loss[r]; dlogits has the shape and dtype of logits.
extern "C" int kvb_ce_loss_bwd(const void* logits, const long long* targets, const float* lse, const float* grad, void* dlogits,
                               long long rows, int V, long long ld, long long ignore_index, int dtype, void* stream) {
  using namespace kvb;
  if (rows <= 0 || V <= 0 || ld < V) return KVB_ERR_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == 0)
    ce_bwd_kernel<float><<<(unsigned)rows, CE_THREADS, 0, s>>>((const float*)logits, targets, lse, grad, (float*)dlogits, V, ld, ignore_index);
  else if (dtype == 1)
    ce_bwd_kernel<__nv_bfloat16><<<(unsigned)rows, CE_THREADS, 0, s>>>((const __nv_bfloat16*)logits, targets, lse, grad,
                                                                      (__nv_bfloat16*)dlogits, V, ld, ignore_index);
  else return KVB_ERR_ARG;
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

// ---------------------------------------------------------------------------------------------
// Greedy sampling: index of the largest logit of every row (the first one among equals, as
// torch.argmax), in two stages so that a handful of rows of a 128k vocabulary use the whole GPU:
// ARGMAX_SPLITS CTAs per row reduce a slice each, the last CTA to finish a row combines them.
// ---------------------------------------------------------------------------------------------
namespace kvb {
constexpr int ARGMAX_SPLITS = 32;
constexpr int ARGMAX_THREADS = 256;

__device__ __forceinline__ void argmax_combine(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) {
    v = ov;
    i = oi;
  }
}

template <typename T>
__global__ void __launch_bounds__(ARGMAX_THREADS)
argmax_rows_kernel(const T* __restrict__ logits, long long* __restrict__ out, float* __restrict__ part_v, int* __restrict__ part_i,
                   unsigned* __restrict__ counters, int V, long long ld) {
  __shared__ float sv[ARGMAX_THREADS / 32];
  __shared__ int si[ARGMAX_THREADS / 32];
  __shared__ int last;
  const int row = blockIdx.y, split = blockIdx.x, tid = threadIdx.x;
  const T* x = logits + (long long)row * ld;
  const int per = (V + ARGMAX_SPLITS - 1) / ARGMAX_SPLITS;
  const int j0 = split * per, j1 = min(V, j0 + per);
  float v = -INFINITY;
  int idx = 0x7fffffff;
  for (int j = j0 + tid; j < j1; j += ARGMAX_THREADS) {
    float f = to_f32(x[j]);
    if (f != f) f = INFINITY;  // a NaN ranks with +inf: it wins, like in torch.argmax
    if (f > v || (f == v && j < idx)) {
      v = f;
      idx = j;
    }
  }
  auto block_reduce = [&]() {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) argmax_combine(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if ((tid & 31) == 0) {
      sv[tid >> 5] = v;
      si[tid >> 5] = idx;
    }
    __syncthreads();
    if (tid < 32) {
      v = tid < ARGMAX_THREADS / 32 ? sv[tid] : -INFINITY;
      idx = tid < ARGMAX_THREADS / 32 ? si[tid] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) argmax_combine(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
    }
  };
  block_reduce();
  if (tid == 0) {
    part_v[row * ARGMAX_SPLITS + split] = v;
    part_i[row * ARGMAX_SPLITS + split] = idx;
    __threadfence();
    last = atomicAdd(counters + row, 1u) == ARGMAX_SPLITS - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  if (tid < 32) {
    v = tid < ARGMAX_SPLITS ? reinterpret_cast<volatile float*>(part_v)[row * ARGMAX_SPLITS + tid] : -INFINITY;
    idx = tid < ARGMAX_SPLITS ? reinterpret_cast<volatile int*>(part_i)[row * ARGMAX_SPLITS + tid] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) argmax_combine(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if (tid == 0) {
      out[row] = idx == 0x7fffffff ? 0 : idx;
      counters[row] = 0;  // ready for the next call
    }
  }
}
}  // namespace kvb

// logits (rows, V), row stride ld (elements), dtype 0 = fp32, 1 = bf16; out int64 (rows), rows <= 65535.
// scratch: kvb_argmax_scratch_bytes(rows) bytes. Its first ARGMAX_MAX_ROWS words are the per-row counters,
// at the same place for every number of rows: zero before the first call, left zero by every call; the
// partial results of the current call lie behind them.
namespace kvb { constexpr long long ARGMAX_MAX_ROWS = 65536; }
extern "C" long long kvb_argmax_scratch_bytes(long long rows) { return kvb::ARGMAX_MAX_ROWS * 4 + rows * kvb::ARGMAX_SPLITS * 8; }

extern "C" int kvb_argmax_rows(const void* logits, long long* out, void* scratch, long long rows, int V, long long ld, int dtype,
                               void* stream) {
  using namespace kvb;
  if (rows <= 0 || rows > 65535 || V <= 0 || ld < V || !scratch) return KVB_ERR_ARG;
  unsigned* counters = reinterpret_cast<unsigned*>(scratch);
  float* part_v = reinterpret_cast<float*>(counters + ARGMAX_MAX_ROWS);
  int* part_i = reinterpret_cast<int*>(part_v + rows * ARGMAX_SPLITS);
  dim3 grid(ARGMAX_SPLITS, (unsigned)rows);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == 0) argmax_rows_kernel<float><<<grid, ARGMAX_THREADS, 0, s>>>((const float*)logits, out, part_v, part_i, counters, V, ld);
  else if (dtype == 1)
    argmax_rows_kernel<__nv_bfloat16><<<grid, ARGMAX_THREADS, 0, s>>>((const __nv_bfloat16*)logits, out, part_v, part_i, counters, V, ld);
  else return KVB_ERR_ARG;
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}
