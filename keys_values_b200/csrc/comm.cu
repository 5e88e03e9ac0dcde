// Collectives over NVLink peer memory, written as kernels that read the peers'
// buffers directly (P2P loads/stores through the NVSwitch fabric; no NCCL call, no TMA
// load from peer memory, no cluster multicast).
//
// Symmetric memory: every rank allocates an arena of the same size with cudaMalloc,
// exports it with cudaIpcGetMemHandle and maps every peer's arena with
// cudaIpcOpenMemHandle (handle exchange happens in Python over torch.distributed). A
// small flag area at the end of each arena carries the inter-GPU barriers.
//
// kvb_allreduce_mean: in-place all-reduce of a slice of the arena, fused with the 1/world
// scale and the dtype cast:
//   barrier  ->  rank r pulls shard r from all ranks (several 16-byte loads per peer in flight
//   per thread), sums in fp32 in a fixed rank order, so every run and every rank gives identical
//   bits, and pushes scale·sum into shard r of every rank's arena (posted stores)
//   barrier  (nobody reads its arena before every push has landed)
// Every wait is bounded: on timeout the kernel records STATUS_TIMEOUT_PEER_FLAG and
// returns.
//
// Replaces the flatten -> NCCL all_reduce -> copy-back sequence of
// keys_values/optimize/grad_accumulate.py:196-245.
#include <string.h>

#include "common.cuh"
#include "kvb200.h"

namespace kvb {

constexpr int COMM_MAX_RANKS = 16;
constexpr int COMM_THREADS = 512;

struct CommPeers {
  void* base[COMM_MAX_RANKS];       // arena of every rank, mapped into this process
  uint32_t* flags[COMM_MAX_RANKS];  // flag area of every rank: [COMM_MAX_RANKS] words, one per writer
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Barrier across ranks for a whole grid. `sync` points to two words owned by this rank:
// sync[0] = release (last epoch completed), sync[1] = number of local CTAs that arrived.
// Every CTA arrives locally (after making its writes visible system-wide); CTA 0 waits
// for all of them, exchanges flags with the peers and releases the other CTAs. `epoch`
// must increase by one for every barrier of the communicator. All CTAs of the grid must
// be resident at the same time (the launcher keeps the grid far below the SM count).
__device__ bool cross_gpu_barrier(const CommPeers& peers, int rank, int world, uint32_t epoch, uint32_t* sync, int* status,
                                  long long limit) {
  __shared__ int ok_s;
  __syncthreads();
  if (threadIdx.x == 0) {
    ok_s = 1;
    __threadfence_system();
    atomicAdd(sync + 1, 1u);
  }
  __syncthreads();
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) {
      long long t0 = clock64();
      while (*((volatile uint32_t*)(sync + 1)) < gridDim.x) {
        if (clock64() - t0 > limit) {
          if (status) atomicCAS(status, 0, STATUS_TIMEOUT_PEER_FLAG);
          ok_s = 0;
          break;
        }
      }
      *((volatile uint32_t*)(sync + 1)) = 0;
      __threadfence_system();
    }
    __syncthreads();
    if ((int)threadIdx.x < world && ok_s) {
      const int peer = threadIdx.x;
      st_release_sys(peers.flags[peer] + rank, epoch);  // tell `peer` that this rank has arrived
      const uint32_t* mine = peers.flags[rank] + peer;  // wait until `peer` has arrived here
      long long t0 = clock64();
      while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
        if (clock64() - t0 > limit) {
          if (status) atomicCAS(status, 0, STATUS_TIMEOUT_PEER_FLAG);
          ok_s = 0;
          break;
        }
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      atomicExch(sync, ok_s ? epoch : 0xFFFFFFFFu);
    }
  } else {
    if (threadIdx.x == 0) {
      long long t0 = clock64();
      while (true) {
        const uint32_t v = *((volatile uint32_t*)sync);
        if (v == 0xFFFFFFFFu) {
          ok_s = 0;
          break;
        }
        if ((int32_t)(v - epoch) >= 0) break;
        if (clock64() - t0 > 3 * limit) {
          if (status) atomicCAS(status, 0, STATUS_TIMEOUT_PEER_FLAG);
          ok_s = 0;
          break;
        }
      }
      __threadfence();
    }
  }
  __syncthreads();
  return ok_s != 0;
}

// Vectors of 16 bytes that one thread keeps in flight per peer. Remote loads take a few
// microseconds, so the bandwidth of the reduction is (bytes in flight) / latency.
constexpr int COMM_UNROLL = 4;

template <typename T>
__global__ void __launch_bounds__(COMM_THREADS)
allreduce_mean_kernel(CommPeers peers, int rank, int world, long long start, long long count, float scale, uint32_t epoch0,
                      uint32_t* sync, int* status, long long limit) {
  constexpr int V = 16 / sizeof(T);
  constexpr int U = COMM_UNROLL;
  if (!cross_gpu_barrier(peers, rank, world, epoch0, sync, status, limit)) return;
  // shards in units of 16-byte vectors
  const long long nvec = count / V;
  const long long per = (nvec + world - 1) / world;
  const long long v0 = min(per * rank, nvec), v1 = min(v0 + per, nvec);
  const long long step = (long long)gridDim.x * blockDim.x * U;
  // pull shard `rank` from every rank (U loads per peer in flight), reduce in fp32 in a fixed
  // rank order, push scale * sum into shard `rank` of every rank
  for (long long base = v0 + (long long)blockIdx.x * blockDim.x * U; base < v1; base += step) {
    float acc[U][V];
#pragma unroll
    for (int k = 0; k < U; ++k)
#pragma unroll
      for (int j = 0; j < V; ++j) acc[k][j] = 0.f;
    for (int r = 0; r < world; ++r) {
      const T* src = reinterpret_cast<const T*>(peers.base[r]) + start;
      uint4 raw[U];
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const long long i = base + (long long)k * blockDim.x + threadIdx.x;
        raw[k] = i < v1 ? __ldcg(reinterpret_cast<const uint4*>(src + i * V)) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const T* e = reinterpret_cast<const T*>(&raw[k]);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[k][j] += to_f32(e[j]);
      }
    }
    uint4 outv[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      T* o = reinterpret_cast<T*>(&outv[k]);
#pragma unroll
      for (int j = 0; j < V; ++j) o[j] = from_f32<T>(acc[k][j] * scale);
    }
    for (int q = 0; q < world; ++q) {
      T* dst = reinterpret_cast<T*>(peers.base[(rank + q) % world]) + start;
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const long long i = base + (long long)k * blockDim.x + threadIdx.x;
        if (i < v1) *reinterpret_cast<uint4*>(dst + i * V) = outv[k];
      }
    }
  }
  // nobody returns before every rank's pushes have landed
  cross_gpu_barrier(peers, rank, world, epoch0 + 1, sync, status, limit);
}

// One-shot all-reduce (sum) for small payloads (decode steps under tensor parallelism: a few rows of the hidden
// state). Every rank's producer kernel has written its partial result into its own slot of symmetric memory
// before this launch (same stream). Each CTA tells every peer "my slot is ready" (one flag word per writer rank
// and CTA, so there is no grid barrier and no assumption on which CTAs are resident together), waits for the
// peers' words, then reads its part of ALL slots with plain peer loads, sums in fp32 in rank order (identical
// bits on every rank), adds an optional residual and writes the local output. One NVLink round trip.
//
// A slot must not be rewritten while a peer may still read it: the caller rotates over several slots
// ("sites"); a rank cannot be more than one call ahead of a peer, because every call waits for the peer's
// word of that call, so a distance of two calls between uses of one site is enough.
//
// The epoch is epoch_base + *epoch_word: in a captured decode step the base is frozen in the graph and the
// device word, which the graph advances once per replay, makes the epochs of later replays larger.
constexpr int ONESHOT_MAX_CTAS = 16;
constexpr int ONESHOT_THREADS = 256;

struct OneShotPeers {
  const void* slot[COMM_MAX_RANKS];  // this site's slot of every rank
  uint32_t* flags[COMM_MAX_RANKS];   // this site's flag words of every rank: [COMM_MAX_RANKS][ONESHOT_MAX_CTAS]
};

__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

template <typename T>
__global__ void __launch_bounds__(ONESHOT_THREADS)
oneshot_allreduce_kernel(OneShotPeers peers, int rank, int world, long long nvec, const T* __restrict__ residual, T* __restrict__ out,
                         uint32_t epoch_base, const uint32_t* epoch_word, int* status, long long limit) {
  constexpr int V = 16 / sizeof(T);
  __shared__ int ok_s;
  const uint32_t epoch = epoch_base + (epoch_word ? *epoch_word : 0u);
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
    const int peer = threadIdx.x;
    st_release_sys(peers.flags[peer] + rank * ONESHOT_MAX_CTAS + blockIdx.x, epoch);
    const uint32_t* mine = peers.flags[rank] + peer * ONESHOT_MAX_CTAS + blockIdx.x;
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - t0 > limit) {
        if (status) atomicCAS(status, 0, STATUS_TIMEOUT_PEER_FLAG);
        ok_s = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!ok_s) return;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    uint4 raw[COMM_MAX_RANKS];
#pragma unroll
    for (int r = 0; r < COMM_MAX_RANKS; ++r)
      if (r < world) raw[r] = ld_volatile_v4(reinterpret_cast<const uint4*>(peers.slot[r]) + i);
#pragma unroll
    for (int r = 0; r < COMM_MAX_RANKS; ++r)
      if (r < world) {
        const T* e = reinterpret_cast<const T*>(&raw[r]);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += to_f32(e[j]);
      }
    if (residual) {
      const uint4 rv = *(reinterpret_cast<const uint4*>(residual) + i);
      const T* e = reinterpret_cast<const T*>(&rv);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += to_f32(e[j]);
    }
    uint4 ov;
    T* o = reinterpret_cast<T*>(&ov);
#pragma unroll
    for (int j = 0; j < V; ++j) o[j] = from_f32<T>(acc[j]);
    *(reinterpret_cast<uint4*>(out) + i) = ov;
  }
}


// One-shot all-reduce fused with the residual add and the RMSNorm that follows it in a transformer block:
//   x_new = Σ_r partial_r + residual      (written to out_x: the residual stream)
//   normed = x_new · rsqrt(mean(x_new²) + eps) · w   (written to out_normed: the input of the next linears)
// One CTA per row (a decode step has a handful of rows), so the row's sum of squares never leaves the CTA; a thread
// keeps its up to ONESHOT_NORM_VEC 16-byte pieces of the row in registers between the two passes. Same flag
// protocol and epochs as oneshot_allreduce_kernel (flag word of CTA = row).
constexpr int ONESHOT_NORM_VEC = 4;  // 16-byte vectors per thread: rows of up to 4 · 256 · 8 = 8192 16-bit features

template <typename T>
__global__ void __launch_bounds__(ONESHOT_THREADS)
oneshot_allreduce_norm_kernel(OneShotPeers peers, int rank, int world, int feat, const T* __restrict__ residual,
                              const T* __restrict__ norm_w, float eps, int unit_offset, T* __restrict__ out_x,
                              T* __restrict__ out_normed, uint32_t epoch_base, const uint32_t* epoch_word, int* status,
                              long long limit) {
  constexpr int V = 16 / sizeof(T);
  __shared__ int ok_s;
  __shared__ float red_s[ONESHOT_THREADS / 32];
  const uint32_t epoch = epoch_base + (epoch_word ? *epoch_word : 0u);
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if ((int)threadIdx.x < world && (int)threadIdx.x != rank) {
    const int peer = threadIdx.x;
    st_release_sys(peers.flags[peer] + rank * ONESHOT_MAX_CTAS + blockIdx.x, epoch);
    const uint32_t* mine = peers.flags[rank] + peer * ONESHOT_MAX_CTAS + blockIdx.x;
    const long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if (clock64() - t0 > limit) {
        if (status) atomicCAS(status, 0, STATUS_TIMEOUT_PEER_FLAG);
        ok_s = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!ok_s) return;
  const int nvec = feat / V;
  const long long row0 = (long long)blockIdx.x * nvec;  // in vectors
  float x[ONESHOT_NORM_VEC][V];
  float sq = 0.f;
#pragma unroll
  for (int k = 0; k < ONESHOT_NORM_VEC; ++k) {
    const int i = k * ONESHOT_THREADS + threadIdx.x;
    if (i < nvec) {
      float acc[V];
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] = 0.f;
      uint4 raw[COMM_MAX_RANKS];  // all ranks' pieces are requested before the first one is used
#pragma unroll
      for (int r = 0; r < COMM_MAX_RANKS; ++r)
        if (r < world) raw[r] = ld_volatile_v4(reinterpret_cast<const uint4*>(peers.slot[r]) + row0 + i);
#pragma unroll
      for (int r = 0; r < COMM_MAX_RANKS; ++r)
        if (r < world) {
          const T* e = reinterpret_cast<const T*>(&raw[r]);
#pragma unroll
          for (int j = 0; j < V; ++j) acc[j] += to_f32(e[j]);
        }
      if (residual) {
        const uint4 rv = *(reinterpret_cast<const uint4*>(residual) + row0 + i);
        const T* e = reinterpret_cast<const T*>(&rv);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += to_f32(e[j]);
      }
      uint4 ov;
      T* o = reinterpret_cast<T*>(&ov);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        o[j] = from_f32<T>(acc[j]);
        x[k][j] = to_f32(o[j]);  // the norm sees the residual stream as it is stored
        sq += x[k][j] * x[k][j];
      }
      *(reinterpret_cast<uint4*>(out_x) + row0 + i) = ov;
    }
  }
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) red_s[threadIdx.x >> 5] = sq;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int w = 0; w < ONESHOT_THREADS / 32; ++w) total += red_s[w];
  const float rstd = rsqrtf(total / (float)feat + eps);
#pragma unroll
  for (int k = 0; k < ONESHOT_NORM_VEC; ++k) {
    const int i = k * ONESHOT_THREADS + threadIdx.x;
    if (i < nvec) {
      const uint4 wv = *(reinterpret_cast<const uint4*>(norm_w) + i);
      const T* we = reinterpret_cast<const T*>(&wv);
      uint4 ov;
      T* o = reinterpret_cast<T*>(&ov);
#pragma unroll
      for (int j = 0; j < V; ++j) {
        const float w = to_f32(we[j]) + (unit_offset ? 1.f : 0.f);
        o[j] = from_f32<T>(x[k][j] * rstd * w);
      }
      *(reinterpret_cast<uint4*>(out_normed) + row0 + i) = ov;
    }
  }
}

}  // namespace kvb

using namespace kvb;

// ---- symmetric memory plumbing -------------------------------------------------------
extern "C" int kvb_symm_alloc(void** ptr, long long bytes) {
  if (cudaMalloc(ptr, (size_t)bytes) != cudaSuccess) return KVB_ERR_CUDA;
  if (cudaMemset(*ptr, 0, (size_t)bytes) != cudaSuccess) return KVB_ERR_CUDA;
  return KVB_OK;
}
extern "C" int kvb_symm_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? KVB_OK : KVB_ERR_CUDA; }
extern "C" int kvb_ipc_handle_size() { return (int)sizeof(cudaIpcMemHandle_t); }
extern "C" int kvb_ipc_get_handle(void* ptr, void* handle_out) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return KVB_ERR_CUDA;
  memcpy(handle_out, &h, sizeof(h));
  return KVB_OK;
}
extern "C" int kvb_ipc_open_handle(const void* handle, void** ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  if (cudaIpcOpenMemHandle(ptr_out, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return KVB_ERR_CUDA;
  return KVB_OK;
}
extern "C" int kvb_ipc_close_handle(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? KVB_OK : KVB_ERR_CUDA; }

// bases/flags: arrays of `world` device pointers valid in this process. dtype: 0 fp32, 1 bf16, 2 fp16.
// start/count in elements; start*sizeof(T) and the arena base must be 16-byte aligned, count a multiple of 16/sizeof(T).
extern "C" int kvb_allreduce_mean(void* const* bases, void* const* flags, int rank, int world, long long start, long long count,
                                  float scale, unsigned epoch0, void* local_sync, int dtype, int n_ctas, int* status,
                                  double timeout_s, void* stream) {
  if (world < 1 || world > COMM_MAX_RANKS || rank < 0 || rank >= world || count <= 0) return KVB_ERR_ARG;
  CommPeers peers;
  for (int r = 0; r < world; ++r) {
    peers.base[r] = bases[r];
    peers.flags[r] = reinterpret_cast<uint32_t*>(flags[r]);
  }
  const long long limit = (long long)(timeout_s * 1.9e9);
  if (n_ctas <= 0) {
    // Enough CTAs to cover the shard once, between 4 and one per SM. The grid barrier needs every CTA
    // of the launch resident at once: one per SM is safe only while nothing else occupies the SMs, so a
    // caller that runs this launch next to compute kernels passes a small n_ctas (the data-parallel
    // reducer uses 32) instead of this default.
    const long long esz = dtype == 0 ? 4 : 2;
    const long long vec_per_rank = (count * esz / 16 + world - 1) / world;
    const long long want = (vec_per_rank + (long long)COMM_THREADS * COMM_UNROLL - 1) / ((long long)COMM_THREADS * COMM_UNROLL);
    n_ctas = (int)(want < 4 ? 4 : (want > 148 ? 148 : want));
  }
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case 0:
      if ((start % 4) || (count % 4)) return KVB_ERR_ALIGN;
      allreduce_mean_kernel<float><<<n_ctas, COMM_THREADS, 0, s>>>(peers, rank, world, start, count, scale, epoch0,
                                                                  (uint32_t*)local_sync, status, limit);
      break;
    case 1:
      if ((start % 8) || (count % 8)) return KVB_ERR_ALIGN;
      allreduce_mean_kernel<__nv_bfloat16><<<n_ctas, COMM_THREADS, 0, s>>>(peers, rank, world, start, count, scale, epoch0,
                                                                          (uint32_t*)local_sync, status, limit);
      break;
    case 2:
      if ((start % 8) || (count % 8)) return KVB_ERR_ALIGN;
      allreduce_mean_kernel<__half><<<n_ctas, COMM_THREADS, 0, s>>>(peers, rank, world, start, count, scale, epoch0,
                                                                   (uint32_t*)local_sync, status, limit);
      break;
    default:
      return KVB_ERR_ARG;
  }
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

// slots/flags: arrays of `world` device pointers (this site's slot and flag block of every rank, mapped into this
// process). count elements, a multiple of 16/sizeof(T); slots, residual and out 16-byte aligned. dtype as above.
extern "C" int kvb_oneshot_allreduce(void* const* slots, void* const* flags, int rank, int world, long long count,
                                     const void* residual, void* out, unsigned epoch_base, const void* epoch_word, int dtype,
                                     int* status, double timeout_s, void* stream) {
  if (world < 1 || world > COMM_MAX_RANKS || rank < 0 || rank >= world || count <= 0) return KVB_ERR_ARG;
  const long long esz = dtype == 0 ? 4 : 2;
  if ((count * esz) % 16) return KVB_ERR_ALIGN;
  OneShotPeers peers;
  for (int r = 0; r < world; ++r) {
    if (((uintptr_t)slots[r]) % 16) return KVB_ERR_ALIGN;
    peers.slot[r] = slots[r];
    peers.flags[r] = reinterpret_cast<uint32_t*>(flags[r]);
  }
  if (((uintptr_t)out) % 16 || ((uintptr_t)residual) % 16) return KVB_ERR_ALIGN;
  const long long nvec = count * esz / 16;
  long long ctas = (nvec + ONESHOT_THREADS - 1) / ONESHOT_THREADS;
  if (ctas > ONESHOT_MAX_CTAS) ctas = ONESHOT_MAX_CTAS;
  const long long limit = (long long)(timeout_s * 1.9e9);
  cudaStream_t s = (cudaStream_t)stream;
  const uint32_t* ew = reinterpret_cast<const uint32_t*>(epoch_word);
  switch (dtype) {
    case 0:
      oneshot_allreduce_kernel<float><<<(int)ctas, ONESHOT_THREADS, 0, s>>>(peers, rank, world, nvec, (const float*)residual, (float*)out,
                                                                           epoch_base, ew, status, limit);
      break;
    case 1:
      oneshot_allreduce_kernel<__nv_bfloat16><<<(int)ctas, ONESHOT_THREADS, 0, s>>>(
          peers, rank, world, nvec, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, epoch_base, ew, status, limit);
      break;
    case 2:
      oneshot_allreduce_kernel<__half><<<(int)ctas, ONESHOT_THREADS, 0, s>>>(peers, rank, world, nvec, (const __half*)residual, (__half*)out,
                                                                           epoch_base, ew, status, limit);
      break;
    default:
      return KVB_ERR_ARG;
  }
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

// The same with the residual add and the RMSNorm of the next sub-block fused in: rows <= 16 (one CTA per row),
// features a multiple of 8 and at most 8192, 16-bit dtypes (1 bf16, 2 fp16). out_x = sum + residual (residual may be
// NULL), out_normed = rmsnorm(out_x) * norm_w (norm_w + 1 with unit_offset).
extern "C" int kvb_oneshot_allreduce_norm(void* const* slots, void* const* flags, int rank, int world, int rows, int features,
                                          const void* residual, const void* norm_w, float eps, int unit_offset, void* out_x,
                                          void* out_normed, unsigned epoch_base, const void* epoch_word, int dtype, int* status,
                                          double timeout_s, void* stream) {
  if (world < 1 || world > COMM_MAX_RANKS || rank < 0 || rank >= world || rows <= 0 || features <= 0) return KVB_ERR_ARG;
  if (rows > ONESHOT_MAX_CTAS || (features % 8) || features > ONESHOT_NORM_VEC * ONESHOT_THREADS * 8) return KVB_ERR_UNSUPPORTED;
  if (dtype != 1 && dtype != 2) return KVB_ERR_UNSUPPORTED;
  OneShotPeers peers;
  for (int r = 0; r < world; ++r) {
    if (((uintptr_t)slots[r]) % 16) return KVB_ERR_ALIGN;
    peers.slot[r] = slots[r];
    peers.flags[r] = reinterpret_cast<uint32_t*>(flags[r]);
  }
  if ((((uintptr_t)out_x) | ((uintptr_t)out_normed) | ((uintptr_t)residual) | ((uintptr_t)norm_w)) % 16) return KVB_ERR_ALIGN;
  const long long limit = (long long)(timeout_s * 1.9e9);
  cudaStream_t s = (cudaStream_t)stream;
  const uint32_t* ew = reinterpret_cast<const uint32_t*>(epoch_word);
  if (dtype == 1)
    oneshot_allreduce_norm_kernel<__nv_bfloat16><<<rows, ONESHOT_THREADS, 0, s>>>(
        peers, rank, world, features, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)norm_w, eps, unit_offset,
        (__nv_bfloat16*)out_x, (__nv_bfloat16*)out_normed, epoch_base, ew, status, limit);
  else
    oneshot_allreduce_norm_kernel<__half><<<rows, ONESHOT_THREADS, 0, s>>>(peers, rank, world, features, (const __half*)residual,
                                                                         (const __half*)norm_w, eps, unit_offset, (__half*)out_x,
                                                                         (__half*)out_normed, epoch_base, ew, status, limit);
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}
