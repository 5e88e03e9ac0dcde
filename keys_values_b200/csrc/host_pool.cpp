// Pinned host memory pool for the side-stream traffic (activation / KV checkpoints, streamed weights and
// their gradients, host-resident optimizer state).
//
// cudaHostAlloc takes milliseconds and synchronises with the device, so buffers that live for one step or one
// layer must not be allocated one by one. A pool takes ONE pinned slab and hands out 256-byte aligned ranges
// from a first-fit free list with coalescing on release; all bookkeeping is host-side and takes microseconds.
// Copies are plain cudaMemcpyAsync calls, one per range, on the stream the caller names.
//
// With pinned = 0 the slab comes from the C allocator (pageable): the same allocator logic for hosts without
// a GPU and for tests.
//
// Role of the pinned staging buffers that the reference allocates through PyTorch in
// keys_values/kvcache/gradient/checkpoints.py and keys_values/optimize/grad_accumulate.py:196-245.
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <map>
#include <mutex>

#include "kvb200.h"

namespace {

struct HostPool {
  uint8_t* base = nullptr;
  size_t bytes = 0;
  bool pinned = false;
  std::map<size_t, size_t> free_by_offset;  // offset -> length
  std::map<size_t, size_t> used;            // offset -> length
  size_t in_use = 0, peak = 0, n_alloc = 0, n_fail = 0;
  std::mutex mu;
};

constexpr size_t kAlign = 256;
inline size_t round_up(size_t n) { return (n + kAlign - 1) / kAlign * kAlign; }

}  // namespace

extern "C" int kvb_host_pool_create(void** pool_out, long long bytes, int pinned) {
  if (!pool_out || bytes <= 0) return KVB_ERR_ARG;
  HostPool* p = new HostPool();
  p->bytes = round_up((size_t)bytes);
  p->pinned = pinned != 0;
  if (p->pinned) {
    void* ptr = nullptr;
    if (cudaHostAlloc(&ptr, p->bytes, cudaHostAllocPortable) != cudaSuccess) {
      cudaGetLastError();
      delete p;
      return KVB_ERR_CUDA;
    }
    p->base = static_cast<uint8_t*>(ptr);
  } else {
    p->base = static_cast<uint8_t*>(aligned_alloc(4096, (p->bytes + 4095) / 4096 * 4096));
    if (!p->base) {
      delete p;
      return KVB_ERR_ARG;
    }
  }
  p->free_by_offset[0] = p->bytes;
  *pool_out = p;
  return KVB_OK;
}

extern "C" int kvb_host_pool_destroy(void* pool) {
  HostPool* p = static_cast<HostPool*>(pool);
  if (!p) return KVB_ERR_ARG;
  if (p->pinned) cudaFreeHost(p->base);
  else free(p->base);
  delete p;
  return KVB_OK;
}

// First fit. Returns KVB_ERR_TOO_LARGE when no free range is long enough (the caller falls back to its own allocation).
extern "C" int kvb_host_pool_alloc(void* pool, long long bytes, void** ptr_out) {
  HostPool* p = static_cast<HostPool*>(pool);
  if (!p || bytes <= 0 || !ptr_out) return KVB_ERR_ARG;
  const size_t need = round_up((size_t)bytes);
  std::lock_guard<std::mutex> lock(p->mu);
  for (auto it = p->free_by_offset.begin(); it != p->free_by_offset.end(); ++it) {
    if (it->second < need) continue;
    const size_t off = it->first, len = it->second;
    p->free_by_offset.erase(it);
    if (len > need) p->free_by_offset[off + need] = len - need;
    p->used[off] = need;
    p->in_use += need;
    if (p->in_use > p->peak) p->peak = p->in_use;
    ++p->n_alloc;
    *ptr_out = p->base + off;
    return KVB_OK;
  }
  ++p->n_fail;
  return KVB_ERR_TOO_LARGE;
}

extern "C" int kvb_host_pool_free(void* pool, void* ptr) {
  HostPool* p = static_cast<HostPool*>(pool);
  if (!p || !ptr) return KVB_ERR_ARG;
  std::lock_guard<std::mutex> lock(p->mu);
  const size_t off = static_cast<uint8_t*>(ptr) - p->base;
  auto it = p->used.find(off);
  if (it == p->used.end()) return KVB_ERR_ARG;
  size_t start = off, len = it->second;
  p->in_use -= len;
  p->used.erase(it);
  // coalesce with the free neighbours
  auto next = p->free_by_offset.lower_bound(start);
  if (next != p->free_by_offset.end() && next->first == start + len) {
    len += next->second;
    next = p->free_by_offset.erase(next);
  }
  if (next != p->free_by_offset.begin()) {
    auto prev = std::prev(next);
    if (prev->first + prev->second == start) {
      start = prev->first;
      len += prev->second;
      p->free_by_offset.erase(prev);
    }
  }
  p->free_by_offset[start] = len;
  return KVB_OK;
}

// out[0..5] = capacity, in use, peak in use, largest free range, successful allocations, failed allocations
extern "C" int kvb_host_pool_stats(void* pool, long long* out) {
  HostPool* p = static_cast<HostPool*>(pool);
  if (!p || !out) return KVB_ERR_ARG;
  std::lock_guard<std::mutex> lock(p->mu);
  size_t largest = 0;
  for (auto& kv : p->free_by_offset)
    if (kv.second > largest) largest = kv.second;
  out[0] = (long long)p->bytes;
  out[1] = (long long)p->in_use;
  out[2] = (long long)p->peak;
  out[3] = (long long)largest;
  out[4] = (long long)p->n_alloc;
  out[5] = (long long)p->n_fail;
  return KVB_OK;
}

// One asynchronous copy; kind: 1 host -> device, 2 device -> host.
extern "C" int kvb_copy_async(void* dst, const void* src, long long bytes, int kind, void* stream) {
  if (!dst || !src || bytes <= 0 || (kind != 1 && kind != 2)) return KVB_ERR_ARG;
  const cudaMemcpyKind k = kind == 1 ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost;
  return cudaMemcpyAsync(dst, src, (size_t)bytes, k, (cudaStream_t)stream) == cudaSuccess ? KVB_OK : KVB_ERR_CUDA;
}
