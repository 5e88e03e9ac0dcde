// Entry point of libkvb200 that allocates nothing. It has no counterpart in the reference
// library: it exists for callers of THIS library that cannot allocate device memory at the
// time of the call (a frozen allocator, a serving loop with a fixed memory plan, a host
// runtime that links only the C symbols).
//
// kvb_decode_attn_noalloc computes exactly what kvb_decode_attn (kvb200.h) computes: the
// attention of one new query token per sequence over a bf16 / int8 / int4 KV cache, plus the
// per-slot summed attention weights. The caller passes inputs and outputs only; the
// workspace is a fixed array of KVB_DECODE_STATIC_SCRATCH_BYTES = 8 MiB inside the library's
// device image (held by every GPU that loads the library until the process exits).
//
//   * Limit: kvb_decode_scratch_bytes(B, H, L) must not exceed
//     kvb_decode_attn_noalloc_max_bytes() (8 MiB; e.g. B=1, H=32, L=32768 needs 4.6 MiB).
//     Larger problems are refused with KVB_ERR_TOO_LARGE and nothing is launched.
//   * The first call on a device looks up the device address of the workspace
//     (cudaGetSymbolAddress, with that device current). Make that first call before any
//     stream capture begins on the device.
//   * It calls no cudaMalloc, cudaFree or allocating library routine.
//   * All calls on a device share the one workspace, which keeps the contents of the last
//     call. Nothing needs to be zeroed between calls (every word that is read is written
//     earlier in the same call), but two calls that overlap on the GPU, e.g. on two
//     streams, race on it: serialise them.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

long long kvb_decode_attn_noalloc_max_bytes(void);
int kvb_decode_attn_noalloc(const void* q, const void* kq, const void* vq, const float* ks, const int32_t* kz, const float* vs,
                            const int32_t* vz, const void* k_new, const void* v_new, const int32_t* new_slot, void* out,
                            float* weights, int B, int H, int G, int L, int C, int bits, float scale, void* stream);

#ifdef __cplusplus
}
#endif
