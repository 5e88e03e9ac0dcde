// Pieces shared by the single-CTA and the CTA-pair GEMM kernels: the parameter block of the fused collectives and the
// role of the CTAs that copy the peers' shards for the all-gather.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace kvb {

// Optional fusion of the GEMM with a collective over NVLink peer memory.
//   * reduce-scatter epilogue (rs_world > 1): the output rows are partitioned over ranks
//     (rows_per_rank each, a multiple of 128). A finished tile is not written to C but
//     stored straight into the *owner rank's* receive buffer, slot [this rank][row][col],
//     with plain peer stores; then the tile is counted on the owner's flag word. Tiles for
//     remote owners are produced first, the rank's own rows last, so the transfers hide
//     behind the remaining MMAs. The owner sums the partials with kvb_reduce_partials.
//   * gated A operand (a_flags != nullptr): rows of A arrive chunk by chunk (an all-gather
//     that copies remote shards into LOCAL staging memory); the TMA producer waits for the
//     chunk's flag before it loads a tile of that chunk. The copy runs in the first
//     `ag_copy_ctas` CTAs of the same grid, which pull the peers' shards with plain loads.
// No TMA load ever targets peer memory and no load uses cluster multicast.
struct GemmExtra {
  // reduce-scatter epilogue
  int rs_world, rs_rank, rows_per_rank;
  uint32_t rs_tile_inc;                  // value added to the owner's flag per finished tile (1)
  __nv_bfloat16* rs_dst[16];             // receive buffer of every rank: [world][rows_per_rank][N]
  uint32_t* rs_flag[16];                 // flag words of every rank: [world] counters, indexed by source rank
  // gated A / all-gather
  const uint32_t* a_flags;               // [world] local counters: chunk q is complete when a_flags[q] >= a_target
  uint32_t a_target;
  int rows_per_chunk;                    // rows of A per source rank
  int ag_copy_ctas;                      // CTAs [0, ag_copy_ctas) copy, the rest compute
  int ag_world, ag_rank;
  const __nv_bfloat16* ag_src[16];       // shard of every rank (peer pointers), [rows_per_chunk][K] with pitch ag_ld
  __nv_bfloat16* ag_stage;               // local staging [world*rows_per_chunk][K] with pitch ag_ld (also operand A)
  uint32_t* ag_flags_w;                  // same memory as a_flags, writable
  long long ag_ld;
  uint32_t* ag_ready[16];                // "shard is ready" word of every rank (each rank publishes its own)
  uint32_t ag_epoch;                     // value of the ready words for this call
  uint32_t* ag_pulled[16];               // "how many copy CTAs have pulled my shard" counter of every rank
  uint32_t ag_pulled_target;             // own counter value at which this rank's shard may be overwritten
  long long wait_limit;
};

__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// The all-gather copy role of CTA blockIdx.x < ex.ag_copy_ctas: pulls the peers' shards into local staging, chunk by
// chunk, and counts every chunk on the local flag word. `ag_smem_raw`: the dynamic shared memory of the kernel (at
// least 12 x 16 KB + 1.3 KB).
__device__ __forceinline__ void gemm_ag_copy_role(const GemmExtra& ex, int K, int* status, uint8_t* ag_smem_raw) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  const long long vec_per_row = (long long)K / 8;
  // everything issued earlier on this stream has completed, so this rank's shard is final: publish it
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    st_release_sys_u32(ex.ag_ready[ex.ag_rank], ex.ag_epoch);
  }
  for (int qi = 1; qi < ex.ag_world; ++qi) {
    const int src = (ex.ag_rank + qi) % ex.ag_world;
    // the peer publishes "shard ready" by writing the epoch into ITS OWN ready word
    if (threadIdx.x == 0) {
      long long t0 = clock64();
      while ((int32_t)(ld_acquire_sys_u32(ex.ag_ready[src]) - ex.ag_epoch) < 0) {
        if (clock64() - t0 > ex.wait_limit) {
          if (status) atomicCAS(status, 0, STATUS_TIMEOUT_PEER_FLAG);
          ok_s = 0;
          break;
        }
      }
    }
    __syncthreads();
    if (!ok_s) return;
    const long long total = (long long)ex.rows_per_chunk * vec_per_row;
    const __nv_bfloat16* sp = ex.ag_src[src];
    __nv_bfloat16* dp = ex.ag_stage + (long long)src * ex.rows_per_chunk * ex.ag_ld;
    if (ex.ag_ld == (long long)K) {
      // Contiguous shard: the TMA engine moves it, peer memory -> shared memory -> local staging, in
      // pieces of AG_PIECE bytes through a ring of AG_RING pieces, driven by one thread. A CTA keeps
      // AG_RING x AG_PIECE bytes in flight, so a few copy CTAs saturate the link and the rest of the
      // SMs stay with the product.
      constexpr uint32_t AG_PIECE = 16384;
      constexpr int AG_RING = 12;
      extern __shared__ uint8_t ag_smem_raw[];
      uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(ag_smem_raw) + 1023) & ~uintptr_t(1023));
      uint64_t* rbar = reinterpret_cast<uint64_t*>(ring + (size_t)AG_RING * AG_PIECE);
      __shared__ int ag_abort;
      if (threadIdx.x == 0) {
        const long long bytes = total * 16;
        const long long n_piece = (bytes + AG_PIECE - 1) / AG_PIECE;
        const uint8_t* gs = reinterpret_cast<const uint8_t*>(sp);
        uint8_t* gd = reinterpret_cast<uint8_t*>(dp);
        if (qi == 1) {
          ag_abort = 0;
          for (int r = 0; r < AG_RING; ++r) mbar_init(&rbar[r], 1);
          mbar_fence_init();
        }
        // pieces blockIdx.x, blockIdx.x + n_copy, ... of this shard
        const long long first = blockIdx.x, step = ex.ag_copy_ctas;
        const long long mine = first < n_piece ? (n_piece - first + step - 1) / step : 0;
        auto piece_bytes = [&](long long k) -> uint32_t {
          const long long off = (first + k * step) * AG_PIECE;
          return (uint32_t)(bytes - off < AG_PIECE ? bytes - off : AG_PIECE);
        };
        auto issue_load = [&](long long k, uint32_t use) {  // `use`: how often this ring slot has been used before
          const int sl = (int)(k % AG_RING);
          (void)use;
          mbar_expect_tx(&rbar[sl], piece_bytes(k));
          bulk_load(ring + (size_t)sl * AG_PIECE, gs + (first + k * step) * AG_PIECE, piece_bytes(k), &rbar[sl]);
        };
        // ring slot sl has been used (qi - 1) * uses_per_shard + ... times: track phases explicitly
        static_assert(AG_RING <= 32, "phase bits");
        uint32_t& phases = *reinterpret_cast<uint32_t*>(&rbar[AG_RING]);
        if (qi == 1) phases = 0;
        for (long long k = 0; k < mine && k < AG_RING; ++k) issue_load(k, 0);
        for (long long k = 0; k < mine && ok_s; ++k) {
          const int sl = (int)(k % AG_RING);
          if (!mbar_wait_bounded(&rbar[sl], (phases >> sl) & 1u, &ag_abort, status, STATUS_TIMEOUT_FULL, ex.wait_limit)) {
            ok_s = 0;
            break;
          }
          phases ^= 1u << sl;
          bulk_store(gd + (first + k * step) * AG_PIECE, ring + (size_t)sl * AG_PIECE, piece_bytes(k));
          bulk_commit();
          if (k + AG_RING < mine) {
            bulk_wait_read_all();  // the slot's store has read it: the slot can take the next piece
            issue_load(k + AG_RING, 0);
          }
        }
        bulk_wait_all();  // the staged pieces are in local memory
      }
      __threadfence();
      __syncthreads();
      if (!ok_s) return;
      if (threadIdx.x == 0) {
        red_release_gpu_add(ex.ag_flags_w + src, 1u);
        red_release_sys_add(ex.ag_pulled[src], 1u);
      }
      continue;
    }
    // remote loads take microseconds: keep 16 of them in flight per thread
    constexpr int CU = 16;
    const long long cstride = (long long)ex.ag_copy_ctas * blockDim.x;
    const bool contig = ex.ag_ld == (long long)K;  // rows back to back: element offset = 8 i
    const unsigned vpr = (unsigned)vec_per_row;
    auto elem_off = [&](long long i) -> long long {
      if (contig) return i * 8;
      const unsigned r = (unsigned)i / vpr, c = (unsigned)i % vpr;  // a shard has far fewer than 2^32 vectors
      return (long long)r * ex.ag_ld + (long long)c * 8;
    };
    for (long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += cstride * CU) {
      uint4 v[CU];
#pragma unroll
      for (int k = 0; k < CU; ++k) {
        const long long i = i0 + k * cstride;
        if (i < total) v[k] = __ldcg(reinterpret_cast<const uint4*>(sp + elem_off(i)));
      }
#pragma unroll
      for (int k = 0; k < CU; ++k) {
        const long long i = i0 + k * cstride;
        if (i < total) *reinterpret_cast<uint4*>(dp + elem_off(i)) = v[k];
      }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      red_release_gpu_add(ex.ag_flags_w + src, 1u);        // local: chunk `src` is (partly) staged
      red_release_sys_add(ex.ag_pulled[src], 1u);          // remote: tell `src` that this CTA is done with its shard
    }
  }
  // do not let this rank overwrite its shard before every peer has pulled it
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys_u32(ex.ag_pulled[ex.ag_rank]) - ex.ag_pulled_target) < 0) {
      if (clock64() - t0 > ex.wait_limit) {
        if (status) atomicCAS(status, 0, STATUS_TIMEOUT_PEER_FLAG);
        break;
      }
    }
  }
}

// defined in gemm2_sm100.cu: the product on CTA pairs (cta_group::2), with the same fused collectives
int launch_gemm_pair(const void* A, const void* B, const void* A2, const void* B2, void* C, const void* residual, int M, int N,
                     int K, int K2, long long lda, long long ldb, long long lda2, long long ldb2, long long ldc, int* status,
                     int max_pairs, cudaStream_t stream, const GemmExtra* extra);

}  // namespace kvb
