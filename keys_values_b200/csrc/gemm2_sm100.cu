// Persistent bf16 GEMM for sm_100a on CTA pairs:  C[M,N] = A[M,K] · B[N,K]^T (+ A2[M,K2] · B2[N,K2]^T) (+ residual)
//
// A cluster of two CTAs (two SMs) works on one 256 x 256 tile with tcgen05.mma.cta_group::2 (M = 256, N = 256,
// K = 16 per instruction):
//   * CTA r of the pair loads rows [m0 + 128 r, +128) of A and rows [n0 + 128 r, +128) of B (its half of the N
//     extent) into its own shared memory, by plain TMA loads (no multicast); the tensor core of each SM reads its own A
//     rows and both halves of B. Per SM that is 8 KB of operand reads per instruction and 32 KB of TMA writes per
//     k-block of 64, half of what a 128 x 256 tile per single CTA needs: the single-CTA kernel is bound by the
//     shared-memory port at about 0.65 of the tensor pipe.
//   * The first CTA of the pair (the leader) issues every MMA. The TMA loads of both CTAs complete on the leader's
//     "full" barrier of the stage (the leader arms it with the bytes of both). When the MMAs of a stage are done the
//     leader's tcgen05.commit arrives on the "empty" barrier of the stage in both CTAs, and when a tile is done on the
//     "accumulator full" barrier of both.
//   * Each CTA holds its 128 rows x 256 columns of the fp32 accumulator in its own TMEM, double-buffered (2 x 256
//     columns), so the epilogue of tile i (tcgen05.ld -> bf16 -> shared memory -> global, 4 rows x 128 contiguous
//     bytes per store instruction) overlaps the main loop of tile i + 1. The epilogue warps of both CTAs hand the
//     buffer back on the leader's "accumulator empty" barrier (the follower's with a remote arrive).
//   * warp roles per CTA: warp 0 = TMA producer, warp 1 = TMEM owner (and MMA issuer in the leader), warps 2..5 =
//     epilogue.
// Every wait is bounded; a CTA that gives up raises the status word and still takes part in the cluster barrier at the
// end, so that neither CTA's shared memory is released while the other may still signal it.
//
// Replaces the cuBLAS calls behind nn.Linear in the reference (keys_values/model.py:596-610, lora_utils.py:159-172).
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "gemm_extra.cuh"
#include "kvb200.h"

namespace kvb {

int make_tmap_2d_bf16(CUtensorMap* tm, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols);

constexpr int G2_BM = 128;      // rows of A per CTA (256 per pair)
constexpr int G2_BNH = 128;     // rows of B per CTA (N = 256 per pair)
constexpr int G2_BN = 256;
constexpr int G2_BK = 64;
constexpr int G2_STAGES = 6;
constexpr int G2_THREADS = 192;

struct G2Smem {
  static constexpr int A_BYTES = G2_BM * G2_BK * 2;
  static constexpr int B_BYTES = G2_BNH * G2_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;          // per CTA
  static constexpr int EPI_OFFSET = G2_STAGES * STAGE_BYTES;     // per epilogue warp: 32 rows x 128 B staging
  static constexpr int EPI_BYTES = 4 * 32 * 128;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;          // barriers + alignment slack
};
static_assert(G2Smem::TOTAL <= 232448, "shared memory of the pair GEMM exceeds the limit of a CTA");

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `local` (a shared::cta address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_u32(uint32_t local, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local), "r"(rank));
  return a;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on a barrier that may live in the other CTA of the cluster (shared::cluster address)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load of a CTA of a pair: the destination is this CTA's shared memory, the barrier (shared::cluster address) may be
// the other CTA's
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(smem_dst)),
      "l"(tmap), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem of both CTAs] (+)= A[256 x 16: 128 rows per CTA] · B[256 x 16: 128 rows per CTA]^T; issued by ONE thread of the leader
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive, in both CTAs of the pair, on the barrier at this shared-memory offset once all MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                  __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ residual, int M, int N, int K, int K2,
                  long long ldc, int* status, const GemmExtra ex, const int diag) {
  using S = G2Smem;
  extern __shared__ uint8_t smem_raw[];
  // ---- all-gather copy CTAs (whole pairs: copy_span CTAs, the last one idle when ag_copy_ctas is odd). They take no
  // part in any cluster barrier, MMA or TMEM allocation.
  const int copy_span = (ex.ag_copy_ctas + 1) & ~1;
  if ((int)blockIdx.x < copy_span) {
    if ((int)blockIdx.x < ex.ag_copy_ctas) gemm_ag_copy_role(ex, K, status, smem_raw);
    return;
  }
  // the same offsets in both CTAs (the window starts at the same shared-memory address in every CTA of the kernel): the
  // leader's descriptors address both
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + G2_STAGES;
  uint64_t* tmem_full = empty_bar + G2_STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: leader
  const int pair = ((int)blockIdx.x - copy_span) >> 1;
  const int n_pairs = ((int)gridDim.x - copy_span) >> 1;
  const int num_m = (M + 2 * G2_BM - 1) / (2 * G2_BM);
  const int num_n = (N + G2_BN - 1) / G2_BN;
  const int num_tiles = num_m * num_n;
  const int kb1 = (K + G2_BK - 1) / G2_BK;
  const int kb2 = (K2 + G2_BK - 1) / G2_BK;
  const int num_kb = kb1 + kb2;
  const bool aligned_ok = (smem_u32(smem) & 1023u) == 0;  // swizzled tiles need a 1024-byte aligned window
  // tile -> (first row of the pair's 256 rows, first column). With a fused collective the order is row-block major and
  // the row blocks are rotated so that the blocks this rank already holds (all-gather) come first, or the rows this
  // rank owns (reduce-scatter) last.
  const bool comm = ex.a_flags != nullptr || ex.rs_world > 1;
  int m_rot = 0;
  if (ex.a_flags) m_rot = (ex.ag_rank * ex.rows_per_chunk) / (2 * G2_BM);
  if (ex.rs_world > 1) m_rot = (((ex.rs_rank + 1) * ex.rows_per_rank + 2 * G2_BM - 1) / (2 * G2_BM)) % num_m;
  auto tile_coords = [&](int tile, int& m0, int& n0) {
    if (comm) {
      m0 = ((tile / num_n + m_rot) % num_m) * (2 * G2_BM);
      n0 = (tile % num_n) * G2_BN;
    } else {
      m0 = (tile % num_m) * (2 * G2_BM);
      n0 = (tile / num_m) * G2_BN;
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < G2_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);    // the leader's producer arms it with the bytes of both CTAs
      mbar_init(&empty_bar[s], 1);   // the leader's commit, in both CTAs
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);   // the leader's commit, in both CTAs
      mbar_init(&tmem_empty[a], 8);  // one arrive per epilogue warp of both CTAs (used in the leader)
    }
    *abort_flag = aligned_ok ? 0 : 1;
    if (!aligned_ok && status) atomicCAS(status, 0, STATUS_TIMEOUT_MISC);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_base_slot, 2 * G2_BN);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // barriers of both CTAs are initialised before either signals the other
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0 && !*abort_flag) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        int m0, n0;
        tile_coords(tile, m0, n0);
        m0 += (int)rank * G2_BM;
        n0 += (int)rank * G2_BNH;
        if (ex.a_flags && m0 < M) {
          // rows of A come from an all-gather: wait until the chunk that holds this CTA's rows is local
          const int chunk = m0 / ex.rows_per_chunk;
          if (chunk != ex.ag_rank) {
            long long t0 = clock64();
            while ((int32_t)(ld_acquire_gpu_u32(ex.a_flags + chunk) - ex.a_target) < 0) {
              if (*abort_flag || clock64() - t0 > ex.wait_limit) {
                if (status) atomicCAS(status, 0, STATUS_TIMEOUT_PEER_FLAG);
                *abort_flag = 1;
                ok = false;
                break;
              }
            }
            if (!ok) break;
            asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy writes -> visible to the TMA reads
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if ((diag == 1 || diag >= 3) && (tile != pair || kb >= G2_STAGES)) continue;  // diagnostics: the ring is filled once, the MMAs re-read it
          // diag 2: loads keep flowing at their own pace (a stage is refilled when its previous load has landed, on this
          // CTA's own barrier), the MMAs never wait
          if (!mbar_wait_bounded(diag == 2 ? &full_bar[stage] : &empty_bar[stage], phase ^ 1, abort_flag, status, STATUS_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          if (diag == 2) mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          else if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * S::STAGE_BYTES);
          const uint32_t bar = mapa_u32(smem_u32(&full_bar[stage]), diag == 2 ? rank : 0);  // the leader's barrier
          if (kb < kb1) {
            tma_load_2d_pair(sa, &tmA, bar, kb * G2_BK, m0);
            tma_load_2d_pair(sb, &tmB, bar, kb * G2_BK, n0);
          } else {
            tma_load_2d_pair(sa, &tmA2, bar, (kb - kb1) * G2_BK, m0);
            tma_load_2d_pair(sb, &tmB2, bar, (kb - kb1) * G2_BK, n0);
          }
          if (++stage == G2_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // unwinding: give the copies that are still in flight a bounded time to land
        long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && rank == 0 && !*abort_flag) {
      // diag 3 / 4 (as diag 1, no operand feed): MMAs of N = 64 / N = 128 instead of 256, to time small instructions
      // diag 5: N = 64 MMAs that alternate between two accumulators (two independent chains of accumulation)
      const uint32_t idesc = (diag == 3 || diag == 5) ? make_idesc_bf16(2 * G2_BM, 64, 0, 0)
                                       : (diag == 4 ? make_idesc_bf16(2 * G2_BM, 128, 0, 0) : make_idesc_bf16(2 * G2_BM, G2_BN, 0, 0));
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        if (!mbar_wait_bounded(&tmem_empty[acc], acc_phase ^ 1, abort_flag, status, STATUS_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * G2_BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          const bool fed = !diag || ((diag == 1 || diag >= 3) && tile == pair && kb < G2_STAGES);
          if (fed && !mbar_wait_bounded(&full_bar[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
          const uint64_t da = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < G2_BK / 16; ++k) {
            // advance 16 elements (32 B) along K inside the 128B swizzle row: +2 in 16 B units
            umma_f16_ss_pair(diag == 5 ? d_tmem + (uint32_t)((k & 1) * 64) : d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc,
                             (kb | k) != 0 ? 1u : 0u);
          }
          if (!diag) umma_commit_pair(&empty_bar[stage]);
          if (++stage == G2_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit_pair(&tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // --------------------------------------------------------------- epilogue (both CTAs)
    const int quarter = warp & 3;  // TMEM sub-partition of this warp
    const int row_in_tile = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t empty_remote = mapa_u32(smem_u32(&tmem_empty[0]), 0);  // the leader's "accumulator empty" barriers
    for (int tile = pair; tile < num_tiles; tile += n_pairs) {
      int m0, n0;
      tile_coords(tile, m0, n0);
      m0 += (int)rank * G2_BM;
      if (!mbar_wait_bounded(&tmem_full[acc], acc_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int m = m0 + row_in_tile;
      // reduce-scatter epilogue: this CTA's 128 rows go to the receive buffer of the rank that owns them
      __nv_bfloat16* out_base = C;
      long long out_row = m;
      int dest = -1;
      if (ex.rs_world > 1 && m0 < M) {
        dest = m0 / ex.rows_per_rank;
        out_base = ex.rs_dst[dest];
        out_row = (long long)ex.rs_rank * ex.rows_per_rank + (m - dest * ex.rows_per_rank);
      }
      const long long out_row0 = out_row - lane;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * G2_BN);
      // 64 columns at a time: thread = row converts its 128 bytes, the warp exchanges them through shared memory
      // (16-byte units XOR-swizzled by row, conflict-free both ways) and stores 4 rows x 128 contiguous bytes per
      // instruction.
      uint8_t* stg = smem + S::EPI_OFFSET + quarter * (32 * 128);
      const int m_warp0 = m0 + quarter * 32;  // first row of this warp
#pragma unroll 1
      for (int c0 = 0; c0 < G2_BN; c0 += 64) {
        const int n = n0 + c0;
        if (n >= N) break;  // warp-uniform
        uint32_t r[64];
        tmem_ld_32x32b_x32(taddr + (uint32_t)c0, r);
        tmem_ld_32x32b_x32(taddr + (uint32_t)(c0 + 32), r + 32);
        tmem_ld_wait();
        if (n + 64 <= N) {
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[8 * v]), __uint_as_float(r[8 * v + 1]));
            o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
            o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
            o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
            *reinterpret_cast<uint4*>(stg + lane * 128 + ((v ^ (lane & 7)) << 4)) = o;
          }
          __syncwarp();
          const int u = lane & 7;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int rr = 4 * j + (lane >> 3);  // row of the warp's 32
            uint4 o = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((u ^ (rr & 7)) << 4));
            if (m_warp0 + rr < M) {
              if (residual) {
                const uint4 rv = *reinterpret_cast<const uint4*>(residual + (long long)(m_warp0 + rr) * ldc + n + u * 8);
                const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
                __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 a = __bfloat1622float2(op[i]), t = __bfloat1622float2(rp[i]);
                  op[i] = __floats2bfloat162_rn(a.x + t.x, a.y + t.y);
                }
              }
              *reinterpret_cast<uint4*>(out_base + (out_row0 + rr) * ldc + n + u * 8) = o;
            }
          }
          __syncwarp();
        } else if (m < M) {
          // ragged right edge: element by element
          __nv_bfloat16* dst = out_base + out_row * ldc + n;
          const __nv_bfloat16* res = residual ? residual + (long long)m * ldc + n : nullptr;
          for (int i = 0; i < 64 && n + i < N; ++i) {
            float f = __uint_as_float(r[i]);
            if (res) f += __bfloat162float(res[i]);
            dst[i] = __float2bfloat16_rn(f);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(empty_remote + (uint32_t)(acc * 8));
      if (dest >= 0) {
        // make this warp's peer stores visible system-wide, then count a quarter of a 128 x 256 block at the owner
        __threadfence_system();
        __syncwarp();
        if (lane == 0) red_release_sys_add(ex.rs_flag[dest] + ex.rs_rank, ex.rs_tile_inc);
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // nothing of either CTA is released while the other one may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * G2_BN);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// The wide variant: one 256 x 512 tile per CTA pair. The operands of a 256 x 256 tile cross L2 -> shared memory at 64
// bytes per clock and SM at full tensor rate, which is what the L2 delivers to 148 SMs at once (measured: the loads of
// the 256 x 256 kernel alone, running at their own pace, take as long as the whole kernel). A 256 x 512 tile re-uses the
// A rows for two B tiles: 25 % fewer operand bytes per flop. Both 256-column accumulators of an SM belong to the same
// tile (acc 0: columns [n0, n0 + 256), acc 1: [n0 + 256, n0 + 512)), so there is no second buffer: eight epilogue warps
// (two per TMEM lane quarter, 128 columns each) drain acc 0 and then acc 1 while the next tile's first MMAs wait for the
// accumulator they need; the producer keeps prefetching.
// ------------------------------------------------------------------------------------------------------------------
constexpr int G2W_STAGES = 4;
constexpr int G2W_THREADS = 64 + 256;
constexpr int G2W_BN = 512;

struct G2WSmem {
  static constexpr int A_BYTES = G2_BM * G2_BK * 2;
  static constexpr int B_BYTES = G2_BNH * G2_BK * 2;             // one half (128 rows) of one 256-row B tile
  static constexpr int STAGE_BYTES = A_BYTES + 2 * B_BYTES;      // per CTA: A | B of acc 0 | B of acc 1
  static constexpr int EPI_OFFSET = G2W_STAGES * STAGE_BYTES;    // per epilogue warp: 32 rows x 128 B staging
  static constexpr int EPI_BYTES = 8 * 32 * 128;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
};
static_assert(G2WSmem::TOTAL + 64 <= 232448, "shared memory of the wide pair GEMM exceeds the limit of a CTA");

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2W_THREADS, 1)
gemm2w_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                   __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ residual, int M, int N, int K, int K2,
                   long long ldc, int* status, const GemmExtra ex) {
  using S = G2WSmem;
  extern __shared__ uint8_t smem_raw[];
  const int copy_span = (ex.ag_copy_ctas + 1) & ~1;
  if ((int)blockIdx.x < copy_span) {
    if ((int)blockIdx.x < ex.ag_copy_ctas) gemm_ag_copy_role(ex, K, status, smem_raw);
    return;
  }
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + G2W_STAGES;
  uint64_t* tmem_full = empty_bar + G2W_STAGES;   // [2]: accumulator h of the current tile is complete
  uint64_t* tmem_empty = tmem_full + 2;           // [2]: accumulator h has been drained (used in the leader)
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0: leader
  const int pair = ((int)blockIdx.x - copy_span) >> 1;
  const int n_pairs = ((int)gridDim.x - copy_span) >> 1;
  const int num_m = (M + 2 * G2_BM - 1) / (2 * G2_BM);
  const int num_n = (N + G2W_BN - 1) / G2W_BN;
  const int num_tiles = num_m * num_n;
  const int kb1 = (K + G2_BK - 1) / G2_BK;
  const int kb2 = (K2 + G2_BK - 1) / G2_BK;
  const int num_kb = kb1 + kb2;
  const bool aligned_ok = (smem_u32(smem) & 1023u) == 0;
  const bool comm = ex.a_flags != nullptr || ex.rs_world > 1;
  int m_rot = 0;
  if (ex.a_flags) m_rot = (ex.ag_rank * ex.rows_per_chunk) / (2 * G2_BM);
  if (ex.rs_world > 1) m_rot = (((ex.rs_rank + 1) * ex.rows_per_rank + 2 * G2_BM - 1) / (2 * G2_BM)) % num_m;
  auto tile_coords = [&](int tile, int& m0, int& n0) {
    if (comm) {
      m0 = ((tile / num_n + m_rot) % num_m) * (2 * G2_BM);
      n0 = (tile % num_n) * G2W_BN;
    } else {
      m0 = (tile % num_m) * (2 * G2_BM);
      n0 = (tile / num_m) * G2W_BN;
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < G2W_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 16);  // one arrive per epilogue warp of both CTAs
    }
    *abort_flag = aligned_ok ? 0 : 1;
    if (!aligned_ok && status) atomicCAS(status, 0, STATUS_TIMEOUT_MISC);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_base_slot, 512);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0 && !*abort_flag) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        int m0, n0;
        tile_coords(tile, m0, n0);
        m0 += (int)rank * G2_BM;
        n0 += (int)rank * G2_BNH;  // this CTA's half of the B tile of acc 0; acc 1: 256 rows further
        if (ex.a_flags && m0 < M) {
          const int chunk = m0 / ex.rows_per_chunk;
          if (chunk != ex.ag_rank) {
            long long t0 = clock64();
            while ((int32_t)(ld_acquire_gpu_u32(ex.a_flags + chunk) - ex.a_target) < 0) {
              if (*abort_flag || clock64() - t0 > ex.wait_limit) {
                if (status) atomicCAS(status, 0, STATUS_TIMEOUT_PEER_FLAG);
                *abort_flag = 1;
                ok = false;
                break;
              }
            }
            if (!ok) break;
            asm volatile("fence.proxy.async;" ::: "memory");
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, status, STATUS_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb0 = sa + S::A_BYTES;
          uint8_t* sb1 = sb0 + S::B_BYTES;
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * S::STAGE_BYTES);
          const uint32_t bar = mapa_u32(smem_u32(&full_bar[stage]), 0);  // the leader's barrier
          const CUtensorMap* ta = kb < kb1 ? &tmA : &tmA2;
          const CUtensorMap* tb = kb < kb1 ? &tmB : &tmB2;
          const int k0 = (kb < kb1 ? kb : kb - kb1) * G2_BK;
          tma_load_2d_pair(sa, ta, bar, k0, m0);
          tma_load_2d_pair(sb0, tb, bar, k0, n0);
          tma_load_2d_pair(sb1, tb, bar, k0, n0 + G2_BN);  // rows beyond N are filled with zeros
          if (++stage == G2W_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (leader only)
    if (lane == 0 && rank == 0 && !*abort_flag) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * G2_BM, G2_BN, 0, 0);
      int stage = 0;
      uint32_t phase = 0, tile_phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint64_t da = make_smem_desc_sw128(sa, 16, 1024);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (kb == 0 && !mbar_wait_bounded(&tmem_empty[h], tile_phase ^ 1, abort_flag, status, STATUS_TIMEOUT_TMEM_EMPTY)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const uint64_t db = make_smem_desc_sw128(sa + S::A_BYTES + h * S::B_BYTES, 16, 1024);
            const uint32_t d_tmem = tmem_base + (uint32_t)(h * G2_BN);
#pragma unroll
            for (int k = 0; k < G2_BK / 16; ++k)
              umma_f16_ss_pair(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
            if (kb == num_kb - 1) umma_commit_pair(&tmem_full[h]);
          }
          if (!ok) break;
          umma_commit_pair(&empty_bar[stage]);
          if (++stage == G2W_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        tile_phase ^= 1;
      }
    }
  } else {
    // --------------------------------------------------------------- epilogue (both CTAs, 8 warps)
    const int e = warp - 2;
    const int quarter = warp & 3;   // TMEM sub-partition of this warp
    const int colhalf = e >> 2;     // which 128 of the 256 columns of an accumulator
    const int row_in_tile = quarter * 32 + lane;
    uint32_t tile_phase = 0;
    const uint32_t empty_remote = mapa_u32(smem_u32(&tmem_empty[0]), 0);
    uint8_t* stg = smem + S::EPI_OFFSET + e * (32 * 128);
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += n_pairs) {
      int m0, n0;
      tile_coords(tile, m0, n0);
      m0 += (int)rank * G2_BM;
      const int m = m0 + row_in_tile;
      __nv_bfloat16* out_base = C;
      long long out_row = m;
      int dest = -1;
      if (ex.rs_world > 1 && m0 < M) {
        dest = m0 / ex.rows_per_rank;
        out_base = ex.rs_dst[dest];
        out_row = (long long)ex.rs_rank * ex.rows_per_rank + (m - dest * ex.rows_per_rank);
      }
      const long long out_row0 = out_row - lane;
      const int m_warp0 = m0 + quarter * 32;
      for (int h = 0; h < 2; ++h) {
        if (!mbar_wait_bounded(&tmem_full[h], tile_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(h * G2_BN + colhalf * 128);
        const int nh = n0 + h * G2_BN + colhalf * 128;  // first column of this warp's 128
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 64) {
          const int n = nh + c0;
          if (n >= N) break;  // warp-uniform
          uint32_t r[64];
          tmem_ld_32x32b_x32(taddr + (uint32_t)c0, r);
          tmem_ld_32x32b_x32(taddr + (uint32_t)(c0 + 32), r + 32);
          tmem_ld_wait();
          if (n + 64 <= N) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(r[8 * v]), __uint_as_float(r[8 * v + 1]));
              o.y = pack_bf16x2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              o.z = pack_bf16x2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              o.w = pack_bf16x2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              *reinterpret_cast<uint4*>(stg + lane * 128 + ((v ^ (lane & 7)) << 4)) = o;
            }
            __syncwarp();
            const int u = lane & 7;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int rr = 4 * j + (lane >> 3);
              uint4 o = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((u ^ (rr & 7)) << 4));
              if (m_warp0 + rr < M) {
                if (residual) {
                  const uint4 rv = *reinterpret_cast<const uint4*>(residual + (long long)(m_warp0 + rr) * ldc + n + u * 8);
                  const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
                  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    const float2 a = __bfloat1622float2(op[i]), t = __bfloat1622float2(rp[i]);
                    op[i] = __floats2bfloat162_rn(a.x + t.x, a.y + t.y);
                  }
                }
                *reinterpret_cast<uint4*>(out_base + (out_row0 + rr) * ldc + n + u * 8) = o;
              }
            }
            __syncwarp();
          } else if (m < M) {
            __nv_bfloat16* dst = out_base + out_row * ldc + n;
            const __nv_bfloat16* res = residual ? residual + (long long)m * ldc + n : nullptr;
            for (int i = 0; i < 64 && n + i < N; ++i) {
              float f = __uint_as_float(r[i]);
              if (res) f += __bfloat162float(res[i]);
              dst[i] = __float2bfloat16_rn(f);
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(empty_remote + (uint32_t)(h * 8));
        if (dest >= 0 && n0 + h * G2_BN < N) {
          // Both warps of this lane quarter have stored their halves of the 128 x 256 block: make the peer stores
          // visible system-wide, then one of them counts a quarter of the block at the owner (the same count per
          // 128 x 256 block as in the other kernels).
          __threadfence_system();
          asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
          if (colhalf == 0 && lane == 0) red_release_sys_add(ex.rs_flag[dest] + ex.rs_rank, ex.rs_tile_inc);
        }
      }
      tile_phase ^= 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

static int g2_max_pairs() {
  static int n[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (!n[dev]) {
    cudaFuncSetAttribute(gemm2_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G2Smem::TOTAL);
    cudaFuncSetAttribute(gemm2w_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, G2WSmem::TOTAL);
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // how many clusters of two can be resident at once (clusters do not span GPCs)
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)(sms / 2 * 2));
    cfg.blockDim = dim3(G2_THREADS);
    cfg.dynamicSmemBytes = G2Smem::TOTAL;
    cudaLaunchAttribute at;
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2;
    at.val.clusterDim.y = 1;
    at.val.clusterDim.z = 1;
    cfg.attrs = &at;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm2_bf16_kernel, &cfg) != cudaSuccess || clusters <= 0) {
      cudaGetLastError();
      clusters = sms / 2 - 2;  // a conservative count
    }
    if (clusters > sms / 2) clusters = sms / 2;
    n[dev] = clusters > 0 ? clusters : 1;
  }
  return n[dev];
}

// KVB200_GEMM2_DIAG=1 (diagnostics, wrong results): the operand ring is filled once per CTA and every later MMA re-reads
// it without waiting, which shows the rate of the issue loop and of the tensor core's own shared-memory reads alone.
// KVB200_GEMM2_DIAG=3 / 4 / 5: as 1 with MMAs of N = 64 / N = 128 / N = 64 alternating between two accumulators (the
// cost of small instructions).
// KVB200_GEMM2_DIAG=2 (wrong results too): all loads are issued, each CTA refills a stage as soon as its previous load
// has landed, and the MMAs never wait: the two sides run at their own pace, without the barrier hand-shake.
static int g2_diag() {
  static const int v = [] {
    const char* e = getenv("KVB200_GEMM2_DIAG");
    return (e && e[0] >= '1' && e[0] <= '5') ? e[0] - '0' : 0;
  }();
  return v;
}

// KVB200_GEMM2_TILE=narrow: always 256 x 256 tiles; =wide: always 256 x 512; otherwise chosen by the number of tiles.
static int g2_wide_mode() {
  static const int v = [] {
    const char* e = getenv("KVB200_GEMM2_TILE");
    return (e && e[0] == 'n') ? 0 : ((e && e[0] == 'w') ? 2 : 1);
  }();
  return v;
}

// Launch on CTA pairs; `extra` (may be NULL) selects a fused collective as in the single-CTA kernel. max_pairs > 0 limits
// the number of compute pairs.
int launch_gemm_pair(const void* A, const void* B, const void* A2, const void* B2, void* C, const void* residual, int M, int N,
                     int K, int K2, long long lda, long long ldb, long long lda2, long long ldb2, long long ldc, int* status,
                     int max_pairs, cudaStream_t stream, const GemmExtra* extra) {
  CUtensorMap tmA, tmB, tmA2, tmB2;
  int rc;
  if ((rc = make_tmap_2d_bf16(&tmA, A, M, K, lda, G2_BM, G2_BK))) return rc;
  if ((rc = make_tmap_2d_bf16(&tmB, B, N, K, ldb, G2_BNH, G2_BK))) return rc;
  if (K2 > 0) {
    if ((rc = make_tmap_2d_bf16(&tmA2, A2, M, K2, lda2, G2_BM, G2_BK))) return rc;
    if ((rc = make_tmap_2d_bf16(&tmB2, B2, N, K2, ldb2, G2_BNH, G2_BK))) return rc;
  } else {
    tmA2 = tmA;
    tmB2 = tmB;
  }
  GemmExtra ex;
  memset(&ex, 0, sizeof(ex));
  if (extra) ex = *extra;
  int pairs = g2_max_pairs();
  if (pairs <= 0) return KVB_ERR_CUDA;
  const int copy_pairs = (ex.ag_copy_ctas + 1) / 2;
  pairs -= copy_pairs;  // copy CTAs and compute CTAs wait on one another: all of them must be resident at once
  if (pairs < 1) return KVB_ERR_ARG;
  if (max_pairs > 0 && max_pairs < pairs) pairs = max_pairs;
  // 256 x 512 tiles (fewer operand bytes per flop) when there are enough of them to keep every pair busy
  const int num_m = (M + 2 * G2_BM - 1) / (2 * G2_BM);
  const int tiles_wide = num_m * ((N + G2W_BN - 1) / G2W_BN);
  // (measured: the wide tile wins for long K loops, where its exposed epilogue is a small share, as long as its fewer
  // tiles still fill the last wave of pairs: 8192^3 0.81 -> 0.92 of the library GEMM, 8192 x 14336 x 4096 0.84 -> 0.88;
  // 8192 x 4096 x 2048 0.92 -> 0.79)
  const int waves_wide = (tiles_wide + pairs - 1) / pairs;
  const bool wide_pays = K + K2 >= 4096 && tiles_wide >= 3 * pairs && 10LL * tiles_wide >= 9LL * waves_wide * pairs;
  if (g2_wide_mode() == 2 || (g2_wide_mode() == 1 && wide_pays && !g2_diag())) {
    if (tiles_wide < pairs) pairs = tiles_wide;
    gemm2w_bf16_kernel<<<2 * (pairs + copy_pairs), G2W_THREADS, G2WSmem::TOTAL, stream>>>(
        tmA, tmB, tmA2, tmB2, (__nv_bfloat16*)C, (const __nv_bfloat16*)residual, M, N, K, K2, ldc, status, ex);
    return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
  }
  const int num_tiles = num_m * ((N + G2_BN - 1) / G2_BN);
  if (num_tiles < pairs) pairs = num_tiles;
  gemm2_bf16_kernel<<<2 * (pairs + copy_pairs), G2_THREADS, G2Smem::TOTAL, stream>>>(
      tmA, tmB, tmA2, tmB2, (__nv_bfloat16*)C, (const __nv_bfloat16*)residual, M, N, K, K2, ldc, status, ex, g2_diag());
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

}  // namespace kvb

// C[M,N] = A[M,K] · B[N,K]^T (+ A2 · B2^T) (+ residual), bf16 with fp32 accumulation, on CTA pairs (cta_group::2).
// max_pairs > 0 limits the number of CTA pairs.
extern "C" int kvb_gemm2_bf16(const void* A, const void* B, const void* A2, const void* B2, void* C, const void* residual,
                              int M, int N, int K, int K2, long long lda, long long ldb, long long lda2, long long ldb2,
                              long long ldc, int* status, int max_pairs, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return KVB_ERR_ARG;
  if ((K % 8) || (lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8)) return KVB_ERR_ALIGN;
  if (K2 > 0 && ((K2 % 8) || (lda2 % 8) || (ldb2 % 8))) return KVB_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return KVB_ERR_ALIGN;
  return kvb::launch_gemm_pair(A, B, A2, B2, C, residual, M, N, K, K2, lda, ldb, lda2, ldb2, ldc, status, max_pairs,
                               reinterpret_cast<cudaStream_t>(stream), nullptr);
}
