// Persistent bf16 GEMM for sm_100a:  C[M,N] = A[M,K] · B[N,K]^T (+ A2[M,K2] · B2[N,K2]^T) (+ residual)
//
//   * operands are staged by TMA (cp.async.bulk.tensor, 128B swizzle, no multicast)
//     into a 4-stage shared-memory ring;
//   * one elected thread issues tcgen05.mma (cta_group::1, kind::f16, M=128, N=BN, K=16)
//     with the fp32 accumulator in TMEM;
//   * the accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of
//     tile i (tcgen05.ld -> bf16 -> global) overlaps the main loop of tile i+1;
//   * warp roles: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
//     warps 2..5 = epilogue (each owns the 32 TMEM lanes of its sub-partition).
//
// The optional second operand pair (A2, B2) extends the K loop: it is how a LoRA
// update  x W^T + (s · x A^T) B^T  is fused into the same accumulator.
//
// Replaces the cuBLAS calls behind nn.Linear in the reference
// (keys_values/model.py:596-610, lora_utils.py:159-172).
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "gemm_extra.cuh"
#include "kvb200.h"

namespace kvb {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_STAGES = 4;
constexpr int GEMM_THREADS = 192;

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_OFFSET = GEMM_STAGES * STAGE_BYTES;   // per epilogue warp: 32 rows x 128 B staging
  static constexpr int EPI_BYTES = 4 * 32 * 128;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + alignment slack
};

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                 __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ residual, int M, int N, int K, int K2,
                 long long ldc, int* status, const GemmExtra ex) {
  using S = GemmSmem<BN>;
  // ---- all-gather copy CTAs: pull the peers' shards into local staging, chunk by chunk
  if (ex.ag_copy_ctas > 0 && (int)blockIdx.x < ex.ag_copy_ctas) {
    extern __shared__ uint8_t ag_smem_raw[];
    gemm_ag_copy_role(ex, K, status, ag_smem_raw);
    return;
  }
  const int cta = (int)blockIdx.x - ex.ag_copy_ctas;
  const int n_ctas = (int)gridDim.x - ex.ag_copy_ctas;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + S::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + GEMM_STAGES;
  uint64_t* tmem_full = empty_bar + GEMM_STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_m = (M + GEMM_BM - 1) / GEMM_BM;
  const int num_n = (N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int kb1 = (K + GEMM_BK - 1) / GEMM_BK;
  const int kb2 = (K2 + GEMM_BK - 1) / GEMM_BK;
  const int num_kb = kb1 + kb2;
  // tile -> (row offset, column offset). Row blocks are rotated so that the blocks this rank
  // already holds (all-gather) come first, or the rows this rank owns (reduce-scatter) last.
  int m_rot = 0;
  if (ex.a_flags) m_rot = (ex.ag_rank * ex.rows_per_chunk) / GEMM_BM;
  if (ex.rs_world > 1) m_rot = ((ex.rs_rank + 1) * ex.rows_per_rank / GEMM_BM) % num_m;
  auto tile_coords = [&](int tile, int& m0, int& n0) {
    const bool comm = ex.a_flags != nullptr || ex.rs_world > 1;
    if (comm) {
      // row-block major: all column tiles of a row block are adjacent in time
      const int mi = (tile / num_n + m_rot) % num_m;
      m0 = mi * GEMM_BM;
      n0 = (tile % num_n) * BN;
    } else {
      m0 = (tile % num_m) * GEMM_BM;
      n0 = (tile / num_m) * BN;
    }
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < GEMM_STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);  // one arrive per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      int stage = 0;
      uint32_t phase = 0;
      long long issued = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += n_ctas) {
        int m0, n0;
        tile_coords(tile, m0, n0);
        if (ex.a_flags) {
          // rows of A come from an all-gather: wait until the chunk that holds this tile is local
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
          if (!mbar_wait_bounded(&empty_bar[stage], phase ^ 1, abort_flag, status, STATUS_TIMEOUT_EMPTY)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * S::STAGE_BYTES;
          uint8_t* sb = sa + S::A_BYTES;
          mbar_expect_tx(&full_bar[stage], S::STAGE_BYTES);
          if (kb < kb1) {
            tma_load_2d(sa, &tmA, &full_bar[stage], kb * GEMM_BK, m0);
            tma_load_2d(sb, &tmB, &full_bar[stage], kb * GEMM_BK, n0);
          } else {
            tma_load_2d(sa, &tmA2, &full_bar[stage], (kb - kb1) * GEMM_BK, m0);
            tma_load_2d(sb, &tmB2, &full_bar[stage], (kb - kb1) * GEMM_BK, n0);
          }
          ++issued;
          if (++stage == GEMM_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Unwinding: give the copies that are still in flight a bounded time to land
        // before this CTA's shared memory can be handed to another CTA.
        long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(GEMM_BM, BN, 0, 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += n_ctas) {
        if (!mbar_wait_bounded(&tmem_empty[acc], acc_phase ^ 1, abort_flag, status, STATUS_TIMEOUT_TMEM_EMPTY)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(&full_bar[stage], phase, abort_flag, status, STATUS_TIMEOUT_FULL)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * S::STAGE_BYTES);
          const uint32_t sb = sa + S::A_BYTES;
          const uint64_t da = make_smem_desc_sw128(sa, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            // advance 16 elements (32 B) along K inside the 128B swizzle row: +2 in 16 B units
            umma_f16_ss(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == GEMM_STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // --------------------------------------------------------------- epilogue
    const int quarter = warp & 3;  // TMEM sub-partition of this warp
    const int row_in_tile = quarter * 32 + lane;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = cta; tile < num_tiles; tile += n_ctas) {
      int m0, n0;
      tile_coords(tile, m0, n0);
      if (!mbar_wait_bounded(&tmem_full[acc], acc_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int m = m0 + row_in_tile;
      // reduce-scatter epilogue: the tile goes to the receive buffer of the rank that owns its rows
      __nv_bfloat16* out_base = C;
      long long out_row = m;
      int dest = -1;
      if (ex.rs_world > 1) {
        dest = m0 / ex.rows_per_rank;
        out_base = ex.rs_dst[dest];
        out_row = (long long)ex.rs_rank * ex.rows_per_rank + (m - dest * ex.rows_per_rank);
      }
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
      // 64 columns at a time: thread = row converts its 128 bytes, the warp exchanges them through
      // shared memory (16-byte units XOR-swizzled by row, conflict-free both ways) and stores 4 rows
      // x 128 contiguous bytes per instruction. Peer memory in particular wants long contiguous
      // writes: a row-per-thread store pattern crosses NVLink in 16-byte pieces.
      uint8_t* stg = smem + S::EPI_OFFSET + quarter * (32 * 128);
      const int m_warp0 = m0 + quarter * 32;  // first row of this warp
      const long long out_row0 = out_row - lane;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 64) {
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
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
      if (dest >= 0) {
        // make this warp's peer stores visible system-wide, then count a quarter tile at the owner
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D bf16 tensor map: inner dimension `cols` (contiguous), outer `rows` with pitch
// `ld` elements; box = box_cols x box_rows, 128B swizzle (box_cols * 2 bytes == 128).
int make_tmap_2d_bf16(CUtensorMap* tm, const void* ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                      uint32_t box_cols) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return KVB_ERR_DRIVER;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? KVB_OK : KVB_ERR_TMAP;
}

static int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  }
  return n;
}

template <int BN>
static int launch_gemm(const void* A, const void* B, const void* A2, const void* B2, void* C, const void* residual, int M,
                       int N, int K, int K2, long long lda, long long ldb, long long lda2, long long ldb2, long long ldc,
                       int* status, int max_ctas, cudaStream_t stream, const GemmExtra* extra = nullptr) {
  using S = GemmSmem<BN>;
  CUtensorMap tmA, tmB, tmA2, tmB2;
  int rc;
  if ((rc = make_tmap_2d_bf16(&tmA, A, M, K, lda, GEMM_BM, GEMM_BK))) return rc;
  if ((rc = make_tmap_2d_bf16(&tmB, B, N, K, ldb, BN, GEMM_BK))) return rc;
  if (K2 > 0) {
    if ((rc = make_tmap_2d_bf16(&tmA2, A2, M, K2, lda2, GEMM_BM, GEMM_BK))) return rc;
    if ((rc = make_tmap_2d_bf16(&tmB2, B2, N, K2, ldb2, BN, GEMM_BK))) return rc;
  } else {
    tmA2 = tmA;
    tmB2 = tmB;
  }
  static kvb::PerDeviceOnce attr_once;
  if (attr_once.first()) {
    cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
  }
  const int num_tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN);
  GemmExtra ex;
  memset(&ex, 0, sizeof(ex));
  if (extra) ex = *extra;
  int ctas = sm_count();
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  int compute = ctas - ex.ag_copy_ctas;
  if (compute < 1) return KVB_ERR_ARG;
  if (num_tiles < compute) compute = num_tiles;
  ctas = compute + ex.ag_copy_ctas;
  gemm_bf16_kernel<BN><<<ctas, GEMM_THREADS, S::TOTAL, stream>>>(tmA, tmB, tmA2, tmB2, (__nv_bfloat16*)C,
                                                               (const __nv_bfloat16*)residual, M, N, K, K2, ldc, status, ex);
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

}  // namespace kvb

extern "C" int kvb_gemm_bf16(const void* A, const void* B, const void* A2, const void* B2, void* C, const void* residual,
                             int M, int N, int K, int K2, long long lda, long long ldb, long long lda2, long long ldb2,
                             long long ldc, int* status, int max_ctas, void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return KVB_ERR_ARG;
  if ((K % 8) || (lda % 8) || (ldb % 8) || (ldc % 8) || (N % 8)) return KVB_ERR_ALIGN;
  if (K2 > 0 && ((K2 % 8) || (lda2 % 8) || (ldb2 % 8))) return KVB_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) return KVB_ERR_ALIGN;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // Wide tiles when there are enough of them to fill the GPU, else narrower ones.
  const long long tiles256 = (long long)((M + 127) / 128) * ((N + 255) / 256);
  if (tiles256 >= 120 || N % 256 == 0 && tiles256 >= 64)
    return kvb::launch_gemm<256>(A, B, A2, B2, C, residual, M, N, K, K2, lda, ldb, lda2, ldb2, ldc, status, max_ctas, s);
  return kvb::launch_gemm<128>(A, B, A2, B2, C, residual, M, N, K, K2, lda, ldb, lda2, ldb2, ldc, status, max_ctas, s);
}


// ------------------------------------------------------------------------------------
// Fused GEMM + collective entry points (tensor parallelism over NVLink peer memory)
// ------------------------------------------------------------------------------------
namespace kvb {

// The fused collectives run on the CTA-pair kernel (cta_group::2) unless KVB200_TP_GEMM=single asks for the single-CTA one.
static bool tp_gemm_on_pairs() {
  static const int v = [] {
    const char* e = getenv("KVB200_TP_GEMM");
    return (e && e[0] == 's') ? 0 : 1;
  }();
  return v != 0;
}

// out[r, :] = sum_src recv[src][r, :] (+ residual[r, :]), after every source has delivered all its tiles
__global__ void reduce_partials_kernel(const __nv_bfloat16* __restrict__ recv, const uint32_t* __restrict__ flags,
                                       uint32_t target, int world, const __nv_bfloat16* __restrict__ residual,
                                       __nv_bfloat16* __restrict__ out, long long rows, int N, long long wait_limit, int* status) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if ((int)threadIdx.x < world) {
    long long t0 = clock64();
    while ((int32_t)(ld_acquire_sys_u32(flags + threadIdx.x) - target) < 0) {
      if (clock64() - t0 > wait_limit) {
        if (status) atomicCAS(status, 0, STATUS_TIMEOUT_PEER_FLAG);
        ok_s = 0;
        break;
      }
    }
  }
  __syncthreads();
  if (!ok_s) return;
  const long long nvec = rows * N / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < world; ++s) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(recv + (long long)s * rows * N) + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    if (residual) {
      const uint4 v = reinterpret_cast<const uint4*>(residual)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

}  // namespace kvb

// GEMM -> reduce-scatter. A (M,K) and B (N,K) are this rank's shards along K; the rows of the
// (M,N) product are owned by ranks in blocks of M/world rows. recv_bufs[r]: rank r's receive
// buffer [world][M/world][N] bf16; flags[r]: rank r's [world] tile counters. After the GEMM the
// rank reduces what it received into `out` (M/world, N) (+ residual). `flag_target`: value every
// counter of this rank reaches when all sources have delivered this call (4 x tiles of 128 x 256 x calls).
extern "C" int kvb_gemm_reduce_scatter(const void* A, const void* B, void* out, const void* residual, void* const* recv_bufs,
                                       void* const* flags, int rank, int world, int M, int N, int K, long long lda,
                                       long long ldb, unsigned flag_target, int* status, double timeout_s, void* stream) {
  using namespace kvb;
  if (world < 2 || world > 16 || M % world || (M / world) % GEMM_BM || N % 8 || K % 8) return KVB_ERR_ARG;
  GemmExtra ex;
  memset(&ex, 0, sizeof(ex));
  ex.rs_world = world;
  ex.rs_rank = rank;
  ex.rows_per_rank = M / world;
  ex.rs_tile_inc = 1;
  for (int r = 0; r < world; ++r) {
    ex.rs_dst[r] = (__nv_bfloat16*)recv_bufs[r];
    ex.rs_flag[r] = (uint32_t*)flags[r];
  }
  ex.wait_limit = (long long)(timeout_s * 1.9e9);
  cudaStream_t s = (cudaStream_t)stream;
  // ldc of the receive buffers is N
  // 128 x 256 tiles: a 128 x 128 tile reads as many operand bytes from shared memory per MMA cycle as
  // the tensor core can take, which leaves nothing for the TMA writes of the next stage
  int rc = tp_gemm_on_pairs()
               ? launch_gemm_pair(A, B, nullptr, nullptr, recv_bufs[rank], nullptr, M, N, K, 0, lda, ldb, 0, 0, N, status, 0, s, &ex)
               : launch_gemm<256>(A, B, nullptr, nullptr, recv_bufs[rank], nullptr, M, N, K, 0, lda, ldb, 0, 0, N, status, 0, s, &ex);
  if (rc) return rc;
  const long long rows = M / world;
  reduce_partials_kernel<<<128, 512, 0, s>>>((const __nv_bfloat16*)recv_bufs[rank], (const uint32_t*)flags[rank], flag_target,
                                             world, (const __nv_bfloat16*)residual, (__nv_bfloat16*)out, rows, N, ex.wait_limit,
                                             status);
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

// all-gather -> GEMM. stage: local staging (world*rows, K) whose block `rank` already holds this
// rank's shard; stages[r]: the same buffer of rank r (peer pointer); chunk_flags: [world] local
// counters; ready[r] / pulled[r]: flag words of rank r. C (world*rows, N) = stage · B^T.
extern "C" int kvb_allgather_gemm(void* stage, void* const* stages, const void* B, void* C, void* chunk_flags,
                                  void* const* ready, void* const* pulled, int rank, int world, int rows, int N, int K,
                                  long long ld_stage, long long ldb, long long ldc, unsigned epoch, unsigned chunk_target,
                                  unsigned pulled_target, int copy_ctas, int* status, double timeout_s, void* stream) {
  using namespace kvb;
  if (world < 2 || world > 16 || rows % GEMM_BM || N % 8 || K % 8 || copy_ctas < 1) return KVB_ERR_ARG;
  GemmExtra ex;
  memset(&ex, 0, sizeof(ex));
  ex.a_flags = (const uint32_t*)chunk_flags;
  ex.ag_flags_w = (uint32_t*)chunk_flags;
  ex.a_target = chunk_target;
  ex.rows_per_chunk = rows;
  ex.ag_copy_ctas = copy_ctas;
  ex.ag_world = world;
  ex.ag_rank = rank;
  ex.ag_stage = (__nv_bfloat16*)stage;
  ex.ag_ld = ld_stage;
  ex.ag_epoch = epoch;
  ex.ag_pulled_target = pulled_target;
  for (int r = 0; r < world; ++r) {
    ex.ag_src[r] = (const __nv_bfloat16*)stages[r] + (long long)r * rows * ld_stage;
    ex.ag_ready[r] = (uint32_t*)ready[r];
    ex.ag_pulled[r] = (uint32_t*)pulled[r];
  }
  ex.wait_limit = (long long)(timeout_s * 1.9e9);
  const int M = world * rows;
  if (tp_gemm_on_pairs())
    return launch_gemm_pair(stage, B, nullptr, nullptr, C, nullptr, M, N, K, 0, ld_stage, ldb, 0, 0, ldc, status, 0,
                            (cudaStream_t)stream, &ex);
  return launch_gemm<256>(stage, B, nullptr, nullptr, C, nullptr, M, N, K, 0, ld_stage, ldb, 0, 0, ldc, status, 0,
                          (cudaStream_t)stream, &ex);
}
