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

#include "common.cuh"
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
  static constexpr int BAR_OFFSET = GEMM_STAGES * STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;  // barriers + alignment slack
};

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmA2, const __grid_constant__ CUtensorMap tmB2,
                 __nv_bfloat16* __restrict__ C, const __nv_bfloat16* __restrict__ residual, int M, int N, int K, int K2,
                 long long ldc, int* status) {
  using S = GemmSmem<BN>;
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
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % num_m) * GEMM_BM;
        const int n0 = (tile / num_m) * BN;
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
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
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
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int m0 = (tile % num_m) * GEMM_BM;
      const int n0 = (tile / num_m) * BN;
      if (!mbar_wait_bounded(&tmem_full[acc], acc_phase, abort_flag, status, STATUS_TIMEOUT_TMEM_FULL)) break;
      tc_fence_after();
      const int m = m0 + row_in_tile;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + (uint32_t)c0, r);
        tmem_ld_wait();
        const int n = n0 + c0;
        if (m < M && n < N) {
          __nv_bfloat16* dst = C + (long long)m * ldc + n;
          const __nv_bfloat16* res = residual ? residual + (long long)m * ldc + n : nullptr;
          if (n + 32 <= N) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[v * 8 + i]);
              if (res) {
                uint4 rv = *reinterpret_cast<const uint4*>(res + v * 8);
                const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  float2 t = __bfloat1622float2(rp[i]);
                  f[2 * i] += t.x;
                  f[2 * i + 1] += t.y;
                }
              }
              uint4 o;
              o.x = pack_bf16x2(f[0], f[1]);
              o.y = pack_bf16x2(f[2], f[3]);
              o.z = pack_bf16x2(f[4], f[5]);
              o.w = pack_bf16x2(f[6], f[7]);
              *reinterpret_cast<uint4*>(dst + v * 8) = o;
            }
          } else {
            for (int i = 0; i < 32 && n + i < N; ++i) {
              float f = __uint_as_float(r[i]);
              if (res) f += __bfloat162float(res[i]);
              dst[i] = __float2bfloat16_rn(f);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
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
                       int* status, int max_ctas, cudaStream_t stream) {
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
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemm_bf16_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
    attr_set = true;
  }
  const int num_tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN);
  int ctas = sm_count();
  if (max_ctas > 0 && max_ctas < ctas) ctas = max_ctas;
  if (num_tiles < ctas) ctas = num_tiles;
  gemm_bf16_kernel<BN><<<ctas, GEMM_THREADS, S::TOTAL, stream>>>(tmA, tmB, tmA2, tmB2, (__nv_bfloat16*)C,
                                                               (const __nv_bfloat16*)residual, M, N, K, K2, ldc, status);
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
