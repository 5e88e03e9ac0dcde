// GQA decode attention (one new query token per sequence) over a bf16, int8 or int4
// KV cache, with de-quantization fused into the tile load and the per-slot summed
// attention weights (H2O score input) as a second output.
//
//   split-KV: grid (B·G, n_splits, head blocks); every CTA scores 256 slots for (up to 8 of) the
//   H/G heads of its KV group, keeps the raw scores in a (B,H,L) scratch, accumulates its
//   partial (max, sum, O); a merge kernel combines the partials; a third kernel turns the raw
//   scores into weights[b,g,j] = (1/(H/G)) Σ_h exp(s_hj − lse_h). A warp reads four cache rows
//   at a time as whole 16-byte units (8 lanes per row), several loads in flight per lane: the
//   kernel is bound by the HBM read of the cache.
//
// The quantized storage is read directly: x = (q − zp)·scale is folded into the dot
// products (q·k = scale·(Σ q_i·code_i − zp·Σ q_i)), so no full-precision copy of the cache
// is ever materialised for decoding. The row of the token that is being decoded is
// taken in full precision from `k_new/v_new` (it has not been through quantization
// from the point of view of this step).
//
// Replaces csrc/kernels/sdpa_decode.cu of the reference (FlashInfer single-decode in a
// host loop over the batch, and its CUDA-core kernels with atomics) plus the per-token
// de/re-quantization of whole layers in keys_values/kvcache/quant_buffers.py:473-503.
#include <float.h>

#include "common.cuh"
#include "kvb200.h"

namespace kvb {

constexpr int DEC_D = 128;
constexpr int DEC_SPLIT = 256;    // slots per CTA (shortest split; the scratch is laid out for it)
constexpr int DEC_SPLIT_MAX = 1024;
constexpr int DEC_THREADS = 128;  // 4 warps
constexpr int DEC_MAX_GS = 16;
constexpr int DEC_HB = 8;         // heads of a group handled by one CTA (more heads: more CTAs along z)

struct DecParams {
  const __nv_bfloat16* q;       // (B,H,D)
  const void* kq;               // (Bmax,G,C,Dq) codes or bf16
  const void* vq;
  const float *ks, *vs;         // (Bmax,G,C)
  const int32_t *kz, *vz;
  const __nv_bfloat16 *k_new, *v_new;  // (B,G,D) or nullptr
  const int32_t* new_slot;      // (B,G) or nullptr
  __nv_bfloat16* out;           // (B,H*D)
  float* weights;               // (B,G,L) or nullptr
  float* logits;                // (B,H,L)
  float* part_m;                // (B,H,nS)
  float* part_l;                // (B,H,nS)
  float* part_o;                // (B,H,nS,D)
  float* lse;                   // (B,H)
  int B, H, G, L, C, gs, nS, split;
  float scale;
  // Logit soft-capping (0: none): scores become softcap · tanh(score / softcap). Sliding window (0: none): slots whose
  // token is at or before query position − window are hidden; tok_pos (B,G,C) with strides gives the tokens of the slots,
  // the query position is *pos_src when that pointer is set (captured decode steps), else query_pos.
  float softcap;
  int window, query_pos;
  const int32_t* tok_pos;
  long long tp_sb, tp_sg;
  const int* pos_src;
};

// ---------------------------------------------------------------------------------------------
// The partial kernel multiplies with mma.sync m16n8k16 (fp32 accumulate): per CTA the problem is
// (256 slots x 128 features) x (128 x up to 8 heads), N = 8 is the whole width of the product, far
// below a tcgen05 tile, and the kernel is bound by the HBM read of the cache; what the tensor
// pipe takes away is the de-quantize + FMA work of the CUDA cores (about 12 instructions per cache
// element and head before), which made the int8 / int4 kernels compute bound.
//
//   S^T (16 slots x 8 heads)    = K tile (16 slots x 128 features) · Q^T      8 k-steps
//   O^T (128 features x 8 heads) = V^T tile (128 features x 16 slots) · P^T   8 m-tiles
//
// No operand passes through shared memory. A dot product does not care about the order of its
// terms, so every lane declares the bytes it loaded (whole 16-byte units of a cache row) to be the
// fragment columns it owns, and the Q fragments are gathered once with the same permutation:
//   pass A, lane (r = lane / 4, c = lane % 4): rows r and r + 8 of the tile, 32 features each;
//   pass B, lane (r, c): 16 features (8 m-tiles x {row r, row r + 8}) of the slots 2c, 2c+1, 2c+8,
//   2c+9 of the tile; the pairs (slot, slot + 1) that an A register wants are put together by
//   the same PRMT / LOP3 that expands the codes.
// Codes become fp16 exactly and without arithmetic: 0x6400 | code is 1024 + code; the offset joins
// the zero point (x = (code' − (zp + 1024)) · scale stays folded into the products, whose terms
// are exact in the fp32 accumulator; the zero-point sum of the output uses P as rounded to fp16). bf16 caches use the bf16 MMA
// on the raw rows. The row of the token being decoded (full precision, k_new / v_new) is in one
// tile of one CTA: there the CUDA cores compute its score and its share of the output.
// ---------------------------------------------------------------------------------------------
// Feature held by element e of fragment register `slot` (0: columns 2c, 2c+1; 1: columns 2c+8, 2c+9)
// in k-step s of pass A for lane column c.
template <int BITS>
__device__ __forceinline__ int deca_feature(int c, int s, int slot, int e) {
  // lane column c holds the 16-byte units c, 4 + c, ... of a row, so that one load instruction of
  // the warp covers contiguous 64 bytes of each row
  if (BITS == 4) return ((s & 1) ? 64 : 0) + 16 * c + 4 * (s >> 1) + slot + 2 * e;
  if (BITS == 8) return 64 * (s >> 2) + 16 * c + 4 * (s & 3) + 2 * slot + e;
  return 32 * (s >> 1) + 8 * c + 4 * (s & 1) + 2 * slot + e;
}
// Feature of row r (e = 0) or r + 8 (e = 1) of m-tile m in pass B.
template <int BITS>
__device__ __forceinline__ int decb_feature(int r, int m, int e) {
  // bf16: row lane r holds the units r and 8 + r of a slot (contiguous 128 bytes per instruction)
  if (BITS == 8) return 16 * r + 2 * m + e;
  return (m >= 4 ? 64 : 0) + 8 * r + 2 * (m & 3) + e;
}

// Two floats as one operand register: fp16 pair for quantized caches, bf16 pair for bf16 caches.
template <int BITS>
__device__ __forceinline__ uint32_t dec_pack2(float lo, float hi) {
  if (BITS == 16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
  }
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <int BITS>
__device__ __forceinline__ void dec_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if (BITS == 16) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

// 16-byte units of one row that a lane holds in pass A / of one slot in pass B
template <int BITS> struct DecRaw { static constexpr int UA = BITS == 16 ? 4 : (BITS == 8 ? 2 : 1), WB = BITS == 16 ? 8 : (BITS == 8 ? 4 : 2); };

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// One tile (16 slots) of a warp in shared memory. The 16 K rows of a tile are contiguous in the
// cache (and so are the V rows, and each of the four scale / zero-point vectors), so the warp copies
// them linearly: every cp.async instruction of the warp covers 512 contiguous bytes, whole 128-byte
// lines (a copy in which each lane fetched the bytes of its own fragments touched eight half lines
// per instruction and kept the load/store pipe busy with five times the wavefronts). The 16-byte
// unit a lane copies is not, in general, one it will read: the destination is the place where the
// lane that owns it in the MMA fragments looks for it, and a __syncwarp() follows the wait.
//   K unit (row, u):  owner r = row & 7, rowsel = row >> 3, c = u & 3, i = u >> 2;
//                     16-byte position (rowsel · UA + i) · 32 + ((r ^ i) · 4 + c)
//   V unit (slot s, u) of bf16 / int8: owner c = (s & 7) >> 1, r = u & 7, j = u >> 3,
//                     islot = (s & 1) + 2 (s >> 3); position (islot · J + j) · 32 + r · 4 + (c ^ (r >> 1))
//   V of int4 (8-byte pieces, two per copied unit): byte ((islot · 4 + c) · 8 + r) · 8
//   scales: [ks | kz | vs | vz][16 slots], one instruction of 16 lanes
// The XOR terms spread the writes of one instruction and the reads of one fragment load evenly over
// the banks (four wavefronts per 512 bytes, the minimum).
template <int BITS>
struct DecStage {
  static constexpr int UA = DecRaw<BITS>::UA, WB = DecRaw<BITS>::WB;
  static constexpr int UR = BITS == 16 ? 16 : (BITS == 8 ? 8 : 4);  // 16-byte units per cache row
  static constexpr int K_BYTES = 16 * UR * 16;
  static constexpr int V_BYTES = 16 * UR * 16;
  static constexpr int S_BYTES = BITS == 16 ? 0 : 4 * 16 * 4;
  static constexpr int BYTES = K_BYTES + V_BYTES + S_BYTES;
  static constexpr int STAGES = BITS == 4 ? 6 : (BITS == 8 ? 4 : 3);  // 96 / 66 / 51 KB per CTA: two or three CTAs per SM
};

// kt / vt: byte address of the first row of the split in the K / V cache (16-byte aligned).
template <int BITS>
__device__ __forceinline__ void dec_stage_issue(uint8_t* st, const DecParams& p, const uint8_t* kt, const uint8_t* vt,
                                                long long row0j0, int tb, int n, int lane) {
  using S = DecStage<BITS>;
  constexpr int UR = S::UR, row_bytes = UR * 16;
#pragma unroll
  for (int k = 0; k < UR / 2; ++k) {
    const int gu = k * 32 + lane;          // unit of the tile
    const int row = gu / UR, u = gu % UR;  // slot of the tile, unit of the row
    const unsigned src = (unsigned)(min(tb + row, n - 1) * row_bytes + u * 16);  // rows beyond the split re-read its last row
    {
      const int r = row & 7, rowsel = row >> 3, c = u & 3, i = u >> 2;
      cp_async16(st + ((rowsel * S::UA + i) * 32 + ((r ^ i) * 4 + c)) * 16, kt + src);
    }
    {
      const int c = (row & 7) >> 1, islot = (row & 1) + 2 * (row >> 3);
      uint8_t* vst = st + S::K_BYTES;
      if (BITS == 4) {
        cp_async16(vst + ((islot * 4 + c) * 8 + 2 * u) * 8, vt + src);
      } else {
        const int r = u & 7, j = u >> 3;
        cp_async16(vst + ((islot * (UR / 8) + j) * 32 + r * 4 + (c ^ (r >> 1))) * 16, vt + src);
      }
    }
  }
  if (BITS != 16 && lane < 16) {
    const int arr = lane >> 2, q4 = lane & 3;
    const int slot = min(tb + 4 * q4, ((n - 1) >> 2) << 2);  // units beyond the split re-read its last one
    const void* base = arr == 0 ? (const void*)p.ks : arr == 1 ? (const void*)p.kz : arr == 2 ? (const void*)p.vs : (const void*)p.vz;
    cp_async16(st + S::K_BYTES + S::V_BYTES + (arr * 16 + 4 * q4) * 4, reinterpret_cast<const uint8_t*>(base) + (row0j0 + slot) * 4);
  }
}

// ... as the A registers of k-step s for this row: x0 = columns (2c, 2c+1), x1 = columns (2c+8, 2c+9)
template <int BITS>
__device__ __forceinline__ void deca_frag(const uint4 (&u)[DecRaw<BITS>::UA], int s, uint32_t& x0, uint32_t& x1) {
  const uint32_t* w = reinterpret_cast<const uint32_t*>(u);
  if (BITS == 16) {
    x0 = w[2 * s];
    x1 = w[2 * s + 1];
  } else if (BITS == 8) {
    x0 = __byte_perm(w[s], 0x64646464u, 0x4140);
    x1 = __byte_perm(w[s], 0x64646464u, 0x4342);
  } else {
    const uint32_t v = w[s >> 1];
    if (s & 1) {  // low nibbles: features 64 + ...
      x0 = (v & 0x000F000Fu) | 0x64006400u;
      x1 = ((v >> 8) & 0x000F000Fu) | 0x64006400u;
    } else {
      x0 = ((v >> 4) & 0x000F000Fu) | 0x64006400u;
      x1 = ((v >> 12) & 0x000F000Fu) | 0x64006400u;
    }
  }
}

// A registers of m-tile m for one pair of slots (wa: the even slot, wb: the odd one):
// x0 = (row r; slot, slot + 1), x1 = (row r + 8; slot, slot + 1)
template <int BITS>
__device__ __forceinline__ void decb_frag(const uint32_t (&wa)[DecRaw<BITS>::WB], const uint32_t (&wb)[DecRaw<BITS>::WB], int m,
                                          uint32_t& x0, uint32_t& x1) {
  if (BITS == 16) {
    x0 = __byte_perm(wa[m], wb[m], 0x5410);
    x1 = __byte_perm(wa[m], wb[m], 0x7632);
  } else if (BITS == 8) {
    const uint32_t t = __byte_perm(wa[m >> 1], wb[m >> 1], (m & 1) ? 0x7362 : 0x5140);
    x0 = __byte_perm(t, 0x64646464u, 0x4140);
    x1 = __byte_perm(t, 0x64646464u, 0x4342);
  } else {
    const int pi = m & 3;  // bytes (2 (pi & 1), +1) of word pi >> 1
    const uint32_t t = __byte_perm(wa[pi >> 1], wb[pi >> 1], (pi & 1) ? 0x7632 : 0x5410);
    if (m >= 4) {  // low nibbles: features 64 + ...
      x0 = (t & 0x000F000Fu) | 0x64006400u;
      x1 = ((t >> 8) & 0x000F000Fu) | 0x64006400u;
    } else {
      x0 = ((t >> 4) & 0x000F000Fu) | 0x64006400u;
      x1 = ((t >> 12) & 0x000F000Fu) | 0x64006400u;
    }
  }
}

// One CTA = (batch, KV group, split of p.split slots, block of up to 8 heads). A warp owns a
// quarter of the split, tile by tile (16 slots), and runs on its own (online softmax per warp): a
// ring of lane-private stages in shared memory is filled with cp.async several tiles ahead, so that
// the HBM latency is covered by bytes in flight, not by registers or occupancy; scores,
// exponentials (handed from the score layout to the P^T operand layout through a warp-private patch
// of shared memory) and the product with V follow without a block-wide barrier; the four warps
// merge their (max, sum, O) once at the end.
// VAR: capped scores and / or a sliding window (a separate instantiation: the plain kernel keeps its registers)
template <int BITS, bool VAR>
__global__ void __launch_bounds__(DEC_THREADS)
decode_partial_kernel(const DecParams p) {
  using ST = DecStage<BITS>;
  constexpr int NW = DEC_THREADS / 32;
  constexpr int PST = 24;                             // row stride of the P patch (floats)
  extern __shared__ __align__(16) uint8_t dec_dsm[];
  __shared__ __align__(16) float psm[NW][DEC_HB][PST];
  __shared__ float wm[NW][DEC_HB], wl[NW][DEC_HB], wz[NW][DEC_HB];
  const int bg = blockIdx.x, split = blockIdx.y, h0 = blockIdx.z * DEC_HB;
  const int nh = min(DEC_HB, p.gs - h0);  // heads of this CTA
  const int b = bg / p.G, g = bg % p.G;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, c = lane & 3;
  const int j0 = split * p.split, j1 = min(j0 + p.split, p.L);
  const int n = j1 - j0;
  const long long row0 = ((long long)b * p.G + g) * p.C;
  const int ns = p.new_slot ? p.new_slot[b * p.G + g] : -1;
  const int ns_tile = (ns >= j0 && ns < j1) ? (ns - j0) >> 4 : -1;  // tile of this CTA that holds the new token
  const long long head0 = (long long)b * p.H + g * p.gs + h0;       // first head of this CTA
  const int wslots = p.split / NW;                                   // slots of a warp (a multiple of 16)
  const int wbase = warp * wslots;                                   // first slot of this warp within the split
  const int ntiles = wbase < n ? (min(wslots, n - wbase) + 15) >> 4 : 0;
  const int ha = 2 * c, hb = 2 * c + 1;                              // heads of this lane's scores and outputs
  uint8_t* wst = dec_dsm + (size_t)warp * ST::STAGES * ST::BYTES;
  constexpr int row_bytes = BITS == 16 ? 256 : (BITS == 8 ? 128 : 64);
  const uint8_t* kb = reinterpret_cast<const uint8_t*>(p.kq) + (row0 + j0) * row_bytes;
  const uint8_t* vb = reinterpret_cast<const uint8_t*>(p.vq) + (row0 + j0) * row_bytes;

  // the first tiles are requested before anything else
#pragma unroll
  for (int t = 0; t < ST::STAGES - 1; ++t) {
    if (t < ntiles) dec_stage_issue<BITS>(wst + t * ST::BYTES, p, kb, vb, row0 + j0, wbase + 16 * t, n, lane);
    cp_async_commit();
  }

  // Q fragments of head r (B operand of the score product) and Σ_f q_f for the heads ha, hb
  uint32_t qb[8][2];
  float qsum0, qsum1;
  {
    float s = 0.f;
    const __nv_bfloat16* qr = p.q + (head0 + min(r, nh - 1)) * DEC_D;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks)
#pragma unroll
      for (int sl = 0; sl < 2; ++sl) {
        float a = __bfloat162float(qr[deca_feature<BITS>(c, ks, sl, 0)]);
        float e = __bfloat162float(qr[deca_feature<BITS>(c, ks, sl, 1)]);
        if (r >= nh) a = e = 0.f;
        const uint32_t pk = dec_pack2<BITS>(a, e);
        qb[ks][sl] = pk;
        if (BITS == 16) {
          s += a + e;
        } else {  // the sum of what the tensor core multiplies with: the fp16 values
          const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&pk));
          s += f.x + f.y;
        }
      }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    qsum0 = __shfl_sync(0xffffffffu, s, 8 * c);
    qsum1 = __shfl_sync(0xffffffffu, s, 8 * c + 4);
  }

  float m0 = -FLT_MAX, m1 = -FLT_MAX;       // running maxima of the heads ha, hb (equal in all row lanes)
  float l0 = 0.f, l1 = 0.f, z0 = 0.f, z1 = 0.f;  // this lane's share of Σ p and Σ p · v_scale · v_zp
  float acc[8][4];
#pragma unroll
  for (int m = 0; m < 8; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0.f;

  for (int t = 0; t < ntiles; ++t) {
    {  // keep the ring full: tile t + STAGES − 1 goes where tile t − 1 was
      const int tn = t + ST::STAGES - 1;
      if (tn < ntiles) dec_stage_issue<BITS>(wst + (tn % ST::STAGES) * ST::BYTES, p, kb, vb, row0 + j0, wbase + 16 * tn, n, lane);
      cp_async_commit();
      cp_async_wait<ST::STAGES - 1>();  // this lane's copies of tile t have landed ...
      __syncwarp();                      // ... and so have those of the other lanes
    }
    const uint8_t* st = wst + (t % ST::STAGES) * ST::BYTES;
    const int tb = wbase + 16 * t;
    const int jlo = tb + r, jhi = tb + r + 8;
    const bool has_new = (tb >> 4) == ns_tile;
    float kslo = 1.f, kshi = 1.f, kzlo = 0.f, kzhi = 0.f, vslo = 1.f, vshi = 1.f, vzlo = 0.f, vzhi = 0.f;
    if (BITS != 16) {
      const float* sst = reinterpret_cast<const float*>(st + ST::K_BYTES + ST::V_BYTES);
      const int32_t* szt = reinterpret_cast<const int32_t*>(sst);
      if (jlo < n) {  // codes enter as 1024 + code: the offset joins the zero point
        kslo = sst[r]; kzlo = (float)szt[16 + r] + 1024.f; vslo = sst[32 + r]; vzlo = (float)szt[48 + r] + 1024.f;
      }
      if (jhi < n) {
        kshi = sst[r + 8]; kzhi = (float)szt[16 + r + 8] + 1024.f; vshi = sst[32 + r + 8]; vzhi = (float)szt[48 + r + 8] + 1024.f;
      }
    }
    // ---- scores: d[0], [1]: slot jlo, heads ha, hb; d[2], [3]: slot jhi
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    {
      uint4 ulo[ST::UA], uhi[ST::UA];
#pragma unroll
      for (int i = 0; i < ST::UA; ++i) {
        ulo[i] = *reinterpret_cast<const uint4*>(st + ((i * 32) + ((r ^ i) * 4 + c)) * 16);
        uhi[i] = *reinterpret_cast<const uint4*>(st + (((ST::UA + i) * 32) + ((r ^ i) * 4 + c)) * 16);
      }
      float d2[4] = {0.f, 0.f, 0.f, 0.f};  // two chains of four dependent MMAs instead of one of eight
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint32_t a[4];
        deca_frag<BITS>(ulo, ks, a[0], a[2]);
        deca_frag<BITS>(uhi, ks, a[1], a[3]);
        if (ks & 1) dec_mma<BITS>(d2, a, qb[ks][0], qb[ks][1]);
        else dec_mma<BITS>(d, a, qb[ks][0], qb[ks][1]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) d[i] += d2[i];
    }
    if (has_new) {
      // The tile with the token being decoded: the cache row of its slot is stale. Its exact
      // score q_h · k_new is computed by the whole warp (lane (r, c): head r, the 32 features of
      // its Q fragments) and replaces what the tensor core made of the stale row.
      const __nv_bfloat16* kr = p.k_new + ((long long)b * p.G + g) * DEC_D;
      float dn = 0.f;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
          float2 qf;
          if (BITS == 16) qf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qb[ks][sl]));
          else qf = __half22float2(*reinterpret_cast<const __half2*>(&qb[ks][sl]));
          dn = fmaf(qf.x, __bfloat162float(kr[deca_feature<BITS>(c, ks, sl, 0)]), dn);
          dn = fmaf(qf.y, __bfloat162float(kr[deca_feature<BITS>(c, ks, sl, 1)]), dn);
        }
      dn += __shfl_xor_sync(0xffffffffu, dn, 1);
      dn += __shfl_xor_sync(0xffffffffu, dn, 2);
      const float dna = __shfl_sync(0xffffffffu, dn, 8 * c), dnb = __shfl_sync(0xffffffffu, dn, 8 * c + 4);  // heads ha, hb
      if (j0 + jlo == ns) { d[0] = dna; d[1] = dnb; kslo = 1.f; kzlo = 0.f; vslo = 1.f; vzlo = 0.f; }
      if (j0 + jhi == ns) { d[2] = dna; d[3] = dnb; kshi = 1.f; kzhi = 0.f; vshi = 1.f; vzhi = 0.f; }
    }
    float s00 = p.scale * kslo * (d[0] - kzlo * qsum0), s01 = p.scale * kslo * (d[1] - kzlo * qsum1);
    float s10 = p.scale * kshi * (d[2] - kzhi * qsum0), s11 = p.scale * kshi * (d[3] - kzhi * qsum1);
    if (VAR && p.softcap > 0.f) {
      const float inv = 1.f / p.softcap;
      s00 = p.softcap * tanhf(s00 * inv); s01 = p.softcap * tanhf(s01 * inv);
      s10 = p.softcap * tanhf(s10 * inv); s11 = p.softcap * tanhf(s11 * inv);
    }
    if (VAR && p.window > 0) {
      // hidden slots keep the mark of "no slot" (their weight and their share of the output are zero)
      const int oldest = (p.pos_src ? *p.pos_src : p.query_pos) - p.window;
      const int32_t* tp = p.tok_pos + b * p.tp_sb + g * p.tp_sg + j0;
      if (jlo < n && tp[jlo] <= oldest) s00 = s01 = -FLT_MAX;
      if (jhi < n && tp[jhi] <= oldest) s10 = s11 = -FLT_MAX;
    }
    float mx0 = -FLT_MAX, mx1 = -FLT_MAX;
    if (jlo < n) {
      if (ha < nh) p.logits[(head0 + ha) * p.L + j0 + jlo] = s00;
      if (hb < nh) p.logits[(head0 + hb) * p.L + j0 + jlo] = s01;
      mx0 = s00;
      mx1 = s01;
    } else {
      s00 = s01 = -FLT_MAX;
    }
    if (jhi < n) {
      if (ha < nh) p.logits[(head0 + ha) * p.L + j0 + jhi] = s10;
      if (hb < nh) p.logits[(head0 + hb) * p.L + j0 + jhi] = s11;
      mx0 = fmaxf(mx0, s10);
      mx1 = fmaxf(mx1, s11);
    } else {
      s10 = s11 = -FLT_MAX;
    }
    // ---- online softmax: new maxima over the row lanes; what has been accumulated shrinks by exp(m − m')
#pragma unroll
    for (int o = 4; o < 32; o <<= 1) {
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
    }
    const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
    const float al0 = __expf(m0 - mn0), al1 = __expf(m1 - mn1);
    m0 = mn0;
    m1 = mn1;
    if (__any_sync(0xffffffffu, al0 != 1.f || al1 != 1.f)) {
      l0 *= al0; z0 *= al0;
      l1 *= al1; z1 *= al1;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        acc[m][0] *= al0; acc[m][2] *= al0;
        acc[m][1] *= al1; acc[m][3] *= al1;
      }
    }
    {
      const float p00 = s00 == -FLT_MAX ? 0.f : __expf(s00 - m0), p01 = s01 == -FLT_MAX ? 0.f : __expf(s01 - m1);
      const float p10 = s10 == -FLT_MAX ? 0.f : __expf(s10 - m0), p11 = s11 == -FLT_MAX ? 0.f : __expf(s11 - m1);
      l0 += p00 + p10;
      l1 += p01 + p11;
      float a00 = p00 * vslo, a01 = p01 * vslo, a10 = p10 * vshi, a11 = p11 * vshi;
      if (BITS != 16) {  // as the tensor core will see them, so that the offset of the codes cancels exactly
        a00 = __half2float(__float2half_rn(a00)); a01 = __half2float(__float2half_rn(a01));
        a10 = __half2float(__float2half_rn(a10)); a11 = __half2float(__float2half_rn(a11));
      }
      z0 += a00 * vzlo + a10 * vzhi;
      z1 += a01 * vzlo + a11 * vzhi;
      psm[warp][ha][r] = a00;
      psm[warp][hb][r] = a01;
      psm[warp][ha][r + 8] = a10;
      psm[warp][hb][r + 8] = a11;
    }
    __syncwarp();
    // ---- O^T += V^T tile · P^T
    if (has_new) {
      // the new token's share p · v_new is added on the CUDA cores (every (feature, head) of the
      // accumulator tile has one owner); its stale cache row then multiplies with zero
      const int sidx = ns - j0 - tb;
      const float pa = psm[warp][ha][sidx], pb = psm[warp][hb][sidx];
      const __nv_bfloat16* vr = p.v_new + ((long long)b * p.G + g) * DEC_D;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const float v0 = __bfloat162float(vr[decb_feature<BITS>(r, m, 0)]), v1 = __bfloat162float(vr[decb_feature<BITS>(r, m, 1)]);
        acc[m][0] = fmaf(pa, v0, acc[m][0]);
        acc[m][1] = fmaf(pb, v0, acc[m][1]);
        acc[m][2] = fmaf(pa, v1, acc[m][2]);
        acc[m][3] = fmaf(pb, v1, acc[m][3]);
      }
      __syncwarp();
      if (lane < DEC_HB) psm[warp][lane][sidx] = 0.f;
      __syncwarp();
    }
    {
      const float2 p0 = *reinterpret_cast<const float2*>(&psm[warp][r][2 * c]);
      const float2 p1 = *reinterpret_cast<const float2*>(&psm[warp][r][2 * c + 8]);
      const uint32_t pb0 = dec_pack2<BITS>(p0.x, p0.y), pb1 = dec_pack2<BITS>(p1.x, p1.y);
      uint32_t vw[4][ST::WB];
      const uint8_t* vst = st + ST::K_BYTES;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int vpos = r * 4 + (c ^ (r >> 1));
        if (BITS == 16) {
          const uint4 x = *reinterpret_cast<const uint4*>(vst + (((2 * i) * 32) + vpos) * 16);
          const uint4 y = *reinterpret_cast<const uint4*>(vst + (((2 * i + 1) * 32) + vpos) * 16);
          vw[i][0] = x.x; vw[i][1] = x.y; vw[i][2] = x.z; vw[i][3] = x.w;
          vw[i][4 % ST::WB] = y.x; vw[i][5 % ST::WB] = y.y; vw[i][6 % ST::WB] = y.z; vw[i][7 % ST::WB] = y.w;
        } else if (BITS == 8) {
          const uint4 x = *reinterpret_cast<const uint4*>(vst + ((i * 32) + vpos) * 16);
          vw[i][0] = x.x; vw[i][1] = x.y; vw[i][2 % ST::WB] = x.z; vw[i][3 % ST::WB] = x.w;
        } else {
          const uint2 x = *reinterpret_cast<const uint2*>(vst + ((i * 4 + c) * 8 + r) * 8);
          vw[i][0] = x.x; vw[i][1] = x.y;
        }
      }
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        uint32_t a[4];
        decb_frag<BITS>(vw[0], vw[1], m, a[0], a[1]);
        decb_frag<BITS>(vw[2], vw[3], m, a[2], a[3]);
        dec_mma<BITS>(acc[m], a, pb0, pb1);
      }
    }
    __syncwarp();  // the P patch is rewritten by the next tile
  }
  cp_async_wait<0>();
  // ---- the warp's totals (over the row lanes), then the merge of the four warps
#pragma unroll
  for (int o = 4; o < 32; o <<= 1) {
    l0 += __shfl_xor_sync(0xffffffffu, l0, o);
    l1 += __shfl_xor_sync(0xffffffffu, l1, o);
    z0 += __shfl_xor_sync(0xffffffffu, z0, o);
    z1 += __shfl_xor_sync(0xffffffffu, z1, o);
  }
  if (r == 0) {
    wm[warp][ha] = m0; wm[warp][hb] = m1;
    wl[warp][ha] = l0; wl[warp][hb] = l1;
    wz[warp][ha] = z0; wz[warp][hb] = z1;
  }
  // acc[m][0], [1]: feature (r, m, 0), heads ha, hb; [2], [3]: feature (r, m, 1). The warp's output
  // tile (8 heads x 128 floats) goes where its own stages were: all its copies have landed and been read.
  float(*ored)[DEC_D] = reinterpret_cast<float(*)[DEC_D]>(wst);
#pragma unroll
  for (int m = 0; m < 8; ++m) {
    const int f0 = decb_feature<BITS>(r, m, 0), f1 = decb_feature<BITS>(r, m, 1);
    ored[ha][f0] = acc[m][0];
    ored[hb][f0] = acc[m][1];
    ored[ha][f1] = acc[m][2];
    ored[hb][f1] = acc[m][3];
  }
  __syncthreads();
  for (int i = tid; i < nh * DEC_D; i += DEC_THREADS) {
    const int h = i / DEC_D, d = i % DEC_D;
    float M = -FLT_MAX;
#pragma unroll
    for (int w2 = 0; w2 < NW; ++w2) M = fmaxf(M, wm[w2][h]);
    float o = 0.f, l = 0.f, z = 0.f;
#pragma unroll
    for (int w2 = 0; w2 < NW; ++w2) {
      const float f = wm[w2][h] == -FLT_MAX ? 0.f : __expf(wm[w2][h] - M);  // a warp without slots has nothing to add
      const float* ow = reinterpret_cast<const float*>(dec_dsm + (size_t)w2 * ST::STAGES * ST::BYTES);
      o += f * ow[h * DEC_D + d];
      l += f * wl[w2][h];
      z += f * wz[w2][h];
    }
    p.part_o[((head0 + h) * p.nS + split) * DEC_D + d] = o - z;
    if (d == 0) {
      const long long idx = (head0 + h) * p.nS + split;
      p.part_m[idx] = M;
      p.part_l[idx] = l;
    }
  }
}

template <int BITS>
constexpr int dec_dyn_smem() { return (DEC_THREADS / 32) * DecStage<BITS>::STAGES * DecStage<BITS>::BYTES; }

__global__ void decode_merge_kernel(const DecParams p) {
  const int bh = blockIdx.x, d = threadIdx.x;  // 128 threads
  __shared__ float wgt[DEC_THREADS];
  __shared__ float red[2][DEC_THREADS / 32];
  const float* pm = p.part_m + (long long)bh * p.nS;
  const float* pl = p.part_l + (long long)bh * p.nS;
  float M = -FLT_MAX;
  for (int s = d; s < p.nS; s += DEC_THREADS) M = fmaxf(M, pm[s]);
  M = warp_max(M);
  if ((d & 31) == 0) red[0][d >> 5] = M;
  __syncthreads();
  M = fmaxf(fmaxf(red[0][0], red[0][1]), fmaxf(red[0][2], red[0][3]));
  float Lsum = 0.f, o = 0.f;
  for (int s0 = 0; s0 < p.nS; s0 += DEC_THREADS) {  // nS <= 128 for every context the scratch was sized for; the loop covers more
    const int cnt = min(DEC_THREADS, p.nS - s0);
    __syncthreads();
    if (d < cnt) {
      const float w = __expf(pm[s0 + d] - M);
      wgt[d] = w;
      Lsum += pl[s0 + d] * w;
    }
    __syncthreads();
    const float* po = p.part_o + ((long long)bh * p.nS + s0) * DEC_D + d;
    int s = 0;
    for (; s + 8 <= cnt; s += 8) {  // eight independent loads in flight
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = po[(long long)(s + u) * DEC_D];
#pragma unroll
      for (int u = 0; u < 8; ++u) o = fmaf(v[u], wgt[s + u], o);
    }
    for (; s < cnt; ++s) o = fmaf(po[(long long)s * DEC_D], wgt[s], o);
  }
  Lsum = warp_sum(Lsum);
  if ((d & 31) == 0) red[1][d >> 5] = Lsum;
  __syncthreads();
  Lsum = red[1][0] + red[1][1] + red[1][2] + red[1][3];
  p.out[(long long)bh * DEC_D + d] = __float2bfloat16_rn(o / Lsum);
  if (d == 0) p.lse[bh] = M + logf(Lsum);
}

__global__ void decode_weights_kernel(const DecParams p) {
  const int bg = blockIdx.y;
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= p.L) return;
  const int b = bg / p.G, g = bg % p.G;
  float s = 0.f;
  for (int h = 0; h < p.gs; ++h) {
    const long long bh = (long long)b * p.H + g * p.gs + h;
    s += __expf(p.logits[bh * p.L + j] - p.lse[bh]);
  }
  p.weights[(long long)bg * p.L + j] = s / p.gs;
}

}  // namespace kvb

extern "C" long long kvb_decode_scratch_bytes(int B, int H, int L) {
  const long long nS = (L + kvb::DEC_SPLIT - 1) / kvb::DEC_SPLIT;
  return ((long long)B * H * L + 2LL * B * H * nS + (long long)B * H * nS * kvb::DEC_D + (long long)B * H) * 4;
}

extern "C" const int* kvb_position_source();

extern "C" int kvb_decode_attn(const void* q, const void* kq, const void* vq, const float* ks, const int32_t* kz, const float* vs,
                               const int32_t* vz, const void* k_new, const void* v_new, const int32_t* new_slot, void* out,
                               float* weights, void* scratch, int B, int H, int G, int L, int C, int bits, float scale,
                               void* stream) {
  return kvb_decode_attn_ex(q, kq, vq, ks, kz, vs, vz, k_new, v_new, new_slot, out, weights, scratch, B, H, G, L, C, bits, scale,
                            0.f, 0, nullptr, 0, 0, 0, stream);
}

// softcap: logit soft-capping threshold (0: none). window: sliding window in tokens (0: none) with token_pos (B,G,C) int32
// (strides tp_sb, tp_sg in elements) and the position of the query token (read from the device-resident position word
// when one is set, so that a captured step serves every later position).
extern "C" int kvb_decode_attn_ex(const void* q, const void* kq, const void* vq, const float* ks, const int32_t* kz,
                                  const float* vs, const int32_t* vz, const void* k_new, const void* v_new,
                                  const int32_t* new_slot, void* out, float* weights, void* scratch, int B, int H, int G, int L,
                                  int C, int bits, float scale, float softcap, int window, const int32_t* token_pos,
                                  long long tp_sb, long long tp_sg, int query_pos, void* stream) {
  using namespace kvb;
  if (B <= 0 || H <= 0 || G <= 0 || L <= 0 || C < L || H % G) return KVB_ERR_ARG;
  if (softcap < 0.f || window < 0 || (window > 0 && !token_pos)) return KVB_ERR_ARG;
  const int gs = H / G;
  if (gs > DEC_MAX_GS) return KVB_ERR_UNSUPPORTED;
  if (bits != 16 && bits != 8 && bits != 4) return KVB_ERR_ARG;
  if (bits != 16 && (!ks || !kz || !vs || !vz)) return KVB_ERR_ARG;
  // the warp copies rows and scale vectors as 16-byte units
  if (bits != 16 && (C & 3)) return KVB_ERR_UNSUPPORTED;
  if (((uintptr_t)kq | (uintptr_t)vq | (uintptr_t)ks | (uintptr_t)kz | (uintptr_t)vs | (uintptr_t)vz) & 15) return KVB_ERR_UNSUPPORTED;
  DecParams p;
  p.q = (const __nv_bfloat16*)q; p.kq = kq; p.vq = vq; p.ks = ks; p.kz = kz; p.vs = vs; p.vz = vz;
  p.k_new = (const __nv_bfloat16*)k_new; p.v_new = (const __nv_bfloat16*)v_new; p.new_slot = k_new ? new_slot : nullptr;
  p.out = (__nv_bfloat16*)out; p.weights = weights;
  p.B = B; p.H = H; p.G = G; p.L = L; p.C = C; p.gs = gs; p.scale = scale;
  p.softcap = softcap; p.window = window; p.query_pos = query_pos; p.tok_pos = token_pos; p.tp_sb = tp_sb; p.tp_sg = tp_sg;
  p.pos_src = window > 0 ? kvb_position_source() : nullptr;
  // Slots per CTA: longer splits spend less on the per-CTA prologue and merge, as long as there are
  // CTAs for a few waves over the SMs. The scratch is laid out for the shortest split.
  const int zb = (gs + DEC_HB - 1) / DEC_HB;
  p.split = DEC_SPLIT;
  while (p.split < DEC_SPLIT_MAX && (long long)B * G * zb * ((L + 2 * p.split - 1) / (2 * p.split)) >= 4 * 148) p.split *= 2;
  p.nS = (L + p.split - 1) / p.split;
  float* sc = reinterpret_cast<float*>(scratch);
  p.logits = sc; sc += (long long)B * H * L;
  p.part_m = sc; sc += (long long)B * H * p.nS;
  p.part_l = sc; sc += (long long)B * H * p.nS;
  p.part_o = sc; sc += (long long)B * H * p.nS * DEC_D;
  p.lse = sc;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(B * G, p.nS, zb);
  static bool attr_set[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return KVB_ERR_CUDA;
  if (!attr_set[dev]) {
    cudaFuncSetAttribute(decode_partial_kernel<16, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, dec_dyn_smem<16>());
    cudaFuncSetAttribute(decode_partial_kernel<8, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, dec_dyn_smem<8>());
    cudaFuncSetAttribute(decode_partial_kernel<4, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, dec_dyn_smem<4>());
    cudaFuncSetAttribute(decode_partial_kernel<16, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, dec_dyn_smem<16>());
    cudaFuncSetAttribute(decode_partial_kernel<8, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, dec_dyn_smem<8>());
    cudaFuncSetAttribute(decode_partial_kernel<4, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, dec_dyn_smem<4>());
    attr_set[dev] = true;
  }
  if (softcap > 0.f || window > 0) {
    if (bits == 16) decode_partial_kernel<16, true><<<grid, DEC_THREADS, dec_dyn_smem<16>(), s>>>(p);
    else if (bits == 8) decode_partial_kernel<8, true><<<grid, DEC_THREADS, dec_dyn_smem<8>(), s>>>(p);
    else decode_partial_kernel<4, true><<<grid, DEC_THREADS, dec_dyn_smem<4>(), s>>>(p);
  } else {
    if (bits == 16) decode_partial_kernel<16, false><<<grid, DEC_THREADS, dec_dyn_smem<16>(), s>>>(p);
    else if (bits == 8) decode_partial_kernel<8, false><<<grid, DEC_THREADS, dec_dyn_smem<8>(), s>>>(p);
    else decode_partial_kernel<4, false><<<grid, DEC_THREADS, dec_dyn_smem<4>(), s>>>(p);
  }
  decode_merge_kernel<<<B * H, DEC_D, 0, s>>>(p);
  if (weights) {
    dim3 g2((L + 255) / 256, B * G);
    decode_weights_kernel<<<g2, 256, 0, s>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? KVB_OK : KVB_ERR_LAUNCH;
}

// ------------------------------------------------------------------------------------
// Decode attention for callers that must not allocate.
//
// Some callers cannot hand this library a scratch buffer because they cannot create one
// at the point of the call: code running while the CUDA caching allocator is frozen,
// latency-critical serving loops that pre-plan every byte of device memory at start-up and
// forbid cudaMalloc afterwards, or host runtimes in other languages that only link the C
// symbols and have no tensor allocator at all. For them the workspace of the decode kernels
// (raw scores, per-split partial results, log-sum-exp) lives in a fixed array inside this
// library's device image. Every GPU that loads the library holds these
// KVB_DECODE_STATIC_SCRATCH_BYTES until the process exits.
//
// Host code must never hand the array's name to a kernel: in host code the name is only a
// stand-in for the symbol, not a device address. The device address is looked up with
// cudaGetSymbolAddress, once per device, with that device current, and cached here.
// ------------------------------------------------------------------------------------
#define KVB_DECODE_STATIC_SCRATCH_BYTES (8u << 20)
#define KVB_DECODE_STATIC_MAX_DEVICES 64

static __device__ __align__(256) unsigned char kvb_decode_static_scratch[KVB_DECODE_STATIC_SCRATCH_BYTES];
static void* kvb_decode_static_scratch_addr[KVB_DECODE_STATIC_MAX_DEVICES] = {nullptr};

extern "C" long long kvb_decode_attn_noalloc_max_bytes(void) { return (long long)KVB_DECODE_STATIC_SCRATCH_BYTES; }

extern "C" int kvb_decode_attn_noalloc(const void* q, const void* kq, const void* vq, const float* ks, const int32_t* kz,
                                       const float* vs, const int32_t* vz, const void* k_new, const void* v_new,
                                       const int32_t* new_slot, void* out, float* weights, int B, int H, int G, int L, int C,
                                       int bits, float scale, void* stream) {
  if (B <= 0 || H <= 0 || L <= 0) return KVB_ERR_ARG;
  // workspace needed by this problem size; refuse what does not fit the fixed array
  const long long need = kvb_decode_scratch_bytes(B, H, L);
  if (need > (long long)KVB_DECODE_STATIC_SCRATCH_BYTES) return KVB_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= KVB_DECODE_STATIC_MAX_DEVICES) return KVB_ERR_CUDA;
  if (kvb_decode_static_scratch_addr[dev] == nullptr) {
    // first call on this device: resolve the device address of the array (no allocation)
    void* ptr = nullptr;
    if (cudaGetSymbolAddress((void**)&ptr, kvb_decode_static_scratch) != cudaSuccess || ptr == nullptr) return KVB_ERR_CUDA;
    kvb_decode_static_scratch_addr[dev] = ptr;
  }
  // Every word of the workspace that the kernels read (scores, partial max/sum/output,
  // log-sum-exp) is written earlier in the same call, so nothing has to be cleared.
  return kvb_decode_attn(q, kq, vq, ks, kz, vs, vz, k_new, v_new, new_slot, out, weights, kvb_decode_static_scratch_addr[dev], B, H,
                         G, L, C, bits, scale, stream);
}
