// C API of libkvb200: every entry point launches on the given CUDA stream and
// returns KVB_OK or a negative error code; none of them synchronises the device.
// Pointers are device pointers unless stated otherwise. dtype codes: 0 = fp32,
// 1 = bf16, 2 = fp16.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  KVB_OK = 0,
  KVB_ERR_ARG = -1,
  KVB_ERR_ALIGN = -2,
  KVB_ERR_DRIVER = -3,
  KVB_ERR_TMAP = -4,
  KVB_ERR_LAUNCH = -5,
  KVB_ERR_UNSUPPORTED = -6,
  KVB_ERR_TOO_LARGE = -7,
  KVB_ERR_CUDA = -8,
};

// ---- elementwise.cu
// Gradient replay steps (csrc/quant.cu): bf16 caches, head size 128
int kvb_replay_write(void* k_buf, void* v_buf, int32_t* token_pos, const int32_t* slots, const void* key, const void* value,
                     void* old_k, void* old_v, int32_t* old_tp, int B, int G, int n, int D, int C, long long slot_sb,
                     long long slot_sg, long long kv_sb, long long kv_sg, long long kv_sn, int input_pos, int* status, void* stream);
int kvb_replay_undo(void* k_buf, void* v_buf, int32_t* token_pos, float* dk_buf, float* dv_buf, const int32_t* slots,
                    const void* old_k, const void* old_v, const int32_t* old_tp, void* dk_new, void* dv_new, int B, int G, int n,
                    int D, int C, long long slot_sb, long long slot_sg, int* status, void* stream);
// Token cross-entropy (csrc/ce_loss.cu)
int kvb_ce_loss_fwd(const void* logits, const long long* targets, float* loss, float* lse, long long rows, int V, long long ld,
                    long long ignore_index, int dtype, void* stream);
int kvb_ce_loss_bwd(const void* logits, const long long* targets, const float* lse, const float* grad, void* dlogits,
                    long long rows, int V, long long ld, long long ignore_index, int dtype, void* stream);
int kvb_add_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out, float* rstd, long long rows,
                        int dim, float eps, int add_unit_offset, void* stream);
int kvb_rmsnorm_bwd_add(const void* gy, const void* x, const void* w, const float* rstd, const void* gadd, void* dx,
                        long long rows, int dim, int add_unit_offset, void* stream);
int kvb_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int dim, float eps, int add_unit_offset,
                    int dtype, void* stream);
int kvb_rmsnorm_bwd(const void* gy, const void* x, const void* w, const float* rstd, void* dx, float* dw_partial,
                    long long rows, int dim, int add_unit_offset, int dtype, int n_partial, void* stream);
int kvb_qknorm_rope_fwd(const void* qkv, const float* cos, const float* sin, const void* qw, const void* kw, void* q, void* k,
                        void* v, float* rstd, int B, int T, int H, int G, int D, float eps, int rope_n_elem,
                        int add_unit_offset, int dtype, void* stream);
int kvb_qknorm_rope_bwd(const void* gq, const void* gk, const void* gv, const void* qkv, const float* cos, const float* sin,
                        const void* qw, const void* kw, const float* rstd, void* dqkv, float* dw_partial, int B, int T, int H,
                        int G, int D, int rope_n_elem, int add_unit_offset, int dtype, int n_partial, void* stream);
int kvb_swiglu_fwd(const void* a, const void* b, void* y, long long n, int dtype, void* stream);
int kvb_swiglu_bwd(const void* gy, const void* a, const void* b, void* da, void* db, long long n, int dtype, void* stream);

// ---- quant.cu
int kvb_quantize_rows(const void* x, uint8_t* q, float* scale, int32_t* zp, long long rows, int D, int bits, int dtype,
                      void* stream);
int kvb_dequantize_rows(const uint8_t* q, const float* scale, const int32_t* zp, void* out, int B, int G, int n, int D,
                        long long q_sb, long long q_sg, long long q_sn, long long m_sb, long long m_sg, long long o_sb,
                        long long o_sg, long long o_sn, int bits, int dtype, void* stream);
int kvb_cache_write(void* k_buf, void* v_buf, int32_t* token_pos, const int32_t* slots, const void* key, const void* value,
                    uint8_t* qk, float* sk, int32_t* zk, uint8_t* qv, float* sv, int32_t* zv, int B, int G, int n, int D, int C,
                    long long slot_sb, long long slot_sg, int input_pos, int bits, int dtype, int* status, void* stream);
// the same with batch and group strides of key / value in elements (rows D apart)
int kvb_cache_write_strided(void* k_buf, void* v_buf, int32_t* token_pos, const int32_t* slots, const void* key, const void* value,
                            uint8_t* qk, float* sk, int32_t* zk, uint8_t* qv, float* sv, int32_t* zv, int B, int G, int n, int D,
                            int C, long long slot_sb, long long slot_sg, long long kv_sb, long long kv_sg, int input_pos, int bits,
                            int dtype, int* status, void* stream);

// Device word that overrides the host ``input_pos`` of kvb_cache_write / kvb_h2o_update while set
// (NULL clears it): lets a captured decode step be replayed at later positions.
void kvb_set_position_source(const int* device_word);
const int* kvb_position_source();

// ---- h2o.cu (weights may be NULL: selection only, scores unchanged)
int kvb_h2o_update(float* scores, const float* weights, const int32_t* token_pos, int32_t* out_idx, int B, int G, int C,
                   int n_evictable, int k_select, int normalize, int input_pos, int prefill_length, long long sc_sb,
                   long long sc_sg, long long tp_sb, long long tp_sg, void* stream);

// ---- ce_loss.cu: greedy sampling
long long kvb_argmax_scratch_bytes(long long rows);
int kvb_argmax_rows(const void* logits, long long* out, void* scratch, long long rows, int V, long long ld, int dtype, void* stream);

// ---- gemm_sm100.cu
int kvb_gemm_bf16(const void* A, const void* B, const void* A2, const void* B2, void* C, const void* residual, int M, int N,
                  int K, int K2, long long lda, long long ldb, long long lda2, long long ldb2, long long ldc, int* status,
                  int max_ctas, void* stream);

// ---- gemm2_sm100.cu: the same product on CTA pairs (tcgen05.mma.cta_group::2, 256 x 256 tiles)
int kvb_gemm2_bf16(const void* A, const void* B, const void* A2, const void* B2, void* C, const void* residual, int M, int N,
                   int K, int K2, long long lda, long long ldb, long long lda2, long long ldb2, long long ldc, int* status,
                   int max_pairs, void* stream);

// ---- sdpa_sm100.cu
// Diagnostics: per-phase cycle counters of CTA 0 of later kvb_sdpa_fwd launches (4 roles x 8 int64, see sdpa_sm100.cu).
int kvb_sdpa_fwd_set_trace(void* buf);
int kvb_sdpa_bwd_set_trace(void* buf, int cap, int mode);
// scratch: kvb_sdpa_fwd_scratch_bytes(...) bytes of device memory owned by the caller
long long kvb_sdpa_fwd_scratch_bytes(int B, int H, int G, int q_len, int kv_len);
int kvb_sdpa_fwd(const void* q, const void* k, const void* v, const int32_t* token_pos, void* out, float* lse, float* weights,
                 void* scratch, int B, int H, int G, int q_len, int kv_len, long long k_sb, long long k_sg, long long tp_sb,
                 long long tp_sg, float scale, int input_pos, int* status, void* stream);
// the same for head size 128 or 64, q with batch / head strides q_sb, q_sh (elements; 0, 0: contiguous), with a sliding
// window in tokens (0: none) and a logit soft-capping threshold (0: none)
int kvb_sdpa_fwd_ex(const void* q, const void* k, const void* v, const int32_t* token_pos, void* out, float* lse, float* weights,
                    void* scratch, int B, int H, int G, int q_len, int kv_len, int head_size, long long q_sb, long long q_sh,
                    long long k_sb, long long k_sg, long long tp_sb, long long tp_sg, float scale, int input_pos, int window,
                    float softcap, int* status, void* stream);

// ---- sdpa_bwd_sm100.cu: dq (B,H,T,D) bf16 is written, dk/dv (B,G,C,D) fp32 are accumulated into
long long kvb_sdpa_bwd_scratch_bytes(int B, int H, int G, int q_len, int kv_len);
int kvb_sdpa_bwd(const void* q, const void* k, const void* v, const int32_t* token_pos, const void* out, const void* dout,
                 const float* lse, void* dq, float* dk, float* dv, void* scratch, int B, int H, int G, int q_len, int kv_len,
                 long long k_sb, long long k_sg, long long tp_sb, long long tp_sg, long long dk_sb, long long dk_sg, float scale,
                 int input_pos, int* status, void* stream);
int kvb_sdpa_bwd_ex(const void* q, const void* k, const void* v, const int32_t* token_pos, const void* out, const void* dout,
                    const float* lse, void* dq, float* dk, float* dv, void* scratch, int B, int H, int G, int q_len, int kv_len,
                    int head_size, long long q_sb, long long q_sh, long long k_sb, long long k_sg, long long tp_sb,
                    long long tp_sg, long long dk_sb, long long dk_sg, float scale, int input_pos, int window, float softcap,
                    int* status, void* stream);

// ---- decode.cu: q (B,H,D) bf16; K/V either bf16 (bits = 16) or int8/int4 codes with scale / zero point
long long kvb_decode_scratch_bytes(int B, int H, int L);
int kvb_decode_attn(const void* q, const void* kq, const void* vq, const float* ks, const int32_t* kz, const float* vs,
                    const int32_t* vz, const void* k_new, const void* v_new, const int32_t* new_slot, void* out, float* weights,
                    void* scratch, int B, int H, int G, int L, int C, int bits, float scale, void* stream);
// the same with logit soft-capping (0: none) and a sliding window (0: none; token_pos (B,G,C) int32 with strides, query_pos =
// position of the query token, taken from the device-resident position word when one is set)
int kvb_decode_attn_ex(const void* q, const void* kq, const void* vq, const float* ks, const int32_t* kz, const float* vs,
                       const int32_t* vz, const void* k_new, const void* v_new, const int32_t* new_slot, void* out, float* weights,
                       void* scratch, int B, int H, int G, int L, int C, int bits, float scale, float softcap, int window,
                       const int32_t* token_pos, long long tp_sb, long long tp_sg, int query_pos, void* stream);


// ---- comm.cu: symmetric memory over CUDA IPC and the fused all-reduce
int kvb_symm_alloc(void** ptr, long long bytes);
int kvb_symm_free(void* ptr);
int kvb_ipc_handle_size(void);
int kvb_ipc_get_handle(void* ptr, void* handle_out);
int kvb_ipc_open_handle(const void* handle, void** ptr_out);
int kvb_ipc_close_handle(void* ptr);
// In-place mean over ranks of elements [start, start+count) of the symmetric arenas. `epoch0` advances by 3 per call.
// `local_sync`: two zero-initialised uint32 words in this rank's device memory.
int kvb_allreduce_mean(void* const* bases, void* const* flags, int rank, int world, long long start, long long count,
                       float scale, unsigned epoch0, void* local_sync, int dtype, int n_ctas, int* status, double timeout_s,
                       void* stream);
// Sum over ranks of `count` elements that every rank holds in its slot of symmetric memory (small payloads; one
// NVLink round trip), plus an optional local residual, written to the local `out`. Epoch = epoch_base + *epoch_word.
int kvb_oneshot_allreduce(void* const* slots, void* const* flags, int rank, int world, long long count, const void* residual,
                          void* out, unsigned epoch_base, const void* epoch_word, int dtype, int* status, double timeout_s,
                          void* stream);
int kvb_oneshot_allreduce_norm(void* const* slots, void* const* flags, int rank, int world, int rows, int features,
                               const void* residual, const void* norm_w, float eps, int unit_offset, void* out_x, void* out_normed,
                               unsigned epoch_base, const void* epoch_word, int dtype, int* status, double timeout_s, void* stream);
#define KVB_ONESHOT_MAX_CTAS 16
#define KVB_COMM_MAX_RANKS 16

// ---- host_pool.cpp: pinned host memory pool (one slab, first-fit ranges of 256-byte granularity) and async copies
int kvb_host_pool_create(void** pool_out, long long bytes, int pinned);
int kvb_host_pool_destroy(void* pool);
int kvb_host_pool_alloc(void* pool, long long bytes, void** ptr_out);  // KVB_ERR_TOO_LARGE: no free range fits
int kvb_host_pool_free(void* pool, void* ptr);
int kvb_host_pool_stats(void* pool, long long* out6);  // capacity, in use, peak, largest free range, allocations, failures
int kvb_copy_async(void* dst, const void* src, long long bytes, int kind, void* stream);  // kind 1: H2D, 2: D2H


// ---- gemm_sm100.cu: GEMM fused with a collective over peer memory (tensor parallelism)
int kvb_gemm_reduce_scatter(const void* A, const void* B, void* out, const void* residual, void* const* recv_bufs,
                            void* const* flags, int rank, int world, int M, int N, int K, long long lda, long long ldb,
                            unsigned flag_target, int* status, double timeout_s, void* stream);
int kvb_allgather_gemm(void* stage, void* const* stages, const void* B, void* C, void* chunk_flags, void* const* ready,
                       void* const* pulled, int rank, int world, int rows, int N, int K, long long ld_stage, long long ldb,
                       long long ldc, unsigned epoch, unsigned chunk_target, unsigned pulled_target, int copy_ctas, int* status,
                       double timeout_s, void* stream);

#ifdef __cplusplus
}
#endif
