// C ABI of the kernel library. Every launcher takes raw device pointers and a stream,
// returns MB_OK or a negative error code, allocates nothing and never synchronises.
// Kernels that wait on barriers or flags report a timed-out wait through `err`
// (a device int that stays 0 on success).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define MB_OK 0
#define MB_ERR_SHAPE -1
#define MB_ERR_ALIGN -2
#define MB_ERR_DRIVER -3
#define MB_ERR_TMAP -4
#define MB_ERR_LAUNCH -5
#define MB_ERR_TOO_LARGE -6

#ifdef __cplusplus
extern "C" {
#endif

// Programmatic dependent launch for the step kernels (process-wide; see common/launch.h).
void mb_set_pdl(int on);
void mb_set_attn_decode_dense(int on);
void mb_set_attn_fork(int on);
int mb_get_pdl(void);

// ---- GEMM (gemm_tcgen05.cu) -------------------------------------------------------------
void mb_gemm_bf16_plan(int M, int N, int K, int dual, int num_sms, int* bn, int* splits,
                       int* stages);
int mb_gemm_bf16(const void* X, const void* W, void* Y, const void* R, int M, int N, int K,
                 int ldx, int ldw, int ldy, int ldr, int flags, int bn, int splits, int stages,
                 void* workspace, int* err, int num_sms, cudaStream_t stream);

// Gated variants: token tiles wait for the tensor-parallel ready flags (comm_flags.h) of the ranks
// whose rows they read, so the GEMM overlaps the all-gather that fills X. gate_flags = nullptr: off.
int mb_gemm_bf16_gated(const void* X, const void* W, void* Y, const void* R, int M, int N, int K,
                       int ldx, int ldw, int ldy, int ldr, int flags, int bn, int splits, int stages,
                       void* workspace, int* err, int num_sms, const int* gate_flags, int gate_rpr,
                       int gate_world, cudaStream_t stream);
// CTA-pair (cta_group::2, cluster of two) variant of the tiled GEMM; same contract as mb_gemm_bf16_gated.
int mb_gemm_bf16_pair(const void* X, const void* W, void* Y, const void* R, int M, int N, int K, int ldx,
                      int ldw, int ldy, int ldr, int flags, int bn, int splits, int stages, void* workspace,
                      int* err, int num_sms, const int* gate_flags, int gate_rpr, int gate_world,
                      cudaStream_t stream);
void mb_gemm_bf16_pair_plan(int M, int N, int K, int no_split, int num_sms, int* bn_out, int* splits_out);
void mb_set_gemm_pair(int min_m_plain, int min_m_dual);
// 0: never the persistent form of the CTA-pair GEMM (default 1: used when there are more tiles than SM pairs)
int mb_gemm_pair_choice(int M, int N, int dual, int num_sms);
void mb_set_gemm_pair_persistent(int on);
// bit 0: fused SwiGLU, bit 1: plain GEMMs on the token-major persistent pair kernel (tokens on the MMA's M side)
void mb_set_gemm_pair_token_major(int mask);
int mb_gemm_pair_wanted(int M, int dual);
int mb_gemm_bf16_persistent_gated(const void* X, const void* W, void* Y, const void* R, int M, int N, int K,
                                  int ldx, int ldw, int ldy, int ldr, int flags, int bn, int stages,
                                  int force_mode, void* ws, int* counters, int* err, int num_sms,
                                  const int* gate_flags, int gate_rpr, int gate_world, cudaStream_t stream);

size_t mb_gemm_persistent_workspace_bytes(int num_sms);
size_t mb_gemm_persistent_counter_ints(int num_sms);
int mb_gemm_bf16_persistent(const void* X, const void* W, void* Y, const void* R, int M, int N, int K,
                            int ldx, int ldw, int ldy, int ldr, int flags, int bn, int stages,
                            int force_mode, void* ws, int* counters, int* err, int num_sms,
                            cudaStream_t stream);

// Decode-step GEMM (gemm_decode.cu): M <= 256 tokens, equal K-block shares on every SM, epilogue over the
// whole output after one grid-wide meeting point. mode 0 bf16 store, 1 SwiGLU over W = [gate; up],
// 2 all-reduce over `world` ranks (sentinel-polled receive buffers `lam`) + residual `h` + RMSNorm -> `xn`.
int mb_gemm_dec_max_tokens(void);
int mb_gemm_dec_state_ints(void);
size_t mb_gemm_dec_workspace_bytes(int num_sms);
size_t mb_gemm_dec_lamport_elems(int world, int rows, int N);
void mb_set_gemm_dec_smem_kb(int kb);
void mb_set_gemm_dec_trace(void* buf);
// MB_OK when mb_gemm_dec takes the shape with a workspace of `ws_bytes`
int mb_gemm_dec_plan(int M, int N, int K, int mode, size_t ws_bytes, int num_sms);
int mb_gemm_dec(const void* X, const void* W, int M, int N, int K, int ldx, int ldw, int mode, void* Y, int ldy,
                void* h, void* xn, const void* gamma, float eps, float w_off, int mbc, int world, int rank,
                void* const* lam, int lam_rows, void* ws, size_t ws_bytes, int* state, int* err, int num_sms,
                cudaStream_t stream);

// ---- block-scaled fp8 (gemm_fp8_blockscaled.cu, quant_fp8.cu) ----------------------------
int mb_quant_fp8_group128(const void* x_bf16, void* q_fp8, float* scales, int M, int K, int ldx,
                          int scale_ld, int scales_k_major, cudaStream_t stream);
int mb_gemm_fp8_blockscaled(const void* Xq, const float* Xs, const void* Wq, const float* Ws, void* Y,
                            const void* R, int M, int N, int K, int flags, int bn, int stages, int splits,
                            void* workspace, size_t workspace_bytes, int num_sms, int* err,
                            cudaStream_t stream);
int mb_grouped_gemm_fp8_blockscaled(const void* Xq, const float* Xs, const void* Wq, const float* Ws, void* Y,
                                    const int32_t* expert_offsets, int n_experts, int total_rows, int max_rows,
                                    int N, int K, int ldx, int bn, int stages, int* err, cudaStream_t stream);

// ---- elementwise / normalisation / rope (elementwise.cu) ---------------------------------
int mb_rmsnorm(const void* x, const void* w, void* out, int rows, int cols, int ldx, int ldo,
               float eps, float weight_offset, int multiply_before_cast, cudaStream_t stream);
int mb_add_rmsnorm(const void* x, void* residual, const void* w, void* out, int rows, int cols,
                   float eps, float weight_offset, int multiply_before_cast, cudaStream_t stream);
// RMSNorm over head_dim of every query and key head of a fused [T, (n_q + 2 n_kv) * head_dim] projection, in place
int mb_qk_norm(void* qkv, const void* q_w, const void* k_w, int T, int n_q, int n_kv, int head_dim, int ld, float eps,
               cudaStream_t stream);
// x[r, 0:cols] += bias (bf16; rows `ld` elements apart, cols and ld multiples of 8)
int mb_add_bias(void* x, const void* bias, int rows, int cols, int ld, cudaStream_t stream);
int mb_silu_mul(const void* gate_up, void* out, int rows, int inter, cudaStream_t stream);
int mb_silu_mul_quant_fp8(const void* gate_up, void* q_fp8, float* scales, int M, int inter, int ld_s,
                          const int32_t* n_rows_dev, cudaStream_t stream);
void mb_set_mla_split_workspace(void* ws, size_t ws_bytes, int* counters, int n_counters);
void mb_set_mla_split(int mode);
size_t mb_mla_split_workspace_bytes(int num_sms);
int mb_mla_prefill_tc(const void* q_lat, const void* q_rope, void* out, const void* cache, long long page_stride,
                      long long n_pages, const int32_t* block_table, int bt_stride, const int32_t* q_start,
                      const int32_t* q_len, const int32_t* kv_len, int T, int B, int n_heads, int page_size, float scale,
                      int32_t* tok_scratch, int* err, cudaStream_t stream);
int mb_mla_post_down(const void* qkv_a, int ld, int q_lora, int R, const void* gamma_q, const void* gamma_kv, float eps,
                     const int32_t* positions, const float* cos_sin, const int64_t* slots, void* q_a_out, void* cache,
                     int T, int page_size, long long page_stride, cudaStream_t stream);
int mb_mla_q_rope(const void* q, int n_heads, int nope, const int32_t* positions, const float* cos_sin, void* q_rope,
                  int T, cudaStream_t stream);
int mb_gemm_dec_w8(const void* X, const void* Wq, const float* Ws, int M, int N, int K, int ldx, int mode, void* Y, int ldy,
                   void* h, void* xn, const void* gamma, float eps, float w_off, int mbc, int world, int rank,
                   void* const* lam, int lam_rows, void* ws, size_t ws_bytes, int* state, int* err, int num_sms,
                   cudaStream_t stream);
int mb_gemm_dec_wq(int wfmt, const void* X, const void* Wq, const void* block_scales, const float* global_scale, int M,
                   int N, int K, int ldx, int mode, void* Y, int ldy, void* h, void* xn, const void* gamma, float eps,
                   float w_off, int mbc, int world, int rank, void* const* lam, int lam_rows, void* ws, size_t ws_bytes,
                   int* state, int* err, int num_sms, cudaStream_t stream);
void mb_set_gemm_dec_tile_epilogue(int on);
void mb_set_gemm_dec_rope(int on);
int mb_gemm_dec_qkv_rope(const void* X, const void* W, int M, int K, int ldx, int ldw, void* qkv, int ldy,
                         const int32_t* positions, const int64_t* slots, const float* cos_sin, void* k_cache,
                         void* v_cache, int n_q, int n_kv, int head_dim, int page_size, long long page_stride,
                         long long head_stride, void* ws, size_t ws_bytes, int* state, int* err, int num_sms,
                         cudaStream_t stream);
int mb_gemm_dec_batched(const void* X, const void* W, void* Y, int B, int M, int N, int K, int ldx, int x_off, int ldy,
                        int y_off, int x_cols, void* ws, size_t ws_bytes, int* state, int* err, int num_sms,
                        cudaStream_t stream);
int mb_batched_gemm_bf16(const void* X, const void* W, void* Y, int B, int M, int N, int K, int ldx, int x_off,
                         int ldy, int y_off, int x_cols, int bn, int* err, cudaStream_t stream);
int mb_dequant_fp8_group128(const void* q_fp8, const float* scales, void* out_bf16, int M, int K, int ld_s,
                            const int32_t* n_rows_dev, cudaStream_t stream);
int mb_ep_recv_compact(const void* recv_x, const int32_t* recv_meta, const int* flags, int world, int cap,
                       int n_experts, int H, int fp8, int rows_bound, int32_t* offsets, int32_t* order, void* xq,
                       float* xs, int ld_s, int num_sms, cudaStream_t stream);
int mb_embedding(const int64_t* ids, const void* table, void* out, int n, int hidden, int vocab,
                 int vocab_start, cudaStream_t stream);
// RoPE on Q and K (in place in the fused QKV buffer) + K/V scatter into the paged cache.
int mb_rope_kv_store(void* qkv, const int32_t* positions, const int64_t* slots,
                     const float* cos_sin, void* k_cache, void* v_cache, int T, int n_q, int n_kv,
                     int head_dim, int page_size, int64_t page_stride, int64_t head_stride,
                     int interleaved, cudaStream_t stream);
int mb_realize_future_tokens(int64_t* tokens, const int32_t* src, const int64_t* prev, int n,
                             cudaStream_t stream);
int mb_gather_rows(const void* src, const int32_t* idx, void* dst, int n, int row_bytes, int ld_src,
                   cudaStream_t stream);

// ---- attention (attention.cu) --------------------------------------------------------------
int mb_paged_attention(const void* q, int ldq, void* out, int ldo, const void* k_cache,
                       const void* v_cache, const int32_t* block_table, int bt_stride,
                       const int32_t* q_start, const int32_t* q_len, const int32_t* kv_len,
                       const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles,
                       int n_decode, const int32_t* decode_seq, int n_q, int n_kv, int head_dim,
                       int page_size, int64_t page_stride, int64_t head_stride, float scale,
                       cudaStream_t stream);

// TMA-fed variant (attention_tma.cu): the KV allocation is addressed as [total_rows, head_dim].
int mb_paged_attention_tma(const void* q, int ldq, void* out, int ldo, const void* kv_base,
                           long long total_rows, long long k_off_rows, long long v_off_rows,
                           long long page_rows, const int32_t* block_table, int bt_stride,
                           const int32_t* q_start, const int32_t* q_len, const int32_t* kv_len,
                           const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles, int n_decode,
                           const int32_t* decode_seq, int n_q, int n_kv, int head_dim, int page_size,
                           float scale, int* err, cudaStream_t stream);

// Split-KV decode (attention_tma.cu): decode-only steps cut the KV tiles of all sequences into equal shares per
// CTA once this process-wide workspace is set (partials + zeroed counters, one per KV head and sequence).
size_t mb_attn_split_workspace_bytes(int num_sms);
void mb_set_attn_split_workspace(void* ws, size_t ws_bytes, int* counters, int counter_ints);
void mb_set_attn_split(int on);

// tcgen05 prefill attention (attention_tc.cu): same addressing as mb_paged_attention_tma, head_dim 128 only.
int mb_paged_attention_prefill_tc(const void* q, int ldq, void* out, int ldo, const void* kv_base,
                                  long long total_rows, long long k_off_rows, long long v_off_rows,
                                  long long page_rows, const int32_t* block_table, int bt_stride,
                                  const int32_t* q_start, const int32_t* q_len, const int32_t* kv_len,
                                  const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles, int n_q,
                                  int n_kv, int head_dim, int page_size, float scale, int* err,
                                  cudaStream_t stream);
// Route the prefill tiles of mb_paged_attention_tma through the tcgen05 kernel when a step has at least
// `min_tiles` 64-row tiles (process-wide; 0 = never).
void mb_set_attn_tc(int min_tiles);
int mb_get_attn_tc(void);

// ---- multi-head latent attention over a paged latent cache (mla.cu) ------------------------
// Decode steps (one query token per sequence) of absorbed MLA on tcgen05 (mla_tc.cu).
void mb_set_mla_tc(int on);
int mb_mla_tc_usable(int T, int B, int n_heads, int R, int page_size);
int mb_mla_decode_tc(const void* q_lat, const void* q_rope, void* out, const void* cache, long long page_stride,
                     long long n_pages, const int32_t* block_table, int bt_stride, const int32_t* q_start,
                     const int32_t* q_len, const int32_t* kv_len, int T, int B, int n_heads, int page_size,
                     float scale, int* err, cudaStream_t stream);
int mb_mla_paged_attention(const void* q_lat, const void* q_rope, void* out, const void* cache,
                           long long page_stride, const int32_t* block_table, int bt_stride,
                           const int32_t* q_start, const int32_t* q_len, const int32_t* kv_len, int T,
                           int B, int n_heads, int R, int page_size, float scale, cudaStream_t stream);
int mb_mla_kv_store(const void* c_kv, const void* k_rope, const int64_t* slots, void* cache, int T, int R,
                    int ld_c, int ld_r, int page_size, long long page_stride, cudaStream_t stream);

// ---- mixture of experts (moe.cu, grouped mode of gemm_tcgen05.cu) ---------------------------
int mb_moe_router_group_limited(const float* logits, const float* bias, int32_t* topk_ids, float* topk_w,
                                int T, int E, int n_group, int topk_group, int top_k, int norm_topk,
                                float scaling, int ld, cudaStream_t stream);
int mb_moe_router_softmax_topk(const float* logits, int32_t* topk_ids, float* topk_w, int T, int E,
                               int top_k, int norm_topk, int ld, cudaStream_t stream);
int mb_moe_create_indices(const int32_t* topk_ids, int n_pairs, int e_begin, int e_end, int32_t* counts,
                          int32_t* offsets, int32_t* cursor, int32_t* order, int32_t* inverse,
                          cudaStream_t stream);
int mb_moe_permute_rows(const void* src, const int32_t* order, const int32_t* n_rows_dev, void* dst,
                        int max_rows, int row_bytes, int top_k, cudaStream_t stream);
int mb_moe_combine(const void* expert_out, const int32_t* inverse, const float* w, const void* shared,
                   void* y, int T, int H, int top_k, cudaStream_t stream);
int mb_grouped_gemm_bf16(const void* X, const void* W, void* Y, const int32_t* expert_offsets,
                         int n_experts, int total_rows, int max_rows, int N, int K, int flags, int bn,
                         int* err, cudaStream_t stream);

// ---- tensor-parallel communication over peer memory (comm.cu) ------------------------------
int mb_tp_flag_ints(void);
int mb_tp_barrier(int world, int rank, int* const* flags, int* err, cudaStream_t stream);
int mb_tp_rs_norm_ag(int world, int rank, void* const* partial_bufs, void* const* xn_bufs,
                     int* const* flags, void* h_local, const void* gamma, int M, int H,
                     int rows_per_rank, float eps, float w_off, int mbc, int has_partials, int* err,
                     cudaStream_t stream);
// mode bit0: partials were pushed by mb_gemm_bf16_comm into partial_bufs[rank] (n_slots slots of
// [rows_per_rank, H]); wait for `expected` counter increments instead of a barrier + pull.
// mode bit1: close with per-source ready flags (for a flag-gated mb_gemm_bf16_comm) instead of a barrier.
int mb_tp_rs_norm_ag_ex(int world, int rank, void* const* partial_bufs, void* const* xn_bufs,
                        int* const* flags, void* h_local, const void* gamma, int M, int H,
                        int rows_per_rank, float eps, float w_off, int mbc, int has_partials, int mode,
                        int n_slots, int expected, int* err, cudaStream_t stream);
// GEMM fused with the neighbouring tensor-parallel collective (gemm_comm.cu).
int mb_gemm_bf16_comm(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw,
                      int ldy, int flags, int bn, int splits, int world, int rank, int rows_per_rank,
                      int* const* flags_all, void* const* partial_all, int max_slots,
                      int* expected_out, int* splits_out, int* err, int num_sms, cudaStream_t stream);
int mb_tp_allgather(int world, int rank, void* const* dst_bufs, int* const* flags, const void* src,
                    int rows, int row_bytes, int ld_src, int ld_dst, long long col_off, int* err,
                    cudaStream_t stream);

int mb_tp_allreduce(int world, int rank, void* const* in_bufs, void* const* out_bufs, void* out,
                    const void* mc_in, int* const* flags, long long n, int algo, int* err,
                    cudaStream_t stream);
// Barrier-free one-shot all-reduce (sentinel-polled receive buffers, three generations), optionally with the
// residual add + RMSNorm epilogue. lam_bufs[r]: [3][world][cap] bf16 on rank r, filled with -0.0 once.
int mb_tp_allreduce_lamport(int world, int rank, void* const* lam_bufs, const void* x, void* out, long long n,
                            long long cap, int* state, void* residual, const void* gamma, int cols, float eps,
                            float w_off, int mbc, int* err, cudaStream_t stream);
// Bounded wait on a flag word (at most 5 s): *ok_out = 1 when reached, else `code` goes to the error word.
int mb_tp_wait_flag(const int* flag, int target, unsigned timeout_ms, int code, int* err, int* ok_out,
                    cudaStream_t stream);
int mb_tp_broadcast(int world, int rank, int root, void* const* in_bufs, void* out, int* const* flags,
                    long long nbytes, int* err, cudaStream_t stream);
// rank r receives bytes [r * chunk_bytes, (r + 1) * chunk_bytes) of the root's symmetric buffer
int mb_tp_scatter(int world, int rank, int root, void* const* in_bufs, void* out, int* const* flags,
                  long long chunk_bytes, int* err, cudaStream_t stream);

// ---- expert-parallel dispatch / combine over peer memory (comm_ep.cu) -----------------------
int mb_ep_flag_ints(void);
int mb_ep_dispatch(int world, int rank, void* const* recv_x, void* const* recv_meta, int* const* flags,
                   const void* x, const int32_t* topk_ids, int32_t* send_pos, int T, int H, int top_k,
                   int e_local, int cap, int fp8, int* err, cudaStream_t stream);
int mb_ep_gather_ids(const int32_t* recv_meta, const int* flags, int32_t* ids, int world, int cap,
                     cudaStream_t stream);
int mb_ep_combine_send(int world, int rank, void* const* ret_x, int* const* flags, const void* out_sorted,
                       const int32_t* order, const int32_t* n_rows_dev, int max_rows, int H, int cap,
                       int* err, cudaStream_t stream);
int mb_ep_combine_reduce(const void* ret_x, const int32_t* topk_ids, const int32_t* send_pos, const float* w,
                         const void* shared, const void* residual, void* y, int T, int H, int top_k, int e_local,
                         int cap, cudaStream_t stream);
int mb_ep_dequant_rows(const void* src, void* dst, int n, int H, const int32_t* n_rows_dev, cudaStream_t stream);

// ---- sampling (sampling.cu) ----------------------------------------------------------------
int mb_argmax(const float* logits, int64_t* out, int rows, int vocab, int ld, cudaStream_t stream);
int mb_sample_topk_topp(const float* logits, int64_t* out, int rows, int vocab, int ld,
                        const float* temperature, const int32_t* top_k, const float* top_p,
                        const float* min_p, const uint64_t* seeds, uint64_t step,
                        cudaStream_t stream);
// 0: rows with a top-k / top-p / min-p filter are not spread over a cluster of CTAs first (default 1)
void mb_set_sample_cluster(int on);
// ---- state-space layers (state_space.cu): ragged batches, per-sequence state slots (-1 = none)
int mb_causal_conv1d_varlen(const void* x, const void* w, const void* bias, void* y, float* conv_state,
                            const int* cu_seqlens, const int* state_idx, const int* has_init, int n_seqs,
                            int D, int width, int ldx, int ldy, int act, cudaStream_t stream);
int mb_selective_scan_varlen(const void* u, const void* delta, const float* A, const void* B, const void* C,
                             const float* Dskip, const void* z, const float* dt_bias, void* y, float* ssm_state,
                             const int* cu_seqlens, const int* state_idx, const int* has_init, int n_seqs,
                             int D, int N, int ld_u, int ld_bc, int dt_softplus, cudaStream_t stream);
int mb_ssd_scan_varlen(const void* x, const void* dt, const float* A, const void* B, const void* C,
                       const float* Dskip, const float* dt_bias, void* y, float* ssm_state,
                       const int* cu_seqlens, const int* state_idx, const int* has_init, int n_seqs, int H,
                       int P, int N, int G, int dt_softplus, cudaStream_t stream);
int mb_apply_token_bitmask(float* logits, const int32_t* bitmask, int rows, int vocab, int ld,
                           cudaStream_t stream);
int mb_apply_penalties(float* logits, int rows, int vocab, int ld, const int32_t* tok,
                       const int32_t* cnt, const int32_t* offsets, const float* freq_pen,
                       const float* pres_pen, const float* rep_pen, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
