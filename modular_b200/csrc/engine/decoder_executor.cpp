#include "decoder_executor.h"

#include <string>

#include "../common/api.h"

namespace mb {

#define MB_TRY(expr)            \
  do {                          \
    int rc__ = (expr);          \
    if (rc__ != MB_OK) return rc__; \
  } while (0)

void DecoderExecutor::mark(const char* label, cudaStream_t stream) {
  if (!profiling) return;
  cudaEvent_t ev;
  if (cudaEventCreate(&ev) != cudaSuccess) return;
  cudaEventRecord(ev, stream);
  marks_.emplace_back(label, ev);
}

std::vector<std::tuple<std::string, int, double>> DecoderExecutor::profile_ms() {
  std::vector<std::tuple<std::string, int, double>> out;
  if (marks_.empty()) return out;
  cudaEventSynchronize(marks_.back().second);
  for (size_t i = 1; i < marks_.size(); ++i) {
    if (std::string(marks_[i].first) == "begin") continue;  // gap between two steps
    float ms = 0.f;
    cudaEventElapsedTime(&ms, marks_[i - 1].second, marks_[i].second);
    bool found = false;
    for (auto& e : out)
      if (std::get<0>(e) == marks_[i].first) { std::get<1>(e) += 1; std::get<2>(e) += ms; found = true; break; }
    if (!found) out.emplace_back(marks_[i].first, 1, ms);
  }
  for (auto& m : marks_) cudaEventDestroy(m.second);
  marks_.clear();
  return out;
}

// Y[M, N] (bf16, contiguous) = X[M, K] · W^T for a block-scaled fp8 weight: quantise X per token and
// 128-wide K group, then the fp8 GEMM (optionally + residual R).
static int linear_fp8(const DecoderBuffers& buf, const DecoderConfig& c, const void* X, int ldx, const void* Wq,
                      const float* Ws, void* Y, const void* R, int M, int N, int K, long* launches,
                      cudaStream_t stream) {
  if (buf.xq == nullptr || buf.xs == nullptr) return MB_ERR_SHAPE;
  MB_TRY(mb_quant_fp8_group128(X, buf.xq, buf.xs, M, K, ldx, M, 1, stream));
  MB_TRY(mb_gemm_fp8_blockscaled(buf.xq, buf.xs, Wq, Ws, Y, R, M, N, K, R != nullptr ? 2 : 0, 0, 0, 0,
                                 buf.workspace, buf.workspace_bytes, c.num_sms, buf.err, stream));
  *launches += 2;
  return MB_OK;
}

bool DecoderExecutor::dec_usable(int T) const {
  const DecoderConfig& c = cfg;
  if (T <= 0 || T > c.dec_max_tokens || buf.dec_ws == nullptr || buf.dec_state == nullptr) return false;
  if (tp.world > 1 && (tp.lam[0] == nullptr || T > tp.lam_rows)) return false;
  const int qkv_dim = (c.n_q + 2 * c.n_kv) * c.head_dim;
  const int q_dim = c.n_q * c.head_dim;
  const size_t wsb = buf.dec_ws_bytes;
  // block-scaled fp8 layers: weight tiles are converted per 128 x 128 scale block
  if (!layers.empty() && layers[0].wqkv_s != nullptr &&
      (qkv_dim % 128 || c.hidden % 128 || q_dim % 128 || c.inter % 128 || !c.fuse_swiglu))
    return false;
  return mb_gemm_dec_plan(T, qkv_dim, c.hidden, 0, wsb, c.num_sms) == MB_OK &&
         mb_gemm_dec_plan(T, c.hidden, q_dim, 2, wsb, c.num_sms) == MB_OK &&
         mb_gemm_dec_plan(T, 2 * c.inter, c.hidden, c.fuse_swiglu ? 1 : 0, wsb, c.num_sms) == MB_OK &&
         mb_gemm_dec_plan(T, c.hidden, c.inter, 2, wsb, c.num_sms) == MB_OK;
}

int DecoderExecutor::forward_dec(const StepInputs& in, cudaStream_t stream) {
  const DecoderConfig& c = cfg;
  const int T = in.T;
  const int W = tp.world, R = tp.rank;
  const int qkv_dim = (c.n_q + 2 * c.n_kv) * c.head_dim;
  const int q_dim = c.n_q * c.head_dim;
  auto dec = [&](const void* X, const void* Wt, const float* Ws, int N, int K, int mode, void* Y, int ldy,
                 const void* gamma) {
    launches += 1;
    if (Ws != nullptr)      // block-scaled fp8 weights, bf16 activations
      return mb_gemm_dec_w8(X, Wt, Ws, T, N, K, K, mode, Y, ldy, buf.h, buf.xn, gamma, c.eps, c.norm_weight_offset,
                            c.multiply_before_cast, W, R, tp.lam, tp.lam_rows, buf.dec_ws, buf.dec_ws_bytes,
                            buf.dec_state, buf.err, c.num_sms, stream);
    return mb_gemm_dec(X, Wt, T, N, K, K, K, mode, Y, ldy, buf.h, buf.xn, gamma, c.eps, c.norm_weight_offset,
                       c.multiply_before_cast, W, R, tp.lam, tp.lam_rows, buf.dec_ws, buf.dec_ws_bytes,
                       buf.dec_state, buf.err, c.num_sms, stream);
  };
  mark("begin", stream);
  if (in.future_src != nullptr) {
    MB_TRY(mb_realize_future_tokens(const_cast<int64_t*>(in.tokens), in.future_src, buf.sampled, T, stream));
    launches += 1;
  }
  MB_TRY(mb_embedding(in.tokens, embed, buf.h, T, c.hidden, c.vocab, 0, stream));
  MB_TRY(mb_rmsnorm(buf.h, layers[0].attn_norm, buf.xn, T, c.hidden, c.hidden, c.hidden, c.eps,
                    c.norm_weight_offset, c.multiply_before_cast, stream));
  launches += 2;
  mark("embed", stream);
  for (int l = 0; l < c.n_layers; ++l) {
    const DecoderLayerWeights& w = layers[l];
    const long long hd = c.head_dim;
    char* kbase = static_cast<char*>(kv.base) + 2 * (static_cast<int64_t>(l) * kv.layer_stride);
    // one launch for the projection, the rotation and the cache store where the kernel takes the shape
    int fused = MB_ERR_SHAPE;
    if (!c.rope_interleaved && w.wqkv_s == nullptr && w.qkv_bias == nullptr && w.q_norm == nullptr)
      fused = mb_gemm_dec_qkv_rope(buf.xn, w.wqkv, T, c.hidden, c.hidden, c.hidden, buf.qkv, qkv_dim, in.positions,
                                   in.slots, cos_sin, kbase, kbase + 2 * kv.kv_stride, c.n_q, c.n_kv, c.head_dim,
                                   c.page_size, kv.page_stride, kv.head_stride, buf.dec_ws, buf.dec_ws_bytes,
                                   buf.dec_state, buf.err, c.num_sms, stream);
    if (fused == MB_OK) {
      launches += 1;
      mark("gemm_qkv+rope+store", stream);
    } else if (fused != MB_ERR_SHAPE) {
      return fused;
    } else {
      MB_TRY(dec(buf.xn, w.wqkv, w.wqkv_s, qkv_dim, c.hidden, 0, buf.qkv, qkv_dim, nullptr));
      if (w.qkv_bias != nullptr) {
        MB_TRY(mb_add_bias(buf.qkv, w.qkv_bias, T, qkv_dim, qkv_dim, stream));
        launches += 1;
      }
      if (w.q_norm != nullptr) {
        MB_TRY(mb_qk_norm(buf.qkv, w.q_norm, w.k_norm, T, c.n_q, c.n_kv, c.head_dim, qkv_dim, c.eps, stream));
        launches += 1;
      }
      mark("gemm_qkv", stream);
      MB_TRY(mb_rope_kv_store(buf.qkv, in.positions, in.slots, cos_sin, kbase, kbase + 2 * kv.kv_stride, T, c.n_q,
                              c.n_kv, c.head_dim, c.page_size, kv.page_stride, kv.head_stride, c.rope_interleaved,
                              stream));
      launches += 1;
      mark("rope_kv_store", stream);
    }
    if (c.attn_impl == 1 && c.page_size % 64 == 0) {
      MB_TRY(mb_paged_attention_tma(
          buf.qkv, qkv_dim, buf.attn, q_dim, kv.base, kv.total_elems / hd,
          static_cast<long long>(l) * kv.layer_stride / hd,
          (static_cast<long long>(l) * kv.layer_stride + kv.kv_stride) / hd, kv.page_stride / hd, in.block_table,
          in.bt_stride, in.q_start, in.q_len, in.kv_len, in.tile_seq, in.tile_q0, in.n_tiles, in.n_decode,
          in.decode_seq, c.n_q, c.n_kv, c.head_dim, c.page_size, c.attn_scale, buf.err, stream));
    } else {
      MB_TRY(mb_paged_attention(buf.qkv, qkv_dim, buf.attn, q_dim, kbase, kbase + 2 * kv.kv_stride, in.block_table,
                                in.bt_stride, in.q_start, in.q_len, in.kv_len, in.tile_seq, in.tile_q0, in.n_tiles,
                                in.n_decode, in.decode_seq, c.n_q, c.n_kv, c.head_dim, c.page_size, kv.page_stride,
                                kv.head_stride, c.attn_scale, stream));
    }
    launches += 1;
    mark("attention", stream);
    MB_TRY(dec(buf.attn, w.wo, w.wo_s, c.hidden, q_dim, 2, nullptr, 0, w.mlp_norm));
    mark("gemm_o+ar+norm", stream);
    if (c.fuse_swiglu) {
      MB_TRY(dec(buf.xn, w.wgu, w.wgu_s, 2 * c.inter, c.hidden, 1, buf.act, c.inter, nullptr));
    } else {
      MB_TRY(dec(buf.xn, w.wgu, w.wgu_s, 2 * c.inter, c.hidden, 0, buf.gu, 2 * c.inter, nullptr));
      MB_TRY(mb_silu_mul(buf.gu, buf.act, T, c.inter, stream));
      launches += 1;
    }
    mark("gemm_gate_up", stream);
    const void* next_norm = l + 1 < c.n_layers ? layers[l + 1].attn_norm : final_norm;
    MB_TRY(dec(buf.act, w.wd, w.wd_s, c.hidden, c.inter, 2, nullptr, 0, next_norm));
    mark("gemm_down+ar+norm", stream);
  }
  if (in.n_logits > 0) {
    // xn holds the final-normalised rows of every token (on every rank)
    MB_TRY(mb_gather_rows(buf.xn, in.logit_rows, buf.last_xn, in.n_logits, c.hidden * 2, c.hidden * 2, stream));
    launches += 1;
    const float* logits = buf.logits;
    if (W > 1) {
      int bn, splits, stages;
      mb_gemm_bf16_plan(in.n_logits, tp.vocab_local, c.hidden, 0, c.num_sms, &bn, &splits, &stages);
      MB_TRY(mb_gemm_bf16(buf.last_xn, lm_head, tp.logits_local, nullptr, in.n_logits, tp.vocab_local, c.hidden,
                          c.hidden, c.hidden, tp.vocab_local, tp.vocab_local, 4, bn, 1, stages, buf.workspace,
                          buf.err, c.num_sms, stream));
      MB_TRY(mb_tp_allgather(W, R, tp.logits, tp.flags, tp.logits_local, in.n_logits, tp.vocab_local * 4,
                             tp.vocab_local * 4, c.vocab * 4, static_cast<long long>(R) * tp.vocab_local * 4,
                             buf.err, stream));
      launches += 2;
      logits = static_cast<const float*>(tp.logits[R]);
      mark("lm_head+allgather", stream);
    } else {
      int bn, splits, stages;
      mb_gemm_bf16_plan(in.n_logits, c.vocab, c.hidden, 0, c.num_sms, &bn, &splits, &stages);
      MB_TRY(mb_gemm_bf16(buf.last_xn, lm_head, buf.logits, nullptr, in.n_logits, c.vocab, c.hidden, c.hidden,
                          c.hidden, c.vocab, c.vocab, 4, bn, 1, stages, buf.workspace, buf.err, c.num_sms, stream));
      launches += 1;
      mark("lm_head", stream);
    }
    if (in.do_sample) {
      MB_TRY(mb_sample_topk_topp(logits, buf.sampled, in.n_logits, c.vocab, c.vocab, in.temperature, in.top_k,
                                 in.top_p, in.min_p, in.seeds, in.sample_step, stream));
      launches += 1;
      mark("sample", stream);
    }
  }
  return MB_OK;
}

int DecoderExecutor::forward(const StepInputs& in, cudaStream_t stream) {
  if (dec_usable(in.T)) return forward_dec(in, stream);
  if (tp.world > 1) return forward_tp(in, stream);
  const DecoderConfig& c = cfg;
  const int T = in.T;
  if (T <= 0) return MB_OK;
  const int qkv_dim = (c.n_q + 2 * c.n_kv) * c.head_dim;
  const int q_dim = c.n_q * c.head_dim;
  auto gemm = [&](const void* X, const void* W, void* Y, const void* R, int M, int N, int K,
                  int ldx, int ldy, int flags) {
    // gemm_impl: 0 = one CTA per tile, 1 = persistent (hybrid stream-K), 2 = per-shape choice
    // from measurements on B200: the persistent kernel in whole-tile mode wins for the fused
    // SwiGLU GEMM (wider token tiles, epilogue overlapped by the second TMEM buffer) and once
    // there are several waves of tiles; small single-wave GEMMs stay on the tiled kernel with
    // split-K, whose separate reduction pass is cheaper than an in-kernel fix-up.
    bool persistent = c.gemm_impl == 1;
    int mode = -1;
    if (c.gemm_impl == 2) {
      const int tiles = ((N + 127) / 128) * ((M + 255) / 256);
      persistent = (flags & 1) || tiles >= 4 * c.num_sms;
      mode = -1;   // the kernel picks whole tiles or whole tiles + a stream-K remainder
    }
    if (mb_gemm_pair_choice(M, N, flags & 1, c.num_sms)) {
      int pbn, psp;
      mb_gemm_bf16_pair_plan(M, N, K, (flags & 5) ? 1 : 0, c.num_sms, &pbn, &psp);
      if (static_cast<size_t>(psp) * M * N * sizeof(float) > buf.workspace_bytes) psp = 1;
      launches += psp > 1 ? 2 : 1;
      return mb_gemm_bf16_pair(X, W, Y, R, M, N, K, ldx, K, ldy, ldy, flags, pbn, psp, 0, buf.workspace, buf.err,
                               c.num_sms, nullptr, 1, 0, stream);
    }
    if (persistent && buf.p_ws != nullptr) {
      launches += 1;
      return mb_gemm_bf16_persistent(X, W, Y, R, M, N, K, ldx, K, ldy, ldy,
                                     flags | (c.use_pdl ? 8 : 0) | (c.prefetch_weights ? 128 : 0), 0, 0, mode, buf.p_ws,
                                     buf.p_counters, buf.err, c.num_sms, stream);
    }
    int bn, splits, stages;
    mb_gemm_bf16_plan(M, N, K, flags & 1, c.num_sms, &bn, &splits, &stages);
    if (static_cast<size_t>(splits) * M * N * sizeof(float) > buf.workspace_bytes) splits = 1;
    launches += splits > 1 ? 2 : 1;
    // bit 7: the weights of the model are written by no kernel of the step
    return mb_gemm_bf16(X, W, Y, R, M, N, K, ldx, K, ldy, ldy, flags | (c.prefetch_weights ? 128 : 0), bn, splits,
                        stages, buf.workspace, buf.err, c.num_sms, stream);
  };

  mark("begin", stream);
  if (in.future_src != nullptr) {
    MB_TRY(mb_realize_future_tokens(const_cast<int64_t*>(in.tokens), in.future_src, buf.sampled, T,
                                    stream));
    launches += 1;
  }
  MB_TRY(mb_embedding(in.tokens, embed, buf.h, T, c.hidden, c.vocab, 0, stream));
  launches += 1;
  mark("embed", stream);
  for (int l = 0; l < c.n_layers; ++l) {
    const DecoderLayerWeights& w = layers[l];
    char* kbase = static_cast<char*>(kv.base) + 2 * (static_cast<int64_t>(l) * kv.layer_stride);
    void* kc = kbase;
    void* vc = kbase + 2 * kv.kv_stride;
    MB_TRY(mb_rmsnorm(buf.h, w.attn_norm, buf.xn, T, c.hidden, c.hidden, c.hidden, c.eps,
                      c.norm_weight_offset, c.multiply_before_cast, stream));
    mark("rmsnorm", stream);
    if (w.wqkv_s != nullptr) {
      MB_TRY(linear_fp8(buf, c, buf.xn, c.hidden, w.wqkv, w.wqkv_s, buf.qkv, nullptr, T, qkv_dim, c.hidden,
                        &launches, stream));
    } else {
      MB_TRY(gemm(buf.xn, w.wqkv, buf.qkv, nullptr, T, qkv_dim, c.hidden, c.hidden, qkv_dim, 0));
    }
    if (w.qkv_bias != nullptr) {
      MB_TRY(mb_add_bias(buf.qkv, w.qkv_bias, T, qkv_dim, qkv_dim, stream));
      launches += 1;
    }
    if (w.q_norm != nullptr) {
      MB_TRY(mb_qk_norm(buf.qkv, w.q_norm, w.k_norm, T, c.n_q, c.n_kv, c.head_dim, qkv_dim, c.eps, stream));
      launches += 1;
    }
    mark("gemm_qkv", stream);
    MB_TRY(mb_rope_kv_store(buf.qkv, in.positions, in.slots, cos_sin, kc, vc, T, c.n_q, c.n_kv,
                            c.head_dim, c.page_size, kv.page_stride, kv.head_stride,
                            c.rope_interleaved, stream));
    mark("rope_kv_store", stream);
    if (c.attn_impl == 1 && c.page_size % 64 == 0) {
      const long long hd = c.head_dim;
      MB_TRY(mb_paged_attention_tma(
          buf.qkv, qkv_dim, buf.attn, q_dim, kv.base, kv.total_elems / hd,
          static_cast<long long>(l) * kv.layer_stride / hd,
          (static_cast<long long>(l) * kv.layer_stride + kv.kv_stride) / hd, kv.page_stride / hd,
          in.block_table, in.bt_stride, in.q_start, in.q_len, in.kv_len, in.tile_seq, in.tile_q0,
          in.n_tiles, in.n_decode, in.decode_seq, c.n_q, c.n_kv, c.head_dim, c.page_size,
          c.attn_scale, buf.err, stream));
      launches += 3;   // rmsnorm, rope+store, attention
    } else {
      MB_TRY(mb_paged_attention(buf.qkv, qkv_dim, buf.attn, q_dim, kc, vc, in.block_table,
                                in.bt_stride, in.q_start, in.q_len, in.kv_len, in.tile_seq,
                                in.tile_q0, in.n_tiles, in.n_decode, in.decode_seq, c.n_q, c.n_kv,
                                c.head_dim, c.page_size, kv.page_stride, kv.head_stride,
                                c.attn_scale, stream));
      launches += 2 + (in.n_tiles > 0) + (in.n_decode > 0);
    }
    mark("attention", stream);
    if (w.wo_s != nullptr) {
      MB_TRY(linear_fp8(buf, c, buf.attn, q_dim, w.wo, w.wo_s, buf.h, buf.h, T, c.hidden, q_dim, &launches, stream));
    } else {
      MB_TRY(gemm(buf.attn, w.wo, buf.h, buf.h, T, c.hidden, q_dim, q_dim, c.hidden, 2));
    }
    mark("gemm_o", stream);
    MB_TRY(mb_rmsnorm(buf.h, w.mlp_norm, buf.xn, T, c.hidden, c.hidden, c.hidden, c.eps,
                      c.norm_weight_offset, c.multiply_before_cast, stream));
    launches += 1;
    mark("rmsnorm", stream);
    if (w.wgu_s != nullptr) {
      if (buf.gu == nullptr) return MB_ERR_SHAPE;
      MB_TRY(linear_fp8(buf, c, buf.xn, c.hidden, w.wgu, w.wgu_s, buf.gu, nullptr, T, 2 * c.inter, c.hidden,
                        &launches, stream));
      MB_TRY(mb_silu_mul(buf.gu, buf.act, T, c.inter, stream));
      launches += 1;
    } else if (c.fuse_swiglu) {
      MB_TRY(gemm(buf.xn, w.wgu, buf.act, nullptr, T, c.inter, c.hidden, c.hidden, c.inter, 1));
    } else {
      MB_TRY(gemm(buf.xn, w.wgu, buf.gu, nullptr, T, 2 * c.inter, c.hidden, c.hidden, 2 * c.inter,
                  0));
      MB_TRY(mb_silu_mul(buf.gu, buf.act, T, c.inter, stream));
      launches += 1;
    }
    mark("gemm_gate_up", stream);
    if (w.wd_s != nullptr) {
      MB_TRY(linear_fp8(buf, c, buf.act, c.inter, w.wd, w.wd_s, buf.h, buf.h, T, c.hidden, c.inter, &launches, stream));
    } else {
      MB_TRY(gemm(buf.act, w.wd, buf.h, buf.h, T, c.hidden, c.inter, c.inter, c.hidden, 2));
    }
    mark("gemm_down", stream);
  }
  if (in.n_logits > 0) {
    MB_TRY(mb_gather_rows(buf.h, in.logit_rows, buf.last_h, in.n_logits, c.hidden * 2,
                          c.hidden * 2, stream));
    MB_TRY(mb_rmsnorm(buf.last_h, final_norm, buf.last_xn, in.n_logits, c.hidden, c.hidden,
                      c.hidden, c.eps, c.norm_weight_offset, c.multiply_before_cast, stream));
    MB_TRY(gemm(buf.last_xn, lm_head, buf.logits, nullptr, in.n_logits, c.vocab, c.hidden,
                c.hidden, c.vocab, 4));
    launches += 2;
    mark("lm_head", stream);
    if (in.do_sample) {
      MB_TRY(mb_sample_topk_topp(buf.logits, buf.sampled, in.n_logits, c.vocab, c.vocab,
                                 in.temperature, in.top_k, in.top_p, in.min_p, in.seeds,
                                 in.sample_step, stream));
      launches += 1;
      mark("sample", stream);
    }
  }
  return MB_OK;
}

// Tensor-parallel step. Config sizes (n_q, n_kv, inter) are this rank's shard; hidden and vocab
// are global. Column-parallel GEMMs (QKV, gate/up, LM head) read the gathered activations;
// row-parallel GEMMs (O, down) write partial sums into the symmetric `partial` buffer, and one
// fused kernel per GEMM does reduce-scatter + residual + RMSNorm + all-gather over NVLink.
int DecoderExecutor::forward_tp(const StepInputs& in, cudaStream_t stream) {
  const DecoderConfig& c = cfg;
  const int T = in.T;
  if (T <= 0) return MB_OK;
  const int W = tp.world, R = tp.rank;
  const int qkv_dim = (c.n_q + 2 * c.n_kv) * c.head_dim;
  const int q_dim = c.n_q * c.head_dim;
  const int rows_per_rank = (T + W - 1) / W;
  void* xn = tp.xn[R];
  void* partial = tp.partial[R];
  auto gemm = [&](const void* X, const void* Wt, void* Y, int M, int N, int K, int ldx, int ldy, int flags) {
    if ((flags & 1) && buf.p_ws != nullptr) {
      launches += 1;
      return mb_gemm_bf16_persistent(X, Wt, Y, nullptr, M, N, K, ldx, K, ldy, ldy, flags | (c.prefetch_weights ? 128 : 0), 0, 0, 0,
                                     buf.p_ws, buf.p_counters, buf.err, c.num_sms, stream);
    }
    int bn, splits, stages;
    mb_gemm_bf16_plan(M, N, K, flags & 1, c.num_sms, &bn, &splits, &stages);
    if (static_cast<size_t>(splits) * M * N * sizeof(float) > buf.workspace_bytes) splits = 1;
    launches += splits > 1 ? 2 : 1;
    return mb_gemm_bf16(X, Wt, Y, nullptr, M, N, K, ldx, K, ldy, ldy, flags | (c.prefetch_weights ? 128 : 0), bn, splits, stages,
                        buf.workspace, buf.err, c.num_sms, stream);
  };
  // Fused paths (tp.fused bit0 / bit1, independent):
  //   push: row-parallel GEMMs store their tiles into the owners' partial slots (GEMM -> reduce-scatter)
  //   gate: reduce+norm closes with ready flags and the next column-parallel GEMM waits per token
  //         tile for the sources it reads (all-gather -> GEMM), instead of a closing barrier
  // fp8 layers: the fp8 GEMM neither pushes its tiles nor waits on ready flags, so the exchange kernel opens
  // and closes with barriers and the GEMMs run on complete inputs
  const bool fp8 = !layers.empty() && layers[0].wqkv_s != nullptr;
  const bool push = !fp8 && (tp.fused & 1) && tp.partial_rows >= static_cast<long long>(W) * rows_per_rank;
  const bool gate_on = !fp8 && (tp.fused & 2) != 0;
  const int max_slots = push ? static_cast<int>(tp.partial_rows / rows_per_rank) : 0;
  // column-parallel GEMM on the gathered activations; its token tiles wait for the ready flags of
  // the ranks that push their rows (same kernel choice as the single-GPU path)
  auto gemm_gathered = [&](const void* Wt, const float* Ws, void* Y, int N, int ldy, int flags, bool wait) {
    if (Ws != nullptr) {
      // column-parallel fp8 GEMM on the gathered activations; SwiGLU (flags bit0: W = [gate; up], N = inter) as a
      // separate pass over the [T, 2 inter] product
      if (flags & 1) {
        if (buf.gu == nullptr) return static_cast<int>(MB_ERR_SHAPE);
        MB_TRY(linear_fp8(buf, c, xn, c.hidden, Wt, Ws, buf.gu, nullptr, T, 2 * N, c.hidden, &launches, stream));
        launches += 1;
        return mb_silu_mul(buf.gu, Y, T, N, stream);
      }
      return linear_fp8(buf, c, xn, c.hidden, Wt, Ws, Y, nullptr, T, N, c.hidden, &launches, stream);
    }
    const int* gate = wait ? tp.flags[R] : nullptr;
    if ((flags & 1) && buf.p_ws != nullptr) {
      launches += 1;
      return mb_gemm_bf16_persistent_gated(xn, Wt, Y, nullptr, T, N, c.hidden, c.hidden, c.hidden, ldy, ldy,
                                           flags, 0, 0, -1, buf.p_ws, buf.p_counters, buf.err, c.num_sms, gate,
                                           rows_per_rank, W, stream);
    }
    int bn, splits, stages;
    mb_gemm_bf16_plan(T, N, c.hidden, flags & 1, c.num_sms, &bn, &splits, &stages);
    if (static_cast<size_t>(splits) * T * N * sizeof(float) > buf.workspace_bytes) splits = 1;
    launches += splits > 1 ? 2 : 1;
    return mb_gemm_bf16_gated(xn, Wt, Y, nullptr, T, N, c.hidden, c.hidden, c.hidden, ldy, ldy, flags, bn,
                              splits, stages, buf.workspace, buf.err, c.num_sms, gate, rows_per_rank, W, stream);
  };
  // row-parallel GEMM, then reduce-scatter + residual + norm + gather of the normalised rows
  auto row_parallel_reduce_norm = [&](const void* X, const void* Wt, const float* Ws, int K, const void* gamma,
                                      bool last) {
    int expected = 0, splits = 1, mode = 0;
    if (Ws != nullptr) {
      MB_TRY(linear_fp8(buf, c, X, K, Wt, Ws, partial, nullptr, T, c.hidden, K, &launches, stream));
    } else if (push) {
      MB_TRY(mb_gemm_bf16_comm(X, Wt, partial, T, c.hidden, K, K, K, c.hidden, 32, 0, 0, W, R, rows_per_rank,
                               tp.flags, tp.partial, max_slots, &expected, &splits, buf.err, c.num_sms, stream));
      launches += 1;
      mode |= 1;
    } else {
      MB_TRY(gemm(X, Wt, partial, T, c.hidden, K, K, c.hidden, 0));
    }
    // the last reduce of the step closes with a barrier: the logits path reads every row of xn
    if (gate_on && !last) mode |= 2;
    launches += 1;
    return mb_tp_rs_norm_ag_ex(W, R, tp.partial, tp.xn, tp.flags, tp.h_local, gamma, T, c.hidden, rows_per_rank,
                               c.eps, c.norm_weight_offset, c.multiply_before_cast, 1, mode, W * splits,
                               expected, buf.err, stream);
  };

  mark("begin", stream);
  if (in.future_src != nullptr) {
    MB_TRY(mb_realize_future_tokens(const_cast<int64_t*>(in.tokens), in.future_src, buf.sampled, T, stream));
    launches += 1;
  }
  // embedding on every rank (replicated table); keep this rank's rows as its residual slice
  MB_TRY(mb_embedding(in.tokens, embed, buf.h, T, c.hidden, c.vocab, 0, stream));
  {
    const int row0 = R * rows_per_rank;
    int n = T - row0;
    if (n > rows_per_rank) n = rows_per_rank;
    if (n > 0 &&
        cudaMemcpyAsync(tp.h_local, static_cast<const char*>(buf.h) + static_cast<size_t>(row0) * c.hidden * 2,
                        static_cast<size_t>(n) * c.hidden * 2, cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
      return MB_ERR_LAUNCH;
  }
  MB_TRY(mb_rmsnorm(buf.h, layers[0].attn_norm, xn, T, c.hidden, c.hidden, c.hidden, c.eps,
                    c.norm_weight_offset, c.multiply_before_cast, stream));
  launches += 3;
  mark("embed", stream);
  for (int l = 0; l < c.n_layers; ++l) {
    const DecoderLayerWeights& w = layers[l];
    const long long hd = c.head_dim;
    MB_TRY(gemm_gathered(w.wqkv, w.wqkv_s, buf.qkv, qkv_dim, qkv_dim, 0, gate_on && l > 0));
    if (w.qkv_bias != nullptr) {
      MB_TRY(mb_add_bias(buf.qkv, w.qkv_bias, T, qkv_dim, qkv_dim, stream));
      launches += 1;
    }
    if (w.q_norm != nullptr) {
      MB_TRY(mb_qk_norm(buf.qkv, w.q_norm, w.k_norm, T, c.n_q, c.n_kv, c.head_dim, qkv_dim, c.eps, stream));
      launches += 1;
    }
    mark("gemm_qkv", stream);
    char* kbase = static_cast<char*>(kv.base) + 2 * (static_cast<int64_t>(l) * kv.layer_stride);
    MB_TRY(mb_rope_kv_store(buf.qkv, in.positions, in.slots, cos_sin, kbase, kbase + 2 * kv.kv_stride, T,
                            c.n_q, c.n_kv, c.head_dim, c.page_size, kv.page_stride, kv.head_stride,
                            c.rope_interleaved, stream));
    mark("rope_kv_store", stream);
    if (c.attn_impl == 1 && c.page_size % 64 == 0) {
      MB_TRY(mb_paged_attention_tma(
          buf.qkv, qkv_dim, buf.attn, q_dim, kv.base, kv.total_elems / hd,
          static_cast<long long>(l) * kv.layer_stride / hd,
          (static_cast<long long>(l) * kv.layer_stride + kv.kv_stride) / hd, kv.page_stride / hd,
          in.block_table, in.bt_stride, in.q_start, in.q_len, in.kv_len, in.tile_seq, in.tile_q0,
          in.n_tiles, in.n_decode, in.decode_seq, c.n_q, c.n_kv, c.head_dim, c.page_size,
          c.attn_scale, buf.err, stream));
    } else {
      MB_TRY(mb_paged_attention(buf.qkv, qkv_dim, buf.attn, q_dim, kbase, kbase + 2 * kv.kv_stride,
                                in.block_table, in.bt_stride, in.q_start, in.q_len, in.kv_len,
                                in.tile_seq, in.tile_q0, in.n_tiles, in.n_decode, in.decode_seq, c.n_q,
                                c.n_kv, c.head_dim, c.page_size, kv.page_stride, kv.head_stride,
                                c.attn_scale, stream));
    }
    launches += 2;
    mark("attention", stream);
    const void* next_norm = l + 1 < c.n_layers ? layers[l + 1].attn_norm : final_norm;
    MB_TRY(row_parallel_reduce_norm(buf.attn, w.wo, w.wo_s, q_dim, w.mlp_norm, false));
    mark("gemm_o+rs_norm_ag", stream);
    MB_TRY(gemm_gathered(w.wgu, w.wgu_s, buf.act, c.inter, c.inter, 1, gate_on));
    mark("gemm_gate_up", stream);
    MB_TRY(row_parallel_reduce_norm(buf.act, w.wd, w.wd_s, c.inter, next_norm, l + 1 == c.n_layers));
    mark("gemm_down+rs_norm_ag", stream);
  }
  if (in.n_logits > 0) {
    // xn already holds the final-normalised rows of every token on every rank
    MB_TRY(mb_gather_rows(xn, in.logit_rows, buf.last_xn, in.n_logits, c.hidden * 2, c.hidden * 2, stream));
    MB_TRY(gemm(buf.last_xn, lm_head, tp.logits_local, in.n_logits, tp.vocab_local, c.hidden, c.hidden,
                tp.vocab_local, 4));
    MB_TRY(mb_tp_allgather(W, R, tp.logits, tp.flags, tp.logits_local, in.n_logits, tp.vocab_local * 4,
                           tp.vocab_local * 4, c.vocab * 4, static_cast<long long>(R) * tp.vocab_local * 4,
                           buf.err, stream));
    launches += 2;
    mark("lm_head+allgather", stream);
    if (in.do_sample) {
      MB_TRY(mb_sample_topk_topp(static_cast<const float*>(tp.logits[R]), buf.sampled, in.n_logits, c.vocab,
                                 c.vocab, in.temperature, in.top_k, in.top_p, in.min_p, in.seeds,
                                 in.sample_step, stream));
      launches += 1;
      mark("sample", stream);
    }
  }
  return MB_OK;
}

}  // namespace mb
