#include "decoder_executor.h"

#include "../common/api.h"

namespace mb {

#define MB_TRY(expr)            \
  do {                          \
    int rc__ = (expr);          \
    if (rc__ != MB_OK) return rc__; \
  } while (0)

int DecoderExecutor::forward(const StepInputs& in, cudaStream_t stream) {
  const DecoderConfig& c = cfg;
  const int T = in.T;
  if (T <= 0) return MB_OK;
  const int qkv_dim = (c.n_q + 2 * c.n_kv) * c.head_dim;
  const int q_dim = c.n_q * c.head_dim;
  auto gemm = [&](const void* X, const void* W, void* Y, const void* R, int M, int N, int K,
                  int ldx, int ldy, int flags) {
    if (c.gemm_impl == 1 && buf.p_ws != nullptr) {
      launches += 1;
      return mb_gemm_bf16_persistent(X, W, Y, R, M, N, K, ldx, K, ldy, ldy, flags | (c.use_pdl ? 8 : 0),
                                     0, 0, -1, buf.p_ws, buf.p_counters, buf.err, c.num_sms, stream);
    }
    int bn, splits, stages;
    mb_gemm_bf16_plan(M, N, K, flags & 1, c.num_sms, &bn, &splits, &stages);
    if (static_cast<size_t>(splits) * M * N * sizeof(float) > buf.workspace_bytes) splits = 1;
    launches += splits > 1 ? 2 : 1;
    return mb_gemm_bf16(X, W, Y, R, M, N, K, ldx, K, ldy, ldy, flags, bn, splits, stages,
                        buf.workspace, buf.err, c.num_sms, stream);
  };

  if (in.future_src != nullptr) {
    MB_TRY(mb_realize_future_tokens(const_cast<int64_t*>(in.tokens), in.future_src, buf.sampled, T,
                                    stream));
    launches += 1;
  }
  MB_TRY(mb_embedding(in.tokens, embed, buf.h, T, c.hidden, c.vocab, 0, stream));
  launches += 1;
  for (int l = 0; l < c.n_layers; ++l) {
    const DecoderLayerWeights& w = layers[l];
    char* kbase = static_cast<char*>(kv.base) + 2 * (static_cast<int64_t>(l) * kv.layer_stride);
    void* kc = kbase;
    void* vc = kbase + 2 * kv.kv_stride;
    MB_TRY(mb_rmsnorm(buf.h, w.attn_norm, buf.xn, T, c.hidden, c.hidden, c.hidden, c.eps,
                      c.norm_weight_offset, c.multiply_before_cast, stream));
    MB_TRY(gemm(buf.xn, w.wqkv, buf.qkv, nullptr, T, qkv_dim, c.hidden, c.hidden, qkv_dim, 0));
    MB_TRY(mb_rope_kv_store(buf.qkv, in.positions, in.slots, cos_sin, kc, vc, T, c.n_q, c.n_kv,
                            c.head_dim, c.page_size, kv.page_stride, kv.head_stride,
                            c.rope_interleaved, stream));
    if (c.attn_impl == 1 && c.page_size % 64 == 0) {
      const long long hd = c.head_dim;
      MB_TRY(mb_paged_attention_tma(
          buf.qkv, qkv_dim, buf.attn, q_dim, kv.base, kv.total_elems / hd,
          static_cast<long long>(l) * kv.layer_stride / hd,
          (static_cast<long long>(l) * kv.layer_stride + kv.kv_stride) / hd, kv.page_stride / hd,
          in.block_table, in.bt_stride, in.q_start, in.q_len, in.kv_len, in.tile_seq, in.tile_q0,
          in.n_tiles, in.n_decode, in.decode_seq, c.n_q, c.n_kv, c.head_dim, c.page_size,
          c.attn_scale, buf.err, stream));
      launches += 3;
    } else {
      MB_TRY(mb_paged_attention(buf.qkv, qkv_dim, buf.attn, q_dim, kc, vc, in.block_table,
                                in.bt_stride, in.q_start, in.q_len, in.kv_len, in.tile_seq,
                                in.tile_q0, in.n_tiles, in.n_decode, in.decode_seq, c.n_q, c.n_kv,
                                c.head_dim, c.page_size, kv.page_stride, kv.head_stride,
                                c.attn_scale, stream));
      launches += 2 + (in.n_tiles > 0) + (in.n_decode > 0);
    }
    MB_TRY(gemm(buf.attn, w.wo, buf.h, buf.h, T, c.hidden, q_dim, q_dim, c.hidden, 2));
    MB_TRY(mb_rmsnorm(buf.h, w.mlp_norm, buf.xn, T, c.hidden, c.hidden, c.hidden, c.eps,
                      c.norm_weight_offset, c.multiply_before_cast, stream));
    launches += 1;
    if (c.fuse_swiglu) {
      MB_TRY(gemm(buf.xn, w.wgu, buf.act, nullptr, T, c.inter, c.hidden, c.hidden, c.inter, 1));
    } else {
      MB_TRY(gemm(buf.xn, w.wgu, buf.gu, nullptr, T, 2 * c.inter, c.hidden, c.hidden, 2 * c.inter,
                  0));
      MB_TRY(mb_silu_mul(buf.gu, buf.act, T, c.inter, stream));
      launches += 1;
    }
    MB_TRY(gemm(buf.act, w.wd, buf.h, buf.h, T, c.hidden, c.inter, c.inter, c.hidden, 2));
  }
  if (in.n_logits > 0) {
    MB_TRY(mb_gather_rows(buf.h, in.logit_rows, buf.last_h, in.n_logits, c.hidden * 2,
                          c.hidden * 2, stream));
    MB_TRY(mb_rmsnorm(buf.last_h, final_norm, buf.last_xn, in.n_logits, c.hidden, c.hidden,
                      c.hidden, c.eps, c.norm_weight_offset, c.multiply_before_cast, stream));
    MB_TRY(gemm(buf.last_xn, lm_head, buf.logits, nullptr, in.n_logits, c.vocab, c.hidden,
                c.hidden, c.vocab, 4));
    launches += 2;
    if (in.do_sample) {
      MB_TRY(mb_sample_topk_topp(buf.logits, buf.sampled, in.n_logits, c.vocab, c.vocab,
                                 in.temperature, in.top_k, in.top_p, in.min_p, in.seeds,
                                 in.sample_step, stream));
      launches += 1;
    }
  }
  return MB_OK;
}

}  // namespace mb
