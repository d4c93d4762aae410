// Native forward executor for Llama-family decoder stacks.
//
// The Python pipeline hands over raw device pointers once (weights, KV cache, scratch
// activations) and then calls `forward` once per scheduler step; the executor issues
// every kernel of the step on the caller's stream without touching the Python
// interpreter, allocating, or synchronising. This plays the role the reference gives to
// its compiled graph (`Model.execute`, max/python/max/engine/api.py:120): one host call
// per step, replayable under CUDA graph capture because every buffer address is fixed.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <tuple>
#include <vector>

namespace mb {

struct DecoderLayerWeights {
  const void* attn_norm;  // [hidden]
  const void* wqkv;       // [(n_q + 2 n_kv) * head_dim, hidden]
  const void* wo;         // [hidden, n_q * head_dim]
  const void* mlp_norm;   // [hidden]
  const void* wgu;        // [2 * inter, hidden]  (gate rows then up rows)
  const void* wd;         // [hidden, inter]
  // Block-scaled fp8 layers: the four matrices above are e4m3 and these are their fp32 scales, one per
  // 128 x 128 block ([ceil(rows/128), ceil(cols/128)]); nullptr = bf16 weights.
  const float* wqkv_s = nullptr;
  const float* wo_s = nullptr;
  const float* wgu_s = nullptr;
  const float* wd_s = nullptr;
  const void* qkv_bias = nullptr;   // [(n_q + 2 n_kv) * head_dim] added to the fused projection (Qwen2), or nullptr
  const void* q_norm = nullptr;     // [head_dim] weights of the RMSNorm on every query / key head (Qwen3), or nullptr
  const void* k_norm = nullptr;
};

struct DecoderConfig {
  int n_layers, hidden, n_q, n_kv, head_dim, inter, vocab;
  float eps;
  float norm_weight_offset;   // 0 for Llama, 1 for Gemma-style (1 + w)
  int multiply_before_cast;   // RMSNorm rounding order
  int rope_interleaved;
  int page_size;
  float attn_scale;
  float logits_scale;
  int fuse_swiglu;            // gate/up GEMM with SwiGLU epilogue
  int gemm_impl;              // 0 = one CTA per tile (+split-K), 1 = persistent stream-K
  int use_pdl;                // launch persistent GEMMs with programmatic dependent launch
  int attn_impl;              // 0 = cp.async kernels, 1 = TMA-fed single-launch kernel (page_size % 64 == 0)
  int num_sms;
  int dec_max_tokens;         // steps of up to this many tokens run the decode-step GEMMs (0 = never)
  int prefetch_weights;       // tiled GEMMs request their first weight tiles before the programmatic-dependency wait
};

struct DecoderBuffers {
  void* h;        // [max_tokens, hidden] residual stream
  void* xn;       // [max_tokens, hidden]
  void* qkv;      // [max_tokens, (n_q + 2 n_kv) * head_dim]
  void* attn;     // [max_tokens, n_q * head_dim]
  void* act;      // [max_tokens, inter] (or [max_tokens, 2*inter] + act when not fused)
  void* gu;       // [max_tokens, 2*inter] only when !fuse_swiglu
  void* last_h;   // [max_seqs, hidden]
  void* last_xn;  // [max_seqs, hidden]
  float* logits;  // [max_seqs, vocab]
  int64_t* sampled;  // [max_seqs] tokens sampled by the latest step (also next step's source)
  void* workspace;  // split-K partials
  size_t workspace_bytes;
  void* p_ws;       // persistent GEMM partial-tile slots
  int* p_counters;  // persistent GEMM tile counters (zeroed)
  int* err;
  // fp8 layers: activations quantised per token and 128-wide K group before every GEMM
  void* xq = nullptr;           // e4m3 [max_tokens, max K]
  float* xs = nullptr;          // fp32 [ceil(max K / 128), max_tokens]
  void* dec_ws = nullptr;       // decode-step GEMM partial tiles
  size_t dec_ws_bytes = 0;
  int* dec_state = nullptr;     // decode-step GEMM counters / all-reduce generation (zeroed once)
};

struct KVCacheView {
  void* base;            // bf16
  int64_t page_stride;   // elements between consecutive pages
  int64_t kv_stride;     // elements between the K and V planes of a page
  int64_t layer_stride;  // elements between layers inside a page
  int64_t head_stride;   // elements between KV heads (= page_size * head_dim)
  int64_t total_elems;   // elements in the whole allocation
};

// Device-resident per-step metadata (one packed H2D copy per step).
struct StepInputs {
  const int64_t* tokens;      // [T]
  const int32_t* positions;   // [T]
  const int64_t* slots;       // [T] flat KV slot (page * page_size + offset), -1 = skip
  const int32_t* block_table; // [B, bt_stride]
  const int32_t* q_start;     // [B]
  const int32_t* q_len;       // [B]
  const int32_t* kv_len;      // [B]
  const int32_t* tile_seq;    // [n_tiles]
  const int32_t* tile_q0;     // [n_tiles]
  const int32_t* decode_seq;  // [n_decode]
  const int32_t* logit_rows;  // [n_logits] token rows whose logits are wanted
  // optional: rows whose token id is still on the device (index into `prev_sampled`, or -1)
  const int32_t* future_src;  // [T] or nullptr
  // optional fused sampling of the logit rows (all arrays [n_logits])
  const float* temperature;
  const int32_t* top_k;
  const float* top_p;
  const float* min_p;
  const uint64_t* seeds;
  uint64_t sample_step;
  int do_sample;
  int T, B, bt_stride, n_tiles, n_decode, n_logits;
};

// Tensor-parallel state: peer addresses of the symmetric buffers (index = rank).
struct TpState {
  int world = 1, rank = 0;
  void* partial[8] = {};   // [max_tokens, hidden] bf16: row-parallel GEMM partial sums
  void* xn[8] = {};        // [max_tokens, hidden] bf16: gathered normalised activations
  void* logits[8] = {};    // [max_seqs, vocab] fp32: gathered logits
  int* flags[8] = {};      // barrier flag words
  void* h_local = nullptr;       // [ceil(max_tokens / world), hidden] bf16 residual slice
  float* logits_local = nullptr; // [max_seqs, vocab / world] fp32
  int vocab_local = 0;
  // fused bit0: row-parallel GEMMs push their partial tiles into the owners' slots (`partial` then
  // holds [slots][rows_per_rank][hidden] and must have room for partial_rows rows).
  // fused bit1: column-parallel GEMMs wait per source on ready flags instead of a closing barrier.
  int fused = 0;
  long long partial_rows = 0;
  // decode steps: receive buffers of the GEMM + all-reduce + norm kernel on every rank
  // ([3][world][lam_rows][hidden] bf16, filled with -0.0 once); the residual stream is then replicated
  void* lam[8] = {};
  int lam_rows = 0;
};

class DecoderExecutor {
 public:
  TpState tp;
  DecoderConfig cfg;
  DecoderBuffers buf;
  KVCacheView kv;
  const void* embed = nullptr;
  const void* final_norm = nullptr;
  const void* lm_head = nullptr;
  const float* cos_sin = nullptr;
  std::vector<DecoderLayerWeights> layers;
  long launches = 0;  // kernels launched since construction (for accounting)

  // Runs embedding -> layers -> final norm -> LM head on `stream`. Returns MB_OK or the
  // first launcher error.
  int forward(const StepInputs& in, cudaStream_t stream);

  // True when a step of T tokens takes the decode-step path (forward_dec).
  bool dec_usable(int T) const;

  // Per-kernel timing of eager (not graph-captured) steps: when `profiling` is set, an event is
  // recorded after every launch group; profile_ms() synchronises and returns, per label, the
  // number of intervals and their summed duration since the last call.
  bool profiling = false;
  void mark(const char* label, cudaStream_t stream);
  std::vector<std::tuple<std::string, int, double>> profile_ms();

 private:
  int forward_tp(const StepInputs& in, cudaStream_t stream);
  // Small steps (T <= cfg.dec_max_tokens), one GPU or tensor parallel: four decode-step GEMMs per layer,
  // the row-parallel ones fused with all-reduce + residual + RMSNorm; no other collective, no stand-alone
  // norm after the first one.
  int forward_dec(const StepInputs& in, cudaStream_t stream);
  std::vector<std::pair<const char*, cudaEvent_t>> marks_;
};

}  // namespace mb
