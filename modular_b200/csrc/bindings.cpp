// Python bindings: torch tensors in, raw pointers + current CUDA stream out.
// No kernel is defined here; every op forwards to the C ABI in common/api.h or to the
// native executor, so the same entry points serve Python, the C++ engine and C callers.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <stdexcept>
#include <string>

#include "common/api.h"
#include "engine/decoder_executor.h"
#include "runtime/runtime.h"

namespace py = pybind11;
using torch::Tensor;

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_rc(int rc, const char* what) {
  if (rc == MB_OK) return;
  const char* msg = "unknown";
  switch (rc) {
    case MB_ERR_SHAPE: msg = "unsupported shape"; break;
    case MB_ERR_ALIGN: msg = "pointer not 16-byte aligned"; break;
    case MB_ERR_DRIVER: msg = "driver entry point unavailable"; break;
    case MB_ERR_TMAP: msg = "tensor-map encode failed"; break;
    case MB_ERR_LAUNCH: msg = "kernel launch failed"; break;
    case MB_ERR_TOO_LARGE: msg = "size beyond the supported maximum"; break;
  }
  throw std::runtime_error(std::string(what) + ": " + msg + " (" + std::to_string(rc) + ")");
}

void need_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
}
const void* optptr(const c10::optional<Tensor>& t) {
  return t.has_value() && t->defined() ? t->data_ptr() : nullptr;
}

// One error word per process (one process per GPU): kernels with bounded waits set it.
int* error_flag() {
  static int* flag = nullptr;
  if (!flag) {
    TORCH_CHECK(cudaMalloc(&flag, sizeof(int)) == cudaSuccess, "cudaMalloc(error flag)");
    cudaMemset(flag, 0, sizeof(int));
  }
  return flag;
}
int read_error_flag(bool reset) {
  int v = 0;
  cudaMemcpy(&v, error_flag(), sizeof(int), cudaMemcpyDeviceToHost);
  if (reset && v) cudaMemset(error_flag(), 0, sizeof(int));
  return v;
}

int num_sms() {
  static int n = 0;
  if (!n) n = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  return n;
}

// y = x @ w.T with optional fusions; see mb_gemm_bf16.
void gemm_bf16(const Tensor& x, const Tensor& w, Tensor& y, const c10::optional<Tensor>& residual,
               bool dual, const c10::optional<Tensor>& workspace, int bn, int splits, int stages,
               bool packed, bool pair) {
  need_cuda(x, "x"); need_cuda(w, "w"); need_cuda(y, "y");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && y.dim() == 2, "gemm_bf16: 2-D tensors expected");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16, "bf16 inputs");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && y.stride(1) == 1, "row-major operands");
  const int M = x.size(0), K = x.size(1);
  const int N = dual ? w.size(0) / 2 : w.size(0);
  TORCH_CHECK(w.size(1) == K && y.size(0) == M && y.size(1) == N, "gemm_bf16: shape mismatch");
  const bool f32 = y.scalar_type() == at::kFloat;
  TORCH_CHECK(f32 || y.scalar_type() == at::kBFloat16, "output must be bf16 or fp32");
  int flags = (dual ? 1 : 0) | (residual.has_value() && residual->defined() ? 2 : 0) | (f32 ? 4 : 0) |
              (packed ? 64 : 0);
  void* ws = nullptr;
  if (workspace.has_value() && workspace->defined()) {
    ws = workspace->data_ptr();
    if (pair) {
      if (splits <= 0 && bn <= 0) {
        int pbn;
        mb_gemm_bf16_pair_plan(M, N, K, (dual || f32) ? 1 : 0, num_sms(), &pbn, &splits);
      } else if (splits <= 0) {
        splits = 1;   // explicit tile width: no automatic split
      }
      const size_t need = static_cast<size_t>(splits > 0 ? splits : 1) * M * N * 4;
      if (need > static_cast<size_t>(workspace->nbytes())) { ws = nullptr; splits = 1; }
    } else if (splits <= 0) {
      int pbn, psp, pst;
      mb_gemm_bf16_plan(M, N, K, dual, num_sms(), &pbn, &psp, &pst);
      splits = psp;
    }
    if (!pair && static_cast<size_t>(splits) * M * N * 4 > static_cast<size_t>(workspace->nbytes())) splits = 1;
  } else {
    splits = 1;
  }
  int ldr = 0;
  if (flags & 2) {
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->stride(1) == 1, "residual");
    ldr = residual->stride(0);
  }
  if (pair) {
    check_rc(mb_gemm_bf16_pair(x.data_ptr(), w.data_ptr(), y.data_ptr(), optptr(residual), M, N, K,
                               x.stride(0), w.stride(0), y.stride(0), ldr, flags, bn, splits, stages, ws,
                               error_flag(), num_sms(), nullptr, 1, 0, cur_stream()),
             "gemm_bf16_pair");
    return;
  }
  check_rc(mb_gemm_bf16(x.data_ptr(), w.data_ptr(), y.data_ptr(), optptr(residual), M, N, K,
                        x.stride(0), w.stride(0), y.stride(0), ldr, flags, bn, splits, stages, ws,
                        error_flag(), num_sms(), cur_stream()),
           "gemm_bf16");
}

// Persistent stream-K variant. `ws` = (float workspace, int32 zeroed counters).
void gemm_bf16_persistent(const Tensor& x, const Tensor& w, Tensor& y,
                          const c10::optional<Tensor>& residual, bool dual, const Tensor& ws,
                          const Tensor& counters, int bn, int stages, int mode, bool pdl, bool packed) {
  need_cuda(x, "x"); need_cuda(w, "w"); need_cuda(y, "y");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && y.dim() == 2, "gemm: 2-D tensors expected");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16, "bf16 inputs");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1 && y.stride(1) == 1, "row-major operands");
  const int M = x.size(0), K = x.size(1);
  const int N = dual ? w.size(0) / 2 : w.size(0);
  TORCH_CHECK(w.size(1) == K && y.size(0) == M && y.size(1) == N, "gemm: shape mismatch");
  const bool f32 = y.scalar_type() == at::kFloat;
  const bool resid = residual.has_value() && residual->defined();
  TORCH_CHECK(static_cast<size_t>(ws.nbytes()) >= mb_gemm_persistent_workspace_bytes(num_sms()) &&
                  static_cast<size_t>(counters.numel()) >= mb_gemm_persistent_counter_ints(num_sms()) &&
                  counters.scalar_type() == at::kInt,
              "gemm: workspace too small");
  int flags = (dual ? 1 : 0) | (resid ? 2 : 0) | (f32 ? 4 : 0) | (pdl ? 8 : 0) | (packed ? 64 : 0);
  check_rc(mb_gemm_bf16_persistent(x.data_ptr(), w.data_ptr(), y.data_ptr(), optptr(residual), M, N, K,
                                   x.stride(0), w.stride(0), y.stride(0),
                                   resid ? residual->stride(0) : 0, flags, bn, stages, mode,
                                   ws.data_ptr(), counters.data_ptr<int>(), error_flag(), num_sms(),
                                   cur_stream()),
           "gemm_bf16_persistent");
}
py::tuple gemm_persistent_sizes() {
  return py::make_tuple(mb_gemm_persistent_workspace_bytes(num_sms()),
                        mb_gemm_persistent_counter_ints(num_sms()));
}

// Per-token-group (1 x 128) dynamic fp8 quantisation. q: [M, K] float8_e4m3fn; scales fp32
// [ceil(K/128), M] when k_major (the layout the fp8 GEMM reads) else [M, ceil(K/128)].
void quant_fp8_group128(const Tensor& x, Tensor& q, Tensor& scales, bool k_major) {
  need_cuda(x, "x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == at::kBFloat16, "x: bf16 [M, K]");
  TORCH_CHECK(q.is_contiguous() && q.element_size() == 1 && scales.scalar_type() == at::kFloat, "q / scales");
  check_rc(mb_quant_fp8_group128(x.data_ptr(), q.data_ptr(), scales.data_ptr<float>(), x.size(0),
                                 x.size(1), x.stride(0), 0, k_major ? 1 : 0, cur_stream()),
           "quant_fp8_group128");
}
// y = (xq * xs) @ (wq * ws).T with 128x128 weight blocks and 1x128 activation groups.
void gemm_fp8_blockscaled(const Tensor& xq, const Tensor& xs, const Tensor& wq, const Tensor& ws,
                          Tensor& y, const c10::optional<Tensor>& residual, int bn, int stages, int splits,
                          const c10::optional<Tensor>& workspace) {
  need_cuda(xq, "xq");
  TORCH_CHECK(xq.is_contiguous() && wq.is_contiguous() && y.is_contiguous() && xs.is_contiguous() &&
                  ws.is_contiguous() && xq.element_size() == 1 && wq.element_size() == 1 &&
                  y.scalar_type() == at::kBFloat16,
              "gemm_fp8: contiguous fp8 operands, bf16 output");
  const int M = xq.size(0), K = xq.size(1), N = wq.size(0);
  TORCH_CHECK(wq.size(1) == K && y.size(0) == M && y.size(1) == N, "gemm_fp8: shape mismatch");
  TORCH_CHECK(xs.numel() == static_cast<int64_t>((K + 127) / 128) * M &&
                  ws.numel() == static_cast<int64_t>((N + 127) / 128) * ((K + 127) / 128),
              "gemm_fp8: scale shapes");
  const bool resid = residual.has_value() && residual->defined();
  if (resid) TORCH_CHECK(residual->is_contiguous() && residual->scalar_type() == at::kBFloat16, "residual");
  const bool has_ws = workspace.has_value() && workspace->defined();
  if (has_ws) TORCH_CHECK(workspace->is_cuda() && workspace->is_contiguous(), "gemm_fp8: workspace");
  check_rc(mb_gemm_fp8_blockscaled(xq.data_ptr(), xs.data_ptr<float>(), wq.data_ptr(), ws.data_ptr<float>(),
                                   y.data_ptr(), optptr(residual), M, N, K, resid ? 2 : 0, bn, stages, splits,
                                   has_ws ? workspace->data_ptr() : nullptr,
                                   has_ws ? static_cast<size_t>(workspace->nbytes()) : 0, num_sms(),
                                   error_flag(), cur_stream()),
           "gemm_fp8_blockscaled");
}

// ---- mixture of experts
void moe_router_group_limited(const Tensor& logits, const c10::optional<Tensor>& bias, Tensor& ids,
                              Tensor& w, int n_group, int topk_group, bool norm_topk, double scaling) {
  need_cuda(logits, "logits");
  TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.stride(1) == 1 && ids.scalar_type() == at::kInt &&
                  w.scalar_type() == at::kFloat && ids.is_contiguous() && w.is_contiguous(),
              "router dtypes");
  check_rc(mb_moe_router_group_limited(logits.data_ptr<float>(), static_cast<const float*>(optptr(bias)),
                                       ids.data_ptr<int32_t>(), w.data_ptr<float>(), logits.size(0),
                                       logits.size(1), n_group, topk_group, ids.size(1), norm_topk, scaling,
                                       logits.stride(0), cur_stream()),
           "moe_router_group_limited");
}
void moe_router_softmax_topk(const Tensor& logits, Tensor& ids, Tensor& w, bool norm_topk) {
  need_cuda(logits, "logits");
  TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.stride(1) == 1 && ids.is_contiguous() && w.is_contiguous(), "router");
  check_rc(mb_moe_router_softmax_topk(logits.data_ptr<float>(), ids.data_ptr<int32_t>(), w.data_ptr<float>(),
                                      logits.size(0), logits.size(1), ids.size(1), norm_topk,
                                      logits.stride(0), cur_stream()),
           "moe_router_softmax_topk");
}
// scratch: int32 [2 * E_local] zeroed once (counts | cursor); offsets int32 [E_local + 1].
void moe_create_indices(const Tensor& ids, int e_begin, int e_end, Tensor& scratch, Tensor& offsets,
                        Tensor& order, Tensor& inverse) {
  need_cuda(ids, "topk_ids");
  const int E = e_end - e_begin;
  TORCH_CHECK(ids.is_contiguous() && ids.scalar_type() == at::kInt && scratch.numel() >= 2 * E &&
                  offsets.numel() >= E + 1 && order.numel() >= ids.numel() && inverse.numel() >= ids.numel(),
              "moe_create_indices buffers");
  check_rc(mb_moe_create_indices(ids.data_ptr<int32_t>(), ids.numel(), e_begin, e_end,
                                 scratch.data_ptr<int32_t>(), offsets.data_ptr<int32_t>(),
                                 scratch.data_ptr<int32_t>() + E, order.data_ptr<int32_t>(),
                                 inverse.data_ptr<int32_t>(), cur_stream()),
           "moe_create_indices");
}
void moe_permute_rows(const Tensor& src, const Tensor& order, const c10::optional<Tensor>& n_rows,
                      Tensor& dst, int top_k) {
  need_cuda(src, "src");
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous(), "contiguous");
  check_rc(mb_moe_permute_rows(src.data_ptr(), order.data_ptr<int32_t>(),
                               static_cast<const int32_t*>(optptr(n_rows)), dst.data_ptr(), dst.size(0),
                               src.size(1) * src.element_size(), top_k, cur_stream()),
           "moe_permute_rows");
}
void moe_combine(const Tensor& expert_out, const Tensor& inverse, const Tensor& w,
                 const c10::optional<Tensor>& shared, Tensor& y, int top_k) {
  need_cuda(expert_out, "expert_out");
  TORCH_CHECK(expert_out.is_contiguous() && y.is_contiguous() && w.is_contiguous(), "contiguous");
  check_rc(mb_moe_combine(expert_out.data_ptr(), inverse.data_ptr<int32_t>(), w.data_ptr<float>(),
                          optptr(shared), y.data_ptr(), y.size(0), y.size(1), top_k, cur_stream()),
           "moe_combine");
}
// x: [rows, K] tokens in expert order; w: [E, N or 2N, K]; offsets int32 [E + 1] on device.
void grouped_gemm_bf16(const Tensor& x, const Tensor& w, Tensor& y, const Tensor& offsets, int max_rows,
                       bool dual, int bn) {
  need_cuda(x, "x");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous() && y.is_contiguous() && w.dim() == 3, "grouped_gemm layout");
  const int E = w.size(0), K = w.size(2), N = dual ? w.size(1) / 2 : w.size(1);
  TORCH_CHECK(x.size(1) == K && y.size(1) == N && y.size(0) == x.size(0) && offsets.numel() >= E + 1, "grouped_gemm shapes");
  check_rc(mb_grouped_gemm_bf16(x.data_ptr(), w.data_ptr(), y.data_ptr(), offsets.data_ptr<int32_t>(), E,
                                x.size(0), max_rows, N, K, dual ? 1 : 0, bn, error_flag(), cur_stream()),
           "grouped_gemm_bf16");
}

py::tuple gemm_plan(int M, int N, int K, bool dual) {
  int bn, sp, st;
  mb_gemm_bf16_plan(M, N, K, dual, num_sms(), &bn, &sp, &st);
  return py::make_tuple(bn, sp, st);
}

void rmsnorm(const Tensor& x, const Tensor& w, Tensor& out, double eps, double w_off, bool mbc) {
  need_cuda(x, "x");
  check_rc(mb_rmsnorm(x.data_ptr(), w.data_ptr(), out.data_ptr(), x.size(0), x.size(1),
                      x.stride(0), out.stride(0), eps, w_off, mbc, cur_stream()),
           "rmsnorm");
}
void add_rmsnorm(const Tensor& x, Tensor& residual, const Tensor& w, Tensor& out, double eps,
                 double w_off, bool mbc) {
  need_cuda(x, "x");
  TORCH_CHECK(x.is_contiguous() && residual.is_contiguous() && out.is_contiguous(), "contiguous");
  check_rc(mb_add_rmsnorm(x.data_ptr(), residual.data_ptr(), w.data_ptr(), out.data_ptr(),
                          x.size(0), x.size(1), eps, w_off, mbc, cur_stream()),
           "add_rmsnorm");
}
void silu_mul(const Tensor& gu, Tensor& out) {
  need_cuda(gu, "gate_up");
  TORCH_CHECK(gu.is_contiguous() && out.is_contiguous(), "contiguous");
  check_rc(mb_silu_mul(gu.data_ptr(), out.data_ptr(), gu.size(0), gu.size(1) / 2, cur_stream()),
           "silu_mul");
}
void embedding(const Tensor& ids, const Tensor& table, Tensor& out, int vocab_start) {
  need_cuda(ids, "ids");
  TORCH_CHECK(ids.scalar_type() == at::kLong && table.is_contiguous() && out.is_contiguous(), "embedding");
  check_rc(mb_embedding(ids.data_ptr<int64_t>(), table.data_ptr(), out.data_ptr(), ids.numel(),
                        table.size(1), table.size(0), vocab_start, cur_stream()),
           "embedding");
}
void gather_rows(const Tensor& src, const Tensor& idx, Tensor& dst) {
  need_cuda(src, "src");
  TORCH_CHECK(idx.scalar_type() == at::kInt && dst.is_contiguous() && src.stride(1) == 1, "gather_rows");
  check_rc(mb_gather_rows(src.data_ptr(), idx.data_ptr<int32_t>(), dst.data_ptr(), idx.numel(),
                          src.size(1) * src.element_size(), src.stride(0) * src.element_size(),
                          cur_stream()),
           "gather_rows");
}

// k_cache / v_cache: views [pages, n_kv, page_size, head_dim] of one layer (any page stride).
void rope_kv_store(Tensor& qkv, const Tensor& positions, const Tensor& slots, const Tensor& cos_sin,
                   Tensor& k_cache, Tensor& v_cache, int n_q, int n_kv, int head_dim,
                   bool interleaved) {
  need_cuda(qkv, "qkv");
  TORCH_CHECK(qkv.is_contiguous() && positions.scalar_type() == at::kInt &&
                  slots.scalar_type() == at::kLong && cos_sin.scalar_type() == at::kFloat,
              "rope_kv_store: dtypes");
  TORCH_CHECK(k_cache.dim() == 4 && k_cache.stride(3) == 1 && k_cache.stride(2) == head_dim, "cache layout");
  TORCH_CHECK(v_cache.stride(0) == k_cache.stride(0) && v_cache.stride(1) == k_cache.stride(1), "k/v strides");
  check_rc(mb_rope_kv_store(qkv.data_ptr(), positions.data_ptr<int32_t>(), slots.data_ptr<int64_t>(),
                            cos_sin.data_ptr<float>(), k_cache.data_ptr(), v_cache.data_ptr(),
                            qkv.size(0), n_q, n_kv, head_dim, k_cache.size(2), k_cache.stride(0),
                            k_cache.stride(1), interleaved, cur_stream()),
           "rope_kv_store");
}

void paged_attention(const Tensor& q, Tensor& out, const Tensor& k_cache, const Tensor& v_cache,
                     const Tensor& block_table, const Tensor& q_start, const Tensor& q_len,
                     const Tensor& kv_len, const c10::optional<Tensor>& tile_seq,
                     const c10::optional<Tensor>& tile_q0, const c10::optional<Tensor>& decode_seq,
                     int n_q, int n_kv, int head_dim, double scale) {
  need_cuda(q, "q");
  TORCH_CHECK(q.dim() == 2 && out.dim() == 2 && q.stride(1) == 1 && out.stride(1) == 1, "q/out 2-D");
  TORCH_CHECK(block_table.scalar_type() == at::kInt && block_table.dim() == 2, "block_table int32 2-D");
  const int n_tiles = tile_seq.has_value() && tile_seq->defined() ? tile_seq->numel() : 0;
  const int n_dec = decode_seq.has_value() && decode_seq->defined() ? decode_seq->numel() : 0;
  check_rc(mb_paged_attention(
               q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), k_cache.data_ptr(),
               v_cache.data_ptr(), block_table.data_ptr<int32_t>(), block_table.stride(0),
               q_start.data_ptr<int32_t>(), q_len.data_ptr<int32_t>(), kv_len.data_ptr<int32_t>(),
               static_cast<const int32_t*>(optptr(tile_seq)),
               static_cast<const int32_t*>(optptr(tile_q0)), n_tiles, n_dec,
               static_cast<const int32_t*>(optptr(decode_seq)), n_q, n_kv, head_dim,
               k_cache.size(2), k_cache.stride(0), k_cache.stride(1), scale, cur_stream()),
           "paged_attention");
}

// TMA-fed attention over the whole cache tensor kv: [pages, 2, layers, n_kv, page_size, head_dim].
void paged_attention_tma(const Tensor& q, Tensor& out, const Tensor& kv, int layer,
                         const Tensor& block_table, const Tensor& q_start, const Tensor& q_len,
                         const Tensor& kv_len, const c10::optional<Tensor>& tile_seq,
                         const c10::optional<Tensor>& tile_q0, const c10::optional<Tensor>& decode_seq,
                         int n_q, int n_kv, int head_dim, double scale) {
  need_cuda(q, "q");
  TORCH_CHECK(kv.dim() == 6 && kv.is_contiguous() && kv.size(1) == 2 && kv.size(5) == head_dim,
              "kv must be the contiguous 6-D cache tensor");
  TORCH_CHECK(block_table.scalar_type() == at::kInt && block_table.dim() == 2, "block_table int32 2-D");
  const int n_tiles = tile_seq.has_value() && tile_seq->defined() ? tile_seq->numel() : 0;
  const int n_dec = decode_seq.has_value() && decode_seq->defined() ? decode_seq->numel() : 0;
  const long long hd = head_dim;
  check_rc(mb_paged_attention_tma(
               q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), kv.data_ptr(), kv.numel() / hd,
               layer * kv.stride(2) / hd, (layer * kv.stride(2) + kv.stride(1)) / hd, kv.stride(0) / hd,
               block_table.data_ptr<int32_t>(), block_table.stride(0), q_start.data_ptr<int32_t>(),
               q_len.data_ptr<int32_t>(), kv_len.data_ptr<int32_t>(),
               static_cast<const int32_t*>(optptr(tile_seq)), static_cast<const int32_t*>(optptr(tile_q0)),
               n_tiles, n_dec, static_cast<const int32_t*>(optptr(decode_seq)), n_q, n_kv, head_dim,
               kv.size(4), scale, error_flag(), cur_stream()),
           "paged_attention_tma");
}

void argmax(const Tensor& logits, Tensor& out) {
  need_cuda(logits, "logits");
  TORCH_CHECK(logits.scalar_type() == at::kFloat && out.scalar_type() == at::kLong, "argmax dtypes");
  check_rc(mb_argmax(logits.data_ptr<float>(), out.data_ptr<int64_t>(), logits.size(0),
                     logits.size(1), logits.stride(0), cur_stream()),
           "argmax");
}
void sample(const Tensor& logits, Tensor& out, const c10::optional<Tensor>& temperature,
            const c10::optional<Tensor>& top_k, const c10::optional<Tensor>& top_p,
            const c10::optional<Tensor>& min_p, const c10::optional<Tensor>& seeds, int64_t step) {
  need_cuda(logits, "logits");
  TORCH_CHECK(logits.scalar_type() == at::kFloat && out.scalar_type() == at::kLong, "sample dtypes");
  check_rc(mb_sample_topk_topp(logits.data_ptr<float>(), out.data_ptr<int64_t>(), logits.size(0),
                               logits.size(1), logits.stride(0),
                               static_cast<const float*>(optptr(temperature)),
                               static_cast<const int32_t*>(optptr(top_k)),
                               static_cast<const float*>(optptr(top_p)),
                               static_cast<const float*>(optptr(min_p)),
                               static_cast<const uint64_t*>(optptr(seeds)),
                               static_cast<uint64_t>(step), cur_stream()),
           "sample");
}
void qk_norm(Tensor& qkv, const Tensor& q_w, const Tensor& k_w, int n_q, int n_kv, int head_dim, double eps) {
  need_cuda(qkv, "qkv");
  TORCH_CHECK(qkv.scalar_type() == at::kBFloat16 && qkv.dim() == 2 && qkv.stride(1) == 1 &&
                  qkv.size(1) >= static_cast<int64_t>(n_q + n_kv) * head_dim && q_w.numel() == head_dim &&
                  k_w.numel() == head_dim && q_w.scalar_type() == at::kBFloat16 && k_w.scalar_type() == at::kBFloat16,
              "qk_norm: bf16 [T, >= (n_q + n_kv) * head_dim] projection and two [head_dim] weights expected");
  check_rc(mb_qk_norm(qkv.data_ptr(), q_w.data_ptr(), k_w.data_ptr(), qkv.size(0), n_q, n_kv, head_dim, qkv.stride(0),
                      static_cast<float>(eps), cur_stream()),
           "qk_norm");
}
void apply_penalties(Tensor& logits, const Tensor& tok, const Tensor& cnt, const Tensor& offsets,
                     const c10::optional<Tensor>& freq, const c10::optional<Tensor>& pres,
                     const c10::optional<Tensor>& rep) {
  need_cuda(logits, "logits");
  check_rc(mb_apply_penalties(logits.data_ptr<float>(), logits.size(0), logits.size(1),
                              logits.stride(0), tok.data_ptr<int32_t>(), cnt.data_ptr<int32_t>(),
                              offsets.data_ptr<int32_t>(), static_cast<const float*>(optptr(freq)),
                              static_cast<const float*>(optptr(pres)),
                              static_cast<const float*>(optptr(rep)), cur_stream()),
           "apply_penalties");
}

// ------------------------------------------------------------------ executor wrapper
class PyDecoderExecutor {
 public:
  mb::DecoderExecutor ex;
  std::vector<Tensor> keep;  // keeps every tensor whose pointer the executor holds alive

  PyDecoderExecutor(py::dict cfg) {
    auto& c = ex.cfg;
    c.n_layers = cfg["n_layers"].cast<int>();
    c.hidden = cfg["hidden"].cast<int>();
    c.n_q = cfg["n_q"].cast<int>();
    c.n_kv = cfg["n_kv"].cast<int>();
    c.head_dim = cfg["head_dim"].cast<int>();
    c.inter = cfg["inter"].cast<int>();
    c.vocab = cfg["vocab"].cast<int>();
    c.eps = cfg["eps"].cast<float>();
    c.norm_weight_offset = cfg.contains("norm_weight_offset") ? cfg["norm_weight_offset"].cast<float>() : 0.f;
    c.multiply_before_cast = cfg.contains("multiply_before_cast") ? cfg["multiply_before_cast"].cast<int>() : 0;
    c.rope_interleaved = cfg.contains("rope_interleaved") ? cfg["rope_interleaved"].cast<int>() : 0;
    c.page_size = cfg["page_size"].cast<int>();
    c.attn_scale = cfg["attn_scale"].cast<float>();
    c.logits_scale = 1.f;
    c.fuse_swiglu = cfg.contains("fuse_swiglu") ? cfg["fuse_swiglu"].cast<int>() : 1;
    c.gemm_impl = cfg.contains("gemm_impl") ? cfg["gemm_impl"].cast<int>() : 0;
    c.use_pdl = cfg.contains("use_pdl") ? cfg["use_pdl"].cast<int>() : 0;
    c.attn_impl = cfg.contains("attn_impl") ? cfg["attn_impl"].cast<int>() : 1;
    c.dec_max_tokens = cfg.contains("dec_max_tokens") ? cfg["dec_max_tokens"].cast<int>() : 0;
    if (c.dec_max_tokens > mb_gemm_dec_max_tokens()) c.dec_max_tokens = mb_gemm_dec_max_tokens();
    c.prefetch_weights = cfg.contains("prefetch_weights") ? cfg["prefetch_weights"].cast<int>() : 0;
    ex.buf.p_ws = nullptr;
    ex.buf.p_counters = nullptr;
    c.num_sms = num_sms();
    ex.buf.err = error_flag();
  }
  const void* hold(const Tensor& t) {
    TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "executor tensors must be contiguous CUDA tensors");
    keep.push_back(t);
    return t.data_ptr();
  }
  void set_globals(const Tensor& embed, const Tensor& final_norm, const Tensor& lm_head,
                   const Tensor& cos_sin) {
    ex.embed = hold(embed);
    ex.final_norm = hold(final_norm);
    ex.lm_head = hold(lm_head);
    ex.cos_sin = static_cast<const float*>(hold(cos_sin));
  }
  // scales: the four block-scale tensors of an fp8 layer (all or none)
  void add_layer(const Tensor& attn_norm, const Tensor& wqkv, const Tensor& wo,
                 const Tensor& mlp_norm, const Tensor& wgu, const Tensor& wd,
                 const c10::optional<std::vector<Tensor>>& scales, const c10::optional<Tensor>& qkv_bias,
                 const c10::optional<Tensor>& q_norm, const c10::optional<Tensor>& k_norm) {
    mb::DecoderLayerWeights w;
    if (q_norm.has_value() && q_norm->defined()) {
      TORCH_CHECK(k_norm.has_value() && k_norm->defined() && q_norm->scalar_type() == at::kBFloat16 &&
                      k_norm->scalar_type() == at::kBFloat16 && q_norm->dim() == 1 && k_norm->dim() == 1 &&
                      q_norm->size(0) == ex.cfg.head_dim && k_norm->size(0) == ex.cfg.head_dim &&
                      q_norm->is_contiguous() && k_norm->is_contiguous(),
                  "add_layer: q_norm / k_norm must be contiguous bf16 vectors of head_dim entries");
      w.q_norm = hold(*q_norm);
      w.k_norm = hold(*k_norm);
    }
    if (qkv_bias.has_value() && qkv_bias->defined()) {
      TORCH_CHECK(qkv_bias->scalar_type() == at::kBFloat16 && qkv_bias->dim() == 1 &&
                      qkv_bias->size(0) == wqkv.size(0) && qkv_bias->is_contiguous(),
                  "add_layer: qkv_bias must be a contiguous bf16 vector with one entry per row of wqkv");
      w.qkv_bias = hold(*qkv_bias);
    }
    w.attn_norm = hold(attn_norm); w.wqkv = hold(wqkv); w.wo = hold(wo);
    w.mlp_norm = hold(mlp_norm); w.wgu = hold(wgu); w.wd = hold(wd);
    if (scales.has_value()) {
      TORCH_CHECK(scales->size() == 4, "add_layer: four scale tensors (qkv, o, gate_up, down) expected");
      const Tensor* ws[4] = {&wqkv, &wo, &wgu, &wd};
      const float* ptr[4];
      for (int i = 0; i < 4; ++i) {
        const Tensor& s = (*scales)[i];
        TORCH_CHECK(s.scalar_type() == at::kFloat && s.dim() == 2 && ws[i]->element_size() == 1 &&
                        s.size(0) == (ws[i]->size(0) + 127) / 128 && s.size(1) == (ws[i]->size(1) + 127) / 128,
                    "add_layer: scales must be fp32 [ceil(N/128), ceil(K/128)] of an 8-bit weight");
        ptr[i] = static_cast<const float*>(hold(s));
      }
      w.wqkv_s = ptr[0]; w.wo_s = ptr[1]; w.wgu_s = ptr[2]; w.wd_s = ptr[3];
    }
    ex.layers.push_back(w);
  }
  void set_fp8_buffers(const Tensor& xq, const Tensor& xs, const Tensor& gu) {
    ex.buf.xq = const_cast<void*>(hold(xq));
    TORCH_CHECK(xs.scalar_type() == at::kFloat, "xs must be fp32");
    ex.buf.xs = static_cast<float*>(const_cast<void*>(hold(xs)));
    ex.buf.gu = const_cast<void*>(hold(gu));
  }
  // kv: [pages, 2, n_layers, n_kv, page_size, head_dim]
  void set_kv_cache(const Tensor& kv) {
    TORCH_CHECK(kv.dim() == 6 && kv.is_contiguous(), "kv cache must be 6-D contiguous");
    ex.kv.base = const_cast<void*>(hold(kv));
    ex.kv.page_stride = kv.stride(0);
    ex.kv.kv_stride = kv.stride(1);
    ex.kv.layer_stride = kv.stride(2);
    ex.kv.head_stride = kv.stride(3);
    ex.kv.total_elems = kv.numel();
  }
  void set_buffers(const Tensor& h, const Tensor& xn, const Tensor& qkv, const Tensor& attn,
                   const Tensor& act, const c10::optional<Tensor>& gu, const Tensor& last_h,
                   const Tensor& last_xn, const Tensor& logits, const Tensor& sampled,
                   const Tensor& workspace, const c10::optional<Tensor>& p_ws,
                   const c10::optional<Tensor>& p_counters) {
    auto& b = ex.buf;
    b.h = const_cast<void*>(hold(h)); b.xn = const_cast<void*>(hold(xn));
    b.qkv = const_cast<void*>(hold(qkv)); b.attn = const_cast<void*>(hold(attn));
    b.act = const_cast<void*>(hold(act));
    b.gu = gu.has_value() && gu->defined() ? const_cast<void*>(hold(*gu)) : nullptr;
    b.last_h = const_cast<void*>(hold(last_h)); b.last_xn = const_cast<void*>(hold(last_xn));
    b.logits = static_cast<float*>(const_cast<void*>(hold(logits)));
    TORCH_CHECK(sampled.scalar_type() == at::kLong, "sampled must be int64");
    b.sampled = static_cast<int64_t*>(const_cast<void*>(hold(sampled)));
    b.workspace = const_cast<void*>(hold(workspace));
    b.workspace_bytes = workspace.nbytes();
    if (p_ws.has_value() && p_ws->defined() && p_counters.has_value() && p_counters->defined()) {
      TORCH_CHECK(static_cast<size_t>(p_ws->nbytes()) >= mb_gemm_persistent_workspace_bytes(num_sms()) &&
                      static_cast<size_t>(p_counters->numel()) >= mb_gemm_persistent_counter_ints(num_sms()),
                  "persistent GEMM workspace too small");
      b.p_ws = const_cast<void*>(hold(*p_ws));
      b.p_counters = static_cast<int*>(const_cast<void*>(hold(*p_counters)));
    }
  }
  // meta: one int32 device tensor holding every per-step array; offsets are in int32 units
  // (tokens and slots are int64 and 8-byte aligned inside it).
  void forward(const Tensor& meta, py::dict off, int T, int B, int bt_stride, int n_tiles,
               int n_decode, int n_logits, bool has_future, bool do_sample, int64_t sample_step) {
    const int32_t* base = meta.data_ptr<int32_t>();
    auto at32 = [&](const char* k) { return base + off[k].cast<int64_t>(); };
    mb::StepInputs in;
    in.tokens = reinterpret_cast<const int64_t*>(at32("tokens"));
    in.slots = reinterpret_cast<const int64_t*>(at32("slots"));
    in.positions = at32("positions");
    in.block_table = at32("block_table");
    in.q_start = at32("q_start"); in.q_len = at32("q_len"); in.kv_len = at32("kv_len");
    in.tile_seq = at32("tile_seq"); in.tile_q0 = at32("tile_q0");
    in.decode_seq = at32("decode_seq"); in.logit_rows = at32("logit_rows");
    in.T = T; in.B = B; in.bt_stride = bt_stride; in.n_tiles = n_tiles; in.n_decode = n_decode;
    in.n_logits = n_logits;
    in.future_src = has_future ? at32("future_src") : nullptr;
    in.temperature = reinterpret_cast<const float*>(at32("temperature"));
    in.top_k = at32("top_k");
    in.top_p = reinterpret_cast<const float*>(at32("top_p"));
    in.min_p = reinterpret_cast<const float*>(at32("min_p"));
    in.seeds = reinterpret_cast<const uint64_t*>(at32("seeds"));
    in.sample_step = static_cast<uint64_t>(sample_step);
    in.do_sample = do_sample ? 1 : 0;
    check_rc(ex.forward(in, cur_stream()), "DecoderExecutor.forward");
  }
  // peer pointers are integers (device addresses valid in this process: symmetric memory)
  void set_tp(int world, int rank, const std::vector<int64_t>& partial, const std::vector<int64_t>& xn,
              const std::vector<int64_t>& logits, const std::vector<int64_t>& flags, const Tensor& h_local,
              const Tensor& logits_local, int vocab_local, int fused, int64_t partial_rows) {
    TORCH_CHECK(world >= 1 && world <= 8 && static_cast<int>(partial.size()) == world &&
                    static_cast<int>(xn.size()) == world && static_cast<int>(logits.size()) == world &&
                    static_cast<int>(flags.size()) == world,
                "set_tp: one pointer per rank expected");
    ex.tp.world = world;
    ex.tp.rank = rank;
    for (int i = 0; i < world; ++i) {
      ex.tp.partial[i] = reinterpret_cast<void*>(partial[i]);
      ex.tp.xn[i] = reinterpret_cast<void*>(xn[i]);
      ex.tp.logits[i] = reinterpret_cast<void*>(logits[i]);
      ex.tp.flags[i] = reinterpret_cast<int*>(flags[i]);
    }
    ex.tp.h_local = const_cast<void*>(hold(h_local));
    ex.tp.logits_local = static_cast<float*>(const_cast<void*>(hold(logits_local)));
    ex.tp.vocab_local = vocab_local;
    ex.tp.fused = fused;
    ex.tp.partial_rows = partial_rows;
  }
  // workspace (fp32) and zeroed state words of the decode-step GEMMs
  void set_dec(const Tensor& ws, const Tensor& state) {
    TORCH_CHECK(state.scalar_type() == at::kInt && state.numel() >= mb_gemm_dec_state_ints(), "dec state too small");
    ex.buf.dec_ws = const_cast<void*>(hold(ws));
    ex.buf.dec_ws_bytes = ws.nbytes();
    ex.buf.dec_state = static_cast<int*>(const_cast<void*>(hold(state)));
  }
  // receive buffers of the fused all-reduce on every rank (symmetric memory, filled with bf16 -0.0)
  void set_tp_lamport(const std::vector<int64_t>& lam, int lam_rows) {
    TORCH_CHECK(static_cast<int>(lam.size()) == ex.tp.world, "set_tp_lamport: one pointer per rank expected");
    for (int i = 0; i < ex.tp.world; ++i) ex.tp.lam[i] = reinterpret_cast<void*>(lam[i]);
    ex.tp.lam_rows = lam_rows;
  }
  bool dec_usable(int T) const { return ex.dec_usable(T); }
  long launches() const { return ex.launches; }
  void set_profiling(bool on) { ex.profiling = on; }
  py::list profile() {
    py::list out;
    for (auto& e : ex.profile_ms()) out.append(py::make_tuple(std::get<0>(e), std::get<1>(e), std::get<2>(e)));
    return out;
  }
};

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "modular_b200 native kernels and runtime (sm_100a)";
  m.def("gemm_bf16", &gemm_bf16, py::arg("x"), py::arg("w"), py::arg("y"),
        py::arg("residual") = py::none(), py::arg("dual") = false,
        py::arg("workspace") = py::none(), py::arg("bn") = 0, py::arg("splits") = 0,
        py::arg("stages") = 0, py::arg("packed") = false, py::arg("pair") = false);
  m.def("gemm_plan", &gemm_plan);
  m.def("moe_router_group_limited", &moe_router_group_limited);
  m.def("moe_router_softmax_topk", &moe_router_softmax_topk);
  m.def("moe_create_indices", &moe_create_indices);
  m.def("moe_permute_rows", &moe_permute_rows);
  m.def("moe_combine", &moe_combine);
  m.def("grouped_gemm_bf16", &grouped_gemm_bf16);
  m.def("quant_fp8_group128", &quant_fp8_group128);
  m.def("gemm_fp8_blockscaled", &gemm_fp8_blockscaled, py::arg("xq"), py::arg("xs"), py::arg("wq"),
        py::arg("ws"), py::arg("y"), py::arg("residual") = py::none(), py::arg("bn") = 0,
        py::arg("stages") = 0, py::arg("splits") = 0, py::arg("workspace") = py::none());
  m.def("gemm_bf16_persistent", &gemm_bf16_persistent, py::arg("x"), py::arg("w"), py::arg("y"),
        py::arg("residual") = py::none(), py::arg("dual") = false, py::arg("ws"), py::arg("counters"),
        py::arg("bn") = 0, py::arg("stages") = 0, py::arg("mode") = -1, py::arg("pdl") = false,
        py::arg("packed") = false);
  m.def("gemm_persistent_sizes", &gemm_persistent_sizes);
  // QKV projection + rotary embedding + KV-cache store of a decode step in one launch (head_dim 128, rotate-half)
  m.def("gemm_dec_qkv_rope", [](const Tensor& x, const Tensor& w, Tensor& qkv, const Tensor& positions,
                                const Tensor& slots, const Tensor& cos_sin, Tensor& k_cache, Tensor& v_cache, int n_q,
                                int n_kv, Tensor& ws, Tensor& state) {
    need_cuda(x, "x");
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1 && qkv.stride(1) == 1 &&
                    x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 && qkv.scalar_type() == at::kBFloat16 &&
                    positions.scalar_type() == at::kInt && slots.scalar_type() == at::kLong &&
                    cos_sin.scalar_type() == at::kFloat && cos_sin.is_contiguous() && cos_sin.size(1) == 128 &&
                    w.size(0) == (n_q + 2 * n_kv) * 128 && qkv.size(1) == w.size(0) && qkv.size(0) >= x.size(0) &&
                    positions.numel() >= x.size(0) && slots.numel() >= x.size(0),
                "gemm_dec_qkv_rope: operands");
    TORCH_CHECK(k_cache.dim() == 4 && k_cache.stride(3) == 1 && k_cache.stride(2) == 128 && k_cache.size(3) == 128 &&
                    v_cache.stride(0) == k_cache.stride(0) && v_cache.stride(1) == k_cache.stride(1) &&
                    state.scalar_type() == at::kInt && state.numel() >= mb_gemm_dec_state_ints(),
                "gemm_dec_qkv_rope: cache layout / state");
    check_rc(mb_gemm_dec_qkv_rope(x.data_ptr(), w.data_ptr(), x.size(0), x.size(1), x.stride(0), w.stride(0),
                                  qkv.data_ptr(), qkv.stride(0), positions.data_ptr<int32_t>(), slots.data_ptr<int64_t>(),
                                  cos_sin.data_ptr<float>(), k_cache.data_ptr(), v_cache.data_ptr(), n_q, n_kv, 128,
                                  k_cache.size(2), k_cache.stride(0), k_cache.stride(1), ws.data_ptr(), ws.nbytes(),
                                  state.data_ptr<int>(), error_flag(), num_sms(), cur_stream()),
             "gemm_dec_qkv_rope");
  });
  m.def("set_gemm_dec_rope", [](bool on) { mb_set_gemm_dec_rope(on ? 1 : 0); }, py::arg("on"));
  m.def("set_sample_cluster", [](bool on) { mb_set_sample_cluster(on ? 1 : 0); }, py::arg("on"));
  m.def("set_gemm_dec_tile_epilogue", [](bool on) { mb_set_gemm_dec_tile_epilogue(on ? 1 : 0); }, py::arg("on"));
  m.def("gemm_dec_sizes", []() {
    return py::make_tuple(static_cast<int64_t>(mb_gemm_dec_workspace_bytes(num_sms())), mb_gemm_dec_state_ints(),
                          mb_gemm_dec_max_tokens());
  });
  m.def("gemm_dec_lamport_elems", [](int world, int rows, int N) {
    return static_cast<int64_t>(mb_gemm_dec_lamport_elems(world, rows, N));
  });
  m.def("set_gemm_dec_smem_kb", [](int kb) { mb_set_gemm_dec_smem_kb(kb); });
  m.def("set_gemm_dec_trace", [](const c10::optional<Tensor>& buf) {
    TORCH_CHECK(!buf.has_value() || (buf->is_cuda() && buf->nbytes() >= static_cast<size_t>(num_sms()) * 64), "trace buffer");
    mb_set_gemm_dec_trace(buf.has_value() ? buf->data_ptr() : nullptr);
  });
  m.def("gemm_dec_plan", [](int M, int N, int K, int mode, int64_t ws_bytes) {
    return mb_gemm_dec_plan(M, N, K, mode, static_cast<size_t>(ws_bytes), num_sms()) == MB_OK;
  });
  // Decode-step GEMM; see mb_gemm_dec. mode 0/1: `y` is the output; mode 2: `h` (in place) and `xn`.
  m.def("gemm_dec", [](const Tensor& x, const Tensor& w, int mode, const c10::optional<Tensor>& y,
                       const c10::optional<Tensor>& h, const c10::optional<Tensor>& xn,
                       const c10::optional<Tensor>& gamma, double eps, double w_off, bool mbc, int world, int rank,
                       const std::vector<int64_t>& lam, int lam_rows, const Tensor& ws, Tensor& state,
                       const c10::optional<Tensor>& w_scale, int w_format, const c10::optional<Tensor>& w_block_scale,
                       const c10::optional<Tensor>& w_global_scale) {
    need_cuda(x, "x"); need_cuda(w, "w");
    TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.stride(1) == 1 && w.stride(1) == 1, "gemm_dec: row-major 2-D operands");
    if (w_format == 2 || w_format == 3) {
      // weight-only NVFP4 (w: [N, K / 2] bytes) or MXFP8 (w: [N, K] e4m3) with per-block scale bytes
      const int M = x.size(0), K = x.size(1), N = w.size(0);
      TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.element_size() == 1 && w.is_contiguous() &&
                      w.size(1) == (w_format == 2 ? K / 2 : K) && w_block_scale && w_block_scale->is_contiguous() &&
                      w_block_scale->element_size() == 1 && w_block_scale->numel() == static_cast<int64_t>(N) * (K / (w_format == 2 ? 16 : 32)) &&
                      (w_format == 3 || (w_global_scale && w_global_scale->scalar_type() == at::kFloat && w_global_scale->is_cuda())),
                  "gemm_dec: quantised weight layout");
      TORCH_CHECK(state.scalar_type() == at::kInt && state.numel() >= mb_gemm_dec_state_ints(), "gemm_dec: state");
      void* yp = nullptr;
      int ldy = 0;
      if (mode == 2) {
        TORCH_CHECK(h.has_value() && xn.has_value() && gamma.has_value() && h->is_contiguous() && xn->is_contiguous() &&
                        h->size(1) == N && xn->size(1) == N && gamma->numel() == N, "gemm_dec mode 2: h / xn / gamma");
      } else {
        TORCH_CHECK(y.has_value() && y->stride(1) == 1 && y->size(0) >= M && y->size(1) == (mode == 1 ? N / 2 : N) &&
                        y->scalar_type() == at::kBFloat16, "gemm_dec: output shape");
        yp = y->data_ptr();
        ldy = y->stride(0);
      }
      void* lamq[8] = {};
      for (size_t i = 0; i < lam.size() && i < 8; ++i) lamq[i] = reinterpret_cast<void*>(lam[i]);
      check_rc(mb_gemm_dec_wq(w_format, x.data_ptr(), w.data_ptr(), w_block_scale->data_ptr(),
                              w_global_scale ? w_global_scale->data_ptr<float>() : nullptr, M, N, K, x.stride(0), mode, yp, ldy,
                              const_cast<void*>(optptr(h)), const_cast<void*>(optptr(xn)), optptr(gamma),
                              static_cast<float>(eps), static_cast<float>(w_off), mbc ? 1 : 0, world, rank, lamq, lam_rows,
                              ws.data_ptr(), ws.nbytes(), state.data_ptr<int>(), error_flag(), num_sms(), cur_stream()),
               "gemm_dec_wq");
      return;
    }
    // w_scale: block-scaled fp8 weights (e4m3 [N, K] contiguous, fp32 scales [N / 128, K / 128]); activations stay bf16
    TORCH_CHECK(x.scalar_type() == at::kBFloat16 &&
                    (w_scale ? (w.element_size() == 1 && w.is_contiguous() && w_scale->is_contiguous() &&
                                w_scale->scalar_type() == at::kFloat &&
                                w_scale->numel() == (w.size(0) / 128) * ((w.size(1) + 127) / 128))
                             : w.scalar_type() == at::kBFloat16),
                "gemm_dec: bf16 activations; bf16 weights or e4m3 weights with block scales");
    const int M = x.size(0), K = x.size(1), N = w.size(0);
    TORCH_CHECK(w.size(1) == K, "gemm_dec: shape mismatch");
    TORCH_CHECK(state.scalar_type() == at::kInt && state.numel() >= mb_gemm_dec_state_ints(), "gemm_dec: state");
    void* yp = nullptr;
    int ldy = 0;
    if (mode == 2) {
      TORCH_CHECK(h.has_value() && xn.has_value() && gamma.has_value(), "gemm_dec mode 2 needs h, xn, gamma");
      TORCH_CHECK(h->is_contiguous() && xn->is_contiguous() && h->size(0) >= M && h->size(1) == N &&
                      xn->size(0) >= M && xn->size(1) == N && gamma->numel() == N,
                  "gemm_dec mode 2: h / xn must be contiguous [>=M, N]");
      TORCH_CHECK(world == 1 || static_cast<int>(lam.size()) == world, "gemm_dec: one receive buffer per rank");
    } else {
      TORCH_CHECK(y.has_value() && y->stride(1) == 1 && y->size(0) >= M && y->size(1) == (mode == 1 ? N / 2 : N) &&
                      y->scalar_type() == at::kBFloat16,
                  "gemm_dec: output shape");
      yp = y->data_ptr();
      ldy = y->stride(0);
    }
    void* lamp[8] = {};
    for (size_t i = 0; i < lam.size() && i < 8; ++i) lamp[i] = reinterpret_cast<void*>(lam[i]);
    if (w_scale) {
      check_rc(mb_gemm_dec_w8(x.data_ptr(), w.data_ptr(), w_scale->data_ptr<float>(), M, N, K, x.stride(0), mode, yp, ldy,
                              const_cast<void*>(optptr(h)), const_cast<void*>(optptr(xn)), optptr(gamma),
                              static_cast<float>(eps), static_cast<float>(w_off), mbc ? 1 : 0, world, rank, lamp,
                              lam_rows, ws.data_ptr(), ws.nbytes(), state.data_ptr<int>(), error_flag(), num_sms(),
                              cur_stream()),
               "gemm_dec_w8");
      return;
    }
    check_rc(mb_gemm_dec(x.data_ptr(), w.data_ptr(), M, N, K, x.stride(0), w.stride(0), mode, yp, ldy,
                         const_cast<void*>(optptr(h)), const_cast<void*>(optptr(xn)), optptr(gamma),
                         static_cast<float>(eps), static_cast<float>(w_off), mbc ? 1 : 0, world, rank, lamp, lam_rows,
                         ws.data_ptr(), ws.nbytes(), state.data_ptr<int>(), error_flag(), num_sms(), cur_stream()),
             "gemm_dec");
  }, py::arg("x"), py::arg("w"), py::arg("mode"), py::arg("y"), py::arg("h"), py::arg("xn"), py::arg("gamma"),
     py::arg("eps"), py::arg("w_off"), py::arg("mbc"), py::arg("world"), py::arg("rank"), py::arg("lam"),
     py::arg("lam_rows"), py::arg("ws"), py::arg("state"), py::arg("w_scale") = py::none(), py::arg("w_format") = 0,
     py::arg("w_block_scale") = py::none(), py::arg("w_global_scale") = py::none());
  m.def("rmsnorm", &rmsnorm);
  m.def("add_rmsnorm", &add_rmsnorm);
  m.def("silu_mul", &silu_mul);
  m.def("embedding", &embedding);
  m.def("gather_rows", &gather_rows);
  m.def("rope_kv_store", &rope_kv_store);
  m.def("paged_attention", &paged_attention);
  m.def("paged_attention_tma", &paged_attention_tma);
  m.def("argmax", &argmax);
  m.def("sample", &sample);
  m.def("apply_penalties", &apply_penalties);
  // state-space layers
  m.def("causal_conv1d_varlen", [](const Tensor& x, const Tensor& w, const c10::optional<Tensor>& bias, Tensor& y,
                                   const c10::optional<Tensor>& conv_state, const Tensor& cu_seqlens,
                                   const c10::optional<Tensor>& state_idx, const c10::optional<Tensor>& has_init,
                                   bool silu) {
    need_cuda(x, "x");
    TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && y.stride(1) == 1 && x.scalar_type() == at::kBFloat16 &&
                    w.is_contiguous() && w.scalar_type() == at::kBFloat16 && w.size(0) == x.size(1),
                "causal_conv1d: x [T, D] bf16, w [D, W] bf16");
    TORCH_CHECK(cu_seqlens.scalar_type() == at::kInt, "cu_seqlens int32");
    check_rc(mb_causal_conv1d_varlen(x.data_ptr(), w.data_ptr(), optptr(bias), y.data_ptr(),
                                     conv_state.has_value() ? conv_state->data_ptr<float>() : nullptr,
                                     cu_seqlens.data_ptr<int>(),
                                     state_idx.has_value() ? state_idx->data_ptr<int>() : nullptr,
                                     has_init.has_value() ? has_init->data_ptr<int>() : nullptr,
                                     cu_seqlens.numel() - 1, x.size(1), w.size(1), x.stride(0), y.stride(0),
                                     silu ? 1 : 0, cur_stream()),
             "causal_conv1d_varlen");
  });
  m.def("selective_scan_varlen", [](const Tensor& u, const Tensor& delta, const Tensor& A, const Tensor& B,
                                    const Tensor& C, const c10::optional<Tensor>& D, const c10::optional<Tensor>& z,
                                    const c10::optional<Tensor>& dt_bias, Tensor& y,
                                    const c10::optional<Tensor>& ssm_state, const Tensor& cu_seqlens,
                                    const c10::optional<Tensor>& state_idx, const c10::optional<Tensor>& has_init,
                                    bool dt_softplus) {
    need_cuda(u, "u");
    TORCH_CHECK(u.is_contiguous() && delta.is_contiguous() && y.is_contiguous() && B.is_contiguous() &&
                    C.is_contiguous() && A.is_contiguous() && A.scalar_type() == at::kFloat &&
                    u.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16,
                "selective_scan: contiguous bf16 u/delta/B/C, fp32 A");
    TORCH_CHECK(!z.has_value() || z->is_contiguous(), "selective_scan: z contiguous");
    check_rc(mb_selective_scan_varlen(u.data_ptr(), delta.data_ptr(), A.data_ptr<float>(), B.data_ptr(),
                                      C.data_ptr(), D.has_value() ? D->data_ptr<float>() : nullptr, optptr(z),
                                      dt_bias.has_value() ? dt_bias->data_ptr<float>() : nullptr, y.data_ptr(),
                                      ssm_state.has_value() ? ssm_state->data_ptr<float>() : nullptr,
                                      cu_seqlens.data_ptr<int>(),
                                      state_idx.has_value() ? state_idx->data_ptr<int>() : nullptr,
                                      has_init.has_value() ? has_init->data_ptr<int>() : nullptr,
                                      cu_seqlens.numel() - 1, u.size(1), A.size(1), u.size(1), B.size(1),
                                      dt_softplus ? 1 : 0, cur_stream()),
             "selective_scan_varlen");
  });
  m.def("ssd_scan_varlen", [](const Tensor& x, const Tensor& dt, const Tensor& A, const Tensor& B, const Tensor& C,
                              const c10::optional<Tensor>& D, const c10::optional<Tensor>& dt_bias, Tensor& y,
                              const c10::optional<Tensor>& ssm_state, const Tensor& cu_seqlens,
                              const c10::optional<Tensor>& state_idx, const c10::optional<Tensor>& has_init,
                              bool dt_softplus) {
    need_cuda(x, "x");
    TORCH_CHECK(x.dim() == 3 && x.is_contiguous() && dt.is_contiguous() && B.dim() == 3 && B.is_contiguous() &&
                    C.is_contiguous() && y.is_contiguous() && A.scalar_type() == at::kFloat &&
                    x.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16,
                "ssd_scan: x [T, H, P], dt [T, H], B/C [T, G, N] contiguous bf16, A fp32 [H]");
    check_rc(mb_ssd_scan_varlen(x.data_ptr(), dt.data_ptr(), A.data_ptr<float>(), B.data_ptr(), C.data_ptr(),
                                D.has_value() ? D->data_ptr<float>() : nullptr,
                                dt_bias.has_value() ? dt_bias->data_ptr<float>() : nullptr, y.data_ptr(),
                                ssm_state.has_value() ? ssm_state->data_ptr<float>() : nullptr,
                                cu_seqlens.data_ptr<int>(),
                                state_idx.has_value() ? state_idx->data_ptr<int>() : nullptr,
                                has_init.has_value() ? has_init->data_ptr<int>() : nullptr,
                                cu_seqlens.numel() - 1, x.size(1), x.size(2), B.size(2), B.size(1),
                                dt_softplus ? 1 : 0, cur_stream()),
             "ssd_scan_varlen");
  });
  // grouped block-scaled fp8 GEMM: xq [rows, K] e4m3 (tokens in expert order), xs fp32 [ceil(K/128), rows],
  // wq [E, N, K] e4m3, ws fp32 [E, N/128, ceil(K/128)], offsets int32 [E + 1]
  m.def("grouped_gemm_fp8", [](const Tensor& xq, const Tensor& xs, const Tensor& wq, const Tensor& ws, Tensor& y,
                               const Tensor& offsets, int max_rows, int bn) {
    need_cuda(xq, "xq");
    TORCH_CHECK(xq.dim() == 2 && wq.dim() == 3 && xq.stride(1) == 1 && wq.is_contiguous() && xs.is_contiguous() &&
                    ws.is_contiguous() && y.is_contiguous() && xq.element_size() == 1 && wq.element_size() == 1 &&
                    y.scalar_type() == at::kBFloat16 && offsets.scalar_type() == at::kInt,
                "grouped_gemm_fp8: contiguous fp8 operands, bf16 output, int32 offsets");
    const int rows = xq.size(0), K = xq.size(1), E = wq.size(0), N = wq.size(1);
    TORCH_CHECK(wq.size(2) == K && y.size(0) == rows && y.size(1) == N && offsets.numel() >= E + 1,
                "grouped_gemm_fp8: shape mismatch");
    TORCH_CHECK(xs.numel() == static_cast<int64_t>((K + 127) / 128) * rows &&
                    ws.numel() == static_cast<int64_t>(E) * (N / 128) * ((K + 127) / 128),
                "grouped_gemm_fp8: scale shapes");
    check_rc(mb_grouped_gemm_fp8_blockscaled(xq.data_ptr(), xs.data_ptr<float>(), wq.data_ptr(),
                                             ws.data_ptr<float>(), y.data_ptr(), offsets.data_ptr<int>(), E, rows,
                                             max_rows, N, K, static_cast<int>(xq.stride(0)), bn, 0, error_flag(),
                                             cur_stream()),
             "grouped_gemm_fp8");
  }, py::arg("xq"), py::arg("xs"), py::arg("wq"), py::arg("ws"), py::arg("y"), py::arg("offsets"),
     py::arg("max_rows") = 0, py::arg("bn") = 0);
  m.def("apply_token_bitmask", [](Tensor& logits, const Tensor& bitmask) {
    need_cuda(logits, "logits");
    TORCH_CHECK(logits.scalar_type() == at::kFloat && logits.stride(1) == 1 && bitmask.is_contiguous() &&
                    bitmask.scalar_type() == at::kInt && bitmask.size(0) >= logits.size(0) &&
                    bitmask.size(1) == (logits.size(1) + 31) / 32,
                "apply_token_bitmask: fp32 logits [rows, vocab], int32 bitmask [rows, ceil(vocab/32)]");
    check_rc(mb_apply_token_bitmask(logits.data_ptr<float>(), bitmask.data_ptr<int32_t>(), logits.size(0),
                                    logits.size(1), logits.stride(0), cur_stream()),
             "apply_token_bitmask");
  });
  m.def("read_error_flag", &read_error_flag, py::arg("reset") = true);
  m.def("num_sms", &num_sms);
  m.def("attn_split_workspace_bytes", []() { return static_cast<int64_t>(mb_attn_split_workspace_bytes(num_sms())); });
  // partial-state workspace (fp32) and zeroed int32 counters of the split-KV decode attention; the caller keeps
  // both tensors alive for the life of the process
  m.def("set_attn_split_workspace", [](const Tensor& ws, const Tensor& counters) {
    need_cuda(ws, "ws"); need_cuda(counters, "counters");
    TORCH_CHECK(counters.scalar_type() == at::kInt && ws.is_contiguous() && counters.is_contiguous(), "workspace types");
    mb_set_attn_split_workspace(ws.data_ptr(), ws.nbytes(), counters.data_ptr<int>(), static_cast<int>(counters.numel()));
  });
  // 0 = never, 1 = by the partition heuristic (few sequences x KV heads), 2 = every decode-only step
  m.def("set_attn_split", [](int mode) { mb_set_attn_split(mode); });
  m.def("set_attn_tc", [](int min_tiles) { mb_set_attn_tc(min_tiles); });
  m.def("get_attn_tc", []() { return mb_get_attn_tc(); });
  m.def("qk_norm", &qk_norm, py::arg("qkv"), py::arg("q_w"), py::arg("k_w"), py::arg("n_q"), py::arg("n_kv"),
        py::arg("head_dim"), py::arg("eps"));
  m.def("set_gemm_pair_token_major", [](int mask) { mb_set_gemm_pair_token_major(mask); }, py::arg("mask"));
  m.def("set_gemm_pair_persistent", [](bool on) { mb_set_gemm_pair_persistent(on ? 1 : 0); }, py::arg("on"));
  m.def("set_gemm_pair", [](int min_m_plain, int min_m_dual) { mb_set_gemm_pair(min_m_plain, min_m_dual); },
        py::arg("min_m_plain"), py::arg("min_m_dual"));
  m.def("set_attn_decode_dense", [](bool on) { mb_set_attn_decode_dense(on ? 1 : 0); }, py::arg("on"));
  m.def("set_attn_fork", [](bool on) { mb_set_attn_fork(on ? 1 : 0); }, py::arg("on"));
  m.def("set_pdl", [](bool on) { mb_set_pdl(on ? 1 : 0); });
  m.def("get_pdl", []() { return mb_get_pdl() != 0; });
  m.def("tp_flag_ints", []() { return mb_tp_flag_ints(); });
  m.def("tp_barrier", [](int world, int rank, const std::vector<int64_t>& flags) {
    int* f[8] = {};
    for (int i = 0; i < world && i < 8; ++i) f[i] = reinterpret_cast<int*>(flags[i]);
    check_rc(mb_tp_barrier(world, rank, f, error_flag(), cur_stream()), "tp_barrier");
  });
  m.def("tp_rs_norm_ag", [](int world, int rank, const std::vector<int64_t>& partial,
                            const std::vector<int64_t>& xn, const std::vector<int64_t>& flags,
                            Tensor& h_local, const Tensor& gamma, int M, int rows_per_rank, double eps,
                            bool has_partials) {
    void* a[8] = {}; void* b[8] = {}; int* f[8] = {};
    for (int i = 0; i < world && i < 8; ++i) {
      a[i] = reinterpret_cast<void*>(partial[i]);
      b[i] = reinterpret_cast<void*>(xn[i]);
      f[i] = reinterpret_cast<int*>(flags[i]);
    }
    check_rc(mb_tp_rs_norm_ag(world, rank, a, b, f, h_local.data_ptr(), gamma.data_ptr(), M,
                              h_local.size(1), rows_per_rank, eps, 0.f, 0, has_partials ? 1 : 0,
                              error_flag(), cur_stream()),
             "tp_rs_norm_ag");
  });
  // mode bit0: pushed partials (n_slots, expected); bit1: close with ready flags instead of a barrier
  m.def("tp_rs_norm_ag_ex", [](int world, int rank, const std::vector<int64_t>& partial,
                               const std::vector<int64_t>& xn, const std::vector<int64_t>& flags,
                               Tensor& h_local, const Tensor& gamma, int M, int rows_per_rank, double eps,
                               bool has_partials, int mode, int n_slots, int expected) {
    void* a[8] = {}; void* b[8] = {}; int* f[8] = {};
    for (int i = 0; i < world && i < 8; ++i) {
      a[i] = reinterpret_cast<void*>(partial[i]);
      b[i] = reinterpret_cast<void*>(xn[i]);
      f[i] = reinterpret_cast<int*>(flags[i]);
    }
    check_rc(mb_tp_rs_norm_ag_ex(world, rank, a, b, f, h_local.data_ptr(), gamma.data_ptr(), M,
                                 h_local.size(1), rows_per_rank, eps, 0.f, 0, has_partials ? 1 : 0, mode,
                                 n_slots, expected, error_flag(), cur_stream()),
             "tp_rs_norm_ag_ex");
  });
  // GEMM fused with its collective; returns (expected counter increments on this rank, splits used)
  m.def("gemm_bf16_comm", [](const Tensor& x, const Tensor& w, const c10::optional<Tensor>& y, int M, bool dual,
                             bool wait_ready, bool push, int bn, int splits, int world, int rank,
                             int rows_per_rank, const std::vector<int64_t>& flags,
                             const std::vector<int64_t>& partial, int max_slots) {
    need_cuda(x, "x");
    TORCH_CHECK(x.stride(1) == 1 && w.is_contiguous(), "gemm_bf16_comm layout");
    int* f[8] = {}; void* a[8] = {};
    for (int i = 0; i < world && i < 8; ++i) {
      f[i] = reinterpret_cast<int*>(flags[i]);
      if (push) a[i] = reinterpret_cast<void*>(partial[i]);
    }
    const int K = x.size(1), N = dual ? w.size(0) / 2 : w.size(0);
    int expected = 0, used = 1;
    void* yp = y.has_value() ? y->data_ptr() : a[rank];
    check_rc(mb_gemm_bf16_comm(x.data_ptr(), w.data_ptr(), yp, M, N, K, x.stride(0), K,
                               y.has_value() ? static_cast<int>(y->stride(0)) : N,
                               (dual ? 1 : 0) | (wait_ready ? 16 : 0) | (push ? 32 : 0), bn, splits, world, rank,
                               rows_per_rank, f, push ? a : nullptr, max_slots, &expected, &used, error_flag(),
                               num_sms(), cur_stream()),
             "gemm_bf16_comm");
    return py::make_tuple(expected, used);
  });
  m.def("tp_allgather", [](int world, int rank, const std::vector<int64_t>& dst, const std::vector<int64_t>& flags,
                           const Tensor& src, int rows, int row_bytes, int ld_src, int ld_dst, int64_t col_off) {
    void* d[8] = {}; int* f[8] = {};
    for (int i = 0; i < world && i < 8; ++i) {
      d[i] = reinterpret_cast<void*>(dst[i]);
      f[i] = reinterpret_cast<int*>(flags[i]);
    }
    check_rc(mb_tp_allgather(world, rank, d, f, src.data_ptr(), rows, row_bytes, ld_src, ld_dst, col_off,
                             error_flag(), cur_stream()),
             "tp_allgather");
  });
  // all-reduce of symmetric bf16 buffers; algo 0 auto / 1 one-shot / 2 two-shot / 3 multimem
  m.def("tp_allreduce", [](int world, int rank, const std::vector<int64_t>& in_bufs,
                           const std::vector<int64_t>& out_bufs, Tensor& out, int64_t mc_in,
                           const std::vector<int64_t>& flags, int64_t n, int algo) {
    void* a[8] = {}; void* b[8] = {}; int* f[8] = {};
    for (int i = 0; i < world && i < 8; ++i) {
      a[i] = reinterpret_cast<void*>(in_bufs[i]);
      if (!out_bufs.empty()) b[i] = reinterpret_cast<void*>(out_bufs[i]);
      f[i] = reinterpret_cast<int*>(flags[i]);
    }
    check_rc(mb_tp_allreduce(world, rank, a, out_bufs.empty() ? nullptr : b, out.data_ptr(),
                             reinterpret_cast<const void*>(mc_in), f, n, algo, error_flag(), cur_stream()),
             "tp_allreduce");
  });
  m.def("tp_allreduce_lamport", [](int world, int rank, const std::vector<int64_t>& lam, const Tensor& x, Tensor& out,
                                   int64_t cap, Tensor& state, const c10::optional<Tensor>& residual,
                                   const c10::optional<Tensor>& gamma, double eps) {
    need_cuda(x, "x");
    TORCH_CHECK(x.is_contiguous() && out.is_contiguous() && x.scalar_type() == at::kBFloat16 && state.numel() >= 8 &&
                    state.scalar_type() == at::kInt && static_cast<int>(lam.size()) == world,
                "tp_allreduce_lamport: contiguous bf16 tensors, 8 state ints, one buffer per rank");
    void* a[8] = {};
    for (int i = 0; i < world && i < 8; ++i) a[i] = reinterpret_cast<void*>(lam[i]);
    const bool norm = gamma.has_value() && gamma->defined();
    check_rc(mb_tp_allreduce_lamport(world, rank, a, x.data_ptr(), out.data_ptr(), x.numel(), cap, state.data_ptr<int>(),
                                     norm ? const_cast<void*>(optptr(residual)) : nullptr, norm ? optptr(gamma) : nullptr,
                                     norm ? static_cast<int>(x.size(-1)) : 0, static_cast<float>(eps), 0.f, 0,
                                     error_flag(), cur_stream()),
             "tp_allreduce_lamport");
  });
  m.def("tp_wait_flag", [](const Tensor& flag, int target, int timeout_ms, int code, Tensor& ok_out) {
    need_cuda(flag, "flag");
    check_rc(mb_tp_wait_flag(flag.data_ptr<int32_t>(), target, timeout_ms, code, error_flag(),
                             ok_out.data_ptr<int32_t>(), cur_stream()),
             "tp_wait_flag");
  });
  m.def("tp_scatter", [](int world, int rank, int root, const std::vector<int64_t>& in_bufs, Tensor& out,
                         const std::vector<int64_t>& flags, int64_t chunk_bytes) {
    void* a[8] = {}; int* f[8] = {};
    for (int i = 0; i < world && i < 8; ++i) {
      a[i] = reinterpret_cast<void*>(in_bufs[i]);
      f[i] = reinterpret_cast<int*>(flags[i]);
    }
    check_rc(mb_tp_scatter(world, rank, root, a, out.data_ptr(), f, chunk_bytes, error_flag(), cur_stream()),
             "tp_scatter");
  });
  m.def("tp_broadcast", [](int world, int rank, int root, const std::vector<int64_t>& in_bufs, Tensor& out,
                           const std::vector<int64_t>& flags, int64_t nbytes) {
    void* a[8] = {}; int* f[8] = {};
    for (int i = 0; i < world && i < 8; ++i) {
      a[i] = reinterpret_cast<void*>(in_bufs[i]);
      f[i] = reinterpret_cast<int*>(flags[i]);
    }
    check_rc(mb_tp_broadcast(world, rank, root, a, out.data_ptr(), f, nbytes, error_flag(), cur_stream()),
             "tp_broadcast");
  });
  // ---- multi-head latent attention ----
  // cache: [pages, page_size, R + 64] view of one layer (page stride free, rows contiguous)
  m.def("mla_kv_store", [](const Tensor& c_kv, const Tensor& k_rope, const Tensor& slots, Tensor& cache) {
    need_cuda(c_kv, "c_kv");
    TORCH_CHECK(c_kv.stride(1) == 1 && k_rope.stride(1) == 1 && k_rope.size(1) == 64 &&
                    cache.stride(2) == 1 && cache.stride(1) == cache.size(2) &&
                    cache.size(2) == c_kv.size(1) + 64 && slots.scalar_type() == at::kLong,
                "mla_kv_store layout");
    check_rc(mb_mla_kv_store(c_kv.data_ptr(), k_rope.data_ptr(), slots.data_ptr<int64_t>(), cache.data_ptr(),
                             c_kv.size(0), c_kv.size(1), c_kv.stride(0), k_rope.stride(0), cache.size(1),
                             cache.stride(0), cur_stream()),
             "mla_kv_store");
  });
  m.def("mla_paged_attention", [](const Tensor& q_lat, const Tensor& q_rope, const Tensor& cache,
                                  const Tensor& block_table, const Tensor& q_start, const Tensor& q_len,
                                  const Tensor& kv_len, Tensor& out, double scale, bool decode_only) {
    need_cuda(q_lat, "q_lat");
    TORCH_CHECK(q_lat.is_contiguous() && q_rope.is_contiguous() && out.is_contiguous() && q_rope.size(2) == 64 &&
                    cache.stride(2) == 1 && cache.stride(1) == cache.size(2) &&
                    cache.size(2) == q_lat.size(2) + 64 && block_table.stride(1) == 1,
                "mla_paged_attention layout");
    // decode_only: the caller knows that every sequence has exactly one query token
    if (decode_only && mb_mla_tc_usable(q_lat.size(0), block_table.size(0), q_lat.size(1), q_lat.size(2),
                                        cache.size(1))) {
      check_rc(mb_mla_decode_tc(q_lat.data_ptr(), q_rope.data_ptr(), out.data_ptr(), cache.data_ptr(),
                                cache.stride(0), cache.size(0), block_table.data_ptr<int32_t>(),
                                block_table.stride(0), q_start.data_ptr<int32_t>(), q_len.data_ptr<int32_t>(),
                                kv_len.data_ptr<int32_t>(), q_lat.size(0), block_table.size(0), q_lat.size(1),
                                cache.size(1), scale, error_flag(), cur_stream()),
               "mla_decode_tc");
      return;
    }
    // ragged steps with 512-wide latents and a multiple of 128 heads: the tensor-core kernel, one CTA pair per token
    if (!decode_only && mb_mla_tc_usable(q_lat.size(0), q_lat.size(0), q_lat.size(1), q_lat.size(2), cache.size(1))) {
      auto scratch = at::empty({2 * q_lat.size(0)}, q_start.options().dtype(at::kInt));
      check_rc(mb_mla_prefill_tc(q_lat.data_ptr(), q_rope.data_ptr(), out.data_ptr(), cache.data_ptr(),
                                 cache.stride(0), cache.size(0), block_table.data_ptr<int32_t>(),
                                 block_table.stride(0), q_start.data_ptr<int32_t>(), q_len.data_ptr<int32_t>(),
                                 kv_len.data_ptr<int32_t>(), q_lat.size(0), block_table.size(0), q_lat.size(1),
                                 cache.size(1), scale, scratch.data_ptr<int32_t>(), error_flag(), cur_stream()),
               "mla_prefill_tc");
      return;
    }
    check_rc(mb_mla_paged_attention(q_lat.data_ptr(), q_rope.data_ptr(), out.data_ptr(), cache.data_ptr(),
                                    cache.stride(0), block_table.data_ptr<int32_t>(), block_table.stride(0),
                                    q_start.data_ptr<int32_t>(), q_len.data_ptr<int32_t>(),
                                    kv_len.data_ptr<int32_t>(), q_lat.size(0), block_table.size(0),
                                    q_lat.size(1), q_lat.size(2), cache.size(1), scale, cur_stream()),
             "mla_paged_attention");
  }, py::arg("q_lat"), py::arg("q_rope"), py::arg("cache"), py::arg("block_table"), py::arg("q_start"),
     py::arg("q_len"), py::arg("kv_len"), py::arg("out"), py::arg("scale"), py::arg("decode_only") = false);
  // after the fused down-projections of an MLA layer: norms, key rotation and the latent-cache store in one launch
  m.def("mla_post_down", [](const Tensor& qkv_a, int q_lora, const c10::optional<Tensor>& gamma_q, const Tensor& gamma_kv,
                            double eps, const Tensor& positions, const Tensor& cos_sin, const Tensor& slots,
                            const c10::optional<Tensor>& q_a_out, Tensor& cache) {
    need_cuda(qkv_a, "qkv_a");
    const int R = cache.size(2) - 64;
    TORCH_CHECK(qkv_a.dim() == 2 && qkv_a.stride(1) == 1 && qkv_a.scalar_type() == at::kBFloat16 &&
                    qkv_a.size(1) >= q_lora + R + 64 && positions.scalar_type() == at::kInt &&
                    slots.scalar_type() == at::kLong && cos_sin.scalar_type() == at::kFloat && cos_sin.is_contiguous() &&
                    cos_sin.size(1) == 64 && cache.stride(2) == 1 && cache.stride(1) == cache.size(2) &&
                    gamma_kv.numel() == R && positions.numel() >= qkv_a.size(0) && slots.numel() >= qkv_a.size(0),
                "mla_post_down layout");
    TORCH_CHECK(q_lora == 0 || (gamma_q.has_value() && q_a_out.has_value() && gamma_q->numel() == q_lora &&
                                q_a_out->is_contiguous() && q_a_out->size(0) >= qkv_a.size(0) && q_a_out->size(1) == q_lora),
                "mla_post_down: q_a outputs");
    check_rc(mb_mla_post_down(qkv_a.data_ptr(), qkv_a.stride(0), q_lora, R, q_lora ? gamma_q->data_ptr() : gamma_kv.data_ptr(),
                              gamma_kv.data_ptr(), eps, positions.data_ptr<int32_t>(), cos_sin.data_ptr<float>(),
                              slots.data_ptr<int64_t>(), q_lora ? q_a_out->data_ptr() : cache.data_ptr(), cache.data_ptr(),
                              qkv_a.size(0), cache.size(1), cache.stride(0), cur_stream()),
             "mla_post_down");
  });
  m.def("mla_q_rope", [](const Tensor& q, int n_heads, int nope, const Tensor& positions, const Tensor& cos_sin,
                         Tensor& q_rope) {
    need_cuda(q, "q");
    TORCH_CHECK(q.is_contiguous() && q_rope.is_contiguous() && q.scalar_type() == at::kBFloat16 &&
                    q.numel() == q.size(0) * static_cast<int64_t>(n_heads) * (nope + 64) &&
                    q_rope.numel() >= q.size(0) * static_cast<int64_t>(n_heads) * 64 && positions.scalar_type() == at::kInt &&
                    cos_sin.scalar_type() == at::kFloat && cos_sin.is_contiguous() && cos_sin.size(1) == 64,
                "mla_q_rope layout");
    check_rc(mb_mla_q_rope(q.data_ptr(), n_heads, nope, positions.data_ptr<int32_t>(), cos_sin.data_ptr<float>(),
                           q_rope.data_ptr(), q.size(0), cur_stream()),
             "mla_q_rope");
  });
  m.def("mla_split_workspace_bytes", []() { return static_cast<int64_t>(mb_mla_split_workspace_bytes(num_sms())); });
  m.def("set_mla_split_workspace", [](const Tensor& ws, const Tensor& counters) {
    need_cuda(ws, "ws"); need_cuda(counters, "counters");
    TORCH_CHECK(counters.scalar_type() == at::kInt && ws.is_contiguous() && counters.is_contiguous(), "workspace types");
    mb_set_mla_split_workspace(ws.data_ptr(), ws.nbytes(), counters.data_ptr<int>(), static_cast<int>(counters.numel()));
  });
  m.def("set_mla_split", [](int mode) { mb_set_mla_split(mode); }, py::arg("mode"));
  m.def("set_mla_tc", [](bool on) { mb_set_mla_tc(on ? 1 : 0); }, py::arg("on"));
  // ---- expert parallelism ----
  m.def("ep_flag_ints", []() { return mb_ep_flag_ints(); });
  m.def("ep_dispatch", [](int world, int rank, const std::vector<int64_t>& recv_x,
                          const std::vector<int64_t>& recv_meta, const std::vector<int64_t>& flags,
                          const Tensor& x, const Tensor& topk_ids, Tensor& send_pos, int e_local, int cap,
                          bool fp8) {
    need_cuda(x, "x");
    TORCH_CHECK(x.is_contiguous() && topk_ids.is_contiguous() && topk_ids.scalar_type() == at::kInt &&
                    send_pos.numel() >= topk_ids.numel(), "ep_dispatch layout");
    void* a[8] = {}; void* b[8] = {}; int* f[8] = {};
    for (int i = 0; i < world && i < 8; ++i) {
      a[i] = reinterpret_cast<void*>(recv_x[i]);
      b[i] = reinterpret_cast<void*>(recv_meta[i]);
      f[i] = reinterpret_cast<int*>(flags[i]);
    }
    check_rc(mb_ep_dispatch(world, rank, a, b, f, x.data_ptr(), topk_ids.data_ptr<int32_t>(),
                            send_pos.data_ptr<int32_t>(), x.size(0), x.size(1), topk_ids.size(1), e_local,
                            cap, fp8 ? 1 : 0, error_flag(), cur_stream()),
             "ep_dispatch");
  });
  m.def("ep_gather_ids", [](const Tensor& recv_meta, const Tensor& flags, Tensor& ids, int world, int cap) {
    need_cuda(recv_meta, "recv_meta");
    TORCH_CHECK(ids.numel() >= static_cast<int64_t>(world) * cap, "ids too small");
    check_rc(mb_ep_gather_ids(recv_meta.data_ptr<int32_t>(), flags.data_ptr<int32_t>(), ids.data_ptr<int32_t>(),
                              world, cap, cur_stream()),
             "ep_gather_ids");
  });
  m.def("ep_combine_send", [](int world, int rank, const std::vector<int64_t>& ret_x,
                              const std::vector<int64_t>& flags, const Tensor& out_sorted, const Tensor& order,
                              const Tensor& n_rows, int cap) {
    need_cuda(out_sorted, "out_sorted");
    TORCH_CHECK(out_sorted.is_contiguous(), "contiguous");
    void* a[8] = {}; int* f[8] = {};
    for (int i = 0; i < world && i < 8; ++i) {
      a[i] = reinterpret_cast<void*>(ret_x[i]);
      f[i] = reinterpret_cast<int*>(flags[i]);
    }
    check_rc(mb_ep_combine_send(world, rank, a, f, out_sorted.data_ptr(), order.data_ptr<int32_t>(),
                                n_rows.data_ptr<int32_t>(), out_sorted.size(0), out_sorted.size(1), cap,
                                error_flag(), cur_stream()),
             "ep_combine_send");
  });
  m.def("ep_combine_reduce", [](const Tensor& ret_x, const Tensor& topk_ids, const Tensor& send_pos,
                                const Tensor& w, const c10::optional<Tensor>& shared, Tensor& y, int e_local,
                                int cap, const c10::optional<Tensor>& residual) {
    need_cuda(ret_x, "ret_x");
    TORCH_CHECK(y.is_contiguous() && w.is_contiguous() && w.scalar_type() == at::kFloat &&
                    (!residual || (residual->is_contiguous() && residual->sizes() == y.sizes())) &&
                    (!shared || (shared->is_contiguous() && shared->sizes() == y.sizes())),
                "ep_combine_reduce layout");
    check_rc(mb_ep_combine_reduce(ret_x.data_ptr(), topk_ids.data_ptr<int32_t>(), send_pos.data_ptr<int32_t>(),
                                  w.data_ptr<float>(), optptr(shared), optptr(residual), y.data_ptr(), y.size(0),
                                  y.size(1), topk_ids.size(1), e_local, cap, cur_stream()),
             "ep_combine_reduce");
  }, py::arg("ret_x"), py::arg("topk_ids"), py::arg("send_pos"), py::arg("w"), py::arg("shared"), py::arg("y"),
     py::arg("e_local"), py::arg("cap"), py::arg("residual") = py::none());
  // receive buffers -> rows in expert order + offsets + order, one launch; fp8 rows are split into payload and
  // group-major scales
  m.def("ep_recv_compact", [](const Tensor& recv_x, const Tensor& recv_meta, const Tensor& flags, int world, int cap,
                              int n_experts, int hidden, bool fp8, int rows_bound, Tensor& offsets, Tensor& order,
                              Tensor& xq, const c10::optional<Tensor>& xs) {
    need_cuda(recv_x, "recv_x");
    TORCH_CHECK(recv_meta.scalar_type() == at::kInt && offsets.scalar_type() == at::kInt &&
                    order.scalar_type() == at::kInt && offsets.numel() >= n_experts + 1 && xq.is_contiguous() &&
                    xq.dim() == 2 && order.numel() >= xq.size(0) && xq.size(0) >= rows_bound &&
                    xq.size(1) * xq.element_size() == (fp8 ? hidden : hidden * 2),
                "ep_recv_compact layout");
    TORCH_CHECK(!fp8 || (xs.has_value() && xs->is_contiguous() && xs->scalar_type() == at::kFloat && xs->dim() == 2 &&
                         xs->size(0) == hidden / 128 && xs->size(1) >= rows_bound),
                "ep_recv_compact: scales [hidden / 128, >= rows_bound]");
    check_rc(mb_ep_recv_compact(recv_x.data_ptr(), recv_meta.data_ptr<int32_t>(), flags.data_ptr<int32_t>(), world,
                                cap, n_experts, hidden, fp8 ? 1 : 0, rows_bound, offsets.data_ptr<int32_t>(),
                                order.data_ptr<int32_t>(), xq.data_ptr(), xs ? xs->data_ptr<float>() : nullptr,
                                xs ? static_cast<int>(xs->size(1)) : 0, num_sms(), cur_stream()),
             "ep_recv_compact");
  });
  // y[m, b * y_off + n] = sum_k x[m, b * x_off + k] * w[b, n, k]: per-head products on column blocks of x and y
  m.def("batched_gemm_bf16", [](const Tensor& x, const Tensor& w, Tensor& y, int x_off, int y_off) {
    need_cuda(x, "x");
    TORCH_CHECK(x.dim() == 2 && y.dim() == 2 && w.dim() == 3 && x.stride(1) == 1 && y.stride(1) == 1 &&
                    w.is_contiguous() && x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 &&
                    y.scalar_type() == at::kBFloat16 && y.size(0) == x.size(0),
                "batched_gemm_bf16: bf16 x [M, *], w [B, N, K], y [M, *]");
    const int B = w.size(0), N = w.size(1), K = w.size(2);
    TORCH_CHECK(static_cast<int64_t>(B - 1) * x_off + K <= x.size(1) && static_cast<int64_t>(B - 1) * y_off + N <= y.size(1),
                "batched_gemm_bf16: column blocks out of range");
    check_rc(mb_batched_gemm_bf16(x.data_ptr(), w.data_ptr(), y.data_ptr(), B, x.size(0), N, K, x.stride(0), x_off,
                                  y.stride(0), y_off, x.size(1), 0, error_flag(), cur_stream()),
             "batched_gemm_bf16");
  });
  // the same on the persistent decode-step GEMM (at most 256 rows, N % 128 == 0): one launch over all heads
  m.def("gemm_dec_batched", [](const Tensor& x, const Tensor& w, Tensor& y, int x_off, int y_off, Tensor& ws,
                               Tensor& state) {
    need_cuda(x, "x");
    TORCH_CHECK(x.dim() == 2 && y.dim() == 2 && w.dim() == 3 && x.stride(1) == 1 && y.stride(1) == 1 &&
                    w.is_contiguous() && x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16 &&
                    y.scalar_type() == at::kBFloat16 && y.size(0) == x.size(0) && state.scalar_type() == at::kInt,
                "gemm_dec_batched: bf16 x [M, *], w [B, N, K], y [M, *]");
    const int B = w.size(0), N = w.size(1), K = w.size(2);
    TORCH_CHECK(static_cast<int64_t>(B - 1) * x_off + K <= x.size(1) && static_cast<int64_t>(B - 1) * y_off + N <= y.size(1),
                "gemm_dec_batched: column blocks out of range");
    check_rc(mb_gemm_dec_batched(x.data_ptr(), w.data_ptr(), y.data_ptr(), B, x.size(0), N, K, x.stride(0), x_off,
                                 y.stride(0), y_off, x.size(1), ws.data_ptr(), ws.nbytes(), state.data_ptr<int>(),
                                 error_flag(), num_sms(), cur_stream()),
             "gemm_dec_batched");
  });
  m.def("dequant_fp8_group128", [](const Tensor& q, const Tensor& scales, Tensor& out, const c10::optional<Tensor>& n_rows) {
    need_cuda(q, "q");
    TORCH_CHECK(q.is_contiguous() && q.element_size() == 1 && q.dim() == 2 && out.is_contiguous() &&
                    out.scalar_type() == at::kBFloat16 && out.size(0) == q.size(0) && out.size(1) == q.size(1) &&
                    scales.is_contiguous() && scales.scalar_type() == at::kFloat && scales.dim() == 2 &&
                    scales.size(0) == q.size(1) / 128 && scales.size(1) >= q.size(0),
                "dequant_fp8_group128 layout");
    check_rc(mb_dequant_fp8_group128(q.data_ptr(), scales.data_ptr<float>(), out.data_ptr(), q.size(0), q.size(1),
                                     static_cast<int>(scales.size(1)), n_rows ? n_rows->data_ptr<int32_t>() : nullptr,
                                     cur_stream()),
             "dequant_fp8_group128");
  });
  m.def("silu_mul_quant_fp8", [](const Tensor& gu, Tensor& q, Tensor& scales, const c10::optional<Tensor>& n_rows) {
    need_cuda(gu, "gate_up");
    const int M = gu.size(0), I = gu.size(1) / 2;
    TORCH_CHECK(gu.is_contiguous() && gu.scalar_type() == at::kBFloat16 && q.is_contiguous() && q.element_size() == 1 &&
                    q.size(0) == M && q.size(1) == I && scales.is_contiguous() && scales.scalar_type() == at::kFloat &&
                    scales.dim() == 2 && scales.size(0) == I / 128 && scales.size(1) >= M,
                "silu_mul_quant_fp8 layout");
    check_rc(mb_silu_mul_quant_fp8(gu.data_ptr(), q.data_ptr(), scales.data_ptr<float>(), M, I,
                                   static_cast<int>(scales.size(1)), n_rows ? n_rows->data_ptr<int32_t>() : nullptr,
                                   cur_stream()),
             "silu_mul_quant_fp8");
  });
  m.def("ep_dequant_rows", [](const Tensor& src, Tensor& dst, int n, const c10::optional<Tensor>& n_rows) {
    need_cuda(src, "src");
    check_rc(mb_ep_dequant_rows(src.data_ptr(), dst.data_ptr(), n, dst.size(1),
                                static_cast<const int32_t*>(optptr(n_rows)), cur_stream()),
             "ep_dequant_rows");
  });
  py::class_<PyDecoderExecutor>(m, "DecoderExecutor")
      .def(py::init<py::dict>())
      .def("set_globals", &PyDecoderExecutor::set_globals)
      .def("add_layer", &PyDecoderExecutor::add_layer, py::arg("attn_norm"), py::arg("wqkv"), py::arg("wo"),
           py::arg("mlp_norm"), py::arg("wgu"), py::arg("wd"), py::arg("scales") = py::none(),
           py::arg("qkv_bias") = py::none(), py::arg("q_norm") = py::none(), py::arg("k_norm") = py::none())
      .def("set_fp8_buffers", &PyDecoderExecutor::set_fp8_buffers)
      .def("set_kv_cache", &PyDecoderExecutor::set_kv_cache)
      .def("set_buffers", &PyDecoderExecutor::set_buffers)
      .def("set_tp", &PyDecoderExecutor::set_tp)
      .def("set_dec", &PyDecoderExecutor::set_dec)
      .def("set_tp_lamport", &PyDecoderExecutor::set_tp_lamport)
      .def("dec_usable", &PyDecoderExecutor::dec_usable)
      .def("forward", &PyDecoderExecutor::forward)
      .def("launches", &PyDecoderExecutor::launches)
      .def("set_profiling", &PyDecoderExecutor::set_profiling)
      .def("profile", &PyDecoderExecutor::profile);
  mb::bind_runtime(m);
}
