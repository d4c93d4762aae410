// Bandwidth-bound helper kernels: RMSNorm (+ fused residual add), SwiGLU, embedding
// gather, row gather, and the fused RoPE + QKV split + paged-KV store.
//
// All of them move 16 bytes per thread per access and keep statistics in fp32.
// Behavioural counterparts in the reference: max/kernels/src/nn/normalization.mojo
// (rms_norm, rms_norm_fused_residual), max/kernels/src/nn/rope_split_store.mojo:430
// (rope_split_store_paged_ragged).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace mb {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = lane < nw ? scratch[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

// out = rmsnorm(x [+ residual]) * (w + offset). When ADD, residual <- x + residual first.
// MBC (multiply before cast): Gemma rounding order; otherwise Llama order
// (normalise, round to bf16, then multiply by the bf16 weight).
template <bool ADD>
__global__ void __launch_bounds__(256)
rmsnorm_kernel(const bf16* __restrict__ x, bf16* __restrict__ residual, const bf16* __restrict__ w,
               bf16* __restrict__ out, int cols, int ldx, int ldo, float eps, float w_off,
               int mbc) {
  __shared__ float scratch[32];
  extern __shared__ uint4 row_cache[];  // cols/8 packed values (the summed row)
  pdl_wait();
  pdl_trigger();
  const int row = blockIdx.x;
  const bf16* xr = x + static_cast<size_t>(row) * ldx;
  bf16* rr = ADD ? residual + static_cast<size_t>(row) * cols : nullptr;
  const int nvec = cols >> 3;
  float ss = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 a = *reinterpret_cast<const uint4*>(xr + v * 8);
    bf162* ap = reinterpret_cast<bf162*>(&a);
    if (ADD) {
      const uint4 b = *reinterpret_cast<const uint4*>(rr + v * 8);
      const bf162* bp = reinterpret_cast<const bf162*>(&b);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 fa = __bfloat1622float2(ap[i]), fb = __bfloat1622float2(bp[i]);
        ap[i] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
      }
      *reinterpret_cast<uint4*>(rr + v * 8) = a;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(ap[i]);
      ss += f.x * f.x + f.y * f.y;
    }
    row_cache[v] = a;
  }
  const float tot = block_sum(ss, scratch);
  const float inv = rsqrtf(tot / static_cast<float>(cols) + eps);
  bf16* orow = out + static_cast<size_t>(row) * ldo;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 a = row_cache[v];
    const uint4 wv = *reinterpret_cast<const uint4*>(w + v * 8);
    bf162* ap = reinterpret_cast<bf162*>(&a);
    const bf162* wp = reinterpret_cast<const bf162*>(&wv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(ap[i]);
      const float2 g = __bfloat1622float2(wp[i]);
      if (mbc) {
        ap[i] = __floats2bfloat162_rn(f.x * inv * (g.x + w_off), f.y * inv * (g.y + w_off));
      } else {
        const bf162 n = __floats2bfloat162_rn(f.x * inv, f.y * inv);
        const float2 nf = __bfloat1622float2(n);
        ap[i] = __floats2bfloat162_rn(nf.x * (g.x + w_off), nf.y * (g.y + w_off));
      }
    }
    *reinterpret_cast<uint4*>(orow + v * 8) = a;
  }
}

// RMSNorm over head_dim of every query and key head of a fused projection, in place: one warp per (token, head),
// head_dim / 8 lanes hold 8 values each (head_dim <= 256). Llama rounding order: normalise, round to bf16, multiply
// by the bf16 weight.
__global__ void qk_norm_kernel(bf16* __restrict__ qkv, const bf16* __restrict__ qw, const bf16* __restrict__ kw,
                               int T, int n_q, int n_kv, int hd, int ld, float eps) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long unit = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int heads = n_q + n_kv;
  if (unit >= static_cast<long long>(T) * heads) return;
  const int t = static_cast<int>(unit / heads), h = static_cast<int>(unit % heads);
  const bf16* w = h < n_q ? qw : kw;
  bf16* p = qkv + static_cast<size_t>(t) * ld + static_cast<size_t>(h) * hd;   // key heads follow the query heads
  const bool on = lane * 8 < hd;
  uint4 a = make_uint4(0u, 0u, 0u, 0u);
  if (on) a = *reinterpret_cast<const uint4*>(p + lane * 8);
  bf162* ap = reinterpret_cast<bf162*>(&a);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(ap[i]);
    ss += f.x * f.x + f.y * f.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (!on) return;
  const float inv = rsqrtf(ss / static_cast<float>(hd) + eps);
  const uint4 wv = *reinterpret_cast<const uint4*>(w + lane * 8);
  const bf162* wp = reinterpret_cast<const bf162*>(&wv);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(ap[i]);
    const float2 g = __bfloat1622float2(wp[i]);
    const float2 n = __bfloat1622float2(__floats2bfloat162_rn(f.x * inv, f.y * inv));
    ap[i] = __floats2bfloat162_rn(n.x * g.x, n.y * g.y);
  }
  *reinterpret_cast<uint4*>(p + lane * 8) = a;
}

// x[r, c] += bias[c] (bias of a fused projection; rows of `ld` elements, cols a multiple of 8)
__global__ void add_bias_kernel(bf16* __restrict__ x, const bf16* __restrict__ bias, int rows, int cols, int ld) {
  pdl_wait();
  pdl_trigger();
  const int per_row = cols >> 3;
  const size_t vec = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (vec >= static_cast<size_t>(rows) * per_row) return;
  const int r = static_cast<int>(vec / per_row), c = static_cast<int>(vec % per_row) * 8;
  bf16* xp = x + static_cast<size_t>(r) * ld + c;
  uint4 a = *reinterpret_cast<const uint4*>(xp);
  const uint4 b = *reinterpret_cast<const uint4*>(bias + c);
  bf162* ap = reinterpret_cast<bf162*>(&a);
  const bf162* bp = reinterpret_cast<const bf162*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = __bfloat1622float2(ap[i]), fb = __bfloat1622float2(bp[i]);
    ap[i] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
  }
  *reinterpret_cast<uint4*>(xp) = a;
}

// out[r, i] = silu(gu[r, i]) * gu[r, inter + i]
__global__ void silu_mul_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int rows,
                                int inter) {
  const size_t vec = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_row = inter >> 3;
  if (vec >= static_cast<size_t>(rows) * per_row) return;
  const int r = static_cast<int>(vec / per_row), c = static_cast<int>(vec % per_row) * 8;
  const bf16* g = gu + static_cast<size_t>(r) * 2 * inter + c;
  uint4 a = *reinterpret_cast<const uint4*>(g);
  const uint4 b = *reinterpret_cast<const uint4*>(g + inter);
  bf162* ap = reinterpret_cast<bf162*>(&a);
  const bf162* bp = reinterpret_cast<const bf162*>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = __bfloat1622float2(ap[i]), fb = __bfloat1622float2(bp[i]);
    ap[i] = __floats2bfloat162_rn(fa.x / (1.f + __expf(-fa.x)) * fb.x,
                                  fa.y / (1.f + __expf(-fa.y)) * fb.y);
  }
  *reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * inter + c) = a;
}

// Vocabulary-shard aware embedding lookup: ids outside [vocab_start, vocab_start+vocab)
// produce zero rows (the tensor-parallel reduction then restores them).
__global__ void embedding_kernel(const int64_t* __restrict__ ids, const bf16* __restrict__ table,
                                 bf16* __restrict__ out, int n, int hidden, int vocab,
                                 int vocab_start) {
  pdl_wait();
  pdl_trigger();
  const int per_row = hidden >> 3;
  const size_t vec = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (vec >= static_cast<size_t>(n) * per_row) return;
  const int r = static_cast<int>(vec / per_row), c = static_cast<int>(vec % per_row) * 8;
  const int64_t id = ids[r] - vocab_start;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (id >= 0 && id < vocab) v = *reinterpret_cast<const uint4*>(table + id * hidden + c);
  *reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * hidden + c) = v;
}

__global__ void gather_rows_kernel(const uint8_t* __restrict__ src, const int32_t* __restrict__ idx,
                                   uint8_t* __restrict__ dst, int n, int row_bytes, int ld_src) {
  pdl_wait();
  pdl_trigger();
  const int per_row = row_bytes >> 4;
  const size_t vec = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (vec >= static_cast<size_t>(n) * per_row) return;
  const int r = static_cast<int>(vec / per_row), c = static_cast<int>(vec % per_row) * 16;
  *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * row_bytes + c) =
      *reinterpret_cast<const uint4*>(src + static_cast<size_t>(idx[r]) * ld_src + c);
}

// One thread handles 8 consecutive dims d..d+7 of the first half of a head and the
// matching 8 dims of the second half (rotate-half convention), or 8 consecutive dims
// as 4 (even, odd) pairs (interleaved convention). cos_sin is [max_pos, head_dim]:
// the first head_dim/2 entries of a row are cos, the rest sin.
__global__ void rope_kv_store_kernel(bf16* __restrict__ qkv, const int32_t* __restrict__ positions,
                                     const int64_t* __restrict__ slots,
                                     const float* __restrict__ cos_sin, bf16* __restrict__ k_cache,
                                     bf16* __restrict__ v_cache, int T, int n_q, int n_kv,
                                     int head_dim, int page_size, int64_t page_stride,
                                     int64_t head_stride, int interleaved) {
  pdl_wait();
  pdl_trigger();
  const int half = head_dim >> 1;
  const int vec_per_head = half >> 3;           // threads per (token, head) for q/k
  const int heads_rot = n_q + n_kv;             // heads that get rotated
  const int work_per_tok = heads_rot * vec_per_head + n_kv * (head_dim >> 3);
  const size_t gid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (gid >= static_cast<size_t>(T) * work_per_tok) return;
  const int t = static_cast<int>(gid / work_per_tok);
  int w = static_cast<int>(gid % work_per_tok);
  const int row_elems = (n_q + 2 * n_kv) * head_dim;
  bf16* row = qkv + static_cast<size_t>(t) * row_elems;
  const int64_t slot = slots[t];
  const int64_t page = slot / page_size;
  const int off = static_cast<int>(slot % page_size);

  if (w >= heads_rot * vec_per_head) {
    // V copy: 8 dims per thread
    w -= heads_rot * vec_per_head;
    const int h = w / (head_dim >> 3), d = (w % (head_dim >> 3)) * 8;
    if (slot < 0) return;
    const uint4 v = *reinterpret_cast<const uint4*>(row + (n_q + n_kv + h) * head_dim + d);
    *reinterpret_cast<uint4*>(v_cache + page * page_stride + h * head_stride +
                              static_cast<int64_t>(off) * head_dim + d) = v;
    return;
  }
  const int h = w / vec_per_head, d = (w % vec_per_head) * 8;
  const float* cs = cos_sin + static_cast<size_t>(positions[t]) * head_dim;
  bf16* hp = row + h * head_dim;
  uint4 lo, hi;
  if (!interleaved) {
    lo = *reinterpret_cast<const uint4*>(hp + d);
    hi = *reinterpret_cast<const uint4*>(hp + half + d);
    bf16* l = reinterpret_cast<bf16*>(&lo);
    bf16* u = reinterpret_cast<bf16*>(&hi);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float c = cs[d + i], s = cs[half + d + i];
      const float a = __bfloat162float(l[i]), b = __bfloat162float(u[i]);
      l[i] = __float2bfloat16(a * c - b * s);
      u[i] = __float2bfloat16(b * c + a * s);
    }
  } else {
    // dims [2d, 2d+16): pairs (2j, 2j+1) use frequency j
    lo = *reinterpret_cast<const uint4*>(hp + 2 * d);
    hi = *reinterpret_cast<const uint4*>(hp + 2 * d + 8);
    bf16* l = reinterpret_cast<bf16*>(&lo);
    bf16* u = reinterpret_cast<bf16*>(&hi);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float c = cs[d + i], s = cs[half + d + i];
      float a = __bfloat162float(l[2 * i]), b = __bfloat162float(l[2 * i + 1]);
      l[2 * i] = __float2bfloat16(a * c - b * s);
      l[2 * i + 1] = __float2bfloat16(b * c + a * s);
      c = cs[d + 4 + i]; s = cs[half + d + 4 + i];
      a = __bfloat162float(u[2 * i]); b = __bfloat162float(u[2 * i + 1]);
      u[2 * i] = __float2bfloat16(a * c - b * s);
      u[2 * i + 1] = __float2bfloat16(b * c + a * s);
    }
  }
  if (h < n_q) {
    if (!interleaved) {
      *reinterpret_cast<uint4*>(hp + d) = lo;
      *reinterpret_cast<uint4*>(hp + half + d) = hi;
    } else {
      *reinterpret_cast<uint4*>(hp + 2 * d) = lo;
      *reinterpret_cast<uint4*>(hp + 2 * d + 8) = hi;
    }
  } else if (slot >= 0) {
    bf16* kc = k_cache + page * page_stride + (h - n_q) * head_stride +
               static_cast<int64_t>(off) * head_dim;
    if (!interleaved) {
      *reinterpret_cast<uint4*>(kc + d) = lo;
      *reinterpret_cast<uint4*>(kc + half + d) = hi;
    } else {
      *reinterpret_cast<uint4*>(kc + 2 * d) = lo;
      *reinterpret_cast<uint4*>(kc + 2 * d + 8) = hi;
    }
  }
}

// tokens[i] <- prev_sampled[src[i]] where src[i] >= 0: fills in ids that were sampled on the
// device by the previous step and never visited the host.
__global__ void realize_future_kernel(int64_t* __restrict__ tokens, const int32_t* __restrict__ src,
                                      const int64_t* __restrict__ prev, int n) {
  pdl_wait();
  pdl_trigger();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n && src[i] >= 0) tokens[i] = prev[src[i]];
}

}  // namespace mb

namespace mb {
static bool g_pdl = false;
bool pdl_enabled() { return g_pdl; }
}  // namespace mb

using namespace mb;

// Process-wide switch for programmatic dependent launch of the step kernels (see common/launch.h).
extern "C" void mb_set_pdl(int on) { mb::g_pdl = on != 0; }
extern "C" int mb_get_pdl(void) { return mb::g_pdl ? 1 : 0; }

extern "C" int mb_realize_future_tokens(int64_t* tokens, const int32_t* src, const int64_t* prev,
                                        int n, cudaStream_t stream) {
  if (n <= 0) return MB_OK;
  launch_k(realize_future_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, tokens, src, prev, n);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

static inline unsigned blocks_for(size_t n, int threads) {
  return static_cast<unsigned>((n + threads - 1) / threads);
}
#define MB_LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH)

extern "C" int mb_rmsnorm(const void* x, const void* w, void* out, int rows, int cols, int ldx,
                          int ldo, float eps, float weight_offset, int mbc, cudaStream_t stream) {
  if (rows <= 0) return MB_OK;
  if (cols % 8 || ldx % 8 || ldo % 8 || cols > 32768) return MB_ERR_SHAPE;
  launch_k(rmsnorm_kernel<false>, dim3(rows), dim3(256), cols * 2, stream, static_cast<const bf16*>(x),
           static_cast<bf16*>(nullptr), static_cast<const bf16*>(w), static_cast<bf16*>(out), cols, ldx, ldo, eps,
           weight_offset, mbc);
  return MB_LAUNCH_OK();
}

extern "C" int mb_add_rmsnorm(const void* x, void* residual, const void* w, void* out, int rows,
                              int cols, float eps, float weight_offset, int mbc,
                              cudaStream_t stream) {
  if (rows <= 0) return MB_OK;
  if (cols % 8 || cols > 32768) return MB_ERR_SHAPE;
  launch_k(rmsnorm_kernel<true>, dim3(rows), dim3(256), cols * 2, stream, static_cast<const bf16*>(x),
           static_cast<bf16*>(residual), static_cast<const bf16*>(w), static_cast<bf16*>(out), cols, cols, cols,
           eps, weight_offset, mbc);
  return MB_LAUNCH_OK();
}

extern "C" int mb_qk_norm(void* qkv, const void* q_w, const void* k_w, int T, int n_q, int n_kv, int head_dim, int ld,
                          float eps, cudaStream_t stream) {
  if (T <= 0) return MB_OK;
  if (head_dim % 8 || head_dim > 256 || ld % 8) return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q_w) | reinterpret_cast<uintptr_t>(k_w)) & 15)
    return MB_ERR_ALIGN;
  const size_t units = static_cast<size_t>(T) * (n_q + n_kv);
  launch_k(qk_norm_kernel, dim3(blocks_for(units * 32, 256)), dim3(256), 0, stream, static_cast<bf16*>(qkv),
           static_cast<const bf16*>(q_w), static_cast<const bf16*>(k_w), T, n_q, n_kv, head_dim, ld, eps);
  return MB_LAUNCH_OK();
}

extern "C" int mb_add_bias(void* x, const void* bias, int rows, int cols, int ld, cudaStream_t stream) {
  if (rows <= 0) return MB_OK;
  if (cols % 8 || ld % 8) return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(bias)) & 15) return MB_ERR_ALIGN;
  const size_t n = static_cast<size_t>(rows) * (cols / 8);
  launch_k(add_bias_kernel, dim3(blocks_for(n, 256)), dim3(256), 0, stream, static_cast<bf16*>(x),
           static_cast<const bf16*>(bias), rows, cols, ld);
  return MB_LAUNCH_OK();
}

extern "C" int mb_silu_mul(const void* gate_up, void* out, int rows, int inter,
                           cudaStream_t stream) {
  if (rows <= 0) return MB_OK;
  if (inter % 8) return MB_ERR_SHAPE;
  const size_t n = static_cast<size_t>(rows) * (inter / 8);
  silu_mul_kernel<<<blocks_for(n, 256), 256, 0, stream>>>(static_cast<const bf16*>(gate_up),
                                                          static_cast<bf16*>(out), rows, inter);
  return MB_LAUNCH_OK();
}

extern "C" int mb_embedding(const int64_t* ids, const void* table, void* out, int n, int hidden,
                            int vocab, int vocab_start, cudaStream_t stream) {
  if (n <= 0) return MB_OK;
  if (hidden % 8) return MB_ERR_SHAPE;
  const size_t work = static_cast<size_t>(n) * (hidden / 8);
  launch_k(embedding_kernel, dim3(blocks_for(work, 256)), dim3(256), 0, stream, ids,
           static_cast<const bf16*>(table), static_cast<bf16*>(out), n, hidden, vocab, vocab_start);
  return MB_LAUNCH_OK();
}

extern "C" int mb_gather_rows(const void* src, const int32_t* idx, void* dst, int n, int row_bytes,
                              int ld_src, cudaStream_t stream) {
  if (n <= 0) return MB_OK;
  if (row_bytes % 16 || ld_src % 16) return MB_ERR_SHAPE;
  const size_t work = static_cast<size_t>(n) * (row_bytes / 16);
  launch_k(gather_rows_kernel, dim3(blocks_for(work, 256)), dim3(256), 0, stream,
           static_cast<const uint8_t*>(src), idx, static_cast<uint8_t*>(dst), n, row_bytes, ld_src);
  return MB_LAUNCH_OK();
}

extern "C" int mb_rope_kv_store(void* qkv, const int32_t* positions, const int64_t* slots,
                                const float* cos_sin, void* k_cache, void* v_cache, int T, int n_q,
                                int n_kv, int head_dim, int page_size, int64_t page_stride,
                                int64_t head_stride, int interleaved, cudaStream_t stream) {
  if (T <= 0) return MB_OK;
  if (head_dim % 16) return MB_ERR_SHAPE;
  const int work_per_tok = (n_q + n_kv) * (head_dim / 16) + n_kv * (head_dim / 8);
  const size_t work = static_cast<size_t>(T) * work_per_tok;
  launch_k(rope_kv_store_kernel, dim3(blocks_for(work, 256)), dim3(256), 0, stream, static_cast<bf16*>(qkv),
           positions, slots, cos_sin, static_cast<bf16*>(k_cache), static_cast<bf16*>(v_cache), T, n_q, n_kv,
           head_dim, page_size, page_stride, head_stride, interleaved);
  return MB_LAUNCH_OK();
}
