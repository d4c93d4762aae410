// Mixture-of-experts routing and token shuffling.
//
//   moe_router_group_limited  DeepSeek-V3 routing: sigmoid scores (+ correction bias for the
//                             choice only), sum of the top-2 scores per expert group, keep the
//                             best `topk_group` groups, top-k experts inside them, weights from
//                             the un-biased scores, optional normalisation, times a scaling factor.
//   moe_router_softmax_topk   plain softmax top-k routing (Mixtral / Qwen style).
//   moe_create_indices        counting sort of (token, slot) pairs by expert: CSR offsets per
//                             expert, the permutation and its inverse.
//   moe_permute_rows          gather token rows into expert order (optionally fused with the
//                             1x128 fp8 quantisation of the activations).
//   moe_combine               y[t] = sum_k w[t,k] * expert_out[pos(t,k)] (+ shared-expert rows).
//
// Reference counterparts: max/kernels/src/nn/moe.mojo:789 (group_limited_router_kernel), :435
// (moe_create_indices), max/python/max/nn/moe/moe.py:743-865 (gather / un-permute / weighted sum).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "../common/api.h"

namespace mb {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

struct ArgMaxF {
  float v;
  int i;
};
__device__ __forceinline__ ArgMaxF amax(ArgMaxF a, ArgMaxF b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}
__device__ __forceinline__ ArgMaxF block_amax(ArgMaxF a, ArgMaxF* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMaxF b{__shfl_xor_sync(0xffffffffu, a.v, o), __shfl_xor_sync(0xffffffffu, a.i, o)};
    a = amax(a, b);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = (blockDim.x + 31) >> 5;
  if (lane == 0) sh[warp] = a;
  __syncthreads();
  ArgMaxF r = lane < nw ? sh[lane] : ArgMaxF{-FLT_MAX, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMaxF b{__shfl_xor_sync(0xffffffffu, r.v, o), __shfl_xor_sync(0xffffffffu, r.i, o)};
    r = amax(r, b);
  }
  __syncthreads();
  return r;
}

// One CTA per token, one thread per expert (E <= 1024).
__global__ void router_group_limited_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                            int32_t* __restrict__ topk_ids, float* __restrict__ topk_w,
                                            int E, int n_group, int topk_group, int top_k,
                                            int norm_topk, float scaling, int ld) {
  extern __shared__ float sh[];            // scores_for_choice [E] | group score [n_group] | keep [n_group]
  __shared__ ArgMaxF red[32];
  __shared__ float wsum;
  float* choice = sh;
  float* gscore = sh + E;
  int* gkeep = reinterpret_cast<int*>(gscore + n_group);
  const int t = blockIdx.x, e = threadIdx.x;
  const int gsize = E / n_group;
  float score = 0.f;
  if (e < E) {
    score = 1.f / (1.f + __expf(-logits[static_cast<size_t>(t) * ld + e]));
    choice[e] = score + (bias ? bias[e] : 0.f);
  }
  __syncthreads();
  // group score = sum of the two largest choice scores of the group
  if (e < n_group) {
    float m1 = -FLT_MAX, m2 = -FLT_MAX;
    for (int j = 0; j < gsize; ++j) {
      const float v = choice[e * gsize + j];
      if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
    }
    gscore[e] = gsize > 1 ? m1 + m2 : m1;
    gkeep[e] = 0;
  }
  __syncthreads();
  if (e == 0) {
    for (int k = 0; k < topk_group; ++k) {
      int best = -1;
      float bv = -FLT_MAX;
      for (int g = 0; g < n_group; ++g)
        if (!gkeep[g] && gscore[g] > bv) { bv = gscore[g]; best = g; }
      if (best >= 0) gkeep[best] = 1;
    }
    wsum = 0.f;
  }
  __syncthreads();
  float mine = (e < E && gkeep[e / gsize]) ? choice[e] : -FLT_MAX;
  for (int k = 0; k < top_k; ++k) {
    const ArgMaxF w = block_amax(ArgMaxF{mine, e < E ? e : 0x7fffffff}, red);
    if (e == w.i) {
      topk_ids[static_cast<size_t>(t) * top_k + k] = e;
      topk_w[static_cast<size_t>(t) * top_k + k] = score;
      atomicAdd(&wsum, score);
      mine = -FLT_MAX;
    }
  }
  __syncthreads();
  if (e < top_k) {
    float w = topk_w[static_cast<size_t>(t) * top_k + e];
    if (norm_topk) w /= (wsum + 1e-20f);
    topk_w[static_cast<size_t>(t) * top_k + e] = w * scaling;
  }
}

__global__ void router_softmax_topk_kernel(const float* __restrict__ logits, int32_t* __restrict__ topk_ids,
                                           float* __restrict__ topk_w, int E, int top_k, int norm_topk,
                                           int ld) {
  __shared__ ArgMaxF red[32];
  __shared__ float ssum, wsum;
  const int t = blockIdx.x, e = threadIdx.x;
  const float x = e < E ? logits[static_cast<size_t>(t) * ld + e] : -FLT_MAX;
  const ArgMaxF mx = block_amax(ArgMaxF{x, e}, red);
  if (e == 0) { ssum = 0.f; wsum = 0.f; }
  __syncthreads();
  const float p = e < E ? __expf(x - mx.v) : 0.f;
  atomicAdd(&ssum, p);
  __syncthreads();
  const float prob = p / ssum;
  float mine = e < E ? prob : -FLT_MAX;
  for (int k = 0; k < top_k; ++k) {
    const ArgMaxF w = block_amax(ArgMaxF{mine, e < E ? e : 0x7fffffff}, red);
    if (e == w.i) {
      topk_ids[static_cast<size_t>(t) * top_k + k] = e;
      topk_w[static_cast<size_t>(t) * top_k + k] = prob;
      atomicAdd(&wsum, prob);
      mine = -FLT_MAX;
    }
  }
  __syncthreads();
  if (e < top_k && norm_topk) topk_w[static_cast<size_t>(t) * top_k + e] /= (wsum + 1e-20f);
}

// ---- counting sort by expert -------------------------------------------------------------
__global__ void moe_count_kernel(const int32_t* __restrict__ ids, int n, int32_t* __restrict__ counts,
                                 int E, int e_begin, int e_end) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = ids[i];
  if (e >= e_begin && e < e_end) atomicAdd(&counts[e - e_begin], 1);
}
// offsets[0..E] = exclusive scan of counts; cursor[e] = offsets[e]; counts are cleared.
__global__ void moe_scan_kernel(int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                                int32_t* __restrict__ cursor, int E) {
  __shared__ int32_t s[1025];
  const int e = threadIdx.x;
  s[e] = e < E ? counts[e] : 0;
  __syncthreads();
  if (e == 0) {
    int32_t acc = 0;
    for (int i = 0; i < E; ++i) { const int32_t c = s[i]; s[i] = acc; acc += c; }
    s[E] = acc;
  }
  __syncthreads();
  if (e <= E) offsets[e] = s[e];
  if (e < E) { cursor[e] = s[e]; counts[e] = 0; }
}
// order[pos] = flat (token*top_k + slot); inverse[flat] = pos (or -1 for experts outside the range)
__global__ void moe_scatter_kernel(const int32_t* __restrict__ ids, int n, int32_t* __restrict__ cursor,
                                   int32_t* __restrict__ order, int32_t* __restrict__ inverse,
                                   int e_begin, int e_end) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = ids[i];
  if (e >= e_begin && e < e_end) {
    const int pos = atomicAdd(&cursor[e - e_begin], 1);
    order[pos] = i;
    inverse[i] = pos;
  } else {
    inverse[i] = -1;
  }
}

// dst[p] = src[order[p] / top_k]  (16 bytes per thread)
__global__ void moe_permute_rows_kernel(const uint8_t* __restrict__ src, const int32_t* __restrict__ order,
                                        const int32_t* __restrict__ n_rows_dev, uint8_t* __restrict__ dst,
                                        int max_rows, int row_bytes, int top_k) {
  const int per_row = row_bytes >> 4;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int n_rows = n_rows_dev ? min(*n_rows_dev, max_rows) : max_rows;
  if (i >= static_cast<long long>(n_rows) * per_row) return;
  const int p = static_cast<int>(i / per_row), c = static_cast<int>(i % per_row) * 16;
  const int t = order[p] / top_k;
  *reinterpret_cast<uint4*>(dst + static_cast<size_t>(p) * row_bytes + c) =
      *reinterpret_cast<const uint4*>(src + static_cast<size_t>(t) * row_bytes + c);
}

// y[t] = (shared ? shared[t] : 0) + sum_k w[t,k] * expert_out[inverse[t*top_k+k]]
__global__ void moe_combine_kernel(const bf16* __restrict__ expert_out, const int32_t* __restrict__ inverse,
                                   const float* __restrict__ w, const bf16* __restrict__ shared,
                                   bf16* __restrict__ y, int T, int H, int top_k) {
  const int per_row = H >> 3;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(T) * per_row) return;
  const int t = static_cast<int>(i / per_row), c = static_cast<int>(i % per_row) * 8;
  float acc[8];
  if (shared) {
    const uint4 sv = *reinterpret_cast<const uint4*>(shared + static_cast<size_t>(t) * H + c);
    const bf162* sp = reinterpret_cast<const bf162*>(&sv);
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(sp[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  }
  for (int k = 0; k < top_k; ++k) {
    const int pos = inverse[static_cast<size_t>(t) * top_k + k];
    if (pos < 0) continue;
    const float wk = w[static_cast<size_t>(t) * top_k + k];
    const uint4 ev = *reinterpret_cast<const uint4*>(expert_out + static_cast<size_t>(pos) * H + c);
    const bf162* ep = reinterpret_cast<const bf162*>(&ev);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(ep[j]);
      acc[2 * j] = fmaf(wk, f.x, acc[2 * j]);
      acc[2 * j + 1] = fmaf(wk, f.y, acc[2 * j + 1]);
    }
  }
  uint4 out;
  bf162* op = reinterpret_cast<bf162*>(&out);
#pragma unroll
  for (int j = 0; j < 4; ++j) op[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
  *reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * H + c) = out;
}

}  // namespace mb

using namespace mb;
#define MB_OK_OR_LAUNCH() (cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH)

extern "C" int mb_moe_router_group_limited(const float* logits, const float* bias, int32_t* topk_ids,
                                           float* topk_w, int T, int E, int n_group, int topk_group,
                                           int top_k, int norm_topk, float scaling, int ld,
                                           cudaStream_t stream) {
  if (T <= 0) return MB_OK;
  if (E > 1024 || n_group < 1 || E % n_group || top_k > E || topk_group > n_group) return MB_ERR_SHAPE;
  const int threads = ((E + 31) / 32) * 32;
  router_group_limited_kernel<<<T, threads, (E + 2 * n_group) * sizeof(float), stream>>>(
      logits, bias, topk_ids, topk_w, E, n_group, topk_group, top_k, norm_topk, scaling, ld);
  return MB_OK_OR_LAUNCH();
}

extern "C" int mb_moe_router_softmax_topk(const float* logits, int32_t* topk_ids, float* topk_w, int T,
                                          int E, int top_k, int norm_topk, int ld, cudaStream_t stream) {
  if (T <= 0) return MB_OK;
  if (E > 1024 || top_k > E) return MB_ERR_SHAPE;
  router_softmax_topk_kernel<<<T, ((E + 31) / 32) * 32, 0, stream>>>(logits, topk_ids, topk_w, E, top_k,
                                                                     norm_topk, ld);
  return MB_OK_OR_LAUNCH();
}

// counts: int32[E_local] zeroed scratch (left zeroed); offsets: int32[E_local+1]; cursor: int32[E_local].
// Only experts in [e_begin, e_end) are kept (expert parallel: this rank's experts).
extern "C" int mb_moe_create_indices(const int32_t* topk_ids, int n_pairs, int e_begin, int e_end,
                                     int32_t* counts, int32_t* offsets, int32_t* cursor, int32_t* order,
                                     int32_t* inverse, cudaStream_t stream) {
  const int E = e_end - e_begin;
  if (E <= 0 || E > 1024) return MB_ERR_SHAPE;
  if (n_pairs > 0)
    moe_count_kernel<<<(n_pairs + 255) / 256, 256, 0, stream>>>(topk_ids, n_pairs, counts, E, e_begin, e_end);
  moe_scan_kernel<<<1, 1024, 0, stream>>>(counts, offsets, cursor, E);
  if (n_pairs > 0)
    moe_scatter_kernel<<<(n_pairs + 255) / 256, 256, 0, stream>>>(topk_ids, n_pairs, cursor, order, inverse,
                                                                 e_begin, e_end);
  return MB_OK_OR_LAUNCH();
}

extern "C" int mb_moe_permute_rows(const void* src, const int32_t* order, const int32_t* n_rows_dev,
                                   void* dst, int max_rows, int row_bytes, int top_k, cudaStream_t stream) {
  if (max_rows <= 0) return MB_OK;
  if (row_bytes % 16) return MB_ERR_SHAPE;
  const long long work = static_cast<long long>(max_rows) * (row_bytes / 16);
  moe_permute_rows_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint8_t*>(src), order, n_rows_dev, static_cast<uint8_t*>(dst), max_rows, row_bytes,
      top_k);
  return MB_OK_OR_LAUNCH();
}

extern "C" int mb_moe_combine(const void* expert_out, const int32_t* inverse, const float* w,
                              const void* shared, void* y, int T, int H, int top_k, cudaStream_t stream) {
  if (T <= 0) return MB_OK;
  if (H % 8) return MB_ERR_SHAPE;
  const long long work = static_cast<long long>(T) * (H / 8);
  moe_combine_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, stream>>>(
      static_cast<const bf16*>(expert_out), inverse, w, static_cast<const bf16*>(shared),
      static_cast<bf16*>(y), T, H, top_k);
  return MB_OK_OR_LAUNCH();
}
