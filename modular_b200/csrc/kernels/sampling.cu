// Token sampling on the device: greedy argmax, temperature / top-k / top-p / min-p
// sampling with per-request seeds, and frequency / presence / repetition penalties.
//
// One CTA of 1024 threads owns one batch row. Top-k and top-p cut-offs are found by
// bisection on the order-preserving integer image of the fp32 logits, so no sort and
// no scratch memory is needed; pure temperature sampling takes the one-pass Gumbel-max
// route. Behavioural counterparts in the reference: max/kernels/src/nn/topk.mojo
// (fused token sampling :2037, Gumbel argmax :2369), nn/sampling/topk_fi.mojo,
// nn/sampling/sampling.mojo:31 (penalties).
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace mb {

constexpr int kSampThreads = 1024;

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t step, uint64_t idx) {
  const uint64_t h = mix64(mix64(seed ^ (step * 0xD1342543DE82EF95ull)) + idx);
  return (static_cast<float>(h >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0,1)
}
// Monotone map fp32 -> uint32 (larger float <=> larger key).
__device__ __forceinline__ uint32_t fkey(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float fkey_inv(uint32_t k) {
  const uint32_t u = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
  return __uint_as_float(u);
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax amax2(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ ArgMax block_argmax(ArgMax a, ArgMax* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = amax2(a, b);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sh[warp] = a;
  __syncthreads();
  ArgMax r = lane < (blockDim.x >> 5) ? sh[lane] : ArgMax{-FLT_MAX, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, r.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, r.i, o);
    r = amax2(r, b);
  }
  __syncthreads();
  return r;
}
__device__ __forceinline__ float block_sum_f(float v, float* sh) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) sh[warp] = v;
  __syncthreads();
  float r = lane < (blockDim.x >> 5) ? sh[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
  __syncthreads();
  return r;
}

// Visit every element of a row as f(value, index). Rows that start on a 16-byte boundary are read as float4 with
// four loads in flight per thread: with one scalar load per iteration a pass over 128 k logits is bound by
// the latency of its 125 dependent round trips (about 60 us per pass on B200), not by bandwidth.
template <typename F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ row, int vocab, F&& f) {
  if ((reinterpret_cast<uintptr_t>(row) & 15) != 0) {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) f(row[i], i);
    return;
  }
  const int n4 = vocab >> 2;
  const float4* __restrict__ r4 = reinterpret_cast<const float4*>(row);
  const int step = blockDim.x;
  int i = threadIdx.x;
  for (; i + 3 * step < n4; i += 4 * step) {
    const float4 a = r4[i];
    const float4 b = r4[i + step];
    const float4 c = r4[i + 2 * step];
    const float4 d = r4[i + 3 * step];
    const int ia = i << 2, ib = (i + step) << 2, ic = (i + 2 * step) << 2, id = (i + 3 * step) << 2;
    f(a.x, ia); f(a.y, ia + 1); f(a.z, ia + 2); f(a.w, ia + 3);
    f(b.x, ib); f(b.y, ib + 1); f(b.z, ib + 2); f(b.w, ib + 3);
    f(c.x, ic); f(c.y, ic + 1); f(c.z, ic + 2); f(c.w, ic + 3);
    f(d.x, id); f(d.y, id + 1); f(d.z, id + 2); f(d.w, id + 3);
  }
  for (; i < n4; i += step) {
    const float4 a = r4[i];
    const int ia = i << 2;
    f(a.x, ia); f(a.y, ia + 1); f(a.z, ia + 2); f(a.w, ia + 3);
  }
  for (int t = (n4 << 2) + threadIdx.x; t < vocab; t += blockDim.x) f(row[t], t);
}

__global__ void __launch_bounds__(kSampThreads)
argmax_kernel(const float* __restrict__ logits, int64_t* __restrict__ out, int vocab, int ld) {
  __shared__ ArgMax sh[32];
  const float* row = logits + static_cast<size_t>(blockIdx.x) * ld;
  ArgMax a{-FLT_MAX, 0x7fffffff};
  for_each_logit(row, vocab, [&](float v, int i) { a = amax2(a, ArgMax{v, i}); });
  a = block_argmax(a, sh);
  if (threadIdx.x == 0) out[blockIdx.x] = a.i;
}

// ---- threshold search for the top-k / top-p filters
// Wanted: the largest key t with measure{ i : fkey(x_i) >= t } >= target, where the measure is a count
// (MASS = false) or the softmax mass exp(x_i - mx) (MASS = true). The search keeps an interval [lo, hi]
// that holds t and `above` = measure{ key > hi }. One sixteen-way pass evaluates fifteen thresholds at
// once (per-thread bucket accumulators, one block reduction) and shrinks the interval sixteen-fold. A pass
// over the whole row costs about 70 instructions per element, so before every such pass the elements that
// still lie inside [lo, hi] are collected into shared memory; as soon as they fit (they do after one or
// two passes for any peaked distribution) the rest of the search runs on that list alone.
constexpr int kListPerWarp = 256;

struct SearchSmem {
  float list[(kSampThreads / 32) * kListPerWarp];   // per warp, in index order: x_i / T of the candidates
  float acc[(kSampThreads / 32) * 16];
  int wcnt[kSampThreads / 32];
  int over;
};

// Per warp (warp w scans its own contiguous share of the row): x / T of the elements with key in [lo, hi].
// Returns false if some warp found more than it can hold.
__device__ bool compact_range(const float* __restrict__ row, int vocab, float invT, uint32_t lo, uint32_t hi,
                              SearchSmem* sm) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) sm->over = 0;
  __syncthreads();
  // each warp owns a contiguous share of the row (a multiple of 128 elements, so float4 loads stay aligned);
  // candidates are appended in a fixed order (element slot of the float4, then lane), which keeps the list -
  // and with it every later floating-point sum - the same from run to run
  const int seg = (((vocab + 31) / 32) + 127) & ~127;
  const int beg = warp * seg;
  const int end = beg + seg < vocab ? beg + seg : vocab;
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  int cnt = 0;   // warp-uniform
  for (int i0 = beg; i0 < end && cnt <= kListPerWarp; i0 += 128) {
    const int i = i0 + 4 * lane;
    float xv[4] = {0.f, 0.f, 0.f, 0.f};
    if (vec && i + 3 < end) {
      const float4 q = *reinterpret_cast<const float4*>(row + i);
      xv[0] = q.x; xv[1] = q.y; xv[2] = q.z; xv[3] = q.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) xv[e] = i + e < end ? row[i + e] : 0.f;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float x = xv[e] * invT;
      const uint32_t key = fkey(x);
      const bool in = i + e < end && key >= lo && key <= hi;
      const uint32_t m = __ballot_sync(0xffffffffu, in);
      if (in) {
        const int pos = cnt + __popc(m & ((1u << lane) - 1u));
        if (pos < kListPerWarp) sm->list[warp * kListPerWarp + pos] = x;
      }
      cnt += __popc(m);
    }
  }
  if (lane == 0) {
    sm->wcnt[warp] = cnt < kListPerWarp ? cnt : kListPerWarp;
    if (cnt > kListPerWarp) sm->over = 1;
  }
  __syncthreads();
  return sm->over == 0;
}

// One sixteen-way pass over the row (LIST = false) or over the collected candidates (LIST = true).
template <bool MASS, bool LIST>
__device__ void multiway_pass(const float* __restrict__ row, int vocab, float invT, float mx, SearchSmem* sm,
                              uint32_t& lo, uint32_t& hi, float target, float& above) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // bucket j = [lo + (j << sh), lo + ((j + 1) << sh)): a power-of-two width makes the bucket index a shift
  // (a division per element costs as much as the sixteen accumulations); sixteen buckets cover [lo, hi]
  const uint32_t span16 = (hi - lo) >> 4;
  const int sh = span16 == 0 ? 0 : 32 - __clz(span16);
  const uint32_t width = 1u << sh;
  float acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.f;
  auto visit = [&](float x) {
    const uint32_t key = fkey(x);
    if (key < lo || key > hi) return;
    const int b = static_cast<int>((key - lo) >> sh);
    const float w = MASS ? __expf(x - mx) : 1.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) acc[j] += (b == j) ? w : 0.f;
  };
  if (LIST) {
    const int n = sm->wcnt[warp];
    for (int q = lane; q < n; q += 32) visit(sm->list[warp * kListPerWarp + q]);
  } else {
    for_each_logit(row, vocab, [&](float v, int) { visit(v * invT); });
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    if (lane == 0) sm->acc[warp * 16 + j] = acc[j];
  }
  __syncthreads();
  // every thread derives the same decision: the highest bucket whose suffix measure reaches the target
  float run = above, above_new = 0.f;
  int best = 0;
  bool found = false;
  for (int j = 15; j >= 1; --j) {
    float t = 0.f;
    for (int q = 0; q < (kSampThreads / 32); ++q) t += sm->acc[q * 16 + j];
    if (!found && run + t >= target) { best = j; found = true; above_new = run; }
    run += t;
  }
  if (!found) above_new = run;   // bucket 0 (its lower end is lo itself, which qualifies by the invariant)
  __syncthreads();
  // a qualifying bucket holds a key, so lo + best * width cannot wrap; the bucket's upper end can
  lo += static_cast<uint32_t>(best) * width;
  const uint64_t new_hi = static_cast<uint64_t>(lo) + width - 1;
  hi = new_hi < hi ? static_cast<uint32_t>(new_hi) : hi;
  above = above_new;
}

// Count (or softmax mass) of the collected candidates; every thread gets the same value.
template <bool MASS>
__device__ float list_measure(SearchSmem* sm, float mx) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float v = 0.f;
  if (MASS) {
    const int n = sm->wcnt[warp];
    for (int q = lane; q < n; q += 32) v += __expf(sm->list[warp * kListPerWarp + q] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  } else {
    v = static_cast<float>(sm->wcnt[warp]);
  }
  __syncthreads();
  if (lane == 0) sm->acc[warp] = v;
  __syncthreads();
  float tot = 0.f;
  for (int q = 0; q < kSampThreads / 32; ++q) tot += sm->acc[q];
  __syncthreads();
  return tot;
}

// Requires measure{ key >= lo } >= target and measure{ key > hi } == 0 on entry (hi = key of the maximum).
template <bool MASS>
__device__ uint32_t find_threshold(const float* __restrict__ row, int vocab, float invT, float mx, uint32_t lo,
                                   uint32_t hi, float target, SearchSmem* sm) {
  float above = 0.f;
  // Shortcut for the usual case that the wanted set sits within a few units below the maximum: collect the
  // elements of a window under the maximum in one cheap pass; if they fit and already reach the target, the
  // whole search runs on that list. Windows that hold too much (flat distributions) or too little fall
  // through to the general search.
  for (int wi = 0; wi < 3 && lo < hi; ++wi) {
    const float window = wi == 0 ? 2.f : (wi == 1 ? 6.f : 12.f);
    const uint32_t wlo = fkey(mx - window);
    if (wlo <= lo) break;                                   // the window is the whole remaining range
    if (!compact_range(row, vocab, invT, wlo, hi, sm)) break;   // too many candidates
    if (list_measure<MASS>(sm, mx) >= target) {
      lo = wlo;
      while (lo < hi) multiway_pass<MASS, true>(row, vocab, invT, mx, sm, lo, hi, target, above);
      return lo;
    }
  }
  while (lo < hi) {
    if (compact_range(row, vocab, invT, lo, hi, sm)) {
      while (lo < hi) multiway_pass<MASS, true>(row, vocab, invT, mx, sm, lo, hi, target, above);
      return lo;
    }
    multiway_pass<MASS, false>(row, vocab, invT, mx, sm, lo, hi, target, above);
  }
  return lo;
}

__global__ void __launch_bounds__(kSampThreads, 1)
sample_kernel(const float* __restrict__ logits, int64_t* __restrict__ out, int vocab, int ld,
              const float* __restrict__ temperature, const int32_t* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p,
              const uint64_t* __restrict__ seeds, uint64_t step) {
  __shared__ ArgMax sh_am[32];
  __shared__ float sh_f[32];
  __shared__ float sh_scan[kSampThreads / 32];
  __shared__ SearchSmem sh_search;
  __shared__ int sh_pick;
  pdl_wait();
  pdl_trigger();
  const int rowi = blockIdx.x;
  const float* row = logits + static_cast<size_t>(rowi) * ld;
  const float T = temperature ? temperature[rowi] : 1.f;
  const int k = top_k ? top_k[rowi] : 0;
  const float tp = top_p ? top_p[rowi] : 1.f;
  const float mp = min_p ? min_p[rowi] : 0.f;
  const uint64_t seed = seeds ? seeds[rowi] : 0x1234ull + rowi;

  // greedy
  if (T <= 0.f || k == 1) {
    ArgMax a{-FLT_MAX, 0x7fffffff};
    for_each_logit(row, vocab, [&](float v, int i) { a = amax2(a, ArgMax{v, i}); });
    a = block_argmax(a, sh_am);
    if (threadIdx.x == 0) out[rowi] = a.i;
    return;
  }
  const float invT = 1.f / T;
  const bool use_k = k > 0 && k < vocab, use_p = tp < 1.f, use_m = mp > 0.f;
  if (!use_k && !use_p && !use_m) {
    // Gumbel-max: argmax(x/T + g), g = -log(-log u)
    ArgMax a{-FLT_MAX, 0x7fffffff};
    for_each_logit(row, vocab, [&](float v, int i) {
      const float u = uniform01(seed, step, i);
      a = amax2(a, ArgMax{v * invT - __logf(-__logf(u)), i});
    });
    a = block_argmax(a, sh_am);
    if (threadIdx.x == 0) out[rowi] = a.i;
    return;
  }
  // max of scaled logits
  ArgMax a{-FLT_MAX, 0x7fffffff};
  for_each_logit(row, vocab, [&](float v, int i) { a = amax2(a, ArgMax{v * invT, i}); });
  a = block_argmax(a, sh_am);
  const float mx = a.v;
  uint32_t thr_key = 0;  // keep x with fkey(x*invT) >= thr_key
  if (use_k) {
    // largest key t with count(key >= t) >= k
    const uint32_t lo = find_threshold<false>(row, vocab, invT, mx, 0u, fkey(mx), static_cast<float>(k), &sh_search);
    thr_key = lo;
  }
  if (use_m) {
    const uint32_t km = fkey(mx + __logf(mp));
    thr_key = max(thr_key, km);
  }
  float Z = 0.f;
  for_each_logit(row, vocab, [&](float v, int) {
    const float x = v * invT;
    Z += fkey(x) >= thr_key ? __expf(x - mx) : 0.f;
  });
  Z = block_sum_f(Z, sh_f);
  if (use_p) {
    // largest key t (>= thr_key) with mass(key >= t) >= tp * Z
    const float target = tp * Z;
    const uint32_t lo = find_threshold<true>(row, vocab, invT, mx, thr_key, fkey(mx), target, &sh_search);
    thr_key = lo;
    Z = 0.f;
    for_each_logit(row, vocab, [&](float v, int) {
      const float x = v * invT;
      Z += fkey(x) >= thr_key ? __expf(x - mx) : 0.f;
    });
    Z = block_sum_f(Z, sh_f);
  }
  // inverse-CDF draw over the kept set, in index order
  const float target = uniform01(seed, step, 0xffffffffull) * Z;
  if (threadIdx.x == 0) sh_pick = -1;
  __syncthreads();
  float base = 0.f;
  int last_kept = -1;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  for (int c0 = 0; c0 < vocab; c0 += 4 * kSampThreads) {
    // four consecutive elements per thread and iteration
    const int i = c0 + 4 * threadIdx.x;
    float xv[4] = {0.f, 0.f, 0.f, 0.f};
    if (vec && i + 3 < vocab) {
      const float4 q = *reinterpret_cast<const float4*>(row + i);
      xv[0] = q.x; xv[1] = q.y; xv[2] = q.z; xv[3] = q.w;
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) xv[e] = i + e < vocab ? row[i + e] : 0.f;
    }
    float w[4];
    float mine = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float x = xv[e] * invT;
      w[e] = (i + e < vocab && fkey(x) >= thr_key) ? __expf(x - mx) : 0.f;
      mine += w[e];
    }
    float incl = mine;  // warp inclusive scan of the per-thread sums
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) sh_scan[warp] = incl;
    __syncthreads();
    float woff = 0.f, total = 0.f;
    for (int q = 0; q < kSampThreads / 32; ++q) {
      const float t = sh_scan[q];
      if (q < warp) woff += t;
      total += t;
    }
    float cum = base + woff + incl - mine;   // mass before this thread's first element
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (w[e] > 0.f) {
        if (cum + w[e] >= target && cum < target) atomicMax(&sh_pick, i + e);
        last_kept = i + e;
      }
      cum += w[e];
    }
    base += total;
    __syncthreads();
    if (sh_pick >= 0) break;
  }
  if (sh_pick < 0) {
    // rounding left the target just above the total mass: take the last kept index
    ArgMax b{static_cast<float>(last_kept), last_kept < 0 ? 0x7fffffff : -last_kept};
    b = block_argmax(b, sh_am);
    if (threadIdx.x == 0) out[rowi] = b.v >= 0.f ? static_cast<int64_t>(b.v) : a.i;
  } else if (threadIdx.x == 0) {
    out[rowi] = sh_pick;
  }
}

// One thread per (row, distinct history token). counts > 0 are output-token counts for
// frequency/presence; repetition applies to every listed token.
__global__ void penalties_kernel(float* __restrict__ logits, int rows, int vocab, int ld,
                                 const int32_t* __restrict__ tok, const int32_t* __restrict__ cnt,
                                 const int32_t* __restrict__ offsets, const float* __restrict__ freq,
                                 const float* __restrict__ pres, const float* __restrict__ rep) {
  const int row = blockIdx.y;
  const int beg = offsets[row], end = offsets[row + 1];
  for (int j = beg + blockIdx.x * blockDim.x + threadIdx.x; j < end; j += gridDim.x * blockDim.x) {
    const int t = tok[j];
    if (t < 0 || t >= vocab) continue;
    float x = logits[static_cast<size_t>(row) * ld + t];
    const float r = rep ? rep[row] : 1.f;
    if (r != 1.f) x = x > 0.f ? x / r : x * r;
    const int c = cnt[j];
    if (c > 0) x -= (freq ? freq[row] : 0.f) * c + (pres ? pres[row] : 0.f);
    logits[static_cast<size_t>(row) * ld + t] = x;
  }
}

}  // namespace mb

using namespace mb;

extern "C" int mb_argmax(const float* logits, int64_t* out, int rows, int vocab, int ld,
                         cudaStream_t stream) {
  if (rows <= 0) return MB_OK;
  argmax_kernel<<<rows, kSampThreads, 0, stream>>>(logits, out, vocab, ld);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_sample_topk_topp(const float* logits, int64_t* out, int rows, int vocab, int ld,
                                   const float* temperature, const int32_t* top_k,
                                   const float* top_p, const float* min_p, const uint64_t* seeds,
                                   uint64_t step, cudaStream_t stream) {
  if (rows <= 0) return MB_OK;
  return launch_k(sample_kernel, dim3(rows), dim3(kSampThreads), 0, stream, logits, out, vocab, ld, temperature,
                  top_k, top_p, min_p, seeds, step) == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

// logits[r, v] = -inf where bit (v % 32) of bitmask[r, v / 32] is clear (grammar-constrained decoding)
__global__ void token_bitmask_kernel(float* __restrict__ logits, const int32_t* __restrict__ bitmask, int vocab,
                                     int ld, int words) {
  const int r = blockIdx.y;
  for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < vocab; v += gridDim.x * blockDim.x)
    if (!((static_cast<uint32_t>(bitmask[static_cast<size_t>(r) * words + (v >> 5)]) >> (v & 31)) & 1u))
      logits[static_cast<size_t>(r) * ld + v] = -INFINITY;
}

extern "C" int mb_apply_token_bitmask(float* logits, const int32_t* bitmask, int rows, int vocab, int ld,
                                      cudaStream_t stream) {
  if (rows <= 0) return MB_OK;
  token_bitmask_kernel<<<dim3(16, rows), 256, 0, stream>>>(logits, bitmask, vocab, ld, (vocab + 31) / 32);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_apply_penalties(float* logits, int rows, int vocab, int ld, const int32_t* tok,
                                  const int32_t* cnt, const int32_t* offsets, const float* freq,
                                  const float* pres, const float* rep, cudaStream_t stream) {
  if (rows <= 0) return MB_OK;
  penalties_kernel<<<dim3(8, rows), 256, 0, stream>>>(logits, rows, vocab, ld, tok, cnt, offsets,
                                                      freq, pres, rep);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}
