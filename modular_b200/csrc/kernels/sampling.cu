// Token sampling on the device: greedy argmax, temperature / top-k / top-p / min-p
// sampling with per-request seeds, and frequency / presence / repetition penalties.
//
// sample_kernel: one CTA of 1024 threads owns one batch row. Top-k and top-p cut-offs are found by
// bisection on the order-preserving integer image of the fp32 logits, so no sort and
// no scratch memory is needed; pure temperature sampling takes the one-pass Gumbel-max
// route. sample_cluster_kernel, launched before it for rows with a filter, spreads a row over a thread-block
// cluster and leaves only the rows it cannot take. Behavioural counterparts in the reference: max/kernels/src/nn/topk.mojo
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
  float tot[16];
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
  bool empty = false;   // warp-uniform: a warp without candidates has nothing to add up
  if (LIST) {
    const int n = sm->wcnt[warp];
    empty = n == 0;
    for (int q = lane; q < n; q += 32) visit(sm->list[warp * kListPerWarp + q]);
  } else {
    for_each_logit(row, vocab, [&](float v, int) { visit(v * invT); });
  }
  if (empty) {
    if (lane < 16) sm->acc[warp * 16 + lane] = 0.f;
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
      if (lane == 0) sm->acc[warp * 16 + j] = acc[j];
    }
  }
  __syncthreads();
  // warp j adds bucket j over the 32 warps (lane q holds warp q's share); a loop over all of them in every
  // thread would cost 480 shared-memory reads per thread and pass, several microseconds
  if (warp < 16) {
    float t = sm->acc[lane * 16 + warp];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) sm->tot[warp] = t;
  }
  __syncthreads();
  // every thread derives the same decision: the highest bucket whose suffix measure reaches the target
  float run = above, above_new = 0.f;
  int best = 0;
  bool found = false;
  for (int j = 15; j >= 1; --j) {
    const float t = sm->tot[j];
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
              const uint64_t* __restrict__ seeds, uint64_t step, int only_pending) {
  __shared__ ArgMax sh_am[32];
  __shared__ float sh_f[32];
  __shared__ float sh_scan[kSampThreads / 32];
  __shared__ SearchSmem sh_search;
  __shared__ int sh_pick;
  pdl_wait();
  pdl_trigger();
  const int rowi = blockIdx.x;
  if (only_pending && out[rowi] >= 0) return;   // sample_cluster_kernel already drew this row
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

// ---- truncated sampling with a row spread over a cluster of eight CTAs
// sample_kernel walks a row with one CTA, so a batch of 64 rows keeps 64 SMs busy with eight or more
// latency-bound passes each. Here the 256 warps of a cluster each own a contiguous share of the row and
// read it three times (L2 hits after the first): maximum; candidate counts and softmax mass inside three
// windows below the maximum; then the candidates of the smallest window that provably holds the whole kept
// set are written, in index order, into the list of the cluster's first CTA through distributed shared
// memory. That CTA finds the top-k / top-p cut-offs and draws the token on the list alone. A row whose kept
// set does not fit a window (flat distributions, huge k) gets out[row] = -1 and is left to sample_kernel,
// as are greedy and plain-temperature rows.
constexpr int kClu = 8;   // largest cluster; the launcher picks 8, 4, 2 or 1 CTAs per row from the batch size
constexpr int kCluList = (kSampThreads / 32) * kListPerWarp;
// Histogram under the maximum: bin b holds the elements with b <= mx - x / T < b + 1. "Window w" is bins 0..w.
constexpr int kCntBins = 32;    // counts reach 32 units down (a top-k of a few hundred on a peaked row)
static_assert(kListPerWarp * (kSampThreads / 32) >= 4 * kSampThreads, "room for the rank-ordered copies");
static_assert(kCntBins == kSampThreads / 32, "one warp adds up one count bin");
constexpr int kMassBins = 16;   // masses only 16: what lies lower weighs less than e^-16 of the maximum each

struct ClusterSmem {
  SearchSmem search;            // search.list: x / T of the candidates (filled in the first CTA only)
  int idx[kCluList];            // their vocabulary indices
  ArgMax cmax;                  // maximum of this CTA's share
  int cnt[kCntBins][32];        // per warp: elements with floor(mx - x / T) == bin
  float mass[kMassBins][32];    // per warp: their softmax mass
  float zall[32];               // per warp: softmax mass of the whole share
  int cta_cnt[kCntBins];        // the same over this CTA's warps (what the peers read)
  float cta_mass[kMassBins];
  float cta_z;
  int peer_cnt[kClu][kCntBins]; // every CTA's figures, gathered
  int tot_cnt[kCntBins];        // over the cluster
  float tot_mass[kMassBins];
  float tot_z;
  float red[32];
  int pick, last, cut;
};

__device__ __forceinline__ void load4(const float* __restrict__ row, int i, int end, bool vec, float (&xv)[4]) {
  if (vec && i + 3 < end) {
    const float4 q = *reinterpret_cast<const float4*>(row + i);
    xv[0] = q.x; xv[1] = q.y; xv[2] = q.z; xv[3] = q.w;
  } else {
#pragma unroll
    for (int e = 0; e < 4; ++e) xv[e] = i + e < end ? row[i + e] : -FLT_MAX;
  }
}

// softmax mass of the list entries with key >= thr; every thread gets the same value
__device__ float list_mass_ge(SearchSmem* sm, float mx, uint32_t thr) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float v = 0.f;
  const int n = sm->wcnt[warp];
  for (int q = lane; q < n; q += 32) {
    const float x = sm->list[warp * kListPerWarp + q];
    v += fkey(x) >= thr ? __expf(x - mx) : 0.f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) sm->acc[warp] = v;
  __syncthreads();
  float tot = 0.f;
  for (int q = 0; q < kSampThreads / 32; ++q) tot += sm->acc[q];
  __syncthreads();
  return tot;
}

__global__ void __launch_bounds__(kSampThreads, 1)
sample_cluster_kernel(const float* __restrict__ logits, int64_t* __restrict__ out, int vocab, int ld,
                      const float* __restrict__ temperature, const int32_t* __restrict__ top_k,
                      const float* __restrict__ top_p, const float* __restrict__ min_p,
                      const uint64_t* __restrict__ seeds, uint64_t step) {
  extern __shared__ __align__(16) unsigned char sm_raw[];
  ClusterSmem* sm = reinterpret_cast<ClusterSmem*>(sm_raw);
  __shared__ ArgMax sh_am[32];
  const int rowi = blockIdx.y;
  const uint32_t rank = cluster_ctarank(), nclu = cluster_nctarank();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* row = logits + static_cast<size_t>(rowi) * ld;
  const float T = temperature ? temperature[rowi] : 1.f;
  const int k = top_k ? top_k[rowi] : 0;
  const float tp = top_p ? top_p[rowi] : 1.f;
  const float mp = min_p ? min_p[rowi] : 0.f;
  const bool use_k = k > 0 && k < vocab, use_p = tp < 1.f, use_m = mp > 0.f;
  // the same decision in all eight CTAs, so a row is left by the whole cluster at once
  if (T <= 0.f || k == 1 || !(use_k || use_p || use_m)) {
    if (rank == 0 && threadIdx.x == 0) out[rowi] = -1;
    return;
  }
  const float invT = 1.f / T;
  const bool vec = (reinterpret_cast<uintptr_t>(row) & 15) == 0;
  // warp g of the cluster owns [g * seg, (g + 1) * seg): a multiple of 128 elements (aligned float4 loads)
  const int nwarps = static_cast<int>(nclu) * 32;
  const int seg = (((vocab + nwarps - 1) / nwarps) + 127) & ~127;
  const int gw = static_cast<int>(rank) * 32 + warp;
  const int beg = gw * seg < vocab ? gw * seg : vocab;
  const int end = beg + seg < vocab ? beg + seg : vocab;

  // 1. maximum of x / T
  ArgMax a{-FLT_MAX, 0x7fffffff};
  for (int i0 = beg; i0 < end; i0 += 512) {
    float xv[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) load4(row, i0 + u * 128 + 4 * lane, end, vec, xv[u]);
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = i0 + u * 128 + 4 * lane + e;
        if (i < end) a = amax2(a, ArgMax{__fmul_rn(xv[u][e], invT), i});
      }
  }
  a = block_argmax(a, sh_am);
  if (threadIdx.x == 0) sm->cmax = a;
  cluster_sync_all();
  {
    ArgMax g{-FLT_MAX, 0x7fffffff};
    for (uint32_t r = 0; r < nclu; ++r) {
      ArgMax b;
      b.v = __uint_as_float(ld_cluster_u32(mapa_shared(&sm->cmax.v, r)));
      b.i = static_cast<int>(ld_cluster_u32(mapa_shared(&sm->cmax.i, r)));
      g = amax2(g, b);
    }
    a = g;
  }
  const float mx = a.v;
  const uint32_t hi_key = fkey(mx);

  // 2. histogram of mx - x / T in unit bins: counts (two 16-bit counters per register) and softmax mass
  {
    uint32_t c[kCntBins / 2];
    float m[kMassBins];
#pragma unroll
    for (int j = 0; j < kCntBins / 2; ++j) c[j] = 0u;
#pragma unroll
    for (int j = 0; j < kMassBins; ++j) m[j] = 0.f;
    float z = 0.f;
    for (int i0 = beg; i0 < end; i0 += 512) {
      float xv[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) load4(row, i0 + u * 128 + 4 * lane, end, vec, xv[u]);
#pragma unroll
      for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = i0 + u * 128 + 4 * lane + e;
          if (i >= end) continue;
          const float d = __fsub_rn(mx, __fmul_rn(xv[u][e], invT));   // no contraction: step 3 must agree
          const float w = __expf(-d);
          z += w;
          if (d < static_cast<float>(kCntBins)) {
            const int b = static_cast<int>(d);
            const uint32_t inc = (b & 1) ? 0x10000u : 1u;
#pragma unroll
            for (int j = 0; j < kCntBins / 2; ++j) c[j] += ((b >> 1) == j) ? inc : 0u;
#pragma unroll
            for (int j = 0; j < kMassBins; ++j) m[j] += (b == j) ? w : 0.f;
          }
        }
    }
    // a warp's share is below 65536 elements for any vocabulary under 16 M, so the packed sums cannot carry
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      z += __shfl_xor_sync(0xffffffffu, z, o);
#pragma unroll
      for (int j = 0; j < kCntBins / 2; ++j) c[j] += __shfl_xor_sync(0xffffffffu, c[j], o);
#pragma unroll
      for (int j = 0; j < kMassBins; ++j) m[j] += __shfl_xor_sync(0xffffffffu, m[j], o);
    }
    if (lane == 0) {
      sm->zall[warp] = z;
#pragma unroll
      for (int j = 0; j < kCntBins / 2; ++j) {
        sm->cnt[2 * j][warp] = static_cast<int>(c[j] & 0xffffu);
        sm->cnt[2 * j + 1][warp] = static_cast<int>(c[j] >> 16);
      }
#pragma unroll
      for (int j = 0; j < kMassBins; ++j) sm->mass[j][warp] = m[j];
    }
  }
  __syncthreads();
  // this CTA's sums: warp b adds bin b over the warps (lane q holds warp q's figure)
  {
    int cb = sm->cnt[warp][lane];
    float mb_ = warp < kMassBins ? sm->mass[warp][lane] : (warp == kMassBins ? sm->zall[lane] : 0.f);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      cb += __shfl_xor_sync(0xffffffffu, cb, o);
      mb_ += __shfl_xor_sync(0xffffffffu, mb_, o);
    }
    if (lane == 0) {
      sm->cta_cnt[warp] = cb;
      if (warp < kMassBins) sm->cta_mass[warp] = mb_;
      if (warp == kMassBins) sm->cta_z = mb_;
    }
  }
  cluster_sync_all();
  // the cluster's sums, added in CTA order by one thread per figure: all eight CTAs get the same numbers
  if (threadIdx.x < kCntBins) {
    int t = 0;
    for (uint32_t r = 0; r < nclu; ++r) {
      const int v = static_cast<int>(ld_cluster_u32(mapa_shared(&sm->cta_cnt[threadIdx.x], r)));
      sm->peer_cnt[r][threadIdx.x] = v;
      t += v;
    }
    sm->tot_cnt[threadIdx.x] = t;
  } else if (threadIdx.x < kCntBins + kMassBins + 1) {
    const int j = threadIdx.x - kCntBins;
    const float* src = j < kMassBins ? &sm->cta_mass[j] : &sm->cta_z;
    float t = 0.f;
    for (uint32_t r = 0; r < nclu; ++r) t += __uint_as_float(ld_cluster_u32(mapa_shared(src, r)));
    if (j < kMassBins) sm->tot_mass[j] = t; else sm->tot_z = t;
  }
  __syncthreads();
  const float z_all = sm->tot_z;
  // smallest window that holds the whole kept set: the k-th largest lies in it, the min-p bound does, and
  // without either of those the nucleus does (its mass is at most tp times the total, which the window has)
  const float d_m = use_m ? -__logf(mp) : 0.f;
  int wsel = -1, n = 0;
  {
    int cum = 0;
    float cum_m = 0.f;
    for (int w = 0; w < kCntBins; ++w) {
      cum += sm->tot_cnt[w];
      if (w < kMassBins) cum_m += sm->tot_mass[w];
      if (cum > kCluList) break;
      const bool ok = (!use_k || cum >= k) && (!use_m || d_m + 0.01f < static_cast<float>(w + 1)) &&
                      (use_k || use_m || (w < kMassBins && cum_m >= tp * z_all));
      if (ok) { wsel = w; n = cum; break; }
    }
  }
  if (wsel < 0) {
    if (rank == 0 && threadIdx.x == 0) out[rowi] = -1;
    cluster_sync_all();   // nobody leaves while a peer may still read its counters
    return;
  }
  const float d_max = static_cast<float>(wsel + 1);       // candidates: mx - x / T < d_max
  const uint32_t wlo = fkey(mx - d_max - 1.f);            // a key below every candidate's
  const uint32_t km = use_m ? fkey(mx + __logf(mp)) : 0u;
  int off = 0;   // candidates of the warps before this one, in index order
  {
    int mine = 0;   // lane l: candidates of this CTA's warp l
    for (int b = 0; b <= wsel; ++b) mine += sm->cnt[b][lane];
    int before = lane < warp ? mine : 0;
    for (int r = lane; r < static_cast<int>(rank); r += 32)
      for (int b = 0; b <= wsel; ++b) before += sm->peer_cnt[r][b];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) before += __shfl_xor_sync(0xffffffffu, before, o);
    off = before;
  }

  // 3. candidates of the chosen window into the first CTA's list, in index order
  {
    const uint32_t list0 = mapa_shared(&sm->search.list[0], 0);
    const uint32_t idx0 = mapa_shared(&sm->idx[0], 0);
    for (int i0 = beg; i0 < end; i0 += 128) {
      float xv[4];
      load4(row, i0 + 4 * lane, end, vec, xv);
      bool in[4];
      int c = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        xv[e] = __fmul_rn(xv[e], invT);
        in[e] = i0 + 4 * lane + e < end && __fsub_rn(mx, xv[e]) < d_max;
        c += in[e] ? 1 : 0;
      }
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      int pos = off + incl - c;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (in[e]) {
          if (pos < kCluList) {
            st_cluster_u32(list0 + 4u * pos, __float_as_uint(xv[e]));
            st_cluster_u32(idx0 + 4u * pos, static_cast<uint32_t>(i0 + 4 * lane + e));
          }
          ++pos;
        }
      off += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  cluster_sync_all();
  if (rank != 0) return;

  // 4. cut-offs and the draw, on the list alone
  SearchSmem* ss = &sm->search;
  if (threadIdx.x < kSampThreads / 32) {
    const int left = n - static_cast<int>(threadIdx.x) * kListPerWarp;
    ss->wcnt[threadIdx.x] = left < 0 ? 0 : (left > kListPerWarp ? kListPerWarp : left);
  }
  if (threadIdx.x == 0) { sm->pick = -1; sm->last = -1; sm->cut = -1; }
  __syncthreads();
  uint32_t thr_key = wlo;
  float Z;
  if (n <= kSampThreads) {
    // Short list (the usual case): one candidate per thread. Its rank in descending order is the number of
    // candidates ahead of it, counted directly; masses are then prefix-summed in rank order, and both
    // cut-offs are read off the sorted values - a few microseconds instead of a dozen bisection passes.
    float* sx = ss->list + kSampThreads;        // x / T by rank
    float* sw = ss->list + 2 * kSampThreads;    // softmax mass by rank
    float* sp = ss->list + 3 * kSampThreads;    // inclusive prefix of sw
    const int t = threadIdx.x;
    const int n4 = (n + 3) & ~3;
    if (t >= n && t < n4) ss->list[t] = -FLT_MAX;
    __syncthreads();
    if (t < n) {
      const float x = ss->list[t];
      const float4* l4 = reinterpret_cast<const float4*>(ss->list);
      int rk = 0;
      for (int j = 0; j < n4; j += 4) {
        const float4 q = l4[j >> 2];
        rk += (q.x > x || (q.x == x && j < t)) ? 1 : 0;
        rk += (q.y > x || (q.y == x && j + 1 < t)) ? 1 : 0;
        rk += (q.z > x || (q.z == x && j + 2 < t)) ? 1 : 0;
        rk += (q.w > x || (q.w == x && j + 3 < t)) ? 1 : 0;
      }
      sx[rk] = x;
      sw[rk] = __expf(x - mx);
    }
    __syncthreads();
    {
      const float mine = t < n ? sw[t] : 0.f;
      float incl = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float u = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += u;
      }
      if (lane == 31) sm->red[warp] = incl;
      __syncthreads();
      float woff = 0.f;
      for (int q = 0; q < warp; ++q) woff += sm->red[q];
      if (t < n) sp[t] = woff + incl;
    }
    __syncthreads();
    if (use_k) thr_key = max(thr_key, fkey(sx[k - 1]));   // k <= n by the choice of the window
    if (use_m) thr_key = max(thr_key, km);
    if (thr_key > hi_key) thr_key = hi_key;               // a min_p above one keeps the maximum alone
    int m = __syncthreads_count(t < n && fkey(sx[t]) >= thr_key);
    Z = (use_k || use_m) ? sp[m - 1] : z_all;
    if (use_p) {
      const float target = tp * Z;
      if (t < m && sp[t] >= target && (t == 0 || sp[t - 1] < target)) sm->cut = t;
      __syncthreads();
      const int r = sm->cut >= 0 ? sm->cut : m - 1;
      thr_key = max(thr_key, fkey(sx[r]));
      m = __syncthreads_count(t < n && fkey(sx[t]) >= thr_key);
      Z = sp[m - 1];
    }
  } else {
    if (use_k) {
      uint32_t lo = wlo, hi = hi_key;
      float above = 0.f;
      while (lo < hi) multiway_pass<false, true>(row, vocab, invT, mx, ss, lo, hi, static_cast<float>(k), above);
      thr_key = lo;
    }
    if (use_m) thr_key = max(thr_key, km);
    if (thr_key > hi_key) thr_key = hi_key;
    Z = (use_k || use_m) ? list_mass_ge(ss, mx, thr_key) : z_all;
    if (use_p) {
      uint32_t lo = thr_key, hi = hi_key;
      float above = 0.f;
      const float target = tp * Z;
      while (lo < hi) multiway_pass<true, true>(row, vocab, invT, mx, ss, lo, hi, target, above);
      thr_key = lo;
      Z = list_mass_ge(ss, mx, thr_key);
    }
  }
  // inverse-CDF draw over the kept entries, which sit in index order: eight consecutive entries per thread
  const uint64_t seed = seeds ? seeds[rowi] : 0x1234ull + rowi;
  const float target = uniform01(seed, step, 0xffffffffull) * Z;
  constexpr int kPer = kCluList / kSampThreads;
  float w[kPer];
  float mine = 0.f;
  int last_kept = -1;
#pragma unroll
  for (int e = 0; e < kPer; ++e) {
    const int p = threadIdx.x * kPer + e;
    const float x = p < n ? ss->list[p] : 0.f;
    w[e] = (p < n && fkey(x) >= thr_key) ? __expf(x - mx) : 0.f;
    mine += w[e];
    if (w[e] > 0.f) last_kept = p;
  }
  float incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) sm->red[warp] = incl;
  __syncthreads();
  float woff = 0.f;
  for (int q = 0; q < warp; ++q) woff += sm->red[q];
  float cum = woff + incl - mine;
#pragma unroll
  for (int e = 0; e < kPer; ++e) {
    if (w[e] > 0.f && cum + w[e] >= target && cum < target) atomicMax(&sm->pick, static_cast<int>(threadIdx.x) * kPer + e);
    cum += w[e];
  }
  if (last_kept >= 0) atomicMax(&sm->last, last_kept);
  __syncthreads();
  if (threadIdx.x == 0) {
    // rounding can leave the target just above the total mass: the last kept entry then
    const int p = sm->pick >= 0 ? sm->pick : sm->last;
    out[rowi] = p >= 0 ? sm->idx[p] : a.i;
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

static bool g_sample_cluster = true;

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
  // rows with a top-k / top-p / min-p filter go to the cluster kernel first; what it leaves (out = -1: greedy
  // and plain-temperature rows, kept sets too wide for its list) is drawn by the one-CTA kernel after it
  bool clustered = g_sample_cluster && (top_k || top_p || min_p) && rows <= 65535;
  if (clustered) {
    static PerDeviceOnce once;
    if (once.needed()) {
      if (cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(sizeof(ClusterSmem))) != cudaSuccess)
        return MB_ERR_LAUNCH;
      once.done();
    }
    // as many CTAs per row as still lets the whole batch run at once (one CTA of this size per SM)
    static int sms = 0;
    if (sms == 0) {
      int dev = 0;
      cudaGetDevice(&dev);
      if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    int c = kClu;
    while (c > 1 && rows * c > sms) c >>= 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(c, rows);
    cfg.blockDim = dim3(kSampThreads);
    cfg.dynamicSmemBytes = sizeof(ClusterSmem);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = c;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, sample_cluster_kernel, logits, out, vocab, ld, temperature, top_k, top_p, min_p,
                           seeds, step) != cudaSuccess) {
      // a device (or partition) that cannot place such clusters: every row goes to the one-CTA kernel from now on
      cudaGetLastError();
      g_sample_cluster = false;
      clustered = false;
    }
  }
  return launch_k(sample_kernel, dim3(rows), dim3(kSampThreads), 0, stream, logits, out, vocab, ld, temperature,
                  top_k, top_p, min_p, seeds, step, clustered ? 1 : 0) == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

// 0: every row is sampled by the one-CTA kernel (the cluster kernel is not launched)
extern "C" void mb_set_sample_cluster(int on) { g_sample_cluster = on != 0; }

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
