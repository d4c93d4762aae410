// Expert-parallel dispatch and combine over NVLink peer memory.
//
// Every rank owns `E_local = E / W` experts. For a batch of T local tokens with top-k routing:
//
//   ep_dispatch   one warp per (token, slot) pair: the token row is written straight into the
//                 owner rank's receive buffer  recv_x[owner][src = me][pos]  (remote 16-byte
//                 stores; optionally quantised to fp8 e4m3 with one scale per 128 values on the
//                 way, which halves the NVLink bytes), together with a meta word (local expert,
//                 source pair index). `pos` comes from a per-destination cursor. The last CTA
//                 publishes the per-destination counts and an epoch flag to every peer and waits
//                 for theirs, so when the kernel ends the rank knows how many rows it received.
//   ep_gather_ids turns the received meta words into an expert-id array (or -1 for empty slots)
//                 that the MoE index kernel sorts; the grouped GEMMs then run on local experts.
//   ep_recv_compact   the same in one launch, and with the rows moved: per-expert offsets, the rows of the
//                 receive buffer copied into expert order (fp8 payload and scales split into the operand
//                 layout of the block-scaled grouped GEMM), and the order array that the combine needs.
//   ep_combine_send   expert outputs go back to  ret_x[src][owner = me][pos]  on the source rank.
//   ep_combine_reduce on the source: y[t] = shared[t] + sum_k w[t,k] * ret_x[owner(t,k)][pos(t,k)].
//
// Flags and epochs work as in comm.cu (epoch words live in device memory, so CUDA graphs
// replay); all waits are bounded and report through the error word.
//
// Reference counterparts: max/kernels/src/shmem/ep_comm.mojo:2913 (dispatch_async), :3036
// (dispatch_wait), :3757 (combine_async), :3860 (combine_wait), BlockwiseFP8TokenFormat :621.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"

namespace mb {
namespace ep {

typedef __nv_bfloat16 bf16;
constexpr int kMaxRanks = 8;
// flag words (int32) per rank: [0..7] dispatch epoch from src, [8..15] combine epoch from owner,
// [16..23] counts from src (rows sent to me), [24] epoch, [25] done-CTA counter, [32..39] send cursors
constexpr int kDispFlag = 0, kCombFlag = 8, kCount = 16, kEpoch = 24, kDone = 25, kCursor = 32;

struct Peers {
  int world, rank;
  uint8_t* recv_x[kMaxRanks];   // [W src][cap][row_bytes]
  int32_t* recv_meta[kMaxRanks];// [W src][cap][2]  (local expert, source pair index)
  uint8_t* ret_x[kMaxRanks];    // [W owner][cap][H bf16]
  int* flags[kMaxRanks];
};

// Last CTA of the grid: publish (optional payload +) epoch to every peer, wait for all peers.
__device__ __forceinline__ bool grid_last_cta(int* done_word) {
  __shared__ int is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) is_last = atomicAdd(done_word, 1) == static_cast<int>(gridDim.x) - 1;
  __syncthreads();
  return is_last != 0;
}

// x: [T, H] bf16. row_bytes = H*2 (bf16) or H + H/128*4 (fp8 payload followed by fp32 scales).
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(Peers p, const bf16* __restrict__ x, const int32_t* __restrict__ topk_ids,
                   int32_t* __restrict__ send_pos, int T, int H, int top_k, int e_local, int cap,
                   int row_bytes, int fp8, int* err) {
  int* my = p.flags[p.rank];
  const int epoch = ld_volatile(my + kEpoch) + 1;
  const int warps_per_cta = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_pairs = T * top_k;
  for (int pair = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); pair < n_pairs;
       pair += gridDim.x * warps_per_cta) {
    const int e = topk_ids[pair];
    const int owner = e / e_local;
    int pos = 0;
    if (lane == 0) pos = atomicAdd(my + kCursor + owner, 1);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (lane == 0) send_pos[pair] = pos < cap ? pos : -1;
    if (pos >= cap) continue;  // capacity overflow: the pair is dropped (reported through counts)
    const int t = pair / top_k;
    uint8_t* dst = p.recv_x[owner] + (static_cast<size_t>(p.rank) * cap + pos) * row_bytes;
    const bf16* src = x + static_cast<size_t>(t) * H;
    if (!fp8) {
      for (int v = lane; v < (H >> 3); v += 32)
        *reinterpret_cast<uint4*>(dst + v * 16) = *reinterpret_cast<const uint4*>(src + v * 8);
    } else {
      // 128 values per group: each lane holds 4, the warp one group per iteration
      float* scales = reinterpret_cast<float*>(dst + H);
      for (int g = 0; g < (H >> 7); ++g) {
        const uint2 raw = *reinterpret_cast<const uint2*>(src + g * 128 + lane * 4);
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
        const float2 a = __bfloat1622float2(b[0]), c = __bfloat1622float2(b[1]);
        float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(c.x), fabsf(c.y)));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float scale = fmaxf(amax, 1e-12f) / 448.0f, inv = 1.0f / scale;
        const __nv_fp8x4_e4m3 q(make_float4(a.x * inv, a.y * inv, c.x * inv, c.y * inv));
        *reinterpret_cast<uint32_t*>(dst + g * 128 + lane * 4) = q.__x;
        if (lane == 0) scales[g] = scale;
      }
    }
    if (lane == 0) {
      int32_t* meta = p.recv_meta[owner] + (static_cast<size_t>(p.rank) * cap + pos) * 2;
      meta[0] = e - owner * e_local;
      meta[1] = pair;
    }
  }
  if (!grid_last_cta(my + kDone)) return;
  // publish counts + epoch, reset cursors, wait for every source's epoch
  if (threadIdx.x < p.world) {
    const int r = threadIdx.x;
    int cnt = my[kCursor + r];
    if (cnt > cap) cnt = cap;
    p.flags[r][kCount + p.rank] = cnt;
    __threadfence_system();
    st_release_sys(p.flags[r] + kDispFlag + p.rank, epoch);
    my[kCursor + r] = 0;
    wait_flag_ge(my + kDispFlag + r, epoch, err, 601);
  }
  __syncthreads();
  if (threadIdx.x == 0) { my[kDone] = 0; my[kEpoch] = epoch; }
}

// ids[src*cap + pos] = local expert of that received row, or -1 beyond the received count.
__global__ void ep_gather_ids_kernel(const int32_t* __restrict__ recv_meta, const int* __restrict__ flags,
                                     int32_t* __restrict__ ids, int world, int cap) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= world * cap) return;
  const int src = i / cap, pos = i % cap;
  ids[i] = pos < flags[kCount + src] ? recv_meta[static_cast<size_t>(i) * 2] : -1;
}

// Received rows -> grouped-GEMM operands, one launch. Every CTA ranks ALL received rows (a counting sort
// by local expert that keeps the order of (source, position), so the result does not depend on the grid),
// then moves its own share of them.
//   virtual row v in [0, total): source s with base[s] <= v < base[s + 1], position v - base[s]
//   thread th owns the v of chunk th (ceil(total / 256) each); hist[e][th] counts them per expert
//   rank of a row = offsets[e] + rows of expert e in earlier chunks + earlier rows of e in its own chunk
// Outputs: offsets [E + 1]; order[pos] = s * cap + position; rows: fp8 -> xq [rows, H] e4m3 and
// xs [H / 128, ld_s] fp32 (group-major), bf16 -> xq [rows, H] bf16. E <= 128 (uint16 histogram in 64 KB).
constexpr int kCompactThreads = 256;
constexpr int kCompactMaxExperts = 128;

__global__ void __launch_bounds__(kCompactThreads)
ep_recv_compact_kernel(const uint8_t* __restrict__ recv_x, const int32_t* __restrict__ recv_meta,
                       const int* __restrict__ flags, int world, int cap, int E, int H, int row_bytes, int fp8,
                       int share_cap, int32_t* __restrict__ offsets, int32_t* __restrict__ order,
                       uint8_t* __restrict__ xq, float* __restrict__ xs, int ld_s) {
  extern __shared__ uint8_t dyn[];
  uint16_t* hist = reinterpret_cast<uint16_t*>(dyn);                               // [E][256]
  int2* todo = reinterpret_cast<int2*>(dyn + static_cast<size_t>(E) * kCompactThreads * 2);  // [share_cap]
  __shared__ int base[kMaxRanks + 1];
  __shared__ int off_s[kCompactMaxExperts + 1];
  const int th = threadIdx.x, lane = th & 31, warp = th >> 5;
  if (th == 0) {
    int acc = 0;
    for (int s = 0; s < world; ++s) {
      base[s] = acc;
      int c = flags[kCount + s];
      acc += c < cap ? (c < 0 ? 0 : c) : cap;
    }
    for (int s = world; s <= kMaxRanks; ++s) base[s] = acc;
  }
  for (int i = th; i < E * kCompactThreads; i += kCompactThreads) hist[i] = 0;
  __syncthreads();
  const int total = base[world];
  const int chunk = (total + kCompactThreads - 1) / kCompactThreads;
  const int v0 = th * chunk, v1 = min(total, v0 + chunk);
  // pass 1: histogram of this thread's chunk
  {
    int s = 0;
    for (int v = v0; v < v1; ++v) {
      while (v >= base[s + 1]) ++s;
      const int e = recv_meta[(static_cast<size_t>(s) * cap + (v - base[s])) * 2];
      if (e >= 0 && e < E) hist[e * kCompactThreads + th] += 1;
    }
  }
  __syncthreads();
  // exclusive scan over the 256 chunks of every expert (one warp per expert, 8 entries per lane)
  for (int e = warp; e < E; e += kCompactThreads / 32) {
    uint16_t* h = hist + e * kCompactThreads + lane * 8;
    int loc[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { loc[j] = h[j]; sum += loc[j]; }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    int run = incl - sum;
#pragma unroll
    for (int j = 0; j < 8; ++j) { h[j] = static_cast<uint16_t>(run); run += loc[j]; }
    if (lane == 31) off_s[e + 1] = incl;       // rows of expert e
  }
  __syncthreads();
  if (th == 0) {
    off_s[0] = 0;
    for (int e = 0; e < E; ++e) off_s[e + 1] += off_s[e];
  }
  __syncthreads();
  if (blockIdx.x == 0)
    for (int e = th; e <= E; e += kCompactThreads) offsets[e] = off_s[e];
  // pass 2: positions of the rows in this CTA's share [r0, r1) of the virtual rows
  const int share = (total + gridDim.x - 1) / gridDim.x;
  const int r0 = blockIdx.x * share, r1 = min(total, r0 + share);
  if (v0 < r1 && v1 > r0) {
    int s = 0;
    for (int v = v0; v < v1; ++v) {
      while (v >= base[s + 1]) ++s;
      const int flat = s * cap + (v - base[s]);
      const int e = recv_meta[static_cast<size_t>(flat) * 2];
      const bool mine = v >= r0 && v < r1 && v - r0 < share_cap;
      if (e < 0 || e >= E) {          // not an id the dispatch writes: the row gets no position
        if (mine) todo[v - r0] = make_int2(-1, flat);
        continue;
      }
      const int pos = off_s[e] + hist[e * kCompactThreads + th];
      hist[e * kCompactThreads + th] += 1;
      if (mine) todo[v - r0] = make_int2(pos, flat);
    }
  }
  __syncthreads();
  const int n_mine = max(0, min(r1 - r0, share_cap));
  // move the rows: one warp per row, 16 bytes per lane and iteration
  const int payload = fp8 ? H : H * 2;
  for (int i = warp; i < n_mine; i += kCompactThreads / 32) {
    const int2 pf = todo[i];
    if (pf.x < 0) continue;
    const uint8_t* src = recv_x + static_cast<size_t>(pf.y) * row_bytes;
    uint8_t* dst = xq + static_cast<size_t>(pf.x) * payload;
    for (int c = lane * 16; c < payload; c += 512)
      *reinterpret_cast<uint4*>(dst + c) = *reinterpret_cast<const uint4*>(src + c);
    if (fp8) {
      const float* sc = reinterpret_cast<const float*>(src + H);
      for (int g = lane; g < (H >> 7); g += 32) xs[static_cast<size_t>(g) * ld_s + pf.x] = sc[g];
    }
    if (lane == 0) order[pf.x] = pf.y;
  }
}

// out_sorted: [n_rows, H] expert outputs in expert order; order[p] = src*cap + pos.
__global__ void __launch_bounds__(256)
ep_combine_send_kernel(Peers p, const bf16* __restrict__ out_sorted, const int32_t* __restrict__ order,
                       const int32_t* __restrict__ n_rows_dev, int H, int cap, int* err) {
  int* my = p.flags[p.rank];
  const int epoch = ld_volatile(my + kEpoch) + 1;
  const int n_rows = *n_rows_dev;
  const int warps_per_cta = blockDim.x >> 5, lane = threadIdx.x & 31;
  for (int r = blockIdx.x * warps_per_cta + (threadIdx.x >> 5); r < n_rows; r += gridDim.x * warps_per_cta) {
    const int flat = order[r];
    const int src = flat / cap, pos = flat % cap;
    uint8_t* dst = p.ret_x[src] + (static_cast<size_t>(p.rank) * cap + pos) * (static_cast<size_t>(H) * 2);
    const bf16* s = out_sorted + static_cast<size_t>(r) * H;
    for (int v = lane; v < (H >> 3); v += 32)
      *reinterpret_cast<uint4*>(dst + v * 16) = *reinterpret_cast<const uint4*>(s + v * 8);
  }
  if (!grid_last_cta(my + kDone)) return;
  if (threadIdx.x < p.world) {
    const int r = threadIdx.x;
    __threadfence_system();
    st_release_sys(p.flags[r] + kCombFlag + p.rank, epoch);
    wait_flag_ge(my + kCombFlag + r, epoch, err, 602);
  }
  __syncthreads();
  if (threadIdx.x == 0) { my[kDone] = 0; my[kEpoch] = epoch; }
}

// y[t] = residual[t] + shared[t] + sum_k w[t,k] * ret_x[owner][pos]   (all local reads; y may alias residual)
__global__ void ep_combine_reduce_kernel(const uint8_t* __restrict__ ret_x, const int32_t* __restrict__ topk_ids,
                                         const int32_t* __restrict__ send_pos, const float* __restrict__ w,
                                         const bf16* __restrict__ shared, const bf16* residual, bf16* y, int T, int H,
                                         int top_k, int e_local, int cap) {
  const int per_row = H >> 3;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(T) * per_row) return;
  const int t = static_cast<int>(i / per_row), c = static_cast<int>(i % per_row) * 8;
  float acc[8];
  if (shared) {
    const uint4 sv = *reinterpret_cast<const uint4*>(shared + static_cast<size_t>(t) * H + c);
    const __nv_bfloat162* sp = reinterpret_cast<const __nv_bfloat162*>(&sv);
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(sp[j]); acc[2 * j] = f.x; acc[2 * j + 1] = f.y; }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  }
  if (residual) {
    const uint4 rv = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(t) * H + c);
    const __nv_bfloat162* rp = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(rp[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
  }
  for (int k = 0; k < top_k; ++k) {
    const int pair = t * top_k + k;
    const int pos = send_pos[pair];
    if (pos < 0) continue;
    const int owner = topk_ids[pair] / e_local;
    const float wk = w[pair];
    const bf16* row = reinterpret_cast<const bf16*>(ret_x) + (static_cast<size_t>(owner) * cap + pos) * H;
    const uint4 ev = *reinterpret_cast<const uint4*>(row + c);
    const __nv_bfloat162* ep_ = reinterpret_cast<const __nv_bfloat162*>(&ev);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(ep_[j]);
      acc[2 * j] = fmaf(wk, f.x, acc[2 * j]);
      acc[2 * j + 1] = fmaf(wk, f.y, acc[2 * j + 1]);
    }
  }
  uint4 out;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
  for (int j = 0; j < 4; ++j) op[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
  *reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * H + c) = out;
}

// fp8 rows [n, H + H/128*4] -> bf16 rows (used after dispatch when the experts run in bf16)
__global__ void ep_dequant_rows_kernel(const uint8_t* __restrict__ src, bf16* __restrict__ dst, int n, int H,
                                       int row_bytes, const int32_t* __restrict__ n_rows_dev) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_row = H >> 2;
  if (n_rows_dev != nullptr && *n_rows_dev < n) n = *n_rows_dev;   // only the rows that were received
  if (i >= static_cast<long long>(n) * per_row) return;
  const int r = static_cast<int>(i / per_row), c = static_cast<int>(i % per_row) * 4;
  const uint8_t* row = src + static_cast<size_t>(r) * row_bytes;
  const float scale = reinterpret_cast<const float*>(row + H)[c >> 7];
  __nv_fp8x4_e4m3 q;
  q.__x = *reinterpret_cast<const uint32_t*>(row + c);
  const float4 f = static_cast<float4>(q);
  __nv_bfloat162 lo = __floats2bfloat162_rn(f.x * scale, f.y * scale), hi = __floats2bfloat162_rn(f.z * scale, f.w * scale);
  uint2 o;
  o.x = *reinterpret_cast<uint32_t*>(&lo);
  o.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(dst + static_cast<size_t>(r) * H + c) = o;
}

static Peers make_peers(int world, int rank, void* const* recv_x, void* const* recv_meta, void* const* ret_x,
                        int* const* flags) {
  Peers p;
  p.world = world; p.rank = rank;
  for (int i = 0; i < kMaxRanks; ++i) {
    const bool ok = i < world;
    p.recv_x[i] = ok && recv_x ? static_cast<uint8_t*>(recv_x[i]) : nullptr;
    p.recv_meta[i] = ok && recv_meta ? static_cast<int32_t*>(recv_meta[i]) : nullptr;
    p.ret_x[i] = ok && ret_x ? static_cast<uint8_t*>(ret_x[i]) : nullptr;
    p.flags[i] = ok ? flags[i] : nullptr;
  }
  return p;
}

}  // namespace ep
}  // namespace mb

using namespace mb;
#define EP_LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH)

extern "C" int mb_ep_flag_ints(void) { return 64; }

extern "C" int mb_ep_dispatch(int world, int rank, void* const* recv_x, void* const* recv_meta,
                              int* const* flags, const void* x, const int32_t* topk_ids, int32_t* send_pos,
                              int T, int H, int top_k, int e_local, int cap, int fp8, int* err,
                              cudaStream_t stream) {
  if (world < 1 || world > ep::kMaxRanks || H % 128) return MB_ERR_SHAPE;
  const int row_bytes = fp8 ? H + (H / 128) * 4 : H * 2;
  int grid = (T * top_k + 7) / 8;
  if (grid > 592) grid = 592;
  if (grid < 1) grid = 1;
  ep::ep_dispatch_kernel<<<grid, 256, 0, stream>>>(
      ep::make_peers(world, rank, recv_x, recv_meta, nullptr, flags), static_cast<const ep::bf16*>(x),
      topk_ids, send_pos, T, H, top_k, e_local, cap, row_bytes, fp8, err);
  return EP_LAUNCH_OK();
}

extern "C" int mb_ep_gather_ids(const int32_t* recv_meta, const int* flags, int32_t* ids, int world, int cap,
                                cudaStream_t stream) {
  const int n = world * cap;
  if (n <= 0) return MB_OK;
  ep::ep_gather_ids_kernel<<<(n + 255) / 256, 256, 0, stream>>>(recv_meta, flags, ids, world, cap);
  return EP_LAUNCH_OK();
}

// One launch from receive buffers to grouped-GEMM operands (see ep_recv_compact_kernel). `rows_bound`: an upper
// bound of the rows this rank can have received (<= world * cap); `ld_s` >= rows_bound.
extern "C" int mb_ep_recv_compact(const void* recv_x, const int32_t* recv_meta, const int* flags, int world, int cap,
                                  int n_experts, int H, int fp8, int rows_bound, int32_t* offsets, int32_t* order,
                                  void* xq, float* xs, int ld_s, int num_sms, cudaStream_t stream) {
  if (world < 1 || world > ep::kMaxRanks || H % 128 || n_experts < 1 || n_experts > ep::kCompactMaxExperts)
    return MB_ERR_SHAPE;
  if (rows_bound <= 0 || rows_bound > world * cap) rows_bound = world * cap;
  if (fp8 && (xs == nullptr || ld_s < rows_bound)) return MB_ERR_SHAPE;
  const int row_bytes = fp8 ? H + (H / 128) * 4 : H * 2;
  // rows move as 16-byte vectors: the received rows (payload + scales) must keep that alignment
  if (row_bytes % 16 || (reinterpret_cast<uintptr_t>(recv_x) | reinterpret_cast<uintptr_t>(xq)) & 15) return MB_ERR_ALIGN;
  int grid = (rows_bound + 7) / 8;                  // at least a warp-load of rows per CTA
  if (num_sms <= 0) num_sms = 148;
  if (grid > num_sms) grid = num_sms;
  if (grid < 1) grid = 1;
  const int share_cap = (rows_bound + grid - 1) / grid;
  const size_t smem = static_cast<size_t>(n_experts) * ep::kCompactThreads * 2 + static_cast<size_t>(share_cap) * 8;
  if (smem > 200 * 1024) return MB_ERR_TOO_LARGE;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    cudaFuncSetAttribute(ep::ep_recv_compact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    configured.done();
  }
  ep::ep_recv_compact_kernel<<<grid, ep::kCompactThreads, smem, stream>>>(
      static_cast<const uint8_t*>(recv_x), recv_meta, flags, world, cap, n_experts, H, row_bytes, fp8, share_cap,
      offsets, order, static_cast<uint8_t*>(xq), xs, ld_s);
  return EP_LAUNCH_OK();
}

extern "C" int mb_ep_combine_send(int world, int rank, void* const* ret_x, int* const* flags,
                                  const void* out_sorted, const int32_t* order, const int32_t* n_rows_dev,
                                  int max_rows, int H, int cap, int* err, cudaStream_t stream) {
  if (world < 1 || world > ep::kMaxRanks || H % 8) return MB_ERR_SHAPE;
  int grid = (max_rows + 7) / 8;
  if (grid > 592) grid = 592;
  if (grid < 1) grid = 1;
  ep::ep_combine_send_kernel<<<grid, 256, 0, stream>>>(
      ep::make_peers(world, rank, nullptr, nullptr, ret_x, flags), static_cast<const ep::bf16*>(out_sorted),
      order, n_rows_dev, H, cap, err);
  return EP_LAUNCH_OK();
}

extern "C" int mb_ep_combine_reduce(const void* ret_x, const int32_t* topk_ids, const int32_t* send_pos,
                                    const float* w, const void* shared, const void* residual, void* y, int T, int H,
                                    int top_k, int e_local, int cap, cudaStream_t stream) {
  if (T <= 0) return MB_OK;
  const long long work = static_cast<long long>(T) * (H / 8);
  ep::ep_combine_reduce_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint8_t*>(ret_x), topk_ids, send_pos, w, static_cast<const ep::bf16*>(shared),
      static_cast<const ep::bf16*>(residual), static_cast<ep::bf16*>(y), T, H, top_k, e_local, cap);
  return EP_LAUNCH_OK();
}

extern "C" int mb_ep_dequant_rows(const void* src, void* dst, int n, int H, const int32_t* n_rows_dev,
                                  cudaStream_t stream) {
  if (n <= 0) return MB_OK;
  const long long work = static_cast<long long>(n) * (H / 4);
  ep::ep_dequant_rows_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, stream>>>(
      static_cast<const uint8_t*>(src), static_cast<ep::bf16*>(dst), n, H, H + (H / 128) * 4, n_rows_dev);
  return EP_LAUNCH_OK();
}
