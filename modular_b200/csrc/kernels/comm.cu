// Tensor-parallel communication kernels over NVLink peer memory (one process per GPU).
//
// Every rank owns a set of *symmetric* buffers (same size and role on every rank) whose peer
// addresses are known to all ranks. Kernels read and write peers' buffers directly with
// 16-byte loads/stores and synchronise through flag words in peer memory (release/acquire at
// system scope); NVSwitch gives every pair of GPUs full bandwidth, so the algorithms are
// all-to-all in one or two shots, never rings.
//
//   tp_rs_norm_ag    row-parallel GEMM partials -> reduce-scatter (each rank sums the rows it
//                    owns over all ranks' partials, pulled from peer memory) + residual add +
//                    RMSNorm -> all-gather (the normalised rows are pushed into every rank's
//                    activation buffer). The residual stream stays sharded by rows
//                    (sequence-parallel layout), so only normalised activations cross NVLink.
//   tp_allgather     push a local [rows, cols] block into a column slot of every peer's buffer.
//   tp_allreduce     one-shot (small), two-shot (large) and in-switch multimem.ld_reduce variants.
//   tp_broadcast     pull from the root's buffer.
//   tp_barrier       all-rank barrier (used between phases that are not fused).
//
// Flags: each rank has an int array in symmetric memory. Word layout: [slot][src_rank] where a
// rank writes its current epoch into word [slot][my_rank] of every peer; EPOCH lives in the
// rank's own array and is advanced by the kernels themselves, so captured CUDA graphs replay
// with fresh epochs. All waits are bounded (1 s); a timeout sets the error word and the kernel
// carries on, leaving the context usable.
//
// Reference counterparts: max/kernels/src/comm/sync.mojo:336 (_multi_gpu_barrier),
// comm/reducescatter_rmsnorm.mojo:390, comm/allgather_rmsnorm.mojo:288, comm/allgather.mojo:167.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/ptx.cuh"
#include "comm_flags.h"

namespace mb {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

struct TpPeers {
  int world, rank;
  void* a[kMaxRanks];    // buffer A on every rank (meaning depends on the kernel)
  void* b[kMaxRanks];    // buffer B on every rank
  int* flags[kMaxRanks]; // flag arrays
};

// Barrier across ranks, executed by every CTA: CTA 0 publishes `epoch` to all peers, every CTA
// waits until all peers have published it. `slot` selects an independent set of words.
__device__ __forceinline__ void tp_barrier_dev(const TpPeers& p, int slot, int epoch, int* err) {
  if (blockIdx.x == 0 && threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + slot * kMaxRanks + p.rank, epoch);
  }
  if (threadIdx.x < p.world)
    wait_flag_ge(p.flags[p.rank] + slot * kMaxRanks + threadIdx.x, epoch, err, 400 + slot);
  __syncthreads();
}

// Closing barrier of a multi-CTA kernel: the last CTA of this rank to finish publishes `epoch`
// to all peers (so a peer sees it only when *all* of this rank's remote reads and writes are
// done), waits for every peer's epoch, then advances the epoch word. Other CTAs just leave.
__device__ __forceinline__ void tp_finish_barrier(const TpPeers& p, int slot, int epoch, int* err,
                                                  int push_target = -1) {
  __shared__ int is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(p.flags[p.rank] + kDoneWord, 1);
    is_last = prev == static_cast<int>(gridDim.x) - 1;
  }
  __syncthreads();
  if (!is_last) return;
  if (threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + slot * kMaxRanks + p.rank, epoch);
    wait_flag_ge(p.flags[p.rank] + slot * kMaxRanks + threadIdx.x, epoch, err, 400 + slot);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    p.flags[p.rank][kDoneWord] = 0;
    p.flags[p.rank][kEpochWord] = epoch;
    if (push_target >= 0) p.flags[p.rank][kPushTarget] = push_target;
  }
}

__global__ void tp_barrier_kernel(TpPeers p, int* err) {
  const int epoch = ld_volatile(p.flags[p.rank] + kEpochWord) + 1;
  __syncthreads();
  tp_barrier_dev(p, 0, epoch, err);
  if (threadIdx.x == 0) p.flags[p.rank][kEpochWord] = epoch;
}

// Closing step without a barrier: the last CTA of this rank to finish tells every peer that this
// rank's rows have landed in the peer's activation buffer (ready epoch) and leaves. The consumer
// (the TMA producer of the next GEMM) does the waiting, tile by tile.
__device__ __forceinline__ void tp_finish_signal(const TpPeers& p, int ready_epoch, int push_target) {
  __shared__ int is_last_s;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(p.flags[p.rank] + kDoneWord, 1);
    is_last_s = prev == static_cast<int>(gridDim.x) - 1;
  }
  __syncthreads();
  if (!is_last_s) return;
  if (threadIdx.x < p.world) {
    __threadfence_system();
    st_release_sys(p.flags[threadIdx.x] + kReady + p.rank, ready_epoch);
  }
  if (threadIdx.x == 0) {
    // written by the last CTA only: every CTA has read these words at its start
    p.flags[p.rank][kDoneWord] = 0;
    p.flags[p.rank][kPushTarget] = push_target;
    p.flags[p.rank][kReadyEpoch] = ready_epoch;
  }
}

// b[r] = gathered normalised activations [M, H] of rank r.
// h_local = this rank's slice of the residual stream, rows [row0, row0 + n_rows).
// has_partials = 0 skips the reduction (h_local is used as is): layer-0 entry.
// mode bit0 = 0: a[r] = partial sums [M, H] of rank r, pulled from peers after a barrier.
// mode bit0 = 1: the GEMMs pushed their partials into a[rank] = [n_slots][rows_per_rank][H]; the
//                kernel waits until the push counter has grown by `expected` and sums local slots.
// mode bit1 = 0: closing barrier (every rank's rows have landed everywhere when the kernel ends).
// mode bit1 = 1: closing signal only (per-source ready flags for a flag-gated consumer GEMM).
__global__ void __launch_bounds__(256)
tp_rs_norm_ag_kernel(TpPeers p, bf16* __restrict__ h_local, const bf16* __restrict__ gamma, int M,
                     int H, int rows_per_rank, float eps, float w_off, int mbc, int has_partials,
                     int mode, int n_slots, int expected, int* err) {
  __shared__ float red[32];
  extern __shared__ uint4 row_cache[];
  int* my = p.flags[p.rank];
  const int epoch = ld_volatile(my + kEpochWord) + 1;
  const int ready_epoch = ld_volatile(my + kReadyEpoch) + 1;
  const int push_target = ld_volatile(my + kPushTarget) + ((mode & 1) ? expected : 0);
  __syncthreads();
  if (mode & 1) {
    // every partial tile destined for this rank has landed
    if (threadIdx.x == 0) wait_flag_ge(my + kPushCount, push_target, err, 410);
    __syncthreads();
  } else {
    // all ranks' GEMMs have written their partials
    tp_barrier_dev(p, 0, epoch, err);
  }

  const int row0 = p.rank * rows_per_rank;
  int n_rows = M - row0;
  if (n_rows > rows_per_rank) n_rows = rows_per_rank;
  const int nvec = H >> 3;
  for (int r = blockIdx.x; r < n_rows; r += gridDim.x) {
    const int t = row0 + r;
    float ss = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float acc[8];
      {
        const uint4 hv = *reinterpret_cast<const uint4*>(h_local + static_cast<size_t>(r) * H + v * 8);
        const bf162* hp = reinterpret_cast<const bf162*>(&hv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(hp[i]);
          acc[2 * i] = f.x; acc[2 * i + 1] = f.y;
        }
      }
      if (has_partials && (mode & 1)) {
        const bf16* base = static_cast<const bf16*>(p.a[p.rank]) + static_cast<size_t>(r) * H + v * 8;
        const size_t slot_stride = static_cast<size_t>(rows_per_rank) * H;
        for (int s0 = 0; s0 < n_slots; s0 += 4) {
          uint4 pv[4];
#pragma unroll
          for (int s = 0; s < 4; ++s)
            if (s0 + s < n_slots) pv[s] = *reinterpret_cast<const uint4*>(base + (s0 + s) * slot_stride);
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            if (s0 + s < n_slots) {
              const bf162* pp = reinterpret_cast<const bf162*>(&pv[s]);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(pp[i]);
                acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
              }
            }
          }
        }
      } else if (has_partials) {
        uint4 pv[kMaxRanks];
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s) {
          if (s < p.world) {
            // start with the next rank so that the eight GPUs do not all pull from rank 0 first
            const int src = (p.rank + 1 + s) % p.world;
            pv[s] = *reinterpret_cast<const uint4*>(static_cast<const bf16*>(p.a[src]) +
                                                    static_cast<size_t>(t) * H + v * 8);
          }
        }
        // a row is reduced by exactly one rank, always in the same order: deterministic
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s) {
          if (s < p.world) {
            const bf162* pp = reinterpret_cast<const bf162*>(&pv[s]);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 f = __bfloat1622float2(pp[i]);
              acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
            }
          }
        }
      }
      uint4 out;
      bf162* op = reinterpret_cast<bf162*>(&out);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        op[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
        const float2 f = __bfloat1622float2(op[i]);
        ss += f.x * f.x + f.y * f.y;
      }
      *reinterpret_cast<uint4*>(h_local + static_cast<size_t>(r) * H + v * 8) = out;
      row_cache[v] = out;
    }
    // block reduction of the sum of squares
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
    __syncthreads();
    const float inv = rsqrtf(tot / static_cast<float>(H) + eps);
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      uint4 a = row_cache[v];
      const uint4 wv = *reinterpret_cast<const uint4*>(gamma + v * 8);
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
      // all-gather: push the normalised row into every rank's activation buffer
#pragma unroll
      for (int s = 0; s < kMaxRanks; ++s) {
        if (s < p.world) {
          const int dst = (p.rank + s) % p.world;
          *reinterpret_cast<uint4*>(static_cast<bf16*>(p.b[dst]) + static_cast<size_t>(t) * H + v * 8) = a;
        }
      }
    }
    __syncthreads();
  }
  if (mode & 2) {
    tp_finish_signal(p, ready_epoch, push_target);
    return;
  }
  // every rank's pushes have landed (and every rank is done pulling) before anyone continues
  tp_finish_barrier(p, 1, epoch, err, push_target);
}

// Push local block src[rows, cols] (row stride ld_src bytes) to a[dst] + col_off bytes on every
// rank (row stride ld_dst bytes), then barrier.
__global__ void __launch_bounds__(256)
tp_allgather_kernel(TpPeers p, const uint8_t* __restrict__ src, int rows, int row_bytes, int ld_src,
                    int ld_dst, long long col_off, int* err) {
  const int epoch = ld_volatile(p.flags[p.rank] + kEpochWord) + 1;
  __syncthreads();
  const int per_row = row_bytes >> 4;
  const long long total = static_cast<long long>(rows) * per_row;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / per_row), c = static_cast<int>(i % per_row) * 16;
    const uint4 v = *reinterpret_cast<const uint4*>(src + static_cast<size_t>(r) * ld_src + c);
#pragma unroll
    for (int s = 0; s < kMaxRanks; ++s) {
      if (s < p.world) {
        const int dst = (p.rank + s) % p.world;
        *reinterpret_cast<uint4*>(static_cast<uint8_t*>(p.a[dst]) + static_cast<size_t>(r) * ld_dst +
                                  col_off + c) = v;
      }
    }
  }
  tp_finish_barrier(p, 2, epoch, err);
}

// ---------------------------------------------------------------------------- all-reduce
// Sum of every rank's symmetric input buffer a[r] (bf16, n elements, n % 8 == 0) into out (local).
// One-shot: after a barrier every rank reads all ranks' data itself (W reads of n over NVLink per
// rank; best for small n). All ranks add in rank order in fp32, so results are bit-identical.
__device__ __forceinline__ void accum8(float (&acc)[8], const uint4& v) {
  const bf162* p = reinterpret_cast<const bf162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p[i]);
    acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&acc)[8]) {
  uint4 o;
  bf162* p = reinterpret_cast<bf162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  return o;
}

__global__ void __launch_bounds__(256)
tp_allreduce_1shot_kernel(TpPeers p, bf16* __restrict__ out, long long n, int* err) {
  const int epoch = ld_volatile(p.flags[p.rank] + kEpochWord) + 1;
  __syncthreads();
  tp_barrier_dev(p, 0, epoch, err);  // every rank's input is complete
  const long long nvec = n >> 3;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 in[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < p.world) in[r] = reinterpret_cast<const uint4*>(p.a[r])[v];
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < p.world) accum8(acc, in[r]);
    reinterpret_cast<uint4*>(out)[v] = pack8(acc);
  }
  tp_finish_barrier(p, 1, epoch, err);  // nobody overwrites its input while a peer still reads it
}

// Two-shot: each rank reduces the 1/W slice it owns (pulling that slice from every peer), then
// pushes the reduced slice into every rank's output buffer b[r] (symmetric). 2(W-1)/W * n bytes per
// rank over NVLink instead of (W-1) * n: the choice for large n.
__global__ void __launch_bounds__(256)
tp_allreduce_2shot_kernel(TpPeers p, long long n, int* err) {
  const int epoch = ld_volatile(p.flags[p.rank] + kEpochWord) + 1;
  __syncthreads();
  tp_barrier_dev(p, 0, epoch, err);
  const long long nvec = n >> 3;
  const long long per = (nvec + p.world - 1) / p.world;
  const long long v0 = per * p.rank;
  const long long v1 = v0 + per < nvec ? v0 + per : nvec;
  for (long long v = v0 + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < v1;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 in[kMaxRanks];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < p.world) in[r] = reinterpret_cast<const uint4*>(p.a[r])[v];
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r)
      if (r < p.world) accum8(acc, in[r]);
    const uint4 o = pack8(acc);
#pragma unroll
    for (int s = 0; s < kMaxRanks; ++s)
      if (s < p.world) reinterpret_cast<uint4*>(p.b[(p.rank + s) % p.world])[v] = o;
  }
  tp_finish_barrier(p, 1, epoch, err);  // every slice has landed everywhere
}

// One-shot through the NVSwitch: `mc_in` is the multicast address of the symmetric input, one
// multimem.ld_reduce returns the sum over all ranks computed inside the switch.
__global__ void __launch_bounds__(256)
tp_allreduce_multimem_kernel(TpPeers p, const bf16* __restrict__ mc_in, bf16* __restrict__ out, long long n,
                             int* err) {
  const int epoch = ld_volatile(p.flags[p.rank] + kEpochWord) + 1;
  __syncthreads();
  tp_barrier_dev(p, 0, epoch, err);
  const long long nvec = n >> 3;
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 o;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(o.x), "=r"(o.y), "=r"(o.z), "=r"(o.w)
                 : "l"(mc_in + v * 8)
                 : "memory");
    reinterpret_cast<uint4*>(out)[v] = o;
  }
  tp_finish_barrier(p, 1, epoch, err);
}

// ---------------------------------------------------------------------------- barrier-free all-reduce
// One-shot all-reduce without any barrier or flag (sentinel protocol): every rank writes its 16-byte packs
// straight into every peer's receive buffer lam[peer][generation][my rank] and then polls its own receive
// buffer until no pack holds the sentinel bf16 -0.0 any more - the data is its own arrival signal. Inputs are
// sanitised (a real -0.0 is sent as +0.0). Three generations rotate: while generation g is in use, peers that
// run one call ahead already write g+1, and g+2 (read two calls ago) is reset to sentinels, so no rank ever
// waits for another one to finish reading. All ranks add in rank order: results are bit-identical.
// Optional epilogue per row of `cols` elements: residual += sum (in place), out = RMSNorm(residual) * gamma.
//   lam[r]   receive buffer of rank r, [3][world][cap] bf16, every element -0.0 before the first call
//   state    local ints (zeroed once): [0] generation, [1..3] elements written when a generation was last used,
//            [4] CTAs that have left
// Reference: max/kernels/src/comm/allreduce.mojo:1051 (_allreduce_lamport_kernel), comm/lamport.mojo,
// comm/allreduce_lamport_rmsnorm.mojo:62.
__device__ __forceinline__ bool lam_pending(const uint4& v) {
  auto bad = [](uint32_t w) { return (w & 0xffffu) == 0x8000u || (w >> 16) == 0x8000u; };
  return bad(v.x) || bad(v.y) || bad(v.z) || bad(v.w);
}
__device__ __forceinline__ uint32_t lam_clean(uint32_t w) {
  if ((w & 0xffffu) == 0x8000u) w &= 0xffff0000u;
  if ((w >> 16) == 0x8000u) w &= 0x0000ffffu;
  return w;
}
__device__ __forceinline__ uint4 ld_volatile_u4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Sum over ranks of pack `v` (this rank's contribution `mine` is pushed first). Returns fp32 sums in acc.
__device__ __forceinline__ void lam_exchange(const TpPeers& p, long long v, long long cap_vec, int g3, uint4 mine,
                                             float (&acc)[8], int* err) {
  mine.x = lam_clean(mine.x); mine.y = lam_clean(mine.y); mine.z = lam_clean(mine.z); mine.w = lam_clean(mine.w);
  const long long gen_off = static_cast<long long>(g3) * p.world * cap_vec;
#pragma unroll
  for (int s = 1; s < kMaxRanks; ++s) {
    if (s < p.world) {
      const int dst = (p.rank + s) % p.world;
      reinterpret_cast<uint4*>(p.a[dst])[gen_off + static_cast<long long>(p.rank) * cap_vec + v] = mine;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  const uint4* inbox = reinterpret_cast<const uint4*>(p.a[p.rank]) + gen_off + v;
  uint64_t t0 = 0;
  for (int src = 0; src < p.world; ++src) {
    if (src == p.rank) { accum8(acc, mine); continue; }
    const uint4* a = inbox + static_cast<long long>(src) * cap_vec;
    uint4 in = ld_volatile_u4(a);
    uint32_t spins = 0;
    while (lam_pending(in)) {
      if (((++spins) & 0x3f) == 0) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > 1000000000ull) { if (err) atomicCAS(err, 0, 420); break; }
      }
      in = ld_volatile_u4(a);
    }
    accum8(acc, in);
  }
}

__global__ void __launch_bounds__(256)
tp_allreduce_lamport_kernel(TpPeers p, const bf16* __restrict__ x, bf16* __restrict__ out, long long n, long long cap,
                            int* state, bf16* __restrict__ residual, const bf16* __restrict__ gamma, int cols,
                            float eps, float w_off, int mbc, int* err) {
  __shared__ float red[8];
  extern __shared__ uint4 lam_row[];
  const int gen = ld_volatile(state + 0);
  const int g3 = gen % 3, gclr = (gen + 2) % 3;
  const long long old_vec = ld_volatile(state + 1 + gclr) >> 3;
  const long long nvec = n >> 3, cap_vec = cap >> 3;
  const uint4 sentinel = make_uint4(0x80008000u, 0x80008000u, 0x80008000u, 0x80008000u);
  if (gamma == nullptr) {
    for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
         v += static_cast<long long>(gridDim.x) * blockDim.x) {
      float acc[8];
      lam_exchange(p, v, cap_vec, g3, reinterpret_cast<const uint4*>(x)[v], acc, err);
      reinterpret_cast<uint4*>(out)[v] = pack8(acc);
    }
  } else {
    const int rvec = cols >> 3;
    const long long rows = nvec / rvec;
    for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
      float ss = 0.f;
      for (int c = threadIdx.x; c < rvec; c += blockDim.x) {
        const long long v = r * rvec + c;
        float acc[8];
        const uint4 hv = reinterpret_cast<const uint4*>(residual)[v];
        lam_exchange(p, v, cap_vec, g3, reinterpret_cast<const uint4*>(x)[v], acc, err);
        accum8(acc, hv);
        const uint4 o = pack8(acc);
        const bf162* q = reinterpret_cast<const bf162*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(q[i]);
          ss += f.x * f.x + f.y * f.y;
        }
        reinterpret_cast<uint4*>(residual)[v] = o;
        lam_row[c] = o;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) tot += red[i];
      const float inv = rsqrtf(tot / static_cast<float>(cols) + eps);
      for (int c = threadIdx.x; c < rvec; c += blockDim.x) {
        uint4 a = lam_row[c];
        const uint4 wv = reinterpret_cast<const uint4*>(gamma)[c];
        bf162* ap = reinterpret_cast<bf162*>(&a);
        const bf162* wp = reinterpret_cast<const bf162*>(&wv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(ap[i]);
          const float2 gm = __bfloat1622float2(wp[i]);
          if (mbc) {
            ap[i] = __floats2bfloat162_rn(f.x * inv * (gm.x + w_off), f.y * inv * (gm.y + w_off));
          } else {
            const bf162 nrm = __floats2bfloat162_rn(f.x * inv, f.y * inv);
            const float2 nf = __bfloat1622float2(nrm);
            ap[i] = __floats2bfloat162_rn(nf.x * (gm.x + w_off), nf.y * (gm.y + w_off));
          }
        }
        reinterpret_cast<uint4*>(out)[r * rvec + c] = a;
      }
      __syncthreads();
    }
  }
  // the generation read two calls ago becomes sentinels again
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < old_vec;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    for (int src = 0; src < p.world; ++src)
      if (src != p.rank)
        reinterpret_cast<uint4*>(p.a[p.rank])[(static_cast<long long>(gclr) * p.world + src) * cap_vec + v] = sentinel;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(state + 4, 1);
    if (prev == static_cast<int>(gridDim.x) - 1) {
      state[4] = 0;
      state[1 + g3] = static_cast<int>(n);
      state[0] = gen + 1;
    }
  }
}

// Broadcast n bytes (n % 16 == 0) of root's symmetric buffer a[root] into out on every rank (pull).
__global__ void __launch_bounds__(256)
tp_broadcast_kernel(TpPeers p, int root, uint8_t* __restrict__ out, long long n, int* err) {
  const int epoch = ld_volatile(p.flags[p.rank] + kEpochWord) + 1;
  __syncthreads();
  tp_barrier_dev(p, 0, epoch, err);
  const long long nvec = n >> 4;
  const uint4* src = reinterpret_cast<const uint4*>(p.a[root]);
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x)
    reinterpret_cast<uint4*>(out)[v] = src[v];
  tp_finish_barrier(p, 1, epoch, err);
}

// Scatter: rank r pulls chunk r (n bytes, n % 16 == 0) of root's symmetric buffer a[root] into out.
// Reference: max/kernels/src/comm/scatter.mojo:61 (pull scatter).
__global__ void __launch_bounds__(256)
tp_scatter_kernel(TpPeers p, int root, uint8_t* __restrict__ out, long long n, int* err) {
  const int epoch = ld_volatile(p.flags[p.rank] + kEpochWord) + 1;
  __syncthreads();
  tp_barrier_dev(p, 0, epoch, err);
  const long long nvec = n >> 4;
  const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.a[root]) + static_cast<long long>(p.rank) * n);
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec;
       v += static_cast<long long>(gridDim.x) * blockDim.x)
    reinterpret_cast<uint4*>(out)[v] = src[v];
  tp_finish_barrier(p, 1, epoch, err);   // the root may not overwrite its buffer while a peer still reads it
}

// Waits (bounded) until *flag >= target; on timeout the error word receives `code` and the kernel
// returns normally, so the context stays usable. Used to probe a peer's progress flag from the host
// side of failure detection without ever blocking a GPU.
__global__ void tp_wait_flag_kernel(const int* flag, int target, unsigned long long timeout_ns, int code,
                                    int* err, int* ok_out) {
  const bool ok = wait_flag_ge(flag, target, err, code, timeout_ns);
  if (ok_out) *ok_out = ok ? 1 : 0;
}

static TpPeers make_peers(int world, int rank, void* const* a, void* const* b, int* const* flags) {
  TpPeers p;
  p.world = world; p.rank = rank;
  for (int i = 0; i < kMaxRanks; ++i) {
    p.a[i] = i < world && a ? a[i] : nullptr;
    p.b[i] = i < world && b ? b[i] : nullptr;
    p.flags[i] = i < world ? flags[i] : nullptr;
  }
  return p;
}

}  // namespace mb

using namespace mb;

extern "C" int mb_tp_flag_ints(void) { return kTpFlagInts; }

extern "C" int mb_tp_barrier(int world, int rank, int* const* flags, int* err, cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks) return MB_ERR_SHAPE;
  tp_barrier_kernel<<<1, 32, 0, stream>>>(make_peers(world, rank, nullptr, nullptr, flags), err);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_tp_rs_norm_ag(int world, int rank, void* const* partial_bufs, void* const* xn_bufs,
                                int* const* flags, void* h_local, const void* gamma, int M, int H,
                                int rows_per_rank, float eps, float w_off, int mbc, int has_partials,
                                int* err, cudaStream_t stream) {
  return mb_tp_rs_norm_ag_ex(world, rank, partial_bufs, xn_bufs, flags, h_local, gamma, M, H, rows_per_rank,
                             eps, w_off, mbc, has_partials, 0, 0, 0, err, stream);
}

extern "C" int mb_tp_rs_norm_ag_ex(int world, int rank, void* const* partial_bufs, void* const* xn_bufs,
                                   int* const* flags, void* h_local, const void* gamma, int M, int H,
                                   int rows_per_rank, float eps, float w_off, int mbc, int has_partials,
                                   int mode, int n_slots, int expected, int* err, cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || H % 8 || H > 32768) return MB_ERR_SHAPE;
  if (M <= 0) return MB_OK;
  int grid = rows_per_rank < 1 ? 1 : rows_per_rank;
  if (grid > 592) grid = 592;
  tp_rs_norm_ag_kernel<<<grid, 256, H * 2, stream>>>(
      make_peers(world, rank, partial_bufs, xn_bufs, flags), static_cast<bf16*>(h_local),
      static_cast<const bf16*>(gamma), M, H, rows_per_rank, eps, w_off, mbc, has_partials, mode, n_slots,
      expected, err);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_tp_allgather(int world, int rank, void* const* dst_bufs, int* const* flags,
                               const void* src, int rows, int row_bytes, int ld_src, int ld_dst,
                               long long col_off, int* err, cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || row_bytes % 16 || ld_src % 16 || ld_dst % 16 || col_off % 16)
    return MB_ERR_SHAPE;
  if (rows <= 0) return MB_OK;
  long long work = static_cast<long long>(rows) * (row_bytes / 16);
  int grid = static_cast<int>((work + 255) / 256);
  if (grid > 296) grid = 296;
  if (grid < 1) grid = 1;
  tp_allgather_kernel<<<grid, 256, 0, stream>>>(make_peers(world, rank, dst_bufs, nullptr, flags),
                                                static_cast<const uint8_t*>(src), rows, row_bytes,
                                                ld_src, ld_dst, col_off, err);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

// algo: 0 = choose by size (one-shot up to 512 KiB, two-shot above), 1 = one-shot, 2 = two-shot,
// 3 = multimem one-shot (needs `mc_in`). Two-shot writes the result into out_bufs[rank] (symmetric);
// the others write `out` (local). n = bf16 elements, multiple of 8.
extern "C" int mb_tp_allreduce(int world, int rank, void* const* in_bufs, void* const* out_bufs, void* out,
                               const void* mc_in, int* const* flags, long long n, int algo, int* err,
                               cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || n % 8) return MB_ERR_SHAPE;
  if (n <= 0) return MB_OK;
  if (algo == 0) algo = n * 2 <= (512 << 10) || out_bufs == nullptr ? 1 : 2;
  if (algo == 3 && mc_in == nullptr) return MB_ERR_SHAPE;
  if (algo == 2 && out_bufs == nullptr) return MB_ERR_SHAPE;
  const long long nvec = n >> 3;
  long long work = algo == 2 ? (nvec + world - 1) / world : nvec;
  int grid = static_cast<int>((work + 255) / 256);
  if (grid > 592) grid = 592;
  if (grid < 1) grid = 1;
  TpPeers p = make_peers(world, rank, in_bufs, out_bufs, flags);
  if (algo == 1)
    tp_allreduce_1shot_kernel<<<grid, 256, 0, stream>>>(p, static_cast<bf16*>(out), n, err);
  else if (algo == 2)
    tp_allreduce_2shot_kernel<<<grid, 256, 0, stream>>>(p, n, err);
  else if (algo == 3)
    tp_allreduce_multimem_kernel<<<grid, 256, 0, stream>>>(p, static_cast<const bf16*>(mc_in),
                                                           static_cast<bf16*>(out), n, err);
  else
    return MB_ERR_SHAPE;
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

// Barrier-free one-shot all-reduce of `x` (local bf16, n % 8 == 0, n <= cap) into `out` (local); see the kernel.
// gamma != nullptr: rows of `cols` elements, residual += sum (in place), out = RMSNorm(residual) * (gamma + w_off).
// `state` holds 8 zeroed ints that live as long as the receive buffers; every rank must issue the same calls.
extern "C" int mb_tp_allreduce_lamport(int world, int rank, void* const* lam_bufs, const void* x, void* out,
                                       long long n, long long cap, int* state, void* residual, const void* gamma,
                                       int cols, float eps, float w_off, int mbc, int* err, cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || n % 8 || cap % 8 || n > cap || n >= (1ll << 31)) return MB_ERR_SHAPE;
  if (n <= 0) return MB_OK;
  if (gamma != nullptr && (residual == nullptr || cols <= 0 || cols % 8 || n % cols || cols > 32768)) return MB_ERR_SHAPE;
  TpPeers p = make_peers(world, rank, lam_bufs, nullptr, lam_bufs ? reinterpret_cast<int* const*>(lam_bufs) : nullptr);
  for (int i = 0; i < kMaxRanks; ++i) p.flags[i] = nullptr;
  int grid;
  size_t smem = 0;
  if (gamma != nullptr) {
    grid = static_cast<int>(n / cols);
    smem = static_cast<size_t>(cols) * 2;
  } else {
    grid = static_cast<int>(((n >> 3) + 255) / 256);
  }
  if (grid > 592) grid = 592;
  if (grid < 1) grid = 1;
  tp_allreduce_lamport_kernel<<<grid, 256, smem, stream>>>(
      p, static_cast<const bf16*>(x), static_cast<bf16*>(out), n, cap, state, static_cast<bf16*>(residual),
      static_cast<const bf16*>(gamma), cols, eps, w_off, mbc, err);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_tp_broadcast(int world, int rank, int root, void* const* in_bufs, void* out, int* const* flags,
                               long long nbytes, int* err, cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || nbytes % 16 || root < 0 || root >= world) return MB_ERR_SHAPE;
  if (nbytes <= 0) return MB_OK;
  int grid = static_cast<int>(((nbytes >> 4) + 255) / 256);
  if (grid > 592) grid = 592;
  if (grid < 1) grid = 1;
  tp_broadcast_kernel<<<grid, 256, 0, stream>>>(make_peers(world, rank, in_bufs, nullptr, flags), root,
                                                static_cast<uint8_t*>(out), nbytes, err);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_tp_scatter(int world, int rank, int root, void* const* in_bufs, void* out, int* const* flags,
                             long long chunk_bytes, int* err, cudaStream_t stream) {
  if (world < 1 || world > kMaxRanks || chunk_bytes % 16 || root < 0 || root >= world) return MB_ERR_SHAPE;
  if (chunk_bytes <= 0) return MB_OK;
  int grid = static_cast<int>(((chunk_bytes >> 4) + 255) / 256);
  if (grid > 592) grid = 592;
  if (grid < 1) grid = 1;
  tp_scatter_kernel<<<grid, 256, 0, stream>>>(make_peers(world, rank, in_bufs, nullptr, flags), root,
                                              static_cast<uint8_t*>(out), chunk_bytes, err);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_tp_wait_flag(const int* flag, int target, unsigned timeout_ms, int code, int* err, int* ok_out,
                               cudaStream_t stream) {
  if (timeout_ms > 5000) timeout_ms = 5000;  // a wait in a kernel never exceeds a few seconds
  tp_wait_flag_kernel<<<1, 1, 0, stream>>>(flag, target, static_cast<unsigned long long>(timeout_ms) * 1000000ull,
                                           code, err, ok_out);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}
