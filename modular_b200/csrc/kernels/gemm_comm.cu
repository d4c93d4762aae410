// tcgen05 GEMMs fused with the tensor-parallel collective that precedes or follows them.
//
//   all-gather -> GEMM   (column-parallel linear: QKV, gate/up, LM head)
//       The activation rows of the other ranks are pushed into this rank's buffer by the
//       reduce+norm kernel of the producing rank, which then raises a per-source "ready" flag.
//       The GEMM's TMA producer waits only for the flags of the sources its token tile covers,
//       so tiles whose rows have landed start while the rest of the gather is still in flight;
//       there is no barrier between the gather and the GEMM.
//
//   GEMM -> reduce-scatter   (row-parallel linear: attention output, MLP down)
//       The epilogue stores every output row straight into the partial-sum slot of the rank that
//       owns the row (16-byte stores over NVLink, 256 contiguous bytes per row and tile). CTAs
//       count their finished tiles per owner on a local word; the last one forwards the count to
//       the owner with one remote add. The owner's reduce+norm kernel waits for that counter, so
//       the transfer of tile i overlaps the math of tile i+1 and nothing is ever staged in a
//       local partial buffer. With split-K every split owns a slot.
//
// Tile structure is that of gemm_tcgen05.cu: weights on the UMMA M side (128 rows per CTA),
// tokens on the N side (runtime BN), warp 0 = TMA, warp 1 = MMA issue, warps 2-5 = epilogue.
// All waits are bounded; a timed-out wait raises the error word and the CTA drains and leaves.
//
// Reference counterparts (separate kernels there): max/kernels/src/comm/allgather.mojo:167 +
// linalg matmul, max/kernels/src/comm/reducescatter.mojo, and the distributed matmul+allreduce
// split in max/kernels/src/linalg/distributed_matmul.mojo.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "comm_flags.h"
#include "gemm_common.h"

namespace mb {
namespace gc {

typedef __nv_bfloat16 bf16;
constexpr int kBM = 128, kBK = 64, kUmmaK = 16;
constexpr int kATileBytes = kBM * kBK * 2;
constexpr int kStageWarpBytes = 32 * 32 * 2;
constexpr int kThreads = 192;

struct CommArgs {
  int world, rank;
  int rows_per_rank;  // token rows owned by each rank (reduce-scatter) / contributed (all-gather)
  int wait_ready;     // 1: wait for the ready flags of the sources covered by the token tile
  int push;           // 1: epilogue writes into the owners' partial slots and signals them
  int* flags_local;
  int* peer_flags[kMaxRanks];
  bf16* partial[kMaxRanks];  // [world * splits slots][rows_per_rank][N] on every rank
};

struct SmemTail {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full;
  uint32_t tmem_base;
  int abort_word;
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

template <bool DUAL>
__global__ void __launch_bounds__(kThreads)
gemm_comm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                 bf16* __restrict__ Y, int M, int N, int K, int ldy, int dual_rows, int k_per_split,
                 int BN, int stages, uint32_t tmem_cols, int* err, const __grid_constant__ CommArgs ca) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int a_bytes = kATileBytes * (DUAL ? 2 : 1);
  const int b_bytes = BN * kBK * 2;
  const int stage_bytes = a_bytes + b_bytes;
  uint8_t* stage_buf = smem + stages * stage_bytes;
  SmemTail* tail = reinterpret_cast<SmemTail*>(stage_buf + 4 * kStageWarpBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t0 = blockIdx.x * BN, n0 = blockIdx.y * kBM, split = blockIdx.z;
  const int k_begin = split * k_per_split;
  const int k_end = min(K, k_begin + k_per_split);
  const int k_iters = (k_end - k_begin + kBK - 1) / kBK;
  const int t_last = min(t0 + BN, M) - 1;  // last valid token row of this tile

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&tail->full[s], 1);
      mbar_init(&tail->empty[s], 1);
    }
    mbar_init(&tail->tmem_full, 1);
    tail->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(&tail->tmem_base, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tail->tmem_base;
  volatile int* abort_word = &tail->abort_word;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    bool ready = true;
    if (ca.wait_ready) {
      // rows [s*rpr, (s+1)*rpr) come from rank s; this rank's own rows are signalled the same way
      const int s_lo = t0 / ca.rows_per_rank, s_hi = t_last / ca.rows_per_rank;
      const int want = ld_volatile(ca.flags_local + kReadyEpoch);
      bool mine = true;
      if (lane >= s_lo && lane <= s_hi && lane < ca.world)
        mine = wait_flag_ge(ca.flags_local + kReady + lane, want, err, 301);
      ready = __all_sync(0xffffffffu, mine);
      // the rows were written by other GPUs; order the TMA (async proxy) reads after the acquire
      asm volatile("fence.proxy.async;" ::: "memory");
      if (!ready && lane == 0) *abort_word = 301;
    }
    if (lane == 0 && ready) {
      int s = 0;       // stage and phase are carried: no division on the pipeline's latency path
      uint32_t ph = 0;
      for (int it = 0; it < k_iters; ++it) {
        if (!mbar_wait(&tail->empty[s], ph ^ 1, abort_word, err, 302)) break;
        uint8_t* sa = smem + s * stage_bytes;
        uint64_t* full_s = &tail->full[s];
        mbar_arrive_expect_tx(full_s, stage_bytes);
        const int kc = k_begin + it * kBK;
        tma_load_2d(sa, &tmW, full_s, kc, n0);
        if (DUAL) tma_load_2d(sa + kATileBytes, &tmW, full_s, kc, dual_rows + n0);
        tma_load_2d(sa + a_bytes, &tmX, full_s, kc, t0);
        if (++s == stages) { s = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kBM, BN, 1, 1);
      const uint64_t da0_first = umma_desc_sw128(smem);
      const uint64_t d_a1 = static_cast<uint64_t>(kATileBytes >> 4), d_b = static_cast<uint64_t>(a_bytes >> 4);
      const uint64_t d_stage = static_cast<uint64_t>(stage_bytes >> 4);
      uint64_t da0 = da0_first;
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0; it < k_iters; ++it) {
        if (!mbar_wait(&tail->full[s], ph, abort_word, err, 303)) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k) {
          const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
          const uint64_t koff = static_cast<uint64_t>(k * kUmmaK * 2 >> 4);
          umma_bf16(tmem_base, da0 + koff, da0 + d_b + koff, idesc, acc);
          if (DUAL) umma_bf16(tmem_base + BN, da0 + d_a1 + koff, da0 + d_b + koff, idesc, acc);
        }
        tc_commit(&tail->empty[s]);
        if (++s == stages) { s = 0; ph ^= 1; da0 = da0_first; } else { da0 += d_stage; }
      }
      tc_commit(&tail->tmem_full);
    }
  } else {
    // ---------------------------------------------------------------- epilogue (warps 2..5)
    const int quad = warp & 3;
    const bool ok = mbar_wait(&tail->tmem_full, 0, abort_word, err, 304);
    tc_fence_after();
    if (ok && k_iters > 0) {
      bf16* stg = reinterpret_cast<bf16*>(stage_buf + quad * kStageWarpBytes);
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      const int slot = ca.rank * static_cast<int>(gridDim.z) + split;
      for (int c0 = 0; c0 < BN; c0 += 16) {
        if (t0 + c0 >= M) break;  // warp-uniform
        uint32_t g[16];
        tmem_ld_32x16(lane_addr + c0, g);
        float v[16];
        if (DUAL) {
          uint32_t u[16];
          tmem_ld_32x16(lane_addr + BN + c0, u);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = silu_f(__uint_as_float(g[j])) * __uint_as_float(u[j]);
        } else {
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(g[j]);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) stg[j * 32 + lane] = __float2bfloat16(v[j]);
        __syncwarp();
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          const int j = pass * 8 + (lane >> 2);
          const int seg = lane & 3;
          const int t = t0 + c0 + j;
          const int n = n0 + quad * 32 + seg * 8;
          if (t < M && n < N) {
            const uint4 val = *reinterpret_cast<const uint4*>(stg + j * 32 + seg * 8);
            bf16* dst;
            if (ca.push) {
              const int owner = t / ca.rows_per_rank;
              const int r = t - owner * ca.rows_per_rank;
              dst = ca.partial[owner] +
                    (static_cast<size_t>(slot) * ca.rows_per_rank + r) * static_cast<size_t>(ldy) + n;
            } else {
              dst = Y + static_cast<size_t>(t) * ldy + n;
            }
            *reinterpret_cast<uint4*>(dst) = val;
          }
        }
        __syncwarp();
      }
      if (ca.push) __threadfence_system();  // this thread's remote stores before the CTA's signal
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
  if (ca.push && warp == 2 && k_iters > 0 && *abort_word == 0) {
    // Tell each owner this CTA touched that its tile has landed. Remote atomics on one word are
    // slow (they serialise over NVLink), so CTAs count on a local word per owner and only the last
    // one of this GEMM forwards the whole count with a single remote add.
    const int o_lo = t0 / ca.rows_per_rank, o_hi = t_last / ca.rows_per_rank;
    if (lane >= o_lo && lane <= o_hi && lane < ca.world) {
      const int lo = lane * ca.rows_per_rank;
      const int hi = min(lo + ca.rows_per_rank, M) - 1;
      const int total = (hi / BN - lo / BN + 1) * static_cast<int>(gridDim.y * gridDim.z);
      __threadfence_system();  // this CTA's remote stores are visible before it is counted
      const int prev = atomicAdd(ca.flags_local + kPushLocal + lane, 1);
      if (prev == total - 1) {
        ca.flags_local[kPushLocal + lane] = 0;  // every CTA of this GEMM has arrived: reset for the next
        __threadfence_system();
        red_release_sys_add(ca.peer_flags[lane] + kPushCount, total);
      }
    }
  }
}

template <bool DUAL>
static int launch(const CUtensorMap& tw, const CUtensorMap& tx, void* Y, int M, int N, int K, int ldy,
                  int dual_rows, int k_per_split, int splits, int BN, int stages, int* err,
                  const CommArgs& ca, cudaStream_t stream) {
  const int stage_bytes = kATileBytes * (DUAL ? 2 : 1) + BN * kBK * 2;
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + 4 * kStageWarpBytes + sizeof(SmemTail) + 1024;
  auto kern = gemm_comm_kernel<DUAL>;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return MB_ERR_LAUNCH;
    configured.done();
  }
  uint32_t tmem_cols = 32;
  while (static_cast<int>(tmem_cols) < (DUAL ? 2 * BN : BN)) tmem_cols <<= 1;
  dim3 grid((M + BN - 1) / BN, (N + kBM - 1) / kBM, splits);
  kern<<<grid, kThreads, smem, stream>>>(tw, tx, static_cast<bf16*>(Y), M, N, K, ldy, dual_rows, k_per_split,
                                         BN, stages, tmem_cols, err, ca);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

}  // namespace gc
}  // namespace mb

using namespace mb;

// Y = X · W^T for one tensor-parallel rank, fused with the neighbouring collective.
//   flags bit0  dual (SwiGLU over W = [gate; up])
//         bit4  wait_ready: X is this rank's gathered activation buffer; tiles wait for the
//               per-source ready flags in `flags_all[rank]`
//         bit5  push: rows go to `partial_all[owner]` (reduce-scatter layout
//               [world*splits][rows_per_rank][N]); `*expected_out` receives the number of counter
//               increments the owner `rank` must wait for (identical shapes on every rank)
// Without bit5 the result is stored to the local Y (ldy). Split-K (`splits` > 1) only with bit5.
extern "C" int mb_gemm_bf16_comm(const void* X, const void* W, void* Y, int M, int N, int K, int ldx, int ldw,
                                 int ldy, int flags, int bn, int splits, int world, int rank, int rows_per_rank,
                                 int* const* flags_all, void* const* partial_all, int max_slots,
                                 int* expected_out, int* splits_out, int* err, int num_sms, cudaStream_t stream) {
  if (expected_out) *expected_out = 0;
  if (M <= 0 || N <= 0) return MB_OK;
  const bool dual = flags & 1, wait_ready = flags & 16, push = flags & 32;
  if (world < 1 || world > kMaxRanks || rows_per_rank < 1) return MB_ERR_SHAPE;
  if (K % 8 || ldx % 8 || ldw % 8 || N % 8 || ldy % 8 || (dual && push)) return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(Y)) & 15)
    return MB_ERR_ALIGN;
  int pbn, psp, pst;
  mb_gemm_bf16_plan(M, N, K, dual, num_sms > 0 ? num_sms : 148, &pbn, &psp, &pst);
  if (bn <= 0) bn = pbn;
  if (bn % 16 || bn > (dual ? 128 : 256)) return MB_ERR_SHAPE;
  if (splits <= 0) splits = psp;
  if (!push) splits = 1;
  int k_per_split = K;
  if (splits > 1) {
    const int k_blocks = (K + gc::kBK - 1) / gc::kBK;
    k_per_split = ((k_blocks + splits - 1) / splits) * gc::kBK;
    splits = (K + k_per_split - 1) / k_per_split;
  }
  if (push && world * splits > max_slots) {
    splits = max_slots / world;
    if (splits < 1) return MB_ERR_TOO_LARGE;
    const int k_blocks = (K + gc::kBK - 1) / gc::kBK;
    k_per_split = ((k_blocks + splits - 1) / splits) * gc::kBK;
    splits = (K + k_per_split - 1) / k_per_split;
  }
  const int stage_bytes = gc::kATileBytes * (dual ? 2 : 1) + bn * gc::kBK * 2;
  int stages = (227 * 1024 - 1024 - 4 * gc::kStageWarpBytes - 512) / stage_bytes;
  if (stages > 8) stages = 8;
  if (pst < stages) stages = pst;  // keeps two CTAs per SM where the plan asks for it
  if (stages < 1) return MB_ERR_SHAPE;

  gc::CommArgs ca;
  ca.world = world; ca.rank = rank; ca.rows_per_rank = rows_per_rank;
  ca.wait_ready = wait_ready ? 1 : 0; ca.push = push ? 1 : 0;
  ca.flags_local = flags_all ? flags_all[rank] : nullptr;
  for (int i = 0; i < kMaxRanks; ++i) {
    ca.peer_flags[i] = i < world && flags_all ? flags_all[i] : nullptr;
    ca.partial[i] = i < world && partial_all ? static_cast<gc::bf16*>(partial_all[i]) : nullptr;
  }
  if ((wait_ready || push) && ca.flags_local == nullptr) return MB_ERR_SHAPE;
  if (push && partial_all == nullptr) return MB_ERR_SHAPE;

  if (push && expected_out) {
    // token tiles that intersect this rank's rows, times weight tiles, splits and source ranks
    const int lo = rank * rows_per_rank;
    const int hi = (lo + rows_per_rank < M ? lo + rows_per_rank : M) - 1;
    int m_tiles_mine = 0;
    if (hi >= lo) m_tiles_mine = hi / bn - lo / bn + 1;
    *expected_out = m_tiles_mine * ((N + gc::kBM - 1) / gc::kBM) * splits * world;
  }
  if (splits_out) *splits_out = splits;

  CUtensorMap tw, tx;
  int rc = cached_tmap(&tw, W, dual ? 2 * N : N, K, ldw, gc::kBM, 2);
  if (rc != MB_OK) return rc;
  rc = cached_tmap(&tx, X, M, K, ldx, bn, 2);
  if (rc != MB_OK) return rc;
  if (dual)
    return gc::launch<true>(tw, tx, Y, M, N, K, ldy, N, k_per_split, splits, bn, stages, err, ca, stream);
  return gc::launch<false>(tw, tx, Y, M, N, K, ldy, 0, k_per_split, splits, bn, stages, err, ca, stream);
}
