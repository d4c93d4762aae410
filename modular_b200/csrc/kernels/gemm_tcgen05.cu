// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   Y[M, N] = X[M, K] · W[N, K]^T            (nn.Linear layout, both operands K-major)
//
// The weight matrix always sits on the UMMA "M" side (128 weight rows per CTA tile)
// and the activations on the UMMA "N" side (BN tokens, any multiple of 16 up to 256,
// chosen at run time). Serving batches are ragged in the token count, so putting the
// tokens on the side with 16-granularity keeps the tensor cores full at M = 64..600
// where a 128-row token tile would waste up to half of every instruction.
//
// One CTA = 6 warps:
//   warp 0     TMA producer   (cp.async.bulk.tensor 2-D, 128B swizzle, no multicast)
//   warp 1     MMA issuer     (tcgen05.mma kind::f16, fp32 accumulators in TMEM)
//   warps 2-5  epilogue       (tcgen05.ld -> registers -> smem transpose -> 16-byte stores)
//
// Fused epilogues: bf16 store, bf16 store with residual add, fp32 store (split-K
// partials / logits), and a "dual" mode where two weight tiles (gate, up) feed two
// accumulators and the epilogue writes silu(gate) * up.
//
// Behavioural counterpart in the reference: the warp-specialised sm100 matmul
// (max/kernels/src/linalg/matmul/gpu/sm100_structured/default/matmul_kernels.mojo:348)
// and its fused SwiGLU variant (sm100_structured/fused_swiglu/matmul_swiglu_kernels.mojo).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <unordered_map>

#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "../common/api.h"
#include "comm_flags.h"
#include "gemm_common.h"

namespace mb {

constexpr int kBM = 128;          // weight rows per tile (UMMA M)
constexpr int kBK = 64;           // bf16 elements per 128-byte swizzle row
constexpr int kUmmaK = 16;        // K of one tcgen05.mma kind::f16
constexpr int kATileBytes = kBM * kBK * 2;  // 16 KiB
constexpr int kStageWarpBytes = 32 * 32 * 2;  // per-epilogue-warp transpose buffer
constexpr int kGemmThreads = 192;

enum GemmEpi { EPI_BF16 = 0, EPI_BF16_RESIDUAL = 1, EPI_F32 = 2 };

struct GemmSmemTail {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full;
  uint32_t tmem_base;
  int abort_word;
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// Epilogue of one accumulator tile by one warp: TMEM lanes [quad*32, +32) = weight rows
// n0 + quad*32 + lane, columns [0, BN) = tokens t0.. (DUAL: gate at column 0, up at column BN).
template <bool DUAL, int EPI>
__device__ __forceinline__ void epilogue_tile(uint32_t tmem_base, uint8_t* stage_buf, int quad, int lane,
                                              void* __restrict__ Yv, const __nv_bfloat16* __restrict__ R,
                                              int M, int N, int ldy, int ldr, int BN, int n0, int t0,
                                              int Mlim, int split) {
    __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(stage_buf + quad * kStageWarpBytes);
    const int n_row = n0 + quad * 32 + lane;  // weight row (= output column) of this thread
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    // Residual rows are fetched one 16-token chunk ahead: a load issued only after the transpose would put a
    // global round trip (two per chunk) on the epilogue's critical path, which is longer than the TMEM read,
    // the transpose and the stores together.
    uint4 rv[2];
    auto fetch_residual = [&](int c0) {
#pragma unroll
      for (int pass = 0; pass < 2; ++pass) {
        const int t = t0 + c0 + pass * 8 + (lane >> 2);
        const int n = n0 + quad * 32 + (lane & 3) * 8;
        rv[pass] = make_uint4(0u, 0u, 0u, 0u);
        if (c0 < BN && t < Mlim && n < N)
          rv[pass] = *reinterpret_cast<const uint4*>(R + static_cast<size_t>(t) * ldr + n);
      }
    };
    if (EPI == EPI_BF16_RESIDUAL) fetch_residual(0);
    for (int c0 = 0; c0 < BN; c0 += 16) {
      if (t0 + c0 >= Mlim) break;  // warp-uniform
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
      if (EPI == EPI_F32) {
        float* Y = reinterpret_cast<float*>(Yv) + static_cast<size_t>(split) * M * ldy;
        if (n_row < N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int t = t0 + c0 + j;
            if (t < Mlim) Y[static_cast<size_t>(t) * ldy + n_row] = v[j];
          }
        }
      } else {
        __nv_bfloat16* Y = reinterpret_cast<__nv_bfloat16*>(Yv);
        // transpose through this warp's private buffer: stg[token j][weight row lane]
#pragma unroll
        for (int j = 0; j < 16; ++j) stg[j * 32 + lane] = __float2bfloat16(v[j]);
        __syncwarp();
        uint4 cur[2];
        if (EPI == EPI_BF16_RESIDUAL) {
          cur[0] = rv[0];
          cur[1] = rv[1];
          fetch_residual(c0 + 16);   // in flight while this chunk is added up and stored
        }
        // 16 tokens x 64 bytes: 4 lanes cover one token row, 8 tokens per pass
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          const int j = pass * 8 + (lane >> 2);
          const int seg = lane & 3;
          const int t = t0 + c0 + j;
          const int n = n0 + quad * 32 + seg * 8;
          if (t < Mlim && n < N) {
            uint4 val = *reinterpret_cast<const uint4*>(stg + j * 32 + seg * 8);
            if (EPI == EPI_BF16_RESIDUAL) {
              __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&val);
              const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&cur[pass]);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float2 fa = __bfloat1622float2(a[q]);
                const float2 fb = __bfloat1622float2(b[q]);
                a[q] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
              }
            }
            *reinterpret_cast<uint4*>(Y + static_cast<size_t>(t) * ldy + n) = val;
          }
        }
        __syncwarp();
      }
    }
}

template <bool DUAL, int EPI>
__global__ void __launch_bounds__(kGemmThreads)
gemm_wx_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
               void* __restrict__ Yv, const __nv_bfloat16* __restrict__ R, int M, int N, int K,
               int ldy, int ldr, int dual_rows, int k_per_split, int BN, int stages,
               uint32_t tmem_cols, int* err, const int32_t* __restrict__ expert_offsets,
               int w_rows_per_expert, const int* gate_flags, int gate_rpr, int gate_world,
               int packed_kb, int x_batch_off, int y_batch_off, int w_static) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int a_bytes = kATileBytes * (DUAL ? 2 : 1);
  const int b_bytes = BN * kBK * 2;
  const int stage_bytes = a_bytes + b_bytes;
  uint8_t* stage_buf = smem + stages * stage_bytes;  // 4 * 2 KiB epilogue transpose buffers
  GemmSmemTail* tail = reinterpret_cast<GemmSmemTail*>(stage_buf + 4 * kStageWarpBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tile = blockIdx.x;  // token tile (fast index: CTAs sharing a weight tile co-run)
  const int n_tile = blockIdx.y;  // weight-row tile
  // Grouped (mixture-of-experts) mode: blockIdx.z is the expert, its token rows are
  // [expert_offsets[e], expert_offsets[e+1]) of X / Y and its weights start at row
  // e * w_rows_per_expert of W. CTAs beyond an expert's rows leave before touching TMEM.
  int split = blockIdx.z;
  const int n0 = n_tile * kBM;
  int t0 = m_tile * BN;
  int Mlim = M, w_row0 = 0;
  if (expert_offsets != nullptr) {
    pdl_wait();  // the offsets are produced by the routing kernels
    const int e = blockIdx.z;
    const int row_begin = expert_offsets[e], row_end = expert_offsets[e + 1];
    t0 = row_begin + m_tile * BN;
    if (t0 >= row_end) return;
    Mlim = row_end;
    w_row0 = e * w_rows_per_expert;
    split = 0;
  }
  // Batched mode (x_batch_off > 0): blockIdx.z is the batch entry b (an attention head); it reads the K columns
  // of X that start at b * x_batch_off, weights W[b] and writes the N columns of Y that start at b * y_batch_off.
  int xk0 = 0;
  if (x_batch_off > 0) {
    const int b = blockIdx.z;
    w_row0 = b * w_rows_per_expert;
    xk0 = b * x_batch_off;
    Yv = static_cast<__nv_bfloat16*>(Yv) + static_cast<size_t>(b) * y_batch_off;
    split = 0;
  }
  const int k_begin = split * k_per_split;
  const int k_end = min(K, k_begin + k_per_split);
  const int k_iters = (k_end - k_begin + kBK - 1) / kBK;

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
  // Weights that no kernel on the stream writes (w_static) are requested before the wait: the first ring stages
  // fill while the previous kernel drains, the activation tiles follow after the wait on the same barriers.
  int pre = 0;
  if (w_static && expert_offsets == nullptr && gate_flags == nullptr && warp == 0 && lane == 0) {
    pre = k_iters < stages ? k_iters : stages;
    for (int it = 0; it < pre; ++it) {
      uint8_t* sa = smem + it * stage_bytes;
      uint64_t* full_s = &tail->full[it];
      mbar_arrive_expect_tx(full_s, stage_bytes);
      const int kc = k_begin + it * kBK;
      if (packed_kb > 0) {
        const int kb = kc / kBK;
        tma_load_2d(sa, &tmW, full_s, 0, (((w_row0 + n0) >> 7) * packed_kb + kb) << 7);
        if (DUAL) tma_load_2d(sa + kATileBytes, &tmW, full_s, 0, (((w_row0 + dual_rows + n0) >> 7) * packed_kb + kb) << 7);
      } else {
        tma_load_2d(sa, &tmW, full_s, kc, w_row0 + n0);
        if (DUAL) tma_load_2d(sa + kATileBytes, &tmW, full_s, kc, w_row0 + dual_rows + n0);
      }
    }
  }
  // everything above touched only this CTA's own resources and static weights; the other operands are produced
  // by earlier kernels on the stream (no-op unless launched as a programmatic dependent)
  pdl_wait();
  pdl_trigger();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    bool ready = true;
    if (gate_flags != nullptr) {
      // Tensor-parallel all-gather -> GEMM: token rows [s*rpr, (s+1)*rpr) are pushed into X by rank
      // s, which then raises flag kReady+s; wait only for the sources this token tile covers.
      const int t_last = min(t0 + BN, M) - 1;
      const int s_lo = t0 / gate_rpr, s_hi = t_last / gate_rpr;
      const int want = ld_volatile(gate_flags + kReadyEpoch);
      bool mine = true;
      if (lane >= s_lo && lane <= s_hi && lane < gate_world)
        mine = wait_flag_ge(gate_flags + kReady + lane, want, err, 105);
      ready = __all_sync(0xffffffffu, mine);
      asm volatile("fence.proxy.async;" ::: "memory");  // TMA reads after the acquire
      if (!ready && lane == 0) *abort_word = 105;
    }
    if (lane == 0 && ready) {
      // the stage index and phase are carried, not divided out of `it`: this loop and the MMA loop below sit
      // on the latency path of the pipeline (a stage is refilled only after both have turned around)
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0; it < k_iters; ++it) {
        uint8_t* sa = smem + s * stage_bytes;
        uint8_t* sb = sa + a_bytes;
        uint64_t* full_s = &tail->full[s];
        const int kc = k_begin + it * kBK;
        if (it < pre) {
          // the stage was armed and its weight tile requested before the wait
          if (++s == stages) { s = 0; ph ^= 1; }
          tma_load_2d(sb, &tmX, full_s, xk0 + kc, t0);
          continue;
        }
        if (!mbar_wait(&tail->empty[s], ph ^ 1, abort_word, err, 101)) break;
        mbar_arrive_expect_tx(full_s, stage_bytes);
        if (++s == stages) { s = 0; ph ^= 1; }
        if (packed_kb > 0) {
          // pre-tiled weights: tile (row block, K block) is one contiguous 16 KiB run in memory,
          // addressed as 128 rows of the [tiles * 128, 64] view
          const int kb = kc / kBK;
          tma_load_2d(sa, &tmW, full_s, 0, (((w_row0 + n0) >> 7) * packed_kb + kb) << 7);
          if (DUAL)
            tma_load_2d(sa + kATileBytes, &tmW, full_s, 0,
                        (((w_row0 + dual_rows + n0) >> 7) * packed_kb + kb) << 7);
        } else {
          tma_load_2d(sa, &tmW, full_s, kc, w_row0 + n0);
          if (DUAL) tma_load_2d(sa + kATileBytes, &tmW, full_s, kc, w_row0 + dual_rows + n0);
        }
        tma_load_2d(sb, &tmX, full_s, xk0 + kc, t0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kBM, BN, 1, 1);
      bool ok = true;
      // descriptors advance by one stage per iteration (the address field counts 16-byte units)
      const uint64_t da0_first = umma_desc_sw128(smem);
      const uint64_t d_a1 = static_cast<uint64_t>(kATileBytes >> 4), d_b = static_cast<uint64_t>(a_bytes >> 4);
      const uint64_t d_stage = static_cast<uint64_t>(stage_bytes >> 4);
      uint64_t da0 = da0_first;
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0; it < k_iters && ok; ++it) {
        ok = mbar_wait(&tail->full[s], ph, abort_word, err, 102);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k) {
          const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
          const uint64_t koff = static_cast<uint64_t>(k * kUmmaK * 2 >> 4);
          umma_bf16(tmem_base, da0 + koff, da0 + d_b + koff, idesc, acc);
          if (DUAL) umma_bf16(tmem_base + BN, da0 + d_a1 + koff, da0 + d_b + koff, idesc, acc);
        }
        tc_commit(&tail->empty[s]);  // frees the smem stage when these MMAs retire
        if (++s == stages) { s = 0; ph ^= 1; da0 = da0_first; } else { da0 += d_stage; }
      }
      tc_commit(&tail->tmem_full);
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    const bool ok = mbar_wait(&tail->tmem_full, 0, abort_word, err, 103);
    tc_fence_after();
    if (ok && k_iters > 0)
      epilogue_tile<DUAL, EPI>(tmem_base, stage_buf, quad, lane, Yv, R, M, N, ldy, ldr, BN, n0, t0, Mlim, split);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ------------------------------------------------------------------ CTA-pair variant
// Same GEMM with cta_group::2 MMAs: a cluster of two CTAs owns 256 weight rows x BN tokens. Each CTA
// loads its own 128 weight rows and HALF of the token tile; the leader (even) CTA issues
// 256 x BN x 16 MMAs that read both halves, and each CTA's TMEM receives the accumulator of its own
// weight rows. Per CTA and K step the shared-memory traffic is 128 + BN/2 rows instead of
// 128 + BN, which is what lifts the tensor pipe past the one-CTA shared-memory bound.
//   full[s]   lives in the leader: its producer posts the byte count of both CTAs' loads, and both
//             CTAs' TMA loads complete on it.
//   empty[s]  one per CTA, released by the leader's commits (one commit per CTA).
//   tmem_full one per CTA, likewise.
// grid = (2 * token tiles, weight-row pairs, K splits), cluster = (2, 1, 1).
template <bool DUAL, int EPI>
__global__ void __launch_bounds__(kGemmThreads)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                 void* __restrict__ Yv, const __nv_bfloat16* __restrict__ R, int M, int N, int K,
                 int ldy, int ldr, int dual_rows, int k_per_split, int BN, int stages,
                 uint32_t tmem_cols, int* err, const int* gate_flags, int gate_rpr, int gate_world,
                 int packed_kb) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int half = BN >> 1;
  const int a_bytes = kATileBytes * (DUAL ? 2 : 1);
  const int b_bytes = half * kBK * 2;
  const int stage_bytes = a_bytes + b_bytes;
  uint8_t* stage_buf = smem + stages * stage_bytes;
  GemmSmemTail* tail = reinterpret_cast<GemmSmemTail*>(stage_buf + 4 * kStageWarpBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const int m_tile = blockIdx.x >> 1;
  const int n0 = blockIdx.y * (2 * kBM) + static_cast<int>(rank) * kBM;   // this CTA's weight rows
  const int t0 = m_tile * BN;                                              // the pair's token tile
  const int tb0 = t0 + static_cast<int>(rank) * half;                      // this CTA's half of it
  const int split = blockIdx.z;
  const int k_begin = split * k_per_split;
  const int k_end = min(K, k_begin + k_per_split);
  const int k_iters = (k_end - k_begin + kBK - 1) / kBK;

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
    tmem_alloc_pair(&tail->tmem_base, tmem_cols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = tail->tmem_base;
  volatile int* abort_word = &tail->abort_word;
  pdl_wait();
  pdl_trigger();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    bool ready = true;
    if (gate_flags != nullptr) {
      const int t_last = min(tb0 + half, M) - 1;
      const int s_lo = tb0 / gate_rpr, s_hi = t_last / gate_rpr;   // empty range when tb0 >= M
      const int want = ld_volatile(gate_flags + kReadyEpoch);
      bool mine = true;
      if (lane >= s_lo && lane <= s_hi && lane < gate_world)
        mine = wait_flag_ge(gate_flags + kReady + lane, want, err, 115);
      ready = __all_sync(0xffffffffu, mine);
      asm volatile("fence.proxy.async;" ::: "memory");
      if (!ready && lane == 0) *abort_word = 115;
    }
    if (lane == 0 && ready) {
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0; it < k_iters; ++it) {
        if (!mbar_wait(&tail->empty[s], ph ^ 1, abort_word, err, 111)) break;
        uint8_t* sa = smem + s * stage_bytes;
        uint8_t* sb = sa + a_bytes;
        if (rank == 0) mbar_arrive_expect_tx(&tail->full[s], 2 * stage_bytes);
        const uint32_t full_leader = mapa_shared(&tail->full[s], 0);
        const int kc = k_begin + it * kBK;
        if (++s == stages) { s = 0; ph ^= 1; }
        if (packed_kb > 0) {
          const int kb = kc / kBK;
          tma_load_2d_pair(sa, &tmW, full_leader, 0, ((n0 >> 7) * packed_kb + kb) << 7);
          if (DUAL)
            tma_load_2d_pair(sa + kATileBytes, &tmW, full_leader, 0,
                             (((dual_rows + n0) >> 7) * packed_kb + kb) << 7);
        } else {
          tma_load_2d_pair(sa, &tmW, full_leader, kc, n0);
          if (DUAL) tma_load_2d_pair(sa + kATileBytes, &tmW, full_leader, kc, dual_rows + n0);
        }
        tma_load_2d_pair(sb, &tmX, full_leader, kc, tb0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc(2 * kBM, BN, 1, 1);
      bool ok = true;
      const uint64_t da0_first = umma_desc_sw128(smem);
      const uint64_t d_a1 = static_cast<uint64_t>(kATileBytes >> 4), d_b = static_cast<uint64_t>(a_bytes >> 4);
      const uint64_t d_stage = static_cast<uint64_t>(stage_bytes >> 4);
      const uint32_t empty0 = mapa_shared(&tail->empty[0], 0), empty1 = mapa_shared(&tail->empty[0], 1);
      uint64_t da0 = da0_first;
      int s = 0;
      uint32_t ph = 0;
      for (int it = 0; it < k_iters && ok; ++it) {
        ok = mbar_wait(&tail->full[s], ph, abort_word, err, 112);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k) {
          const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
          const uint64_t koff = static_cast<uint64_t>(k * kUmmaK * 2 >> 4);
          umma_bf16_pair(tmem_base, da0 + koff, da0 + d_b + koff, idesc, acc);
          if (DUAL) umma_bf16_pair(tmem_base + BN, da0 + d_a1 + koff, da0 + d_b + koff, idesc, acc);
        }
        tc_commit_pair(empty0 + 8u * s);   // mbarriers are 8 bytes apart, at the same offset in both CTAs
        tc_commit_pair(empty1 + 8u * s);
        if (++s == stages) { s = 0; ph ^= 1; da0 = da0_first; } else { da0 += d_stage; }
      }
      tc_commit_pair(mapa_shared(&tail->tmem_full, 0));
      tc_commit_pair(mapa_shared(&tail->tmem_full, 1));
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    const bool ok = mbar_wait(&tail->tmem_full, 0, abort_word, err, 113);
    tc_fence_after();
    if (ok && k_iters > 0)
      epilogue_tile<DUAL, EPI>(tmem_base, stage_buf, quad, lane, Yv, R, M, N, ldy, ldr, BN, n0, t0, M, split);
  }

  // neither CTA may leave (or free TMEM) while the other can still read its shared memory, signal
  // its barriers or run MMAs into its TMEM
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, tmem_cols);
  }
}

// ------------------------------------------------------------------ persistent CTA-pair variant
// The pair kernel above spends a TMEM allocation, a cluster barrier, a cold TMA ring and an epilogue that no
// MMA overlaps on every tile. Here one pair per two SMs walks over tiles t = cluster, cluster + clusters, ...
// (token tile fastest, so the pairs running at the same time share weight panels in L2). The operand ring
// keeps running across tiles, and the accumulator has two TMEM stages of 256 columns: while the epilogue
// warps of both CTAs drain stage a, the leader's MMAs fill stage a ^ 1.
//   tmem_full[a]   one per CTA, completed by the leader's commit after the tile's last MMA
//   tmem_empty[a]  in the leader, one arrival per epilogue warp of either CTA (eight)
struct PairPersistTail {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_word;
};
constexpr int kAccStageCols = 256;

template <bool DUAL, int EPI>
__global__ void __launch_bounds__(kGemmThreads)
gemm_pair_persistent_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                            void* __restrict__ Yv, const __nv_bfloat16* __restrict__ R, int M, int N, int K,
                            int ldy, int ldr, int dual_rows, int BN, int stages, int m_tiles, int total_tiles,
                            int* err, int packed_kb) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int half = BN >> 1;
  const int a_bytes = kATileBytes * (DUAL ? 2 : 1);
  const int b_bytes = half * kBK * 2;
  const int stage_bytes = a_bytes + b_bytes;
  uint8_t* stage_buf = smem + stages * stage_bytes;
  PairPersistTail* tail = reinterpret_cast<PairPersistTail*>(stage_buf + 4 * kStageWarpBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const int cluster = blockIdx.x >> 1, clusters = gridDim.x >> 1;
  const int k_iters = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&tail->full[s], 1);
      mbar_init(&tail->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tail->tmem_full[a], 1);
      mbar_init(&tail->tmem_empty[a], 8);
    }
    tail->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc_pair(&tail->tmem_base, 2 * kAccStageCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = tail->tmem_base;
  volatile int* abort_word = &tail->abort_word;
  pdl_wait();
  pdl_trigger();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = cluster; t < total_tiles && ok; t += clusters) {
        const int n0 = (t / m_tiles) * (2 * kBM) + static_cast<int>(rank) * kBM;
        const int tb0 = (t % m_tiles) * BN + static_cast<int>(rank) * half;
        for (int it = 0; it < k_iters; ++it) {
          if (!mbar_wait(&tail->empty[s], ph ^ 1, abort_word, err, 116)) { ok = false; break; }
          uint8_t* sa = smem + s * stage_bytes;
          if (rank == 0) mbar_arrive_expect_tx(&tail->full[s], 2 * stage_bytes);
          const uint32_t full_leader = mapa_shared(&tail->full[s], 0);
          const int kc = it * kBK;
          if (++s == stages) { s = 0; ph ^= 1; }
          if (packed_kb > 0) {
            tma_load_2d_pair(sa, &tmW, full_leader, 0, ((n0 >> 7) * packed_kb + (kc / kBK)) << 7);
            if (DUAL)
              tma_load_2d_pair(sa + kATileBytes, &tmW, full_leader, 0,
                               (((dual_rows + n0) >> 7) * packed_kb + (kc / kBK)) << 7);
          } else {
            tma_load_2d_pair(sa, &tmW, full_leader, kc, n0);
            if (DUAL) tma_load_2d_pair(sa + kATileBytes, &tmW, full_leader, kc, dual_rows + n0);
          }
          tma_load_2d_pair(sa + a_bytes, &tmX, full_leader, kc, tb0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc(2 * kBM, BN, 1, 1);
      const uint64_t da0_first = umma_desc_sw128(smem);
      const uint64_t d_a1 = static_cast<uint64_t>(kATileBytes >> 4), d_b = static_cast<uint64_t>(a_bytes >> 4);
      const uint64_t d_stage = static_cast<uint64_t>(stage_bytes >> 4);
      const uint32_t empty0 = mapa_shared(&tail->empty[0], 0), empty1 = mapa_shared(&tail->empty[0], 1);
      const uint32_t tfull0 = mapa_shared(&tail->tmem_full[0], 0), tfull1 = mapa_shared(&tail->tmem_full[0], 1);
      uint64_t da0 = da0_first;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int i = 0;   // tiles done by this pair
      for (int t = cluster; t < total_tiles && ok; t += clusters, ++i) {
        const int a = i & 1;
        // the epilogues of the tile that used this accumulator stage two tiles ago have read it out
        ok = mbar_wait(&tail->tmem_empty[a], ((i >> 1) & 1) ^ 1, abort_word, err, 117);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(a * kAccStageCols);
        for (int it = 0; it < k_iters; ++it) {
          ok = mbar_wait(&tail->full[s], ph, abort_word, err, 118);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
            const uint64_t koff = static_cast<uint64_t>(k * kUmmaK * 2 >> 4);
            umma_bf16_pair(d_tmem, da0 + koff, da0 + d_b + koff, idesc, acc);
            if (DUAL) umma_bf16_pair(d_tmem + BN, da0 + d_a1 + koff, da0 + d_b + koff, idesc, acc);
          }
          tc_commit_pair(empty0 + 8u * s);   // mbarriers are 8 bytes apart, at the same offset in both CTAs
          tc_commit_pair(empty1 + 8u * s);
          if (++s == stages) { s = 0; ph ^= 1; da0 = da0_first; } else { da0 += d_stage; }
        }
        if (!ok) break;
        tc_commit_pair(tfull0 + 8u * a);
        tc_commit_pair(tfull1 + 8u * a);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    const uint32_t tempty_leader = mapa_shared(&tail->tmem_empty[0], 0);
    int i = 0;
    for (int t = cluster; t < total_tiles; t += clusters, ++i) {
      const int a = i & 1;
      if (!mbar_wait(&tail->tmem_full[a], (i >> 1) & 1, abort_word, err, 119)) break;
      tc_fence_after();
      const int n0 = (t / m_tiles) * (2 * kBM) + static_cast<int>(rank) * kBM;
      const int t0 = (t % m_tiles) * BN;
      if (k_iters > 0)
        epilogue_tile<DUAL, EPI>(tmem_base + static_cast<uint32_t>(a * kAccStageCols), stage_buf, quad, lane, Yv, R,
                                  M, N, ldy, ldr, BN, n0, t0, M, 0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader + 8u * a);
    }
  }

  // neither CTA may leave (or free TMEM) while the other can still read its shared memory, signal
  // its barriers or run MMAs into its TMEM
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * kAccStageCols);
  }
}

// ------------------------------------------------------------------ persistent CTA pairs, tokens on the MMA's M side
// Same schedule as gemm_pair_persistent_kernel with the operand roles swapped: the pair's A operand is 256 token
// rows (128 per CTA) and its B operand 256 weight rows, half of them loaded by each CTA. For the fused SwiGLU
// GEMM the leader loads 128 gate rows and the peer the matching 128 up rows, so ONE 256 x 256 x 16 MMA produces
// gate (accumulator columns 0..127) and up (128..255) of 128 features for 256 tokens: per CTA and K block
// that is 32 KB of operands for the FLOPs the weight-major form spends 40-48 KB (and two N = 128 MMAs, which
// are bound by their shared-memory reads) on, and the accumulator still fits a 256-column stage, so the epilogue
// runs under the next tile. TMEM lanes are token rows here: a thread owns one output row and stores 32-byte
// runs of it, no transpose. Plain GEMMs: the peer loads weight rows n0 + 128.., 256 features per tile.
template <bool DUAL, int EPI>
__device__ __forceinline__ void epilogue_rows(uint32_t tmem_acc, int quad, int lane, __nv_bfloat16* __restrict__ Y,
                                              const __nv_bfloat16* __restrict__ R, int M, int N, int ldy, int ldr,
                                              int token, int n0) {
  const uint32_t lane_addr = tmem_acc + (static_cast<uint32_t>(quad * 32) << 16);
  constexpr int kCols = DUAL ? 128 : 256;
  const bool row_ok = token < M;
  // The residual is fetched one 128-byte line (64 features) ahead. The output is usually written in place over
  // the residual, and a load that follows a store of the same thread to the same line waits for that store to
  // be acknowledged: with a look-ahead of one 16-feature chunk every chunk paid two round trips to L2 (139
  // against 61 us for a 2112 x 4096 x 4096 GEMM); a whole line ahead, loads and stores in flight never share one.
  uint4 nxt[8];
  auto fetch_line = [&](int l0) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      nxt[q] = make_uint4(0u, 0u, 0u, 0u);
      if (row_ok && l0 < kCols && n0 + l0 + 8 * q + 8 <= N)
        nxt[q] = __ldcg(reinterpret_cast<const uint4*>(R + static_cast<size_t>(token) * ldr + n0 + l0 + 8 * q));
    }
  };
  if (EPI == EPI_BF16_RESIDUAL) fetch_line(0);
  for (int l0 = 0; l0 < kCols; l0 += 64) {
    if (n0 + l0 >= N) break;   // warp-uniform
    uint4 cur[8];
    if (EPI == EPI_BF16_RESIDUAL) {
#pragma unroll
      for (int q = 0; q < 8; ++q) cur[q] = nxt[q];
      fetch_line(l0 + 64);
    }
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int c0 = l0 + cc * 16;
      if (n0 + c0 >= N) break;   // warp-uniform
      uint32_t g[16];
      tmem_ld_32x16(lane_addr + c0, g);
      float v[16];
      if (DUAL) {
        uint32_t u[16];
        tmem_ld_32x16(lane_addr + 128 + c0, u);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = silu_f(__uint_as_float(g[j])) * __uint_as_float(u[j]);
      } else {
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(g[j]);
      }
      uint4 o[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&o[h]);
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&cur[2 * cc + h]);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float x0 = v[h * 8 + 2 * q], x1 = v[h * 8 + 2 * q + 1];
          if (EPI == EPI_BF16_RESIDUAL) {
            const float2 fb = __bfloat1622float2(b[q]);
            // the weight-major kernels round the product to bf16 before the residual is added
            x0 = __bfloat162float(__float2bfloat16(x0)) + fb.x;
            x1 = __bfloat162float(__float2bfloat16(x1)) + fb.y;
          }
          a[q] = __floats2bfloat162_rn(x0, x1);
        }
      }
      if (row_ok) {
        __nv_bfloat16* y = Y + static_cast<size_t>(token) * ldy + n0 + c0;
        if (n0 + c0 + 8 <= N) *reinterpret_cast<uint4*>(y) = o[0];
        if (n0 + c0 + 16 <= N) *reinterpret_cast<uint4*>(y + 8) = o[1];
      }
    }
  }
}

template <bool DUAL, int EPI>
__global__ void __launch_bounds__(kGemmThreads)
gemm_pair_xw_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                    __nv_bfloat16* __restrict__ Y, const __nv_bfloat16* __restrict__ R, int M, int N, int K,
                    int ldy, int ldr, int dual_rows, int stages, int m_tiles, int total_tiles, int* err,
                    int packed_kb) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int kStage = 2 * kATileBytes;           // 128 token rows + 128 weight rows of one 64-wide K block
  constexpr int kTileN = DUAL ? kBM : 2 * kBM;      // output features per tile
  PairPersistTail* tail = reinterpret_cast<PairPersistTail*>(smem + stages * kStage);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const int cluster = blockIdx.x >> 1, clusters = gridDim.x >> 1;
  const int k_iters = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&tail->full[s], 1);
      mbar_init(&tail->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tail->tmem_full[a], 1);
      mbar_init(&tail->tmem_empty[a], 8);
    }
    tail->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc_pair(&tail->tmem_base, 2 * kAccStageCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything is sent to them
  tc_fence_after();
  const uint32_t tmem_base = tail->tmem_base;
  volatile int* abort_word = &tail->abort_word;
  pdl_wait();
  pdl_trigger();

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      for (int t = cluster; t < total_tiles && ok; t += clusters) {
        const int n0 = (t / m_tiles) * kTileN;
        const int w0 = DUAL ? (rank == 0 ? n0 : dual_rows + n0) : n0 + static_cast<int>(rank) * kBM;   // my weight rows
        const int tk0 = (t % m_tiles) * (2 * kBM) + static_cast<int>(rank) * kBM;                     // my token rows
        for (int it = 0; it < k_iters; ++it) {
          if (!mbar_wait(&tail->empty[s], ph ^ 1, abort_word, err, 120)) { ok = false; break; }
          uint8_t* sa = smem + s * kStage;
          if (rank == 0) mbar_arrive_expect_tx(&tail->full[s], 2 * kStage);
          const uint32_t full_leader = mapa_shared(&tail->full[s], 0);
          const int kc = it * kBK;
          if (++s == stages) { s = 0; ph ^= 1; }
          tma_load_2d_pair(sa, &tmX, full_leader, kc, tk0);
          if (packed_kb > 0)
            tma_load_2d_pair(sa + kATileBytes, &tmW, full_leader, 0, ((w0 >> 7) * packed_kb + it) << 7);
          else
            tma_load_2d_pair(sa + kATileBytes, &tmW, full_leader, kc, w0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = umma_idesc(2 * kBM, 2 * kBM, 1, 1);
      const uint64_t da0_first = umma_desc_sw128(smem);
      const uint64_t d_b = static_cast<uint64_t>(kATileBytes >> 4);
      const uint64_t d_stage = static_cast<uint64_t>(kStage >> 4);
      const uint32_t empty0 = mapa_shared(&tail->empty[0], 0), empty1 = mapa_shared(&tail->empty[0], 1);
      const uint32_t tfull0 = mapa_shared(&tail->tmem_full[0], 0), tfull1 = mapa_shared(&tail->tmem_full[0], 1);
      uint64_t da0 = da0_first;
      int s = 0;
      uint32_t ph = 0;
      bool ok = true;
      int i = 0;
      for (int t = cluster; t < total_tiles && ok; t += clusters, ++i) {
        const int a = i & 1;
        ok = mbar_wait(&tail->tmem_empty[a], ((i >> 1) & 1) ^ 1, abort_word, err, 121);
        if (!ok) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(a * kAccStageCols);
        for (int it = 0; it < k_iters; ++it) {
          ok = mbar_wait(&tail->full[s], ph, abort_word, err, 122);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
            const uint64_t koff = static_cast<uint64_t>(k * kUmmaK * 2 >> 4);
            umma_bf16_pair(d_tmem, da0 + koff, da0 + d_b + koff, idesc, acc);
          }
          tc_commit_pair(empty0 + 8u * s);
          tc_commit_pair(empty1 + 8u * s);
          if (++s == stages) { s = 0; ph ^= 1; da0 = da0_first; } else { da0 += d_stage; }
        }
        if (!ok) break;
        tc_commit_pair(tfull0 + 8u * a);
        tc_commit_pair(tfull1 + 8u * a);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quad = warp & 3;
    const uint32_t tempty_leader = mapa_shared(&tail->tmem_empty[0], 0);
    int i = 0;
    for (int t = cluster; t < total_tiles; t += clusters, ++i) {
      const int a = i & 1;
      if (!mbar_wait(&tail->tmem_full[a], (i >> 1) & 1, abort_word, err, 123)) break;
      tc_fence_after();
      const int n0 = (t / m_tiles) * kTileN;
      const int token = (t % m_tiles) * (2 * kBM) + static_cast<int>(rank) * kBM + quad * 32 + lane;
      if (k_iters > 0)
        epilogue_rows<DUAL, EPI>(tmem_base + static_cast<uint32_t>(a * kAccStageCols), quad, lane, Y, R, M, N, ldy,
                                 ldr, token, n0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader + 8u * a);
    }
  }

  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * kAccStageCols);
  }
}

// Sum split-K fp32 partials [splits, M, N] -> bf16 Y (+ optional residual).
__global__ void splitk_reduce_kernel(const float* __restrict__ part, const __nv_bfloat16* __restrict__ R,
                                     __nv_bfloat16* __restrict__ Y, int M, int N, int splits,
                                     int ldy, int ldr) {
  pdl_wait();
  pdl_trigger();
  const size_t idx = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  const size_t total = static_cast<size_t>(M) * N;
  if (idx >= total) return;
  const int t = static_cast<int>(idx / N);
  const int n = static_cast<int>(idx % N);
  float4 acc = *reinterpret_cast<const float4*>(part + idx);
  for (int s = 1; s < splits; ++s) {
    const float4 p = *reinterpret_cast<const float4*>(part + s * total + idx);
    acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
  }
  __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x, acc.y);
  __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z, acc.w);
  if (R != nullptr) {
    const uint2 rv = *reinterpret_cast<const uint2*>(R + static_cast<size_t>(t) * ldr + n);
    const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&rv);
    float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(rb[0]);
    lo = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
    a = __bfloat1622float2(hi); b = __bfloat1622float2(rb[1]);
    hi = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
  }
  uint2 out;
  out.x = *reinterpret_cast<uint32_t*>(&lo);
  out.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(Y + static_cast<size_t>(t) * ldy + n) = out;
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D row-major [rows, cols] tensor of `elt_bytes` elements; box = [box_rows, 128 bytes].
int make_tmap_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                 uint32_t box_rows, int elt_bytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return MB_ERR_DRIVER;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld * static_cast<uint64_t>(elt_bytes)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elt_bytes), box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt =
      elt_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? MB_OK : MB_ERR_TMAP;
}

struct TmapKey {
  const void* p;
  uint64_t rows, cols, ld;
  uint32_t box;
  bool operator==(const TmapKey& o) const {
    return p == o.p && rows == o.rows && cols == o.cols && ld == o.ld && box == o.box;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.p);
    h ^= k.rows * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.cols * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= (k.ld * 31 + k.box) + (h << 6) + (h >> 2);
    return h;
  }
};

// Descriptors are pure functions of (pointer, shape, box): cache them so the steady
// state of a serving loop encodes nothing on the host.
int cached_tmap(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                       uint64_t ld, uint32_t box_rows, int elt_bytes) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  TmapKey key{base, rows, cols, ld, box_rows * 4 + static_cast<uint32_t>(elt_bytes)};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return MB_OK;
  }
  int rc = make_tmap_2d(out, base, rows, cols, ld, box_rows, elt_bytes);
  if (rc == MB_OK) {
    if (cache.size() > 65536) cache.clear();
    cache.emplace(key, *out);
  }
  return rc;
}

// Unswizzled byte tiles: `box_bytes` bytes (a multiple of 16) of `box_rows` rows of a [rows, cols] byte matrix with
// row pitch `ld` bytes.
int cached_tmap_raw(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows,
                    uint32_t box_bytes) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  TmapKey key{base, rows, cols, ld, box_rows * 1024 + box_bytes};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return MB_OK;
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return MB_ERR_DRIVER;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {ld};
  const cuuint32_t box[2] = {box_bytes, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return MB_ERR_TMAP;
  if (cache.size() > 65536) cache.clear();
  cache.emplace(key, *out);
  return MB_OK;
}

static uint32_t pow2_cols(int c) {
  uint32_t p = 32;
  while (static_cast<int>(p) < c) p <<= 1;
  return p;
}

template <bool DUAL, int EPI>
static int launch_cfg(const CUtensorMap& tw, const CUtensorMap& tx, void* Y, const void* R, int M,
                      int N, int K, int ldy, int ldr, int dual_rows, int k_per_split, int splits,
                      int BN, int stages, int* err, cudaStream_t stream,
                      const int32_t* expert_offsets = nullptr, int n_experts = 0,
                      int w_rows_per_expert = 0, const int* gate_flags = nullptr, int gate_rpr = 1,
                      int gate_world = 0, int packed_kb = 0, int batch = 0, int x_batch_off = 0,
                      int y_batch_off = 0, int w_static = 0) {
  const int stage_bytes = kATileBytes * (DUAL ? 2 : 1) + BN * kBK * 2;
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + 4 * kStageWarpBytes +
                      sizeof(GemmSmemTail) + 1024;
  auto kern = gemm_wx_kernel<DUAL, EPI>;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) !=
        cudaSuccess)
      return MB_ERR_LAUNCH;
    configured.done();
  }
  dim3 grid((M + BN - 1) / BN, (N + kBM - 1) / kBM, expert_offsets ? n_experts : (batch > 0 ? batch : splits));
  const uint32_t tmem_cols = pow2_cols(DUAL ? 2 * BN : BN);
  const cudaError_t e = launch_k(kern, grid, dim3(kGemmThreads), smem, stream, tw, tx, Y,
                                 static_cast<const __nv_bfloat16*>(R), M, N, K, ldy, ldr, dual_rows, k_per_split,
                                 BN, stages, tmem_cols, err, expert_offsets, w_rows_per_expert, gate_flags,
                                 gate_rpr, gate_world, packed_kb, x_batch_off, y_batch_off, w_static);
  return e == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

template <bool DUAL, int EPI>
static int launch_pair_cfg(const CUtensorMap& tw, const CUtensorMap& tx, void* Y, const void* R, int M, int N,
                           int K, int ldy, int ldr, int dual_rows, int k_per_split, int splits, int BN,
                           int stages, int* err, cudaStream_t stream, const int* gate_flags, int gate_rpr,
                           int gate_world, int packed_kb) {
  const int stage_bytes = kATileBytes * (DUAL ? 2 : 1) + (BN / 2) * kBK * 2;
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + 4 * kStageWarpBytes +
                      sizeof(GemmSmemTail) + 1024;
  auto kern = gemm_pair_kernel<DUAL, EPI>;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return MB_ERR_LAUNCH;
    configured.done();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * ((M + BN - 1) / BN), (N + 2 * kBM - 1) / (2 * kBM), splits);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.numAttrs = 1;
  if (pdl_enabled()) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attr;
  const uint32_t tmem_cols = pow2_cols(DUAL ? 2 * BN : BN);
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, tx, Y, static_cast<const __nv_bfloat16*>(R), M, N, K,
                                           ldy, ldr, dual_rows, k_per_split, BN, stages, tmem_cols, err,
                                           gate_flags, gate_rpr, gate_world, packed_kb);
  return e == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

template <bool DUAL, int EPI>
static int launch_pair_persistent(const CUtensorMap& tw, const CUtensorMap& tx, void* Y, const void* R, int M, int N,
                                  int K, int ldy, int ldr, int dual_rows, int BN, int stages, int num_sms, int* err,
                                  cudaStream_t stream, int packed_kb) {
  const int stage_bytes = kATileBytes * (DUAL ? 2 : 1) + (BN / 2) * kBK * 2;
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + 4 * kStageWarpBytes +
                      sizeof(PairPersistTail) + 1024;
  auto kern = gemm_pair_persistent_kernel<DUAL, EPI>;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return MB_ERR_LAUNCH;
    configured.done();
  }
  const int m_tiles = (M + BN - 1) / BN;
  const int total = m_tiles * ((N + 2 * kBM - 1) / (2 * kBM));
  const int clusters = total < num_sms / 2 ? total : num_sms / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.numAttrs = 1;
  if (pdl_enabled()) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attr;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, tx, Y, static_cast<const __nv_bfloat16*>(R), M, N, K, ldy,
                                           ldr, dual_rows, BN, stages, m_tiles, total, err, packed_kb);
  return e == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

template <bool DUAL, int EPI>
static int launch_pair_xw(const CUtensorMap& tw, const CUtensorMap& tx, void* Y, const void* R, int M, int N, int K,
                          int ldy, int ldr, int dual_rows, int num_sms, int* err, cudaStream_t stream,
                          int packed_kb) {
  constexpr int kStage = 2 * kATileBytes;
  const int stages = 6;
  const size_t smem = static_cast<size_t>(stages) * kStage + sizeof(PairPersistTail) + 1024;
  auto kern = gemm_pair_xw_kernel<DUAL, EPI>;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return MB_ERR_LAUNCH;
    configured.done();
  }
  const int tile_n = DUAL ? kBM : 2 * kBM;
  const int m_tiles = (M + 2 * kBM - 1) / (2 * kBM);
  const int total = m_tiles * ((N + tile_n - 1) / tile_n);
  const int clusters = total < num_sms / 2 ? total : num_sms / 2;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * clusters);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.numAttrs = 1;
  if (pdl_enabled()) {
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.numAttrs = 2;
  }
  cfg.attrs = attr;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, tx, static_cast<__nv_bfloat16*>(Y),
                                           static_cast<const __nv_bfloat16*>(R), M, N, K, ldy, ldr, dual_rows, stages,
                                           m_tiles, total, err, packed_kb);
  return e == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

}  // namespace mb

using namespace mb;

// Tile-shape heuristic: the token tile is the smallest multiple of 16 that covers M in
// ceil(M/256) passes; split-K only when the grid would leave most SMs idle.
extern "C" void mb_gemm_bf16_plan(int M, int N, int K, int dual, int num_sms, int* bn_out,
                                  int* splits_out, int* stages_out) {
  const int max_bn = dual ? 128 : 256;
  const int n_tiles = (N + kBM - 1) / kBM;
  int m_tiles = (M + max_bn - 1) / max_bn;
  if (!dual && n_tiles * m_tiles > num_sms) {
    // More CTAs than SMs: every SM runs ceil(CTAs / SMs) tiles one after the other, and a tile of `b`
    // tokens costs about (128 + b) units (its bytes per K block). A narrower tile that needs no extra round
    // is cheaper: 1024 tokens x 48 weight tiles run as 6 x 176 (288 CTAs, two rounds) instead of 4 x 256
    // (192 CTAs, also two rounds).
    long best_cost = -1;
    int best = m_tiles;
    for (int c = m_tiles; c <= m_tiles + 2; ++c) {
      const int b = ((M + c - 1) / c + 15) / 16 * 16;
      const long rounds = (static_cast<long>(c) * n_tiles + num_sms - 1) / num_sms;
      const long cost = rounds * (128 + b);
      if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = c; }
    }
    m_tiles = best;
  }
  int bn = ((M + m_tiles - 1) / m_tiles + 15) / 16 * 16;
  if (bn < 16) bn = 16;
  int splits = 1;
  const int ctas = n_tiles * m_tiles;
  if (!dual && ctas * 2 <= num_sms) {
    splits = num_sms / ctas;
    const int k_blocks = (K + kBK - 1) / kBK;
    if (splits > k_blocks / 8) splits = k_blocks / 8 > 0 ? k_blocks / 8 : 1;
    if (splits > 8) splits = 8;
  }
  const int stage_bytes = kATileBytes * (dual ? 2 : 1) + bn * kBK * 2;
  const int tmem_need = dual ? 2 * bn : bn;
  // Two CTAs per SM when both the pipeline and the accumulators fit twice - but only when the grid
  // has more CTAs than SMs: a single-wave grid (the decode GEMMs) runs one CTA per SM, and then a
  // deeper pipeline (more bytes in flight per SM) is what brings the weight stream up to HBM speed.
  const bool one_wave = ctas * splits <= num_sms;
  int budget = (!one_wave && tmem_need <= 256 && stage_bytes * 4 + 12 * 1024 <= 112 * 1024) ? 100 * 1024
                                                                                           : 212 * 1024;
  int stages = budget / stage_bytes;
  if (stages > 8) stages = 8;
  if (stages < 2) stages = 2;
  *bn_out = bn;
  *splits_out = splits;
  *stages_out = stages;
}

// Y = X · W^T with optional fusions. flags: bit0 dual (SwiGLU over W = [gate; up]),
// bit1 residual add, bit2 fp32 output. `bn`/`splits`/`stages` <= 0 selects the plan above.
// Split-K needs `workspace` of splits*M*N floats.
extern "C" int mb_gemm_bf16(const void* X, const void* W, void* Y, const void* R, int M, int N,
                            int K, int ldx, int ldw, int ldy, int ldr, int flags, int bn,
                            int splits, int stages, void* workspace, int* err, int num_sms,
                            cudaStream_t stream) {
  return mb_gemm_bf16_gated(X, W, Y, R, M, N, K, ldx, ldw, ldy, ldr, flags, bn, splits, stages, workspace, err,
                            num_sms, nullptr, 1, 0, stream);
}

// Same GEMM whose token tiles wait for the tensor-parallel ready flags of the ranks that push the
// rows of X (`gate_flags` = this rank's flag array; nullptr = no gating).
extern "C" int mb_gemm_bf16_gated(const void* X, const void* W, void* Y, const void* R, int M, int N,
                                  int K, int ldx, int ldw, int ldy, int ldr, int flags, int bn,
                                  int splits, int stages, void* workspace, int* err, int num_sms,
                                  const int* gate_flags, int gate_rpr, int gate_world,
                                  cudaStream_t stream) {
  if (M <= 0 || N <= 0) return MB_OK;
  if (gate_flags != nullptr && (gate_rpr < 1 || gate_world < 1 || gate_world > kMaxRanks)) return MB_ERR_SHAPE;
  const bool dual = flags & 1, resid = flags & 2, f32 = flags & 4, packed = flags & 64;
  // bit6: W is pre-tiled as [rows/128][K/64][128][64] (mb_pack_weight_tiles layout)
  // bit7: W is written by no kernel on this stream (model weights): its first tiles may be requested before the
  //       programmatic-dependency wait
  const int w_static = (flags & 128) ? 1 : 0;
  if (packed && (K % kBK || N % kBM || ldw != K)) return MB_ERR_SHAPE;
  const int packed_kb = packed ? K / kBK : 0;
  if (K % 8 || ldx % 8 || ldw % 8 || N % 8 || (!f32 && ldy % 8) || (resid && ldr % 8))
    return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W) |
       reinterpret_cast<uintptr_t>(Y) | reinterpret_cast<uintptr_t>(R)) & 15)
    return MB_ERR_ALIGN;
  int pbn, psp, pst;
  mb_gemm_bf16_plan(M, N, K, dual, num_sms > 0 ? num_sms : 148, &pbn, &psp, &pst);
  if (bn <= 0) bn = pbn;
  if (splits <= 0) splits = psp;
  if (bn % 16 || bn > 256 || (dual && bn > 256)) return MB_ERR_SHAPE;
  if (dual && f32) return MB_ERR_SHAPE;
  if (splits > 1 && (workspace == nullptr || dual || f32)) splits = 1;
  {
    const int stage_bytes = kATileBytes * (dual ? 2 : 1) + bn * kBK * 2;
    const int max_stages = (227 * 1024 - 1024 - 4 * kStageWarpBytes - 512) / stage_bytes;
    if (stages <= 0) stages = pst;
    if (stages > max_stages) stages = max_stages;
    if (stages > 8) stages = 8;
    if (stages < 1) return MB_ERR_SHAPE;
  }
  const int w_rows = dual ? 2 * N : N;
  CUtensorMap tw, tx;
  int rc = packed ? cached_tmap(&tw, W, static_cast<uint64_t>(w_rows) * packed_kb, kBK, kBK, kBM, 2)
                  : cached_tmap(&tw, W, w_rows, K, ldw, kBM, 2);
  if (rc != MB_OK) return rc;
  rc = cached_tmap(&tx, X, M, K, ldx, bn, 2);
  if (rc != MB_OK) return rc;

  int k_per_split = K;
  if (splits > 1) {
    const int k_blocks = (K + kBK - 1) / kBK;
    k_per_split = ((k_blocks + splits - 1) / splits) * kBK;
    splits = (K + k_per_split - 1) / k_per_split;
  }
  if (splits > 1) {
    rc = launch_cfg<false, EPI_F32>(tw, tx, workspace, nullptr, M, N, K, N, 0, 0, k_per_split,
                                    splits, bn, stages, err, stream, nullptr, 0, 0, gate_flags, gate_rpr,
                                    gate_world, packed_kb, 0, 0, 0, w_static);
    if (rc != MB_OK) return rc;
    if (f32) return MB_ERR_SHAPE;  // fp32 output is never split
    const size_t total4 = (static_cast<size_t>(M) * N + 3) / 4;
    const cudaError_t e = launch_k(
        splitk_reduce_kernel, dim3(static_cast<unsigned>((total4 + 255) / 256)), dim3(256), 0, stream,
        static_cast<const float*>(workspace), resid ? static_cast<const __nv_bfloat16*>(R) : nullptr,
        static_cast<__nv_bfloat16*>(Y), M, N, splits, ldy, ldr);
    return e == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
  }
  if (dual)
    return launch_cfg<true, EPI_BF16>(tw, tx, Y, nullptr, M, N, K, ldy, 0, N, K, 1, bn, stages, err,
                                      stream, nullptr, 0, 0, gate_flags, gate_rpr, gate_world, packed_kb, 0, 0, 0, w_static);
  if (f32)
    return launch_cfg<false, EPI_F32>(tw, tx, Y, nullptr, M, N, K, ldy, 0, 0, K, 1, bn, stages, err,
                                      stream, nullptr, 0, 0, gate_flags, gate_rpr, gate_world, packed_kb, 0, 0, 0, w_static);
  if (resid)
    return launch_cfg<false, EPI_BF16_RESIDUAL>(tw, tx, Y, R, M, N, K, ldy, ldr, 0, K, 1, bn,
                                                stages, err, stream, nullptr, 0, 0, gate_flags, gate_rpr,
                                                gate_world, packed_kb, 0, 0, 0, w_static);
  return launch_cfg<false, EPI_BF16>(tw, tx, Y, nullptr, M, N, K, ldy, 0, 0, K, 1, bn, stages, err,
                                     stream, nullptr, 0, 0, gate_flags, gate_rpr, gate_world, packed_kb, 0, 0, 0, w_static);
}

// Process-wide choice of the CTA-pair kernel by token count: plain (and residual) GEMMs with
// M >= min_m_plain and fused SwiGLU GEMMs with M >= min_m_dual use it; 0 = never.
static int g_pair_min_m[2] = {0, 0};
static bool g_pair_persistent = true;
static int g_pair_token_major = 3;
// More tiles than pairs of SMs, and for plain GEMMs a last round that is not mostly idle (the weight-major
// kernel picks its token-tile width by rounds x tile cost; this one has fixed 256 x 256 tiles).
static bool pair_token_major_fits(int M, int N, bool dual, int num_sms) {
  const int tile_n = dual ? kBM : 2 * kBM;
  const int total = ((M + 2 * kBM - 1) / (2 * kBM)) * ((N + tile_n - 1) / tile_n);
  const int clusters = num_sms / 2;
  if (total <= clusters) return false;
  const int rounds = (total + clusters - 1) / clusters;
  return dual || 5 * total >= 4 * rounds * clusters;
}
// bit 0: fused SwiGLU GEMMs with more tiles than SM pairs run the token-major persistent pair kernel, bit 1: plain ones
extern "C" void mb_set_gemm_pair_token_major(int mask) { g_pair_token_major = mask; }
// 0: the CTA-pair GEMM launches one pair per tile even when there are more tiles than pairs of SMs
extern "C" void mb_set_gemm_pair_persistent(int on) { g_pair_persistent = on != 0; }
extern "C" void mb_set_gemm_pair(int min_m_plain, int min_m_dual) {
  g_pair_min_m[0] = min_m_plain;
  g_pair_min_m[1] = min_m_dual;
}
extern "C" int mb_gemm_pair_wanted(int M, int dual) {
  const int m = g_pair_min_m[dual ? 1 : 0];
  return m > 0 && M >= m;
}
// The same question with the problem's width known: fused SwiGLU GEMMs also take the pair path from the plain
// threshold up when the token-major persistent kernel would run them.
extern "C" int mb_gemm_pair_choice(int M, int N, int dual, int num_sms) {
  if (mb_gemm_pair_wanted(M, dual)) return 1;
  if (num_sms <= 0) num_sms = 148;
  return dual && g_pair_min_m[0] > 0 && M >= g_pair_min_m[0] && g_pair_persistent && (g_pair_token_major & 1) &&
         pair_token_major_fits(M, N, true, num_sms);
}

// Token-tile width and K splits the pair kernel picks by itself (no_split: fused SwiGLU or fp32 output).
// Callers use it to check that their workspace holds splits * M * N floats.
extern "C" void mb_gemm_bf16_pair_plan(int M, int N, int K, int no_split, int num_sms, int* bn_out,
                                       int* splits_out) {
  if (num_sms <= 0) num_sms = 148;
  int mt = (M + 255) / 256;
  const int pairs = (N + 2 * kBM - 1) / (2 * kBM);
  if (!no_split && 2 * pairs * mt > num_sms) {   // same rounds x tile-cost choice as the one-CTA plan
    long best_cost = -1;
    int best = mt;
    for (int c = mt; c <= mt + 2; ++c) {
      const int b = ((M + c - 1) / c + 31) / 32 * 32;
      const long rounds = (2L * c * pairs + num_sms - 1) / num_sms;
      const long cost = rounds * (128 + b / 2);
      if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = c; }
    }
    mt = best;
  }
  const int bn = ((M + mt - 1) / mt + 31) / 32 * 32;
  const int m_tiles = (M + bn - 1) / bn;
  const int k_blocks = (K + kBK - 1) / kBK;
  int splits = 1;
  const int ctas = 2 * m_tiles * pairs;
  if (!no_split && ctas * 2 <= num_sms) {
    splits = num_sms / ctas;
    if (splits > k_blocks / 8) splits = k_blocks / 8 > 0 ? k_blocks / 8 : 1;
    if (splits > 8) splits = 8;
  }
  *bn_out = bn;
  *splits_out = splits;
}

// CTA-pair (cta_group::2) GEMM: same contract and flags as mb_gemm_bf16_gated. The token tile is a
// multiple of 32 (each CTA of a pair loads half of it).
extern "C" int mb_gemm_bf16_pair(const void* X, const void* W, void* Y, const void* R, int M, int N, int K,
                                 int ldx, int ldw, int ldy, int ldr, int flags, int bn, int splits,
                                 int stages, void* workspace, int* err, int num_sms, const int* gate_flags,
                                 int gate_rpr, int gate_world, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return MB_OK;
  if (gate_flags != nullptr && (gate_rpr < 1 || gate_world < 1 || gate_world > kMaxRanks)) return MB_ERR_SHAPE;
  const bool dual = flags & 1, resid = flags & 2, f32 = flags & 4, packed = flags & 64;
  if (packed && (K % kBK || N % kBM || ldw != K)) return MB_ERR_SHAPE;
  const int packed_kb = packed ? K / kBK : 0;
  if (K % 8 || ldx % 8 || ldw % 8 || N % 8 || (!f32 && ldy % 8) || (resid && ldr % 8)) return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(Y) |
       reinterpret_cast<uintptr_t>(R)) & 15)
    return MB_ERR_ALIGN;
  if (dual && f32) return MB_ERR_SHAPE;
  if (num_sms <= 0) num_sms = 148;
  // token-major persistent pairs: bit 0 of the switch = fused SwiGLU GEMMs, bit 1 = plain ones
  if (g_pair_persistent && gate_flags == nullptr && !f32 && splits <= 1 &&
      (g_pair_token_major & (dual ? 1 : 2)) != 0) {
    if (pair_token_major_fits(M, N, dual, num_sms)) {
      const int w_rows_x = dual ? 2 * N : N;
      CUtensorMap twx, txx;
      int rcx = packed ? cached_tmap(&twx, W, static_cast<uint64_t>(w_rows_x) * packed_kb, kBK, kBK, kBM, 2)
                       : cached_tmap(&twx, W, w_rows_x, K, ldw, kBM, 2);
      if (rcx != MB_OK) return rcx;
      rcx = cached_tmap(&txx, X, M, K, ldx, kBM, 2);
      if (rcx != MB_OK) return rcx;
      if (dual)
        return launch_pair_xw<true, EPI_BF16>(twx, txx, Y, nullptr, M, N, K, ldy, 0, N, num_sms, err, stream, packed_kb);
      if (resid)
        return launch_pair_xw<false, EPI_BF16_RESIDUAL>(twx, txx, Y, R, M, N, K, ldy, ldr, 0, num_sms, err, stream,
                                                        packed_kb);
      return launch_pair_xw<false, EPI_BF16>(twx, txx, Y, nullptr, M, N, K, ldy, 0, 0, num_sms, err, stream, packed_kb);
    }
  }
  if (dual && bn <= 0 && g_pair_persistent && gate_flags == nullptr) {
    // fused SwiGLU with many tiles: the persistent form needs gate and up side by side in one 256-column
    // accumulator stage, i.e. token tiles of at most 128
    const int mt = (M + 127) / 128;
    const int b = ((M + mt - 1) / mt + 31) / 32 * 32;
    if (((M + b - 1) / b) * ((N + 2 * kBM - 1) / (2 * kBM)) > num_sms / 2) bn = b;
  }
  {
    int pbn, psp;
    mb_gemm_bf16_pair_plan(M, N, K, (dual || f32) ? 1 : 0, num_sms, &pbn, &psp);
    if (bn <= 0) bn = pbn;
    if (splits <= 0) splits = (bn == pbn) ? psp : 1;
  }
  if (bn % 32 || bn < 32 || bn > 256) return MB_ERR_SHAPE;
  const int k_blocks = (K + kBK - 1) / kBK;
  if (splits > 1 && (workspace == nullptr || dual || f32)) splits = 1;
  const int stage_bytes = kATileBytes * (dual ? 2 : 1) + (bn / 2) * kBK * 2;
  const int max_stages = (227 * 1024 - 1024 - 4 * kStageWarpBytes - 512) / stage_bytes;
  if (stages <= 0 || stages > max_stages) stages = max_stages;
  if (stages > 8) stages = 8;
  if (stages < 2) return MB_ERR_SHAPE;
  const int w_rows = dual ? 2 * N : N;
  CUtensorMap tw, tx;
  int rc = packed ? cached_tmap(&tw, W, static_cast<uint64_t>(w_rows) * packed_kb, kBK, kBK, kBM, 2)
                  : cached_tmap(&tw, W, w_rows, K, ldw, kBM, 2);
  if (rc != MB_OK) return rc;
  rc = cached_tmap(&tx, X, M, K, ldx, bn / 2, 2);
  if (rc != MB_OK) return rc;
  int k_per_split = K;
  if (splits > 1) {
    k_per_split = ((k_blocks + splits - 1) / splits) * kBK;
    splits = (K + k_per_split - 1) / k_per_split;
  }
  if (splits > 1) {
    rc = launch_pair_cfg<false, EPI_F32>(tw, tx, workspace, nullptr, M, N, K, N, 0, 0, k_per_split, splits, bn,
                                         stages, err, stream, gate_flags, gate_rpr, gate_world, packed_kb);
    if (rc != MB_OK) return rc;
    const size_t total4 = (static_cast<size_t>(M) * N + 3) / 4;
    const cudaError_t e = launch_k(
        splitk_reduce_kernel, dim3(static_cast<unsigned>((total4 + 255) / 256)), dim3(256), 0, stream,
        static_cast<const float*>(workspace), resid ? static_cast<const __nv_bfloat16*>(R) : nullptr,
        static_cast<__nv_bfloat16*>(Y), M, N, splits, ldy, ldr);
    return e == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
  }
  const bool many_tiles = ((M + bn - 1) / bn) * ((N + 2 * kBM - 1) / (2 * kBM)) > num_sms / 2;
  if (dual && g_pair_persistent && gate_flags == nullptr && many_tiles && bn <= 128)
    return launch_pair_persistent<true, EPI_BF16>(tw, tx, Y, nullptr, M, N, K, ldy, 0, N, bn, stages, num_sms, err,
                                                  stream, packed_kb);
  if (dual)
    return launch_pair_cfg<true, EPI_BF16>(tw, tx, Y, nullptr, M, N, K, ldy, 0, N, K, 1, bn, stages, err, stream,
                                           gate_flags, gate_rpr, gate_world, packed_kb);
  if (f32)
    return launch_pair_cfg<false, EPI_F32>(tw, tx, Y, nullptr, M, N, K, ldy, 0, 0, K, 1, bn, stages, err, stream,
                                           gate_flags, gate_rpr, gate_world, packed_kb);
  // more tiles than pairs of SMs: persistent pairs with two accumulator stages (epilogue under the next tile)
  if (g_pair_persistent && gate_flags == nullptr && many_tiles) {
    if (resid)
      return launch_pair_persistent<false, EPI_BF16_RESIDUAL>(tw, tx, Y, R, M, N, K, ldy, ldr, 0, bn, stages, num_sms,
                                                              err, stream, packed_kb);
    return launch_pair_persistent<false, EPI_BF16>(tw, tx, Y, nullptr, M, N, K, ldy, 0, 0, bn, stages, num_sms, err,
                                                   stream, packed_kb);
  }
  if (resid)
    return launch_pair_cfg<false, EPI_BF16_RESIDUAL>(tw, tx, Y, R, M, N, K, ldy, ldr, 0, K, 1, bn, stages, err,
                                                     stream, gate_flags, gate_rpr, gate_world, packed_kb);
  return launch_pair_cfg<false, EPI_BF16>(tw, tx, Y, nullptr, M, N, K, ldy, 0, 0, K, 1, bn, stages, err, stream,
                                          gate_flags, gate_rpr, gate_world, packed_kb);
}

// Grouped GEMM for mixture-of-experts layers: rows [offsets[e], offsets[e+1]) of X (tokens in
// expert order) are multiplied by expert e's weights W[e] ([N, K], or [2N, K] = [gate; up] with
// the SwiGLU epilogue when flags bit0 is set). `max_rows` bounds the rows any expert can have
// (the grid is sized for it; CTAs past an expert's rows exit at once).
// Reference: max/kernels/src/linalg/grouped_matmul_sm100.mojo (grouped_matmul_ragged).
// Batched product over the column blocks of one activation matrix (the per-head weight absorption of multi-head
// latent attention): Y[m, b * y_off + n] = sum_k X[m, b * x_off + k] * W[b, n, k] for b < B. X: [M, >= B * x_off]
// with row stride ldx, W: [B, N, K] contiguous, Y row stride ldy. No operand is transposed or copied: the head
// is a coordinate offset of the TMA loads and of the stores.
extern "C" int mb_batched_gemm_bf16(const void* X, const void* W, void* Y, int B, int M, int N, int K, int ldx,
                                    int x_off, int ldy, int y_off, int x_cols, int bn, int* err,
                                    cudaStream_t stream) {
  if (B <= 0 || M <= 0) return MB_OK;
  if (K % kBK || N % 8 || ldx % 8 || ldy % 8 || x_off % 8 || y_off % 8 || x_off <= 0 || y_off < N) return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(Y)) & 15)
    return MB_ERR_ALIGN;
  if (bn <= 0) {
    bn = M >= 256 ? 256 : (M + 15) / 16 * 16;
    if (bn < 16) bn = 16;
  }
  if (bn % 16 || bn > 256) return MB_ERR_SHAPE;
  const int stage_bytes = kATileBytes + bn * kBK * 2;
  int stages = (212 * 1024) / stage_bytes;
  if (stages > 8) stages = 8;
  CUtensorMap tw, tx;
  int rc = cached_tmap(&tw, W, static_cast<uint64_t>(N) * B, K, K, kBM, 2);
  if (rc != MB_OK) return rc;
  rc = cached_tmap(&tx, X, M, x_cols, ldx, bn, 2);
  if (rc != MB_OK) return rc;
  return launch_cfg<false, EPI_BF16>(tw, tx, Y, nullptr, M, N, K, ldy, 0, 0, K, 1, bn, stages, err, stream, nullptr, 0,
                                     N, nullptr, 1, 0, 0, B, x_off, y_off);
}

extern "C" int mb_grouped_gemm_bf16(const void* X, const void* W, void* Y, const int32_t* expert_offsets,
                                    int n_experts, int total_rows, int max_rows, int N, int K, int flags,
                                    int bn, int* err, cudaStream_t stream) {
  if (n_experts <= 0 || total_rows <= 0 || max_rows <= 0) return MB_OK;
  const bool dual = flags & 1;
  if (K % 8 || N % 8) return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(Y)) & 15)
    return MB_ERR_ALIGN;
  if (bn <= 0) {
    bn = max_rows >= 128 ? 128 : (max_rows + 15) / 16 * 16;
    if (bn < 16) bn = 16;
  }
  if (bn % 16 || bn > (dual ? 128 : 256)) return MB_ERR_SHAPE;
  const int w_rows = dual ? 2 * N : N;
  const int stage_bytes = kATileBytes * (dual ? 2 : 1) + bn * kBK * 2;
  int stages = (212 * 1024) / stage_bytes;
  if (stages > 8) stages = 8;
  CUtensorMap tw, tx;
  int rc = cached_tmap(&tw, W, static_cast<uint64_t>(w_rows) * n_experts, K, K, kBM, 2);
  if (rc != MB_OK) return rc;
  rc = cached_tmap(&tx, X, total_rows, K, K, bn, 2);
  if (rc != MB_OK) return rc;
  if (dual)
    return launch_cfg<true, EPI_BF16>(tw, tx, Y, nullptr, max_rows, N, K, N, 0, N, K, 1, bn, stages, err,
                                      stream, expert_offsets, n_experts, w_rows);
  return launch_cfg<false, EPI_BF16>(tw, tx, Y, nullptr, max_rows, N, K, N, 0, 0, K, 1, bn, stages, err,
                                     stream, expert_offsets, n_experts, w_rows);
}
