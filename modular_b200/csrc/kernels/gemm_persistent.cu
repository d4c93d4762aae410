// Persistent bf16 GEMM for sm_100a: one CTA per SM, stream-K work split, double-buffered
// TMEM accumulators.
//
//   Y[M, N] = X[M, K] · W[N, K]^T   (+ residual | SwiGLU over W = [gate; up] | fp32 out)
//
// Work is counted in units of one 64-wide K block of one 128(weight rows) x BN(tokens) tile.
//
//   mode 0 (round robin): CTA g owns whole tiles g, g+G, ... Concurrent CTAs then work on
//       neighbouring tiles and share weight/activation tiles in L2. Used when there are
//       many tiles per SM.
//   mode 1 (stream-K): the unit range [0, tiles*kb) is cut into G equal contiguous shares,
//       so every SM streams the same number of weight bytes no matter how the tile count
//       divides the SM count - this is what keeps decode-sized GEMMs (a few dozen tiles)
//       at HBM speed. A tile cut across CTAs is finished by whichever contributor arrives
//       last: every contributor writes its fp32 partial to a private workspace slot, bumps
//       a per-(tile, lane-quadrant) counter, and the last one sums the slots in CTA order
//       (deterministic) and runs the fused epilogue. Nobody waits on anybody.
//
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer (tcgen05.mma, fp32 accumulate in
// TMEM), warps 2-5 epilogue. Two accumulator buffers in TMEM let the epilogue of one
// segment overlap the main loop of the next. Every mbarrier wait is bounded.
//
// The workspace and the counter array belong to one stream at a time: launches that may
// overlap on the device need separate ones.
//
// Reference counterpart: max/kernels/src/linalg/matmul/gpu/sm100_structured/default/
// matmul_kernels.mojo:348 (persistent warp-specialised kernel with accumulator stages).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/ptx.cuh"
#include "gemm_common.h"

namespace mb {

namespace pg {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kUmmaK = 16;
constexpr int kATile = kBM * kBK * 2;
constexpr int kThreads = 192;
constexpr int kStgWarp = 16 * 32 * 2;  // bf16 [16 tokens][32 rows] per epilogue warp

enum Epi { EPI_BF16 = 0, EPI_RESID = 1, EPI_F32 = 2 };

struct Params {
  void* Y;
  const __nv_bfloat16* R;
  float* ws;
  int* counters;
  int* err;
  int M, N, K, ldy, ldr, dual_rows;
  int BN, stages, acc_cols;
  uint32_t tmem_cols;
  int m_tiles, tiles, kb, mode;
  long long units;
};

struct Tail {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_word;
};

struct Seg {
  int tile, kb0, kb1, idx;
};

// Enumerates this CTA's segments; identical in every warp role.
struct SegIter {
  int mode, G, g, tiles, kb, idx, next_tile;
  long long u, u1;
  __device__ SegIter(const Params& p, int g_, int G_)
      : mode(p.mode), G(G_), g(g_), tiles(p.tiles), kb(p.kb), idx(0), next_tile(g_) {
    u = p.units * g_ / G_;
    u1 = p.units * (g_ + 1) / G_;
  }
  __device__ bool next(Seg& s) {
    if (mode == 0) {
      if (next_tile >= tiles) return false;
      s.tile = next_tile; s.kb0 = 0; s.kb1 = kb; s.idx = idx++;
      next_tile += G;
      return true;
    }
    if (u >= u1) return false;
    const int tile = static_cast<int>(u / kb);
    const int kb0 = static_cast<int>(u - static_cast<long long>(tile) * kb);
    long long len = kb - kb0;
    if (len > u1 - u) len = u1 - u;
    s.tile = tile; s.kb0 = kb0; s.kb1 = kb0 + static_cast<int>(len); s.idx = idx++;
    u += len;
    return true;
  }
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// Final store of 16 tokens (c0..c0+15 of the tile) for weight row `n_row` held by this lane.
template <int EPI>
__device__ __forceinline__ void store_chunk(const float (&v)[16], const Params& p, int t0, int c0,
                                            int n_base, int lane, __nv_bfloat16* stg) {
  if (EPI == EPI_F32) {
    float* Y = reinterpret_cast<float*>(p.Y);
    const int n_row = n_base + lane;
    if (n_row < p.N) {
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int t = t0 + c0 + j;
        if (t < p.M) Y[static_cast<size_t>(t) * p.ldy + n_row] = v[j];
      }
    }
    return;
  }
  __nv_bfloat16* Y = reinterpret_cast<__nv_bfloat16*>(p.Y);
#pragma unroll
  for (int j = 0; j < 16; ++j) stg[j * 32 + lane] = __float2bfloat16(v[j]);
  __syncwarp();
#pragma unroll
  for (int pass = 0; pass < 2; ++pass) {
    const int j = pass * 8 + (lane >> 2);
    const int seg = lane & 3;
    const int t = t0 + c0 + j;
    const int n = n_base + seg * 8;
    if (t < p.M && n < p.N) {
      uint4 val = *reinterpret_cast<const uint4*>(stg + j * 32 + seg * 8);
      if (EPI == EPI_RESID) {
        const uint4 rv = *reinterpret_cast<const uint4*>(p.R + static_cast<size_t>(t) * p.ldr + n);
        __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&val);
        const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 fa = __bfloat1622float2(a[q]);
          const float2 fb = __bfloat1622float2(b[q]);
          a[q] = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
        }
      }
      *reinterpret_cast<uint4*>(Y + static_cast<size_t>(t) * p.ldy + n) = val;
    }
  }
  __syncwarp();
}

template <bool DUAL, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_persistent_kernel(const __grid_constant__ CUtensorMap tmW,
                       const __grid_constant__ CUtensorMap tmX, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int a_bytes = kATile * (DUAL ? 2 : 1);
  const int stage_bytes = a_bytes + p.BN * kBK * 2;
  uint8_t* stg_base = smem + p.stages * stage_bytes;
  Tail* tail = reinterpret_cast<Tail*>(stg_base + 4 * kStgWarp);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.x, G = gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&tail->full[s], 1);
      mbar_init(&tail->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tail->tmem_full[b], 1);
      mbar_init(&tail->tmem_empty[b], 4);
    }
    tail->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(&tail->tmem_base, p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tail->tmem_base;
  volatile int* abort_word = &tail->abort_word;
  // Everything above touched only this CTA's resources; wait here for the producing kernels
  // when launched with programmatic dependent launch (no-op otherwise).
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      SegIter it(p, g, G);
      Seg s;
      int n = 0;
      bool ok = true;
      while (ok && it.next(s)) {
        const int n0 = (s.tile / p.m_tiles) * kBM;
        const int t0 = (s.tile % p.m_tiles) * p.BN;
        for (int kbi = s.kb0; kbi < s.kb1; ++kbi, ++n) {
          const int st = n % p.stages;
          const uint32_t ph = (n / p.stages) & 1;
          if (!mbar_wait(&tail->empty[st], ph ^ 1, abort_word, p.err, 201)) { ok = false; break; }
          uint8_t* sa = smem + st * stage_bytes;
          mbar_arrive_expect_tx(&tail->full[st], stage_bytes);
          const int kc = kbi * kBK;
          tma_load_2d(sa, &tmW, &tail->full[st], kc, n0);
          if (DUAL) tma_load_2d(sa + kATile, &tmW, &tail->full[st], kc, p.dual_rows + n0);
          tma_load_2d(sa + a_bytes, &tmX, &tail->full[st], kc, t0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kBM, p.BN, 1, 1);
      SegIter it(p, g, G);
      Seg s;
      int n = 0;
      bool ok = true;
      while (ok && it.next(s)) {
        const int buf = s.idx & 1;
        const uint32_t bph = (s.idx >> 1) & 1;
        if (!mbar_wait(&tail->tmem_empty[buf], bph ^ 1, abort_word, p.err, 202)) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * p.acc_cols;
        for (int kbi = s.kb0; kbi < s.kb1; ++kbi, ++n) {
          const int st = n % p.stages;
          const uint32_t ph = (n / p.stages) & 1;
          if (!mbar_wait(&tail->full[st], ph, abort_word, p.err, 203)) { ok = false; break; }
          tc_fence_after();
          uint8_t* sa = smem + st * stage_bytes;
          const uint64_t da0 = umma_desc_sw128(sa);
          const uint64_t da1 = umma_desc_sw128(sa + kATile);
          const uint64_t db = umma_desc_sw128(sa + a_bytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint32_t accum = (kbi > s.kb0 || k > 0) ? 1u : 0u;
            const uint64_t koff = static_cast<uint64_t>(k * kUmmaK * 2 >> 4);
            umma_bf16(acc, da0 + koff, db + koff, idesc, accum);
            if (DUAL) umma_bf16(acc + p.BN, da1 + koff, db + koff, idesc, accum);
          }
          tc_commit(&tail->empty[st]);
        }
        if (ok) tc_commit(&tail->tmem_full[buf]);
      }
      // main loops issued: let a dependent kernel start its prologue
      asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
  } else {
    const int quad = warp & 3;
    __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(stg_base + quad * kStgWarp);
    const size_t slot_floats = static_cast<size_t>(p.acc_cols) * kBM;
    SegIter it(p, g, G);
    Seg s;
    while (it.next(s)) {
      const int buf = s.idx & 1;
      const uint32_t bph = (s.idx >> 1) & 1;
      if (!mbar_wait(&tail->tmem_full[buf], bph, abort_word, p.err, 204)) break;
      tc_fence_after();
      const int n0 = (s.tile / p.m_tiles) * kBM;
      const int t0 = (s.tile % p.m_tiles) * p.BN;
      const int n_base = n0 + quad * 32;
      const uint32_t acc = tmem_base + buf * p.acc_cols + (static_cast<uint32_t>(quad * 32) << 16);
      const bool full_tile = s.kb0 == 0 && s.kb1 == p.kb;
      if (full_tile) {
        for (int c0 = 0; c0 < p.BN; c0 += 16) {
          if (t0 + c0 >= p.M) break;
          uint32_t a[16];
          float v[16];
          tmem_ld_32x16(acc + c0, a);
          if (DUAL) {
            uint32_t b[16];
            tmem_ld_32x16(acc + p.BN + c0, b);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = silu_f(__uint_as_float(a[j])) * __uint_as_float(b[j]);
          } else {
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(a[j]);
          }
          store_chunk<EPI>(v, p, t0, c0, n_base, lane, stg);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tail->tmem_empty[buf]);
        continue;
      }
      // ---- partial tile: publish, then maybe reduce
      const int row = quad * 32 + lane;
      float* mine = p.ws + (static_cast<size_t>(g) * 2 + (s.idx == 0 ? 0 : 1)) * slot_floats;
      for (int c0 = 0; c0 < p.BN; c0 += 16) {
        if (t0 + c0 >= p.M) break;
        uint32_t a[16];
        tmem_ld_32x16(acc + c0, a);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) mine[static_cast<size_t>(c0 + j) * kBM + row] = __uint_as_float(a[j]);
        if (DUAL) {
          tmem_ld_32x16(acc + p.BN + c0, a);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            mine[static_cast<size_t>(p.BN + c0 + j) * kBM + row] = __uint_as_float(a[j]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tail->tmem_empty[buf]);
      const long long first_unit = static_cast<long long>(s.tile) * p.kb;
      const int g_first = static_cast<int>(((first_unit + 1) * G - 1) / p.units);
      const int g_last = static_cast<int>(((first_unit + p.kb) * G - 1) / p.units);
      __threadfence();
      __syncwarp();
      int old = 0;
      if (lane == 0) old = atomicAdd(&p.counters[s.tile * 4 + quad], 1);
      old = __shfl_sync(0xffffffffu, old, 0);
      if (old != g_last - g_first) continue;  // someone else finishes this tile
      __threadfence();
      for (int c0 = 0; c0 < p.BN; c0 += 16) {
        if (t0 + c0 >= p.M) break;
        float v[16], w[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) { v[j] = 0.f; w[j] = 0.f; }
        for (int gc = g_first; gc <= g_last; ++gc) {
          const long long b0 = p.units * gc / G;
          const float* src = p.ws + (static_cast<size_t>(gc) * 2 + (b0 >= first_unit ? 0 : 1)) * slot_floats;
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] += __ldcg(src + static_cast<size_t>(c0 + j) * kBM + row);
          if (DUAL) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              w[j] += __ldcg(src + static_cast<size_t>(p.BN + c0 + j) * kBM + row);
          }
        }
        if (DUAL) {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = silu_f(v[j]) * w[j];
        }
        store_chunk<EPI>(v, p, t0, c0, n_base, lane, stg);
      }
      if (lane == 0) p.counters[s.tile * 4 + quad] = 0;  // ready for the next launch
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

static uint32_t pow2_cols(int c) {
  uint32_t v = 32;
  while (static_cast<int>(v) < c) v <<= 1;
  return v;
}

template <bool DUAL, int EPI>
static int launch(const CUtensorMap& tw, const CUtensorMap& tx, const Params& p, int grid,
                  bool pdl, cudaStream_t stream) {
  const int stage_bytes = kATile * (DUAL ? 2 : 1) + p.BN * kBK * 2;
  const size_t smem = static_cast<size_t>(p.stages) * stage_bytes + 4 * kStgWarp + sizeof(Tail) + 1024;
  auto kern = gemm_persistent_kernel<DUAL, EPI>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return MB_ERR_LAUNCH;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, tw, tx, p) == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

}  // namespace pg
}  // namespace mb

using namespace mb;

// Workspace requirement of the persistent kernel: 2 slots per CTA of acc_cols*128 floats,
// plus 4 counters per tile. Both are bounded by these constants for every supported shape.
extern "C" size_t mb_gemm_persistent_workspace_bytes(int num_sms) {
  return static_cast<size_t>(num_sms) * 2 * 256 * 128 * sizeof(float);
}
extern "C" size_t mb_gemm_persistent_counter_ints(int num_sms) { return static_cast<size_t>(num_sms) * 4 * 4 * 4; }

// flags: bit0 dual (SwiGLU), bit1 residual add, bit2 fp32 output, bit3 programmatic dependent launch.
// `bn` <= 0 selects the tile width automatically. `ws` must hold
// mb_gemm_persistent_workspace_bytes(), `counters` mb_gemm_persistent_counter_ints() zeroed ints.
extern "C" int mb_gemm_bf16_persistent(const void* X, const void* W, void* Y, const void* R, int M,
                                       int N, int K, int ldx, int ldw, int ldy, int ldr, int flags,
                                       int bn, int stages, int force_mode, void* ws, int* counters,
                                       int* err, int num_sms, cudaStream_t stream) {
  using namespace mb::pg;
  if (M <= 0 || N <= 0) return MB_OK;
  const bool dual = flags & 1, resid = flags & 2, f32 = flags & 4, pdl = flags & 8;
  if (K % 8 || ldx % 8 || ldw % 8 || N % 8 || (!f32 && ldy % 8) || (resid && ldr % 8)) return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(Y) |
       reinterpret_cast<uintptr_t>(R)) & 15)
    return MB_ERR_ALIGN;
  if (dual && f32) return MB_ERR_SHAPE;
  if (num_sms <= 0) num_sms = 148;
  const int max_bn = dual ? 128 : 256;
  if (bn <= 0) {
    const int mt = (M + max_bn - 1) / max_bn;
    bn = ((M + mt - 1) / mt + 15) / 16 * 16;
  }
  if (bn % 16 || bn < 16 || bn > max_bn) return MB_ERR_SHAPE;
  Params p;
  p.Y = Y; p.R = static_cast<const __nv_bfloat16*>(R);
  p.ws = static_cast<float*>(ws); p.counters = counters; p.err = err;
  p.M = M; p.N = N; p.K = K; p.ldy = ldy; p.ldr = ldr; p.dual_rows = N;
  p.BN = bn;
  p.acc_cols = bn * (dual ? 2 : 1);
  p.tmem_cols = pow2_cols(2 * p.acc_cols);
  if (p.tmem_cols > 512) return MB_ERR_SHAPE;
  const int stage_bytes = kATile * (dual ? 2 : 1) + bn * kBK * 2;
  const int max_stages = (227 * 1024 - 1024 - 4 * kStgWarp - 512) / stage_bytes;
  if (stages <= 0 || stages > max_stages) stages = max_stages;
  if (stages > 8) stages = 8;
  if (stages < 2) return MB_ERR_SHAPE;
  p.stages = stages;
  p.m_tiles = (M + bn - 1) / bn;
  const int n_tiles = (N + kBM - 1) / kBM;
  p.tiles = p.m_tiles * n_tiles;
  p.kb = (K + kBK - 1) / kBK;
  p.units = static_cast<long long>(p.tiles) * p.kb;
  int mode = p.tiles >= 4 * num_sms ? 0 : 1;
  if (force_mode == 0 || force_mode == 1) mode = force_mode;
  if (mode == 1 && (ws == nullptr || counters == nullptr || p.tiles * 4 > static_cast<int>(mb_gemm_persistent_counter_ints(num_sms))))
    mode = 0;
  p.mode = mode;
  int grid;
  if (mode == 0) {
    grid = p.tiles < num_sms ? p.tiles : num_sms;
  } else {
    long long g = p.units / 4;  // at least four K blocks per CTA
    if (g < 1) g = 1;
    grid = g < num_sms ? static_cast<int>(g) : num_sms;
  }
  CUtensorMap tw, tx;
  int rc = cached_tmap(&tw, W, dual ? 2 * N : N, K, ldw, kBM, 2);
  if (rc != MB_OK) return rc;
  rc = cached_tmap(&tx, X, M, K, ldx, bn, 2);
  if (rc != MB_OK) return rc;
  if (dual) return launch<true, EPI_BF16>(tw, tx, p, grid, pdl, stream);
  if (f32) return launch<false, EPI_F32>(tw, tx, p, grid, pdl, stream);
  if (resid) return launch<false, EPI_RESID>(tw, tx, p, grid, pdl, stream);
  return launch<false, EPI_BF16>(tw, tx, p, grid, pdl, stream);
}
