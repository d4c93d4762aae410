// Decode-step GEMM for sm_100a: Y[M, N] = X[M, K] · W[N, K]^T for small M (one decode batch,
// M <= 256 tokens), with the whole tail of the half layer fused behind it.
//
// A decode GEMM streams its weights once and does almost no math, so what decides its time is
// (a) whether all 148 SMs stream the same number of bytes and (b) how many launches, barriers and
// re-reads follow it. This kernel therefore
//
//   * cuts the K-block range of all weight tiles into equal contiguous shares, one per CTA
//     (stream-K over every tile, one CTA per SM): every SM streams the same bytes no matter how
//     the tile count divides the SM count;
//   * writes each share's fp32 partial tile to an L2-resident workspace and meets the other CTAs
//     at one grid-wide arrival counter (all CTAs are resident by construction);
//   * then runs the epilogue with ALL threads of ALL CTAs over the output, not per tile:
//       mode 0  bf16 store
//       mode 1  SwiGLU: W = [gate; up] rows, out[t, i] = silu(acc[t, i]) * acc[t, inter + i]
//       mode 2  all-reduce over the tensor-parallel ranks + residual add + RMSNorm: the CTA that
//               owns a token row sums the local partials, pushes the bf16 row into every peer's
//               receive buffer with plain 16-byte peer stores, polls its own receive buffer until
//               no sentinel value is left (no flags, no barrier: the data is its own arrival
//               signal, Lamport style, three buffer generations), adds the residual, writes the new
//               residual row and the normalised row. Every rank ends up with the full residual
//               stream and the full normalised activations, bit-identical (fixed summation order),
//               so the next column-parallel GEMM needs no gather and no flags. With one rank the
//               push and poll vanish and the same code is GEMM + residual + RMSNorm.
//   * starts streaming weights before the previous kernel has finished: launched as a programmatic
//     dependent, the producer fills its pipeline with weight tiles (which no kernel writes) ahead
//     of `griddepcontrol.wait`, and the activation tiles follow after it.
//
// Warp roles in the main loop: warp 0 TMA producer, warp 1 MMA issuer (tcgen05.mma, fp32
// accumulators in TMEM, two buffers), warps 2-5 drain accumulators into the workspace.
// Every wait (mbarrier, arrival counter, sentinel poll) is bounded and reports through `err`.
//
// Reference counterparts: max/kernels/src/comm/allreduce.mojo:1051 (_allreduce_lamport_kernel),
// comm/allreduce_lamport_rmsnorm.mojo:62, comm/lamport.mojo (sentinel protocol, 3 generations),
// linalg/matmul/gpu/sm100_structured/default/matmul_kernels.mojo:348 (the GEMM it follows),
// nn/gemv_partial_norm.mojo:131 (GEMV fused with norm statistics).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "comm_flags.h"
#include "gemm_common.h"

namespace mb {
namespace dec {

constexpr int kBM = 128;       // weight rows per tile (UMMA M)
constexpr int kBK = 64;        // bf16 per 128-byte swizzle row
constexpr int kUmmaK = 16;
constexpr int kATile = kBM * kBK * 2;
constexpr int kThreads = 512;     // warps 0-5 run the main loop, all sixteen run the epilogue
constexpr int kSlots = 6;      // most workspace slots per CTA (segments of different tiles)
constexpr int kRawTile = 128 * 64;   // fp8 weight tile of one K block: 128 rows x 64 bytes, unswizzled
constexpr int kConvWarps = 10;       // warps 6..15 convert fp8 weight tiles: two per ring stage (at most 5 stages)
constexpr uint32_t kSentinel2 = 0x80008000u;   // two bf16 -0.0

struct Params {
  int M, N, K, BN, stages, nbufs;
  uint32_t tmem_cols;
  int m_tiles, tiles, kb, G;
  uint32_t units;          // tiles * kb
  int slot_floats;         // BN * 128
  int slots;               // workspace slots per CTA = most tiles one share can touch
  float* ws;               // [G][slots][BN][128]
  int* state;              // kDecState* words
  int* err;
  int mode;
  __nv_bfloat16* Y;        // mode 0/1 output
  int ldy;
  // batched mode 0 (bN > 0): W stacks B matrices of bN rows; rows [b bN, (b + 1) bN) multiply the K columns of X
  // that start at b * x_boff and produce the bN columns of Y that start at b * y_boff
  int bN, x_boff, y_boff;
  int inter;               // mode 1: gate rows [0, inter), up rows [inter, 2 inter)
  // modes 0 / 1 without the grid-wide meeting point: the CTA whose partial completes an output tile (mode 1: a
  // gate tile and its up tile) reduces and stores that tile; the other CTAs leave as soon as their partials are
  // written
  int tile_epi;
  // Block-scaled fp8 weights (e4m3, one fp32 scale per 128 x 128 block) with bf16 activations: the weight tile of a
  // K block arrives as 128 rows x 64 bytes, eight converter warps write it as scaled bf16 into the operand layout,
  // the accumulation then runs in bf16 x bf16 as for bf16 weights. w_scale = nullptr: bf16 weights.
  const float* w_scale;    // [N / 128, sw_ld]
  int sw_ld;
  // Other weight-only formats through the same converter warps (wfmt): 2 = NVFP4 (two e2m1 values per byte, one
  // e4m3 scale per 16 values along K in w_bscale, one fp32 scale per tensor at *w_gscale), 3 = MXFP8 (e4m3 values,
  // one power-of-two ue8m0 scale per 32 values in w_bscale). 0 = bf16 weights, 1 = e4m3 with 128 x 128 fp32 scales.
  int wfmt;
  const uint8_t* w_bscale;  // [N, bs_ld] bytes
  int bs_ld;
  const float* w_gscale;
  // QKV projection with the rotation and the cache store in the tile epilogue (head_dim 128: an output tile is
  // one head; rotate-half convention). rope = 1: tiles [0, n_q) are query heads (rotated, stored to Y), the next
  // n_kv key heads (rotated, stored to Y and to the K cache at the token's slot), the last n_kv value heads
  // (stored to Y and to the V cache). Values are rounded to bf16 before the rotation, like the stand-alone kernel.
  int rope, n_q, n_kv, page_size;
  long long page_stride, head_stride;
  const int32_t* positions;
  const int64_t* kv_slots; // cache slot of every token row (-1: none)
  const float* cos_sin;    // [max_pos, 128]: 64 cos then 64 sin
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  __nv_bfloat16* h;        // mode 2: residual stream [M, N], updated in place
  __nv_bfloat16* xn;       // mode 2: normalised rows [M, N]
  const __nv_bfloat16* gamma;
  float eps, w_off;
  int mbc;
  int world, rank, lam_rows;
  __nv_bfloat16* lam[kMaxRanks];   // receive buffers of every rank: [3][world][lam_rows][N]
  unsigned long long* trace;       // optional [G][8] globaltimer stamps of the phases (measurement aid), or nullptr
};

struct Tail {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t raw_full[8];    // fp8 weights: the raw tile (and the activation tile) of the stage has landed
  uint32_t tmem_base;
  int abort_word;
  int flag;
  int tile_last;
  float red[kThreads / 32];
};

struct Seg {
  int tile, kb0, kb1, idx;
};

// first K-block unit of CTA g: the partition every role and the reduction agree on
__device__ __forceinline__ uint32_t share_begin(const Params& p, int g) {
  return p.units * static_cast<uint32_t>(g) / static_cast<uint32_t>(p.G);   // units * G < 2^31 (checked by the host)
}

struct SegIter {
  uint32_t u, u1;
  int kb, idx;
  __device__ SegIter(const Params& p, int g) : kb(p.kb), idx(0) {
    u = share_begin(p, g);
    u1 = share_begin(p, g + 1);
  }
  __device__ bool next(Seg& s) {
    if (u >= u1) return false;
    const int tile = static_cast<int>(u / static_cast<uint32_t>(kb));
    const int kb0 = static_cast<int>(u - static_cast<uint32_t>(tile) * kb);
    int len = kb - kb0;
    if (static_cast<uint32_t>(len) > u1 - u) len = static_cast<int>(u1 - u);
    s.tile = tile; s.kb0 = kb0; s.kb1 = kb0 + len; s.idx = idx++;
    u += len;
    return true;
  }
};

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ bool has_sentinel(uint32_t w) {
  return (w & 0xffffu) == 0x8000u || (w >> 16) == 0x8000u;
}
__device__ __forceinline__ uint32_t sanitize2(uint32_t w) {
  // a real -0.0 must not look like "not arrived yet": store it as +0.0
  if ((w & 0xffffu) == 0x8000u) w &= 0xffff0000u;
  if ((w >> 16) == 0x8000u) w &= 0x0000ffffu;
  return w;
}

// Sum of the fp32 partials of output elements (token t, weight rows n..n+7) over the CTAs that share
// the tile, in CTA order (deterministic).
__device__ __forceinline__ void reduce8(const Params& p, int t, int n, float (&acc)[8]) {
  const int n_tile = n >> 7;
  const int m_tile = t / p.BN;
  const int tile = n_tile * p.m_tiles + m_tile;
  const uint32_t fu = static_cast<uint32_t>(tile) * p.kb;
  const int g_first = static_cast<int>(((fu + 1u) * static_cast<uint32_t>(p.G) - 1u) / p.units);
  const int g_last = static_cast<int>(((fu + static_cast<uint32_t>(p.kb)) * static_cast<uint32_t>(p.G) - 1u) / p.units);
  const size_t off = static_cast<size_t>(t - m_tile * p.BN) * kBM + (n & 127);
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  // four contributors per round: all their loads are issued before the first add
  for (int gc0 = g_first; gc0 <= g_last; gc0 += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      a[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      b[j] = a[j];
      const int gc = gc0 + j;
      if (gc <= g_last) {
        const int tau0 = static_cast<int>(share_begin(p, gc) / static_cast<uint32_t>(p.kb));
        const float* src = p.ws + (static_cast<size_t>(gc) * p.slots + (tile - tau0)) * p.slot_floats + off;
        a[j] = __ldcg(reinterpret_cast<const float4*>(src));
        b[j] = __ldcg(reinterpret_cast<const float4*>(src + 4));
      }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[0] += a[j].x; acc[1] += a[j].y; acc[2] += a[j].z; acc[3] += a[j].w;
      acc[4] += b[j].x; acc[5] += b[j].y; acc[6] += b[j].z; acc[7] += b[j].w;
    }
  }
}

// CTAs whose shares touch `tile`
__device__ __forceinline__ int tile_contributors(const Params& p, int tile) {
  const uint32_t fu = static_cast<uint32_t>(tile) * p.kb;
  const int g_first = static_cast<int>(((fu + 1u) * static_cast<uint32_t>(p.G) - 1u) / p.units);
  const int g_last = static_cast<int>(((fu + static_cast<uint32_t>(p.kb)) * static_cast<uint32_t>(p.G) - 1u) / p.units);
  return g_last - g_first + 1;
}

__device__ __forceinline__ uint4 pack_bf16x8(const float (&v)[8]) {
  uint4 o;
  __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) q[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  return o;
}
__device__ __forceinline__ void unpack_add(const uint4& v, float (&acc)[8]) {
  const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(q[i]);
    acc[2 * i] += f.x; acc[2 * i + 1] += f.y;
  }
}

// One work item of the QKV epilogue with rotation: token t, head `head`, dims [d, d + 8) and their partners 64
// further on (rotate-half). Query heads go to Y, key heads to Y and the K cache.
__device__ __forceinline__ void qkv_rotate_item(const Params& p, int t, int head, int d) {
  const int n0 = head << 7;
  float lo[8], hi[8];
  reduce8(p, t, n0 + d, lo);
  reduce8(p, t, n0 + 64 + d, hi);
  const float* cs = p.cos_sin + static_cast<size_t>(p.positions[t]) * 128;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float a = __bfloat162float(__float2bfloat16_rn(lo[i])), b = __bfloat162float(__float2bfloat16_rn(hi[i]));
    const float cc = cs[d + i], sn = cs[64 + d + i];
    lo[i] = a * cc - b * sn;
    hi[i] = b * cc + a * sn;
  }
  const uint4 vlo = pack_bf16x8(lo), vhi = pack_bf16x8(hi);
  __nv_bfloat16* y = p.Y + static_cast<size_t>(t) * p.ldy + n0;
  *reinterpret_cast<uint4*>(y + d) = vlo;
  *reinterpret_cast<uint4*>(y + 64 + d) = vhi;
  if (head >= p.n_q) {
    const int64_t slot = p.kv_slots[t];
    if (slot >= 0) {
      __nv_bfloat16* kc = p.k_cache + (slot / p.page_size) * p.page_stride + (head - p.n_q) * p.head_stride +
                          (slot % p.page_size) * 128;
      *reinterpret_cast<uint4*>(kc + d) = vlo;
      *reinterpret_cast<uint4*>(kc + 64 + d) = vhi;
    }
  }
}

// Value heads: token t, head `head` (>= n_q + n_kv), dims [d, d + 8): to Y and to the V cache.
__device__ __forceinline__ void qkv_value_item(const Params& p, int t, int head, int d) {
  const int n0 = head << 7;
  float v[8];
  reduce8(p, t, n0 + d, v);
  const uint4 o = pack_bf16x8(v);
  *reinterpret_cast<uint4*>(p.Y + static_cast<size_t>(t) * p.ldy + n0 + d) = o;
  const int64_t slot = p.kv_slots[t];
  if (slot >= 0)
    *reinterpret_cast<uint4*>(p.v_cache + (slot / p.page_size) * p.page_stride + (head - p.n_q - p.n_kv) * p.head_stride +
                              (slot % p.page_size) * 128 + d) = o;
}

__global__ void __launch_bounds__(kThreads)
gemm_dec_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int b_bytes = p.BN * kBK * 2;
  const bool w8 = p.wfmt != 0;
  const int raw_row = p.wfmt == 2 ? 32 : 64;            // raw bytes of one weight row of a K block
  const int raw_bytes = 128 * raw_row;
  const int stage_bytes = kATile + b_bytes + (w8 ? kRawTile : 0);
  Tail* tail = reinterpret_cast<Tail*>(smem + p.stages * stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.x;
#define MB_DEC_STAMP(i) do { if (p.trace != nullptr && threadIdx.x == 0) p.trace[g * 8 + (i)] = globaltimer_ns(); } while (0)
  MB_DEC_STAMP(0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&tail->full[s], w8 ? 2 : 1);   // the TMA transaction count, or the two converter warps of the stage
      mbar_init(&tail->empty[s], 1);
      mbar_init(&tail->raw_full[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tail->tmem_full[b], 1);
      mbar_init(&tail->tmem_empty[b], 4);
    }
    tail->abort_word = 0;
    tail->flag = 0;
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

  // ------------------------------------------------------------------ main loop (phase A)
  if (warp == 0) {
    if (lane == 0) {
      // weights are written by no kernel: fill the ring with weight tiles before waiting for the
      // kernels this one depends on; their activation tiles follow after the wait
      int pre = 0;
      {
        SegIter it(p, g);
        Seg s;
        int st = 0;
        while (pre < p.stages && it.next(s)) {
          const int n0 = (s.tile / p.m_tiles) * kBM;
          for (int kbi = s.kb0; kbi < s.kb1 && pre < p.stages; ++kbi) {
            if (w8) {
              // fp8 weights: the raw tile goes behind the operand tiles of the stage and signals the converters
              mbar_arrive_expect_tx(&tail->raw_full[st], raw_bytes + b_bytes);
              tma_load_2d(smem + st * stage_bytes + kATile + b_bytes, &tmW, &tail->raw_full[st], kbi * raw_row, n0);
            } else {
              mbar_arrive_expect_tx(&tail->full[st], stage_bytes);
              tma_load_2d(smem + st * stage_bytes, &tmW, &tail->full[st], kbi * kBK, n0);
            }
            ++st; ++pre;
          }
        }
      }
      MB_DEC_STAMP(1);
      pdl_wait();
      pdl_trigger();
      MB_DEC_STAMP(2);
      SegIter it(p, g);
      Seg s;
      int st = 0, issued = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok && it.next(s)) {
        const int n0 = (s.tile / p.m_tiles) * kBM;
        const int t0 = (s.tile % p.m_tiles) * p.BN;
        for (int kbi = s.kb0; kbi < s.kb1; ++kbi) {
          uint8_t* sa = smem + st * stage_bytes;
          uint64_t* full_st = w8 ? &tail->raw_full[st] : &tail->full[st];
          if (issued >= pre) {
            if (!mbar_wait(&tail->empty[st], ph ^ 1, abort_word, p.err, 301)) { ok = false; break; }
            if (w8) {
              mbar_arrive_expect_tx(full_st, raw_bytes + b_bytes);
              tma_load_2d(sa + kATile + b_bytes, &tmW, full_st, kbi * raw_row, n0);
            } else {
              mbar_arrive_expect_tx(full_st, stage_bytes);
              tma_load_2d(sa, &tmW, full_st, kbi * kBK, n0);
            }
          }
          tma_load_2d(sa + kATile, &tmX, full_st, (p.bN > 0 ? (n0 / p.bN) * p.x_boff : 0) + kbi * kBK, t0);
          ++issued;
          if (++st == p.stages) { st = 0; ph ^= 1; }
        }
      }
    } else {
      pdl_wait();
      pdl_trigger();
    }
  } else if (warp == 1) {
    pdl_wait();
    pdl_trigger();
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kBM, p.BN, 1, 1);
      SegIter it(p, g);
      Seg s;
      const uint64_t da0_first = umma_desc_sw128(smem);
      const uint64_t d_b = static_cast<uint64_t>(kATile >> 4);
      const uint64_t d_stage = static_cast<uint64_t>(stage_bytes >> 4);
      uint64_t da0 = da0_first;
      int st = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok && it.next(s)) {
        const int buf = s.idx % p.nbufs;
        const uint32_t bph = (s.idx / p.nbufs) & 1;
        if (!mbar_wait(&tail->tmem_empty[buf], bph ^ 1, abort_word, p.err, 302)) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * p.BN;
        for (int kbi = s.kb0; kbi < s.kb1; ++kbi) {
          if (!mbar_wait(&tail->full[st], ph, abort_word, p.err, 303)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint32_t accum = (kbi > s.kb0 || k > 0) ? 1u : 0u;
            const uint64_t koff = static_cast<uint64_t>(k * kUmmaK * 2 >> 4);
            umma_bf16(acc, da0 + koff, da0 + d_b + koff, idesc, accum);
          }
          tc_commit(&tail->empty[st]);
          if (++st == p.stages) { st = 0; ph ^= 1; da0 = da0_first; } else { da0 += d_stage; }
        }
        if (ok) tc_commit(&tail->tmem_full[buf]);
      }
    }
  } else if (warp >= 6) {
    pdl_wait();
    pdl_trigger();
    if (w8 && warp < 6 + kConvWarps) {
      // ---------------------------------------------------------------- fp8 weight tiles -> scaled bf16 operand tiles
      // Two converter warps own each ring stage (warps 2s and 2s + 1 take the upper and lower 64 rows of every tile
      // that lands in stage s), so one tile per stage is in conversion at once and the latency of one tile's
      // load-convert-store chain is hidden behind the others'. A stage's barrier is always waited on by the same
      // warps, phase after phase: a waiter that skipped phases could not tell them apart by parity. Per pass a warp reads 512 contiguous raw bytes
      // (8 rows x 64): lane l holds 16 values of row l / 4 and writes two 16-byte chunks of the 128-byte-swizzled
      // K-major tile.
      const int cw = warp - 6;
      SegIter it(p, g);
      Seg s;
      int st = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok && it.next(s)) {
        const int n_tile = s.tile / p.m_tiles;
        const float* srow = p.wfmt == 1 ? p.w_scale + static_cast<size_t>(n_tile) * p.sw_ld : nullptr;
        for (int kbi = s.kb0; kbi < s.kb1; ++kbi) {
          if (st == (cw >> 1)) {
            if (!mbar_wait(&tail->raw_full[st], ph, abort_word, p.err, 307)) { ok = false; break; }
            uint8_t* sa = smem + st * stage_bytes;
            const uint8_t* raw = sa + kATile + b_bytes + lane * 16;
            if (p.wfmt == 2) {
              // NVFP4: 16 rows x 32 raw bytes per pass; lane l holds 32 values of row l / 2 (two scale blocks of 16)
              const float gs = *p.w_gscale;
#pragma unroll 2
              for (int pass = (cw & 1) * 4; pass < (cw & 1) * 4 + 4; ++pass) {
                const uint4 q = *reinterpret_cast<const uint4*>(raw + pass * 512);
                const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
                const int r = pass * 16 + (lane >> 1);
                const uint16_t sb = *reinterpret_cast<const uint16_t*>(
                    p.w_bscale + static_cast<size_t>(n_tile * 128 + r) * p.bs_ld + kbi * 4 + (lane & 1) * 2);
                __nv_fp8_e4m3 s0, s1;
                s0.__x = static_cast<__nv_fp8_storage_t>(sb & 0xff);
                s1.__x = static_cast<__nv_fp8_storage_t>(sb >> 8);
                const float sc2[2] = {static_cast<float>(s0) * gs, static_cast<float>(s1) * gs};
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  float v[8];
                  const uint32_t w4 = qw[c];
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    const uint32_t nib = (w4 >> (4 * j)) & 0xfu, m = nib & 7u;
                    // e2m1 magnitudes {0, .5, 1, 1.5, 2, 3, 4, 6} as bf16 bit patterns, widened to fp32
                    const uint32_t bits = m >= 2u ? 0x3f80u + (m - 2u) * 0x40u : (m ? 0x3f00u : 0u);
                    v[j] = __uint_as_float((bits | ((nib & 8u) << 12)) << 16) * sc2[c >> 1];
                  }
                  const int chunk = (lane & 1) * 4 + c;
                  *reinterpret_cast<uint4*>(sa + r * 128 + ((chunk ^ (r & 7)) << 4)) = pack_bf16x8(v);
                }
              }
            } else {
              // e4m3 values: 8 rows x 64 raw bytes per pass; lane l holds 16 values of row l / 4
              const float sc128 = p.wfmt == 1 ? srow[kbi >> 1] : 0.f;   // one scale per 128 K values = two K blocks
#pragma unroll 4
              for (int pass = (cw & 1) * 8; pass < (cw & 1) * 8 + 8; ++pass) {
                const uint4 q = *reinterpret_cast<const uint4*>(raw + pass * 512);
                const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
                const int r = pass * 8 + (lane >> 2);
                float sc = sc128;
                if (p.wfmt == 3) {
                  // MXFP8: a power-of-two scale per 32 values (ue8m0: 2^(e - 127))
                  const uint32_t e = p.w_bscale[static_cast<size_t>(n_tile * 128 + r) * p.bs_ld + kbi * 2 + ((lane & 3) >> 1)];
                  sc = __uint_as_float(e << 23);
                }
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                  float v[8];
#pragma unroll
                  for (int j = 0; j < 2; ++j) {
                    __nv_fp8x4_e4m3 e;
                    e.__x = qw[c * 2 + j];
                    const float4 f = static_cast<float4>(e);
                    v[4 * j] = f.x * sc; v[4 * j + 1] = f.y * sc; v[4 * j + 2] = f.z * sc; v[4 * j + 3] = f.w * sc;
                  }
                  const int chunk = (lane & 3) * 2 + c;
                  *reinterpret_cast<uint4*>(sa + r * 128 + ((chunk ^ (r & 7)) << 4)) = pack_bf16x8(v);
                }
              }
            }
            fence_proxy_async_smem();        // generic-proxy writes before the tensor core reads the tile
            __syncwarp();
            if (lane == 0) mbar_arrive(&tail->full[st]);
          }
          if (++st == p.stages) { st = 0; ph ^= 1; }
        }
      }
    }
  } else {
    pdl_wait();
    pdl_trigger();
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    SegIter it(p, g);
    Seg s;
    while (it.next(s)) {
      const int buf = s.idx % p.nbufs;
      const uint32_t bph = (s.idx / p.nbufs) & 1;
      if (!mbar_wait(&tail->tmem_full[buf], bph, abort_word, p.err, 304)) break;
      tc_fence_after();
      const int t0 = (s.tile % p.m_tiles) * p.BN;
      const uint32_t acc = tmem_base + buf * p.BN + (static_cast<uint32_t>(quad * 32) << 16);
      float* mine = p.ws + (static_cast<size_t>(g) * p.slots + s.idx) * p.slot_floats;
      for (int c0 = 0; c0 < p.BN; c0 += 16) {
        if (t0 + c0 >= p.M) break;
        uint32_t a[16];
        tmem_ld_32x16(acc + c0, a);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 16; ++j) __stcg(mine + static_cast<size_t>(c0 + j) * kBM + row, __uint_as_float(a[j]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tail->tmem_empty[buf]);
      if (p.tile_epi) {
        // count this CTA's partial of the tile in; the four drain warps act as one group of 128 threads
        const int tiles_inter = p.inter >> 7;
        const int n_tile = s.tile;                       // m_tiles == 1
        const int cnt_idx = (p.mode == 1 && n_tile >= tiles_inter) ? n_tile - tiles_inter : n_tile;
        __threadfence();
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (warp == 2 && lane == 0) {
          int want = tile_contributors(p, cnt_idx);
          if (p.mode == 1) want += tile_contributors(p, cnt_idx + tiles_inter);
          const int prev = atomicAdd(p.state + kDecTileCnt + cnt_idx, 1);
          tail->tile_last = prev == want - 1 ? 1 : 0;
          if (prev == want - 1) p.state[kDecTileCnt + cnt_idx] = 0;     // ready for the next launch
        }
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (tail->tile_last != 0 && p.rope) {
          __threadfence();
          const int tid = (warp - 2) * 32 + lane;
          const int head = cnt_idx;
          if (head < p.n_q + p.n_kv) {
            for (int c = tid; c < p.M * 8; c += 128) qkv_rotate_item(p, c >> 3, head, (c & 7) << 3);
          } else {
            for (int c = tid; c < p.M * 16; c += 128) qkv_value_item(p, c >> 4, head, (c & 15) << 3);
          }
        } else if (tail->tile_last != 0) {
          __threadfence();
          const int tid = (warp - 2) * 32 + lane;
          const int n0 = cnt_idx << 7;
          const int ncols = min(128, (p.mode == 1 ? p.inter : p.N) - n0);
          const int chunks = ncols >> 3;
          for (int c = tid; c < p.M * chunks; c += 128) {
            const int t = c / chunks;
            const int n = n0 + ((c - t * chunks) << 3);
            float v[8];
            reduce8(p, t, n, v);
            if (p.mode == 1) {
              float u[8];
              reduce8(p, t, p.inter + n, u);
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = silu_f(v[i]) * u[i];
            }
            const int col = p.bN > 0 ? (n / p.bN) * p.y_boff + n % p.bN : n;
            *reinterpret_cast<uint4*>(p.Y + static_cast<size_t>(t) * p.ldy + col) = pack_bf16x8(v);
          }
        }
      }
    }
  }

  if (p.tile_epi) {
    // no meeting point: leave once every role of this CTA is done
    tc_fence_before();
    __syncthreads();
    MB_DEC_STAMP(5);
    if (warp == 1) {
      tc_fence_after();
      tmem_dealloc(tmem_base, p.tmem_cols);
    }
    return;
  }

  // ------------------------------------------------------------------ grid-wide meeting point
  // The CTA barrier orders every thread's partial-tile stores before thread 0's release below, and a
  // release is cumulative: one fence per CTA, then a fire-and-forget add, then acquire polls.
  __syncthreads();
  MB_DEC_STAMP(3);
  if (threadIdx.x == 0) {
    asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.state + kDecArrive) : "memory");
    bool ok = *abort_word == 0;
    if (ok && ld_acquire_gpu(p.state + kDecArrive) < p.G) {
      const uint64_t t_start = globaltimer_ns();
      uint32_t spins = 0;
      while (ld_acquire_gpu(p.state + kDecArrive) < p.G) {
        if (((++spins) & 0xff) == 0 && globaltimer_ns() - t_start > 1000000000ull) {
          atomicCAS(p.err, 0, 305);
          ok = false;
          break;
        }
      }
    }
    tail->flag = ok ? 1 : 0;
  }
  __syncthreads();
  MB_DEC_STAMP(4);
  const bool run_epilogue = tail->flag != 0;

  // ------------------------------------------------------------------ epilogue over the output (phase B)
  if (run_epilogue && p.rope) {
    // QKV projection with rotation and cache store: rotated items first (8 per token and head), then the values
    const int rot = p.M * (p.n_q + p.n_kv) * 8;
    const int total = rot + p.M * p.n_kv * 16;
    for (int c = g * kThreads + threadIdx.x; c < total; c += p.G * kThreads) {
      if (c < rot) {
        const int t = c / ((p.n_q + p.n_kv) * 8), r = c - t * ((p.n_q + p.n_kv) * 8);
        qkv_rotate_item(p, t, r >> 3, (r & 7) << 3);
      } else {
        const int c2 = c - rot;
        const int t = c2 / (p.n_kv * 16), r = c2 - t * (p.n_kv * 16);
        qkv_value_item(p, t, p.n_q + p.n_kv + (r >> 4), (r & 15) << 3);
      }
    }
  } else if (run_epilogue && p.mode != 2) {
    const int ncols = p.mode == 1 ? p.inter : p.N;
    const int chunks_per_row = ncols >> 3;
    const int total = p.M * chunks_per_row;
    for (int c = g * kThreads + threadIdx.x; c < total; c += p.G * kThreads) {
      const int t = c / chunks_per_row;
      const int n = (c - t * chunks_per_row) << 3;
      float v[8];
      reduce8(p, t, n, v);
      if (p.mode == 1) {
        float u[8];
        reduce8(p, t, p.inter + n, u);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = silu_f(v[i]) * u[i];
      }
      const int col = p.bN > 0 ? (n / p.bN) * p.y_boff + n % p.bN : n;
      *reinterpret_cast<uint4*>(p.Y + static_cast<size_t>(t) * p.ldy + col) = pack_bf16x8(v);
    }
  } else if (run_epilogue) {
    // all ring stages are idle: reuse them as the row cache (N * 2 bytes)
    uint4* row_cache = reinterpret_cast<uint4*>(smem);
    const int gen = ld_volatile(p.state + kDecGen);
    const int g3 = gen % 3, gclr = (gen + 2) % 3;
    const int old_rows = ld_volatile(p.state + kDecGenRows + gclr);
    const int nvec = p.N >> 3;
    const int W = p.world;
    const int r_hi = p.M > old_rows ? p.M : old_rows;
    const size_t gen_stride = static_cast<size_t>(W) * p.lam_rows * p.N;
    const size_t src_stride = static_cast<size_t>(p.lam_rows) * p.N;
    for (int r = g; r < r_hi; r += p.G) {
      if (r < p.M) {
        float ss = 0.f;
        for (int v = threadIdx.x; v < nvec; v += kThreads) {
          float acc[8];
          // the residual row does not depend on the partials: its load travels together with theirs
          const uint4 hv = *reinterpret_cast<const uint4*>(p.h + static_cast<size_t>(r) * p.N + (v << 3));
          reduce8(p, r, v << 3, acc);
          if (W > 1) {
            // push this rank's bf16 partial row to every peer, then collect the peers' rows
            uint4 mine = pack_bf16x8(acc);
            mine.x = sanitize2(mine.x); mine.y = sanitize2(mine.y);
            mine.z = sanitize2(mine.z); mine.w = sanitize2(mine.w);
            const size_t off = g3 * gen_stride + static_cast<size_t>(p.rank) * src_stride +
                               static_cast<size_t>(r) * p.N + (v << 3);
#pragma unroll
            for (int s = 1; s < kMaxRanks; ++s) {
              if (s < W) {
                const int dst = (p.rank + s) % W;
                *reinterpret_cast<uint4*>(p.lam[dst] + off) = mine;
              }
            }
            // sum in rank order so that every rank computes the same bits
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.f;
            const __nv_bfloat16* inbox = p.lam[p.rank] + g3 * gen_stride + static_cast<size_t>(r) * p.N + (v << 3);
            uint64_t t_start = 0;
            for (int src = 0; src < W; ++src) {
              if (src == p.rank) { unpack_add(mine, acc); continue; }
              const void* a = inbox + static_cast<size_t>(src) * src_stride;
              uint4 in = ld_volatile_v4(a);
              uint32_t spins = 0;
              while (has_sentinel(in.x) || has_sentinel(in.y) || has_sentinel(in.z) || has_sentinel(in.w)) {
                if (((++spins) & 0x3f) == 0) {
                  const uint64_t now = globaltimer_ns();
                  if (t_start == 0) t_start = now;
                  if (now - t_start > 1000000000ull) { atomicCAS(p.err, 0, 306); break; }
                }
                in = ld_volatile_v4(a);
              }
              unpack_add(in, acc);
            }
          }
          unpack_add(hv, acc);
          const uint4 out = pack_bf16x8(acc);
          const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&out);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(q[i]);
            ss += f.x * f.x + f.y * f.y;
          }
          *reinterpret_cast<uint4*>(p.h + static_cast<size_t>(r) * p.N + (v << 3)) = out;
          row_cache[v] = out;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) tail->red[warp] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int i = 0; i < kThreads / 32; ++i) tot += tail->red[i];
        const float inv = rsqrtf(tot / static_cast<float>(p.N) + p.eps);
        for (int v = threadIdx.x; v < nvec; v += kThreads) {
          uint4 a = row_cache[v];
          const uint4 wv = *reinterpret_cast<const uint4*>(p.gamma + (v << 3));
          __nv_bfloat162* ap = reinterpret_cast<__nv_bfloat162*>(&a);
          const __nv_bfloat162* wp = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(ap[i]);
            const float2 gm = __bfloat1622float2(wp[i]);
            if (p.mbc) {
              ap[i] = __floats2bfloat162_rn(f.x * inv * (gm.x + p.w_off), f.y * inv * (gm.y + p.w_off));
            } else {
              const __nv_bfloat162 nrm = __floats2bfloat162_rn(f.x * inv, f.y * inv);
              const float2 nf = __bfloat1622float2(nrm);
              ap[i] = __floats2bfloat162_rn(nf.x * (gm.x + p.w_off), nf.y * (gm.y + p.w_off));
            }
          }
          *reinterpret_cast<uint4*>(p.xn + static_cast<size_t>(r) * p.N + (v << 3)) = a;
        }
        __syncthreads();   // row cache and `red` are reused by the next row
      }
      if (W > 1 && r < old_rows) {
        // rows of the generation that was read two kernels ago become sentinels again
        const uint4 sv = make_uint4(kSentinel2, kSentinel2, kSentinel2, kSentinel2);
        for (int src = 0; src < W; ++src) {
          if (src == p.rank) continue;
          uint4* row = reinterpret_cast<uint4*>(p.lam[p.rank] + gclr * gen_stride + static_cast<size_t>(src) * src_stride +
                                                static_cast<size_t>(r) * p.N);
          for (int v = threadIdx.x; v < nvec; v += kThreads) row[v] = sv;
        }
      }
    }
  }

  // ------------------------------------------------------------------ leave
  tc_fence_before();
  __syncthreads();
  MB_DEC_STAMP(5);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, p.tmem_cols);
  }
  if (threadIdx.x == 0) {
    __threadfence();
    const int prev = atomicAdd(p.state + kDecDepart, 1);
    if (prev == p.G - 1) {
      // last CTA out: every CTA has passed the meeting point and read the generation words
      p.state[kDecArrive] = 0;
      p.state[kDecDepart] = 0;
      if (p.mode == 2 && p.world > 1) {
        const int gen = ld_volatile(p.state + kDecGen);
        p.state[kDecGenRows + gen % 3] = p.M;
        p.state[kDecGen] = gen + 1;
      }
    }
  }
}

static uint32_t pow2_cols(int c) {
  uint32_t v = 32;
  while (static_cast<int>(v) < c) v <<= 1;
  return v;
}

}  // namespace dec
}  // namespace mb

using namespace mb;

extern "C" int mb_gemm_dec_max_tokens(void) { return 256; }
extern "C" int mb_gemm_dec_state_ints(void) { return kDecStateInts; }
// enough for kSlots slots of 128-token tiles (or half as many 256-token ones) on every SM
extern "C" size_t mb_gemm_dec_workspace_bytes(int num_sms) {
  return static_cast<size_t>(num_sms > 0 ? num_sms : 148) * dec::kSlots * 128 * dec::kBM * sizeof(float);
}
// bf16 elements of one rank's receive buffer for the all-reduce mode.
extern "C" size_t mb_gemm_dec_lamport_elems(int world, int rows, int N) {
  return static_cast<size_t>(3) * world * rows * N;
}

static unsigned long long* g_dec_trace = nullptr;
// Measurement aid: `buf` (device, 8 * num_sms uint64) receives per-CTA globaltimer stamps of the next launches:
// [0] start, [1] weight prefetch issued, [2] dependencies done, [3] partials written, [4] all CTAs arrived,
// [5] epilogue done. nullptr turns it off.
extern "C" void mb_set_gemm_dec_trace(void* buf) { g_dec_trace = static_cast<unsigned long long*>(buf); }
static int g_dec_tile_epi = 0;    // modes 0 / 1: per-tile last-arriver epilogue instead of the grid-wide meeting point (off: measured
                                  // slower on B200 from 64 tokens up, 103 vs 53 us per layer at TP8 shapes: one CTA's drain warps
                                  // reduce a whole tile while the meeting point spreads that work over all threads of the grid)
extern "C" void mb_set_gemm_dec_tile_epilogue(int on) { g_dec_tile_epi = on; }
static int g_dec_rope = 0;        // QKV projection with rotation + cache store in its epilogue (mb_gemm_dec_qkv_rope); off:
                                  // measured 2.5 % (TP2) to 9 % (TP1) slower per decode step than the two kernels under a graph
extern "C" void mb_set_gemm_dec_rope(int on) { g_dec_rope = on; }
static int g_dec_smem_kb = 200;   // ring budget (measured on B200: chains of decode GEMMs run 8 % faster with 150-200 KB than with 100)
extern "C" void mb_set_gemm_dec_smem_kb(int kb) { g_dec_smem_kb = kb < 40 ? 40 : (kb > 200 ? 200 : kb); }

static int dec_plan(int M, int N, int K, int mode, size_t ws_bytes, int num_sms, dec::Params* out, bool w8 = false) {
  using namespace mb::dec;
  if (M <= 0 || N <= 0 || M > 256 || K % 8 || N % 8 || K < kBK) return MB_ERR_SHAPE;
  if (mode < 0 || mode > 2 || (mode == 1 && N % 16)) return MB_ERR_SHAPE;
  if (num_sms <= 0) num_sms = 148;
  Params p = {};
  p.M = M; p.N = N; p.K = K;
  p.BN = (M + 15) / 16 * 16;
  p.m_tiles = 1;
  p.nbufs = 2;
  p.tmem_cols = pow2_cols(2 * p.BN);
  const int stage_bytes = kATile + p.BN * kBK * 2 + (w8 ? kRawTile : 0);
  const int budget = (p.BN <= 128 ? g_dec_smem_kb : 200) * 1024;
  int stages = budget / stage_bytes;
  if (stages > 8) stages = 8;
  if (w8 && stages > 5) stages = 5;     // two converter warps per stage, ten converter warps
  if (stages < 2) stages = 2;
  p.stages = stages;
  p.tiles = (N + kBM - 1) / kBM;
  p.kb = (K + kBK - 1) / kBK;
  const long long units = static_cast<long long>(p.tiles) * p.kb;
  if (units * num_sms >= (1ll << 31)) return MB_ERR_SHAPE;
  p.units = static_cast<uint32_t>(units);
  long long G = units / 4;    // at least four K blocks per share
  if (G > num_sms) G = num_sms;
  if (G < 1) G = 1;
  p.G = static_cast<int>(G);
  // segments per CTA: a share of ceil(units / G) blocks touches at most ceil(share / kb) + 1 tiles
  const long long share = (units + p.G - 1) / p.G;
  p.slots = static_cast<int>((share + p.kb - 1) / p.kb + 1);
  if (p.slots > kSlots) return MB_ERR_SHAPE;
  p.slot_floats = p.BN * kBM;
  if (static_cast<size_t>(p.G) * p.slots * p.slot_floats * sizeof(float) > ws_bytes) return MB_ERR_TOO_LARGE;
  // the epilogue of mode 2 keeps one token row in the idle ring
  if (mode == 2 && static_cast<size_t>(N) * 2 > static_cast<size_t>(stages) * stage_bytes) return MB_ERR_SHAPE;
  *out = p;
  return MB_OK;
}

extern "C" int mb_gemm_dec_plan(int M, int N, int K, int mode, size_t ws_bytes, int num_sms) {
  dec::Params p;
  return dec_plan(M, N, K, mode, ws_bytes, num_sms, &p);
}

// mode 0: Y[M, N] bf16.  mode 1: Y[M, N/2] = silu(X Wg^T) * (X Wu^T), W = [Wg; Wu] (N rows in all).
// mode 2: h[M, N] += sum over ranks of X W^T (in place), xn = RMSNorm(h) * (gamma + w_off); `lam` holds
// every rank's receive buffer (mb_gemm_dec_lamport_elems elements, filled with bf16 -0.0 once) and
// `state` mb_gemm_dec_state_ints zeroed ints that live as long as the buffers. world = 1: lam unused.
// All ranks must issue the same sequence of mode-2 calls. Launches that share `ws` / `state` must not
// overlap on the device. Returns MB_ERR_SHAPE / MB_ERR_TOO_LARGE for shapes this kernel does not take
// (see mb_gemm_dec_plan); the caller then uses the tiled kernels.
struct DecRope {
  int n_q, n_kv, page_size;
  long long page_stride, head_stride;
  const int32_t* positions;
  const int64_t* slots;
  const float* cos_sin;
  void* k_cache;
  void* v_cache;
};

static int gemm_dec_impl(const void* X, const void* W, int M, int N, int K, int ldx, int ldw, int mode,
                         void* Y, int ldy, void* h, void* xn, const void* gamma, float eps, float w_off,
                         int mbc, int world, int rank, void* const* lam, int lam_rows, void* ws,
                         size_t ws_bytes, int* state, int* err, int num_sms, cudaStream_t stream, int bN, int x_boff,
                         int y_boff, int x_cols, const DecRope* rope = nullptr, const float* w_scale = nullptr,
                         int wfmt = 0, const uint8_t* w_bscale = nullptr, const float* w_gscale = nullptr) {
  using namespace mb::dec;
  if (M <= 0 || N <= 0) return MB_OK;
  if (ldx % 8 || ldw % 8 || (mode != 2 && ldy % 8)) return MB_ERR_SHAPE;
  if (mode == 2 && (world < 1 || world > kMaxRanks || rank < 0 || rank >= world ||
                    (world > 1 && (lam == nullptr || M > lam_rows))))
    return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(Y) |
       reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(xn) | reinterpret_cast<uintptr_t>(gamma) |
       reinterpret_cast<uintptr_t>(ws)) & 15)
    return MB_ERR_ALIGN;
  if (num_sms <= 0) num_sms = 148;
  Params p;
  if (w_scale != nullptr) wfmt = 1;
  int rc = dec_plan(M, N, K, mode, ws_bytes, num_sms, &p, wfmt != 0);
  if (rc != MB_OK) return rc;
  if (wfmt != 0 && (N % 128 || K % 128 || bN > 0)) return MB_ERR_SHAPE;
  if ((wfmt == 2 && (w_bscale == nullptr || w_gscale == nullptr)) || (wfmt == 3 && w_bscale == nullptr) || wfmt < 0 || wfmt > 3)
    return MB_ERR_SHAPE;
  p.w_scale = w_scale; p.sw_ld = (K + 127) / 128;
  p.wfmt = wfmt; p.w_bscale = w_bscale; p.w_gscale = w_gscale;
  p.bs_ld = wfmt == 2 ? K / 16 : K / 32;
  p.ws = static_cast<float*>(ws);
  p.trace = g_dec_trace;
  p.state = state; p.err = err; p.mode = mode;
  p.Y = static_cast<__nv_bfloat16*>(Y); p.ldy = ldy;
  p.bN = bN; p.x_boff = x_boff; p.y_boff = y_boff;
  p.inter = mode == 1 ? N / 2 : 0;
  p.tile_epi = (g_dec_tile_epi && mode != 2 && p.tiles <= kDecTileCounters && (mode == 0 || p.inter % kBM == 0)) ? 1 : 0;
  p.rope = 0;
  if (rope != nullptr) {
    if (mode != 0 || N != (rope->n_q + 2 * rope->n_kv) * 128) return MB_ERR_SHAPE;
    p.rope = 1; p.n_q = rope->n_q; p.n_kv = rope->n_kv; p.page_size = rope->page_size;
    p.page_stride = rope->page_stride; p.head_stride = rope->head_stride;
    p.positions = rope->positions; p.kv_slots = rope->slots; p.cos_sin = rope->cos_sin;
    p.k_cache = static_cast<__nv_bfloat16*>(rope->k_cache); p.v_cache = static_cast<__nv_bfloat16*>(rope->v_cache);
  }
  p.h = static_cast<__nv_bfloat16*>(h); p.xn = static_cast<__nv_bfloat16*>(xn);
  p.gamma = static_cast<const __nv_bfloat16*>(gamma);
  p.eps = eps; p.w_off = w_off; p.mbc = mbc;
  p.world = mode == 2 ? world : 1; p.rank = mode == 2 ? rank : 0; p.lam_rows = lam_rows;
  for (int i = 0; i < kMaxRanks; ++i)
    p.lam[i] = (mode == 2 && world > 1 && i < world) ? static_cast<__nv_bfloat16*>(lam[i]) : nullptr;
  CUtensorMap tw, tx;
  // fp8 weights: 128 rows x 64 bytes per K block, unswizzled (the converter warps write the operand layout)
  // (NVFP4: two values per byte, so a K block of 64 values is 32 bytes of a [N, K / 2] byte matrix)
  rc = wfmt == 2   ? cached_tmap_raw(&tw, W, N, K / 2, K / 2, kBM, 32)
       : wfmt != 0 ? cached_tmap_raw(&tw, W, N, K, ldw, kBM, 64)
                   : cached_tmap(&tw, W, N, K, ldw, kBM, 2);
  if (rc != MB_OK) return rc;
  rc = cached_tmap(&tx, X, M, bN > 0 ? x_cols : K, ldx, p.BN, 2);
  if (rc != MB_OK) return rc;
  const int stage_bytes = kATile + p.BN * kBK * 2 + (wfmt != 0 ? kRawTile : 0);
  const size_t smem = static_cast<size_t>(p.stages) * stage_bytes + sizeof(Tail) + 1024;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(gemm_dec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return MB_ERR_LAUNCH;
    configured.done();
  }
  const cudaError_t e = launch_k(gemm_dec_kernel, dim3(p.G), dim3(kThreads), smem, stream, tw, tx, p);
  return e == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_gemm_dec(const void* X, const void* W, int M, int N, int K, int ldx, int ldw, int mode,
                           void* Y, int ldy, void* h, void* xn, const void* gamma, float eps, float w_off,
                           int mbc, int world, int rank, void* const* lam, int lam_rows, void* ws,
                           size_t ws_bytes, int* state, int* err, int num_sms, cudaStream_t stream) {
  return gemm_dec_impl(X, W, M, N, K, ldx, ldw, mode, Y, ldy, h, xn, gamma, eps, w_off, mbc, world, rank, lam, lam_rows,
                       ws, ws_bytes, state, err, num_sms, stream, 0, 0, 0, 0);
}

// The decode-step GEMM over the column blocks of one activation matrix (per-head weight absorption with at most
// 256 tokens): Y[m, b * y_off + n] = sum_k X[m, b * x_off + k] * W[b, n, k]. W: [B, N, K] contiguous with
// N % 128 == 0 (a weight tile belongs to one head) and K % 64 == 0. One persistent launch over all heads.
extern "C" int mb_gemm_dec_batched(const void* X, const void* W, void* Y, int B, int M, int N, int K, int ldx,
                                   int x_off, int ldy, int y_off, int x_cols, void* ws, size_t ws_bytes, int* state,
                                   int* err, int num_sms, cudaStream_t stream) {
  if (B <= 0) return MB_OK;
  if (N % mb::dec::kBM || K % mb::dec::kBK || x_off % 8 || y_off % 8 || x_off <= 0 || y_off < N) return MB_ERR_SHAPE;
  return gemm_dec_impl(X, W, M, B * N, K, ldx, K, 0, Y, ldy, nullptr, nullptr, nullptr, 0.f, 0.f, 0, 1, 0, nullptr, 0, ws,
                       ws_bytes, state, err, num_sms, stream, N, x_off, y_off, x_cols);
}

// QKV projection of a decode step with the rotary embedding and the KV-cache store in its tile epilogue
// (head_dim 128, rotate-half convention): what mb_gemm_dec (mode 0) followed by mb_rope_kv_store computes, in
// one launch. Returns MB_ERR_SHAPE when the shape does not fit; the caller then runs the two kernels.
extern "C" int mb_gemm_dec_qkv_rope(const void* X, const void* W, int M, int K, int ldx, int ldw, void* qkv, int ldy,
                                    const int32_t* positions, const int64_t* slots, const float* cos_sin, void* k_cache,
                                    void* v_cache, int n_q, int n_kv, int head_dim, int page_size,
                                    long long page_stride, long long head_stride, void* ws, size_t ws_bytes, int* state,
                                    int* err, int num_sms, cudaStream_t stream) {
  if (head_dim != 128 || !g_dec_rope) return MB_ERR_SHAPE;
  DecRope r{n_q, n_kv, page_size, page_stride, head_stride, positions, slots, cos_sin, k_cache, v_cache};
  return gemm_dec_impl(X, W, M, (n_q + 2 * n_kv) * 128, K, ldx, ldw, 0, qkv, ldy, nullptr, nullptr, nullptr, 0.f, 0.f, 0,
                       1, 0, nullptr, 0, ws, ws_bytes, state, err, num_sms, stream, 0, 0, 0, 0, &r);
}

// The decode-step GEMM on block-scaled fp8 weights (e4m3 [N, K] with fp32 scales [N / 128, K / 128]) and bf16
// activations: weight tiles are converted to scaled bf16 in shared memory, everything else (modes, tails,
// all-reduce) is mb_gemm_dec. N % 128 == 0 and K % 128 == 0.
extern "C" int mb_gemm_dec_w8(const void* X, const void* Wq, const float* Ws, int M, int N, int K, int ldx, int mode,
                              void* Y, int ldy, void* h, void* xn, const void* gamma, float eps, float w_off, int mbc,
                              int world, int rank, void* const* lam, int lam_rows, void* ws, size_t ws_bytes,
                              int* state, int* err, int num_sms, cudaStream_t stream) {
  if (Ws == nullptr) return MB_ERR_SHAPE;
  return gemm_dec_impl(X, Wq, M, N, K, ldx, K, mode, Y, ldy, h, xn, gamma, eps, w_off, mbc, world, rank, lam, lam_rows,
                       ws, ws_bytes, state, err, num_sms, stream, 0, 0, 0, 0, nullptr, Ws);
}

// The decode-step GEMM on NVFP4 (wfmt 2: Wq [N, K / 2] bytes, two e2m1 values per byte with the even index in the low
// nibble; block_scales [N, K / 16] e4m3; *global_scale fp32 on the device) or MXFP8 (wfmt 3: Wq [N, K] e4m3;
// block_scales [N, K / 32] ue8m0) weights with bf16 activations: weight-only quantisation, dequantised tile by tile
// in shared memory. Plain and SwiGLU modes and the all-reduce tail as for the other formats.
extern "C" int mb_gemm_dec_wq(int wfmt, const void* X, const void* Wq, const void* block_scales, const float* global_scale,
                              int M, int N, int K, int ldx, int mode, void* Y, int ldy, void* h, void* xn,
                              const void* gamma, float eps, float w_off, int mbc, int world, int rank, void* const* lam,
                              int lam_rows, void* ws, size_t ws_bytes, int* state, int* err, int num_sms,
                              cudaStream_t stream) {
  if (wfmt != 2 && wfmt != 3) return MB_ERR_SHAPE;
  return gemm_dec_impl(X, Wq, M, N, K, ldx, K, mode, Y, ldy, h, xn, gamma, eps, w_off, mbc, world, rank, lam, lam_rows,
                       ws, ws_bytes, state, err, num_sms, stream, 0, 0, 0, 0, nullptr, nullptr, wfmt,
                       static_cast<const uint8_t*>(block_scales), global_scale);
}
