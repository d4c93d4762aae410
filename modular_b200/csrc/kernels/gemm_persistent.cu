// Persistent bf16 GEMM for sm_100a: one CTA per SM, stream-K work split, double-buffered
// TMEM accumulators.
//
//   Y[M, N] = X[M, K] · W[N, K]^T   (+ residual | SwiGLU over W = [gate; up] | fp32 out)
//
// Work is counted in units of one 64-wide K block of one 128(weight rows) x BN(tokens) tile.
//
// The schedule has two phases:
//   phase 1 (round robin): the first `tiles_dp` tiles - a whole number of waves - go to CTAs
//       as whole tiles g, g+G, ... Concurrent CTAs then work on neighbouring tiles and share
//       weight/activation tiles in L2, and no tile needs a fix-up.
//   phase 2 (stream-K): the K-block range of the remaining tiles (less than one wave) is cut
//       into equal contiguous shares, so every SM streams the same number of weight bytes no
//       matter how the tile count divides the SM count - this is what keeps decode-sized
//       GEMMs (a few dozen tiles) busy on all 148 SMs. A tile cut across CTAs is finished by
//       whichever contributor arrives last: every contributor writes its fp32 partial to a
//       private workspace slot, bumps a per-(tile, lane-quadrant) counter, and the last one
//       sums the slots in CTA order (deterministic) and runs the fused epilogue. Nobody
//       waits on anybody.
//   mode 0 = phase 1 only, mode 1 = phase 2 only, mode 2 = both (default).
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
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "comm_flags.h"
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
  int BN, stages, acc_cols, nbufs;
  uint32_t tmem_cols;
  int m_tiles, tiles, kb;
  int tiles_dp;      // tiles handled round-robin as whole tiles
  int G2;            // CTAs taking part in the stream-K phase
  int dbg;           // measurement aid: bit0 skip the fix-up reduction, bit1 skip the partial store too
  long long units2;  // K blocks in the stream-K phase = (tiles - tiles_dp) * kb
  // Tensor-parallel all-gather -> GEMM gating (nullptr = off): token rows [s*rpr, (s+1)*rpr) are
  // pushed into X by rank s, which then raises flag kReady+s of this rank's flag array.
  const int* gate_flags;
  int gate_rpr, gate_world;
  int packed_kb;     // > 0: W is pre-tiled [rows/128][K/64][128][64]; value = K/64
  int w_static;      // W is written by no kernel of the stream: its first tiles are requested before the dependency wait
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
  int slot;  // workspace slot (0/1) of this CTA when the segment is a partial tile
};

// Enumerates this CTA's segments; identical in every warp role.
struct SegIter {
  int G, g, kb, idx, next_tile, tiles_dp;
  bool sk_first;
  long long u, u1;
  __device__ SegIter(const Params& p, int g_, int G_)
      : G(G_), g(g_), kb(p.kb), idx(0), next_tile(g_), tiles_dp(p.tiles_dp), sk_first(true) {
    if (g_ < p.G2) {
      u = p.units2 * g_ / p.G2;
      u1 = p.units2 * (g_ + 1) / p.G2;
    } else {
      u = u1 = 0;
    }
  }
  __device__ bool next(Seg& s) {
    if (next_tile < tiles_dp) {
      s.tile = next_tile; s.kb0 = 0; s.kb1 = kb; s.idx = idx++; s.slot = 0;
      next_tile += G;
      return true;
    }
    if (u >= u1) return false;
    const int rel = static_cast<int>(u / kb);
    const int kb0 = static_cast<int>(u - static_cast<long long>(rel) * kb);
    long long len = kb - kb0;
    if (len > u1 - u) len = u1 - u;
    s.tile = tiles_dp + rel; s.kb0 = kb0; s.kb1 = kb0 + static_cast<int>(len); s.idx = idx++;
    s.slot = sk_first ? 0 : 1;
    sk_first = false;
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
  // Static weights: fill the ring with this CTA's first weight tiles while the previous kernel drains; their
  // activation tiles follow after the wait on the same barriers.
  int pre = 0;
  if (p.w_static && p.gate_flags == nullptr && warp == 0 && lane == 0) {
    SegIter it(p, g, G);
    Seg s;
    int st = 0;
    while (pre < p.stages && it.next(s)) {
      const int n0 = (s.tile / p.m_tiles) * kBM;
      for (int kbi = s.kb0; kbi < s.kb1 && pre < p.stages; ++kbi, ++st, ++pre) {
        uint8_t* sa = smem + st * stage_bytes;
        uint64_t* full_st = &tail->full[st];
        mbar_arrive_expect_tx(full_st, stage_bytes);
        if (p.packed_kb > 0) {
          tma_load_2d(sa, &tmW, full_st, 0, ((n0 >> 7) * p.packed_kb + kbi) << 7);
          if (DUAL) tma_load_2d(sa + kATile, &tmW, full_st, 0, (((p.dual_rows + n0) >> 7) * p.packed_kb + kbi) << 7);
        } else {
          tma_load_2d(sa, &tmW, full_st, kbi * kBK, n0);
          if (DUAL) tma_load_2d(sa + kATile, &tmW, full_st, kbi * kBK, p.dual_rows + n0);
        }
      }
    }
  }
  // Everything above touched only this CTA's resources and static weights; wait here for the producing kernels
  // when launched with programmatic dependent launch (no-op otherwise).
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == 0) {
    if (lane == 0) {
      SegIter it(p, g, G);
      Seg s;
      // stage index and phase are carried (no division per K block): this loop and the MMA loop are on the
      // latency path of the pipeline
      int st = 0, issued = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok && it.next(s)) {
        const int n0 = (s.tile / p.m_tiles) * kBM;
        const int t0 = (s.tile % p.m_tiles) * p.BN;
        if (p.gate_flags != nullptr) {
          const int t_last = min(t0 + p.BN, p.M) - 1;
          const int want = ld_volatile(p.gate_flags + kReadyEpoch);
          for (int src = t0 / p.gate_rpr; src <= t_last / p.gate_rpr && src < p.gate_world; ++src)
            ok = ok && wait_flag_ge(p.gate_flags + kReady + src, want, p.err, 205);
          asm volatile("fence.proxy.async;" ::: "memory");  // TMA reads after the acquire
          if (!ok) { *abort_word = 205; break; }
        }
        for (int kbi = s.kb0; kbi < s.kb1; ++kbi) {
          uint8_t* sa = smem + st * stage_bytes;
          uint64_t* full_st = &tail->full[st];
          const int kc = kbi * kBK;
          if (issued < pre) {
            // armed, and its weight tile requested, before the wait
            ++issued;
            if (++st == p.stages) { st = 0; ph ^= 1; }
            tma_load_2d(sa + a_bytes, &tmX, full_st, kc, t0);
            continue;
          }
          ++issued;
          if (!mbar_wait(&tail->empty[st], ph ^ 1, abort_word, p.err, 201)) { ok = false; break; }
          mbar_arrive_expect_tx(full_st, stage_bytes);
          if (++st == p.stages) { st = 0; ph ^= 1; }
          if (p.packed_kb > 0) {
            tma_load_2d(sa, &tmW, full_st, 0, ((n0 >> 7) * p.packed_kb + kbi) << 7);
            if (DUAL)
              tma_load_2d(sa + kATile, &tmW, full_st, 0,
                          (((p.dual_rows + n0) >> 7) * p.packed_kb + kbi) << 7);
          } else {
            tma_load_2d(sa, &tmW, full_st, kc, n0);
            if (DUAL) tma_load_2d(sa + kATile, &tmW, full_st, kc, p.dual_rows + n0);
          }
          tma_load_2d(sa + a_bytes, &tmX, full_st, kc, t0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kBM, p.BN, 1, 1);
      SegIter it(p, g, G);
      Seg s;
      // descriptors advance by one stage per K block (the address field counts 16-byte units)
      const uint64_t da0_first = umma_desc_sw128(smem);
      const uint64_t d_a1 = static_cast<uint64_t>(kATile >> 4), d_b = static_cast<uint64_t>(a_bytes >> 4);
      const uint64_t d_stage = static_cast<uint64_t>(stage_bytes >> 4);
      uint64_t da0 = da0_first;
      int st = 0;
      uint32_t ph = 0;
      bool ok = true;
      while (ok && it.next(s)) {
        const int buf = s.idx % p.nbufs;
        const uint32_t bph = (s.idx / p.nbufs) & 1;
        if (!mbar_wait(&tail->tmem_empty[buf], bph ^ 1, abort_word, p.err, 202)) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + buf * p.acc_cols;
        for (int kbi = s.kb0; kbi < s.kb1; ++kbi) {
          if (!mbar_wait(&tail->full[st], ph, abort_word, p.err, 203)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint32_t accum = (kbi > s.kb0 || k > 0) ? 1u : 0u;
            const uint64_t koff = static_cast<uint64_t>(k * kUmmaK * 2 >> 4);
            umma_bf16(acc, da0 + koff, da0 + d_b + koff, idesc, accum);
            if (DUAL) umma_bf16(acc + p.BN, da0 + d_a1 + koff, da0 + d_b + koff, idesc, accum);
          }
          tc_commit(&tail->empty[st]);
          if (++st == p.stages) { st = 0; ph ^= 1; da0 = da0_first; } else { da0 += d_stage; }
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
      const int buf = s.idx % p.nbufs;
      const uint32_t bph = (s.idx / p.nbufs) & 1;
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
      if (p.dbg & 2) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tail->tmem_empty[buf]);
        continue;
      }
      float* mine = p.ws + (static_cast<size_t>(g) * 2 + s.slot) * slot_floats;
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
      const long long first_unit = static_cast<long long>(s.tile - p.tiles_dp) * p.kb;
      const int g_first = static_cast<int>(((first_unit + 1) * p.G2 - 1) / p.units2);
      const int g_last = static_cast<int>(((first_unit + p.kb) * p.G2 - 1) / p.units2);
      __threadfence();
      __syncwarp();
      int old = 0;
      if (lane == 0) old = atomicAdd(&p.counters[(s.tile - p.tiles_dp) * 4 + quad], 1);
      old = __shfl_sync(0xffffffffu, old, 0);
      if (old != g_last - g_first) continue;  // someone else finishes this tile
      if (p.dbg & 1) {
        if (lane == 0) p.counters[(s.tile - p.tiles_dp) * 4 + quad] = 0;
        continue;
      }
      __threadfence();
      // Vectorised reduction of this warp's 32 rows: a lane owns 4 consecutive rows (one float4
      // per partial) and the warp covers 4 tokens per step, 16 per unrolled iteration, so the
      // slots stream in with many independent 16-byte loads in flight.
      {
        const int rq = lane & 7;          // row quad inside the 32-row quadrant
        const int tsub = lane >> 3;       // token inside a 4-token step
        const int n = n_base + rq * 4;
        const int n_contrib = g_last - g_first + 1;
        const float* slots[8];
        int nc = n_contrib < 8 ? n_contrib : 8;
        for (int i = 0; i < nc; ++i) {
          const int gc = g_first + i;
          const long long b0 = p.units2 * gc / p.G2;
          slots[i] = p.ws + (static_cast<size_t>(gc) * 2 + (b0 >= first_unit ? 0 : 1)) * slot_floats +
                     quad * 32 + rq * 4;
        }
        int t_hi = p.M - t0;
        if (t_hi > p.BN) t_hi = p.BN;
        for (int tb = 0; tb < t_hi; tb += 16) {
          float4 acc[4], acc2[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            acc2[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          }
          for (int i = 0; i < n_contrib; ++i) {
            const float* src;
            if (i < 8) {
              src = slots[i];
            } else {
              const int gc = g_first + i;
              const long long b0 = p.units2 * gc / p.G2;
              src = p.ws + (static_cast<size_t>(gc) * 2 + (b0 >= first_unit ? 0 : 1)) * slot_floats +
                    quad * 32 + rq * 4;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int tl = tb + u * 4 + tsub;
              if (tl < t_hi) {
                const float4 x = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(tl) * kBM));
                acc[u].x += x.x; acc[u].y += x.y; acc[u].z += x.z; acc[u].w += x.w;
                if (DUAL) {
                  const float4 y = __ldcg(reinterpret_cast<const float4*>(src + static_cast<size_t>(p.BN + tl) * kBM));
                  acc2[u].x += y.x; acc2[u].y += y.y; acc2[u].z += y.z; acc2[u].w += y.w;
                }
              }
            }
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int tl = tb + u * 4 + tsub;
            const int t = t0 + tl;
            if (tl >= t_hi || n >= p.N) continue;
            float4 r = acc[u];
            if (DUAL) {
              r.x = silu_f(r.x) * acc2[u].x; r.y = silu_f(r.y) * acc2[u].y;
              r.z = silu_f(r.z) * acc2[u].z; r.w = silu_f(r.w) * acc2[u].w;
            }
            if (EPI == EPI_F32) {
              *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.Y) + static_cast<size_t>(t) * p.ldy + n) = r;
            } else {
              __nv_bfloat162 lo = __floats2bfloat162_rn(r.x, r.y), hi = __floats2bfloat162_rn(r.z, r.w);
              if (EPI == EPI_RESID) {
                const uint2 rv = *reinterpret_cast<const uint2*>(p.R + static_cast<size_t>(t) * p.ldr + n);
                const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&rv);
                float2 a = __bfloat1622float2(lo), b = __bfloat1622float2(rb[0]);
                lo = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
                a = __bfloat1622float2(hi); b = __bfloat1622float2(rb[1]);
                hi = __floats2bfloat162_rn(a.x + b.x, a.y + b.y);
              }
              uint2 o2;
              o2.x = *reinterpret_cast<uint32_t*>(&lo);
              o2.y = *reinterpret_cast<uint32_t*>(&hi);
              *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.Y) + static_cast<size_t>(t) * p.ldy + n) = o2;
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) p.counters[(s.tile - p.tiles_dp) * 4 + quad] = 0;  // ready for the next launch
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
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024) != cudaSuccess)
      return MB_ERR_LAUNCH;
    configured.done();
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
  return mb_gemm_bf16_persistent_gated(X, W, Y, R, M, N, K, ldx, ldw, ldy, ldr, flags, bn, stages, force_mode,
                                       ws, counters, err, num_sms, nullptr, 1, 0, stream);
}

// Same kernel with tensor-parallel gating of the token tiles (see Params::gate_flags).
extern "C" int mb_gemm_bf16_persistent_gated(const void* X, const void* W, void* Y, const void* R, int M,
                                             int N, int K, int ldx, int ldw, int ldy, int ldr, int flags,
                                             int bn, int stages, int force_mode, void* ws, int* counters,
                                             int* err, int num_sms, const int* gate_flags, int gate_rpr,
                                             int gate_world, cudaStream_t stream) {
  using namespace mb::pg;
  if (gate_flags != nullptr && (gate_rpr < 1 || gate_world < 1 || gate_world > mb::kMaxRanks)) return MB_ERR_SHAPE;
  if (M <= 0 || N <= 0) return MB_OK;
  const bool dual = flags & 1, resid = flags & 2, f32 = flags & 4, pdl = (flags & 8) || mb::pdl_enabled(), packed = flags & 64;
  if (packed && (K % kBK || N % kBM || ldw != K)) return MB_ERR_SHAPE;
  if (K % 8 || ldx % 8 || ldw % 8 || N % 8 || (!f32 && ldy % 8) || (resid && ldr % 8)) return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(Y) |
       reinterpret_cast<uintptr_t>(R)) & 15)
    return MB_ERR_ALIGN;
  if (dual && f32) return MB_ERR_SHAPE;
  if (num_sms <= 0) num_sms = 148;
  const int max_bn = 256;
  if (bn <= 0) {
    int mt = (M + max_bn - 1) / max_bn;
    if (dual) {
      // Token-tile count for the fused SwiGLU GEMM in whole-tile rounds: every CTA runs ceil(tiles / SMs)
      // tiles, and a tile of `b` tokens costs about (89 + b) units on B200 (fit to 61 us at b = 256 and
      // 55.5 us at b = 224 with K = 4096), so a slightly narrower tile wins when it saves nothing in rounds
      // but shortens each one (1024 tokens: 5 x 208 instead of 4 x 256, both four rounds on 148 SMs).
      const int n_t = (N + kBM - 1) / kBM;
      long best_cost = -1;
      int best_mt = mt;
      for (int c = mt; c <= mt + 2; ++c) {
        const int b = ((M + c - 1) / c + 15) / 16 * 16;
        const long rounds = (static_cast<long>(c) * n_t + num_sms - 1) / num_sms;
        const long cost = rounds * (89 + b);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_mt = c; }
      }
      mt = best_mt;
    }
    bn = ((M + mt - 1) / mt + 15) / 16 * 16;
  }
  if (bn % 16 || bn < 16 || bn > max_bn) return MB_ERR_SHAPE;
  Params p;
  p.gate_flags = gate_flags; p.gate_rpr = gate_rpr; p.gate_world = gate_world;
  p.packed_kb = packed ? K / kBK : 0;
  p.w_static = (flags & 128) ? 1 : 0;
  p.Y = Y; p.R = static_cast<const __nv_bfloat16*>(R);
  p.ws = static_cast<float*>(ws); p.counters = counters; p.err = err;
  p.M = M; p.N = N; p.K = K; p.ldy = ldy; p.ldr = ldr; p.dual_rows = N;
  p.BN = bn;
  p.acc_cols = bn * (dual ? 2 : 1);
  p.nbufs = 2 * p.acc_cols <= 512 ? 2 : 1;  // double-buffer the accumulators when TMEM allows
  p.tmem_cols = pow2_cols(p.nbufs * p.acc_cols);
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
  // Default schedule: whole tiles round robin (mode 0). The stream-K remainder (mode 2) and pure stream-K
  // (mode 1) measured slower on B200 for every Llama shape, small remainders included (M = 1024 SwiGLU:
  // 245 us in whole tiles, 365 us with the 4 left-over tiles cut stream-K), so they run only when forced.
  int mode = 0;
  p.dbg = force_mode >= 0 ? (force_mode >> 4) & 3 : 0;
  if (force_mode >= 0 && (force_mode & 15) <= 2) mode = force_mode & 15;
  // the workspace holds two 256-column fp32 slots per CTA: wider accumulators (SwiGLU with more than 128
  // tokens per tile) cannot take part in a stream-K fix-up
  const bool sk_ok = ws != nullptr && counters != nullptr && p.acc_cols <= 256;
  if (!sk_ok) mode = 0;
  int grid = num_sms;
  if (mode == 0) {
    p.tiles_dp = p.tiles;
  } else if (mode == 1) {
    p.tiles_dp = 0;
  } else {
    p.tiles_dp = p.tiles / num_sms * num_sms;
  }
  const int rest = p.tiles - p.tiles_dp;
  if (rest * 4 > static_cast<int>(mb_gemm_persistent_counter_ints(num_sms))) return MB_ERR_TOO_LARGE;
  p.units2 = static_cast<long long>(rest) * p.kb;
  long long g2 = p.units2 / 4;  // at least four K blocks per stream-K share
  if (g2 > num_sms) g2 = num_sms;
  if (rest > 0 && g2 < 1) g2 = 1;
  p.G2 = static_cast<int>(g2);
  if (p.tiles_dp == 0) grid = p.G2;
  else if (p.tiles < num_sms) grid = p.tiles;
  if (grid < 1) grid = 1;
  CUtensorMap tw, tx;
  int rc = packed ? cached_tmap(&tw, W, static_cast<uint64_t>(dual ? 2 * N : N) * p.packed_kb, kBK, kBK, kBM, 2)
                  : cached_tmap(&tw, W, dual ? 2 * N : N, K, ldw, kBM, 2);
  if (rc != MB_OK) return rc;
  rc = cached_tmap(&tx, X, M, K, ldx, bn, 2);
  if (rc != MB_OK) return rc;
  if (dual) return launch<true, EPI_BF16>(tw, tx, p, grid, pdl, stream);
  if (f32) return launch<false, EPI_F32>(tw, tx, p, grid, pdl, stream);
  if (resid) return launch<false, EPI_RESID>(tw, tx, p, grid, pdl, stream);
  return launch<false, EPI_BF16>(tw, tx, p, grid, pdl, stream);
}
