// Block-scaled fp8 (e4m3) GEMM for sm_100a and the matching activation quantiser.
//
//   Y[M, N] = (Xq ⊙ sx)[M, K] · (Wq ⊙ sw)[N, K]^T
//
//   Wq  e4m3 [N, K], sw fp32 [ceil(N/128), ceil(K/128)]   one scale per 128x128 weight block
//   Xq  e4m3 [M, K], sx fp32 [ceil(K/128), M]             one scale per token per 128-wide K group
//                                                          (stored K-group-major so that a tile's
//                                                          tokens are contiguous)
//
// tcgen05.mma kind::f8f6f4 accumulates 128 K (four K=32 instructions) into one of four TMEM
// buffers; two epilogue warpgroups then "promote" that partial: read it back with tcgen05.ld,
// multiply by sw * sx and add it into fp32 register accumulators while the tensor core already
// works on the next K groups in the other buffers. The combined scales of a K group are fetched
// one group ahead and staged per warp in shared memory, so no global load sits between the
// accumulator barrier and the promotion. Token counts that give fewer CTAs than SMs split K
// over grid.z: every split writes fp32 partials that a small kernel sums (and adds the residual). For decode-sized token counts the promotion
// hides completely under the weight stream; for large token counts it bounds the kernel at
// roughly the bf16 rate, which is the price of arbitrary (non power-of-two) fp32 scales.
//
// Warp roles (320 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 promote token
// columns [0, BN/2), warps 6-9 columns [BN/2, BN). Weights sit on the UMMA M side (128 rows),
// tokens on the N side (BN = 32..128, multiple of 32).
//
// Reference counterparts: max/kernels/src/linalg/matmul/gpu/sm100/
// warp_specialized_blockwise_fp8.mojo:898 (promote_accumulators :520) and
// linalg/fp8_quantization.mojo:369 (per-token-group dynamic quantisation).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "gemm_common.h"

namespace mb {
namespace f8 {

constexpr int kBM = 128;
constexpr int kBKBytes = 128;     // one swizzle row = 128 fp8 elements
constexpr int kThreads = 320;
constexpr int kATile = kBM * kBKBytes;
constexpr int kStgWarp = 16 * 32 * 2;

struct Params {
  __nv_bfloat16* Y;
  const __nv_bfloat16* R;
  const float* sw;
  const float* sx;
  int* err;
  int M, N, K, ldy, ldr, sw_ld, BN, stages;
  int splits, kb_per_split;
  float* partial;   // [splits, M, N] fp32 when splits > 1
  // grouped (mixture-of-experts) mode: blockIdx.x walks the token tiles of all experts in expert order
  // (expert e owns rows [offsets[e], offsets[e+1]) and ceil(rows / BN) tiles); weights / weight scales of
  // expert e start at row e * w_rows / e * sw_rows
  const int* expert_offsets;
  int w_rows, sw_rows, n_experts;
};

constexpr int kAccBufs = 4;

struct Tail {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t acc_full[kAccBufs];
  uint64_t acc_empty[kAccBufs];
  uint32_t tmem_base;
  int abort_word;
  alignas(16) float scales[8][2][64];   // per promotion warp, double-buffered: sw * sx of its token columns
};

template <bool RESID>
__global__ void __launch_bounds__(kThreads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int stage_bytes = kATile + p.BN * kBKBytes;
  uint8_t* stg_base = smem + p.stages * stage_bytes;
  Tail* tail = reinterpret_cast<Tail*>(stg_base + 8 * kStgWarp);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.y * kBM;
  int t0 = blockIdx.x * p.BN;
  int Mlim = p.M, w_row0 = 0, sw_row0 = 0, zsplit = blockIdx.z;
  if (p.expert_offsets != nullptr) {
    // every warp finds the expert of this CTA's tile: a prefix sum of the experts' tile counts, 32 experts
    // per round. The grid is sized for the worst case, so CTAs past the last tile leave here, before any
    // barrier or TMEM allocation.
    const int tile = blockIdx.x;
    int e = -1, row_end = 0, base = 0;
    for (int c = 0; c < p.n_experts; c += 32) {
      const int j = c + lane;
      const int b = j < p.n_experts ? p.expert_offsets[j] : 0;
      const int en = j < p.n_experts ? p.expert_offsets[j + 1] : 0;
      const int nt = (en - b + p.BN - 1) / p.BN;
      int incl = nt;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const int before = base + incl - nt;
      const unsigned hit = __ballot_sync(0xffffffffu, tile >= before && tile < before + nt);
      if (hit != 0) {
        const int src = __ffs(hit) - 1;
        e = c + src;
        row_end = __shfl_sync(0xffffffffu, en, src);
        t0 = __shfl_sync(0xffffffffu, b, src) + (tile - __shfl_sync(0xffffffffu, before, src)) * p.BN;
        break;
      }
      base += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (e < 0) return;
    Mlim = row_end;
    w_row0 = e * p.w_rows;
    sw_row0 = e * p.sw_rows;
    zsplit = 0;
  }
  const int kb_all = (p.K + 127) / 128;
  const int kb_begin = zsplit * p.kb_per_split;
  const int kb_end = kb_begin + p.kb_per_split < kb_all ? kb_begin + p.kb_per_split : kb_all;
  const int kb_total = kb_end - kb_begin;          // K groups of this split
  const uint32_t want_cols = p.BN * kAccBufs;
  const uint32_t tmem_cols = want_cols <= 128 ? 128 : (want_cols <= 256 ? 256 : 512);

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&tail->full[s], 1);
      mbar_init(&tail->empty[s], 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      mbar_init(&tail->acc_full[b], 1);
      mbar_init(&tail->acc_empty[b], 8);
    }
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
    if (lane == 0) {
      int s = 0;       // stage and phase are carried: no division on the pipeline's latency path
      uint32_t ph = 0;
      for (int kb = 0; kb < kb_total; ++kb, s = (s + 1 == p.stages ? 0 : s + 1), ph ^= (s == 0)) {
        if (!mbar_wait(&tail->empty[s], ph ^ 1, abort_word, p.err, 501)) break;
        uint8_t* sa = smem + s * stage_bytes;
        mbar_arrive_expect_tx(&tail->full[s], stage_bytes);
        tma_load_2d(sa, &tmW, &tail->full[s], (kb_begin + kb) * 128, w_row0 + n0);
        tma_load_2d(sa + kATile, &tmX, &tail->full[s], (kb_begin + kb) * 128, t0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(kBM, p.BN, 0, 0);  // e4m3 x e4m3 -> fp32
      int s = 0;
      uint32_t ph = 0;
      for (int kb = 0; kb < kb_total; ++kb, s = (s + 1 == p.stages ? 0 : s + 1), ph ^= (s == 0)) {
        const int buf = kb % kAccBufs;
        const uint32_t bph = (kb / kAccBufs) & 1;
        if (!mbar_wait(&tail->acc_empty[buf], bph ^ 1, abort_word, p.err, 502)) break;
        if (!mbar_wait(&tail->full[s], ph, abort_word, p.err, 503)) break;
        tc_fence_after();
        uint8_t* sa = smem + s * stage_bytes;
        const uint64_t da = umma_desc_sw128(sa);
        const uint64_t db = umma_desc_sw128(sa + kATile);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t koff = static_cast<uint64_t>(k * 32 >> 4);  // 32 bytes per K=32 step
          umma_fp8(tmem_base + buf * p.BN, da + koff, db + koff, idesc, k > 0 ? 1u : 0u);
        }
        tc_commit(&tail->empty[s]);
        tc_commit(&tail->acc_full[buf]);
      }
    }
  } else {
    // ---------------------------------------------------------------- promotion + epilogue
    const int ew = warp - 2;            // 0..7
    const int quad = warp & 3;          // TMEM lane quadrant
    const int half = ew >> 2;           // which half of the token columns
    const int cols = p.BN >> 1;         // columns handled by this warpgroup (multiple of 16)
    const int c_base = half * cols;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] = 0.f;
    const float* sw_row = p.sw + static_cast<size_t>(sw_row0 + blockIdx.y) * p.sw_ld + kb_begin;
    const float* sx_base = p.sx + static_cast<size_t>(kb_begin) * p.M + t0 + c_base;
    float* sc = &tail->scales[ew][0][0];
    // lane l owns the scales of token columns l and l + 32 of this warpgroup's half
    const bool in0 = lane < cols && t0 + c_base + lane < Mlim;
    const bool in1 = lane + 32 < cols && t0 + c_base + lane + 32 < Mlim;
    float s0 = 0.f, s1 = 0.f;
    if (kb_total > 0) {
      const float w = sw_row[0];
      s0 = in0 ? sx_base[lane] * w : 0.f;
      s1 = in1 ? sx_base[lane + 32] * w : 0.f;
    }
    sc[lane] = s0;
    sc[lane + 32] = s1;
    __syncwarp();
    bool ok = true;
    for (int kb = 0; kb < kb_total && ok; ++kb) {
      const int buf = kb % kAccBufs;
      const uint32_t bph = (kb / kAccBufs) & 1;
      // next group's scales: in flight while this group's accumulator is awaited and promoted
      if (kb + 1 < kb_total) {
        const float w = sw_row[kb + 1];
        const float* sx_row = sx_base + static_cast<size_t>(kb + 1) * p.M;
        s0 = in0 ? sx_row[lane] * w : 0.f;
        s1 = in1 ? sx_row[lane + 32] * w : 0.f;
      }
      ok = mbar_wait(&tail->acc_full[buf], bph, abort_word, p.err, 504);
      if (!ok) break;
      tc_fence_after();
      const float* scur = sc + (kb & 1) * 64;
#pragma unroll
      for (int c = 0; c < 64; c += 16) {
        if (c < cols) {
          uint32_t v[16];
          tmem_ld_32x16(lane_addr + buf * p.BN + c_base + c, v);
          float4 sv[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) sv[q] = *reinterpret_cast<const float4*>(scur + c + q * 4);
          tc_wait_ld();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            acc[c + q * 4 + 0] = fmaf(__uint_as_float(v[q * 4 + 0]), sv[q].x, acc[c + q * 4 + 0]);
            acc[c + q * 4 + 1] = fmaf(__uint_as_float(v[q * 4 + 1]), sv[q].y, acc[c + q * 4 + 1]);
            acc[c + q * 4 + 2] = fmaf(__uint_as_float(v[q * 4 + 2]), sv[q].z, acc[c + q * 4 + 2]);
            acc[c + q * 4 + 3] = fmaf(__uint_as_float(v[q * 4 + 3]), sv[q].w, acc[c + q * 4 + 3]);
          }
        }
      }
      tc_fence_before();
      float* snext = sc + ((kb + 1) & 1) * 64;
      snext[lane] = s0;
      snext[lane + 32] = s1;
      __syncwarp();
      if (lane == 0) mbar_arrive(&tail->acc_empty[buf]);
    }
    if (ok && p.splits > 1) {
      // fp32 partials of this split: lane = weight row, so each token's 32 floats are contiguous
      const int n = n0 + quad * 32 + lane;
      float* dst = p.partial + static_cast<size_t>(zsplit) * p.M * p.N;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        const int t = t0 + c_base + c;
        if (c < cols && t < Mlim && n < p.N) dst[static_cast<size_t>(t) * p.N + n] = acc[c];
      }
      ok = false;   // nothing left for the bf16 epilogue
    }
    if (ok) {
      __nv_bfloat16* stg = reinterpret_cast<__nv_bfloat16*>(stg_base + ew * kStgWarp);
      const int n_base = n0 + quad * 32;
#pragma unroll
      for (int c = 0; c < 64; c += 16) {
        if (c < cols && t0 + c_base + c < Mlim) {
#pragma unroll
          for (int j = 0; j < 16; ++j) stg[j * 32 + lane] = __float2bfloat16(acc[c + j]);
          __syncwarp();
#pragma unroll
          for (int pass = 0; pass < 2; ++pass) {
            const int j = pass * 8 + (lane >> 2);
            const int seg = lane & 3;
            const int t = t0 + c_base + c + j;
            const int n = n_base + seg * 8;
            if (t < Mlim && n < p.N) {
              uint4 val = *reinterpret_cast<const uint4*>(stg + j * 32 + seg * 8);
              if (RESID) {
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
              *reinterpret_cast<uint4*>(p.Y + static_cast<size_t>(t) * p.ldy + n) = val;
            }
          }
          __syncwarp();
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

// Sum of the split-K partials [splits, M, N] (+ residual) -> bf16 Y; N % 4 == 0.
__global__ void fp8_splitk_reduce_kernel(const float* __restrict__ part, const __nv_bfloat16* __restrict__ R,
                                         __nv_bfloat16* __restrict__ Y, int M, int N, int splits) {
  const size_t idx = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  const size_t total = static_cast<size_t>(M) * N;
  if (idx >= total) return;
  float4 a = *reinterpret_cast<const float4*>(part + idx);
  for (int s = 1; s < splits; ++s) {
    const float4 b = *reinterpret_cast<const float4*>(part + s * total + idx);
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
  }
  if (R != nullptr) {
    const uint2 rv = *reinterpret_cast<const uint2*>(R + idx);
    const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&rv);
    const float2 r0 = __bfloat1622float2(rb[0]), r1 = __bfloat1622float2(rb[1]);
    a.x += r0.x; a.y += r0.y; a.z += r1.x; a.w += r1.y;
  }
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a.x, a.y), hi = __floats2bfloat162_rn(a.z, a.w);
  uint2 out;
  out.x = *reinterpret_cast<const uint32_t*>(&lo);
  out.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(Y + idx) = out;
}

// One warp per (token, 128-wide K group): amax -> scale = amax / 448, q = x / scale.
__global__ void quant_fp8_group128_kernel(const __nv_bfloat16* __restrict__ x, uint8_t* __restrict__ q,
                                          float* __restrict__ scales, int M, int K, int ldx,
                                          int k_major) {
  const int groups = (K + 127) / 128;
  const long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (wid >= static_cast<long long>(M) * groups) return;
  const int t = static_cast<int>(wid / groups), g = static_cast<int>(wid % groups);
  const int k0 = g * 128 + lane * 4;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (k0 < K) {
    const uint2 raw = *reinterpret_cast<const uint2*>(x + static_cast<size_t>(t) * ldx + k0);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&raw);
    const float2 a = __bfloat1622float2(b[0]), c = __bfloat1622float2(b[1]);
    v[0] = a.x; v[1] = a.y; v[2] = c.x; v[3] = c.y;
  }
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-12f) / 448.0f;
  const float inv = 1.0f / scale;
  if (k0 < K) {
    const __nv_fp8x4_e4m3 packed(make_float4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv));
    *reinterpret_cast<uint32_t*>(q + static_cast<size_t>(t) * K + k0) = packed.__x;
  }
  if (lane == 0) scales[k_major ? static_cast<size_t>(g) * M + t : static_cast<size_t>(t) * groups + g] = scale;
}

// SwiGLU and the 1x128 quantisation of its result in one pass: gu [M, 2I] bf16 (gate | up) -> q [M, I] e4m3
// and scales [I/128, ld_s] (group-major). The product is rounded to bf16 first, so the result equals the
// two-pass form bit for bit. Rows at or past *n_rows_dev (when given) are skipped: grouped GEMMs whose row
// count is only known on the device pay for the rows that exist. One warp per (row, group), grid-stride.
__global__ void silu_mul_quant_fp8_kernel(const __nv_bfloat16* __restrict__ gu, uint8_t* __restrict__ q,
                                          float* __restrict__ scales, int M, int I, int ld_s,
                                          const int32_t* __restrict__ n_rows_dev) {
  const int rows = n_rows_dev != nullptr ? min(M, *n_rows_dev) : M;
  const int groups = I >> 7;
  const long long total = static_cast<long long>(rows) * groups;
  const long long stride = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (long long wid = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; wid < total;
       wid += stride) {
    const int t = static_cast<int>(wid / groups), g = static_cast<int>(wid % groups);
    const int k0 = g * 128 + lane * 4;
    const __nv_bfloat16* row = gu + static_cast<size_t>(t) * 2 * I;
    const uint2 graw = *reinterpret_cast<const uint2*>(row + k0);
    const uint2 uraw = *reinterpret_cast<const uint2*>(row + I + k0);
    const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&graw);
    const __nv_bfloat162* ub = reinterpret_cast<const __nv_bfloat162*>(&uraw);
    const float2 g0 = __bfloat1622float2(gb[0]), g1 = __bfloat1622float2(gb[1]);
    const float2 u0 = __bfloat1622float2(ub[0]), u1 = __bfloat1622float2(ub[1]);
    float v[4] = {g0.x / (1.f + __expf(-g0.x)) * u0.x, g0.y / (1.f + __expf(-g0.y)) * u0.y,
                  g1.x / (1.f + __expf(-g1.x)) * u1.x, g1.y / (1.f + __expf(-g1.y)) * u1.y};
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __bfloat162float(__float2bfloat16_rn(v[j]));
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = fmaxf(amax, 1e-12f) / 448.0f;
    const float inv = 1.0f / scale;
    const __nv_fp8x4_e4m3 packed(make_float4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv));
    *reinterpret_cast<uint32_t*>(q + static_cast<size_t>(t) * I + k0) = packed.__x;
    if (lane == 0) scales[static_cast<size_t>(g) * ld_s + t] = scale;
  }
}

// The inverse of the 1x128 quantisation: q [M, K] e4m3 with group-major scales [K/128, ld_s] -> bf16 [M, K].
// Rows at or past *n_rows_dev (when given) are skipped.
__global__ void dequant_fp8_group128_kernel(const uint8_t* __restrict__ q, const float* __restrict__ scales,
                                            __nv_bfloat16* __restrict__ out, int M, int K, int ld_s,
                                            const int32_t* __restrict__ n_rows_dev) {
  const int rows = n_rows_dev != nullptr ? min(M, *n_rows_dev) : M;
  const int per_row = K >> 2;
  const long long total = static_cast<long long>(rows) * per_row;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int r = static_cast<int>(i / per_row), c = static_cast<int>(i % per_row) * 4;
    const float scale = scales[static_cast<size_t>(c >> 7) * ld_s + r];
    __nv_fp8x4_e4m3 v;
    v.__x = *reinterpret_cast<const uint32_t*>(q + static_cast<size_t>(r) * K + c);
    const float4 f = static_cast<float4>(v);
    const __nv_bfloat162 lo = __floats2bfloat162_rn(f.x * scale, f.y * scale);
    const __nv_bfloat162 hi = __floats2bfloat162_rn(f.z * scale, f.w * scale);
    uint2 o;
    o.x = *reinterpret_cast<const uint32_t*>(&lo);
    o.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(r) * K + c) = o;
  }
}

}  // namespace f8
}  // namespace mb

using namespace mb;

extern "C" int mb_dequant_fp8_group128(const void* q_fp8, const float* scales, void* out_bf16, int M, int K, int ld_s,
                                       const int32_t* n_rows_dev, cudaStream_t stream) {
  if (M <= 0) return MB_OK;
  if (K % 128 || ld_s < M) return MB_ERR_SHAPE;
  long long blocks = (static_cast<long long>(M) * (K / 4) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  f8::dequant_fp8_group128_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const uint8_t*>(q_fp8), scales, static_cast<__nv_bfloat16*>(out_bf16), M, K, ld_s, n_rows_dev);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_silu_mul_quant_fp8(const void* gate_up, void* q_fp8, float* scales, int M, int inter, int ld_s,
                                     const int32_t* n_rows_dev, cudaStream_t stream) {
  if (M <= 0) return MB_OK;
  if (inter % 128 || ld_s < M) return MB_ERR_SHAPE;
  const long long warps = static_cast<long long>(M) * (inter / 128);
  long long blocks = (warps + 7) / 8;
  if (blocks > 148 * 16) blocks = 148 * 16;
  f8::silu_mul_quant_fp8_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gate_up), static_cast<uint8_t*>(q_fp8), scales, M, inter, ld_s, n_rows_dev);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_quant_fp8_group128(const void* x_bf16, void* q_fp8, float* scales, int M, int K,
                                     int ldx, int scale_ld, int scales_k_major, cudaStream_t stream) {
  (void)scale_ld;
  if (M <= 0) return MB_OK;
  if (K % 4 || ldx % 4) return MB_ERR_SHAPE;
  const long long warps = static_cast<long long>(M) * ((K + 127) / 128);
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  f8::quant_fp8_group128_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x_bf16), static_cast<uint8_t*>(q_fp8), scales, M, K, ldx,
      scales_k_major);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

// Number of K splits for a grid of `ctas` output tiles: the split count (<= 8, at least four K groups
// each) that fills whole waves of SMs best, with a small bias towards fewer splits.
static int fp8_pick_splits(int ctas, int kb_total, int num_sms) {
  if (ctas >= num_sms || num_sms <= 0) return 1;
  int best = 1;
  float best_score = -1.f;
  for (int s = 1; s <= 8 && kb_total / s >= 4; ++s) {
    const int total = ctas * s;
    const int waves = (total + num_sms - 1) / num_sms;
    const float score = static_cast<float>(total) / (waves * num_sms) - 0.02f * s;
    if (score > best_score) { best_score = score; best = s; }
  }
  return best;
}

// flags: bit1 residual add. Xs is K-group-major [ceil(K/128), M]; Ws is [ceil(N/128), ceil(K/128)].
// splits <= 0: chosen here (1 without a workspace of splits*M*N floats); num_sms is used for that choice.
extern "C" int mb_gemm_fp8_blockscaled(const void* Xq, const float* Xs, const void* Wq, const float* Ws,
                                       void* Y, const void* R, int M, int N, int K, int flags, int bn,
                                       int stages, int splits, void* workspace, size_t workspace_bytes,
                                       int num_sms, int* err, cudaStream_t stream) {
  using namespace mb::f8;
  if (M <= 0 || N <= 0) return MB_OK;
  if (K % 16 || N % 8) return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(Xq) | reinterpret_cast<uintptr_t>(Wq) | reinterpret_cast<uintptr_t>(Y) |
       reinterpret_cast<uintptr_t>(R)) & 15)
    return MB_ERR_ALIGN;
  if (bn <= 0) {
    const int mt = (M + 127) / 128;
    bn = ((M + mt - 1) / mt + 31) / 32 * 32;
  }
  if (bn % 32 || bn < 32 || bn > 128) return MB_ERR_SHAPE;
  Params p;
  p.Y = static_cast<__nv_bfloat16*>(Y);
  p.R = static_cast<const __nv_bfloat16*>(R);
  p.sw = Ws; p.sx = Xs; p.err = err;
  p.M = M; p.N = N; p.K = K; p.ldy = N; p.ldr = N; p.sw_ld = (K + 127) / 128; p.BN = bn;
  const int stage_bytes = kATile + bn * kBKBytes;
  const int max_stages = (227 * 1024 - 1024 - 8 * kStgWarp - static_cast<int>(sizeof(Tail)) - 256) / stage_bytes;
  if (stages <= 0 || stages > max_stages) stages = max_stages;
  if (stages > 8) stages = 8;
  p.stages = stages;
  CUtensorMap tw, tx;
  int rc = cached_tmap(&tw, Wq, N, K, K, kBM, 1);
  if (rc != MB_OK) return rc;
  rc = cached_tmap(&tx, Xq, M, K, K, bn, 1);
  if (rc != MB_OK) return rc;
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + 8 * kStgWarp + sizeof(Tail) + 1024;
  const int kb_all = (K + 127) / 128;
  const int tiles = ((M + bn - 1) / bn) * ((N + kBM - 1) / kBM);
  if (splits <= 0) splits = fp8_pick_splits(tiles, kb_all, num_sms);
  if (splits > kb_all) splits = kb_all;
  if (workspace == nullptr || N % 4 ||
      static_cast<size_t>(splits) * M * N * sizeof(float) > workspace_bytes)
    splits = 1;
  p.kb_per_split = (kb_all + splits - 1) / splits;
  splits = (kb_all + p.kb_per_split - 1) / p.kb_per_split;
  p.splits = splits;
  p.partial = static_cast<float*>(workspace);
  p.expert_offsets = nullptr; p.w_rows = 0; p.sw_rows = 0; p.n_experts = 0;
  dim3 grid((M + bn - 1) / bn, (N + kBM - 1) / kBM, splits);
  const bool resid = (flags & 2) && splits == 1;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    cudaFuncSetAttribute(gemm_fp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    cudaFuncSetAttribute(gemm_fp8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    configured.done();
  }
  if (resid)
    gemm_fp8_kernel<true><<<grid, kThreads, smem, stream>>>(tw, tx, p);
  else
    gemm_fp8_kernel<false><<<grid, kThreads, smem, stream>>>(tw, tx, p);
  if (splits > 1) {
    const size_t total4 = static_cast<size_t>(M) * N / 4;
    fp8_splitk_reduce_kernel<<<static_cast<unsigned>((total4 + 255) / 256), 256, 0, stream>>>(
        p.partial, (flags & 2) ? p.R : nullptr, p.Y, M, N, splits);
  }
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

// Grouped block-scaled fp8 GEMM for mixture-of-experts layers: rows [offsets[e], offsets[e+1]) of Xq
// (tokens in expert order, scales Xs K-group-major over all `total_rows`) times expert e's weights
// Wq[e] ([N, K] e4m3 with 128x128 block scales Ws[e]). N % 128 == 0. `max_rows` bounds the rows of any
// expert (the grid is sized for it; CTAs past an expert's rows exit at once). `ldx` = byte stride of
// Xq rows (0 = K).
// Reference: max/python/max/nn/moe/moe_fp8.py:48 (MoEQuantized, fp8-blockwise strategy) over
// max/kernels/src/linalg/grouped_matmul_sm100_blockwise_fp8.mojo.
extern "C" int mb_grouped_gemm_fp8_blockscaled(const void* Xq, const float* Xs, const void* Wq, const float* Ws,
                                               void* Y, const int32_t* expert_offsets, int n_experts,
                                               int total_rows, int max_rows, int N, int K, int ldx, int bn,
                                               int stages, int* err, cudaStream_t stream) {
  using namespace mb::f8;
  if (total_rows <= 0 || N <= 0 || n_experts <= 0) return MB_OK;
  if (ldx <= 0) ldx = K;            // row stride of Xq in bytes (rows may carry trailing scale bytes)
  if (K % 16 || N % 128 || ldx % 16 || ldx < K) return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(Xq) | reinterpret_cast<uintptr_t>(Wq) | reinterpret_cast<uintptr_t>(Y)) & 15)
    return MB_ERR_ALIGN;
  if (max_rows <= 0 || max_rows > total_rows) max_rows = total_rows;
  if (bn <= 0) {
    // expected rows per expert decide the token tile: small tiles when experts see few tokens
    const int avg = (total_rows + n_experts - 1) / n_experts;
    bn = avg <= 32 ? 32 : (avg <= 64 ? 64 : 128);
  }
  if (bn % 32 || bn < 32 || bn > 128) return MB_ERR_SHAPE;
  Params p;
  p.Y = static_cast<__nv_bfloat16*>(Y);
  p.R = nullptr;
  p.sw = Ws; p.sx = Xs; p.err = err;
  p.M = total_rows; p.N = N; p.K = K; p.ldy = N; p.ldr = N; p.sw_ld = (K + 127) / 128; p.BN = bn;
  const int stage_bytes = kATile + bn * kBKBytes;
  const int max_stages = (227 * 1024 - 1024 - 8 * kStgWarp - static_cast<int>(sizeof(Tail)) - 256) / stage_bytes;
  if (stages <= 0 || stages > max_stages) stages = max_stages;
  if (stages > 8) stages = 8;
  p.stages = stages;
  p.splits = 1;
  p.kb_per_split = (K + 127) / 128;
  p.partial = nullptr;
  p.expert_offsets = expert_offsets;
  p.n_experts = n_experts;
  p.w_rows = N;
  p.sw_rows = N / 128;
  CUtensorMap tw, tx;
  int rc = cached_tmap(&tw, Wq, static_cast<uint64_t>(n_experts) * N, K, K, kBM, 1);
  if (rc != MB_OK) return rc;
  rc = cached_tmap(&tx, Xq, total_rows, K, ldx, bn, 1);
  if (rc != MB_OK) return rc;
  const size_t smem = static_cast<size_t>(stages) * stage_bytes + 8 * kStgWarp + sizeof(Tail) + 1024;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    cudaFuncSetAttribute(gemm_fp8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    configured.done();
  }
  // an upper bound of the number of token tiles: every expert wastes less than one tile, and no expert has
  // more than max_rows rows
  long long tiles = (total_rows + bn - 1) / bn + n_experts;
  const long long by_expert = static_cast<long long>(n_experts) * ((max_rows + bn - 1) / bn);
  if (by_expert < tiles) tiles = by_expert;
  dim3 grid(static_cast<unsigned>(tiles), N / kBM, 1);
  gemm_fp8_kernel<false><<<grid, kThreads, smem, stream>>>(tw, tx, p);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}
