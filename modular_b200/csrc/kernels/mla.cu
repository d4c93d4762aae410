// Multi-head latent attention (DeepSeek-V2/V3) in the absorbed form, over a paged latent cache.
//
// Every token has ONE cached row  [c_kv (R values) | k_rope (64 values)]  shared by all heads.
// Queries arrive already multiplied by W_uk:  q_lat [T, h, R]  and  q_rope [T, h, 64].
//     S[t, head, j] = (q_lat . c_kv[j] + q_rope . k_rope[j]) * scale          (causal)
//     out[t, head]  = softmax(S) . c_kv                                         -> [T, h, R]
// This is multi-query attention with key width R + 64 and value width R, where the values are
// the first R columns of the keys: one shared-memory tile serves both GEMMs.
//
// One CTA (8 warps) owns 64 query rows = (64 / HB tokens) x (HB heads) of one sequence and walks
// the sequence's KV pages 64 tokens at a time (cp.async double buffer, XOR-swizzled rows,
// ldmatrix + mma.sync m16n8k16, online softmax in fp32). Warps 0-3 and 4-7 hold the same four
// 16-row blocks but different halves of the R output columns, so the fp32 output accumulator
// (16 x R/2 per warp) fits in registers for R = 512; both halves compute the (cheap) score
// tile. Decode and prefill share the kernel; tiles are located from q_start/q_len on the device,
// so no host-side plan is needed.
//
// Reference counterparts: max/kernels/src/nn/mla.mojo (flare_mla_decoding / flare_mla_prefill),
// max/python/max/nn/attention/multi_latent_attention.py.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/launch.h"

namespace mb {
namespace mla {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;
constexpr int DR = 64;  // rotary part of the key

struct Params {
  const bf16* q_lat;   // [T, h, R]
  const bf16* q_rope;  // [T, h, DR]
  bf16* out;           // [T, h, R]
  const bf16* cache;   // page p, slot s at cache + p * page_stride + s * (R + DR)
  const int32_t* block_table;
  const int32_t* q_start;
  const int32_t* q_len;
  const int32_t* kv_len;
  int64_t page_stride;
  int B, bt_stride, n_heads, HB, page_size;
  float scale_log2;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(sz)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// element offset of 16-byte chunk `chunk` of row `row` in a [rows][LD] tile, chunks XOR-swizzled
template <int LD>
__device__ __forceinline__ int swz(int row, int chunk) {
  return row * LD + ((chunk ^ (row & 7)) << 3);
}

template <int R>
__device__ __forceinline__ void load_kv_tile(bf16* sK, const Params& p, const int32_t* bt, int kv0,
                                             int kv_end, int tid) {
  constexpr int LD = R + DR, CH = LD / 8;
  for (int idx = tid; idx < 64 * CH; idx += 256) {
    const int row = idx / CH, chunk = idx % CH;
    const int tok = kv0 + row;
    const bool valid = tok < kv_end;
    const int pg = valid ? bt[tok / p.page_size] : 0;
    const int off = valid ? tok % p.page_size : 0;
    const bf16* src = p.cache + static_cast<int64_t>(pg) * p.page_stride + static_cast<int64_t>(off) * LD + chunk * 8;
    cp_async16(sK + swz<LD>(row, chunk), src, valid);
  }
}

template <int R>
__global__ void __launch_bounds__(256, 1) mla_kernel(const Params p) {
  constexpr int LD = R + DR, CH = LD / 8, KS = LD / 16;
  constexpr int HALF = R / 2, DT = HALF / 8;  // output columns / n-tiles per warp
  extern __shared__ __align__(128) uint8_t smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);  // [64][LD]
  bf16* sK = sQ + 64 * LD;                       // [2][64][LD]
  __shared__ int s_seq, s_tq0;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tokens_per_tile = 64 / p.HB;

  // locate this CTA's (sequence, first query token): tiles are enumerated sequence by sequence
  if (tid == 0) {
    int acc = 0, seq = -1, tq0 = 0;
    for (int b = 0; b < p.B; ++b) {
      const int nt = (p.q_len[b] + tokens_per_tile - 1) / tokens_per_tile;
      if (static_cast<int>(blockIdx.x) < acc + nt) { seq = b; tq0 = (blockIdx.x - acc) * tokens_per_tile; break; }
      acc += nt;
    }
    s_seq = seq; s_tq0 = tq0;
  }
  __syncthreads();
  const int seq = s_seq, tq0 = s_tq0;
  if (seq < 0) return;
  const int head0 = blockIdx.y * p.HB;
  const int qs = p.q_start[seq], ql = p.q_len[seq], kl = p.kv_len[seq];
  const int32_t* bt = p.block_table + static_cast<int64_t>(seq) * p.bt_stride;

  for (int idx = tid; idx < 64 * CH; idx += 256) {
    const int row = idx / CH, chunk = idx % CH;
    const int tq = tq0 + row / p.HB, head = head0 + row % p.HB;
    const bool valid = tq < ql;
    const int64_t tok = qs + (valid ? tq : 0);
    const bf16* src = chunk < R / 8
                          ? p.q_lat + (tok * p.n_heads + head) * R + chunk * 8
                          : p.q_rope + (tok * p.n_heads + head) * DR + (chunk - R / 8) * 8;
    cp_async16(sQ + swz<LD>(row, chunk), src, valid);
  }
  int last_tq = tq0 + tokens_per_tile;
  if (last_tq > ql) last_tq = ql;
  const int kv_hi = kl - ql + last_tq;  // exclusive bound of the KV positions any row here may see
  const int ntiles = (kv_hi + 63) / 64;
  load_kv_tile<R>(sK, p, bt, 0, kv_hi, tid);
  cp_async_commit();
  cp_async_wait_all();
  __syncthreads();

  const int rb = warp & 3;        // 16-row block
  const int chalf = warp >> 2;    // which half of the output columns
  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  int limit[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = rb * 16 + (lane >> 2) + h * 8;
    const int tq = tq0 + r / p.HB;
    limit[h] = tq < ql ? kl - ql + tq : -1;
  }

  for (int it = 0; it < ntiles; ++it) {
    const int buf = it & 1;
    if (it + 1 < ntiles) {
      load_kv_tile<R>(sK + (buf ^ 1) * 64 * LD, p, bt, (it + 1) * 64, kv_hi, tid);
      cp_async_commit();
    }
    const bf16* tK = sK + buf * 64 * LD;
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll 4
    for (int ks = 0; ks < KS; ++ks) {
      uint32_t qf[4];
      ldsm_x4(qf, sQ + swz<LD>(rb * 16 + (lane & 15), 2 * ks + (lane >> 4)));
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        const int mi = lane >> 3;
        ldsm_x4(b, tK + swz<LD>(np * 16 + (mi >> 1) * 8 + (lane & 7), 2 * ks + (mi & 1)));
        mma_bf16(s[2 * np], qf, b[0], b[1]);
        mma_bf16(s[2 * np + 1], qf, b[2], b[3]);
      }
    }
    const int kv0 = it * 64;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = kv0 + nt * 8 + 2 * (lane & 3) + (e & 1);
        const int h = e >> 1;
        const float v = col <= limit[h] ? s[nt][e] * p.scale_log2 : -INFINITY;
        s[nt][e] = v;
        mx[h] = fmaxf(mx[h], v);
      }
    }
    float alpha[2], msafe[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float mn = fmaxf(m[h], mx[h]);
      msafe[h] = mn == -INFINITY ? 0.f : mn;
      alpha[h] = exp2f(m[h] - msafe[h]);
      m[h] = mn;
      l[h] *= alpha[h];
    }
#pragma unroll
    for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = exp2f(s[nt][e] - msafe[e >> 1]);
        s[nt][e] = pv;
        l[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) {
      o[dt][0] *= alpha[0]; o[dt][1] *= alpha[0];
      o[dt][2] *= alpha[1]; o[dt][3] *= alpha[1];
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dp = 0; dp < DT / 2; ++dp) {
        uint32_t b[4];
        const int mi = lane >> 3;
        // values = the first R columns of the key tile; this warp's half starts at chunk chalf*HALF/8
        ldsm_x4_t(b, tK + swz<LD>(kk * 16 + (mi & 1) * 8 + (lane & 7), chalf * (HALF / 8) + 2 * dp + (mi >> 1)));
        mma_bf16(o[2 * dp], a, b[0], b[1]);
        mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
      }
    }
    cp_async_wait_all();
    __syncthreads();
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
    const int r = rb * 16 + (lane >> 2) + h * 8;
    const int tq = tq0 + r / p.HB, head = head0 + r % p.HB;
    if (tq < ql) {
      bf16* orow = p.out + (static_cast<int64_t>(qs + tq) * p.n_heads + head) * R + chalf * HALF + 2 * (lane & 3);
#pragma unroll
      for (int dt = 0; dt < DT; ++dt)
        *reinterpret_cast<uint32_t*>(orow + dt * 8) = pack_bf16(o[dt][2 * h] * inv, o[dt][2 * h + 1] * inv);
    }
  }
}

// cache[slot] = [c_kv | k_rope]; one warp per token, 16-byte copies
__global__ void mla_kv_store_kernel(const bf16* __restrict__ c_kv, const bf16* __restrict__ k_rope,
                                    const int64_t* __restrict__ slots, bf16* __restrict__ cache, int T, int R,
                                    int ld_c, int ld_r, int page_size, int64_t page_stride) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int64_t slot = slots[t];
  if (slot < 0) return;
  const int LD = R + DR;
  bf16* dst = cache + (slot / page_size) * page_stride + (slot % page_size) * LD;
  for (int c = threadIdx.x & 31; c < LD / 8; c += 32) {
    const bf16* src = c < R / 8 ? c_kv + static_cast<int64_t>(t) * ld_c + c * 8
                                : k_rope + static_cast<int64_t>(t) * ld_r + (c - R / 8) * 8;
    *reinterpret_cast<uint4*>(dst + c * 8) = *reinterpret_cast<const uint4*>(src);
  }
}

// What follows the two down-projections of an MLA layer, in one pass over the fused projection output
// qkv_a[t] = [q_a (QL) | c_kv (R) | k_rope (64)]:
//   q_a_out[t] = rms_norm(q_a) * gamma_q              (input of the q_b projection; skipped when QL == 0)
//   cache[slot[t]] = [rms_norm(c_kv) * gamma_kv | rope(k_rope, position[t])]   (interleaved pairs)
// One CTA of 256 threads per token. The norm rounds to bf16 before the weight is applied, like rmsnorm_kernel.
__device__ __forceinline__ float block_sum_256(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = threadIdx.x < (blockDim.x >> 5) ? scratch[threadIdx.x] : 0.f;
  if (threadIdx.x < 32) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) scratch[0] = t;
  }
  __syncthreads();
  return scratch[0];
}

__device__ __forceinline__ uint4 norm8(const uint4 raw, const uint4 wraw, float inv) {
  uint4 o;
  const bf162* xp = reinterpret_cast<const bf162*>(&raw);
  const bf162* wp = reinterpret_cast<const bf162*>(&wraw);
  bf162* op = reinterpret_cast<bf162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(xp[i]), g = __bfloat1622float2(wp[i]);
    const float2 nf = __bfloat1622float2(__floats2bfloat162_rn(f.x * inv, f.y * inv));
    op[i] = __floats2bfloat162_rn(nf.x * g.x, nf.y * g.y);
  }
  return o;
}

__global__ void __launch_bounds__(256)
mla_post_down_kernel(const bf16* __restrict__ qkv_a, int ld, int QL, int R, const bf16* __restrict__ gamma_q,
                     const bf16* __restrict__ gamma_kv, float eps, const int32_t* __restrict__ positions,
                     const float* __restrict__ cos_sin, const int64_t* __restrict__ slots,
                     bf16* __restrict__ q_a_out, bf16* __restrict__ cache, int page_size, int64_t page_stride) {
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const bf16* row = qkv_a + static_cast<int64_t>(t) * ld;
  if (QL > 0) {
    float ss = 0.f;
    for (int v = threadIdx.x; v < QL / 8; v += blockDim.x) {
      const uint4 a = *reinterpret_cast<const uint4*>(row + v * 8);
      const bf162* ap = reinterpret_cast<const bf162*>(&a);
#pragma unroll
      for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(ap[i]); ss += f.x * f.x + f.y * f.y; }
    }
    const float inv = rsqrtf(block_sum_256(ss, scratch) / static_cast<float>(QL) + eps);
    for (int v = threadIdx.x; v < QL / 8; v += blockDim.x)
      *reinterpret_cast<uint4*>(q_a_out + static_cast<int64_t>(t) * QL + v * 8) =
          norm8(*reinterpret_cast<const uint4*>(row + v * 8), *reinterpret_cast<const uint4*>(gamma_q + v * 8), inv);
  }
  const int64_t slot = slots[t];
  if (slot < 0) return;            // a dummy row: nothing to store (uniform over the CTA)
  const bf16* ckv = row + QL;
  float ss = 0.f;
  for (int v = threadIdx.x; v < R / 8; v += blockDim.x) {
    const uint4 a = *reinterpret_cast<const uint4*>(ckv + v * 8);
    const bf162* ap = reinterpret_cast<const bf162*>(&a);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(ap[i]); ss += f.x * f.x + f.y * f.y; }
  }
  const float inv = rsqrtf(block_sum_256(ss, scratch) / static_cast<float>(R) + eps);
  bf16* dst = cache + (slot / page_size) * page_stride + (slot % page_size) * (R + DR);
  for (int v = threadIdx.x; v < R / 8; v += blockDim.x)
    *reinterpret_cast<uint4*>(dst + v * 8) =
        norm8(*reinterpret_cast<const uint4*>(ckv + v * 8), *reinterpret_cast<const uint4*>(gamma_kv + v * 8), inv);
  if (threadIdx.x < DR / 2) {
    const int i = threadIdx.x;
    const float* cs = cos_sin + static_cast<int64_t>(positions[t]) * DR;
    const float c = cs[i], sn = cs[DR / 2 + i];
    const float2 ab = __bfloat1622float2(*reinterpret_cast<const bf162*>(ckv + R + 2 * i));
    *reinterpret_cast<bf162*>(dst + R + 2 * i) = __floats2bfloat162_rn(ab.x * c - ab.y * sn, ab.y * c + ab.x * sn);
  }
}

// q: [T, h, NOPE + 64] -> q_rope [T, h, 64] = rope(q[..., NOPE:], position) (interleaved pairs), contiguous.
__global__ void mla_q_rope_kernel(const bf16* __restrict__ q, int n_heads, int nope, const int32_t* __restrict__ positions,
                                  const float* __restrict__ cos_sin, bf16* __restrict__ q_rope, int T) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // one rotated pair per thread
  if (i >= static_cast<int64_t>(T) * n_heads * (DR / 2)) return;
  const int pr = static_cast<int>(i % (DR / 2));
  const int64_t th = i / (DR / 2);
  const int t = static_cast<int>(th / n_heads);
  const float* cs = cos_sin + static_cast<int64_t>(positions[t]) * DR;
  const float c = cs[pr], sn = cs[DR / 2 + pr];
  const float2 ab = __bfloat1622float2(*reinterpret_cast<const bf162*>(q + th * (nope + DR) + nope + 2 * pr));
  *reinterpret_cast<bf162*>(q_rope + th * DR + 2 * pr) = __floats2bfloat162_rn(ab.x * c - ab.y * sn, ab.y * c + ab.x * sn);
}

template <int R>
static int launch(const Params& p, int grid_x, cudaStream_t stream) {
  constexpr int LD = R + DR;
  const size_t smem = static_cast<size_t>(3) * 64 * LD * sizeof(bf16);
  auto kern = mla_kernel<R>;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
      return MB_ERR_LAUNCH;
    configured.done();
  }
  dim3 grid(grid_x, p.n_heads / p.HB);
  kern<<<grid, 256, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

}  // namespace mla
}  // namespace mb

using namespace mb;

extern "C" int mb_mla_post_down(const void* qkv_a, int ld, int q_lora, int R, const void* gamma_q, const void* gamma_kv,
                                float eps, const int32_t* positions, const float* cos_sin, const int64_t* slots,
                                void* q_a_out, void* cache, int T, int page_size, long long page_stride,
                                cudaStream_t stream) {
  if (T <= 0) return MB_OK;
  if (R % 8 || q_lora % 8 || ld % 8 || page_stride % 8) return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(qkv_a) | reinterpret_cast<uintptr_t>(q_a_out) | reinterpret_cast<uintptr_t>(cache) |
       reinterpret_cast<uintptr_t>(gamma_q) | reinterpret_cast<uintptr_t>(gamma_kv)) & 15)
    return MB_ERR_ALIGN;
  mla::mla_post_down_kernel<<<T, 256, 0, stream>>>(
      static_cast<const mla::bf16*>(qkv_a), ld, q_lora, R, static_cast<const mla::bf16*>(gamma_q),
      static_cast<const mla::bf16*>(gamma_kv), eps, positions, cos_sin, slots, static_cast<mla::bf16*>(q_a_out),
      static_cast<mla::bf16*>(cache), page_size, page_stride);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_mla_q_rope(const void* q, int n_heads, int nope, const int32_t* positions, const float* cos_sin,
                             void* q_rope, int T, cudaStream_t stream) {
  if (T <= 0) return MB_OK;
  if (nope % 2) return MB_ERR_SHAPE;
  const long long work = static_cast<long long>(T) * n_heads * (mla::DR / 2);
  mla::mla_q_rope_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, stream>>>(
      static_cast<const mla::bf16*>(q), n_heads, nope, positions, cos_sin, static_cast<mla::bf16*>(q_rope), T);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

// T = total query tokens, B = sequences. kv_lora_rank R in {128, 256, 512}; rope width 64.
extern "C" int mb_mla_paged_attention(const void* q_lat, const void* q_rope, void* out, const void* cache,
                                      long long page_stride, const int32_t* block_table, int bt_stride,
                                      const int32_t* q_start, const int32_t* q_len, const int32_t* kv_len,
                                      int T, int B, int n_heads, int R, int page_size, float scale,
                                      cudaStream_t stream) {
  if (T <= 0 || B <= 0) return MB_OK;
  int HB = 64;
  while (HB > 1 && n_heads % HB) HB >>= 1;
  mla::Params p;
  p.q_lat = static_cast<const mla::bf16*>(q_lat);
  p.q_rope = static_cast<const mla::bf16*>(q_rope);
  p.out = static_cast<mla::bf16*>(out);
  p.cache = static_cast<const mla::bf16*>(cache);
  p.block_table = block_table; p.q_start = q_start; p.q_len = q_len; p.kv_len = kv_len;
  p.page_stride = page_stride; p.B = B; p.bt_stride = bt_stride; p.n_heads = n_heads; p.HB = HB;
  p.page_size = page_size;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int tpt = 64 / HB;
  const int grid_x = (T + tpt - 1) / tpt + B;  // >= sum over sequences of ceil(q_len / tpt)
  switch (R) {
    case 128: return mla::launch<128>(p, grid_x, stream);
    case 256: return mla::launch<256>(p, grid_x, stream);
    case 512: return mla::launch<512>(p, grid_x, stream);
    default: return MB_ERR_SHAPE;
  }
}

extern "C" int mb_mla_kv_store(const void* c_kv, const void* k_rope, const int64_t* slots, void* cache, int T,
                               int R, int ld_c, int ld_r, int page_size, long long page_stride,
                               cudaStream_t stream) {
  if (T <= 0) return MB_OK;
  if (R % 8 || ld_c % 8 || ld_r % 8) return MB_ERR_SHAPE;
  mla::mla_kv_store_kernel<<<(T + 7) / 8, 256, 0, stream>>>(
      static_cast<const mla::bf16*>(c_kv), static_cast<const mla::bf16*>(k_rope), slots,
      static_cast<mla::bf16*>(cache), T, R, ld_c, ld_r, page_size, page_stride);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}
