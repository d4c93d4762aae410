// Paged, ragged flash attention for MHA/GQA over a block-table KV cache.
//
// One launch serves a continuous-batching step: sequences with new-token count > a few
// (prefill chunks) go through `attn_prefill_kernel`, single-token (or short speculative)
// sequences through `attn_decode_kernel`. Both pack the G = n_q / n_kv query heads that
// share a KV head into the row dimension of the MMA tile, so one pass over a K/V tile
// serves the whole group (decode reads every KV byte exactly once).
//
//   prefill: CTA = 64 packed rows (64/G query tokens x G heads) x one KV head, 4 warps,
//            64-token K/V tiles double-buffered with cp.async, online softmax in fp32.
//   decode : CTA = one sequence x one KV head; the 4 warps split every 64-token tile
//            (16 tokens each), keep private (m, l, O) and merge through shared memory.
//
// Behavioural counterpart in the reference: flash_attention_ragged over PagedKVCache
// (max/kernels/src/nn/attention/gpu/mha.mojo, nn/kv_cache_ragged.mojo).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/launch.h"

namespace mb {

typedef __nv_bfloat16 bf16;

struct AttnParams {
  const bf16* q;
  bf16* out;
  const bf16* k_cache;
  const bf16* v_cache;
  const int32_t* block_table;
  const int32_t* q_start;
  const int32_t* q_len;
  const int32_t* kv_len;
  const int32_t* tile_seq;   // prefill: sequence of each CTA tile
  const int32_t* tile_q0;    // prefill: first query token (within the sequence) of the tile
  const int32_t* decode_seq; // decode: sequence of each CTA
  int ldq, ldo, bt_stride, page_size;
  int64_t page_stride, head_stride;
  float scale_log2;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src),
               "r"(sz)
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
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Element offset of 16-byte chunk `chunk` of row `row` in a [rows][HD] bf16 tile whose
// chunks are XOR-swizzled with the low row bits (conflict-free ldmatrix).
template <int HD>
__device__ __forceinline__ int swz(int row, int chunk) {
  return row * HD + ((chunk ^ (row & 7)) << 3);
}

// Load a 64-token K and V tile (tokens kv0 .. kv0+63 of one sequence, one KV head).
template <int HD>
__device__ __forceinline__ void load_kv_tile(bf16* sK, bf16* sV, const AttnParams& p,
                                             const int32_t* bt, int kvh, int kv0, int kv_end,
                                             int tid) {
  constexpr int CH = HD / 8;
#pragma unroll
  for (int i = 0; i < 64 * CH / 128; ++i) {
    const int idx = tid + i * 128;
    const int row = idx / CH, chunk = idx % CH;
    const int tok = kv0 + row;
    const bool valid = tok < kv_end;
    const int pg = valid ? bt[tok / p.page_size] : 0;
    const int off = valid ? tok % p.page_size : 0;
    const int64_t e = static_cast<int64_t>(pg) * p.page_stride + kvh * p.head_stride +
                      static_cast<int64_t>(off) * HD + chunk * 8;
    cp_async16(sK + swz<HD>(row, chunk), p.k_cache + e, valid);
    cp_async16(sV + swz<HD>(row, chunk), p.v_cache + e, valid);
  }
}

template <int HD, int G>
__global__ void __launch_bounds__(128) attn_prefill_kernel(const AttnParams p) {
  constexpr int BM = 64, CH = HD / 8, KS = HD / 16, DT = HD / 8;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
  bf16* sK = sQ + BM * HD;       // [2][64*HD]
  bf16* sV = sK + 2 * 64 * HD;   // [2][64*HD]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.y;
  const int seq = p.tile_seq[blockIdx.x];
  const int tq0 = p.tile_q0[blockIdx.x];
  const int qs = p.q_start[seq], ql = p.q_len[seq], kl = p.kv_len[seq];
  const int32_t* bt = p.block_table + static_cast<int64_t>(seq) * p.bt_stride;

#pragma unroll
  for (int i = 0; i < BM * CH / 128; ++i) {
    const int idx = tid + i * 128;
    const int row = idx / CH, chunk = idx % CH;
    const int tq = tq0 + row / G, head = kvh * G + row % G;
    const bool valid = tq < ql;
    const bf16* src = p.q + static_cast<int64_t>(qs + (valid ? tq : 0)) * p.ldq + head * HD + chunk * 8;
    cp_async16(sQ + swz<HD>(row, chunk), src, valid);
  }
  int last_tq = tq0 + BM / G;
  if (last_tq > ql) last_tq = ql;
  const int kv_hi = kl - ql + last_tq;  // exclusive bound of KV indices any row of this CTA sees
  const int ntiles = (kv_hi + 63) / 64;
  load_kv_tile<HD>(sK, sV, p, bt, kvh, 0, kv_hi, tid);
  cp_async_commit();
  cp_async_wait_all();
  __syncthreads();

  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks)
    ldsm_x4(qf[ks], sQ + swz<HD>(warp * 16 + (lane & 15), 2 * ks + (lane >> 4)));

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  int limit[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = warp * 16 + (lane >> 2) + h * 8;
    const int tq = tq0 + r / G;
    limit[h] = tq < ql ? kl - ql + tq : -1;
  }

  for (int it = 0; it < ntiles; ++it) {
    const int buf = it & 1;
    if (it + 1 < ntiles) {
      load_kv_tile<HD>(sK + (buf ^ 1) * 64 * HD, sV + (buf ^ 1) * 64 * HD, p, bt, kvh,
                       (it + 1) * 64, kv_hi, tid);
      cp_async_commit();
    }
    const bf16* tK = sK + buf * 64 * HD;
    const bf16* tV = sV + buf * 64 * HD;
    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        const int mi = lane >> 3;
        ldsm_x4(b, tK + swz<HD>(np * 16 + (mi >> 1) * 8 + (lane & 7), 2 * ks + (mi & 1)));
        mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
        mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
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
        ldsm_x4_t(b, tV + swz<HD>(kk * 16 + (mi & 1) * 8 + (lane & 7), 2 * dp + (mi >> 1)));
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
    const int r = warp * 16 + (lane >> 2) + h * 8;
    const int tq = tq0 + r / G, head = kvh * G + r % G;
    if (tq < ql) {
      bf16* orow = p.out + static_cast<int64_t>(qs + tq) * p.ldo + head * HD + 2 * (lane & 3);
#pragma unroll
      for (int dt = 0; dt < DT; ++dt)
        *reinterpret_cast<uint32_t*>(orow + dt * 8) =
            pack_bf16(o[dt][2 * h] * inv, o[dt][2 * h + 1] * inv);
    }
  }
}

// Decode: up to 16/G new tokens per sequence (1 for plain decode).
template <int HD, int G>
__global__ void __launch_bounds__(128) attn_decode_kernel(const AttnParams p) {
  constexpr int CH = HD / 8, KS = HD / 16, DT = HD / 8;
  extern __shared__ __align__(128) uint8_t smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);   // [16*HD]
  bf16* sK = sQ + 16 * HD;                        // [2][64*HD]
  bf16* sV = sK + 2 * 64 * HD;                    // [2][64*HD]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.y;
  const int seq = p.decode_seq[blockIdx.x];
  const int qs = p.q_start[seq], ql = p.q_len[seq], kl = p.kv_len[seq];
  const int32_t* bt = p.block_table + static_cast<int64_t>(seq) * p.bt_stride;

  for (int idx = tid; idx < 16 * CH; idx += 128) {
    const int row = idx / CH, chunk = idx % CH;
    const int tq = row / G, head = kvh * G + row % G;
    const bool valid = tq < ql;
    const bf16* src = p.q + static_cast<int64_t>(qs + (valid ? tq : 0)) * p.ldq + head * HD + chunk * 8;
    cp_async16(sQ + swz<HD>(row, chunk), src, valid);
  }
  const int ntiles = (kl + 63) / 64;
  load_kv_tile<HD>(sK, sV, p, bt, kvh, 0, kl, tid);
  cp_async_commit();
  cp_async_wait_all();
  __syncthreads();

  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks)
    ldsm_x4(qf[ks], sQ + swz<HD>(lane & 15, 2 * ks + (lane >> 4)));

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  int limit[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (lane >> 2) + h * 8;
    const int tq = r / G;
    limit[h] = tq < ql ? kl - ql + tq : -1;
  }

  for (int it = 0; it < ntiles; ++it) {
    const int buf = it & 1;
    if (it + 1 < ntiles) {
      load_kv_tile<HD>(sK + (buf ^ 1) * 64 * HD, sV + (buf ^ 1) * 64 * HD, p, bt, kvh,
                       (it + 1) * 64, kl, tid);
      cp_async_commit();
    }
    const bf16* tK = sK + buf * 64 * HD;
    const bf16* tV = sV + buf * 64 * HD;
    const int kv0 = it * 64 + warp * 16;  // this warp's 16 tokens of the tile
    if (kv0 < kl) {
      float s[2][4];
      s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
      s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
      const int mi = lane >> 3;
#pragma unroll
      for (int ks = 0; ks < KS; ++ks) {
        uint32_t b[4];
        ldsm_x4(b, tK + swz<HD>(warp * 16 + (mi >> 1) * 8 + (lane & 7), 2 * ks + (mi & 1)));
        mma_bf16(s[0], qf[ks], b[0], b[1]);
        mma_bf16(s[1], qf[ks], b[2], b[3]);
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
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
      for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float pv = exp2f(s[nt][e] - msafe[e >> 1]);
          s[nt][e] = pv;
          l[e >> 1] += pv;
        }
      }
      uint32_t a[4];
      a[0] = pack_bf16(s[0][0], s[0][1]);
      a[1] = pack_bf16(s[0][2], s[0][3]);
      a[2] = pack_bf16(s[1][0], s[1][1]);
      a[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
      for (int dp = 0; dp < DT / 2; ++dp) {
        o[2 * dp][0] *= alpha[0]; o[2 * dp][1] *= alpha[0];
        o[2 * dp][2] *= alpha[1]; o[2 * dp][3] *= alpha[1];
        o[2 * dp + 1][0] *= alpha[0]; o[2 * dp + 1][1] *= alpha[0];
        o[2 * dp + 1][2] *= alpha[1]; o[2 * dp + 1][3] *= alpha[1];
        uint32_t b[4];
        ldsm_x4_t(b, tV + swz<HD>(warp * 16 + (mi & 1) * 8 + (lane & 7), 2 * dp + (mi >> 1)));
        mma_bf16(o[2 * dp], a, b[0], b[1]);
        mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
      }
    }
    cp_async_wait_all();
    __syncthreads();
  }

  // merge the four warps: shared layout  O[4][16][HD] fp32, M[4][16], L[4][16]
  float* mO = reinterpret_cast<float*>(sK);
  float* mM = mO + 4 * 16 * HD;
  float* mL = mM + 64;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    const int r = (lane >> 2) + h * 8;
    if ((lane & 3) == 0) {
      mM[warp * 16 + r] = m[h];
      mL[warp * 16 + r] = l[h];
    }
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) {
      float2 v = make_float2(o[dt][2 * h], o[dt][2 * h + 1]);
      *reinterpret_cast<float2*>(mO + (warp * 16 + r) * HD + dt * 8 + 2 * (lane & 3)) = v;
    }
  }
  __syncthreads();
  {
    const int r = tid >> 3;                 // 16 rows, 8 threads per row
    const int tq = r / G, head = kvh * G + r % G;
    if (tq < ql) {
      float mm = -INFINITY;
#pragma unroll
      for (int w = 0; w < 4; ++w) mm = fmaxf(mm, mM[w * 16 + r]);
      float wgt[4], L = 0.f;
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float mw = mM[w * 16 + r];
        wgt[w] = mw == -INFINITY ? 0.f : exp2f(mw - mm);
        L += wgt[w] * mL[w * 16 + r];
      }
      const float inv = L > 0.f ? 1.f / L : 0.f;
      bf16* orow = p.out + static_cast<int64_t>(qs + tq) * p.ldo + head * HD;
      constexpr int PER = HD / 8;  // dims per thread
      const int d0 = (tid & 7) * PER;
#pragma unroll
      for (int d = 0; d < PER; d += 2) {
        float a = 0.f, b = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const float2 v = *reinterpret_cast<const float2*>(mO + (w * 16 + r) * HD + d0 + d);
          a += wgt[w] * v.x;
          b += wgt[w] * v.y;
        }
        *reinterpret_cast<uint32_t*>(orow + d0 + d) = pack_bf16(a * inv, b * inv);
      }
    }
  }
}

template <int HD, int G>
static int launch_attn(const AttnParams& p, int n_tiles, int n_decode, int n_kv,
                       cudaStream_t stream) {
  const size_t smem_pf = (64 + 4 * 64) * HD * 2;
  const size_t smem_dc = (16 + 4 * 64) * HD * 2;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    cudaFuncSetAttribute(attn_prefill_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(smem_pf));
    cudaFuncSetAttribute(attn_decode_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         static_cast<int>(smem_dc));
    configured.done();
  }
  if (n_tiles > 0)
    attn_prefill_kernel<HD, G><<<dim3(n_tiles, n_kv), 128, smem_pf, stream>>>(p);
  if (n_decode > 0)
    attn_decode_kernel<HD, G><<<dim3(n_decode, n_kv), 128, smem_dc, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

}  // namespace mb

using namespace mb;

// Prefill tiles cover 64/G query tokens each (host builds tile_seq / tile_q0); decode
// sequences must have q_len * G <= 16.
extern "C" int mb_paged_attention(const void* q, int ldq, void* out, int ldo, const void* k_cache,
                                  const void* v_cache, const int32_t* block_table, int bt_stride,
                                  const int32_t* q_start, const int32_t* q_len,
                                  const int32_t* kv_len, const int32_t* tile_seq,
                                  const int32_t* tile_q0, int n_tiles, int n_decode,
                                  const int32_t* decode_seq, int n_q, int n_kv, int head_dim,
                                  int page_size, int64_t page_stride, int64_t head_stride,
                                  float scale, cudaStream_t stream) {
  if (n_tiles <= 0 && n_decode <= 0) return MB_OK;
  if (n_kv <= 0 || n_q % n_kv) return MB_ERR_SHAPE;
  AttnParams p;
  p.q = static_cast<const bf16*>(q);
  p.out = static_cast<bf16*>(out);
  p.k_cache = static_cast<const bf16*>(k_cache);
  p.v_cache = static_cast<const bf16*>(v_cache);
  p.block_table = block_table;
  p.q_start = q_start; p.q_len = q_len; p.kv_len = kv_len;
  p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.decode_seq = decode_seq;
  p.ldq = ldq; p.ldo = ldo; p.bt_stride = bt_stride; p.page_size = page_size;
  p.page_stride = page_stride; p.head_stride = head_stride;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int G = n_q / n_kv;
#define MB_ATTN_CASE(HD_, G_) \
  if (head_dim == HD_ && G == G_) return launch_attn<HD_, G_>(p, n_tiles, n_decode, n_kv, stream);
  MB_ATTN_CASE(128, 1) MB_ATTN_CASE(128, 2) MB_ATTN_CASE(128, 4) MB_ATTN_CASE(128, 8)
  MB_ATTN_CASE(128, 16)
  MB_ATTN_CASE(64, 1) MB_ATTN_CASE(64, 2) MB_ATTN_CASE(64, 4) MB_ATTN_CASE(64, 8)
  MB_ATTN_CASE(64, 16)
#undef MB_ATTN_CASE
  return MB_ERR_SHAPE;
}
