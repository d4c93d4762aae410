// Paged GQA flash attention fed by TMA, one launch for a whole ragged batch.
//
// Differences from attention.cu (which stays as the path for page sizes that are not a
// multiple of 64):
//   * K/V tiles (64 tokens) arrive through cp.async.bulk.tensor from a single 2-D tensor map
//     laid over the whole KV allocation ([rows, head_dim], a (page, plane, layer, head) slice
//     being `page_size` consecutive rows), 128-byte swizzled, into a 3-stage ring guarded by
//     full/empty mbarriers. A dedicated producer warp walks the block table; the four
//     compute warps never compute a global address for K or V and never hit a CTA barrier
//     inside the loop.
//   * prefill tiles and decode sequences are CTAs of the same grid (prefill first), so the
//     compute-bound and the bandwidth-bound part of a mixed step overlap on the machine.
//
// Rows of the last tile that lie beyond kv_len are whatever the cache holds; they are masked
// to -inf before the softmax. The cache is zero-initialised and only ever holds finite
// values, which keeps 0 * garbage finite in the PV product.
//
// Reference counterpart: flash_attention_ragged over PagedKVCache
// (max/kernels/src/nn/attention/gpu/nvidia/sm100/attention.mojo:62, load_warp.mojo).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "gemm_common.h"

namespace mb {
namespace at2 {

typedef __nv_bfloat16 bf16;
constexpr int kStages = 3;          // ring depth of the mixed launch (and the size of the barrier arrays)
constexpr int kStagesDecode = 2;    // decode-only launch: 2 stages and <= 136 registers, three CTAs per SM
constexpr int kThreads = 160;  // 4 compute warps + 1 producer warp

struct Params {
  const bf16* q;
  bf16* out;
  const int32_t* block_table;
  const int32_t* q_start;
  const int32_t* q_len;
  const int32_t* kv_len;
  const int32_t* tile_seq;
  const int32_t* tile_q0;
  const int32_t* decode_seq;
  int* err;
  int ldq, ldo, bt_stride, page_size, n_tiles;
  long long k_off_rows, v_off_rows, page_rows;
  float scale_log2;
  int q_rows_alloc;      // rows of shared memory reserved for Q (64, or 16 in a decode-only launch)
};

struct Bars {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  int abort_word;
};

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
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
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Q tile layout: [rows][HD] with 16-byte chunks XOR-swizzled by the low row bits.
template <int HD>
__device__ __forceinline__ int qswz(int row, int chunk) {
  return row * HD + ((chunk ^ (row & 7)) << 3);
}
// K/V tile layout as written by TMA: HD/64 sub-tiles of [64 rows][64 dims], 128B swizzle.
__device__ __forceinline__ int kvswz(int row, int chunk) {
  return (chunk >> 3) * (64 * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
}

// One online-softmax step of 16 packed query rows against NP*16 tokens starting at row
// `tok_in_tile` of the K/V tile (global KV index kv0).
template <int HD, int NP>
__device__ __forceinline__ void process_block(const bf16* tK, const bf16* tV, int tok_in_tile, int kv0,
                                              const uint32_t (&qf)[HD / 16][4], float (&o)[HD / 8][4],
                                              float (&m)[2], float (&l)[2], const int (&limit)[2],
                                              float scale_log2, int lane) {
  constexpr int KS = HD / 16, DT = HD / 8;
  const int mi = lane >> 3;
  float sc[2 * NP][4];
#pragma unroll
  for (int i = 0; i < 2 * NP; ++i) sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
    for (int np = 0; np < NP; ++np) {
      uint32_t b[4];
      ldsm_x4(b, tK + kvswz(tok_in_tile + np * 16 + (mi >> 1) * 8 + (lane & 7), 2 * ks + (mi & 1)));
      mma_bf16(sc[2 * np], qf[ks], b[0], b[1]);
      mma_bf16(sc[2 * np + 1], qf[ks], b[2], b[3]);
    }
  }
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < 2 * NP; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int col = kv0 + nt * 8 + 2 * (lane & 3) + (e & 1);
      const int h = e >> 1;
      const float v = col <= limit[h] ? sc[nt][e] * scale_log2 : -INFINITY;
      sc[nt][e] = v;
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
  for (int nt = 0; nt < 2 * NP; ++nt) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float pv = exp2f(sc[nt][e] - msafe[e >> 1]);
      sc[nt][e] = pv;
      l[e >> 1] += pv;
    }
  }
#pragma unroll
  for (int dt = 0; dt < DT; ++dt) {
    o[dt][0] *= alpha[0]; o[dt][1] *= alpha[0];
    o[dt][2] *= alpha[1]; o[dt][3] *= alpha[1];
  }
#pragma unroll
  for (int kk = 0; kk < NP; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(sc[2 * kk][0], sc[2 * kk][1]);
    a[1] = pack_bf16(sc[2 * kk][2], sc[2 * kk][3]);
    a[2] = pack_bf16(sc[2 * kk + 1][0], sc[2 * kk + 1][1]);
    a[3] = pack_bf16(sc[2 * kk + 1][2], sc[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < DT / 2; ++dp) {
      uint32_t b[4];
      ldsm_x4_t(b, tV + kvswz(tok_in_tile + kk * 16 + (mi & 1) * 8 + (lane & 7), 2 * dp + (mi >> 1)));
      mma_bf16(o[2 * dp], a, b[0], b[1]);
      mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
    }
  }
}

// STAGES / MINB: ring depth and CTAs per SM the kernel is compiled for. The decode path is bound by the latency
// of each warp's ldmatrix -> mma -> softmax -> mma chain, so more resident warps matter more than ring depth.
template <int HD, int G, int STAGES, int MINB>
__global__ void __launch_bounds__(kThreads, MINB)
attn_tma_kernel(const __grid_constant__ CUtensorMap tmKV, const Params p) {
  constexpr int CH = HD / 8, KS = HD / 16, DT = HD / 8;
  constexpr int kTileElems = 64 * HD;          // one K (or V) tile
  constexpr uint32_t kStageBytes = 2 * kTileElems * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  bf16* sKV = reinterpret_cast<bf16*>(smem);                       // [stages][K tile | V tile]
  bf16* sQ = sKV + STAGES * 2 * kTileElems;                         // [64][HD]
  Bars* bars = reinterpret_cast<Bars*>(sQ + p.q_rows_alloc * HD);   // Q region: 64 rows (prefill) or 16 (decode-only launch)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.y;
  pdl_wait();      // Q, the KV pages of this step and the batch metadata come from earlier work on the stream
  pdl_trigger();
  const bool is_prefill = static_cast<int>(blockIdx.x) < p.n_tiles;
  const int seq = is_prefill ? p.tile_seq[blockIdx.x] : p.decode_seq[blockIdx.x - p.n_tiles];
  const int tq0 = is_prefill ? p.tile_q0[blockIdx.x] : 0;
  const int qs = p.q_start[seq], ql = p.q_len[seq], kl = p.kv_len[seq];
  const int32_t* bt = p.block_table + static_cast<int64_t>(seq) * p.bt_stride;
  int kv_hi = kl;
  if (is_prefill) {
    int last_tq = tq0 + 64 / G;
    if (last_tq > ql) last_tq = ql;
    kv_hi = kl - ql + last_tq;
  }
  const int ntiles = (kv_hi + 63) / 64;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 4);
    }
    bars->abort_word = 0;
    fence_mbar_init();
  }
  __syncthreads();
  volatile int* abort_word = &bars->abort_word;

  if (warp == 4) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tmKV);
      // This loop is on the latency path of the ring: the page index is walked (no division) and the block
      // table entry of the next tile is loaded before the wait for a free stage, so its latency hides there.
      int s = 0;
      uint32_t ph = 0;
      int page_i = 0, page_off = 0;
      int32_t page_next = ntiles > 0 ? bt[0] : 0;
      const long long head_row = static_cast<long long>(kvh) * p.page_size;
      for (int t = 0; t < ntiles; ++t, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0)) {
        const long long row = static_cast<long long>(page_next) * p.page_rows + head_row + page_off;
        page_off += 64;
        if (page_off == p.page_size) { page_off = 0; ++page_i; }
        if (t + 1 < ntiles && page_off == 0) page_next = bt[page_i];
        if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_word, p.err, 301)) break;
        bf16* dK = sKV + s * 2 * kTileElems;
        bf16* dV = dK + kTileElems;
        mbar_arrive_expect_tx(&bars->full[s], kStageBytes);
#pragma unroll
        for (int sub = 0; sub < HD / 64; ++sub) {
          tma_load_2d(dK + sub * 64 * 64, &tmKV, &bars->full[s], sub * 64,
                      static_cast<int32_t>(p.k_off_rows + row));
          tma_load_2d(dV + sub * 64 * 64, &tmKV, &bars->full[s], sub * 64,
                      static_cast<int32_t>(p.v_off_rows + row));
        }
      }
    }
    return;
  }

  // ------------------------------------------------------------ compute warps
  const int q_rows = is_prefill ? 64 : 16;
  for (int idx = tid; idx < q_rows * CH; idx += 128) {
    const int row = idx / CH, chunk = idx % CH;
    const int tq = tq0 + row / G, head = kvh * G + row % G;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (tq < ql)
      v = *reinterpret_cast<const uint4*>(p.q + static_cast<int64_t>(qs + tq) * p.ldq + head * HD + chunk * 8);
    *reinterpret_cast<uint4*>(sQ + qswz<HD>(row, chunk)) = v;
  }
  consumer_sync();
  const int row_base = is_prefill ? warp * 16 : 0;   // this warp's 16 packed rows
  uint32_t qf[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks)
    ldsm_x4(qf[ks], sQ + qswz<HD>(row_base + (lane & 15), 2 * ks + (lane >> 4)));

  float o[DT][4];
#pragma unroll
  for (int i = 0; i < DT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  int limit[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_base + (lane >> 2) + h * 8;
    const int tq = tq0 + r / G;
    limit[h] = tq < ql ? kl - ql + tq : -1;
  }
  int s = 0;
  uint32_t ph = 0;
  for (int t = 0; t < ntiles; ++t, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0)) {
    if (!mbar_wait(&bars->full[s], ph, abort_word, p.err, 302)) break;
    const bf16* tK = sKV + s * 2 * kTileElems;
    const bf16* tV = tK + kTileElems;
    if (is_prefill) {
      // every warp runs its 16 rows against all 64 tokens of the tile
      process_block<HD, 4>(tK, tV, 0, t * 64, qf, o, m, l, limit, p.scale_log2, lane);
    } else if (t * 64 + warp * 16 < kv_hi) {
      // the 16 packed rows are shared; each warp takes 16 tokens of the tile
      process_block<HD, 1>(tK, tV, warp * 16, t * 64 + warp * 16, qf, o, m, l, limit, p.scale_log2, lane);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&bars->empty[s]);
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
    l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
  }
  if (is_prefill) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
      const int r = row_base + (lane >> 2) + h * 8;
      const int tq = tq0 + r / G, head = kvh * G + r % G;
      if (tq < ql) {
        bf16* orow = p.out + static_cast<int64_t>(qs + tq) * p.ldo + head * HD + 2 * (lane & 3);
#pragma unroll
        for (int dt = 0; dt < DT; ++dt)
          *reinterpret_cast<uint32_t*>(orow + dt * 8) = pack_bf16(o[dt][2 * h] * inv, o[dt][2 * h + 1] * inv);
      }
    }
    return;
  }
  // ---- decode: merge the four warps' partial states through shared memory
  consumer_sync();  // every warp is done reading the K/V ring
  float* mO = reinterpret_cast<float*>(sKV);   // [4][16][HD]
  float* mM = mO + 4 * 16 * HD;                // [4][16]
  float* mL = mM + 64;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (lane >> 2) + h * 8;
    if ((lane & 3) == 0) {
      mM[warp * 16 + r] = m[h];
      mL[warp * 16 + r] = l[h];
    }
#pragma unroll
    for (int dt = 0; dt < DT; ++dt)
      *reinterpret_cast<float2*>(mO + (warp * 16 + r) * HD + dt * 8 + 2 * (lane & 3)) =
          make_float2(o[dt][2 * h], o[dt][2 * h + 1]);
  }
  consumer_sync();
  {
    const int r = tid >> 3;
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
      constexpr int PER = HD / 8;
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

// ---------------------------------------------------------------------------- split-KV decode
// Decode-only steps: the 64-token KV tiles of all decode sequences of one KV head form one list of
// work units that is cut into equal contiguous shares, one per CTA (grid = CTAs per head x KV heads,
// two CTAs per SM), so every SM streams the same number of KV bytes whatever the batch size, the
// context lengths or the number of KV heads on this rank (one head at tensor-parallel degree 8).
// A CTA that holds a whole sequence writes its output; a sequence cut across CTAs is combined by
// whichever contributor arrives last: each writes its running maximum, sum and unnormalised output
// (fp32, in MMA fragment order) to a workspace slot and bumps a per-(sequence, head) counter, and the
// last one merges the slots in CTA order (deterministic) and stores the rows. Nobody waits.
//
// Reference counterparts: max/kernels/src/nn/attention/gpu/mha_decode_partition_heuristic.mojo (how
// many partitions), nn/attention/gpu/nvidia/sm100/fa4_splitk_combine.mojo (the combine step).
struct SplitParams {
  float* ws;         // [n_kv][GX][2][part_floats]
  int* counters;     // [n_kv][n_decode], zero between launches
  int n_decode, GX;
};

constexpr int kMaxSplitDecode = 1024;

template <int HD>
struct PartLayout {
  static constexpr int DT = HD / 8;
  static constexpr int kFloats = (DT * 4 + 4) * 32;
};

template <int DT>
__device__ __forceinline__ void store_state(const float (&o)[DT][4], const float (&m)[2], const float (&l)[2],
                                            float* dst, int lane, bool hi) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (h == 1 && !hi) break;
    dst[(DT * 4 + h) * 32 + lane] = m[h];
    dst[(DT * 4 + 2 + h) * 32 + lane] = l[h];
#pragma unroll
    for (int dt = 0; dt < DT; ++dt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) dst[((h * DT + dt) * 2 + e) * 32 + lane] = o[dt][2 * h + e];
    }
  }
}

template <int HD, int G, int STAGES>
__global__ void __launch_bounds__(kThreads, 2)
attn_decode_split_kernel(const __grid_constant__ CUtensorMap tmKV, const Params p, const SplitParams sp) {
  constexpr int CH = HD / 8, KS = HD / 16, DT = HD / 8;
  constexpr int kTileElems = 64 * HD;
  constexpr uint32_t kStageBytes = 2 * kTileElems * 2;
  constexpr int kPart = PartLayout<HD>::kFloats;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  bf16* sKV = reinterpret_cast<bf16*>(smem);
  bf16* sQ = sKV + STAGES * 2 * kTileElems;                 // [16][HD]
  float* sM = reinterpret_cast<float*>(sQ + 16 * HD);       // two merge slots, one row half each
  constexpr int kMergeFloats = (DT * 2 + 4) * 32;           // o of one row half + m, l of both
  Bars* bars = reinterpret_cast<Bars*>(sM + 2 * kMergeFloats);
  int* prefix = reinterpret_cast<int*>(bars + 1);           // [n_decode + 1] tile prefix sums
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.y, gx = blockIdx.x;
  const int nd = sp.n_decode;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 4);
    }
    bars->abort_word = 0;
    fence_mbar_init();
  }
  pdl_wait();
  pdl_trigger();
  // tile counts of the decode sequences (one round of loads by all threads), then their prefix sums
  // (warp 0: lanes own consecutive chunks of the shared-memory array)
  for (int i = tid; i < nd; i += kThreads) prefix[i + 1] = (p.kv_len[p.decode_seq[i]] + 63) >> 6;
  __syncthreads();
  if (warp == 0) {
    const int per = (nd + 31) / 32;
    const int i0 = lane * per;
    int sum = 0;
    for (int i = i0; i < i0 + per && i < nd; ++i) sum += prefix[i + 1];
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - sum;
    if (lane == 0) prefix[0] = 0;
    for (int i = i0; i < i0 + per && i < nd; ++i) {
      run += prefix[i + 1];
      prefix[i + 1] = run;
    }
  }
  __syncthreads();
  volatile int* abort_word = &bars->abort_word;
  const long long U = prefix[nd];
  // never more shares than tiles: every CTA that stays has at least one tile, so the contributors of a
  // sequence are consecutive CTAs;
  // and no share shorter than four tiles (256 tokens): below that the per-share costs outweigh the balance
  const long long gmax = U >= 8 ? U / 4 : 1;
  const int GX = gmax < sp.GX ? static_cast<int>(gmax) : sp.GX;
  if (gx >= GX) return;
  const int u0 = static_cast<int>(U * gx / GX), u1 = static_cast<int>(U * (gx + 1) / GX);
  // first sequence of this CTA's share: largest i with prefix[i] <= u0
  int i_first;
  {
    int lo = 0, hi = nd - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (prefix[mid] <= u0) lo = mid; else hi = mid - 1;
    }
    i_first = lo;
  }

  if (warp == 4) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tmKV);
      int s = 0;
      uint32_t ph = 0;
      const long long head_row = static_cast<long long>(kvh) * p.page_size;
      bool ok = true;
      for (int i = i_first, u = u0; ok && u < u1; ++i) {
        const int fu = prefix[i], nt = prefix[i + 1] - fu;
        const int t0 = u - fu;
        int t1 = nt;
        if (fu + t1 > u1) t1 = u1 - fu;
        u = fu + t1;
        if (t1 <= t0) continue;   // a sequence without tiles
        const int32_t* bt = p.block_table + static_cast<int64_t>(p.decode_seq[i]) * p.bt_stride;
        int page_i = (t0 * 64) / p.page_size, page_off = (t0 * 64) % p.page_size;
        int32_t page_next = bt[page_i];
        for (int t = t0; t < t1; ++t) {
          const long long row = static_cast<long long>(page_next) * p.page_rows + head_row + page_off;
          page_off += 64;
          if (page_off == p.page_size) { page_off = 0; ++page_i; }
          if (t + 1 < t1 && page_off == 0) page_next = bt[page_i];
          if (!mbar_wait(&bars->empty[s], ph ^ 1, abort_word, p.err, 311)) { ok = false; break; }
          bf16* dK = sKV + s * 2 * kTileElems;
          bf16* dV = dK + kTileElems;
          mbar_arrive_expect_tx(&bars->full[s], kStageBytes);
#pragma unroll
          for (int sub = 0; sub < HD / 64; ++sub) {
            tma_load_2d(dK + sub * 64 * 64, &tmKV, &bars->full[s], sub * 64, static_cast<int32_t>(p.k_off_rows + row));
            tma_load_2d(dV + sub * 64 * 64, &tmKV, &bars->full[s], sub * 64, static_cast<int32_t>(p.v_off_rows + row));
          }
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
    return;
  }

  // ------------------------------------------------------------ compute warps
  int s = 0;
  uint32_t ph = 0;
  bool ok = true;
  for (int i = i_first, u = u0; u < u1; ++i) {
    const int fu = prefix[i], nt = prefix[i + 1] - fu;
    const int t0 = u - fu;
    int t1 = nt;
    if (fu + t1 > u1) t1 = u1 - fu;
    u = fu + t1;
    if (t1 <= t0) continue;
    const int seq = p.decode_seq[i];
    const int qs = p.q_start[seq], ql = p.q_len[seq], kl = p.kv_len[seq];
    const bool hi = ql * G > 8;   // rows 8..15 of the packed query tile are in use
    consumer_sync();              // the previous segment no longer reads sQ or the merge slots
    for (int idx = tid; idx < 16 * CH; idx += 128) {
      const int row = idx / CH, chunk = idx % CH;
      const int tq = row / G, head = kvh * G + row % G;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (tq < ql)
        v = *reinterpret_cast<const uint4*>(p.q + static_cast<int64_t>(qs + tq) * p.ldq + head * HD + chunk * 8);
      *reinterpret_cast<uint4*>(sQ + qswz<HD>(row, chunk)) = v;
    }
    consumer_sync();
    uint32_t qf[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) ldsm_x4(qf[ks], sQ + qswz<HD>(lane & 15, 2 * ks + (lane >> 4)));
    float o[DT][4];
#pragma unroll
    for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    int limit[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int tq = ((lane >> 2) + h * 8) / G;
      limit[h] = tq < ql ? kl - ql + tq : -1;
    }
    for (int t = t0; t < t1 && ok; ++t) {
      // after a failed wait this warp skips the remaining tiles but keeps meeting the other warps at
      // every barrier below (a warp that left early would leave them waiting)
      if (!mbar_wait(&bars->full[s], ph, abort_word, p.err, 312)) { ok = false; break; }
      const bf16* tK = sKV + s * 2 * kTileElems;
      const bf16* tV = tK + kTileElems;
      if (t * 64 + warp * 16 < kl)
        process_block<HD, 1>(tK, tV, warp * 16, t * 64 + warp * 16, qf, o, m, l, limit, p.scale_log2, lane);
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->empty[s]);
      if (++s == STAGES) { s = 0; ph ^= 1; }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
      l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    // tree merge of the four warps' states, one row half at a time through two small slots:
    // warps 2,3 -> slots; warps 0,1 fold them in; warp 1 -> slot 0; warp 0 folds it in
    for (int half = 0; half < (hi ? 2 : 1); ++half) {
      float* slot = sM + (warp & 1) * kMergeFloats;
      auto put = [&]() {
        slot[(DT * 2 + 0) * 32 + lane] = m[half];
        slot[(DT * 2 + 1) * 32 + lane] = l[half];
#pragma unroll
        for (int dt = 0; dt < DT; ++dt) {
          slot[(dt * 2 + 0) * 32 + lane] = o[dt][2 * half];
          slot[(dt * 2 + 1) * 32 + lane] = o[dt][2 * half + 1];
        }
      };
      auto fold = [&]() {
        const float m2 = slot[(DT * 2 + 0) * 32 + lane], l2 = slot[(DT * 2 + 1) * 32 + lane];
        const float mn = fmaxf(m[half], m2);
        const float a = m[half] == -INFINITY ? 0.f : exp2f(m[half] - mn);
        const float b = m2 == -INFINITY ? 0.f : exp2f(m2 - mn);
        m[half] = mn;
        l[half] = a * l[half] + b * l2;
#pragma unroll
        for (int dt = 0; dt < DT; ++dt) {
          o[dt][2 * half] = a * o[dt][2 * half] + b * slot[(dt * 2 + 0) * 32 + lane];
          o[dt][2 * half + 1] = a * o[dt][2 * half + 1] + b * slot[(dt * 2 + 1) * 32 + lane];
        }
      };
      if (warp >= 2) put();
      consumer_sync();
      if (warp < 2) fold();
      consumer_sync();
      if (warp == 1) put();     // (warp & 1) == 1: slot 1
      consumer_sync();
      if (warp == 0) {
        slot = sM + kMergeFloats;
        fold();
      }
      if (half == 0 && hi) consumer_sync();   // slot 1 is read before the second half overwrites it
    }
    if (warp != 0 || *abort_word != 0) continue;
    // ---- warp 0 holds the state of this segment
    const bool whole = t0 == 0 && t1 == nt;
    bool finish = whole;
    if (!whole) {
      const int g_first = static_cast<int>(((static_cast<long long>(fu) + 1) * GX - 1) / U);
      const int g_last = static_cast<int>(((static_cast<long long>(fu) + nt) * GX - 1) / U);
      float* base = sp.ws + static_cast<size_t>(kvh) * sp.GX * 2 * kPart;
      float* mine = base + (static_cast<size_t>(gx) * 2 + (fu <= u0 ? 0 : 1)) * kPart;
      store_state<DT>(o, m, l, mine, lane, hi);
      __threadfence();
      __syncwarp();
      int old = 0;
      int* cnt = sp.counters + static_cast<size_t>(kvh) * nd + i;
      if (lane == 0) old = atomicAdd(cnt, 1);
      old = __shfl_sync(0xffffffffu, old, 0);
      if (old == g_last - g_first) {
        __threadfence();
        // merge every contributor's slot in CTA order, starting from an empty state
#pragma unroll
        for (int d = 0; d < DT; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
        for (int gc = g_first; gc <= g_last; ++gc) {
          const int c0 = static_cast<int>(U * gc / GX);
          const float* src = base + (static_cast<size_t>(gc) * 2 + (fu <= c0 ? 0 : 1)) * kPart;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (h == 1 && !hi) break;
            const float m2 = __ldcg(src + (DT * 4 + h) * 32 + lane);
            const float l2 = __ldcg(src + (DT * 4 + 2 + h) * 32 + lane);
            float v[DT][2];
#pragma unroll
            for (int dt = 0; dt < DT; ++dt) {
              v[dt][0] = __ldcg(src + ((h * DT + dt) * 2 + 0) * 32 + lane);
              v[dt][1] = __ldcg(src + ((h * DT + dt) * 2 + 1) * 32 + lane);
            }
            const float mn = fmaxf(m[h], m2);
            const float a = m[h] == -INFINITY ? 0.f : exp2f(m[h] - mn);
            const float b = m2 == -INFINITY ? 0.f : exp2f(m2 - mn);
            m[h] = mn;
            l[h] = a * l[h] + b * l2;
#pragma unroll
            for (int dt = 0; dt < DT; ++dt) {
              o[dt][2 * h] = a * o[dt][2 * h] + b * v[dt][0];
              o[dt][2 * h + 1] = a * o[dt][2 * h + 1] + b * v[dt][1];
            }
          }
        }
        if (lane == 0) *cnt = 0;   // ready for the next launch
        finish = true;
      }
    }
    if (finish) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
        const int r = (lane >> 2) + h * 8;
        const int tq = r / G, head = kvh * G + r % G;
        if (tq < ql) {
          bf16* orow = p.out + static_cast<int64_t>(qs + tq) * p.ldo + head * HD + 2 * (lane & 3);
#pragma unroll
          for (int dt = 0; dt < DT; ++dt)
            *reinterpret_cast<uint32_t*>(orow + dt * 8) = pack_bf16(o[dt][2 * h] * inv, o[dt][2 * h + 1] * inv);
        }
      }
    }
  }
}

static float* g_split_ws = nullptr;
static size_t g_split_ws_bytes = 0;
static int* g_split_counters = nullptr;
static int g_split_counter_ints = 0;
static int g_split_on = 1;

template <int HD, int G>
static int launch_split(const CUtensorMap& tm, const Params& p, int n_decode, int n_kv, int num_sms,
                        cudaStream_t stream) {
  constexpr int STAGES = kStages;
  constexpr int kPart = PartLayout<HD>::kFloats;
  int GX = 2 * num_sms / n_kv;
  if (GX < 1) GX = 1;
  const size_t need = static_cast<size_t>(n_kv) * GX * 2 * kPart * sizeof(float);
  if (need > g_split_ws_bytes || static_cast<long long>(n_kv) * n_decode > g_split_counter_ints) return MB_ERR_TOO_LARGE;
  SplitParams sp;
  sp.ws = g_split_ws; sp.counters = g_split_counters; sp.n_decode = n_decode; sp.GX = GX;
  constexpr int kMergeFloats = (HD / 8 * 2 + 4) * 32;
  const size_t smem = static_cast<size_t>(STAGES) * 2 * 64 * HD * 2 + 16 * HD * 2 + 2 * kMergeFloats * sizeof(float) +
                      sizeof(Bars) + (static_cast<size_t>(n_decode) + 1) * sizeof(int) + 1024;
  auto kern = attn_decode_split_kernel<HD, G, STAGES>;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)
      return MB_ERR_LAUNCH;
    configured.done();
  }
  if (launch_k(kern, dim3(GX, n_kv), dim3(kThreads), smem, stream, tm, p, sp) != cudaSuccess) return MB_ERR_LAUNCH;
  return MB_OK;
}

template <int HD, int G, int STAGES, int MINB>
static int launch_one(const CUtensorMap& tm, Params p, int n_ctas, int n_kv, int q_rows, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(STAGES) * 2 * 64 * HD * 2 + static_cast<size_t>(q_rows) * HD * 2 +
                      sizeof(Bars) + 1024;
  auto kern = attn_tma_kernel<HD, G, STAGES, MINB>;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    const size_t smem_max = static_cast<size_t>(STAGES) * 2 * 64 * HD * 2 + 64 * HD * 2 + sizeof(Bars) + 1024;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_max)) !=
        cudaSuccess)
      return MB_ERR_LAUNCH;
    configured.done();
  }
  p.q_rows_alloc = q_rows;
  if (launch_k(kern, dim3(n_ctas, n_kv), dim3(kThreads), smem, stream, tm, p) != cudaSuccess) return MB_ERR_LAUNCH;
  return MB_OK;
}

// Decode-only launches may run the 2-stage / three-CTAs-per-SM build (switch below). Off by default: on B200
// it measured 83 us against 70 us for the three-stage / two-CTAs-per-SM build (64 sequences x 1152 tokens) -
// the depth of the TMA ring matters more than the number of resident warps.
static int g_decode_dense = 0;

// One launch covers prefill tiles and decode sequences. A decode-only step reserves shared memory for 16
// query rows instead of 64, so two CTAs (eight compute warps, six 32 KiB stages in flight) share an SM.
template <int HD, int G>
static int launch(const CUtensorMap& tm, const Params& p, int n_decode, int n_kv, const int32_t* decode_seq,
                  cudaStream_t stream) {
  (void)decode_seq;
  const int nd = n_decode < 0 ? 0 : n_decode;
  if (p.n_tiles == 0 && g_decode_dense && HD == 128)
    return launch_one<HD, G, kStagesDecode, 3>(tm, p, nd, n_kv, 16, stream);
  return launch_one<HD, G, kStages, 2>(tm, p, p.n_tiles + nd, n_kv, p.n_tiles > 0 ? 64 : 16, stream);
}

}  // namespace at2
}  // namespace mb

using namespace mb;

// Prefill tiles go to the tcgen05 kernel (attention_tc.cu) when a step has at least this many 64-row
// tiles (0 = never). Small prefill chunks next to many decode rows are cheaper in this file's single
// combined launch; measured crossover on B200: about 32 tiles (512 tokens at 4 query heads per KV head).
static int g_attn_tc_min_tiles = 0;
static int g_attn_fork = 1;                 // decode launch on a side stream next to the tcgen05 prefill launch
static cudaEvent_t g_fork_join = nullptr;
extern "C" void mb_set_attn_fork(int on) { g_attn_fork = on; }
// 1: decode-only launches use the denser build; 0 (default): the three-stage build for every launch
extern "C" void mb_set_attn_decode_dense(int on) { mb::at2::g_decode_dense = on; }
// Workspace of the split-KV decode kernel: `ws` holds partial states (mb_attn_split_workspace_bytes), `counters`
// zeroed ints, one per (KV head, decode sequence) of the largest batch. Process-wide (one process per GPU);
// without it, or with mb_set_attn_split(0), decode-only steps run one CTA per (sequence, KV head).
extern "C" size_t mb_attn_split_workspace_bytes(int num_sms) {
  // at most 2 * num_sms CTAs in all, two slots each, head_dim 128
  return static_cast<size_t>(2 * (num_sms > 0 ? num_sms : 148) + 16) * 2 * mb::at2::PartLayout<128>::kFloats * sizeof(float);
}
extern "C" void mb_set_attn_split_workspace(void* ws, size_t ws_bytes, int* counters, int counter_ints) {
  mb::at2::g_split_ws = static_cast<float*>(ws);
  mb::at2::g_split_ws_bytes = ws_bytes;
  mb::at2::g_split_counters = counters;
  mb::at2::g_split_counter_ints = counter_ints;
}
extern "C" void mb_set_attn_split(int on) { mb::at2::g_split_on = on; }
extern "C" void mb_set_attn_tc(int min_tiles) { g_attn_tc_min_tiles = min_tiles < 0 ? 0 : min_tiles; }
extern "C" int mb_get_attn_tc(void) { return g_attn_tc_min_tiles; }

// kv_base: start of the KV allocation, viewed as [total_rows, head_dim] bf16. A token of page
// `pg`, KV head `h`, offset `o` lives at row  k_off_rows (or v_off_rows) + pg*page_rows +
// h*page_size + o. Requires page_size % 64 == 0.
extern "C" int mb_paged_attention_tma(const void* q, int ldq, void* out, int ldo, const void* kv_base,
                                      long long total_rows, long long k_off_rows, long long v_off_rows,
                                      long long page_rows, const int32_t* block_table, int bt_stride,
                                      const int32_t* q_start, const int32_t* q_len,
                                      const int32_t* kv_len, const int32_t* tile_seq,
                                      const int32_t* tile_q0, int n_tiles, int n_decode,
                                      const int32_t* decode_seq, int n_q, int n_kv, int head_dim,
                                      int page_size, float scale, int* err, cudaStream_t stream) {
  using namespace mb::at2;
  if (n_tiles <= 0 && n_decode <= 0) return MB_OK;
  if (n_kv <= 0 || n_q % n_kv || page_size % 64 || total_rows >= (1ll << 31)) return MB_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(kv_base) & 15) return MB_ERR_ALIGN;
  Params p;
  p.q = static_cast<const bf16*>(q);
  p.out = static_cast<bf16*>(out);
  p.block_table = block_table;
  p.q_start = q_start; p.q_len = q_len; p.kv_len = kv_len;
  p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.decode_seq = decode_seq;
  p.err = err;
  p.ldq = ldq; p.ldo = ldo; p.bt_stride = bt_stride; p.page_size = page_size;
  p.n_tiles = n_tiles < 0 ? 0 : n_tiles;
  p.k_off_rows = k_off_rows; p.v_off_rows = v_off_rows; p.page_rows = page_rows;
  p.scale_log2 = scale * 1.4426950408889634f;
  CUtensorMap tm;
  const int rc = cached_tmap(&tm, kv_base, static_cast<uint64_t>(total_rows), head_dim, head_dim, 64, 2);
  if (rc != MB_OK) return rc;
  const int G = n_q / n_kv;
  cudaStream_t dstream = stream;   // stream of the decode launch
  bool forked = false;
  if (g_attn_tc_min_tiles > 0 && p.n_tiles >= g_attn_tc_min_tiles && head_dim == 128 && G <= 16 &&
      (G & (G - 1)) == 0) {
    // Prefill tiles on the tcgen05 kernel, decode sequences (if any) on this file's kernel. The prefill
    // kernel takes one SM per CTA and a step's prompt chunk rarely gives it 148 CTAs, so the decode launch
    // goes to a side stream and fills the remaining SMs at the same time (fork / join with two events; not
    // while the stream is being captured into a graph).
    if (n_decode > 0 && g_attn_fork) {
      cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
      if (cudaStreamIsCapturing(stream, &cap) == cudaSuccess && cap == cudaStreamCaptureStatusNone) {
        static cudaStream_t side = nullptr;
        static cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
        if (side == nullptr) {
          if (cudaStreamCreateWithFlags(&side, cudaStreamNonBlocking) != cudaSuccess ||
              cudaEventCreateWithFlags(&ev_fork, cudaEventDisableTiming) != cudaSuccess ||
              cudaEventCreateWithFlags(&ev_join, cudaEventDisableTiming) != cudaSuccess)
            side = nullptr;
        }
        if (side != nullptr && cudaEventRecord(ev_fork, stream) == cudaSuccess &&
            cudaStreamWaitEvent(side, ev_fork, 0) == cudaSuccess) {
          dstream = side;
          forked = true;
          g_fork_join = ev_join;
        }
      }
    }
    const int rc2 = mb_paged_attention_prefill_tc(q, ldq, out, ldo, kv_base, total_rows, k_off_rows, v_off_rows,
                                                  page_rows, block_table, bt_stride, q_start, q_len, kv_len, tile_seq,
                                                  tile_q0, p.n_tiles, n_q, n_kv, head_dim, page_size, scale, err,
                                                  stream);
    if (rc2 != MB_OK && !forked) return rc2;
    if (n_decode <= 0) return rc2;
    p.n_tiles = 0;
    if (rc2 != MB_OK) {   // still join the side stream before reporting
      cudaEventRecord(g_fork_join, dstream);
      cudaStreamWaitEvent(stream, g_fork_join, 0);
      return rc2;
    }
  }
  int sms = 0;
  {
    int dev = 0;
    cudaGetDevice(&dev);
    static int sm_count[64] = {};
    if (dev >= 0 && dev < 64) {
      if (sm_count[dev] == 0) cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
      sms = sm_count[dev];
    }
    if (sms <= 0) sms = 148;
  }
  // Partition heuristic, measured on B200 under graph replay (64 sequences x 1152 tokens, 8 / 4 / 2 / 1 KV heads:
  // one CTA per (sequence, head) 52.9 / 29.1 / 17.3 / 15.0 us, split 54.2 / 32.3 / 22.7 / 17.3 us; one sequence
  // of 8192 tokens: 76.1 against 28.6 us): with at least one CTA per (sequence, head) for every second SM the
  // unsplit kernel already streams at 0.85-0.99 of the copy bandwidth and the split costs ~2 us of fixed work;
  // below that a long context would be read by a handful of CTAs, so the KV tiles are shared out.
  // g_split_on = 2 forces the split kernel for every decode-only step.
  const bool want_split = g_split_on == 2 || (g_split_on == 1 && static_cast<long long>(n_decode) * n_kv * 2 <= sms);
  if (p.n_tiles == 0 && n_decode > 0 && n_decode <= kMaxSplitDecode && want_split && g_split_ws != nullptr && !forked) {
    // decode-only step: equal KV shares per CTA with an in-kernel combine
    int rcs = MB_ERR_SHAPE;
#define MB_ATTN_SPLIT_CASE(HD_, G_) \
  if (head_dim == HD_ && G == G_) rcs = launch_split<HD_, G_>(tm, p, n_decode, n_kv, sms, stream);
    MB_ATTN_SPLIT_CASE(128, 1) MB_ATTN_SPLIT_CASE(128, 2) MB_ATTN_SPLIT_CASE(128, 4) MB_ATTN_SPLIT_CASE(128, 8)
    MB_ATTN_SPLIT_CASE(128, 16)
    MB_ATTN_SPLIT_CASE(64, 1) MB_ATTN_SPLIT_CASE(64, 2) MB_ATTN_SPLIT_CASE(64, 4) MB_ATTN_SPLIT_CASE(64, 8)
#undef MB_ATTN_SPLIT_CASE
    if (rcs == MB_OK || rcs == MB_ERR_LAUNCH) return rcs;   // other codes: the one-CTA-per-sequence kernel below
  }
  int rc3 = MB_ERR_SHAPE;
#define MB_ATTN2_CASE(HD_, G_) \
  if (head_dim == HD_ && G == G_) rc3 = launch<HD_, G_>(tm, p, n_decode, n_kv, decode_seq, dstream);
  MB_ATTN2_CASE(128, 1) MB_ATTN2_CASE(128, 2) MB_ATTN2_CASE(128, 4) MB_ATTN2_CASE(128, 8)
  MB_ATTN2_CASE(128, 16)
  MB_ATTN2_CASE(64, 1) MB_ATTN2_CASE(64, 2) MB_ATTN2_CASE(64, 4) MB_ATTN2_CASE(64, 8)
  MB_ATTN2_CASE(64, 16)
#undef MB_ATTN2_CASE
  if (forked) {
    if (cudaEventRecord(g_fork_join, dstream) != cudaSuccess || cudaStreamWaitEvent(stream, g_fork_join, 0) != cudaSuccess)
      return MB_ERR_LAUNCH;
  }
  return rc3;
}
