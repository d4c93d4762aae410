// Absorbed multi-head latent attention, decode (one query token per sequence), on tcgen05 + TMEM + TMA.
//
// The 128 heads of one token are the 128 rows of the MMA (all heads share the one latent "KV head"), the
// key is the 576-wide latent row (512 compressed + 64 rotary), the value its first 512 columns. A CTA owns
// (sequence, block of 128 heads, half of the 512 output columns): the 128 x 512 fp32 output would fill all
// 512 TMEM columns and leave none for the scores, so two CTAs each keep 256 of them and both compute the
// scores.
//
//   shared memory  Q: nine [128 heads x 64 columns] blocks, resident (144 KiB)
//                  ring of seven 8 KiB slots, each one [64 tokens x 64 columns] block of the latent cache
//                  P: [128 x 64] probabilities of the current tile (16 KiB)
//   warp 0   TMA producer. Per 64-token tile the nine column blocks for S = Q . K^T, and later the four
//            blocks of this CTA's output half again for O += P . V (they come from L2 the second time);
//            the same [tokens x 64 columns] block is a K-major operand for S and an MN-major one for P . V
//   warp 1   MMA issuer, in the order S(0) S(1) PV(0) S(2) PV(1) ... so that the scores of the next tile are
//            computed while the softmax warps work on this one (two S buffers in TMEM)
//   warps 2-5  softmax: one head per thread (TMEM lane = head); running maximum with lazy rescaling of the
//            accumulator (only when a row's maximum grew by more than 2^8), P written bf16 in the swizzled
//            K-major layout
//
// Every mbarrier wait is bounded; on a time-out the CTA raises the error word, drains and frees its TMEM.
// Steps with more than one query token per sequence run the same kernel in token mode (one CTA pair per query
// token over the causal prefix of its sequence); other latent widths or head counts stay on the mma.sync kernel of
// mla.cu.
//
// Reference counterpart: max/kernels/src/nn/attention/gpu/nvidia/sm100/mla_decode_*.mojo (absorbed MLA decode
// with split-K partitions) behind nn/attention/multi_latent_attention.py:511.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "gemm_common.h"

namespace mb {
namespace mlatc {

typedef __nv_bfloat16 bf16;
constexpr int R = 512, DR = 64, LD = R + DR;
constexpr int kQBlocks = LD / 64;             // 9
constexpr int kQBlockBytes = 128 * 128;       // 128 heads x 64 columns
constexpr int kSlotBytes = 64 * 128;          // 64 tokens x 64 columns
constexpr int kSlots = 7;
constexpr int kPBytes = 128 * 128;
constexpr int kThreads = 192;
constexpr uint32_t kTmemCols = 512;           // S0 | S1 (64 each) | O half (256)
constexpr int kVBlocks = 4;                   // 256 output columns = four 64-column blocks
constexpr int kPartFloats = 256 * 128 + 2 * 128;   // one partial: O [256 columns][128 heads], m [128], l [128]

struct Params {
  bf16* out;                       // [T, h, 512]
  const int32_t* block_table;
  const int32_t* q_start;
  const int32_t* q_len;
  const int32_t* kv_len;
  // token mode (prefill): grid x walks query tokens; token t belongs to sequence tok_seq[t] and sees the first
  // tok_kvlen[t] cache rows of it (causal). nullptr: grid x walks sequences with one query token each.
  const int32_t* tok_seq;
  const int32_t* tok_kvlen;
  // KV split (decode with few sequences): grid x = sequence * nsplit + part; every part walks its share of the
  // 64-token tiles and leaves an unnormalised partial (256 x 128 fp32 + running maximum and sum per head) in `ws`;
  // the last part to arrive at the (sequence, head block, half) counter combines them. nsplit = 1: no workspace.
  int nsplit;
  float* ws;
  int* counters;
  int* err;
  long long page_rows;             // rows of the [rows, 576] view between consecutive pages
  int bt_stride, n_heads, page_size;
  float scale_log2;
};

struct Bars {
  uint64_t full[kSlots];
  uint64_t empty[kSlots];
  uint64_t q_full;
  uint64_t s_full[2];
  uint64_t s_free[2];
  uint64_t p_full;
  uint64_t pv_full;
  uint32_t tmem_base;
  int abort_word;
  int last_flag;
};

__device__ __forceinline__ uint64_t desc_mn_sw128(const void* smem_tile, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_u32(smem_tile) & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(sbo_bytes >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__global__ void __launch_bounds__(kThreads, 1)
mla_tc_kernel(const __grid_constant__ CUtensorMap tmQl, const __grid_constant__ CUtensorMap tmQr,
              const __grid_constant__ CUtensorMap tmKV, const Params p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0 && p.err) atomicCAS(p.err, 0, 899);
    return;
  }
  uint8_t* sQ = smem_raw;
  uint8_t* sRing = sQ + kQBlocks * kQBlockBytes;
  uint8_t* sP = sRing + kSlots * kSlotBytes;
  Bars* bars = reinterpret_cast<Bars*>(sP + kPBytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hb = blockIdx.y, half = blockIdx.z;

  pdl_wait();
  pdl_trigger();
  int seq = blockIdx.x, qs, ql, kl;
  int part = 0;
  if (p.nsplit > 1) {
    part = seq % p.nsplit;
    seq /= p.nsplit;
  }
  if (p.tok_seq != nullptr) {
    qs = blockIdx.x;                    // one CTA pair per query token
    seq = p.tok_seq[qs];
    kl = p.tok_kvlen[qs];
    ql = seq >= 0 ? 1 : 0;
  } else {
    qs = p.q_start[seq]; ql = p.q_len[seq]; kl = p.kv_len[seq];
  }
  if (ql <= 0) return;   // whole CTA, before any barrier or TMEM allocation
  const int32_t* bt = p.block_table + static_cast<int64_t>(seq) * p.bt_stride;
  const int tiles_all = (kl + 63) / 64;
  // this part's tiles [t_begin, t_begin + ntiles); parts are as even as possible and the trailing ones may be empty
  const int tiles_per = p.nsplit > 1 ? (tiles_all + p.nsplit - 1) / p.nsplit : tiles_all;
  const int t_begin = part * tiles_per;
  const int ntiles = max(0, min(tiles_all, t_begin + tiles_per) - t_begin);
  const int n_parts = tiles_per > 0 ? (tiles_all + tiles_per - 1) / tiles_per : 1;   // parts that have tiles
  if (part > 0 && ntiles == 0) return;            // whole CTA, before any barrier or TMEM allocation
  const int q_row = qs * p.n_heads + hb * 128;   // row of the [T*h, .] views of q_lat / q_rope / out

  if (tid == 0) {
    for (int s = 0; s < kSlots; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    mbar_init(&bars->q_full, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->s_full[b], 1);
      mbar_init(&bars->s_free[b], 4);
    }
    mbar_init(&bars->p_full, 4);
    mbar_init(&bars->pv_full, 1);
    bars->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  volatile int* abort_word = &bars->abort_word;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmKV);
      mbar_arrive_expect_tx(&bars->q_full, kQBlocks * kQBlockBytes);
#pragma unroll
      for (int j = 0; j < kQBlocks - 1; ++j) tma_load_2d(sQ + j * kQBlockBytes, &tmQl, &bars->q_full, j * 64, q_row);
      tma_load_2d(sQ + (kQBlocks - 1) * kQBlockBytes, &tmQr, &bars->q_full, 0, q_row);
      int slot = 0;
      uint32_t ph = 0;
      bool ok = true;
      auto load_block = [&](int col_block, long long row) {
        if (!ok) return;
        ok = mbar_wait(&bars->empty[slot], ph ^ 1, abort_word, p.err, 801);
        if (!ok) return;
        mbar_arrive_expect_tx(&bars->full[slot], kSlotBytes);
        tma_load_2d(sRing + slot * kSlotBytes, &tmKV, &bars->full[slot], col_block * 64, static_cast<int32_t>(row));
        if (++slot == kSlots) { slot = 0; ph ^= 1; }
      };
      // pages are walked without divisions; row_prev is the tile whose P . V blocks follow the next S blocks
      int page_i = (t_begin * 64) / p.page_size, page_off = (t_begin * 64) % p.page_size;
      long long row_prev = 0;
      for (int i = 0; i <= ntiles && ok; ++i) {
        long long row_cur = 0;
        if (i < ntiles) {
          row_cur = static_cast<long long>(bt[page_i]) * p.page_rows + page_off;
          page_off += 64;
          if (page_off == p.page_size) { page_off = 0; ++page_i; }
          for (int j = 0; j < kQBlocks; ++j) load_block(j, row_cur);
        }
        if (i >= 1)
          for (int v = 0; v < kVBlocks; ++v) load_block(half * kVBlocks + v, row_prev);
        row_prev = row_cur;
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(128, 64, 1, 1);
      const uint32_t idesc_pv = umma_idesc(128, 64, 1, 1) | (1u << 16);   // B operand (V) is MN-major
      const uint64_t dq0 = umma_desc_sw128(sQ);
      const uint64_t dp0 = umma_desc_sw128(sP);
      const uint64_t dring0 = umma_desc_sw128(sRing);
      int slot = 0;
      uint32_t ph = 0;
      bool ok = mbar_wait(&bars->q_full, 0, abort_word, p.err, 802);
      for (int i = 0; i <= ntiles && ok; ++i) {
        if (i < ntiles) {
          // S(i) = Q . K^T over the nine column blocks
          const int b = i & 1;
          ok = mbar_wait(&bars->s_free[b], ((i >> 1) & 1) ^ 1, abort_word, p.err, 803);
          for (int j = 0; j < kQBlocks && ok; ++j) {
            ok = mbar_wait(&bars->full[slot], ph, abort_word, p.err, 804);
            if (!ok) break;
            tc_fence_after();
            const uint64_t da = dq0 + static_cast<uint64_t>(j * (kQBlockBytes >> 4));
            const uint64_t db = dring0 + static_cast<uint64_t>(slot * (kSlotBytes >> 4));
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16(tmem_base + b * 64, da + 2 * k, db + 2 * k, idesc_s, (j > 0 || k > 0) ? 1u : 0u);
            tc_commit(&bars->empty[slot]);
            if (++slot == kSlots) { slot = 0; ph ^= 1; }
          }
          if (ok) tc_commit(&bars->s_full[b]);
        }
        if (i >= 1 && ok) {
          // O += P(i-1) . V(i-1), 64 output columns per ring block
          const int t = i - 1;
          ok = mbar_wait(&bars->p_full, t & 1, abort_word, p.err, 805);
          for (int v = 0; v < kVBlocks && ok; ++v) {
            ok = mbar_wait(&bars->full[slot], ph, abort_word, p.err, 806);
            if (!ok) break;
            tc_fence_after();
            const uint8_t* sV = sRing + slot * kSlotBytes;
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_bf16(tmem_base + 128 + v * 64, dp0 + 2 * k, desc_mn_sw128(sV + k * 2048, 8192, 1024), idesc_pv,
                        (t > 0 || k > 0) ? 1u : 0u);
            tc_commit(&bars->empty[slot]);
            if (++slot == kSlots) { slot = 0; ph ^= 1; }
          }
          if (ok) tc_commit(&bars->pv_full);
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax (warps 2-5)
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
    const int r = quad * 32 + lane;            // head within the block
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t o_addr = lane_addr + 128;
    float m_ref = 0.f, l = 0.f;
    bool ok = true;
    for (int t = 0; t < ntiles && ok; ++t) {
      const int b = t & 1;
      ok = mbar_wait(&bars->s_full[b], (t >> 1) & 1, abort_word, p.err, 807);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[2][32];
      tmem_ld_32x32(lane_addr + b * 64, sr[0]);
      tmem_ld_32x32(lane_addr + b * 64 + 32, sr[1]);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->s_free[b]);
      const int kv0 = (t_begin + t) * 64;
      float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (kv0 + 64 <= kl) {
#pragma unroll
        for (int c = 0; c < 64; ++c) mxa[c & 3] = fmaxf(mxa[c & 3], __uint_as_float(sr[c >> 5][c & 31]));
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const float v = (kv0 + c) < kl ? __uint_as_float(sr[c >> 5][c & 31]) : -INFINITY;
          sr[c >> 5][c & 31] = __float_as_uint(v);
          mxa[c & 3] = fmaxf(mxa[c & 3], v);
        }
      }
      const float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])) * p.scale_log2;   // scale > 0
      // the previous P . V has retired: the P buffer is free and the accumulator is quiescent
      if (t > 0) {
        ok = mbar_wait(&bars->pv_full, (t - 1) & 1, abort_word, p.err, 808);
        if (!ok) break;
        tc_fence_after();
      }
      bool grow = false;
      if (t == 0) {
        m_ref = mx == -INFINITY ? 0.f : mx;
      } else {
        grow = mx - m_ref > 8.0f;
      }
      if (__any_sync(0xffffffffu, grow)) {
        const float factor = grow ? exp2f(m_ref - mx) : 1.0f;
        if (grow) { m_ref = mx; l *= factor; }
#pragma unroll 1
        for (int q8 = 0; q8 < 8; ++q8) {
          uint32_t tr[32];
          tmem_ld_32x32(o_addr + q8 * 32, tr);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) tr[c] = __float_as_uint(__uint_as_float(tr[c]) * factor);
          tmem_st_32x32(o_addr + q8 * 32, tr);
        }
        tc_wait_st();
      }
      float la[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        uint32_t pk[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = c8 * 8 + 2 * j;
          const float p0 = exp2f(fmaf(__uint_as_float(sr[c >> 5][c & 31]), p.scale_log2, -m_ref));
          const float p1 = exp2f(fmaf(__uint_as_float(sr[(c + 1) >> 5][(c + 1) & 31]), p.scale_log2, -m_ref));
          la[j] += p0 + p1;
          __nv_bfloat162 v2 = __floats2bfloat162_rn(p0, p1);
          pk[j] = *reinterpret_cast<uint32_t*>(&v2);
        }
        *reinterpret_cast<uint4*>(sP + r * 128 + ((c8 ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l += (la[0] + la[1]) + (la[2] + la[3]);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full);
    }
    if (ok && ntiles > 0) ok = mbar_wait(&bars->pv_full, (ntiles - 1) & 1, abort_word, p.err, 809);
    tc_fence_after();
    // ---- epilogue: O / l -> bf16, 256 columns of this CTA's half
    bf16* orow = p.out + (static_cast<int64_t>(q_row) + r) * R + half * 256;
    if (n_parts <= 1) {
      const float inv = (ok && ntiles > 0 && l > 0.f) ? 1.f / l : 0.f;
      if (ntiles > 0 && ok) {
#pragma unroll 1
        for (int q8 = 0; q8 < 8; ++q8) {
          uint32_t ta[32];
          tmem_ld_32x32(o_addr + q8 * 32, ta);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              __nv_bfloat162 v2 = __floats2bfloat162_rn(__uint_as_float(ta[c * 8 + 2 * j]) * inv,
                                                        __uint_as_float(ta[c * 8 + 2 * j + 1]) * inv);
              pk[j] = *reinterpret_cast<uint32_t*>(&v2);
            }
            *reinterpret_cast<uint4*>(orow + q8 * 32 + c * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
      } else if (ntiles == 0) {
        for (int c = 0; c < 256; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
      }
    } else {
      // ---- this part's partial goes to the workspace; the last part to arrive combines all of them
      const int unit = (seq * (p.n_heads / 128) + hb) * 2 + half;
      float* base = p.ws + static_cast<size_t>(unit) * p.nsplit * kPartFloats;
      float* mine = base + static_cast<size_t>(part) * kPartFloats;
#pragma unroll 1
      for (int q8 = 0; q8 < 8; ++q8) {
        uint32_t ta[32];
        tmem_ld_32x32(o_addr + q8 * 32, ta);
        tc_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; ++c) __stcg(mine + (q8 * 32 + c) * 128 + r, ok ? __uint_as_float(ta[c]) : 0.f);
      }
      __stcg(mine + 256 * 128 + r, m_ref);
      __stcg(mine + 256 * 128 + 128 + r, ok ? l : 0.f);
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");           // the four softmax warps
      if (r == 0) bars->last_flag = atomicAdd(p.counters + unit, 1) == n_parts - 1 ? 1 : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (bars->last_flag != 0) {
        __threadfence();
        float M = -INFINITY;
        for (int q = 0; q < n_parts; ++q) {
          const float* pp = base + static_cast<size_t>(q) * kPartFloats;
          if (__ldcg(pp + 256 * 128 + 128 + r) > 0.f) M = fmaxf(M, __ldcg(pp + 256 * 128 + r));
        }
        float wq[16];                                         // nsplit <= 16
        float L = 0.f;
        for (int q = 0; q < n_parts; ++q) {
          const float* pp = base + static_cast<size_t>(q) * kPartFloats;
          const float lq = __ldcg(pp + 256 * 128 + 128 + r);
          wq[q] = lq > 0.f ? exp2f(__ldcg(pp + 256 * 128 + r) - M) : 0.f;
          L += lq * wq[q];
        }
        const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll 1
        for (int c8 = 0; c8 < 32; ++c8) {
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int q = 0; q < n_parts; ++q) {
            const float* pp = base + static_cast<size_t>(q) * kPartFloats + (c8 * 8) * 128 + r;
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = fmaf(__ldcg(pp + j * 128), wq[q], acc[j]);
          }
          uint32_t pk[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            __nv_bfloat162 v2 = __floats2bfloat162_rn(acc[2 * j] * inv, acc[2 * j + 1] * inv);
            pk[j] = *reinterpret_cast<uint32_t*>(&v2);
          }
          *reinterpret_cast<uint4*>(orow + c8 * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        if (r == 0) p.counters[unit] = 0;                     // ready for the next launch
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// Per-token view of a ragged batch for the token mode: tok_seq[t] = sequence of query token t (-1 for rows
// that belong to none), tok_kvlen[t] = cache rows it attends to = kv_len - q_len + (t - q_start) + 1.
__global__ void mla_expand_tokens_kernel(const int32_t* __restrict__ q_start, const int32_t* __restrict__ q_len,
                                         const int32_t* __restrict__ kv_len, int B, int T, int32_t* __restrict__ tok_seq,
                                         int32_t* __restrict__ tok_kvlen) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  // sequences are laid out in order: binary search for the last q_start <= t
  int lo = 0, hi = B - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (q_start[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int off = t - q_start[lo];
  const bool in = off >= 0 && off < q_len[lo];
  tok_seq[t] = in ? lo : -1;
  tok_kvlen[t] = in ? kv_len[lo] - q_len[lo] + off + 1 : 0;
}

}  // namespace mlatc
}  // namespace mb

using namespace mb;

static float* g_mla_ws = nullptr;
static size_t g_mla_ws_bytes = 0;
static int* g_mla_counters = nullptr;
static int g_mla_n_counters = 0;
static int g_mla_split = 1;       // 0: never split the KV, 1: when the sequences leave SMs idle
// Workspace of the KV-split decode path: `ws` fp32 scratch for the partials, `counters` zeroed int32 (one per
// (sequence, 128-head block, output half)); both live as long as the process uses the kernel.
extern "C" void mb_set_mla_split_workspace(void* ws, size_t ws_bytes, int* counters, int n_counters) {
  g_mla_ws = static_cast<float*>(ws); g_mla_ws_bytes = ws_bytes; g_mla_counters = counters; g_mla_n_counters = n_counters;
}
extern "C" void mb_set_mla_split(int mode) { g_mla_split = mode; }
extern "C" size_t mb_mla_split_workspace_bytes(int num_sms) {
  // at most 2 * num_sms partials are in flight by construction of the split count
  return static_cast<size_t>(2) * (num_sms > 0 ? num_sms : 148) * mb::mlatc::kPartFloats * sizeof(float);
}

static int g_mla_tc = 1;
// 1 (default): decode steps with 512-wide latents and a multiple of 128 heads run on the tcgen05 kernel
extern "C" void mb_set_mla_tc(int on) { g_mla_tc = on; }
extern "C" int mb_mla_tc_usable(int T, int B, int n_heads, int R, int page_size) {
  return g_mla_tc && T == B && R == 512 && n_heads % 128 == 0 && page_size % 64 == 0;
}

// Decode-only absorbed MLA: T == B (one query token per sequence; sequences with q_len 0 are skipped),
// R = 512, n_heads % 128 == 0, page_size % 64 == 0. `cache` is one layer's [pages, page_size, 576] view with
// `page_stride` elements between pages (a multiple of 576); `n_pages` bounds the tensor map.
static int mla_tc_launch(const void* q_lat, const void* q_rope, void* out, const void* cache, long long page_stride,
                         long long n_pages, const int32_t* block_table, int bt_stride, const int32_t* q_start,
                         const int32_t* q_len, const int32_t* kv_len, int T, int B, int n_heads, int page_size,
                         float scale, int32_t* tok_scratch, int* err, cudaStream_t stream);

extern "C" int mb_mla_decode_tc(const void* q_lat, const void* q_rope, void* out, const void* cache,
                                long long page_stride, long long n_pages, const int32_t* block_table, int bt_stride,
                                const int32_t* q_start, const int32_t* q_len, const int32_t* kv_len, int T, int B,
                                int n_heads, int page_size, float scale, int* err, cudaStream_t stream) {
  return mla_tc_launch(q_lat, q_rope, out, cache, page_stride, n_pages, block_table, bt_stride, q_start, q_len, kv_len,
                       T, B, n_heads, page_size, scale, nullptr, err, stream);
}

// Any ragged batch (prefill, chunks, mixed steps) on the same tensor-core kernel: every query token is one CTA
// pair that walks the causal prefix of its sequence. `tok_scratch`: 2 * T int32 of device scratch. The KV tiles of
// a sequence are read once from HBM and again from L2 by the tokens that share them.
extern "C" int mb_mla_prefill_tc(const void* q_lat, const void* q_rope, void* out, const void* cache,
                                 long long page_stride, long long n_pages, const int32_t* block_table, int bt_stride,
                                 const int32_t* q_start, const int32_t* q_len, const int32_t* kv_len, int T, int B,
                                 int n_heads, int page_size, float scale, int32_t* tok_scratch, int* err,
                                 cudaStream_t stream) {
  if (tok_scratch == nullptr) return MB_ERR_SHAPE;
  return mla_tc_launch(q_lat, q_rope, out, cache, page_stride, n_pages, block_table, bt_stride, q_start, q_len, kv_len,
                       T, B, n_heads, page_size, scale, tok_scratch, err, stream);
}

static int mla_tc_launch(const void* q_lat, const void* q_rope, void* out, const void* cache, long long page_stride,
                         long long n_pages, const int32_t* block_table, int bt_stride, const int32_t* q_start,
                         const int32_t* q_len, const int32_t* kv_len, int T, int B, int n_heads, int page_size,
                         float scale, int32_t* tok_scratch, int* err, cudaStream_t stream) {
  using namespace mb::mlatc;
  if (T <= 0 || B <= 0) return MB_OK;
  if (n_heads % 128 || page_size % 64 || page_stride % LD || n_pages <= 0) return MB_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(q_lat) | reinterpret_cast<uintptr_t>(q_rope) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(cache)) & 15)
    return MB_ERR_ALIGN;
  const long long page_rows = page_stride / LD;
  const long long total_rows = (n_pages - 1) * page_rows + page_size;
  if (total_rows >= (1ll << 31)) return MB_ERR_SHAPE;
  Params p;
  p.out = static_cast<bf16*>(out);
  p.block_table = block_table; p.q_start = q_start; p.q_len = q_len; p.kv_len = kv_len;
  p.tok_seq = tok_scratch; p.tok_kvlen = tok_scratch ? tok_scratch + T : nullptr;
  p.nsplit = 1; p.ws = nullptr; p.counters = nullptr;
  const int units = B * (n_heads / 128) * 2;
  if (tok_scratch == nullptr && g_mla_split && g_mla_ws != nullptr && g_mla_counters != nullptr) {
    static int sms = 0;
    if (sms == 0) {
      int dev = 0;
      cudaGetDevice(&dev);
      if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    }
    // as many parts as fill the SMs once, at least four tiles each (the block table bounds the tiles of a sequence)
    const long long max_tiles = static_cast<long long>(bt_stride) * page_size / 64;
    long long ns = sms / units;
    if (ns > max_tiles / 4) ns = max_tiles / 4;
    if (ns > 16) ns = 16;
    while (ns > 1 && (static_cast<size_t>(units) * ns * kPartFloats * sizeof(float) > g_mla_ws_bytes)) --ns;
    if (ns > 1 && units <= g_mla_n_counters) {
      p.nsplit = static_cast<int>(ns); p.ws = g_mla_ws; p.counters = g_mla_counters;
    }
  }
  if (tok_scratch != nullptr)
    mla_expand_tokens_kernel<<<(T + 255) / 256, 256, 0, stream>>>(q_start, q_len, kv_len, B, T, tok_scratch, tok_scratch + T);
  p.err = err;
  p.page_rows = page_rows; p.bt_stride = bt_stride; p.n_heads = n_heads; p.page_size = page_size;
  p.scale_log2 = scale * 1.4426950408889634f;
  CUtensorMap tql, tqr, tkv;
  int rc = cached_tmap(&tql, q_lat, static_cast<uint64_t>(T) * n_heads, R, R, 128, 2);
  if (rc != MB_OK) return rc;
  rc = cached_tmap(&tqr, q_rope, static_cast<uint64_t>(T) * n_heads, DR, DR, 128, 2);
  if (rc != MB_OK) return rc;
  rc = cached_tmap(&tkv, cache, static_cast<uint64_t>(total_rows), LD, LD, 64, 2);
  if (rc != MB_OK) return rc;
  const size_t smem = kQBlocks * kQBlockBytes + kSlots * kSlotBytes + kPBytes + sizeof(Bars);
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(mla_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess)
      return MB_ERR_LAUNCH;
    configured.done();
  }
  return launch_k(mla_tc_kernel, dim3(tok_scratch ? T : B * p.nsplit, n_heads / 128, 2), dim3(kThreads), smem, stream, tql, tqr,
                  tkv, p) ==
                 cudaSuccess
             ? MB_OK
             : MB_ERR_LAUNCH;
}
