// Paged GQA prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), head_dim 128.
//
// One CTA owns 128 query rows of one (sequence, KV head): 128/G consecutive tokens x the G query
// heads that share the KV head (GQA packing puts them on the MMA M dimension). It walks the
// sequence's KV pages 64 tokens at a time:
//
//   warp 0      TMA producer: K tile and V tile of 64 tokens (two 64-column boxes each, 128B swizzle)
//               into a 4-stage ring
//   warp 1      MMA issuer:   S = Q . K^T   (M=128, N=64, K=128; fp32 in TMEM, two S buffers so the
//               next tile's scores are computed while the softmax warps work on this one)
//                             O  += P . V   (M=128, N=128, K=64; V is read as an MN-major operand
//               straight from the row-major KV page, no transpose pass)
//   warps 2-9   two softmax groups of four warps; group g owns the KV tiles g, g+2, ... with its own
//               accumulator and P buffer, so two score -> probability -> P.V chains are in flight; the
//               partial results are merged at the end. Inside a group:
//               one query row per thread (TMEM lane = row): read S, mask, running max / sum, write
//               P (bf16) into shared memory in the swizzled K-major layout the MMA reads. The output
//               accumulates in TMEM across tiles; it is rescaled only when a row's maximum has grown by
//               more than 2^8 since the reference maximum was taken (exact after the final 1/l
//               normalisation, because P is always computed against that reference), so the common
//               tile costs no read-modify-write of the accumulator
//
// All mbarrier waits are bounded; a timed-out wait raises the error word, and the CTA drains,
// frees its TMEM and leaves. Decode rows (one token per sequence) stay on the mma.sync kernel of
// attention_tma.cu: with one token only G of the 128 MMA rows would be used.
//
// Reference counterpart: max/kernels/src/nn/attention/gpu/nvidia/sm100/attention.mojo (FA4 prefill).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"
#include "../common/launch.h"
#include "../common/ptx.cuh"
#include "gemm_common.h"

namespace mb {
namespace atc {

typedef __nv_bfloat16 bf16;
constexpr int HD = 128;
constexpr int kStages = 4;     // K/V tiles are prefetched three ahead
constexpr int kThreads = 320;  // warp 0 TMA, warp 1 MMA, warps 2-5 softmax group 0, warps 6-9 softmax group 1
constexpr int kQBytes = 2 * 128 * 128;        // two 64-column chunks of 128 rows x 128 B
constexpr int kTileBytes = 2 * 64 * 128;      // K (or V) tile: two chunks of 64 rows x 128 B
constexpr int kStageBytes = 2 * kTileBytes;   // K + V
constexpr int kPBytes = 128 * 128;            // P of one group: 128 rows x 64 bf16
constexpr uint32_t kTmemCols = 512;           // S0 | S1 (64 each) | O group 0 (128) | O group 1 (128)

struct Params {
  const bf16* q;
  bf16* out;
  const int32_t* block_table;
  const int32_t* q_start;
  const int32_t* q_len;
  const int32_t* kv_len;
  const int32_t* tile_seq;
  const int32_t* tile_q0;
  int* err;
  long long k_off_rows, v_off_rows, page_rows;
  int ldq, ldo, bt_stride, page_size, n_tiles, G;
  float scale_log2;
};

struct Bars {
  uint64_t kv_full[kStages];
  uint64_t kv_empty[kStages];
  uint64_t s_full[2];
  uint64_t s_free[2];
  uint64_t p_full[2];
  uint64_t pv_full[2];
  uint32_t tmem_base;
  int abort_word;
  float merge_m[128];   // group 1's reference maximum and sum per row, for the final merge
  float merge_l[128];
};

// MN-major operand with 128B swizzle: rows of 64 contiguous MN elements (128 B), 8 consecutive K rows
// form one 1024 B swizzle atom (SBO = stride between atoms along K), the next 64 MN elements live
// LBO bytes away.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(const void* smem_tile, uint32_t lbo_bytes,
                                                       uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_u32(smem_tile) & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>(lbo_bytes >> 4) << 16;
  d |= static_cast<uint64_t>(sbo_bytes >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__global__ void __launch_bounds__(kThreads, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmKV, const Params p) {
  // No alignment slack (208 KiB of tiles + barriers per CTA). The dynamic shared memory window starts
  // 1024-byte aligned (there is no static shared memory in this kernel); should a future toolchain place
  // it elsewhere the kernel reports it instead of computing garbage.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem_raw) & 1023u) {
    if (threadIdx.x == 0 && p.err) atomicCAS(p.err, 0, 799);
    return;
  }
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + kQBytes;                     // [stage][K chunk0 | K chunk1 | V chunk0 | V chunk1]
  uint8_t* sP = sKV + kStages * kStageBytes;        // [group][128 rows x 128 B]
  Bars* bars = reinterpret_cast<Bars*>(sP + 2 * kPBytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.y;
  const int G = p.G;
  const int tok_per_cta = 128 / G;

  pdl_wait();
  pdl_trigger();
  const int seq = p.tile_seq[blockIdx.x];
  const int tq0 = p.tile_q0[blockIdx.x];
  if (tq0 % tok_per_cta != 0) return;  // the plan lists 64-row tiles; every second one is covered by its predecessor
  const int qs = p.q_start[seq], ql = p.q_len[seq], kl = p.kv_len[seq];
  const int32_t* bt = p.block_table + static_cast<int64_t>(seq) * p.bt_stride;
  int last_tq = tq0 + tok_per_cta;
  if (last_tq > ql) last_tq = ql;
  const int kv_hi = kl - ql + last_tq;
  const int ntiles = (kv_hi + 63) / 64;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->kv_full[s], 1);
      mbar_init(&bars->kv_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&bars->s_full[b], 1);
      mbar_init(&bars->s_free[b], 4);
      mbar_init(&bars->p_full[b], 4);
      mbar_init(&bars->pv_full[b], 1);
    }
    bars->abort_word = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  if (warp >= 2) {
    // Q rows of this CTA into shared memory, K-major with 128B swizzle (row r, 16 B piece c); each softmax
    // group copies one of the two 64-column chunks
    const int grp = (warp - 2) >> 2;
    const int r = (warp & 3) * 32 + lane;
    const int tq = tq0 + r / G, head = kvh * G + r % G;
    const bool valid = tq < ql;
    const bf16* src = p.q + static_cast<int64_t>(qs + (valid ? tq : 0)) * p.ldq + head * HD + grp * 64;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (valid) v = *reinterpret_cast<const uint4*>(src + c * 8);
      *reinterpret_cast<uint4*>(sQ + grp * 16384 + r * 128 + ((c ^ (r & 7)) << 4)) = v;
    }
    fence_proxy_async_smem();
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
      // pages are walked (no division) and the next block-table entry is loaded ahead of the wait for a free
      // stage: this loop is on the latency path of the KV ring
      int page_i = 0, page_off = 0;
      int32_t page_next = ntiles > 0 ? bt[0] : 0;
      const long long head_row = static_cast<long long>(kvh) * p.page_size;
      for (int t = 0; t < ntiles; ++t) {
        const int s = t % kStages;
        const uint32_t ph = (t / kStages) & 1;
        const long long row = static_cast<long long>(page_next) * p.page_rows + head_row + page_off;
        page_off += 64;
        if (page_off == p.page_size) { page_off = 0; ++page_i; }
        if (t + 1 < ntiles && page_off == 0) page_next = bt[page_i];
        if (!mbar_wait(&bars->kv_empty[s], ph ^ 1, abort_word, p.err, 701)) break;
        uint8_t* dK = sKV + s * kStageBytes;
        uint8_t* dV = dK + kTileBytes;
        mbar_arrive_expect_tx(&bars->kv_full[s], kStageBytes);
        tma_load_2d(dK, &tmKV, &bars->kv_full[s], 0, static_cast<int32_t>(p.k_off_rows + row));
        tma_load_2d(dK + 8192, &tmKV, &bars->kv_full[s], 64, static_cast<int32_t>(p.k_off_rows + row));
        tma_load_2d(dV, &tmKV, &bars->kv_full[s], 0, static_cast<int32_t>(p.v_off_rows + row));
        tma_load_2d(dV + 8192, &tmKV, &bars->kv_full[s], 64, static_cast<int32_t>(p.v_off_rows + row));
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = umma_idesc(128, 64, 1, 1);
      const uint32_t idesc_pv = umma_idesc(128, 128, 1, 1) | (1u << 16);   // B operand (V) is MN-major
      bool ok = true;
      auto issue_s = [&](int t) {
        const int s = t % kStages, b = t & 1;
        ok = ok && mbar_wait(&bars->kv_full[s], (t / kStages) & 1, abort_word, p.err, 702);
        ok = ok && mbar_wait(&bars->s_free[b], ((t >> 1) & 1) ^ 1, abort_word, p.err, 703);
        if (!ok) return;
        tc_fence_after();
        const uint8_t* sK = sKV + s * kStageBytes;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint64_t da = umma_desc_sw128(sQ + (k >> 2) * 16384) + static_cast<uint64_t>((k & 3) * 2);
          const uint64_t db = umma_desc_sw128(sK + (k >> 2) * 8192) + static_cast<uint64_t>((k & 3) * 2);
          umma_bf16(tmem_base + b * 64, da, db, idesc_s, k > 0 ? 1u : 0u);
        }
        tc_commit(&bars->s_full[b]);
      };
      if (ntiles > 0) issue_s(0);
      for (int t = 0; t < ntiles && ok; ++t) {
        if (t + 1 < ntiles) issue_s(t + 1);
        const int g = t & 1, u = t >> 1;       // tile t belongs to softmax group g, its u-th tile
        ok = ok && mbar_wait(&bars->p_full[g], u & 1, abort_word, p.err, 704);
        if (!ok) break;
        tc_fence_after();
        const int s = t % kStages;
        const uint8_t* sV = sKV + s * kStageBytes + kTileBytes;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint64_t da = umma_desc_sw128(sP + g * kPBytes) + static_cast<uint64_t>(k * 2);
          const uint64_t db = umma_desc_mn_sw128(sV + k * 2048, 8192, 1024);
          umma_bf16(tmem_base + 128 + g * 128, da, db, idesc_pv, (u > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&bars->pv_full[g]);
        tc_commit(&bars->kv_empty[s]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax groups
    // Group g takes the KV tiles t = g, g+2, ... of the same 128 query rows, with its own reference
    // maximum, sum and TMEM accumulator; the two partial results are merged at the end. Two groups keep
    // two dependent chains (scores -> probabilities -> P.V) in flight per CTA.
    const int grp = (warp - 2) >> 2;
    const int quad = warp & 3;
    const int r = quad * 32 + lane;
    const int tq = tq0 + r / G, head = kvh * G + r % G;
    const int limit = tq < ql ? kl - ql + tq : -1;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t o_addr = lane_addr + 128 + grp * 128;
    uint8_t* myP = sP + grp * kPBytes;
    float m_ref = 0.f, l = 0.f;       // P and l are relative to m_ref (a lagging running maximum)
    bool ok = true;
    const int n_mine = (ntiles - grp + 1) / 2;
    for (int u = 0; u < n_mine && ok; ++u) {
      const int t = 2 * u + grp;
      ok = mbar_wait(&bars->s_full[grp], u & 1, abort_word, p.err, 706);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[2][32];
      tmem_ld_32x32(lane_addr + grp * 64, sr[0]);
      tmem_ld_32x32(lane_addr + grp * 64 + 32, sr[1]);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->s_free[grp]);
      const int kv0 = t * 64;
      // row maximum of the raw scores (four independent chains); only tiles that touch the causal
      // diagonal or the end of the sequence need the mask
      float mxa[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (kv0 + 63 <= limit) {
#pragma unroll
        for (int c = 0; c < 64; ++c) mxa[c & 3] = fmaxf(mxa[c & 3], __uint_as_float(sr[c >> 5][c & 31]));
      } else {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const float v = (kv0 + c) <= limit ? __uint_as_float(sr[c >> 5][c & 31]) : -INFINITY;
          sr[c >> 5][c & 31] = __float_as_uint(v);
          mxa[c & 3] = fmaxf(mxa[c & 3], v);
        }
      }
      const float mx = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])) * p.scale_log2;   // scale > 0
      // this group's previous P . V has retired: its P buffer is free and its accumulator is quiescent
      if (u > 0) {
        ok = mbar_wait(&bars->pv_full[grp], (u - 1) & 1, abort_word, p.err, 707);
        if (!ok) break;
        tc_fence_after();
      }
      bool grow = false;
      if (u == 0) {
        m_ref = mx == -INFINITY ? 0.f : mx;
      } else {
        grow = mx - m_ref > 8.0f;      // probabilities would exceed 2^8: move the reference
      }
      if (__any_sync(0xffffffffu, grow)) {
        // rescale this warp's 32 accumulator rows (factor 1 for rows whose reference stays)
        const float factor = grow ? exp2f(m_ref - mx) : 1.0f;
        if (grow) { m_ref = mx; l *= factor; }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t tr[32];
          tmem_ld_32x32(o_addr + q4 * 32, tr);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c) tr[c] = __float_as_uint(__uint_as_float(tr[c]) * factor);
          tmem_st_32x32(o_addr + q4 * 32, tr);
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
        *reinterpret_cast<uint4*>(myP + r * 128 + ((c8 ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l += (la[0] + la[1]) + (la[2] + la[3]);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->p_full[grp]);
    }
    if (ok && n_mine > 0) ok = mbar_wait(&bars->pv_full[grp], (n_mine - 1) & 1, abort_word, p.err, 708);
    // ---- merge the two groups' partial results (group 1 publishes, group 0 combines and stores)
    const bool has_b = ntiles >= 2;      // CTA-uniform: group 1 worked on at least one tile
    if (grp == 1) {
      bars->merge_m[r] = m_ref;
      bars->merge_l[r] = n_mine > 0 ? l : 0.f;
    }
    tc_fence_before();
    asm volatile("bar.sync 1, 256;" ::: "memory");     // the eight softmax warps
    tc_fence_after();
    if (grp == 0 && ok && n_mine > 0 && *abort_word == 0) {
      float wa = 1.f, wb = 0.f;
      if (has_b) {
        const float mb_ = bars->merge_m[r], lb = bars->merge_l[r];
        const float mm = fmaxf(m_ref, mb_);
        wa = exp2f(m_ref - mm);
        wb = lb > 0.f ? exp2f(mb_ - mm) : 0.f;
        l = l * wa + lb * wb;
      }
      const float inv = l > 0.f ? 1.f / l : 0.f;
      wa *= inv;
      wb *= inv;
      bf16* orow = p.out + static_cast<int64_t>(qs + (tq < ql ? tq : 0)) * p.ldo + head * HD;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        uint32_t ta[32], tb[32];
        tmem_ld_32x32(lane_addr + 128 + q4 * 32, ta);          // warp-collective: every lane takes part
        if (has_b) tmem_ld_32x32(lane_addr + 256 + q4 * 32, tb);
        tc_wait_ld();
        if (tq < ql) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t pk[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float x0 = __uint_as_float(ta[c * 8 + 2 * j]) * wa, x1 = __uint_as_float(ta[c * 8 + 2 * j + 1]) * wa;
              if (has_b) {
                x0 = fmaf(__uint_as_float(tb[c * 8 + 2 * j]), wb, x0);
                x1 = fmaf(__uint_as_float(tb[c * 8 + 2 * j + 1]), wb, x1);
              }
              __nv_bfloat162 v2 = __floats2bfloat162_rn(x0, x1);
              pk[j] = *reinterpret_cast<uint32_t*>(&v2);
            }
            *reinterpret_cast<uint4*>(orow + q4 * 32 + c * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        }
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

}  // namespace atc
}  // namespace mb

using namespace mb;

// Prefill tiles of a ragged batch on the tcgen05 kernel. Same KV addressing as mb_paged_attention_tma
// (kv_base viewed as [total_rows, 128]); head_dim 128, G = n_q / n_kv in {1, 2, 4, 8, 16}, page_size % 64 == 0.
// tile_seq / tile_q0 is the plan of 64-row tiles; CTAs take pairs of them.
extern "C" int mb_paged_attention_prefill_tc(const void* q, int ldq, void* out, int ldo, const void* kv_base,
                                             long long total_rows, long long k_off_rows, long long v_off_rows,
                                             long long page_rows, const int32_t* block_table, int bt_stride,
                                             const int32_t* q_start, const int32_t* q_len, const int32_t* kv_len,
                                             const int32_t* tile_seq, const int32_t* tile_q0, int n_tiles, int n_q,
                                             int n_kv, int head_dim, int page_size, float scale, int* err,
                                             cudaStream_t stream) {
  using namespace mb::atc;
  if (n_tiles <= 0) return MB_OK;
  if (head_dim != 128 || n_kv <= 0 || n_q % n_kv || page_size % 64 || total_rows >= (1ll << 31)) return MB_ERR_SHAPE;
  const int G = n_q / n_kv;
  if (G > 16 || (G & (G - 1))) return MB_ERR_SHAPE;
  if (reinterpret_cast<uintptr_t>(kv_base) & 15 || ldq % 8 || ldo % 8) return MB_ERR_ALIGN;
  Params p;
  p.q = static_cast<const bf16*>(q);
  p.out = static_cast<bf16*>(out);
  p.block_table = block_table;
  p.q_start = q_start; p.q_len = q_len; p.kv_len = kv_len;
  p.tile_seq = tile_seq; p.tile_q0 = tile_q0;
  p.err = err;
  p.k_off_rows = k_off_rows; p.v_off_rows = v_off_rows; p.page_rows = page_rows;
  p.ldq = ldq; p.ldo = ldo; p.bt_stride = bt_stride; p.page_size = page_size; p.n_tiles = n_tiles; p.G = G;
  p.scale_log2 = scale * 1.4426950408889634f;
  CUtensorMap tm;
  const int rc = cached_tmap(&tm, kv_base, static_cast<uint64_t>(total_rows), head_dim, head_dim, 64, 2);
  if (rc != MB_OK) return rc;
  const size_t smem = kQBytes + kStages * kStageBytes + 2 * kPBytes + sizeof(Bars);
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) !=
        cudaSuccess)
      return MB_ERR_LAUNCH;
    configured.done();
  }
  return launch_k(attn_tc_kernel, dim3(n_tiles, n_kv), dim3(kThreads), smem, stream, tm, p) == cudaSuccess
             ? MB_OK
             : MB_ERR_LAUNCH;
}
