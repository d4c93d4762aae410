// State-space layer kernels for ragged (variable-length) batches: causal depthwise conv1d,
// the Mamba-1 selective scan and the Mamba-2 SSD recurrence, each carrying per-sequence state so the
// same kernel serves prefill chunks and single-token decode.
//
// Sequences are rows [cu_seqlens[s], cu_seqlens[s+1]) of the token-major inputs. State tensors are
// indexed by `state_idx[s]` (a slot per live request; -1 = no state: start from zero, write nothing),
// are read when `has_init[s]` is non-zero and always written back.
//
// These are the time-sequential forms: one thread (or one thread per state column) walks a sequence
// and keeps the recurrent state in registers. They are bandwidth-bound for decode and for short
// chunks; a chunked (matmul-form) SSD prefill is not built.
//
// Reference counterparts: max/kernels/src/state_space/causal_conv1d.mojo (varlen fwd + update),
// selective_scan.mojo (selective_scan_fwd / _update) and the Mamba-2 SSD kernels of the same package,
// wrapped by max/python/max/nn/state_space/.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../common/api.h"

namespace mb {
namespace ssm {

__device__ __forceinline__ float silu(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// y[t, d] = act(bias[d] + sum_k w[d, k] * x[t - (W-1) + k, d]); tokens before the sequence start come
// from conv_state[slot, d, :] (the last W-1 inputs of the previous chunk). One thread per channel walks
// the sequence with a sliding window in registers. W <= 8.
template <int W>
__global__ void causal_conv1d_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                     const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y,
                                     float* __restrict__ conv_state, const int* __restrict__ cu_seqlens,
                                     const int* __restrict__ state_idx, const int* __restrict__ has_init,
                                     int D, int ldx, int ldy, int act) {
  const int s = blockIdx.y;
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  if (d >= D) return;
  const int t0 = cu_seqlens[s], t1 = cu_seqlens[s + 1];
  const int slot = state_idx ? state_idx[s] : -1;
  float win[W];
  float wk[W];
#pragma unroll
  for (int k = 0; k < W; ++k) wk[k] = __bfloat162float(w[d * W + k]);
#pragma unroll
  for (int k = 0; k < W - 1; ++k)
    win[k + 1] = (slot >= 0 && has_init && has_init[s]) ? conv_state[(static_cast<size_t>(slot) * D + d) * (W - 1) + k]
                                                        : 0.f;
  const float b = bias ? __bfloat162float(bias[d]) : 0.f;
  for (int t = t0; t < t1; ++t) {
#pragma unroll
    for (int k = 0; k < W - 1; ++k) win[k] = win[k + 1];
    win[W - 1] = __bfloat162float(x[static_cast<size_t>(t) * ldx + d]);
    float acc = b;
#pragma unroll
    for (int k = 0; k < W; ++k) acc = fmaf(wk[k], win[k], acc);
    if (act) acc = silu(acc);
    y[static_cast<size_t>(t) * ldy + d] = __float2bfloat16(acc);
  }
  if (slot >= 0) {
#pragma unroll
    for (int k = 0; k < W - 1; ++k)
      conv_state[(static_cast<size_t>(slot) * D + d) * (W - 1) + k] = win[k + 1];
  }
}

// Mamba-1 selective scan. Per channel d and state n:
//   dt = softplus(delta[t, d] + dt_bias[d]);  h = exp(dt * A[d, n]) * h + dt * B[t, n] * u[t, d]
//   y[t, d] = sum_n C[t, n] * h + Dskip[d] * u[t, d];   y *= silu(z[t, d]) when z is given
// One thread per channel, N (<= 32, compile-time) states in registers; B_t / C_t rows are staged in
// shared memory once per time step for the whole block.
template <int N>
__global__ void selective_scan_kernel(const __nv_bfloat16* __restrict__ u, const __nv_bfloat16* __restrict__ delta,
                                      const float* __restrict__ A, const __nv_bfloat16* __restrict__ B,
                                      const __nv_bfloat16* __restrict__ C, const float* __restrict__ Dskip,
                                      const __nv_bfloat16* __restrict__ z, const float* __restrict__ dt_bias,
                                      __nv_bfloat16* __restrict__ y, float* __restrict__ ssm_state,
                                      const int* __restrict__ cu_seqlens, const int* __restrict__ state_idx,
                                      const int* __restrict__ has_init, int D, int ld_u, int ld_bc,
                                      int dt_softplus) {
  __shared__ float sB[N], sC[N];
  const int s = blockIdx.y;
  const int d = blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = d < D;
  const int t0 = cu_seqlens[s], t1 = cu_seqlens[s + 1];
  const int slot = state_idx ? state_idx[s] : -1;
  float h[N], a[N];
#pragma unroll
  for (int n = 0; n < N; ++n) {
    a[n] = live ? A[static_cast<size_t>(d) * N + n] : 0.f;
    h[n] = (live && slot >= 0 && has_init && has_init[s]) ? ssm_state[(static_cast<size_t>(slot) * D + d) * N + n] : 0.f;
  }
  const float dsk = (live && Dskip) ? Dskip[d] : 0.f;
  const float dtb = (live && dt_bias) ? dt_bias[d] : 0.f;
  for (int t = t0; t < t1; ++t) {
    __syncthreads();
    if (threadIdx.x < N) {
      sB[threadIdx.x] = __bfloat162float(B[static_cast<size_t>(t) * ld_bc + threadIdx.x]);
      sC[threadIdx.x] = __bfloat162float(C[static_cast<size_t>(t) * ld_bc + threadIdx.x]);
    }
    __syncthreads();
    if (!live) continue;
    const float ut = __bfloat162float(u[static_cast<size_t>(t) * ld_u + d]);
    float dt = __bfloat162float(delta[static_cast<size_t>(t) * ld_u + d]) + dtb;
    if (dt_softplus) dt = softplus(dt);
    float acc = dsk * ut;
#pragma unroll
    for (int n = 0; n < N; ++n) {
      h[n] = __expf(dt * a[n]) * h[n] + dt * sB[n] * ut;
      acc = fmaf(sC[n], h[n], acc);
    }
    if (z) acc *= silu(__bfloat162float(z[static_cast<size_t>(t) * ld_u + d]));
    y[static_cast<size_t>(t) * ld_u + d] = __float2bfloat16(acc);
  }
  if (live && slot >= 0) {
#pragma unroll
    for (int n = 0; n < N; ++n) ssm_state[(static_cast<size_t>(slot) * D + d) * N + n] = h[n];
  }
}

// Mamba-2 SSD recurrence. Heads H of width P, state size N, G groups of B/C (H % G == 0):
//   dt = softplus(dt_in[t, h] + dt_bias[h]);  S[p, n] = exp(dt * A[h]) * S[p, n] + dt * x[t, h, p] * B[t, g, n]
//   y[t, h, p] = sum_n S[p, n] * C[t, g, n] + D[h] * x[t, h, p]
// One CTA per (sequence, head): thread (p, j) owns the state columns n = j, j + J, ... of row p
// (J = blockDim.x / P); the row's output is reduced across its J threads with shuffles (J <= 32, power of 2).
template <int NPT>
__global__ void ssd_scan_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dt_in,
                                const float* __restrict__ A, const __nv_bfloat16* __restrict__ B,
                                const __nv_bfloat16* __restrict__ C, const float* __restrict__ Dskip,
                                const float* __restrict__ dt_bias, __nv_bfloat16* __restrict__ y,
                                float* __restrict__ ssm_state, const int* __restrict__ cu_seqlens,
                                const int* __restrict__ state_idx, const int* __restrict__ has_init,
                                int H, int P, int N, int G, int J, int dt_softplus) {
  extern __shared__ float sbc[];   // B_t[N] | C_t[N]
  const int s = blockIdx.y, hd = blockIdx.x;
  const int g = hd / (H / G);
  const int p = threadIdx.x / J, j = threadIdx.x % J;
  const int t0 = cu_seqlens[s], t1 = cu_seqlens[s + 1];
  const int slot = state_idx ? state_idx[s] : -1;
  float S[NPT];
  float* st = slot >= 0 ? ssm_state + ((static_cast<size_t>(slot) * H + hd) * P + p) * N : nullptr;
#pragma unroll
  for (int i = 0; i < NPT; ++i) {
    const int n = j + i * J;
    S[i] = (st && has_init && has_init[s] && n < N) ? st[n] : 0.f;
  }
  const float a = A[hd];
  const float dsk = Dskip ? Dskip[hd] : 0.f;
  const float dtb = dt_bias ? dt_bias[hd] : 0.f;
  for (int t = t0; t < t1; ++t) {
    __syncthreads();
    for (int n = threadIdx.x; n < N; n += blockDim.x) {
      sbc[n] = __bfloat162float(B[(static_cast<size_t>(t) * G + g) * N + n]);
      sbc[N + n] = __bfloat162float(C[(static_cast<size_t>(t) * G + g) * N + n]);
    }
    __syncthreads();
    float dt = __bfloat162float(dt_in[static_cast<size_t>(t) * H + hd]) + dtb;
    if (dt_softplus) dt = softplus(dt);
    const float decay = __expf(dt * a);
    const float xt = __bfloat162float(x[(static_cast<size_t>(t) * H + hd) * P + p]);
    const float dx = dt * xt;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = j + i * J;
      if (n < N) {
        S[i] = decay * S[i] + dx * sbc[n];
        acc = fmaf(S[i], sbc[N + n], acc);
      }
    }
    for (int o = J >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (j == 0) y[(static_cast<size_t>(t) * H + hd) * P + p] = __float2bfloat16(acc + dsk * xt);
  }
  if (st) {
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = j + i * J;
      if (n < N) st[n] = S[i];
    }
  }
}

}  // namespace ssm
}  // namespace mb

using namespace mb::ssm;

extern "C" int mb_causal_conv1d_varlen(const void* x, const void* w, const void* bias, void* y, float* conv_state,
                                       const int* cu_seqlens, const int* state_idx, const int* has_init,
                                       int n_seqs, int D, int width, int ldx, int ldy, int act,
                                       cudaStream_t stream) {
  if (n_seqs <= 0 || D <= 0) return MB_OK;
  dim3 grid((D + 127) / 128, n_seqs);
#define MB_CONV(Wv)                                                                                              \
  causal_conv1d_kernel<Wv><<<grid, 128, 0, stream>>>(                                                            \
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),                                \
      static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(y), conv_state, cu_seqlens, state_idx, \
      has_init, D, ldx, ldy, act)
  switch (width) {
    case 2: MB_CONV(2); break;
    case 3: MB_CONV(3); break;
    case 4: MB_CONV(4); break;
    case 8: MB_CONV(8); break;
    default: return MB_ERR_SHAPE;
  }
#undef MB_CONV
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_selective_scan_varlen(const void* u, const void* delta, const float* A, const void* B,
                                        const void* C, const float* Dskip, const void* z, const float* dt_bias,
                                        void* y, float* ssm_state, const int* cu_seqlens, const int* state_idx,
                                        const int* has_init, int n_seqs, int D, int N, int ld_u, int ld_bc,
                                        int dt_softplus, cudaStream_t stream) {
  if (n_seqs <= 0 || D <= 0) return MB_OK;
  dim3 grid((D + 127) / 128, n_seqs);
#define MB_SCAN(Nv)                                                                                             \
  selective_scan_kernel<Nv><<<grid, 128, 0, stream>>>(                                                          \
      static_cast<const __nv_bfloat16*>(u), static_cast<const __nv_bfloat16*>(delta), A,                        \
      static_cast<const __nv_bfloat16*>(B), static_cast<const __nv_bfloat16*>(C), Dskip,                        \
      static_cast<const __nv_bfloat16*>(z), dt_bias, static_cast<__nv_bfloat16*>(y), ssm_state, cu_seqlens,     \
      state_idx, has_init, D, ld_u, ld_bc, dt_softplus)
  switch (N) {
    case 8: MB_SCAN(8); break;
    case 16: MB_SCAN(16); break;
    case 32: MB_SCAN(32); break;
    default: return MB_ERR_SHAPE;
  }
#undef MB_SCAN
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}

extern "C" int mb_ssd_scan_varlen(const void* x, const void* dt, const float* A, const void* B, const void* C,
                                  const float* Dskip, const float* dt_bias, void* y, float* ssm_state,
                                  const int* cu_seqlens, const int* state_idx, const int* has_init, int n_seqs,
                                  int H, int P, int N, int G, int dt_softplus, cudaStream_t stream) {
  if (n_seqs <= 0 || H <= 0) return MB_OK;
  if (P <= 0 || P > 256 || (P & (P - 1)) || G <= 0 || H % G || N <= 0 || N > 256) return MB_ERR_SHAPE;
  int J = 256 / P;            // threads per state row
  if (J > 32) J = 32;
  if (J < 1) J = 1;
  const int npt = (N + J - 1) / J;
  dim3 grid(H, n_seqs);
  const int threads = P * J;
  const size_t smem = 2 * static_cast<size_t>(N) * sizeof(float);
#define MB_SSD(NPTv)                                                                                            \
  ssd_scan_kernel<NPTv><<<grid, threads, smem, stream>>>(                                                       \
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dt), A,                           \
      static_cast<const __nv_bfloat16*>(B), static_cast<const __nv_bfloat16*>(C), Dskip, dt_bias,               \
      static_cast<__nv_bfloat16*>(y), ssm_state, cu_seqlens, state_idx, has_init, H, P, N, G, J, dt_softplus)
  if (npt <= 4) MB_SSD(4);
  else if (npt <= 8) MB_SSD(8);
  else if (npt <= 16) MB_SSD(16);
  else if (npt <= 32) MB_SSD(32);
  else if (npt <= 64) MB_SSD(64);
  else return MB_ERR_SHAPE;
#undef MB_SSD
  return cudaGetLastError() == cudaSuccess ? MB_OK : MB_ERR_LAUNCH;
}
