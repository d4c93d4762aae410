// Split-K bf16 GEMM entry point that performs no device allocation of any kind.
//
// This entry point has no counterpart in the reference; it exists for callers of this
// library that are not in a position to allocate device memory:
//
//   * a serving process that has already handed every free byte of HBM to its KV cache, so a
//     later cudaMalloc for a GEMM workspace would fail (or force the cache to be shrunk);
//   * latency-critical threads, for which cudaMalloc / cudaFree are off limits because both
//     serialise against all work in flight on the device;
//   * plain-C hosts that embed the kernel library without torch and own no allocator.
//
// Such callers pass only inputs and outputs. The fp32 split-K partial sums live in a
// file-scope `static __device__` array inside the library (MB_SPLITK_STATIC_MAX_FLOATS
// floats = 16 MiB, resident on every GPU that loads the library until the process exits).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#define MB_SPLITK_STATIC_MAX_FLOATS (4u << 20)

#ifdef __cplusplus
extern "C" {
#endif

// Y[M, N] (bf16) = X[M, K] · W[N, K]^T (+ R when R != NULL), computed as `splits` K-slices
// whose fp32 partials are summed in a second kernel. Same numerics and tile shapes as
// mb_gemm_bf16 with a caller-provided workspace.
//
// Returns MB_OK, or MB_ERR_TOO_LARGE when splits * M * N exceeds
// MB_SPLITK_STATIC_MAX_FLOATS (nothing is launched then), or another MB_ERR_* code.
//
// Rules for callers:
//   * The first call on each device resolves the device address of the scratch array (with
//     that device current), clears the library's error word and waits once for the whole device
//     (cudaDeviceSynchronize) so that the clear is ordered before GEMMs on any stream. Make
//     that first call early, outside any stream capture.
//   * No cudaMalloc, cudaFree or allocating library routine is called, on the first call or
//     later.
//   * All calls on one device share the one scratch array. Calls that may overlap on the GPU
//     (different streams, or different host threads) race on it; serialise them.
//   * The scratch keeps whatever the previous call left. This entry point needs no zeroed
//     scratch (every partial it reads it has written in the same call), and it resets the
//     error word it uses at set-up only.
//   * `bn` <= 0 picks the token-tile width automatically.
int mb_gemm_bf16_splitk_static(const void* X, const void* W, void* Y, const void* R, int M, int N,
                               int K, int ldx, int ldw, int ldy, int ldr, int splits, int bn,
                               cudaStream_t stream);

// Reads (and clears) the error word the static entry point hands to its kernels: non-zero means
// a bounded barrier wait inside a kernel timed out. Calls cudaDeviceSynchronize() first, so work on
// every stream of the device (non-blocking streams too) has finished when the word is read; do not
// call it from a thread that must not block, nor during stream capture.
int mb_gemm_bf16_splitk_static_error(void);

#ifdef __cplusplus
}
#endif
