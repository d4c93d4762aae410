// Kernel launch helper with optional programmatic dependent launch (PDL).
//
// With PDL on, a kernel is allowed to start while its predecessor on the stream is still
// running; it executes `griddepcontrol.wait` (pdl_wait() in ptx.cuh) before touching global
// memory, which returns once the predecessor has completed and its writes are visible. What
// overlaps is the launch latency and the kernel's private prologue (barrier init, TMEM allocation,
// descriptor prefetch), which is most of the fixed cost of the small decode-step kernels.
// Only kernels that call pdl_wait() may be launched through launch_k().
#pragma once
#include <cuda_runtime.h>

namespace mb {

// Function attributes such as the dynamic shared-memory opt-in are per device. A launcher keeps one of these in
// a function-local static and sets the attribute the first time it runs on each device of the process
// (setting it twice is harmless, so no lock is taken).
struct PerDeviceOnce {
  bool seen[64] = {};
  int dev = -1;
  bool needed() {
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { dev = -1; return true; }
    return !seen[dev];
  }
  void done() { if (dev >= 0) seen[dev] = true; }
};

// process-wide switch (set once by the engine; see mb_set_pdl in elementwise.cu)
bool pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                            Args&&... args) {
  if (!pdl_enabled()) {
    kern<<<grid, block, smem, stream>>>(static_cast<KArgs>(args)...);
    return cudaGetLastError();
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

}  // namespace mb
