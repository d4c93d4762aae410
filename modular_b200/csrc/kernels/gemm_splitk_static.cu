// See gemm_splitk_static.h. The scratch is a file-scope device array; host code may not use
// its name as a pointer (on the host the name is only a stand-in symbol), so the device
// address is looked up once per device with cudaGetSymbolAddress and cached.
#include "gemm_splitk_static.h"

#include <mutex>

#include "../common/api.h"

static __device__ __align__(256) float g_splitk_scratch[MB_SPLITK_STATIC_MAX_FLOATS];
static __device__ __align__(256) int g_splitk_err;

namespace {

constexpr int kMaxDevices = 64;
struct DeviceSlots {
  float* scratch = nullptr;
  int* err = nullptr;
  bool ready = false;
};
DeviceSlots g_slots[kMaxDevices];
std::mutex g_mu;

// Once per device, with that device current: resolve device addresses, clear the error word.
int setup_current_device(DeviceSlots** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return MB_ERR_DRIVER;
  std::lock_guard<std::mutex> g(g_mu);
  DeviceSlots& s = g_slots[dev];
  if (!s.ready) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_splitk_scratch) != cudaSuccess || p == nullptr) return MB_ERR_DRIVER;
    s.scratch = static_cast<float*>(p);
    p = nullptr;
    if (cudaGetSymbolAddress(&p, g_splitk_err) != cudaSuccess || p == nullptr) return MB_ERR_DRIVER;
    s.err = static_cast<int*>(p);
    // the clear must have landed before a first GEMM on any stream (a non-blocking stream does not wait for
    // the legacy stream the memset runs on), hence the one device-wide synchronisation of the set-up
    if (cudaMemset(s.err, 0, sizeof(int)) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess)
      return MB_ERR_DRIVER;
    s.ready = true;
  }
  *out = &s;
  return MB_OK;
}

}  // namespace

extern "C" int mb_gemm_bf16_splitk_static(const void* X, const void* W, void* Y, const void* R,
                                          int M, int N, int K, int ldx, int ldw, int ldy, int ldr,
                                          int splits, int bn, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return MB_OK;
  if (splits < 1) splits = 1;
  if (static_cast<unsigned long long>(splits) * M * N > MB_SPLITK_STATIC_MAX_FLOATS)
    return MB_ERR_TOO_LARGE;
  DeviceSlots* s = nullptr;
  const int rc = setup_current_device(&s);
  if (rc != MB_OK) return rc;
  const int flags = R != nullptr ? 2 : 0;
  return mb_gemm_bf16(X, W, Y, R, M, N, K, ldx, ldw, ldy, ldr, flags, bn, splits, /*stages=*/0,
                      s->scratch, s->err, /*num_sms=*/0, stream);
}

extern "C" int mb_gemm_bf16_splitk_static_error(void) {
  DeviceSlots* s = nullptr;
  if (setup_current_device(&s) != MB_OK) return MB_ERR_DRIVER;
  // wait for every stream of the device, non-blocking ones included: a plain cudaMemcpy alone would only
  // order itself after the legacy stream and could read the word before a GEMM on another stream has finished
  if (cudaDeviceSynchronize() != cudaSuccess) return MB_ERR_DRIVER;
  int v = 0;
  if (cudaMemcpy(&v, s->err, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return MB_ERR_DRIVER;
  if (v != 0 && (cudaMemset(s->err, 0, sizeof(int)) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess))
    return MB_ERR_DRIVER;
  return v;
}
