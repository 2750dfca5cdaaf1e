// difb200_w8a8_linear_static: the W8A8 linear for callers that must not allocate.
//
// Some hosts of this library cannot call cudaMalloc on the path where they run a layer: a
// runtime that planned its whole device arena up front and forbids later allocations (the
// reference's executors reserve memory at prepare() and check a free-memory floor at run()),
// code running while a CUDA graph is being captured or inside a latency-critical serving loop
// where an allocation would synchronise the device, or a plugin whose owner wants a hard
// guarantee that loading a model never grows the process's footprint. For them this file keeps
// the scratch that the two-kernel W8A8 linear needs (the INT8 activation codes, the per-row
// scales and the status words of the GEMM's bounded waits) in a fixed array that is part of
// the library image.
//
// Cost and limits: every GPU on which the library's device code is loaded holds
// kStaticScratchBytes (40 MiB) of device memory until the process exits, whether or not this
// entry point is used. With CUDA's default lazy module loading that memory is taken when the
// module is first needed on a device, which for a host that only uses this entry point is its
// first call there (with CUDA_MODULE_LOADING=EAGER it is taken when the library is loaded). A
// host that wants every allocation behind it before it starts serving therefore makes one call
// with M = 0 per device at start-up: that call resolves the array's address, launches nothing
// and returns 0. The address is cached per device ordinal for the life of the process; after a
// cudaDeviceReset the cache is stale and this entry point must not be used again in that process.
// A call needs 256 + roundup(4*M, 256) + M*K bytes of it and is rejected with status 2 and a
// clear message when that exceeds the array. All calls share the one array and it keeps what
// the last call left there, so two calls whose kernels may overlap on the GPU (different
// streams, or different host threads without ordering) race on the codes; serialise them.
#include "difb200/difb200.h"

#include "common.cuh"
#include "ops.h"

#include <mutex>

namespace difb200 {
namespace {

constexpr size_t kStaticScratchBytes = 40ull << 20;
constexpr size_t kStatusBytes = 256;
constexpr int kMaxDevices = 64;

// File-scope device array. In host code this name is only a handle for the runtime: its
// device address is obtained with cudaGetSymbolAddress below and never by taking &name.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_setup_mutex;
unsigned char *g_device_address[kMaxDevices]; // per device ordinal, filled on first use

// One-time set-up per device, with that device current: resolve the array's device address.
int static_scratch_base(unsigned char **base) {
  int device = 0;
  if (int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice"))
    return rc;
  if (device < 0 || device >= kMaxDevices)
    return fail(kUnsupported, "difb200_w8a8_linear_static: device ordinal out of range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_device_address[device]) {
    unsigned char *ptr = nullptr;
    if (int rc = check_cuda(cudaGetSymbolAddress(reinterpret_cast<void **>(&ptr), g_static_scratch),
                            "cudaGetSymbolAddress(static scratch)"))
      return rc;
    if (!ptr || (reinterpret_cast<uintptr_t>(ptr) & 255u) != 0)
      return fail(kInternalError, "difb200_w8a8_linear_static: static scratch address is unusable");
    g_device_address[device] = ptr;
  }
  *base = g_device_address[device];
  return kOk;
}

} // namespace
} // namespace difb200

using namespace difb200;

extern "C" int difb200_w8a8_linear_static(const void *x, const int8_t *w, const float *col_scales,
                                          const void *bias, uint32_t epilogue,
                                          int32_t implementation, float clip, uint64_t M, uint64_t N,
                                          uint64_t K, void *out, int32_t check_previous,
                                          void *stream) {
  unsigned char *base = nullptr;
  if (int rc = static_scratch_base(&base))
    return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (check_previous) {
    // Report a bounded wait that ran out in the previous call on this device (synchronises).
    DeviceStatus host{};
    if (int rc = check_cuda(cudaStreamSynchronize(s), "cudaStreamSynchronize"))
      return rc;
    if (int rc = check_cuda(cudaMemcpy(&host, base, sizeof(host), cudaMemcpyDeviceToHost),
                            "cudaMemcpy(status words)"))
      return rc;
    if (host.flag != 0) {
      // clear the sticky words, so that the caller can go on after having seen the error once
      cudaMemset(base, 0, sizeof(DeviceStatus));
      return fail(kExecutionError, "difb200_w8a8_linear_static: a bounded device-side wait ran out in "
                                   "the previous call (role " + std::to_string(host.role) + ", detail " +
                                   std::to_string(host.detail) + ")");
    }
  }
  if (M == 0 || N == 0)
    return kOk;
  if (K == 0 || M > (kStaticScratchBytes >> 2) || K > kStaticScratchBytes)
    return fail(kUnsupported, "difb200_w8a8_linear_static: M or K is beyond the static scratch");
  const size_t scale_bytes = (static_cast<size_t>(M) * 4 + 255) & ~static_cast<size_t>(255);
  const size_t need = kStatusBytes + scale_bytes + static_cast<size_t>(M) * static_cast<size_t>(K);
  if (need > kStaticScratchBytes)
    return fail(kUnsupported,
                "difb200_w8a8_linear_static: needs " + std::to_string(need) +
                    " bytes of scratch (256 + 4*M rounded up to 256 + M*K) but the static array holds " +
                    std::to_string(kStaticScratchBytes) + "; use difb200_w8a8_linear with caller scratch");
  DeviceStatus *status = reinterpret_cast<DeviceStatus *>(base);
  float *scales = reinterpret_cast<float *>(base + kStatusBytes);
  int8_t *codes = reinterpret_cast<int8_t *>(base + kStatusBytes + scale_bytes);
  // The status words must start at zero; codes and scales are fully overwritten by the
  // quantiser before the GEMM reads them, so stale contents there do not matter.
  if (int rc = check_cuda(cudaMemsetAsync(status, 0, sizeof(DeviceStatus), s), "cudaMemsetAsync(status)"))
    return rc;
  return w8a8_linear(x, w, col_scales, bias, epilogue, implementation, clip, M, N, K, codes, scales, out,
                     s, status);
}
