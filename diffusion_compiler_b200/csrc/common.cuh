// Shared device/host helpers for the difb200 kernels (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace difb200 {

// Status codes are numerically identical to dif_backend_status of the reference plugin
// ABI (reference include/dif/backend/abi.h:22-30), so they pass through unchanged.
enum Status : int {
  kOk = 0,
  kInvalidArgument = 1,
  kUnsupported = 2,
  kOutOfMemory = 3,
  kCompileError = 4,
  kExecutionError = 5,
  kInternalError = 6,
};

// Thread-local text of the last failure, returned by difb200_last_error().
void set_last_error(const std::string &text);
int fail(int status, const std::string &text);
int check_cuda(cudaError_t code, const char *what);
// check_cuda for the status of a kernel launch; counts the launches of this process (launch_count).
int launched(cudaError_t code, const char *what);
unsigned long long launch_count();
int sm_count();

// One-time set-up that is per device, not per process (function attributes and occupancy
// figures belong to a context): `init` runs the first time `key` is seen with `device` and its
// result value is cached; a failing `init` is not cached. Thread-safe.
int per_device_once(const void *key, int device, int (*init)(void *arg, int *value), void *arg, int *value);
int current_device_once(const void *key, int (*init)(void *arg, int *value), void *arg, int *value);

// Device-side status words written by kernels whose bounded waits ran out. Index 0 is a
// sticky flag, 1..3 describe where (kernel id, role, iteration).
struct DeviceStatus {
  unsigned int flag;
  unsigned int kernel;
  unsigned int role;
  unsigned int detail;
};
// Limit of the kernels' bounded waits in nanoseconds (default 1.5 s), read at every launch.
unsigned long long wait_limit_ns();
void set_wait_limit_ns(unsigned long long ns); // 0 restores the default
// Test aid for the give-up path: the next LinearInt8Scaled launch leaves out the loads of one
// k-block. take_...() returns that k-block (0xffffffff = none) and disarms.
void withhold_next_gemm_load(uint32_t k_block);
uint32_t take_withheld_gemm_load();
// Per-device scratch that only grows (reallocated, which synchronises the device, when a call
// needs more than any call before it): small work areas whose size follows the row count.
void *device_scratch(size_t bytes);
DeviceStatus *device_status_words();      // per-device, allocated once
int poll_device_status(const char *what); // copies back, clears, maps to kExecutionError

#ifdef __CUDACC__

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}
// Round-to-nearest-even on the raw fp32 bits, the reference's bf16 store
// (reference src/runtime/scalar.cpp:18-22).
__device__ __forceinline__ uint32_t f32_to_bf16_bits(float v) {
  const uint32_t b = __float_as_uint(v);
  return ((b + 0x7fffu + ((b >> 16) & 1u)) >> 16) & 0xffffu;
}
__device__ __forceinline__ float round_bf16(float v) {
  return __uint_as_float(f32_to_bf16_bits(v) << 16);
}

// ---- packed fp32x2 arithmetic (two independent fp32 lanes per 64-bit register) ----
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

#endif // __CUDACC__

} // namespace difb200
