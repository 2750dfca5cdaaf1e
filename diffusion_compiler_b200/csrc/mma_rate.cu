// Measured INT8 tensor-core peak: every SM issues tcgen05.mma kind::i8 (the instruction shape of
// the LinearInt8Scaled kernel, M128 or M256 x N256 x K32) back to back on operands that stay in
// shared memory, into one tensor-memory accumulator. No global traffic, no epilogue: the time of
// the launch gives the rate at which the tensor cores retire INT8 MACs on this GPU at the clock it
// runs at under that load. It is the denominator the benchmark puts beside the nominal dense INT8
// figure (the reference publishes no such number; its GEMM is src/runtime/cutlass_gemm.cu:185-303).
#include "difb200/difb200.h"

#include "common.cuh"
#include "ptx.cuh"

namespace difb200 {
namespace {

constexpr uint32_t kOperandBytes = 64 * 1024; // A 128 x 128 B at 0, B 256 x 128 B at 32 KB (pair: 128 rows)
constexpr size_t kRateSmem = 1024 + kOperandBytes + 64;

template <int CTAS>
__global__ void __launch_bounds__(128, 1)
i8_mma_rate_kernel(uint32_t n_mma, unsigned long long wait_ns, DeviceStatus *status) {
  extern __shared__ uint8_t raw[];
  const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
  const uint32_t bar = base + kOperandBytes, slot = bar + 16;
  volatile uint32_t *slot_ptr = reinterpret_cast<volatile uint32_t *>(raw + (slot - smem_u32(raw)));
  const uint32_t rank = CTAS == 2 ? ptx::cluster_ctarank() : 0u;
  // defined operand bytes (any INT8 values do)
  for (uint32_t i = threadIdx.x; i < kOperandBytes / 4; i += blockDim.x)
    reinterpret_cast<uint32_t *>(raw + (base - smem_u32(raw)))[i] = 0x01ff02feu + i;
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar, 1);
    ptx::fence_barrier_init();
  }
  ptx::fence_proxy_async();
  if (threadIdx.x < 32) {
    if (CTAS == 2) {
      ptx::tmem_alloc_pair(slot, 256);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(slot, 256);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (CTAS == 2)
    ptx::cluster_sync();
  ptx::tc_fence_after();
  const uint32_t tmem = *slot_ptr;
  if (threadIdx.x == 0 && rank == 0) {
    constexpr uint32_t idesc = ptx::make_idesc(2 /*S32*/, 1 /*S8*/, 1 /*S8*/, 0, 0, 128 * CTAS, 256);
    const uint64_t a = ptx::smem_desc_sw128(base, 16, 1024), b = ptx::smem_desc_sw128(base + 32768, 16, 1024);
    for (uint32_t i = 0; i < n_mma; ++i) {
      if (CTAS == 2)
        ptx::mma_i8_ss_pair(tmem, a + 2 * (i & 3), b + 2 * (i & 3), idesc, i != 0);
      else
        ptx::mma_i8_ss(tmem, a + 2 * (i & 3), b + 2 * (i & 3), idesc, i != 0);
    }
    if (CTAS == 2)
      ptx::mma_commit_pair(bar);
    else
      ptx::mma_commit(bar);
    if (!ptx::mbar_wait(bar, 0, wait_ns) && atomicExch(&status->flag, 1u) == 0u) {
      status->kernel = 4u;
      status->role = 0u;
      status->detail = n_mma;
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (CTAS == 2)
    ptx::cluster_sync();
  if (threadIdx.x < 32) {
    ptx::tc_fence_after();
    if (CTAS == 2)
      ptx::tmem_dealloc_pair(tmem, 256);
    else
      ptx::tmem_dealloc(tmem, 256);
  }
}

template <int CTAS>
int run_rate(uint32_t n_mma, double *tops, double *milliseconds, cudaStream_t stream) {
  auto kernel = i8_mma_rate_kernel<CTAS>;
  if (int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kRateSmem),
                          "cudaFuncSetAttribute(i8_mma_rate_kernel)"))
    return rc;
  DeviceStatus *status = device_status_words();
  if (!status)
    return fail(kOutOfMemory, "cannot allocate device status words");
  cudaLaunchConfig_t config{};
  config.blockDim = dim3(128);
  config.dynamicSmemBytes = kRateSmem;
  config.stream = stream;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = CTAS;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  config.attrs = &attr;
  config.numAttrs = 1;
  int ctas = sm_count();
  if (CTAS == 2) {
    config.gridDim = dim3((unsigned)ctas);
    int clusters = 0;
    if (int rc = check_cuda(cudaOccupancyMaxActiveClusters(&clusters, kernel, &config), "cudaOccupancyMaxActiveClusters"))
      return rc;
    ctas = 2 * (clusters > 0 ? clusters : 1); // one wave: only pairs that are resident at once
    if (ctas > sm_count())
      ctas = sm_count() & ~1;
  }
  config.gridDim = dim3((unsigned)ctas);
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  if (int rc = check_cuda(cudaEventCreate(&e0), "cudaEventCreate"))
    return rc;
  if (int rc = check_cuda(cudaEventCreate(&e1), "cudaEventCreate")) {
    cudaEventDestroy(e0);
    return rc;
  }
  int rc = kOk;
  float best = 0.0f;
  for (int rep = 0; rep < 4 && rc == kOk; ++rep) { // first repetition warms up
    cudaEventRecord(e0, stream);
    rc = launched(cudaLaunchKernelEx(&config, kernel, n_mma, wait_limit_ns(), status), "i8_mma_rate_kernel launch");
    cudaEventRecord(e1, stream);
    if (rc == kOk)
      rc = check_cuda(cudaEventSynchronize(e1), "cudaEventSynchronize");
    float ms = 0.0f;
    if (rc == kOk && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess && rep > 0 && (best == 0.0f || ms < best))
      best = ms;
  }
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (rc)
    return rc;
  // every leader issues n_mma MMAs of (128 * CTAS) x 256 x 32 MACs
  const double ops = 2.0 * (double)(ctas / CTAS) * n_mma * (128.0 * CTAS) * 256.0 * 32.0;
  if (milliseconds)
    *milliseconds = best;
  if (tops)
    *tops = best > 0.0f ? ops / (best * 1e-3) / 1e12 : 0.0;
  return kOk;
}

} // namespace
} // namespace difb200

extern "C" int difb200_measure_i8_mma_peak(int32_t ctas_per_mma, uint32_t mma_per_issuer, double *tops,
                                           double *milliseconds, void *stream) {
  using namespace difb200;
  if (mma_per_issuer == 0 || mma_per_issuer > (1u << 20))
    return fail(kInvalidArgument, "difb200_measure_i8_mma_peak: 1 .. 2^20 MMAs per issuing thread");
  if (ctas_per_mma == 2)
    return run_rate<2>(mma_per_issuer, tops, milliseconds, static_cast<cudaStream_t>(stream));
  if (ctas_per_mma == 1)
    return run_rate<1>(mma_per_issuer, tops, milliseconds, static_cast<cudaStream_t>(stream));
  return fail(kInvalidArgument, "difb200_measure_i8_mma_peak: form must be 1 (one CTA) or 2 (CTA pair)");
}
