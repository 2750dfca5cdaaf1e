// extern "C" surface of libdifb200.so for device-resident callers (see difb200/difb200.h).
#include "difb200/difb200.h"

#include "common.cuh"
#include "ops.h"

using namespace difb200;

namespace difb200 {

int w8a8_linear(const void *x_bf16, const int8_t *w, const float *col_scales, const void *bias_bf16,
                uint32_t epilogue, int implementation, float clip, uint64_t M, uint64_t N, uint64_t K,
                int8_t *codes_scratch, float *scales_scratch, void *out_bf16, cudaStream_t stream,
                DeviceStatus *status_words) {
  if (!x_bf16 || !codes_scratch || !scales_scratch)
    return fail(kInvalidArgument, "w8a8_linear: null input or scratch pointer");
  const void *parts[1] = {x_bf16};
  const uint64_t widths[1] = {K};
  if (int rc = quantize_int8_rows(parts, widths, 1, M, implementation, clip, nullptr, codes_scratch,
                                  scales_scratch, nullptr, nullptr, stream))
    return rc;
  return linear_int8_scaled(codes_scratch, w, scales_scratch, col_scales, bias_bf16, epilogue, M, N, K,
                            out_bf16, nullptr, stream, status_words);
}

} // namespace difb200

extern "C" {

const char *difb200_last_error(void) { return last_error().c_str(); }

int difb200_version(void) { return 1; }

int difb200_poll_status(void) {
  if (int rc = check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize"))
    return rc;
  return poll_device_status("difb200_poll_status");
}

int difb200_quantize_int8_rows(const void *const *parts, const uint64_t *part_widths,
                               uint32_t part_count, uint64_t rows, int32_t implementation,
                               float clip, const float *clip_device, int8_t *codes, float *scales,
                               int8_t *residual_codes, float *residual_scales, void *stream) {
  if (!parts || !part_widths)
    return fail(kInvalidArgument, "difb200_quantize_int8_rows: null part arrays");
  return quantize_int8_rows(parts, part_widths, part_count, rows, implementation, clip, clip_device,
                            codes, scales, residual_codes, residual_scales,
                            static_cast<cudaStream_t>(stream));
}

int difb200_linear_int8_scaled(const int8_t *x, const int8_t *w, const float *row_scales,
                               const float *col_scales, const void *bias, uint32_t epilogue,
                               uint64_t M, uint64_t N, uint64_t K, void *out, int32_t *acc_out,
                               void *stream) {
  return linear_int8_scaled(x, w, row_scales, col_scales, bias, epilogue, M, N, K, out, acc_out,
                            static_cast<cudaStream_t>(stream));
}

int difb200_w8a8_linear(const void *x, const int8_t *w, const float *col_scales, const void *bias,
                        uint32_t epilogue, int32_t implementation, float clip, uint64_t M, uint64_t N,
                        uint64_t K, int8_t *codes_scratch, float *scales_scratch, void *out,
                        void *stream) {
  return w8a8_linear(x, w, col_scales, bias, epilogue, implementation, clip, M, N, K, codes_scratch,
                     scales_scratch, out, static_cast<cudaStream_t>(stream));
}

}
