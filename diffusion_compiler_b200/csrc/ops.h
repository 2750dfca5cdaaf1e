// Internal C++ declarations of the operator launchers (one per kernel file).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace difb200 {

struct DeviceStatus;

const std::string &last_error();

int quantize_int8_rows(const void *const *parts, const uint64_t *part_widths, uint32_t part_count,
                       uint64_t rows, int implementation, float clip, const float *clip_device,
                       int8_t *codes, float *scales, int8_t *rcodes, float *rscales,
                       cudaStream_t stream);

int linear_int8_scaled(const int8_t *x, const int8_t *w, const float *row_scales,
                       const float *col_scales, const void *bias_bf16, uint32_t epilogue, uint64_t M,
                       uint64_t N, uint64_t K, void *out_bf16, int32_t *acc_out, cudaStream_t stream,
                       DeviceStatus *status_words = nullptr);

// QuantizeInt8Rows -> LinearInt8Scaled [-> BiasAdd -> Gelu] on a bf16 [M,K] input; codes [M,K]
// and row scales [M] are scratch supplied by the caller.
int w8a8_linear(const void *x_bf16, const int8_t *w, const float *col_scales, const void *bias_bf16,
                uint32_t epilogue, int implementation, float clip, uint64_t M, uint64_t N, uint64_t K,
                int8_t *codes_scratch, float *scales_scratch, void *out_bf16, cudaStream_t stream,
                DeviceStatus *status_words = nullptr);

} // namespace difb200
