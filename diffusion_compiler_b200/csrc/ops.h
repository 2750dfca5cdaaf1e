// Internal C++ declarations of the operator launchers (one per kernel file).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace difb200 {

struct DeviceStatus;

const std::string &last_error();

// RmsNormModulate (explicit scale / shift layout) or, with a bias, LayerNormModulate computed in
// front of the quantiser in the same kernel, all bf16: weight [columns] or null, bias [columns]
// or null (null = RMS statistic), scale / shift [rows / rows_per_modulation, columns].
struct NormPrologue {
  const void *weight, *scale, *shift;
  float epsilon;
  const void *bias = nullptr;
  uint64_t rows_per_modulation = 1;
};

int quantize_int8_rows(const void *const *parts, const uint64_t *part_widths, uint32_t part_count,
                       uint64_t rows, int implementation, float clip, const float *clip_device,
                       int8_t *codes, float *scales, int8_t *rcodes, float *rscales,
                       cudaStream_t stream, bool mse_weight_scale = false, const void *equalise_bf16 = nullptr,
                       const NormPrologue *norm = nullptr);

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

// INT8 attention on already quantised Q/K (QuantizeInt8Rows Direct per token-head) and bf16 V.
size_t attention_int8_scratch_bytes(uint64_t B, uint64_t S, uint64_t KV);
// One launch of a chunked attention: it covers the key tiles (128 keys each) [tile_begin[i],
// tile_begin[i] + tile_count[i]) for i = 0, 1 and may take the unnormalised state of every query
// row (m, l, fp32 outputs) from `state` and / or leave it there instead of writing `out`.
// A sequence of launches over disjoint tile ranges, the first without carry_in and the last
// without carry_out, gives the single launch's result up to the order of the fp32 sums.
struct AttentionChunk {
  uint32_t tile_begin[2], tile_count[2];
  bool carry_in, carry_out;
  void *state; // attention_int8_state_bytes(B, Sq, H) bytes, 16-byte aligned
};
size_t attention_int8_state_bytes(uint64_t B, uint64_t Sq, uint64_t H);
int attention_int8(const int8_t *q8, const float *qs, const int8_t *k8, const float *ks, const void *v_bf16,
                   const uint8_t *key_valid, uint64_t B, uint64_t Sq, uint64_t Sk, uint64_t H, uint64_t KV,
                   uint64_t D, float scale, void *scratch, size_t scratch_bytes, void *out_bf16,
                   cudaStream_t stream, const AttentionChunk *chunk = nullptr);

// DiffIR Attention on bf16 q/k/v in its INT8 lowering: Direct quantisation of q and k per
// token-head, then attention_int8. Scratch holds the codes, scales and the key table.
size_t attention_scratch_bytes(uint64_t B, uint64_t S, uint64_t H, uint64_t KV);
// Where the INT8 lowering keeps its operands inside that scratch buffer: a producer that
// quantises q or k itself writes here and passes a null q / k to attention_bf16_via_int8.
struct AttentionScratch {
  int8_t *q8, *k8;
  float *qs, *ks;
  void *rest;
};
AttentionScratch attention_scratch_layout(void *scratch, uint64_t B, uint64_t S, uint64_t H, uint64_t KV);
int attention_bf16_via_int8(const void *q, const void *k, const void *v, const uint8_t *key_valid, uint64_t B,
                            uint64_t S, uint64_t H, uint64_t KV, uint64_t D, float scale, void *scratch,
                            size_t scratch_bytes, void *out_bf16, cudaStream_t stream);

} // namespace difb200
