// Launchers of the block-glue kernels (glue.cu). dtype codes are the DiffIR ones
// (1 = F32, 2 = BF16, 3 = F16). All return a status code (0 = OK).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace difb200 {
namespace glue {

int binary(const void *a, const void *b, void *o, uint32_t dt, uint64_t n, bool multiply, cudaStream_t s);
// kind: 0 = copy/cast, 1 = gelu tanh, 2 = gelu erf, 3 = silu, 4 = sigmoid
int unary(const void *a, void *o, uint32_t dt_in, uint32_t dt_out, uint64_t n, int kind, cudaStream_t s);
int bias_add(const void *a, const void *bias, void *o, uint32_t dt, uint64_t n, uint64_t width, cudaStream_t s);
int affine_last_dim(const void *a, const void *scale, const void *bias, void *o, uint32_t dt, uint64_t n,
                    uint64_t width, cudaStream_t s);
int fill(void *o, uint32_t dt, uint64_t n, float value, cudaStream_t s);
int rms_norm(const void *x, const void *w, void *o, uint32_t dt, uint64_t rows, uint64_t cols, float eps,
             float weight_offset, cudaStream_t s);
int layer_norm_modulate(const void *x, const void *w, const void *b, const void *scale, const void *shift, void *o,
                        uint32_t dt, uint64_t rows, uint64_t cols, uint64_t rows_per_mod, float eps, cudaStream_t s);
int rms_norm_modulate(const void *x, const void *w, const void *a, const void *b, void *o, uint32_t dt, uint64_t rows,
                      uint64_t cols, float eps, float weight_offset, bool shared_vector, uint64_t rows_per_vector,
                      cudaStream_t s);
int qk_norm_rope(const void *x, const void *w, const void *cosv, const void *sinv, void *o, uint32_t dt,
                 uint32_t dt_table, uint64_t tokens, uint64_t heads, uint64_t dim, uint64_t rotary,
                 uint64_t table_width, uint64_t input_seq, uint64_t table_seq, uint64_t table_start, float eps,
                 bool interleaved_v2, cudaStream_t s);
int rotary_frequency(const float *pos, const int32_t *pair_axes, const int32_t *pair_idx, const int32_t *axis_dims,
                     float *cosv, float *sinv, uint64_t tokens, uint64_t axes, uint64_t pairs, double theta_ntk,
                     unsigned int *bad_flag, cudaStream_t s);
int rotary_apply(const void *x, const float *cosv, const float *sinv, void *o, uint32_t dt, uint64_t tokens,
                 uint64_t heads, uint64_t dim, uint64_t pairs, cudaStream_t s);
int residual_gate(const void *res, const void *branch, const void *gate, void *o, uint32_t dt, uint64_t n,
                  uint64_t width, uint64_t rows_per_gate, cudaStream_t s);
int swiglu(const void *x, void *o, uint32_t dt, uint64_t rows, uint64_t width, uint64_t in_width, uint64_t start,
           bool gate_first, cudaStream_t s);
// out[i] = in[offset + sum_a coord_a(i) * in_strides[a]] (BroadcastTo: stride 0 on broadcast axes;
// Slice: offset = start * stride[axis])
int gather(const void *x, void *o, uint32_t elem_bytes, uint32_t rank, const uint64_t *out_dims,
           const uint64_t *in_strides, uint64_t offset, cudaStream_t s);
int concat_part(const void *x, void *o, uint32_t elem_bytes, uint64_t outer, uint64_t chunk, uint64_t out_chunk,
                uint64_t out_offset, cudaStream_t s);
int mask_to_bias(const uint8_t *mask, void *o, uint32_t dt, uint64_t B, uint64_t L, bool vector_mask,
                 bool mask_queries, cudaStream_t s);
int linear(const void *x, const void *w, const void *bias, void *o, uint32_t dt, uint64_t M, uint64_t N, uint64_t K,
           cudaStream_t s);

// Row statistics of a bf16 [rows, cols] tensor in the reference's own order (one sequential fp32
// chain per row, cpu_executor.cpp:1051-1062, 1119-1129, 1250-1256), so that a normalisation built on
// them has the reference's bits: stats[r] = (0, 1 / sqrt(sum x^2 / cols + eps)) or, with `layer`,
// (mean, 1 / sqrt(sum (x - mean)^2 / cols + eps)). *stats points into per-device scratch that the
// next call of this function reuses. False (nothing launched) when cols is not a multiple of 64,
// x is not 16-byte aligned or DIFB200_EXACT_NORM=0 asks for the parallel sums.
bool row_stats_sequential(const void *x, uint64_t rows, uint64_t cols, float eps, bool layer, const float2 **stats,
                          cudaStream_t s, int *rc);

// bf16 fast paths (glue_fast.cu). Each returns false when dtype, widths or alignment are not
// covered (nothing launched; the caller runs the generic kernel), else true with the launch
// status in *rc.
bool residual_gate_fast(const void *res, const void *branch, const void *gate, void *o, uint32_t dt, uint64_t n,
                        uint64_t width, uint64_t rows_per_gate, cudaStream_t s, int *rc);
bool swiglu_fast(const void *x, void *o, uint32_t dt, uint64_t rows, uint64_t width, uint64_t in_width,
                 uint64_t start, bool gate_first, cudaStream_t s, int *rc);
bool layer_norm_modulate_fast(const void *x, const void *w, const void *b, const void *scale, const void *shift,
                              void *o, uint32_t dt, uint64_t rows, uint64_t cols, uint64_t rows_per_mod, float eps,
                              cudaStream_t s, int *rc);
bool rms_norm_modulate_fast(const void *x, const void *w, const void *a, const void *b, void *o, uint32_t dt,
                            uint64_t rows, uint64_t cols, float eps, cudaStream_t s, int *rc);
// Where QkNormPartialRope reads and writes when it is fused with its neighbours (elements /
// tokens): a token's heads start at x + token * in_token_stride + in_offset (a last-axis Slice
// read in place), and the result goes to token (token / input_seq) * out_seq + out_start +
// token % input_seq of the destination (a Concat along tokens written in place).
struct RopeLayout {
  uint64_t in_token_stride, in_offset, out_seq, out_start;
};
// o (bf16 result) and codes/scales (QuantizeInt8Rows Direct of that result) are each optional;
// layout may be null (dense input, output rows = input rows).
bool qk_norm_rope_fast(const void *x, const void *w, const void *cosv, const void *sinv, void *o, int8_t *codes,
                       float *scales, uint32_t dt, uint32_t dt_table, uint64_t tokens, uint64_t heads, uint64_t dim,
                       uint64_t rotary, uint64_t table_width, uint64_t input_seq, uint64_t table_seq,
                       uint64_t table_start, float eps, bool interleaved_v2, const RopeLayout *layout, cudaStream_t s,
                       int *rc);
bool direct_quant_rows128(const void *x, int8_t *codes, float *scales, uint64_t rows, float clip, cudaStream_t s,
                          int *rc);

} // namespace glue
} // namespace difb200
