// Memory-bound block-glue kernels of the plugin: the non-GEMM, non-attention DiffIR ops that sit
// between the quantized linears and attention in a DiT block. Each follows the reference CPU
// executor's arithmetic and storage-dtype rounding points (file:line cited per kernel; paths in
// the reference project). Row reductions are warp-parallel, so sums differ from the CPU's
// sequential fp32 order in the last bits (covered by the bf16 tolerance, not bit-exact).
#include "glue.h"

#include "common.cuh"

#include <cuda_fp16.h>

namespace difb200 {
namespace glue {
namespace {

enum : uint32_t { kF32 = 1, kBF16 = 2, kF16 = 3 };

__device__ __forceinline__ float ld(const void *p, uint32_t dtype, uint64_t i) {
  if (dtype == kF32)
    return static_cast<const float *>(p)[i];
  if (dtype == kBF16)
    return bf16_bits_to_f32(static_cast<const uint16_t *>(p)[i]);
  return __half2float(static_cast<const __half *>(p)[i]);
}
__device__ __forceinline__ void st(void *p, uint32_t dtype, uint64_t i, float v) {
  if (dtype == kF32)
    static_cast<float *>(p)[i] = v;
  else if (dtype == kBF16)
    static_cast<uint16_t *>(p)[i] = (uint16_t)f32_to_bf16_bits(v);
  else
    static_cast<__half *>(p)[i] = __float2half_rn(v);
}
// reference round_to_storage_dtype: the value as it would read back after a store
__device__ __forceinline__ float rnd(float v, uint32_t dtype) {
  if (dtype == kF32)
    return v;
  if (dtype == kBF16)
    return round_bf16(v);
  return __half2float(__float2half_rn(v));
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

#define GRID_STRIDE(i, n)                                                                     \
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < (n);                 \
       i += (uint64_t)gridDim.x * blockDim.x)

inline unsigned blocks_for(uint64_t n, int threads = 256) {
  uint64_t b = (n + threads - 1) / threads;
  const uint64_t cap = (uint64_t)sm_count() * 32;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}
inline unsigned row_blocks(uint64_t rows) { // one warp per row, 8 warps per block
  uint64_t b = (rows + 7) / 8;
  const uint64_t cap = (uint64_t)sm_count() * 16;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}

// ---- elementwise: Add / Multiply (cpu_executor.cpp:45-55) ----
__global__ void k_binary(const void *a, const void *b, void *o, uint32_t dt, uint64_t n, int multiply) {
  GRID_STRIDE(i, n) {
    const float x = ld(a, dt, i), y = ld(b, dt, i);
    st(o, dt, i, multiply ? __fmul_rn(x, y) : __fadd_rn(x, y));
  }
}
// ---- unary: Gelu (93-113), SiLU (84-91), Sigmoid (115-122), Cast ----
__global__ void k_unary(const void *a, void *o, uint32_t dt_in, uint32_t dt_out, uint64_t n, int kind) {
  GRID_STRIDE(i, n) {
    const float v = ld(a, dt_in, i);
    float r = v;
    if (kind == 1) { // gelu tanh
      const float cubic = __fmul_rn(__fmul_rn(v, v), v);
      const float inner = __fmul_rn(0.7978845608028654f, __fadd_rn(v, __fmul_rn(0.044715f, cubic)));
      r = __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, tanhf(inner)));
    } else if (kind == 2) { // gelu erf
      r = __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, erff(__fmul_rn(v, 0.7071067811865475f))));
    } else if (kind == 3) { // silu
      r = __fdiv_rn(v, __fadd_rn(1.0f, expf(-v)));
    } else if (kind == 4) { // sigmoid
      r = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v)));
    }
    st(o, dt_out, i, r);
  }
}
// ---- BiasAdd (1288-1296), AffineLastDim (57-71) ----
__global__ void k_bias(const void *a, const void *bias, void *o, uint32_t dt, uint64_t n, uint64_t width) {
  GRID_STRIDE(i, n) st(o, dt, i, __fadd_rn(ld(a, dt, i), ld(bias, dt, i % width)));
}
__global__ void k_affine(const void *a, const void *scale, const void *bias, void *o, uint32_t dt, uint64_t n,
                         uint64_t width) {
  GRID_STRIDE(i, n) {
    const uint64_t c = i % width;
    const float scaled = rnd(__fmul_rn(ld(a, dt, i), ld(scale, dt, c)), dt);
    st(o, dt, i, bias ? __fadd_rn(scaled, ld(bias, dt, c)) : scaled);
  }
}
__global__ void k_fill(void *o, uint32_t dt, uint64_t n, float value) {
  GRID_STRIDE(i, n) st(o, dt, i, value);
}
// ---- RmsNorm (1051-1075): one warp per row ----
__global__ void k_rms_norm(const void *x, const void *w, void *o, uint32_t dt, uint64_t rows, uint64_t cols,
                           float eps, float weight_offset, const float2 *stats) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const uint64_t nwarps = (uint64_t)gridDim.x * (blockDim.x >> 5);
  for (uint64_t r = warp; r < rows; r += nwarps) {
    float sum = 0.0f;
    for (uint64_t c = lane; c < cols; c += 32) {
      const float v = ld(x, dt, r * cols + c);
      sum = __fmaf_rn(v, v, sum);
    }
    sum = warp_sum(sum);
    // with `stats` the statistic comes in the reference's sequential order (bit-exact outputs)
    const float inv = stats ? stats[r].y : __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(sum, (float)cols), eps)));
    for (uint64_t c = lane; c < cols; c += 32)
      st(o, dt, r * cols + c,
         __fmul_rn(__fmul_rn(ld(x, dt, r * cols + c), inv), __fadd_rn(ld(w, dt, c), weight_offset)));
  }
}
// ---- LayerNormModulate (1108-1148): rounds after norm, after 1+scale, after the product ----
__global__ void k_layer_norm_modulate(const void *x, const void *w, const void *b, const void *scale,
                                      const void *shift, void *o, uint32_t dt, uint64_t rows, uint64_t cols,
                                      uint64_t rows_per_mod, float eps) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const uint64_t nwarps = (uint64_t)gridDim.x * (blockDim.x >> 5);
  for (uint64_t r = warp; r < rows; r += nwarps) {
    float mean = 0.0f;
    for (uint64_t c = lane; c < cols; c += 32)
      mean += ld(x, dt, r * cols + c);
    mean = __fdiv_rn(warp_sum(mean), (float)cols);
    float var = 0.0f;
    for (uint64_t c = lane; c < cols; c += 32) {
      const float d = __fsub_rn(ld(x, dt, r * cols + c), mean);
      var = __fmaf_rn(d, d, var);
    }
    var = warp_sum(var);
    const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(var, (float)cols), eps)));
    const uint64_t mrow = r / rows_per_mod;
    for (uint64_t c = lane; c < cols; c += 32) {
      const uint64_t i = r * cols + c, mi = mrow * cols + c;
      const float normalized = rnd(
          __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(ld(x, dt, i), mean), inv), ld(w, dt, c)), ld(b, dt, c)), dt);
      const float one_plus = rnd(__fadd_rn(1.0f, ld(scale, dt, mi)), dt);
      const float scaled = rnd(__fmul_rn(normalized, one_plus), dt);
      st(o, dt, i, __fadd_rn(scaled, ld(shift, dt, mi)));
    }
  }
}
// ---- RmsNormModulate (1200-1265) ----
__global__ void k_rms_norm_modulate(const void *x, const void *w, const void *a, const void *b, void *o, uint32_t dt,
                                    uint64_t rows, uint64_t cols, float eps, float weight_offset, int shared_vector,
                                    uint64_t rows_per_vector) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const uint64_t nwarps = (uint64_t)gridDim.x * (blockDim.x >> 5);
  for (uint64_t r = warp; r < rows; r += nwarps) {
    float sum = 0.0f;
    for (uint64_t c = lane; c < cols; c += 32) {
      const float v = ld(x, dt, r * cols + c);
      sum = __fmaf_rn(v, v, sum);
    }
    sum = warp_sum(sum);
    const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(sum, (float)cols), eps)));
    for (uint64_t c = lane; c < cols; c += 32) {
      const uint64_t i = r * cols + c;
      if (shared_vector) { // a = vector [V,H], b = delta [2,H]
        const float base = ld(a, dt, (r / rows_per_vector) * cols + c);
        const float scale = __fadd_rn(base, ld(b, dt, c)), shift = __fadd_rn(base, ld(b, dt, cols + c));
        const float normalized =
            __fmul_rn(__fmul_rn(ld(x, dt, i), inv), __fadd_rn(ld(w, dt, c), weight_offset));
        st(o, dt, i, __fadd_rn(__fmul_rn(__fadd_rn(1.0f, scale), normalized), shift));
      } else { // a = scale, b = shift (full shape)
        const float normalized = __fmul_rn(__fmul_rn(ld(x, dt, i), inv), w ? ld(w, dt, c) : 1.0f);
        st(o, dt, i, __fadd_rn(__fmul_rn(normalized, __fadd_rn(1.0f, ld(a, dt, i))), ld(b, dt, i)));
      }
    }
  }
}
// ---- QkNormPartialRope (1741-1837): one warp per (token, head) ----
struct RopeParams {
  const void *x, *w, *cosv, *sinv;
  void *o;
  uint32_t dt, dt_table;
  uint64_t tokens, heads, dim, rotary, table_width, input_seq, table_seq, table_start;
  float eps;
  int interleaved_v2;
};
__global__ void k_qk_norm_rope(const RopeParams p) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const uint64_t nwarps = (uint64_t)gridDim.x * (blockDim.x >> 5);
  const uint64_t half = p.rotary / 2;
  for (uint64_t r = warp; r < p.tokens * p.heads; r += nwarps) {
    const uint64_t token = r / p.heads, base = r * p.dim;
    float sum = 0.0f;
    for (uint64_t d = lane; d < p.dim; d += 32) {
      const float v = ld(p.x, p.dt, base + d);
      sum = __fmaf_rn(v, v, sum);
    }
    sum = warp_sum(sum);
    const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(sum, (float)p.dim), p.eps)));
    const uint64_t trow = ((token / p.input_seq) * p.table_seq + p.table_start + token % p.input_seq) * p.table_width;
    auto norm = [&](uint64_t d) {
      const float v = ld(p.x, p.dt, base + d);
      if (p.interleaved_v2)
        return rnd(__fmul_rn(rnd(__fmul_rn(v, inv), p.dt), ld(p.w, p.dt, d)), p.dt);
      return __fmul_rn(__fmul_rn(v, inv), ld(p.w, p.dt, d));
    };
    if (p.interleaved_v2) {
      for (uint64_t pair = lane; pair < p.table_width; pair += 32) {
        const float even = norm(2 * pair), odd = norm(2 * pair + 1);
        const float c = ld(p.cosv, p.dt_table, trow + pair), s = ld(p.sinv, p.dt_table, trow + pair);
        st(p.o, p.dt, base + 2 * pair, __fsub_rn(__fmul_rn(even, c), __fmul_rn(odd, s)));
        st(p.o, p.dt, base + 2 * pair + 1, __fadd_rn(__fmul_rn(even, s), __fmul_rn(odd, c)));
      }
    } else {
      for (uint64_t d = lane; d < half; d += 32) {
        const float a = norm(d), b = norm(d + half);
        const uint64_t second = p.table_width == p.rotary ? d + half : d;
        st(p.o, p.dt, base + d,
           __fsub_rn(__fmul_rn(a, ld(p.cosv, p.dt_table, trow + d)), __fmul_rn(b, ld(p.sinv, p.dt_table, trow + d))));
        st(p.o, p.dt, base + d + half,
           __fadd_rn(__fmul_rn(b, ld(p.cosv, p.dt_table, trow + second)),
                     __fmul_rn(a, ld(p.sinv, p.dt_table, trow + second))));
      }
    }
    for (uint64_t d = p.rotary + lane; d < p.dim; d += 32)
      st(p.o, p.dt, base + d, norm(d));
  }
}
// ---- RotaryFrequency (552-595): f64 angle, f32 tables ----
__global__ void k_rotary_frequency(const float *pos, const int32_t *pair_axes, const int32_t *pair_idx,
                                   const int32_t *axis_dims, float *cosv, float *sinv, uint64_t tokens,
                                   uint64_t axes, uint64_t pairs, double theta_ntk, unsigned int *bad) {
  GRID_STRIDE(i, tokens * pairs) {
    const uint64_t token = i / pairs, pair = i % pairs;
    const int32_t axis = pair_axes[pair], idx = pair_idx[pair];
    if (axis < 0 || (uint64_t)axis >= axes || idx < 0 || axis_dims[axis] <= 0 || (axis_dims[axis] & 1) ||
        2 * idx >= axis_dims[axis]) {
      atomicExch(bad, 1u);
      continue;
    }
    const double scale = 2.0 * (double)idx / (double)axis_dims[axis];
    const double omega = 1.0 / pow(theta_ntk, scale);
    const double angle = (double)pos[token * axes + axis] * omega;
    cosv[i] = (float)cos(angle);
    sinv[i] = (float)sin(angle);
  }
}
// ---- RotaryApply (597-625), interleaved pairs; tables F32 [B,S,P] ----
__global__ void k_rotary_apply(const void *x, const float *cosv, const float *sinv, void *o, uint32_t dt,
                               uint64_t tokens, uint64_t heads, uint64_t dim, uint64_t pairs) {
  GRID_STRIDE(i, tokens * heads * dim) {
    const uint64_t d = i % dim, th = i / dim, token = th / heads;
    if (d >= 2 * pairs) {
      st(o, dt, i, ld(x, dt, i));
      continue;
    }
    const uint64_t pair = d >> 1, base = th * dim + 2 * pair;
    const float even = ld(x, dt, base), odd = ld(x, dt, base + 1);
    const float c = cosv[token * pairs + pair], s = sinv[token * pairs + pair];
    st(o, dt, i,
       (d & 1) ? __fadd_rn(__fmul_rn(even, s), __fmul_rn(odd, c)) : __fsub_rn(__fmul_rn(even, c), __fmul_rn(odd, s)));
  }
}
// ---- ResidualGate (1703-1719), SwiGlu (1267-1286) ----
__global__ void k_residual_gate(const void *res, const void *branch, const void *gate, void *o, uint32_t dt,
                                uint64_t n, uint64_t width, uint64_t rows_per_gate) {
  GRID_STRIDE(i, n) {
    const uint64_t row = i / width;
    const float g = ld(gate, dt, (row / rows_per_gate) * width + i % width);
    st(o, dt, i, __fadd_rn(ld(res, dt, i), __fmul_rn(g, ld(branch, dt, i))));
  }
}
__global__ void k_swiglu(const void *x, void *o, uint32_t dt, uint64_t rows, uint64_t width, uint64_t in_width,
                         uint64_t start, int gate_first) {
  GRID_STRIDE(i, rows * width) {
    const uint64_t row = i / width, col = i % width, base = row * in_width + start;
    const float value = ld(x, dt, base + (gate_first ? width : 0) + col);
    const float gate = ld(x, dt, base + (gate_first ? 0 : width) + col);
    st(o, dt, i, __fmul_rn(value, __fdiv_rn(gate, __fadd_rn(1.0f, expf(-gate)))));
  }
}
// ---- layout ops: BroadcastTo (504-526), Slice (528-550), Concat (971-1000) ----
struct Dims8 {
  uint64_t out_dims[8], in_strides[8];
  uint32_t rank;
};
__global__ void k_gather(const void *x, void *o, uint32_t elem, uint64_t n, const Dims8 d, uint64_t offset) {
  GRID_STRIDE(i, n) {
    uint64_t coord = i, src = offset;
    for (int a = (int)d.rank - 1; a >= 0; --a) {
      src += (coord % d.out_dims[a]) * d.in_strides[a];
      coord /= d.out_dims[a];
    }
    if (elem == 4)
      static_cast<uint32_t *>(o)[i] = static_cast<const uint32_t *>(x)[src];
    else if (elem == 2)
      static_cast<uint16_t *>(o)[i] = static_cast<const uint16_t *>(x)[src];
    else
      static_cast<uint8_t *>(o)[i] = static_cast<const uint8_t *>(x)[src];
  }
}
__global__ void k_concat_part(const void *x, void *o, uint32_t elem, uint64_t outer, uint64_t chunk,
                              uint64_t out_chunk, uint64_t out_offset) {
  GRID_STRIDE(i, outer * chunk) {
    const uint64_t r = i / chunk, c = i % chunk, dst = r * out_chunk + out_offset + c;
    if (elem == 4)
      static_cast<uint32_t *>(o)[dst] = static_cast<const uint32_t *>(x)[i];
    else if (elem == 2)
      static_cast<uint16_t *>(o)[dst] = static_cast<const uint16_t *>(x)[i];
    else
      static_cast<uint8_t *>(o)[dst] = static_cast<const uint8_t *>(x)[i];
  }
}
// ---- BooleanMaskToBias (627-650), materialised form ----
__global__ void k_mask_to_bias(const uint8_t *mask, void *o, uint32_t dt, uint64_t B, uint64_t L, int vector_mask,
                               int mask_queries) {
  GRID_STRIDE(i, B * L * L) {
    const uint64_t key = i % L, query = (i / L) % L, b = i / (L * L);
    const bool valid = vector_mask ? ((!mask_queries || mask[b * L + query] != 0) && mask[b * L + key] != 0)
                                   : mask[(b * L + query) * L + key] != 0;
    st(o, dt, i, valid ? 0.0f : -INFINITY);
  }
}
// ---- Linear (1721-1739), plain float form for the small non-quantized linears of a block
// (modulation projections): one warp per output element ----
__global__ void k_linear(const void *x, const void *w, const void *bias, void *o, uint32_t dt, uint64_t M, uint64_t N,
                         uint64_t K) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const uint64_t nwarps = (uint64_t)gridDim.x * (blockDim.x >> 5);
  for (uint64_t e = warp; e < M * N; e += nwarps) {
    const uint64_t m = e / N, n = e % N;
    float acc = 0.0f;
    for (uint64_t k = lane; k < K; k += 32)
      acc = __fmaf_rn(ld(x, dt, m * K + k), ld(w, dt, n * K + k), acc);
    acc = warp_sum(acc);
    if (lane == 0)
      st(o, dt, e, bias ? __fadd_rn(acc, ld(bias, dt, n)) : acc);
  }
}

int done(const char *what) { return launched(cudaGetLastError(), what); }

} // namespace

int binary(const void *a, const void *b, void *o, uint32_t dt, uint64_t n, bool multiply, cudaStream_t s) {
  k_binary<<<blocks_for(n), 256, 0, s>>>(a, b, o, dt, n, multiply ? 1 : 0);
  return done("k_binary");
}
int unary(const void *a, void *o, uint32_t dt_in, uint32_t dt_out, uint64_t n, int kind, cudaStream_t s) {
  k_unary<<<blocks_for(n), 256, 0, s>>>(a, o, dt_in, dt_out, n, kind);
  return done("k_unary");
}
int bias_add(const void *a, const void *bias, void *o, uint32_t dt, uint64_t n, uint64_t width, cudaStream_t s) {
  k_bias<<<blocks_for(n), 256, 0, s>>>(a, bias, o, dt, n, width);
  return done("k_bias");
}
int affine_last_dim(const void *a, const void *scale, const void *bias, void *o, uint32_t dt, uint64_t n,
                    uint64_t width, cudaStream_t s) {
  k_affine<<<blocks_for(n), 256, 0, s>>>(a, scale, bias, o, dt, n, width);
  return done("k_affine");
}
int fill(void *o, uint32_t dt, uint64_t n, float value, cudaStream_t s) {
  k_fill<<<blocks_for(n), 256, 0, s>>>(o, dt, n, value);
  return done("k_fill");
}
int rms_norm(const void *x, const void *w, void *o, uint32_t dt, uint64_t rows, uint64_t cols, float eps,
             float weight_offset, cudaStream_t s) {
  const float2 *stats = nullptr;
  if (dt == 2) { // bf16 rows: the statistic in the reference's own order, by its own kernel
    int rc = 0;
    if (row_stats_sequential(x, rows, cols, eps, false, &stats, s, &rc) && rc)
      return rc;
  }
  k_rms_norm<<<row_blocks(rows), 256, 0, s>>>(x, w, o, dt, rows, cols, eps, weight_offset, stats);
  return done("k_rms_norm");
}
int layer_norm_modulate(const void *x, const void *w, const void *b, const void *scale, const void *shift, void *o,
                        uint32_t dt, uint64_t rows, uint64_t cols, uint64_t rows_per_mod, float eps, cudaStream_t s) {
  int rc = 0;
  if (layer_norm_modulate_fast(x, w, b, scale, shift, o, dt, rows, cols, rows_per_mod, eps, s, &rc))
    return rc;
  k_layer_norm_modulate<<<row_blocks(rows), 256, 0, s>>>(x, w, b, scale, shift, o, dt, rows, cols, rows_per_mod, eps);
  return done("k_layer_norm_modulate");
}
int rms_norm_modulate(const void *x, const void *w, const void *a, const void *b, void *o, uint32_t dt, uint64_t rows,
                      uint64_t cols, float eps, float weight_offset, bool shared_vector, uint64_t rows_per_vector,
                      cudaStream_t s) {
  int rc = 0;
  if (!shared_vector && weight_offset == 0.0f && rms_norm_modulate_fast(x, w, a, b, o, dt, rows, cols, eps, s, &rc))
    return rc;
  k_rms_norm_modulate<<<row_blocks(rows), 256, 0, s>>>(x, w, a, b, o, dt, rows, cols, eps, weight_offset,
                                                       shared_vector ? 1 : 0, rows_per_vector);
  return done("k_rms_norm_modulate");
}
int qk_norm_rope(const void *x, const void *w, const void *cosv, const void *sinv, void *o, uint32_t dt,
                 uint32_t dt_table, uint64_t tokens, uint64_t heads, uint64_t dim, uint64_t rotary,
                 uint64_t table_width, uint64_t input_seq, uint64_t table_seq, uint64_t table_start, float eps,
                 bool interleaved_v2, cudaStream_t s) {
  int rc = 0;
  if (qk_norm_rope_fast(x, w, cosv, sinv, o, nullptr, nullptr, dt, dt_table, tokens, heads, dim, rotary, table_width,
                        input_seq, table_seq, table_start, eps, interleaved_v2, nullptr, s, &rc))
    return rc;
  RopeParams p{x, w, cosv, sinv, o, dt, dt_table, tokens, heads, dim, rotary, table_width, input_seq, table_seq,
               table_start, eps, interleaved_v2 ? 1 : 0};
  k_qk_norm_rope<<<row_blocks(tokens * heads), 256, 0, s>>>(p);
  return done("k_qk_norm_rope");
}
int rotary_frequency(const float *pos, const int32_t *pair_axes, const int32_t *pair_idx, const int32_t *axis_dims,
                     float *cosv, float *sinv, uint64_t tokens, uint64_t axes, uint64_t pairs, double theta_ntk,
                     unsigned int *bad_flag, cudaStream_t s) {
  k_rotary_frequency<<<blocks_for(tokens * pairs), 256, 0, s>>>(pos, pair_axes, pair_idx, axis_dims, cosv, sinv,
                                                                tokens, axes, pairs, theta_ntk, bad_flag);
  return done("k_rotary_frequency");
}
int rotary_apply(const void *x, const float *cosv, const float *sinv, void *o, uint32_t dt, uint64_t tokens,
                 uint64_t heads, uint64_t dim, uint64_t pairs, cudaStream_t s) {
  k_rotary_apply<<<blocks_for(tokens * heads * dim), 256, 0, s>>>(x, cosv, sinv, o, dt, tokens, heads, dim, pairs);
  return done("k_rotary_apply");
}
int residual_gate(const void *res, const void *branch, const void *gate, void *o, uint32_t dt, uint64_t n,
                  uint64_t width, uint64_t rows_per_gate, cudaStream_t s) {
  int rc = 0;
  if (residual_gate_fast(res, branch, gate, o, dt, n, width, rows_per_gate, s, &rc))
    return rc;
  k_residual_gate<<<blocks_for(n), 256, 0, s>>>(res, branch, gate, o, dt, n, width, rows_per_gate);
  return done("k_residual_gate");
}
int swiglu(const void *x, void *o, uint32_t dt, uint64_t rows, uint64_t width, uint64_t in_width, uint64_t start,
           bool gate_first, cudaStream_t s) {
  int rc = 0;
  if (swiglu_fast(x, o, dt, rows, width, in_width, start, gate_first, s, &rc))
    return rc;
  k_swiglu<<<blocks_for(rows * width), 256, 0, s>>>(x, o, dt, rows, width, in_width, start, gate_first ? 1 : 0);
  return done("k_swiglu");
}
int gather(const void *x, void *o, uint32_t elem_bytes, uint32_t rank, const uint64_t *out_dims,
           const uint64_t *in_strides, uint64_t offset, cudaStream_t s) {
  Dims8 d{};
  d.rank = rank;
  uint64_t n = 1;
  for (uint32_t a = 0; a < rank; ++a) {
    d.out_dims[a] = out_dims[a];
    d.in_strides[a] = in_strides[a];
    n *= out_dims[a];
  }
  k_gather<<<blocks_for(n), 256, 0, s>>>(x, o, elem_bytes, n, d, offset);
  return done("k_gather");
}
int concat_part(const void *x, void *o, uint32_t elem_bytes, uint64_t outer, uint64_t chunk, uint64_t out_chunk,
                uint64_t out_offset, cudaStream_t s) {
  k_concat_part<<<blocks_for(outer * chunk), 256, 0, s>>>(x, o, elem_bytes, outer, chunk, out_chunk, out_offset);
  return done("k_concat_part");
}
int mask_to_bias(const uint8_t *mask, void *o, uint32_t dt, uint64_t B, uint64_t L, bool vector_mask,
                 bool mask_queries, cudaStream_t s) {
  k_mask_to_bias<<<blocks_for(B * L * L), 256, 0, s>>>(mask, o, dt, B, L, vector_mask ? 1 : 0, mask_queries ? 1 : 0);
  return done("k_mask_to_bias");
}
int linear(const void *x, const void *w, const void *bias, void *o, uint32_t dt, uint64_t M, uint64_t N, uint64_t K,
           cudaStream_t s) {
  k_linear<<<row_blocks(M * N), 256, 0, s>>>(x, w, bias, o, dt, M, N, K);
  return done("k_linear");
}

} // namespace glue
} // namespace difb200
