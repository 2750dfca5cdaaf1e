/*
 * TEST INFRASTRUCTURE ONLY: a plain-C restatement of the reference project's CPU
 * arithmetic for the quantized DiT hot path. It is the checker the CUDA kernels are
 * compared with; the product library never links, loads or calls it.
 *
 * Parity status: PINNED. Every function that restates a reference function is checked
 * bit-for-bit against the reference's own CPU executor (built from the reference sources
 * by the Makefile in this directory) through the committed fixtures under tests/golden/; the
 * weight packer's functions (equalisation vector, MSE scale search, row encoder) against runs of
 * the reference's own packer, which the Makefile builds as a probe from the tool's source.
 * One exception, UNPINNED: orc_attention_int8. The reference has no CPU form of INT8 attention,
 * so that function defines this repository's own numerical contract; its Q/K codes and scales
 * are the reference's (QuantizeInt8Rows, Direct) and it is additionally compared, with a
 * tolerance, against the reference's exact Attention.
 *
 * Each function cites the reference file:line it follows (paths inside the reference
 * project). Build flags: -O3 without -march, so x86-64 never contracts a*b+c into an fma
 * and sums keep the reference's rounding.
 */
#include <math.h>
#include <pthread.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_EXPORT __attribute__((visibility("default")))


/* A minimal pthread parallel-for. Rows of every function here are independent, so results
 * do not depend on the thread count (orc_set_threads, default 1). */
static int g_threads = 1;
ORC_EXPORT void orc_set_threads(int n) { g_threads = n < 1 ? 1 : (n > 256 ? 256 : n); }
typedef void (*orc_body)(void *ctx, int64_t begin, int64_t end);
typedef struct {
  orc_body body;
  void *ctx;
  int64_t begin, end;
} orc_job;
static void *orc_job_main(void *arg) {
  orc_job *job = (orc_job *)arg;
  job->body(job->ctx, job->begin, job->end);
  return NULL;
}
static void parallel_for(int64_t count, orc_body body, void *ctx) {
  int n = g_threads;
  if (count < n)
    n = count > 0 ? (int)count : 1;
  if (n <= 1) {
    body(ctx, 0, count);
    return;
  }
  pthread_t tid[256];
  orc_job jobs[256];
  const int64_t chunk = (count + n - 1) / n;
  for (int t = 0; t < n; ++t) {
    jobs[t].body = body;
    jobs[t].ctx = ctx;
    jobs[t].begin = t * chunk < count ? t * chunk : count;
    jobs[t].end = jobs[t].begin + chunk < count ? jobs[t].begin + chunk : count;
    pthread_create(&tid[t], NULL, orc_job_main, &jobs[t]);
  }
  for (int t = 0; t < n; ++t)
    pthread_join(tid[t], NULL);
}

/* src/runtime/scalar.cpp:18-26: bf16 store is round-to-nearest-even on the raw bits (no
 * NaN special case); bf16 load is a 16-bit left shift. */
static inline uint16_t f2bf(float value) {
  uint32_t bits;
  memcpy(&bits, &value, 4);
  const uint32_t rounding = 0x7fffU + ((bits >> 16U) & 1U);
  return (uint16_t)((bits + rounding) >> 16U);
}
static inline float bf2f(uint16_t value) {
  const uint32_t bits = (uint32_t)value << 16U;
  float out;
  memcpy(&out, &bits, 4);
  return out;
}
static inline float rbf(float value) { return bf2f(f2bf(value)); }

static inline int clampi(int v, int lo, int hi) {
  return v < lo ? lo : (v > hi ? hi : v);
}

/* src/runtime/cpu_executor.cpp:183-189: fixed Rademacher diagonal of the signed
 * variants, a 3-round integer hash of the (global) column index. */
static inline float rotation_sign(uint64_t column) {
  uint32_t hash = (uint32_t)column + 0x9e3779b9U;
  hash = (hash ^ (hash >> 16U)) * 0x7feb352dU;
  hash = (hash ^ (hash >> 15U)) * 0x846ca68bU;
  hash ^= hash >> 16U;
  return (hash & 1U) != 0U ? -1.0F : 1.0F;
}

/* include/dif/ir/ir.hpp:285-293 */
enum {
  ORC_DIRECT = 1,
  ORC_H256 = 2,
  ORC_H256_SIGNED = 3,
  ORC_H4096_SIGNED = 4,
  ORC_H256_F32 = 5,
  ORC_H256_F32_SIGNED = 6,
  ORC_H4096_F32_SIGNED = 7
};

/*
 * QuantizeInt8Rows: src/runtime/cpu_executor.cpp:124-307.
 * parts/part_widths: the 1..n bf16 inputs that are concatenated on the last axis
 * (:138-147). clip is the static Scale attribute or the dynamic F32[1] input (:179-182).
 * rcodes/rscales may be NULL (two-output form). Returns 0, or 1 on an illegal width.
 */
typedef struct {
  const uint16_t *const *parts;
  const uint64_t *part_widths;
  uint64_t part_count, columns;
  int implementation;
  float clip;
  int8_t *codes;
  float *scales;
  int8_t *rcodes;
  float *rscales;
  int mse; /* weight rows: scale from the offline packer's MSE search */
  const uint16_t *equalise; /* weight rows: bf16 [columns] divisor, or NULL */
} quant_ctx;

/* tools/difflux2sample.cpp:1225-1259 (choose_mse_int8_weight_scale): seven clip factors, the
 * bf16-rounded scale of each, squared error over every fourth element in double, first best
 * wins. Pinned bit for bit against the reference's own function (oracle/_ref/difpacker_scale,
 * which includes the tool's source) and through the committed fixture made from it. */
static float choose_mse_weight_scale(const float *values, uint64_t count) {
  static const float factors[7] = {1.0F, 0.96F, 0.92F, 0.88F, 0.84F, 0.80F, 0.76F};
  float maximum = 0.0F;
  for (uint64_t i = 0; i < count; ++i)
    maximum = fmaxf(maximum, fabsf(values[i]));
  if (maximum == 0.0F)
    return 1.0e-30F;
  float best_scale = INFINITY;
  double best_error = INFINITY;
  for (int f = 0; f < 7; ++f) {
    const float scale = rbf(fmaxf(maximum * factors[f] / 127.0F, 1.0e-30F));
    double error = 0.0;
    for (uint64_t i = 0; i < count; i += 4U) {
      const float value = rbf(values[i]);
      const float divided = rbf(value / scale);
      const int encoded = clampi((int)nearbyintf(divided), -128, 127);
      const double delta = (double)value - (double)encoded * scale;
      error += delta * delta;
    }
    if (error < best_error) {
      best_error = error;
      best_scale = scale;
    }
  }
  return best_scale;
}

/* The search alone, on fp32 rows (what the packer hands it: the rotated weight row). */
ORC_EXPORT void orc_choose_mse_weight_scale(const float *values, uint64_t rows, uint64_t columns,
                                            float *scales) {
  for (uint64_t r = 0; r < rows; ++r)
    scales[r] = choose_mse_weight_scale(values + r * columns, columns);
}

static void quant_body(void *vctx, int64_t row_begin, int64_t row_end) {
  const quant_ctx *ctx = (const quant_ctx *)vctx;
  const uint16_t *const *parts = ctx->parts;
  const uint64_t *part_widths = ctx->part_widths;
  const uint64_t part_count = ctx->part_count, columns = ctx->columns;
  const int implementation = ctx->implementation;
  const float clip = ctx->clip;
  int8_t *codes = ctx->codes, *rcodes = ctx->rcodes;
  float *scales = ctx->scales, *rscales = ctx->rscales;
  const int convrot = implementation != ORC_DIRECT;
  const int f32 = implementation == ORC_H256_F32 ||
                  implementation == ORC_H256_F32_SIGNED ||
                  implementation == ORC_H4096_F32_SIGNED;
  const int sgn = implementation == ORC_H256_SIGNED ||
                  implementation == ORC_H256_F32_SIGNED ||
                  implementation == ORC_H4096_SIGNED ||
                  implementation == ORC_H4096_F32_SIGNED;
  const uint64_t group = (implementation == ORC_H4096_SIGNED ||
                          implementation == ORC_H4096_F32_SIGNED)
                             ? 4096U
                             : 256U;
  {
    float *t = (float *)malloc(sizeof(float) * (size_t)columns);
    for (int64_t srow = row_begin; srow < row_end; ++srow) {
      const uint64_t row = (uint64_t)srow;
      const uint64_t base = row * columns;
      /* gather the logical row (:138-147) */
      uint64_t c0 = 0;
      for (uint64_t p = 0; p < part_count; ++p) {
        const uint16_t *src = parts[p] + row * part_widths[p];
        for (uint64_t c = 0; c < part_widths[p]; ++c)
          t[c0 + c] = bf2f(src[c]);
        c0 += part_widths[p];
      }
      if (ctx->equalise) /* tools/difflux2sample.cpp:3005-3014: w / e, then the sign */
        for (uint64_t c = 0; c < columns; ++c)
          t[c] = t[c] / bf2f(ctx->equalise[c]);
      float maximum = 0.0F;
      if (convrot) {
        if (sgn)
          for (uint64_t c = 0; c < columns; ++c)
            t[c] = t[c] * rotation_sign(c); /* :197-201 */
        /* radix-4 Kronecker stages, stride 1,4,16,64(,256,1024) (:202-229) */
        for (uint64_t stride = 1; stride < group; stride *= 4U) {
          for (uint64_t g = 0; g < columns; g += group) {
            for (uint64_t lane = 0; lane < group / 4U; ++lane) {
              const uint64_t i =
                  g + (lane % stride) + (lane / stride) * (4U * stride);
              const float x0 = t[i], x1 = t[i + stride],
                          x2 = t[i + 2U * stride], x3 = t[i + 3U * stride];
              t[i] = 0.5F * (x0 + x1 + x2 - x3);
              t[i + stride] = 0.5F * (x0 + x1 - x2 + x3);
              t[i + 2U * stride] = 0.5F * (x0 - x1 + x2 + x3);
              t[i + 3U * stride] = 0.5F * (-x0 + x1 + x2 + x3);
            }
          }
        }
      }
      for (uint64_t c = 0; c < columns; ++c)
        maximum = fmaxf(maximum, fabsf(t[c])); /* :230-235 */
      /* :236-237; for weight rows packed with the MSE search,
       * tools/difflux2sample.cpp:3020-3031 (scale) and :3032-3037 (what is stored) */
      const float scale = (ctx->mse && convrot) ? choose_mse_weight_scale(t, columns)
                                                : fmaxf(maximum * clip / 127.0F, 1.0e-30F);
      const float scale_bf16 = rbf(scale);
      const float stored = ((sgn || (ctx->mse && convrot)) && !f32) ? scale_bf16 : scale; /* :239-240 */
      scales[row] = stored;
      for (uint64_t c = 0; c < columns; ++c) {
        int rounded;
        if (f32) { /* :242-246 */
          rounded = clampi((int)nearbyintf(t[c] / scale), -127, 127);
        } else if (convrot) { /* :247-254 */
          const float v = rbf(t[c]);
          const float d = rbf(v / scale_bf16);
          rounded = clampi((int)nearbyintf(d), -128, 127);
        } else { /* :255-260 */
          rounded = clampi((int)nearbyintf(t[c] / scale), -127, 127);
        }
        codes[base + c] = (int8_t)rounded;
      }
      if (!rcodes)
        continue;
      /* residual pair (:262-305) */
      float rmax = 0.0F;
      for (uint64_t c = 0; c < columns; ++c) {
        const float v = f32 ? t[c] : (convrot ? rbf(t[c]) : t[c]);
        rmax = fmaxf(rmax, fabsf(fmaf(-(float)codes[base + c], stored, v)));
      }
      const float rscale = fmaxf(rmax / 127.0F, 1.0e-30F);
      const float rscale_bf16 = rbf(rscale);
      rscales[row] = (sgn && !f32) ? rscale_bf16 : rscale;
      for (uint64_t c = 0; c < columns; ++c) {
        const float v = f32 ? t[c] : (convrot ? rbf(t[c]) : t[c]);
        const float r = fmaf(-(float)codes[base + c], stored, v);
        float d;
        if (f32)
          d = r / rscale;
        else if (convrot)
          d = rbf(rbf(r) / rscale_bf16);
        else
          d = r / rscale;
        rcodes[base + c] = (int8_t)clampi((int)nearbyintf(d),
                                          (convrot && !f32) ? -128 : -127, 127);
      }
    }
    free(t);
  }
}

ORC_EXPORT int orc_quantize_int8_rows(const uint16_t *const *parts,
                                      const uint64_t *part_widths,
                                      uint64_t part_count, uint64_t rows,
                                      int implementation, float clip,
                                      int8_t *codes, float *scales,
                                      int8_t *rcodes, float *rscales) {
  uint64_t columns = 0;
  for (uint64_t p = 0; p < part_count; ++p)
    columns += part_widths[p];
  const uint64_t group = (implementation == ORC_H4096_SIGNED ||
                          implementation == ORC_H4096_F32_SIGNED)
                             ? 4096U
                             : 256U;
  if (implementation < ORC_DIRECT || implementation > ORC_H4096_F32_SIGNED)
    return 1;
  if (implementation != ORC_DIRECT && columns % group != 0U)
    return 1;
  quant_ctx ctx = {parts, part_widths, part_count, columns, implementation,
                   clip,  codes,       scales,     rcodes,  rscales, 0, NULL};
  parallel_for((int64_t)rows, quant_body, &ctx);
  return 0;
}

/* Input equalisation of the offline packer, tools/difflux2sample.cpp:2967-2990: per column the
 * absmax over the rows, their geometric mean as the centre, sqrt(max / centre) clamped to
 * [0.5, 2] and stored as bf16. Pinned through whole runs of the reference packer (its cache
 * file's input_scale tensor). */
ORC_EXPORT void orc_weight_equalization(const uint16_t *weight, uint64_t rows,
                                        uint64_t columns, uint16_t *out) {
  float *maxima = (float *)calloc((size_t)columns, sizeof(float));
  for (uint64_t r = 0; r < rows; ++r)
    for (uint64_t c = 0; c < columns; ++c)
      maxima[c] = fmaxf(maxima[c], fabsf(bf2f(weight[r * columns + c])));
  double log_sum = 0.0;
  for (uint64_t c = 0; c < columns; ++c)
    log_sum += logf(fmaxf(maxima[c], 1.0e-30F));
  const float center = (float)exp(log_sum / (double)columns);
  for (uint64_t c = 0; c < columns; ++c) {
    float v = sqrtf(maxima[c] / fmaxf(center, 1.0e-30F));
    v = v < 0.5F ? 0.5F : (v > 2.0F ? 2.0F : v);
    out[c] = f2bf(v);
  }
  free(maxima);
}

/* Weight-side packing of a bf16 [rows, columns] matrix, tools/difflux2sample.cpp:2994-3059
 * (clip 1, no residual); mse != 0 uses choose_mse_weight_scale. Without mse this is
 * orc_quantize_int8_rows on one part, which is pinned against the reference executor. */
ORC_EXPORT int orc_quantize_weight_rows(const uint16_t *weight,
                                        const uint16_t *equalise, uint64_t rows,
                                        uint64_t columns, int implementation,
                                        int mse, int8_t *codes, float *scales) {
  if (implementation < ORC_H256 || implementation > ORC_H4096_F32_SIGNED)
    return 1;
  const uint64_t group = (implementation == ORC_H4096_SIGNED ||
                          implementation == ORC_H4096_F32_SIGNED)
                             ? 4096U
                             : 256U;
  if (columns % group != 0U)
    return 1;
  const uint16_t *parts[1] = {weight};
  const uint64_t widths[1] = {columns};
  quant_ctx ctx = {parts, widths, 1,     columns, implementation, 1.0F,
                   codes, scales, NULL, NULL,    mse,     equalise};
  parallel_for((int64_t)rows, quant_body, &ctx);
  return 0;
}

/*
 * LinearInt8Scaled: src/runtime/cpu_executor.cpp:309-335.
 * acc_out (may be NULL) receives the raw INT32 accumulators; out receives
 * bf16((float(acc) * row[m]) * col[n]).
 */
typedef struct {
  const int8_t *x, *w;
  const float *row_scales, *col_scales;
  uint64_t N, K;
  int32_t *acc_out;
  uint16_t *out;
} linear_ctx;

static void linear_body(void *vctx, int64_t begin, int64_t end) {
  const linear_ctx *ctx = (const linear_ctx *)vctx;
  const int8_t *x = ctx->x, *w = ctx->w;
  const float *row_scales = ctx->row_scales, *col_scales = ctx->col_scales;
  const uint64_t N = ctx->N, K = ctx->K;
  int32_t *acc_out = ctx->acc_out;
  uint16_t *out = ctx->out;
  for (int64_t sm = begin; sm < end; ++sm) {
    const uint64_t m = (uint64_t)sm;
    for (uint64_t n = 0; n < N; ++n) {
      int32_t acc = 0;
      const int8_t *xr = x + m * K;
      const int8_t *wr = w + n * K;
      for (uint64_t k = 0; k < K; ++k)
        acc += (int32_t)xr[k] * (int32_t)wr[k];
      if (acc_out)
        acc_out[m * N + n] = acc;
      if (out)
        out[m * N + n] = f2bf((float)acc * row_scales[m] * col_scales[n]);
    }
  }
}

ORC_EXPORT void orc_linear_int8_scaled(const int8_t *x, const int8_t *w,
                                       const float *row_scales,
                                       const float *col_scales, uint64_t M,
                                       uint64_t N, uint64_t K, int32_t *acc_out,
                                       uint16_t *out) {
  linear_ctx ctx = {x, w, row_scales, col_scales, N, K, acc_out, out};
  parallel_for((int64_t)M, linear_body, &ctx);
}

/* BiasAdd: src/runtime/cpu_executor.cpp:1288-1296 (bf16 in, bf16 bias, bf16 out). */
ORC_EXPORT void orc_bias_add(const uint16_t *in, const uint16_t *bias,
                             uint64_t count, uint64_t width, uint16_t *out) {
  for (uint64_t i = 0; i < count; ++i)
    out[i] = f2bf(bf2f(in[i]) + bf2f(bias[i % width]));
}

/* Gelu, tanh form: src/runtime/cpu_executor.cpp:93-113. */
ORC_EXPORT void orc_gelu_tanh(const uint16_t *in, uint64_t count,
                              uint16_t *out) {
  const float kSqrtTwoOverPi = 0.7978845608028654F;
  const float kCubic = 0.044715F;
  for (uint64_t i = 0; i < count; ++i) {
    const float v = bf2f(in[i]);
    const float cubic = v * v * v;
    const float inner = kSqrtTwoOverPi * (v + kCubic * cubic);
    out[i] = f2bf(0.5F * v * (1.0F + tanhf(inner)));
  }
}

/* RmsNorm: src/runtime/cpu_executor.cpp:1051-1075 (bf16 storage, weight bf16). */
ORC_EXPORT void orc_rms_norm(const uint16_t *in, const uint16_t *weight,
                             uint64_t rows, uint64_t columns, float epsilon,
                             float weight_offset, uint16_t *out) {
  for (uint64_t r = 0; r < rows; ++r) {
    float sum = 0.0F;
    for (uint64_t c = 0; c < columns; ++c) {
      const float v = bf2f(in[r * columns + c]);
      sum += v * v;
    }
    const float inverse = 1.0F / sqrtf(sum / (float)columns + epsilon);
    for (uint64_t c = 0; c < columns; ++c)
      out[r * columns + c] = f2bf(bf2f(in[r * columns + c]) * inverse *
                                  (bf2f(weight[c]) + weight_offset));
  }
}

/* RotaryApply, interleaved pairs: src/runtime/cpu_executor.cpp:597-625.
 * in/out bf16 [B,S,H,D]; cosine/sine f32 [B,S,P]. */
ORC_EXPORT void orc_rotary_apply(const uint16_t *in, const float *cosine,
                                 const float *sine, uint64_t B, uint64_t S,
                                 uint64_t H, uint64_t D, uint64_t P,
                                 uint16_t *out) {
  for (uint64_t bt = 0; bt < B * S; ++bt) {
    for (uint64_t h = 0; h < H; ++h) {
      const uint64_t base = (bt * H + h) * D;
      for (uint64_t p = 0; p < P; ++p) {
        const float even = bf2f(in[base + 2U * p]);
        const float odd = bf2f(in[base + 2U * p + 1U]);
        const float c = cosine[bt * P + p], s = sine[bt * P + p];
        out[base + 2U * p] = f2bf(even * c - odd * s);
        out[base + 2U * p + 1U] = f2bf(even * s + odd * c);
      }
      for (uint64_t d = 2U * P; d < D; ++d)
        out[base + d] = in[base + d];
    }
  }
}

/*
 * Exact Attention: src/runtime/cpu_executor.cpp:1839-1910, with the key-only boolean
 * mask of BooleanMaskToBias(MaskQueries=false) (:627-650) applied as the 0/-inf bias it
 * would materialise. q/out bf16 [B,S,H,D]; k,v bf16 [B,S,KV,D]; key_valid (may be NULL)
 * uint8 [B,S]. Query rows are independent, so they are spread over threads.
 */
typedef struct {
  const void *q, *k, *v;
  const float *qs, *ks;
  const uint8_t *key_valid;
  uint64_t B, S, H, KV, D;
  float scale;
  int32_t *acc_out;
  uint16_t *out;
  uint64_t Sq;  /* query tokens per batch entry (== S for the DiffIR op, < S for a query sample) */
  int fp32_p;   /* INT8 form only: keep P in fp32 (the reported middle tier) */
} attn_ctx;

static void attention_exact_body(void *vctx, int64_t begin, int64_t end) {
  const attn_ctx *ctx = (const attn_ctx *)vctx;
  const uint16_t *q = (const uint16_t *)ctx->q, *k = (const uint16_t *)ctx->k,
                 *v = (const uint16_t *)ctx->v;
  const uint8_t *key_valid = ctx->key_valid;
  const uint64_t S = ctx->S, Sq = ctx->Sq, H = ctx->H, KV = ctx->KV, D = ctx->D;
  const float scale = ctx->scale;
  uint16_t *out = ctx->out;
  const uint64_t group = H / KV;
  {
    float *prob = (float *)malloc(sizeof(float) * (size_t)S);
    {
      for (int64_t bq = begin; bq < end; ++bq) {
        const uint64_t b = (uint64_t)bq / Sq, query = (uint64_t)bq % Sq;
        for (uint64_t head = 0; head < H; ++head) {
          const uint64_t kvh = head / group;
          const uint16_t *qr = q + ((b * Sq + query) * H + head) * D;
          uint16_t *orow = out + ((b * Sq + query) * H + head) * D;
          float maximum = -INFINITY;
          for (uint64_t key = 0; key < S; ++key) {
            const uint16_t *kr = k + ((b * S + key) * KV + kvh) * D;
            float score = 0.0F;
            for (uint64_t d = 0; d < D; ++d)
              score = fmaf(bf2f(qr[d]), bf2f(kr[d]), score);
            score *= scale;
            if (key_valid)
              score += key_valid[b * S + key] ? 0.0F : -INFINITY;
            prob[key] = score;
            maximum = fmaxf(maximum, score);
          }
          if (!isfinite(maximum)) { /* :1881-1887 */
            for (uint64_t d = 0; d < D; ++d)
              orow[d] = f2bf(0.0F);
            continue;
          }
          float denominator = 0.0F;
          for (uint64_t key = 0; key < S; ++key) {
            prob[key] = expf(prob[key] - maximum);
            denominator += prob[key];
          }
          for (uint64_t d = 0; d < D; ++d) {
            float value = 0.0F;
            for (uint64_t key = 0; key < S; ++key)
              value = fmaf(prob[key] / denominator,
                           bf2f(v[((b * S + key) * KV + kvh) * D + d]), value);
            orow[d] = f2bf(value);
          }
        }
      }
    }
    free(prob);
  }
}

ORC_EXPORT void orc_attention_exact(const uint16_t *q, const uint16_t *k,
                                    const uint16_t *v, const uint8_t *key_valid,
                                    uint64_t B, uint64_t S, uint64_t H,
                                    uint64_t KV, uint64_t D, float scale,
                                    uint16_t *out) {
  attn_ctx ctx = {q, k, v, NULL, NULL, key_valid, B, S, H, KV, D, scale, NULL, out, S, 0};
  parallel_for((int64_t)(B * S), attention_exact_body, &ctx);
}

/* The same op for a sample of queries: q/out [B,Sq,H,D] against all S keys (query rows are
 * independent in cpu_executor.cpp:1853-1908, so a row computed here equals the row of the full op). */
ORC_EXPORT void orc_attention_exact_rows(const uint16_t *q, const uint16_t *k,
                                         const uint16_t *v, const uint8_t *key_valid,
                                         uint64_t B, uint64_t Sq, uint64_t S, uint64_t H,
                                         uint64_t KV, uint64_t D, float scale,
                                         uint16_t *out) {
  attn_ctx ctx = {q, k, v, NULL, NULL, key_valid, B, S, H, KV, D, scale, NULL, out, Sq, 0};
  parallel_for((int64_t)(B * Sq), attention_exact_body, &ctx);
}

/*
 * INT8 attention, the numerical contract of this repository's kernel (no CPU form exists
 * in the reference; the loop structure, the GQA head mapping and the all-masked-row rule
 * follow src/runtime/cpu_executor.cpp:1853-1908).
 *
 *   q8 [B,S,H,D], qs [B,S,H]; k8 [B,S,KV,D], ks [B,S,KV]: codes and scales exactly as
 *   QuantizeInt8Rows(Direct) produces them on the [B,S,H,D] / [B,S,KV,D] tensors
 *   (one row per token-head); v bf16 [B,S,KV,D].
 *
 *   acc   = sum_d q8*k8                      (int32, exact)
 *   u_j   = float(acc) * ks'_j               (fp32; ks'_j = ks_j rounded, nearest-even, to 22
 *                                             significant bits, which lets the kernel fuse the
 *                                             int->float conversion into one exact fma)
 *   A_i   = qs_i * (scale * log2(e))         (fp32; both products rounded to fp32)
 *   m_i   = ceil(max_j(u_j) * A_i)           (an integer; masked keys excluded)
 *   p_j   = exp2(fma(u_j, A_i, -m_i))        (fp32)
 *   P_j   = bf16(p_j)
 *   out   = bf16( (sum_j P_j * v_j) / (sum_j p_j) )   (fp32 accumulation; the kernel adds the
 *                                                      p_j in a different order)
 *
 * The power-of-two (integer) maximum makes every rescaling of an online-softmax kernel an
 * exact power of two, so the kernel's bf16 P agrees with this two-pass form except for
 * rare last-bit differences of the fp32 exponent argument.
 * acc_out (may be NULL) receives the int32 accumulators of (batch 0, head 0) as [S,S].
 */
static void attention_int8_body(void *vctx, int64_t begin, int64_t end) {
  const attn_ctx *ctx = (const attn_ctx *)vctx;
  const int8_t *q8 = (const int8_t *)ctx->q, *k8 = (const int8_t *)ctx->k;
  const uint16_t *v = (const uint16_t *)ctx->v;
  const float *qs = ctx->qs, *ks = ctx->ks;
  const uint8_t *key_valid = ctx->key_valid;
  const uint64_t S = ctx->S, Sq = ctx->Sq, H = ctx->H, KV = ctx->KV, D = ctx->D;
  int32_t *acc_out = ctx->acc_out;
  uint16_t *out = ctx->out;
  const uint64_t group = H / KV;
  const float c = ctx->scale * 1.4426950408889634F;
  {
    float *u = (float *)malloc(sizeof(float) * (size_t)S);
    float *o = (float *)malloc(sizeof(float) * (size_t)D);
    {
      for (int64_t bq = begin; bq < end; ++bq) {
        const uint64_t b = (uint64_t)bq / Sq, query = (uint64_t)bq % Sq;
        for (uint64_t head = 0; head < H; ++head) {
          const uint64_t kvh = head / group;
          const int8_t *qr = q8 + ((b * Sq + query) * H + head) * D;
          uint16_t *orow = out + ((b * Sq + query) * H + head) * D;
          const float A = qs[(b * Sq + query) * H + head] * c;
          float umax = -INFINITY;
          for (uint64_t key = 0; key < S; ++key) {
            const int8_t *kr = k8 + ((b * S + key) * KV + kvh) * D;
            int32_t acc = 0;
            for (uint64_t d = 0; d < D; ++d)
              acc += (int32_t)qr[d] * (int32_t)kr[d];
            if (acc_out && b == 0 && head == 0)
              acc_out[query * S + key] = acc; /* only from the entry point with Sq == S */
            uint32_t kbits;
            memcpy(&kbits, &ks[(b * S + key) * KV + kvh], 4);
            kbits = (kbits + 1U + ((kbits >> 2U) & 1U)) & ~3U;
            float k22;
            memcpy(&k22, &kbits, 4);
            float uj = (float)acc * k22;
            if (key_valid && !key_valid[b * S + key])
              uj = -INFINITY;
            u[key] = uj;
            umax = fmaxf(umax, uj);
          }
          if (!isfinite(umax)) {
            for (uint64_t d = 0; d < D; ++d)
              orow[d] = f2bf(0.0F);
            continue;
          }
          const float m = ceilf(umax * A);
          float denominator = 0.0F;
          for (uint64_t d = 0; d < D; ++d)
            o[d] = 0.0F;
          for (uint64_t key = 0; key < S; ++key) {
            if (u[key] == -INFINITY)
              continue;
            const float p = exp2f(fmaf(u[key], A, -m));
            denominator += p;
            const float P = ctx->fp32_p ? p : rbf(p);
            const uint16_t *vr = v + ((b * S + key) * KV + kvh) * D;
            for (uint64_t d = 0; d < D; ++d)
              o[d] += P * bf2f(vr[d]);
          }
          for (uint64_t d = 0; d < D; ++d)
            orow[d] = f2bf(o[d] / denominator);
        }
      }
    }
    free(u);
    free(o);
  }
}

ORC_EXPORT void orc_attention_int8(const int8_t *q8, const float *qs,
                                   const int8_t *k8, const float *ks,
                                   const uint16_t *v, const uint8_t *key_valid,
                                   uint64_t B, uint64_t S, uint64_t H,
                                   uint64_t KV, uint64_t D, float scale,
                                   int32_t *acc_out, uint16_t *out) {
  attn_ctx ctx = {q8, k8, v, qs, ks, key_valid, B, S, H, KV, D, scale, acc_out, out, S, 0};
  parallel_for((int64_t)(B * S), attention_int8_body, &ctx);
}

/* The same contract for a sample of queries (q8 / qs / out over Sq query tokens, keys and values
 * over S tokens): the token-sharded form, and the way rows of very long sequences are checked.
 * fp32_p != 0 keeps P unrounded: same quantisation, exact fp32 softmax weights -- the middle tier
 * that separates the error of the bf16 P from the error of the INT8 codes. */
ORC_EXPORT void orc_attention_int8_rows(const int8_t *q8, const float *qs,
                                        const int8_t *k8, const float *ks,
                                        const uint16_t *v, const uint8_t *key_valid,
                                        uint64_t B, uint64_t Sq, uint64_t S, uint64_t H,
                                        uint64_t KV, uint64_t D, float scale, int fp32_p,
                                        uint16_t *out) {
  attn_ctx ctx = {q8, k8, v, qs, ks, key_valid, B, S, H, KV, D, scale, NULL, out, Sq, fp32_p};
  parallel_for((int64_t)(B * Sq), attention_int8_body, &ctx);
}

ORC_EXPORT int orc_version(void) { return 1; }
