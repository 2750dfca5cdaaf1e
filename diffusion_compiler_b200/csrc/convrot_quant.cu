// QuantizeInt8Rows for sm_100a: orthogonal block rotation fused with per-row absmax INT8
// quantisation. Semantics follow the reference opcode bit for bit
// (reference src/runtime/cpu_executor.cpp:124-307; generated GPU kernel
// src/compiler/compiler.cpp:635-845). bf16 is read once from HBM, codes and scales are
// written once; the rotation runs in registers with one shared-memory transpose per
// 256-wide group.
//
// ConvRot kernel layout. A 256-wide group is the Kronecker product H4 (x) H4 (x) H4 (x) H4,
// applied as four radix-4 stages with strides 1, 4, 16, 64 in exactly the reference's fp32
// association order ((x0+x1)+x2)-x3 etc. The reference multiplies every stage by 0.5; a
// multiplication by a power of two commutes with fp32 rounding, so the kernel skips it and
// carries values scaled by 16 (64 for the six-stage 4096-wide variants), folding the factor into the
// divisor. Results are bit-identical unless an intermediate leaves the normal fp32 range.
//
// Each thread owns 16 consecutive elements of two neighbouring groups and keeps them as 16
// packed fp32x2 registers (lane 0 of the pair = first group, lane 1 = second group), so every
// butterfly is one packed add/sub for two groups. Stages 0-1 run on the thread's own 16
// elements; a 16x16 transpose through shared memory (XOR-swizzled, conflict-free) gives the
// thread the 16 elements of stride 16, on which stages 2-3 run. The 4096-wide variants add a
// second, CTA-wide transpose across 16 groups for stages 4-5.
#include "common.cuh"
#include "glue.h"
#include "ops.h"

#include <cstdio>

namespace difb200 {
namespace {

constexpr int kMaxParts = 8;

struct QuantParams {
  const uint16_t *part[kMaxParts];
  uint32_t width[kMaxParts];
  uint32_t part_count;
  uint32_t columns;
  uint64_t rows;
  float clip;
  const float *clip_device;
  int8_t *codes;
  float *scales;
  int8_t *rcodes;
  float *rscales;
  uint32_t mse;   // weight rows: choose the row scale by the offline packer's MSE search
  const uint16_t *equalise; // weight rows: bf16 [columns], every element is divided by its entry first
  // RmsNormModulate in front of the quantiser (explicit scale / shift layout), all bf16:
  const uint16_t *norm_weight; // [columns] or nullptr
  const uint16_t *norm_scale;  // [rows, columns]; nullptr = no prologue
  const uint16_t *norm_shift;  // [rows, columns]
  float norm_eps;
  const uint16_t *norm_bias;   // [columns]: LayerNormModulate (mean removed, weight and bias); nullptr = RMS
  uint64_t norm_rows_per_mod;  // rows that share one row of scale / shift
  const float2 *norm_stats;    // per row (mean, inverse deviation) in the reference's order, or nullptr
};

// Fixed Rademacher diagonal of the signed variants (reference cpu_executor.cpp:183-189).
__device__ __forceinline__ uint32_t sign_bit(uint32_t column) {
  uint32_t hash = column + 0x9e3779b9u;
  hash = (hash ^ (hash >> 16)) * 0x7feb352du;
  hash = (hash ^ (hash >> 15)) * 0x846ca68bu;
  hash ^= hash >> 16;
  return hash & 1u;
}

// One radix-4 butterfly on packed pairs, without the reference's exact factor 0.5.
__device__ __forceinline__ void bfly(uint64_t &x0, uint64_t &x1, uint64_t &x2, uint64_t &x3) {
  const uint64_t s = add2(x0, x1);
  const uint64_t t = sub2(x0, x1);
  const uint64_t y0 = sub2(add2(s, x2), x3);
  const uint64_t y1 = add2(sub2(s, x2), x3);
  const uint64_t y2 = add2(add2(t, x2), x3);
  // the reference forms (x1 - x0) + x2: x1 - x0 = -t exactly, and (-t) + x2 = x2 - t
  const uint64_t y3 = add2(sub2(x2, t), x3);
  x0 = y0;
  x1 = y1;
  x2 = y2;
  x3 = y3;
}

__device__ __forceinline__ float absmax2(float m, uint64_t v) {
  float lo, hi;
  unpack2(v, lo, hi);
  asm("max.f32 %0, %0, %1, %2;" : "+f"(m) : "f"(fabsf(lo)), "f"(fabsf(hi))); // one three-input maximum
  return m;
}

// Correctly rounded fp32 quotient a/b from y = RN(1/b): two Markstein refinements.
__device__ __forceinline__ uint64_t div2_exact(uint64_t a, uint64_t y, uint64_t negb) {
  uint64_t q = mul2(a, y);
  uint64_t r = fma2(negb, q, a);
  q = fma2(r, y, q);
  r = fma2(negb, q, a);
  return fma2(r, y, q);
}
// bf16(a / b) for bf16 values a and b (8 significant bits each, integers V and S in [128, 255]
// times powers of two) needs no refinement at all: a rounding boundary of the quotient is M / 2^k
// with M odd in [257, 511], and |V / S - M / 2^k| = |2^k V - M S| / (S 2^k) is either 0 -- which
// would need the odd M > 255 to divide V <= 255, impossible -- or at least 2^-17 of the quotient,
// while a * RN(1 / b) is within 2^-23 of it. So the plain product rounds to the same bf16 value
// as the IEEE quotient, ties cannot occur, and a zero numerator gives zero.
__device__ __forceinline__ uint64_t div2_bf16(uint64_t a, uint64_t y) { return mul2(a, y); }

__device__ __forceinline__ uint64_t round_bf16_2(uint64_t v) {
  float lo, hi;
  unpack2(v, lo, hi);
  uint32_t packed;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
  return pack2(__uint_as_float(packed << 16), __uint_as_float(packed & 0xffff0000u));
}

__device__ __forceinline__ int sat_s8(float v) {
  int r;
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
  return r;
}

template <bool F32>
__device__ __forceinline__ void quantize_pair(uint64_t value, uint64_t y, uint64_t negb, int &c0,
                                              int &c1) {
  float q0, q1;
  if (F32) {
    unpack2(div2_exact(value, y, negb), q0, q1);
    c0 = max(sat_s8(q0), -127);
    c1 = max(sat_s8(q1), -127);
  } else {
    unpack2(round_bf16_2(div2_bf16(round_bf16_2(value), y)), q0, q1);
    c0 = sat_s8(q0);
    c1 = sat_s8(q1);
  }
}

// ---- shared-memory access through 32-bit shared addresses (cheap address arithmetic) ----
__device__ __forceinline__ void sts128(uint32_t addr, float x, float y, float z, float w) {
  asm volatile("st.shared.v4.f32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "f"(x), "f"(y), "f"(z), "f"(w)
               : "memory");
}
template <int OFF>
__device__ __forceinline__ uint64_t lds64(uint32_t addr) {
  uint64_t v;
  asm volatile("ld.shared.b64 %0, [%1+%2];" : "=l"(v) : "r"(addr), "n"(OFF) : "memory");
  return v;
}
template <int OFF>
__device__ __forceinline__ void sts8(uint32_t addr, int v) {
  asm volatile("st.shared.u8 [%0+%1], %2;" ::"r"(addr), "n"(OFF), "r"(v) : "memory");
}
__device__ __forceinline__ void sts32(uint32_t addr, float v) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ float lds32(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

// Shared memory per warp: 4 groups x 256 fp32 (two swizzled 16x32-word transposes), reused
// for the code bytes; plus words for the row maxima after all warps' areas.
constexpr int kWarpBytes = 4096;

// Code bytes of one row are staged at index(col) = col + 64 * (col >> 9): one byte per column
// with a 64-byte skew per 512 columns, so that the two half-warps hit different banks.
template <bool H4096, int J>
__device__ __forceinline__ void stage_pair(uint32_t base_a, uint32_t base_b, int ca, int cb) {
  // 256-wide variants: element J of the thread sits 16*J bytes after its base.
  // 4096-wide variants: group J of the block sits 256*J columns on, i.e. 256*J + 64*(J>>1).
  constexpr int off = H4096 ? (256 * J + 64 * (J >> 1)) : 16 * J;
  sts8<off>(base_a, ca);
  sts8<off>(base_b, cb);
}

// MAXT bounds the block size so that the register budget (about 80 per thread, which the
// prefetch needs) is known at compile time: 256 -> 3 blocks/SM, 384 -> 2, 512 -> 1.
// MSE (weight rows only): the scale is the one of seven clipped candidates with the lowest squared
// error over every fourth rotated element, the offline packer's rule (reference
// tools/difflux2sample.cpp:1225-1259; row encoder :2994-3059).
template <bool SIGNED, bool F32, bool H4096, bool RESIDUAL, bool MSE, int MAXT>
__global__ void __launch_bounds__(MAXT, MAXT == 256 ? 3 : (MAXT == 384 ? 2 : 1))
convrot_quant_kernel(const QuantParams p, const int warps_per_row, const int rows_per_cta) {
  extern __shared__ __align__(128) uint32_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = warp / warps_per_row;         // which row of this CTA's batch
  const int wrow = warp - slot * warps_per_row;  // warp index inside the row
  const int h = lane >> 4, a = lane & 15;
  const uint32_t groups = p.columns >> 8;
  const uint32_t group_a = 4u * wrow + 2u * h;   // first group of this thread's pair
  const bool act_a = group_a < groups, act_b = group_a + 1u < groups;
  const int total_warps = blockDim.x >> 5;
  const uint32_t smem_addr = smem_u32(smem);
  const uint32_t warp_addr = smem_addr + warp * kWarpBytes;
  float *red = reinterpret_cast<float *>(smem + total_warps * (kWarpBytes / 4));
  const float clip = p.clip_device ? __ldg(p.clip_device) : p.clip;
  // The values carried through the rotation are scaled by 2^stages.
  constexpr float kCarry = H4096 ? 64.0f : 16.0f;

  // Where this thread's two 16-element runs live in global memory (the logical row is the
  // concatenation of the parts; widths are multiples of 16, so a run never straddles two).
  const uint16_t *src_a = nullptr, *src_b = nullptr;
  uint32_t pitch_a = 0, pitch_b = 0;
  {
    uint32_t ca = group_a * 256u + 16u * a, cb = ca + 256u;
    bool fa = !act_a, fb = !act_b;
    for (uint32_t i = 0; i < p.part_count; ++i) {
      const uint32_t w = p.width[i];
      if (!fa) {
        if (ca < w) { src_a = p.part[i] + ca; pitch_a = w; fa = true; } else ca -= w;
      }
      if (!fb) {
        if (cb < w) { src_b = p.part[i] + cb; pitch_b = w; fb = true; } else cb -= w;
      }
    }
  }

  // Transpose addressing (per half-warp area of 2048 bytes; rows of 128 bytes = 16 pairs):
  // thread a writes its 8 chunks of 2 pairs at chunk position c ^ (a & 7), and reads pair a of
  // every row j from chunk position (a >> 1) ^ (j & 7).
  const uint32_t half_addr = warp_addr + h * 2048u;
  const uint32_t wr_addr = half_addr + 128u * a + ((a & 7u) << 4);          // ^ (c << 4)
  const uint32_t rd_addr = half_addr + ((uint32_t)(a >> 1) << 4) + 8u * (a & 1u); // ^ ((j&7)<<4), + 128 j

  // Code staging addresses.
  uint32_t code_a, code_b;      // byte address of this thread's element/group 0 (A and B lane)
  uint32_t rowbuf_a = 0, rowbuf_b = 0;
  if (H4096) {
    const uint32_t per = p.columns >> 5;
    const uint32_t u0 = threadIdx.x, u1 = threadIdx.x + per;
    const uint32_t col0 = (u0 >> 8) * 4096u + (u0 & 255u), col1 = (u1 >> 8) * 4096u + (u1 & 255u);
    code_a = smem_addr + col0 + ((col0 >> 9) << 6);
    code_b = smem_addr + col1 + ((col1 >> 9) << 6);
    rowbuf_a = smem_addr + 4u * col0;
    rowbuf_b = smem_addr + 4u * col1;
  } else {
    code_a = warp_addr + 512u * h + a + 64u * h;
    code_b = code_a + 256u;
  }
  const uint32_t copy_addr = (H4096 ? smem_addr + (uint32_t)wrow * 1152u : warp_addr) + 16u * lane;
  const uint32_t copy_col = (uint32_t)wrow * 1024u + 16u * lane;

  // Sign flips of this thread's 32 columns as XOR masks on the packed bf16 pairs (bits 15 and
  // 31 of word i: elements 2i and 2i+1), kept in shared memory: words 0-7 group A, 8-15 group B,
  // stored as four 16-byte vectors per thread, vector q of all threads contiguous.
  const uint32_t mask_addr = smem_addr + (uint32_t)total_warps * (kWarpBytes + 16u) + 64u + threadIdx.x * 16u;
  const uint32_t mask_step = blockDim.x * 16u;
  if (SIGNED) {
    uint32_t mw[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      mw[i] = (sign_bit(group_a * 256u + 16u * a + 2 * i) << 15) |
              (sign_bit(group_a * 256u + 16u * a + 2 * i + 1) << 31);
      mw[8 + i] = (sign_bit((group_a + 1u) * 256u + 16u * a + 2 * i) << 15) |
                  (sign_bit((group_a + 1u) * 256u + 16u * a + 2 * i + 1) << 31);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q)
      asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(mask_addr + q * mask_step), "r"(mw[4 * q]),
                   "r"(mw[4 * q + 1]), "r"(mw[4 * q + 2]), "r"(mw[4 * q + 3])
                   : "memory");
  }

  // Software pipeline: the 64 bytes of the next row are requested before the current row is
  // processed, so the HBM latency of row i+1 hides under the arithmetic of row i.
  auto fetch = [&](uint64_t row, uint4 &a0, uint4 &a1, uint4 &b0, uint4 &b1) {
    a0 = a1 = b0 = b1 = make_uint4(0, 0, 0, 0);
    if (row < p.rows) {
      if (act_a) {
        const uint4 *v = reinterpret_cast<const uint4 *>(src_a + row * pitch_a);
        a0 = __ldg(v);
        a1 = __ldg(v + 1);
      }
      if (act_b) {
        const uint4 *v = reinterpret_cast<const uint4 *>(src_b + row * pitch_b);
        b0 = __ldg(v);
        b1 = __ldg(v + 1);
      }
    }
  };
  uint4 na0, na1, nb0, nb1;
  fetch((uint64_t)blockIdx.x * rows_per_cta + slot, na0, na1, nb0, nb1);

  // Only the warps of one row exchange maxima: a named barrier per row slot, so that the rows a
  // CTA works on at the same time do not wait for each other (the 4096-wide variants have one
  // row per CTA and CTA-wide transposes anyway).
  auto row_barrier = [&]() {
    if (H4096)
      __syncthreads();
    else
      asm volatile("bar.sync %0, %1;" ::"r"(slot + 1), "r"(warps_per_row * 32) : "memory");
  };
  uint32_t parity = 0;
  for (uint64_t row0 = (uint64_t)blockIdx.x * rows_per_cta; row0 < p.rows;
       row0 += (uint64_t)gridDim.x * rows_per_cta, parity ^= 1u) {
    const uint64_t row = row0 + slot;
    const bool row_ok = row < p.rows;
    uint64_t P[16];
    {
      const uint4 a0 = na0, a1 = na1, b0 = nb0, b1 = nb1;
      fetch(row + (uint64_t)gridDim.x * rows_per_cta, na0, na1, nb0, nb1);
      uint32_t wa[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      uint32_t wb[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
      if (MSE && p.norm_scale != nullptr) {
        // RmsNormModulate fused in front (reference cpu_executor.cpp:1241-1264 followed by the
        // quantiser; the reference's own fused precedent is cuda_executor.cpp:5417-5466): the
        // words are replaced by the bf16 result h the unfused op would have stored. The row's sum
        // of squares meets per warp and then per row in a fixed order.
        float xs[32];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          xs[2 * i] = __uint_as_float(wa[i] << 16);
          xs[2 * i + 1] = __uint_as_float(wa[i] & 0xffff0000u);
          xs[16 + 2 * i] = __uint_as_float(wb[i] << 16);
          xs[16 + 2 * i + 1] = __uint_as_float(wb[i] & 0xffff0000u);
        }
        const bool layer = p.norm_bias != nullptr;
        float *stat = red + parity * 2 * total_warps + total_warps;
        auto row_sum = [&](float v, float *slots) { // warp tree, then the row's warps in order
#pragma unroll
          for (int o = 16; o > 0; o >>= 1)
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
          if (lane == 0)
            slots[warp] = v;
          row_barrier();
          v = 0.0f;
          for (int w = 0; w < warps_per_row; ++w)
            v = __fadd_rn(v, slots[slot * warps_per_row + w]);
          return v;
        };
        float mean = 0.0f, ss = 0.0f, inv = 0.0f;
        if (p.norm_stats) {
          // the statistic in the reference's sequential order, from glue::row_stats_sequential
          const float2 st = __ldg(p.norm_stats + (row_ok ? row : 0));
          mean = st.x;
          inv = st.y;
        } else if (layer) {
          // LayerNormModulate (cpu_executor.cpp:1108-1148): mean, then the centred second moment.
          // The second sum uses the other parity's slots: they are free until the next row, which
          // every warp of this row reaches only after the barriers of the maxima exchange below.
#pragma unroll
          for (int i = 0; i < 32; ++i)
            mean = __fadd_rn(mean, xs[i]);
          mean = __fdiv_rn(row_sum(mean, stat), (float)p.columns);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float d = __fsub_rn(xs[i], mean);
            if (i < 16 ? act_a : act_b)
              ss = __fmaf_rn(d, d, ss);
          }
          ss = row_sum(ss, red + (parity ^ 1u) * 2 * total_warps + total_warps);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            ss = __fmaf_rn(xs[i], xs[i], ss);
          ss = row_sum(ss, stat);
        }
        if (!p.norm_stats)
          inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(ss, (float)p.columns), p.norm_eps)));
        const uint32_t col = group_a * 256u + 16u * a;
        const uint64_t at = ((row_ok ? row : 0) / p.norm_rows_per_mod) * (uint64_t)p.columns + col;
        const uint4 one = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u), zero = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int g = 0; g < 2; ++g) {
          const bool act = g == 0 ? act_a : act_b;
          const uint4 *wp = reinterpret_cast<const uint4 *>(p.norm_weight + col + 256u * g);
          const uint4 *sp = reinterpret_cast<const uint4 *>(p.norm_scale + at + 256u * g);
          const uint4 *hp = reinterpret_cast<const uint4 *>(p.norm_shift + at + 256u * g);
          const uint4 *bp = reinterpret_cast<const uint4 *>(p.norm_bias + col + 256u * g);
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            const uint4 bq = (act && layer) ? __ldg(bp + half) : zero;
            const uint32_t bw[4] = {bq.x, bq.y, bq.z, bq.w};
            const uint4 wq = (act && p.norm_weight) ? __ldg(wp + half) : one;
            const uint4 sq = act ? __ldg(sp + half) : zero, hq = act ? __ldg(hp + half) : zero;
            const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w}, sw[4] = {sq.x, sq.y, sq.z, sq.w},
                           hw[4] = {hq.x, hq.y, hq.z, hq.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int e = 16 * g + 8 * half + 2 * i;
              float y[2];
#pragma unroll
              for (int k = 0; k < 2; ++k) {
                const float wv = __uint_as_float(k ? (ww[i] & 0xffff0000u) : (ww[i] << 16));
                const float sv = __uint_as_float(k ? (sw[i] & 0xffff0000u) : (sw[i] << 16));
                const float hv = __uint_as_float(k ? (hw[i] & 0xffff0000u) : (hw[i] << 16));
                if (layer) { // intermediate bf16 roundings of the reference's LayerNormModulate
                  const float bv = __uint_as_float(k ? (bw[i] & 0xffff0000u) : (bw[i] << 16));
                  const float normalized = round_bf16(
                      __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(xs[e + k], mean), inv), wv), bv));
                  const float one_plus = round_bf16(__fadd_rn(1.0f, sv));
                  y[k] = __fadd_rn(round_bf16(__fmul_rn(normalized, one_plus)), hv);
                } else {
                  const float normalized = __fmul_rn(__fmul_rn(xs[e + k], inv), wv);
                  y[k] = __fadd_rn(__fmul_rn(normalized, __fadd_rn(1.0f, sv)), hv);
                }
              }
              uint32_t packed;
              asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(y[1]), "f"(y[0]));
              if (g == 0)
                wa[4 * half + i] = packed;
              else
                wb[4 * half + i] = packed;
            }
          }
        }
      }
      if (SIGNED) {
        const uint4 m0 = lds128(mask_addr), m1 = lds128(mask_addr + mask_step);
        const uint4 m2 = lds128(mask_addr + 2u * mask_step), m3 = lds128(mask_addr + 3u * mask_step);
        const uint32_t ma[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        const uint32_t mb[8] = {m2.x, m2.y, m2.z, m2.w, m3.x, m3.y, m3.z, m3.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          wa[i] ^= ma[i];
          wb[i] ^= mb[i];
        }
      }
      // weight rows with input equalisation: w / e in fp32 before anything else (reference
      // tools/difflux2sample.cpp:3005-3014; the sign flip commutes with the division)
      uint32_t ea[8], eb[8];
      const bool equalise = MSE && p.equalise != nullptr;
      if (equalise) {
        const uint32_t col = group_a * 256u + 16u * a;
        const uint4 z = make_uint4(0x3f803f80u, 0x3f803f80u, 0x3f803f80u, 0x3f803f80u); // bf16 ones
        const uint4 *ep = reinterpret_cast<const uint4 *>(p.equalise + col);
        const uint4 e0 = act_a ? __ldg(ep) : z, e1 = act_a ? __ldg(ep + 1) : z;
        const uint4 e2 = act_b ? __ldg(ep + 32) : z, e3 = act_b ? __ldg(ep + 33) : z;
        ea[0] = e0.x, ea[1] = e0.y, ea[2] = e0.z, ea[3] = e0.w, ea[4] = e1.x, ea[5] = e1.y, ea[6] = e1.z, ea[7] = e1.w;
        eb[0] = e2.x, eb[1] = e2.y, eb[2] = e2.z, eb[3] = e2.w, eb[4] = e3.x, eb[5] = e3.y, eb[6] = e3.z, eb[7] = e3.w;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint32_t alo = wa[i] << 16, ahi = wa[i] & 0xffff0000u;
        uint32_t blo = wb[i] << 16, bhi = wb[i] & 0xffff0000u;
        if (equalise) {
          alo = __float_as_uint(__fdiv_rn(__uint_as_float(alo), __uint_as_float(ea[i] << 16)));
          ahi = __float_as_uint(__fdiv_rn(__uint_as_float(ahi), __uint_as_float(ea[i] & 0xffff0000u)));
          blo = __float_as_uint(__fdiv_rn(__uint_as_float(blo), __uint_as_float(eb[i] << 16)));
          bhi = __float_as_uint(__fdiv_rn(__uint_as_float(bhi), __uint_as_float(eb[i] & 0xffff0000u)));
        }
        P[2 * i] = pack2(__uint_as_float(alo), __uint_as_float(blo));
        P[2 * i + 1] = pack2(__uint_as_float(ahi), __uint_as_float(bhi));
      }
    }
    // stage 0 (stride 1) and stage 1 (stride 4)
#pragma unroll
    for (int q = 0; q < 4; ++q)
      bfly(P[4 * q], P[4 * q + 1], P[4 * q + 2], P[4 * q + 3]);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      bfly(P[q], P[q + 4], P[q + 8], P[q + 12]);
    // 16x16 transpose of pairs through shared memory.
    {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float x0, x1, x2, x3;
        unpack2(P[2 * c], x0, x1);
        unpack2(P[2 * c + 1], x2, x3);
        sts128(wr_addr ^ (uint32_t)(c << 4), x0, x1, x2, x3);
      }
      __syncwarp();
      uint32_t rd[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        rd[j] = rd_addr ^ (uint32_t)(j << 4);
      P[0] = lds64<0 * 128>(rd[0]);
      P[1] = lds64<1 * 128>(rd[1]);
      P[2] = lds64<2 * 128>(rd[2]);
      P[3] = lds64<3 * 128>(rd[3]);
      P[4] = lds64<4 * 128>(rd[4]);
      P[5] = lds64<5 * 128>(rd[5]);
      P[6] = lds64<6 * 128>(rd[6]);
      P[7] = lds64<7 * 128>(rd[7]);
      P[8] = lds64<8 * 128>(rd[0]);
      P[9] = lds64<9 * 128>(rd[1]);
      P[10] = lds64<10 * 128>(rd[2]);
      P[11] = lds64<11 * 128>(rd[3]);
      P[12] = lds64<12 * 128>(rd[4]);
      P[13] = lds64<13 * 128>(rd[5]);
      P[14] = lds64<14 * 128>(rd[6]);
      P[15] = lds64<15 * 128>(rd[7]);
      __syncwarp();
    }
    // Now P[j] = element 16*j + a of both groups. stage 2 (stride 16), stage 3 (stride 64).
#pragma unroll
    for (int q = 0; q < 4; ++q)
      bfly(P[4 * q], P[4 * q + 1], P[4 * q + 2], P[4 * q + 3]);
#pragma unroll
    for (int q = 0; q < 4; ++q)
      bfly(P[q], P[q + 4], P[q + 8], P[q + 12]);

    if (H4096) {
      // Second transpose across the 16 groups of every 4096-wide block (one row per CTA):
      // write the row in natural order (this warp's own 1024 columns), read 16 groups of one
      // element position.
      const uint32_t nat_a = smem_addr + 4u * (group_a * 256u + a), nat_b = nat_a + 1024u;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float x0, x1;
        unpack2(P[j], x0, x1);
        sts32(nat_a + 64u * j, x0);
        sts32(nat_b + 64u * j, x1);
      }
      __syncthreads();
#pragma unroll
      for (int g = 0; g < 16; ++g)
        P[g] = pack2(lds32(rowbuf_a + 1024u * g), lds32(rowbuf_b + 1024u * g));
      __syncthreads();
#pragma unroll
      for (int q = 0; q < 4; ++q)
        bfly(P[4 * q], P[4 * q + 1], P[4 * q + 2], P[4 * q + 3]);
#pragma unroll
      for (int q = 0; q < 4; ++q)
        bfly(P[q], P[q + 4], P[q + 8], P[q + 12]);
    }

    // Row maximum: thread -> warp -> row.
    float m = 0.0f;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      m = absmax2(m, P[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float *redp = red + parity * 2 * total_warps;
    if (lane == 0)
      redp[warp] = m;
    row_barrier();
    m = 0.0f;
    for (int w = 0; w < warps_per_row; ++w)
      m = fmaxf(m, redp[slot * warps_per_row + w]);

    const float maximum = m * (1.0f / kCarry);
    float scale = fmaxf(__fdiv_rn(__fmul_rn(maximum, clip), 127.0f), 1.0e-30f);
    if (MSE && p.mse) {
      // Every thread evaluates the seven candidates on its sampled elements (column % 4 == 0, i.e.
      // a % 4 == 0 in this layout), in double like the reference; partial sums meet per warp and
      // then per row in a fixed order (the reference adds sequentially: its sum can differ in
      // the last bits of a double, which matters only for candidates that tie to 1e-15).
      const float factors[7] = {1.0f, 0.96f, 0.92f, 0.88f, 0.84f, 0.80f, 0.76f};
      double *errors = reinterpret_cast<double *>(
          reinterpret_cast<unsigned char *>(smem) + (size_t)total_warps * (kWarpBytes + 16) + 64 +
          (SIGNED ? (size_t)total_warps * 32 * 64 : 0));
      float candidate[7];
#pragma unroll 1
      for (int f = 0; f < 7; ++f) {
        candidate[f] = round_bf16(fmaxf(__fdiv_rn(__fmul_rn(maximum, factors[f]), 127.0f), 1.0e-30f));
        double e = 0.0;
        if ((a & 3) == 0) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float v[2];
            unpack2(P[j], v[0], v[1]);
#pragma unroll
            for (int g = 0; g < 2; ++g) {
              const float value = round_bf16(v[g] * (1.0f / kCarry));
              const float divided = round_bf16(__fdiv_rn(value, candidate[f]));
              const int encoded = min(max(__float2int_rn(divided), -128), 127);
              const double delta = __dsub_rn((double)value, __dmul_rn((double)encoded, (double)candidate[f]));
              e = __dadd_rn(e, __dmul_rn(delta, delta));
            }
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
          e = __dadd_rn(e, __shfl_xor_sync(0xffffffffu, e, o));
        if (lane == 0)
          errors[f * total_warps + warp] = e;
      }
      row_barrier();
      double best = 0.0;
#pragma unroll 1
      for (int f = 0; f < 7; ++f) {
        double e = 0.0;
        for (int w = 0; w < warps_per_row; ++w)
          e = __dadd_rn(e, errors[f * total_warps + slot * warps_per_row + w]);
        if (f == 0 || e < best) {
          best = e;
          scale = candidate[f];
        }
      }
      if (maximum == 0.0f)
        scale = 1.0e-30f;
      row_barrier(); // the error slots are reused by the next row
    }
    const float scale_bf16 = round_bf16(scale);
    const float stored = ((SIGNED || (MSE && p.mse)) && !F32) ? scale_bf16 : scale;
    const float divisor = (F32 ? scale : scale_bf16) * kCarry;
    const float recip = __frcp_rn(divisor);
    const uint64_t y2 = pack2(recip, recip), nb2 = pack2(-divisor, -divisor);
    if (row_ok && wrow == 0 && lane == 0)
      p.scales[row] = stored;

    auto flush_codes = [&](int8_t *dst) {
      if (H4096)
        __syncthreads();
      else
        __syncwarp();
      // every lane copies 2 x 16 bytes of its warp's 1024 columns
#pragma unroll
      for (int part = 0; part < 2; ++part) {
        const uint32_t col = copy_col + part * 512u;
        if (row_ok && col < p.columns)
          *reinterpret_cast<uint4 *>(dst + row * p.columns + col) = lds128(copy_addr + part * 576u);
      }
      if (H4096)
        __syncthreads();
      else
        __syncwarp();
    };

    int codes_a[RESIDUAL ? 16 : 1], codes_b[RESIDUAL ? 16 : 1];
#define DIFB200_QUANT_STEP(J)                                      \
  {                                                                \
    int ca, cb;                                                    \
    quantize_pair<F32>(P[J], y2, nb2, ca, cb);                     \
    stage_pair<H4096, J>(code_a, code_b, ca, cb);                  \
    if (RESIDUAL) {                                                \
      codes_a[RESIDUAL ? J : 0] = ca;                              \
      codes_b[RESIDUAL ? J : 0] = cb;                              \
    }                                                              \
  }
    DIFB200_QUANT_STEP(0) DIFB200_QUANT_STEP(1) DIFB200_QUANT_STEP(2) DIFB200_QUANT_STEP(3)
    DIFB200_QUANT_STEP(4) DIFB200_QUANT_STEP(5) DIFB200_QUANT_STEP(6) DIFB200_QUANT_STEP(7)
    DIFB200_QUANT_STEP(8) DIFB200_QUANT_STEP(9) DIFB200_QUANT_STEP(10) DIFB200_QUANT_STEP(11)
    DIFB200_QUANT_STEP(12) DIFB200_QUANT_STEP(13) DIFB200_QUANT_STEP(14) DIFB200_QUANT_STEP(15)
#undef DIFB200_QUANT_STEP
    flush_codes(p.codes);

    if (RESIDUAL) {
      // Residual pair (reference cpu_executor.cpp:262-305): r = fma(-code, stored, value).
      float rm = 0.0f;
      float ra[16], rb[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float x0, x1;
        unpack2(P[j], x0, x1);
        x0 *= (1.0f / kCarry);
        x1 *= (1.0f / kCarry);
        if (!F32) {
          x0 = round_bf16(x0);
          x1 = round_bf16(x1);
        }
        ra[j] = __fmaf_rn(-(float)codes_a[RESIDUAL ? j : 0], stored, x0);
        rb[j] = __fmaf_rn(-(float)codes_b[RESIDUAL ? j : 0], stored, x1);
        rm = fmaxf(rm, fmaxf(fabsf(ra[j]), fabsf(rb[j])));
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        rm = fmaxf(rm, __shfl_xor_sync(0xffffffffu, rm, o));
      if (lane == 0)
        redp[total_warps + warp] = rm;
      row_barrier();
      rm = 0.0f;
      for (int w = 0; w < warps_per_row; ++w)
        rm = fmaxf(rm, redp[total_warps + slot * warps_per_row + w]);
      const float rscale = fmaxf(__fdiv_rn(rm, 127.0f), 1.0e-30f);
      const float rscale_bf16 = round_bf16(rscale);
      if (row_ok && wrow == 0 && lane == 0)
        p.rscales[row] = (SIGNED && !F32) ? rscale_bf16 : rscale;
      int ca[16], cb[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        if (F32) {
          ca[j] = max(sat_s8(__fdiv_rn(ra[j], rscale)), -127);
          cb[j] = max(sat_s8(__fdiv_rn(rb[j], rscale)), -127);
        } else {
          ca[j] = sat_s8(round_bf16(__fdiv_rn(round_bf16(ra[j]), rscale_bf16)));
          cb[j] = sat_s8(round_bf16(__fdiv_rn(round_bf16(rb[j]), rscale_bf16)));
        }
      }
      stage_pair<H4096, 0>(code_a, code_b, ca[0], cb[0]);
      stage_pair<H4096, 1>(code_a, code_b, ca[1], cb[1]);
      stage_pair<H4096, 2>(code_a, code_b, ca[2], cb[2]);
      stage_pair<H4096, 3>(code_a, code_b, ca[3], cb[3]);
      stage_pair<H4096, 4>(code_a, code_b, ca[4], cb[4]);
      stage_pair<H4096, 5>(code_a, code_b, ca[5], cb[5]);
      stage_pair<H4096, 6>(code_a, code_b, ca[6], cb[6]);
      stage_pair<H4096, 7>(code_a, code_b, ca[7], cb[7]);
      stage_pair<H4096, 8>(code_a, code_b, ca[8], cb[8]);
      stage_pair<H4096, 9>(code_a, code_b, ca[9], cb[9]);
      stage_pair<H4096, 10>(code_a, code_b, ca[10], cb[10]);
      stage_pair<H4096, 11>(code_a, code_b, ca[11], cb[11]);
      stage_pair<H4096, 12>(code_a, code_b, ca[12], cb[12]);
      stage_pair<H4096, 13>(code_a, code_b, ca[13], cb[13]);
      stage_pair<H4096, 14>(code_a, code_b, ca[14], cb[14]);
      stage_pair<H4096, 15>(code_a, code_b, ca[15], cb[15]);
      flush_codes(p.rcodes);
    }
  }
}

// ---------------------------------------------------------------------------------------
// Direct variant (no rotation; reference cpu_executor.cpp:232-260): one warp per row, any
// width. Used for activations of plain W8A8 linears and for the per-token-per-head
// quantisation of attention Q/K (rows of width 128).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float load_logical(const QuantParams &p, uint64_t row, uint32_t column) {
  uint32_t c = column;
  for (uint32_t i = 0; i < p.part_count; ++i) {
    if (c < p.width[i])
      return bf16_bits_to_f32(__ldg(p.part[i] + row * p.width[i] + c));
    c -= p.width[i];
  }
  return 0.0f;
}

template <bool VEC8>
__global__ void __launch_bounds__(256)
direct_quant_kernel(const QuantParams p) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp_global = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const uint64_t warp_count = (uint64_t)gridDim.x * (blockDim.x >> 5);
  const float clip = p.clip_device ? __ldg(p.clip_device) : p.clip;
  const uint32_t K = p.columns;
  for (uint64_t row = warp_global; row < p.rows; row += warp_count) {
    float m = 0.0f;
    if (VEC8) { // single part, width % 8 == 0, 16-byte aligned rows
      const uint4 *src = reinterpret_cast<const uint4 *>(p.part[0] + row * K);
      for (uint32_t c = lane; c < (K >> 3); c += 32) {
        const uint4 v = __ldg(src + c);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          m = fmaxf(m, fabsf(__uint_as_float(w[i] << 16)));
          m = fmaxf(m, fabsf(__uint_as_float(w[i] & 0xffff0000u)));
        }
      }
    } else {
      for (uint32_t c = lane; c < K; c += 32)
        m = fmaxf(m, fabsf(load_logical(p, row, c)));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float scale = fmaxf(__fdiv_rn(__fmul_rn(m, clip), 127.0f), 1.0e-30f);
    if (lane == 0)
      p.scales[row] = scale;
    const bool residual = p.rcodes != nullptr;
    float rm = 0.0f;
    if (VEC8) {
      const uint4 *src = reinterpret_cast<const uint4 *>(p.part[0] + row * K);
      uint2 *dst = reinterpret_cast<uint2 *>(p.codes + row * K);
      for (uint32_t c = lane; c < (K >> 3); c += 32) {
        const uint4 v = __ldg(src + c);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t out[2] = {0, 0};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float x0 = __uint_as_float(w[i] << 16), x1 = __uint_as_float(w[i] & 0xffff0000u);
          const int c0 = max(sat_s8(__fdiv_rn(x0, scale)), -127);
          const int c1 = max(sat_s8(__fdiv_rn(x1, scale)), -127);
          out[i >> 1] |= ((uint32_t)(c0 & 0xff) << (16 * (i & 1))) |
                         ((uint32_t)(c1 & 0xff) << (16 * (i & 1) + 8));
          if (residual) {
            rm = fmaxf(rm, fabsf(__fmaf_rn(-(float)c0, scale, x0)));
            rm = fmaxf(rm, fabsf(__fmaf_rn(-(float)c1, scale, x1)));
          }
        }
        dst[c] = make_uint2(out[0], out[1]);
      }
    } else {
      for (uint32_t c = lane; c < K; c += 32) {
        const float x = load_logical(p, row, c);
        const int code = max(sat_s8(__fdiv_rn(x, scale)), -127);
        p.codes[row * K + c] = (int8_t)code;
        if (residual)
          rm = fmaxf(rm, fabsf(__fmaf_rn(-(float)code, scale, x)));
      }
    }
    if (residual) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        rm = fmaxf(rm, __shfl_xor_sync(0xffffffffu, rm, o));
      const float rscale = fmaxf(__fdiv_rn(rm, 127.0f), 1.0e-30f);
      if (lane == 0)
        p.rscales[row] = rscale;
      __syncwarp();
      for (uint32_t c = lane; c < K; c += 32) {
        const float x = load_logical(p, row, c);
        const float r = __fmaf_rn(-(float)p.codes[row * K + c], scale, x);
        p.rcodes[row * K + c] = (int8_t)max(sat_s8(__fdiv_rn(r, rscale)), -127);
      }
    }
  }
}

template <bool SIGNED, bool F32, bool H4096, bool RESIDUAL, bool MSE = false>
int launch_convrot_impl(const QuantParams &p, cudaStream_t stream) {
  const uint32_t groups = p.columns >> 8;
  const int warps_per_row = (int)((groups + 3u) / 4u);
  if (warps_per_row > 16)
    return fail(kUnsupported, "QuantizeInt8Rows: ConvRot width above 16384 is not supported");
  int rows_per_cta = H4096 ? 1 : (8 / warps_per_row);
  if (rows_per_cta < 1)
    rows_per_cta = 1;
  if ((uint64_t)rows_per_cta > p.rows)
    rows_per_cta = (int)p.rows;
  const int warps = warps_per_row * rows_per_cta;
  // per warp: transpose / staging area; row maxima; for the signed variants 16 XOR masks per thread
  const size_t smem = (size_t)warps * kWarpBytes + (size_t)warps * 4 * sizeof(float) + 64 +
                      (SIGNED ? (size_t)warps * 32 * 64 : 0) + (MSE ? (size_t)warps * 7 * sizeof(double) : 0);
  const int threads_needed = warps * 32;
  auto kernel = threads_needed <= 256   ? convrot_quant_kernel<SIGNED, F32, H4096, RESIDUAL, MSE, 256>
                : threads_needed <= 384 ? convrot_quant_kernel<SIGNED, F32, H4096, RESIDUAL, MSE, 384>
                                        : convrot_quant_kernel<SIGNED, F32, H4096, RESIDUAL, MSE, 512>;
  if (smem > 48 * 1024) {
    if (int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem),
                            "cudaFuncSetAttribute(convrot)"))
      return rc;
  }
  const uint64_t batches = (p.rows + rows_per_cta - 1) / rows_per_cta;
  const int threads = warps * 32;
  int resident = 1;
  if (int rc = check_cuda(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, threads, smem),
                          "occupancy(convrot)"))
    return rc;
  if (resident < 1)
    resident = 1;
  uint64_t grid = (uint64_t)sm_count() * resident;
  if (grid > batches)
    grid = batches;
  kernel<<<(unsigned)grid, threads, smem, stream>>>(p, warps_per_row, rows_per_cta);
  return launched(cudaGetLastError(), "convrot_quant_kernel launch");
}

template <bool SIGNED, bool F32, bool H4096>
int launch_convrot(const QuantParams &p, cudaStream_t stream) {
  if (p.mse || p.equalise || p.norm_scale) { // the form of the kernel with the rarely used extras
    if (H4096 || p.rcodes)
      return fail(kUnsupported, "QuantizeInt8Rows: weight packing (MSE scale, input equalisation) exists for "
                                "the 256-wide variants without residual outputs");
    return launch_convrot_impl<SIGNED, F32, false, false, true>(p, stream);
  }
  return p.rcodes ? launch_convrot_impl<SIGNED, F32, H4096, true>(p, stream)
                  : launch_convrot_impl<SIGNED, F32, H4096, false>(p, stream);
}

} // namespace

int quantize_int8_rows(const void *const *parts, const uint64_t *part_widths, uint32_t part_count,
                       uint64_t rows, int implementation, float clip, const float *clip_device,
                       int8_t *codes, float *scales, int8_t *rcodes, float *rscales,
                       cudaStream_t stream, bool mse_weight_scale, const void *equalise_bf16,
                       const NormPrologue *norm) {
  if (part_count == 0 || part_count > kMaxParts)
    return fail(kUnsupported, "QuantizeInt8Rows: 1..8 concatenated inputs are supported");
  if (!codes || !scales || (rcodes == nullptr) != (rscales == nullptr))
    return fail(kInvalidArgument, "QuantizeInt8Rows: missing output pointer");
  if (!(clip > 0.0f) && !clip_device)
    return fail(kInvalidArgument, "QuantizeInt8Rows: clip ratio must be positive");
  QuantParams p{};
  uint64_t columns = 0;
  bool aligned16 = true, aligned8 = true;
  for (uint32_t i = 0; i < part_count; ++i) {
    if (!parts[i] || part_widths[i] == 0 || part_widths[i] > 0xffffffffull)
      return fail(kInvalidArgument, "QuantizeInt8Rows: bad input part");
    p.part[i] = static_cast<const uint16_t *>(parts[i]);
    p.width[i] = (uint32_t)part_widths[i];
    columns += part_widths[i];
    aligned16 = aligned16 && part_widths[i] % 16 == 0 && (reinterpret_cast<uintptr_t>(parts[i]) & 15) == 0;
    aligned8 = aligned8 && part_widths[i] % 8 == 0 && (reinterpret_cast<uintptr_t>(parts[i]) & 15) == 0;
  }
  if (columns > 0xffffffffull)
    return fail(kUnsupported, "QuantizeInt8Rows: row too wide");
  p.part_count = part_count;
  p.columns = (uint32_t)columns;
  p.rows = rows;
  p.clip = clip;
  p.clip_device = clip_device;
  p.codes = codes;
  p.scales = scales;
  p.rcodes = rcodes;
  p.rscales = rscales;
  p.mse = mse_weight_scale ? 1u : 0u;
  p.equalise = static_cast<const uint16_t *>(equalise_bf16);
  if (norm) {
    if (!norm->scale || !norm->shift)
      return fail(kInvalidArgument, "QuantizeInt8Rows: norm prologue without scale / shift");
    if (implementation < 2 || implementation == 4 || implementation == 7 || part_count != 1 || rcodes ||
        ((reinterpret_cast<uintptr_t>(norm->scale) | reinterpret_cast<uintptr_t>(norm->shift) |
          reinterpret_cast<uintptr_t>(norm->weight) | reinterpret_cast<uintptr_t>(norm->bias)) & 15) ||
        norm->rows_per_modulation == 0 || (norm->bias && !norm->weight))
      return fail(kUnsupported, "QuantizeInt8Rows: the norm prologue needs one input, a 256-wide ConvRot variant, no "
                                "residual outputs and 16-byte aligned pointers");
    p.norm_weight = static_cast<const uint16_t *>(norm->weight);
    p.norm_scale = static_cast<const uint16_t *>(norm->scale);
    p.norm_shift = static_cast<const uint16_t *>(norm->shift);
    p.norm_eps = norm->epsilon;
    p.norm_bias = static_cast<const uint16_t *>(norm->bias);
    p.norm_rows_per_mod = norm->rows_per_modulation;
    if (rows > 0) { // the row statistic in the reference's order, by its own kernel in front
      int rc = 0;
      if (glue::row_stats_sequential(parts[0], rows, columns, norm->epsilon, norm->bias != nullptr, &p.norm_stats,
                                     stream, &rc) && rc)
        return rc;
    }
  }
  if (rows == 0)
    return kOk;
  if ((mse_weight_scale || equalise_bf16) && (implementation == 1 || clip_device || part_count != 1))
    return fail(kUnsupported, "QuantizeInt8Rows: weight packing applies to one input, the ConvRot variants and a "
                              "static clip");
  if (equalise_bf16 && (reinterpret_cast<uintptr_t>(equalise_bf16) & 15))
    return fail(kUnsupported, "QuantizeInt8Rows: the equalisation vector must be 16-byte aligned");
  if (implementation == 1) {
    const int threads = 256;
    uint64_t blocks = (rows + 7) / 8;
    const uint64_t cap = (uint64_t)sm_count() * 16;
    if (blocks > cap)
      blocks = cap;
    if (part_count == 1 && columns == 128 && !rcodes && !clip_device) { // per token-head rows: a thread per row
      int rc = 0;
      if (glue::direct_quant_rows128(parts[0], codes, scales, rows, clip, stream, &rc))
        return rc;
    }
    const bool vec = part_count == 1 && aligned8 && (reinterpret_cast<uintptr_t>(codes) & 7) == 0;
    if (vec)
      direct_quant_kernel<true><<<(unsigned)blocks, threads, 0, stream>>>(p);
    else
      direct_quant_kernel<false><<<(unsigned)blocks, threads, 0, stream>>>(p);
    return launched(cudaGetLastError(), "direct_quant_kernel launch");
  }
  if (implementation < 2 || implementation > 7)
    return fail(kInvalidArgument, "QuantizeInt8Rows: unknown implementation");
  const bool h4096 = implementation == 4 || implementation == 7;
  if (columns % (h4096 ? 4096u : 256u) != 0)
    return fail(kInvalidArgument, "QuantizeInt8Rows: width is not a multiple of the rotation group");
  if (!aligned16 || (reinterpret_cast<uintptr_t>(codes) & 15) != 0 ||
      (rcodes && (reinterpret_cast<uintptr_t>(rcodes) & 15) != 0))
    return fail(kUnsupported,
                "QuantizeInt8Rows: ConvRot path needs 16-byte aligned pointers and part widths "
                "that are multiples of 16");
  switch (implementation) {
  case 2: return launch_convrot<false, false, false>(p, stream);
  case 3: return launch_convrot<true, false, false>(p, stream);
  case 4: return launch_convrot<true, false, true>(p, stream);
  case 5: return launch_convrot<false, true, false>(p, stream);
  case 6: return launch_convrot<true, true, false>(p, stream);
  default: return launch_convrot<true, true, true>(p, stream);
  }
}

} // namespace difb200
