// bf16 fast paths of the block-glue kernels that carry most of a DiT block's non-GEMM,
// non-attention time: every access is 16 bytes (8 bf16), rows stay in registers between the
// statistic and the normalisation, and the per-(token, head) operators give one thread a whole
// 128-wide row. Arithmetic and rounding points are those of the generic kernels in glue.cu (and
// therefore of the reference CPU executor; file:line per kernel, paths in the reference project).
// glue.cu selects these when dtype, widths and alignment allow and falls back otherwise.
#include "glue.h"

#include "common.cuh"

#include <cstdlib>

namespace difb200 {
namespace glue {
namespace {

__device__ __forceinline__ void unpack8(const uint4 v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t packed;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
  return packed;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                    pack_bf16x2(f[6], f[7]));
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

// ---- ResidualGate (cpu_executor.cpp:1703-1719): out = res + gate * branch ----
__global__ void __launch_bounds__(256)
k_residual_gate_bf16(const uint4 *res, const uint4 *branch, const uint4 *gate, uint4 *o, uint64_t groups,
                     uint64_t width8, uint64_t rows_per_gate) {
  GRID_STRIDE(i, groups) {
    const uint64_t row = i / width8, col = i - row * width8;
    float r[8], b[8], g[8], y[8];
    unpack8(__ldg(res + i), r);
    unpack8(__ldg(branch + i), b);
    unpack8(__ldg(gate + (row / rows_per_gate) * width8 + col), g);
#pragma unroll
    for (int e = 0; e < 8; ++e)
      y[e] = __fadd_rn(r[e], __fmul_rn(g[e], b[e]));
    o[i] = pack8(y);
  }
}

// ---- SwiGlu (cpu_executor.cpp:1267-1286): out = value * (gate / (1 + exp(-gate))) ----
__global__ void __launch_bounds__(256)
k_swiglu_bf16(const uint4 *x, uint4 *o, uint64_t rows, uint64_t width8, uint64_t in_width8, uint64_t start8,
              int gate_first) {
  GRID_STRIDE(i, rows * width8) {
    const uint64_t row = i / width8, col = i - row * width8, base = row * in_width8 + start8 + col;
    float value[8], gate[8], y[8];
    unpack8(__ldg(x + base + (gate_first ? width8 : 0)), value);
    unpack8(__ldg(x + base + (gate_first ? 0 : width8)), gate);
#pragma unroll
    for (int e = 0; e < 8; ++e)
      y[e] = __fmul_rn(value[e], __fdiv_rn(gate[e], __fadd_rn(1.0f, expf(-gate[e]))));
    o[i] = pack8(y);
  }
}


// ---- row statistics in the reference's sequential order ----
// The reference sums a row's squares (or values, then squared deviations) in one fp32 chain, column
// by column (cpu_executor.cpp:1051-1062 RmsNorm, 1119-1129 LayerNormModulate, 1250-1256
// RmsNormModulate). A parallel sum differs from that chain in the last bit of about one row in
// three, which flips one bf16 output in a few thousand -- and every ConvRot quantiser behind the
// norm amplifies such a flip across its 256-wide group. So the statistic is computed here in the
// reference's order: one lane per row walks its row sequentially. A warp owns 32 rows and moves them
// through shared memory 64 columns at a time (asynchronous 16-byte copies in coalesced 128-byte
// runs, rows 9 x 16 bytes apart so that lanes read their own rows without bank conflicts), four
// chunks deep: the memory latency of a chunk hides under the chains of the three before it.
// Squares of bf16 values are exact in fp32, so the
// fused multiply-add equals the reference's multiply followed by add; the deviations of the layer
// form are not, and get the two roundings.
constexpr int kStatCols = 64, kStatPitch = 9; // uint4 per row in shared memory (8 + 1 pad)
constexpr int kStatStages = 4, kStatWarps = 2;  // chunks in flight per warp (hides the HBM latency), warps per CTA

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, bool valid) {
  // 16 bytes global -> shared, asynchronously; zero-filled when the row does not exist
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(valid ? 16 : 0) : "memory");
}

template <bool LAYER>
__global__ void __launch_bounds__(32 * kStatWarps)
k_row_stats_sequential(const uint4 *x, float2 *stats, uint64_t rows, uint32_t cols, float eps) {
  __shared__ uint4 tile[kStatWarps][kStatStages][32 * kStatPitch];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t cols8 = cols >> 3, chunks = cols / kStatCols;
  for (uint64_t row0 = ((uint64_t)blockIdx.x * kStatWarps + warp) * 32; row0 < rows;
       row0 += (uint64_t)gridDim.x * kStatWarps * 32) {
    const uint64_t row = row0 + lane;
    // lane l copies, for j = 0..7, the 16 bytes (row0 + 4 j + l / 8, chunk column l % 8) of a chunk
    auto issue = [&](uint32_t chunk) {
      if (chunk < chunks) {
        uint4 *stage = tile[warp][chunk % kStatStages];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint64_t r = row0 + 4 * j + (lane >> 3);
          const bool valid = r < rows;
          cp_async16(smem_u32(stage + (4 * j + (lane >> 3)) * kStatPitch + (lane & 7)),
                     x + (valid ? r : 0) * cols8 + chunk * (kStatCols / 8) + (lane & 7), valid);
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory"); // one group per chunk slot, also when empty
    };
    float mean = 0.0f, acc = 0.0f;
#pragma unroll 1
    for (int pass = LAYER ? 0 : 1; pass < 2; ++pass) {
      acc = 0.0f;
      __syncwarp();
      for (uint32_t c = 0; c < (uint32_t)kStatStages - 1; ++c)
        issue(c);
#pragma unroll 1
      for (uint32_t chunk = 0; chunk < chunks; ++chunk) {
        issue(chunk + kStatStages - 1);              // its stage was read during chunk - 1
        asm volatile("cp.async.wait_group %0;" ::"n"(kStatStages - 1) : "memory");
        __syncwarp();                                // every lane's copies of this chunk have landed
        const uint4 *stage = tile[warp][chunk % kStatStages];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float f[8];
          unpack8(stage[lane * kStatPitch + c], f);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            if (pass == 0) {
              acc = __fadd_rn(acc, f[e]);
            } else if (LAYER) {
              const float d = __fsub_rn(f[e], mean);
              acc = __fadd_rn(acc, __fmul_rn(d, d));
            } else {
              acc = __fmaf_rn(f[e], f[e], acc);
            }
          }
        }
        __syncwarp();                                // before a later copy overwrites this stage
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      if (pass == 0)
        mean = __fdiv_rn(acc, (float)cols);
    }
    if (row < rows)
      stats[row] = make_float2(mean, __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(acc, (float)cols), eps))));
  }
}

// ---- RmsNormModulate, explicit scale / shift (cpu_executor.cpp:1241-1264) ----
// One warp per row; lane l owns the 8-element groups l, l + 32, ... CHUNKS > 0: the row has
// CHUNKS * 256 columns and stays in registers; CHUNKS == 0: any multiple of 256, read twice.
template <int CHUNKS>
__global__ void __launch_bounds__(256)
k_rms_norm_modulate_bf16(const uint4 *x, const uint4 *w, const uint4 *a, const uint4 *b, uint4 *o, uint64_t rows,
                         uint32_t cols, float eps, const float2 *stats) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const uint64_t nwarps = (uint64_t)gridDim.x * (blockDim.x >> 5);
  const uint32_t cols8 = cols >> 3, chunks = CHUNKS > 0 ? (uint32_t)CHUNKS : cols >> 8;
  for (uint64_t r = warp; r < rows; r += nwarps) {
    const uint4 *xr = x + r * cols8;
    uint4 kept[CHUNKS > 0 ? CHUNKS : 1];
    float sum = 0.0f;
#pragma unroll
    for (uint32_t k = 0; k < chunks; ++k) {
      const uint4 v = __ldg(xr + lane + 32u * k);
      if (CHUNKS > 0)
        kept[CHUNKS > 0 ? k : 0] = v;
      float f[8];
      unpack8(v, f);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        sum = __fmaf_rn(f[e], f[e], sum);
    }
    sum = warp_sum(sum);
    // `stats`: the statistic in the reference's sequential order (row_stats_sequential), which
    // makes every output bit the reference's; else the warp's parallel sum (last bit may differ)
    const float inv = stats ? stats[r].y : __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(sum, (float)cols), eps)));
#pragma unroll
    for (uint32_t k = 0; k < chunks; ++k) {
      const uint32_t c = lane + 32u * k;
      float f[8], wv[8], av[8], bv[8], y[8];
      unpack8(CHUNKS > 0 ? kept[CHUNKS > 0 ? k : 0] : __ldg(xr + c), f);
      unpack8(__ldg(a + r * cols8 + c), av);
      unpack8(__ldg(b + r * cols8 + c), bv);
      if (w)
        unpack8(__ldg(w + c), wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float normalized = __fmul_rn(__fmul_rn(f[e], inv), w ? wv[e] : 1.0f);
        y[e] = __fadd_rn(__fmul_rn(normalized, __fadd_rn(1.0f, av[e])), bv[e]);
      }
      o[r * cols8 + c] = pack8(y);
    }
  }
}

// ---- LayerNormModulate (cpu_executor.cpp:1108-1148): rounds to bf16 after the affine norm,
// after 1 + scale and after their product; scale / shift rows broadcast over rows_per_mod rows ----
template <int CHUNKS>
__global__ void __launch_bounds__(256)
k_layer_norm_modulate_bf16(const uint4 *x, const uint4 *w, const uint4 *b, const uint4 *scale, const uint4 *shift,
                           uint4 *o, uint64_t rows, uint32_t cols, uint64_t rows_per_mod, float eps,
                           const float2 *stats) {
  const int lane = threadIdx.x & 31;
  const uint64_t warp = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const uint64_t nwarps = (uint64_t)gridDim.x * (blockDim.x >> 5);
  const uint32_t cols8 = cols >> 3, chunks = CHUNKS > 0 ? (uint32_t)CHUNKS : cols >> 8;
  for (uint64_t r = warp; r < rows; r += nwarps) {
    const uint4 *xr = x + r * cols8;
    uint4 kept[CHUNKS > 0 ? CHUNKS : 1];
    float mean = 0.0f;
#pragma unroll
    for (uint32_t k = 0; k < chunks; ++k) {
      const uint4 v = __ldg(xr + lane + 32u * k);
      if (CHUNKS > 0)
        kept[CHUNKS > 0 ? k : 0] = v;
      float f[8];
      unpack8(v, f);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        mean += f[e];
    }
    mean = stats ? stats[r].x : __fdiv_rn(warp_sum(mean), (float)cols);
    float var = 0.0f;
#pragma unroll
    for (uint32_t k = 0; k < chunks; ++k) {
      float f[8];
      unpack8(CHUNKS > 0 ? kept[CHUNKS > 0 ? k : 0] : __ldg(xr + lane + 32u * k), f);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float d = __fsub_rn(f[e], mean);
        var = __fmaf_rn(d, d, var);
      }
    }
    var = warp_sum(var);
    const float inv = stats ? stats[r].y : __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(var, (float)cols), eps)));
    const uint64_t mrow = (r / rows_per_mod) * cols8;
#pragma unroll
    for (uint32_t k = 0; k < chunks; ++k) {
      const uint32_t c = lane + 32u * k;
      float f[8], wv[8], bv[8], sc[8], sh[8], y[8];
      unpack8(CHUNKS > 0 ? kept[CHUNKS > 0 ? k : 0] : __ldg(xr + c), f);
      unpack8(__ldg(w + c), wv);
      unpack8(__ldg(b + c), bv);
      unpack8(__ldg(scale + mrow + c), sc);
      unpack8(__ldg(shift + mrow + c), sh);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float normalized =
            round_bf16(__fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(f[e], mean), inv), wv[e]), bv[e]));
        const float one_plus = round_bf16(__fadd_rn(1.0f, sc[e]));
        y[e] = __fadd_rn(round_bf16(__fmul_rn(normalized, one_plus)), sh[e]);
      }
      o[r * cols8 + c] = pack8(y);
    }
  }
}

// ---- QkNormPartialRope on 128-wide heads (cpu_executor.cpp:1741-1837), optionally followed by
// QuantizeInt8Rows(Direct) of the result (cpu_executor.cpp:124-307, Direct branch) ----
// One thread per (token, head) row: the sum of squares runs in the reference's sequential order
// (multiply, then add), so the statistic has the reference's bits; rotation partners are in the
// same thread. ROTARY and the layout are compile-time so that the row stays in registers.
struct RowRopeParams {
  const uint4 *x;
  const uint4 *w;       // [128] bf16
  const void *cosv, *sinv;
  uint4 *o;             // bf16 output or nullptr
  int8_t *codes;        // Direct codes or nullptr
  float *scales;
  uint64_t rows, heads, input_seq, table_seq, table_start;
  uint64_t in_token_stride16, in_offset16; // where a token's heads start in x, in 16-byte units
  uint64_t out_seq, out_start;            // output token = (token / input_seq) * out_seq + out_start + token % input_seq
  uint32_t table_width, table_f32;
  float eps;
};

__device__ __forceinline__ void load_table8(const void *table, uint32_t f32, uint64_t index, float (&v)[8]) {
  if (f32) {
    const float4 *p = reinterpret_cast<const float4 *>(static_cast<const float *>(table) + index);
    const float4 lo = __ldg(p), hi = __ldg(p + 1);
    v[0] = lo.x, v[1] = lo.y, v[2] = lo.z, v[3] = lo.w, v[4] = hi.x, v[5] = hi.y, v[6] = hi.z, v[7] = hi.w;
  } else {
    unpack8(__ldg(reinterpret_cast<const uint4 *>(static_cast<const uint16_t *>(table) + index)), v);
  }
}
__device__ __forceinline__ int sat_s8(float v) {
  int r;
  asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(r) : "f"(v));
  return r;
}

template <int ROTARY, bool V2>
__global__ void __launch_bounds__(128)
k_qk_norm_rope_row128(const RowRopeParams p) {
  const uint64_t row = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= p.rows)
    return;
  const uint64_t token = row / p.heads, head = row - token * p.heads;
  const uint4 *src = p.x + token * p.in_token_stride16 + p.in_offset16 + head * 16;
  const uint64_t out_row = ((token / p.input_seq) * p.out_seq + p.out_start + token % p.input_seq) * p.heads + head;
  float n[128];
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    float f[8];
    unpack8(__ldg(src + c), f);
#pragma unroll
    for (int e = 0; e < 8; ++e)
      n[8 * c + e] = f[e];
  }
  float sum = 0.0f;
#pragma unroll
  for (int d = 0; d < 128; ++d)
    sum = __fadd_rn(sum, __fmul_rn(n[d], n[d]));
  const float inv = __fdiv_rn(1.0f, sqrtf(__fadd_rn(__fdiv_rn(sum, 128.0f), p.eps)));
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    float wv[8];
    unpack8(__ldg(p.w + c), wv);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float scaled = __fmul_rn(n[8 * c + e], inv);
      n[8 * c + e] = V2 ? round_bf16(__fmul_rn(round_bf16(scaled), wv[e])) : __fmul_rn(scaled, wv[e]);
    }
  }
  const uint64_t trow = ((token / p.input_seq) * p.table_seq + p.table_start + token % p.input_seq) * p.table_width;
  if (V2) { // interleaved pairs (2 i, 2 i + 1), one table entry per pair
#pragma unroll
    for (int pc = 0; pc < ROTARY / 16; ++pc) {
      float c[8], s[8];
      load_table8(p.cosv, p.table_f32, trow + 8 * pc, c);
      load_table8(p.sinv, p.table_f32, trow + 8 * pc, s);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float even = n[16 * pc + 2 * e], odd = n[16 * pc + 2 * e + 1];
        n[16 * pc + 2 * e] = __fsub_rn(__fmul_rn(even, c[e]), __fmul_rn(odd, s[e]));
        n[16 * pc + 2 * e + 1] = __fadd_rn(__fmul_rn(even, s[e]), __fmul_rn(odd, c[e]));
      }
    }
  } else { // half-split pairs (d, d + ROTARY / 2)
    constexpr int kHalf = ROTARY / 2;
    const bool wide = p.table_width == (uint32_t)ROTARY; // second half of the pair has its own entries
#pragma unroll
    for (int dc = 0; dc < kHalf / 8; ++dc) {
      float c1[8], s1[8], c2[8], s2[8];
      load_table8(p.cosv, p.table_f32, trow + 8 * dc, c1);
      load_table8(p.sinv, p.table_f32, trow + 8 * dc, s1);
      load_table8(p.cosv, p.table_f32, trow + 8 * dc + (wide ? kHalf : 0), c2);
      load_table8(p.sinv, p.table_f32, trow + 8 * dc + (wide ? kHalf : 0), s2);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float a = n[8 * dc + e], b = n[8 * dc + e + kHalf];
        n[8 * dc + e] = __fsub_rn(__fmul_rn(a, c1[e]), __fmul_rn(b, s1[e]));
        n[8 * dc + e + kHalf] = __fadd_rn(__fmul_rn(b, c2[e]), __fmul_rn(a, s2[e]));
      }
    }
  }
  // the stored bf16 values (what a consumer of the unfused op would read back)
  float m = 0.0f;
#pragma unroll
  for (int d = 0; d < 128; ++d) {
    n[d] = round_bf16(n[d]);
    m = fmaxf(m, fabsf(n[d]));
  }
  if (p.o) {
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e)
        f[e] = n[8 * c + e];
      p.o[out_row * 16 + c] = pack8(f);
    }
  }
  if (p.codes) {
    const float scale = fmaxf(__fdiv_rn(m, 127.0f), 1.0e-30f); // clip 1: max * 1 / 127
    p.scales[out_row] = scale;
    uint4 *dst = reinterpret_cast<uint4 *>(p.codes + out_row * 128);
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint32_t word[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        uint32_t packed = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e)
          packed |= (uint32_t)(max(sat_s8(__fdiv_rn(n[16 * c + 4 * q + e], scale)), -127) & 0xff) << (8 * e);
        word[q] = packed;
      }
      dst[c] = make_uint4(word[0], word[1], word[2], word[3]);
    }
  }
}

// ---- QuantizeInt8Rows(Direct) of 128-wide rows, one thread per row (same arithmetic as the
// warp-per-row kernel in convrot_quant.cu) ----
__global__ void __launch_bounds__(128)
k_direct_quant_row128(const uint4 *x, int8_t *codes, float *scales, uint64_t rows, float clip) {
  const uint64_t row = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows)
    return;
  float n[128], m = 0.0f;
#pragma unroll
  for (int c = 0; c < 16; ++c) {
    float f[8];
    unpack8(__ldg(x + row * 16 + c), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      n[8 * c + e] = f[e];
      m = fmaxf(m, fabsf(f[e]));
    }
  }
  const float scale = fmaxf(__fdiv_rn(__fmul_rn(m, clip), 127.0f), 1.0e-30f);
  scales[row] = scale;
  uint4 *dst = reinterpret_cast<uint4 *>(codes + row * 128);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint32_t word[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t packed = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        packed |= (uint32_t)(max(sat_s8(__fdiv_rn(n[16 * c + 4 * q + e], scale)), -127) & 0xff) << (8 * e);
      word[q] = packed;
    }
    dst[c] = make_uint4(word[0], word[1], word[2], word[3]);
  }
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline unsigned blocks_for(uint64_t n, int threads) {
  uint64_t b = (n + threads - 1) / threads;
  const uint64_t cap = (uint64_t)sm_count() * 32;
  return (unsigned)(b < 1 ? 1 : (b > cap ? cap : b));
}
int done(const char *what) { return launched(cudaGetLastError(), what); }

} // namespace

bool residual_gate_fast(const void *res, const void *branch, const void *gate, void *o, uint32_t dt, uint64_t n,
                        uint64_t width, uint64_t rows_per_gate, cudaStream_t s, int *rc) {
  if (dt != 2 || width % 8 != 0 || !aligned16(res) || !aligned16(branch) || !aligned16(gate) || !aligned16(o))
    return false;
  k_residual_gate_bf16<<<blocks_for(n / 8, 256), 256, 0, s>>>(
      static_cast<const uint4 *>(res), static_cast<const uint4 *>(branch), static_cast<const uint4 *>(gate),
      static_cast<uint4 *>(o), n / 8, width / 8, rows_per_gate);
  *rc = done("k_residual_gate_bf16");
  return true;
}

bool swiglu_fast(const void *x, void *o, uint32_t dt, uint64_t rows, uint64_t width, uint64_t in_width,
                 uint64_t start, bool gate_first, cudaStream_t s, int *rc) {
  if (dt != 2 || width % 8 != 0 || in_width % 8 != 0 || start % 8 != 0 || !aligned16(x) || !aligned16(o))
    return false;
  k_swiglu_bf16<<<blocks_for(rows * (width / 8), 256), 256, 0, s>>>(
      static_cast<const uint4 *>(x), static_cast<uint4 *>(o), rows, width / 8, in_width / 8, start / 8,
      gate_first ? 1 : 0);
  *rc = done("k_swiglu_bf16");
  return true;
}

bool row_stats_sequential(const void *x, uint64_t rows, uint64_t cols, float eps, bool layer, const float2 **stats,
                          cudaStream_t s, int *rc) {
  *stats = nullptr;
  *rc = 0;
  if (const char *v = std::getenv("DIFB200_EXACT_NORM"))
    if (v[0] == '0')
      return false;
  if (rows == 0 || cols == 0 || cols % kStatCols != 0 || cols > 0xffffff00ull || !aligned16(x))
    return false;
  float2 *area = static_cast<float2 *>(device_scratch(rows * sizeof(float2)));
  if (!area) {
    *rc = fail(kOutOfMemory, "cannot allocate the row statistics scratch");
    return true;
  }
  uint64_t blocks = (rows + 32 * kStatWarps - 1) / (32 * kStatWarps);
  const uint64_t cap = (uint64_t)sm_count() * 6; // 37 KB of shared memory per CTA: six resident per SM
  blocks = blocks > cap ? cap : blocks;
  if (layer)
    k_row_stats_sequential<true><<<(unsigned)blocks, 32 * kStatWarps, 0, s>>>(static_cast<const uint4 *>(x), area,
                                                                              rows, (uint32_t)cols, eps);
  else
    k_row_stats_sequential<false><<<(unsigned)blocks, 32 * kStatWarps, 0, s>>>(static_cast<const uint4 *>(x), area,
                                                                               rows, (uint32_t)cols, eps);
  *rc = done("k_row_stats_sequential");
  *stats = area;
  return true;
}

bool rms_norm_modulate_fast(const void *x, const void *w, const void *a, const void *b, void *o, uint32_t dt,
                            uint64_t rows, uint64_t cols, float eps, cudaStream_t s, int *rc) {
  if (dt != 2 || cols == 0 || cols % 256 != 0 || cols > 0xffffff00ull || !aligned16(x) || (w && !aligned16(w)) ||
      !aligned16(a) || !aligned16(b) || !aligned16(o))
    return false;
  uint64_t blocks = (rows + 7) / 8;
  const uint64_t cap = (uint64_t)sm_count() * 16;
  blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
  const auto X = static_cast<const uint4 *>(x), W = static_cast<const uint4 *>(w), A = static_cast<const uint4 *>(a),
             B = static_cast<const uint4 *>(b);
  const float2 *stats = nullptr;
  if (row_stats_sequential(x, rows, cols, eps, false, &stats, s, rc) && *rc)
    return true;
  if (cols == 3072)
    k_rms_norm_modulate_bf16<12><<<(unsigned)blocks, 256, 0, s>>>(X, W, A, B, static_cast<uint4 *>(o), rows,
                                                                  (uint32_t)cols, eps, stats);
  else
    k_rms_norm_modulate_bf16<0><<<(unsigned)blocks, 256, 0, s>>>(X, W, A, B, static_cast<uint4 *>(o), rows,
                                                                 (uint32_t)cols, eps, stats);
  *rc = done("k_rms_norm_modulate_bf16");
  return true;
}

bool layer_norm_modulate_fast(const void *x, const void *w, const void *b, const void *scale, const void *shift,
                              void *o, uint32_t dt, uint64_t rows, uint64_t cols, uint64_t rows_per_mod, float eps,
                              cudaStream_t s, int *rc) {
  if (dt != 2 || cols == 0 || cols % 256 != 0 || cols > 0xffffff00ull || !aligned16(x) || !aligned16(w) ||
      !aligned16(b) || !aligned16(scale) || !aligned16(shift) || !aligned16(o))
    return false;
  uint64_t blocks = (rows + 7) / 8;
  const uint64_t cap = (uint64_t)sm_count() * 16;
  blocks = blocks < 1 ? 1 : (blocks > cap ? cap : blocks);
  const auto X = static_cast<const uint4 *>(x), W = static_cast<const uint4 *>(w), B = static_cast<const uint4 *>(b),
             SC = static_cast<const uint4 *>(scale), SH = static_cast<const uint4 *>(shift);
  const float2 *stats = nullptr;
  if (row_stats_sequential(x, rows, cols, eps, true, &stats, s, rc) && *rc)
    return true;
  if (cols == 3072)
    k_layer_norm_modulate_bf16<12><<<(unsigned)blocks, 256, 0, s>>>(X, W, B, SC, SH, static_cast<uint4 *>(o), rows,
                                                                    (uint32_t)cols, rows_per_mod, eps, stats);
  else
    k_layer_norm_modulate_bf16<0><<<(unsigned)blocks, 256, 0, s>>>(X, W, B, SC, SH, static_cast<uint4 *>(o), rows,
                                                                   (uint32_t)cols, rows_per_mod, eps, stats);
  *rc = done("k_layer_norm_modulate_bf16");
  return true;
}

// QkNormPartialRope (+ optional Direct quantisation) for bf16 rows of 128; false when the shape is
// not covered (the caller then runs the generic kernel).
bool qk_norm_rope_fast(const void *x, const void *w, const void *cosv, const void *sinv, void *o, int8_t *codes,
                       float *scales, uint32_t dt, uint32_t dt_table, uint64_t tokens, uint64_t heads, uint64_t dim,
                       uint64_t rotary, uint64_t table_width, uint64_t input_seq, uint64_t table_seq,
                       uint64_t table_start, float eps, bool interleaved_v2, const RopeLayout *layout, cudaStream_t s,
                       int *rc) {
  const RopeLayout dense{heads * 128, 0, input_seq, 0};
  const RopeLayout &l = layout ? *layout : dense;
  if (l.in_token_stride % 8 != 0 || l.in_offset % 8 != 0)
    return false;
  if (dt != 2 || dim != 128 || (dt_table != 1 && dt_table != 2) || !aligned16(x) || !aligned16(w) ||
      !aligned16(cosv) || !aligned16(sinv) || (o && !aligned16(o)) || (codes && !aligned16(codes)))
    return false;
  if (rotary != 64 && rotary != 96 && rotary != 128)
    return false;
  // table rows must start on 16 bytes and hold what the layout reads
  const uint64_t entry = dt_table == 1 ? 4 : 2;
  if ((table_width * entry) % 16 != 0)
    return false;
  if (interleaved_v2 ? table_width != rotary / 2 : (table_width != rotary && table_width != rotary / 2))
    return false;
  RowRopeParams p{static_cast<const uint4 *>(x), static_cast<const uint4 *>(w), cosv, sinv, static_cast<uint4 *>(o),
                  codes, scales, tokens * heads, heads, input_seq, table_seq, table_start, l.in_token_stride / 8,
                  l.in_offset / 8, l.out_seq, l.out_start, (uint32_t)table_width, dt_table == 1 ? 1u : 0u, eps};
  const unsigned blocks = (unsigned)((p.rows + 127) / 128);
  if (p.rows + 127 > 0x7fffffffull * 128ull)
    return false;
#define DIFB200_ROPE_CASE(R, V)                                                                   \
  if (rotary == R && interleaved_v2 == V) {                                                       \
    k_qk_norm_rope_row128<R, V><<<blocks, 128, 0, s>>>(p);                                        \
    *rc = done("k_qk_norm_rope_row128");                                                          \
    return true;                                                                                  \
  }
  DIFB200_ROPE_CASE(64, false)
  DIFB200_ROPE_CASE(96, false)
  DIFB200_ROPE_CASE(128, false)
  DIFB200_ROPE_CASE(64, true)
  DIFB200_ROPE_CASE(96, true)
  DIFB200_ROPE_CASE(128, true)
#undef DIFB200_ROPE_CASE
  return false;
}

bool direct_quant_rows128(const void *x, int8_t *codes, float *scales, uint64_t rows, float clip, cudaStream_t s,
                          int *rc) {
  if (!aligned16(x) || !aligned16(codes) || rows + 127 > 0x7fffffffull * 128ull)
    return false;
  k_direct_quant_row128<<<(unsigned)((rows + 127) / 128), 128, 0, s>>>(static_cast<const uint4 *>(x), codes, scales,
                                                                      rows, clip);
  *rc = done("k_direct_quant_row128");
  return true;
}

} // namespace glue
} // namespace difb200
