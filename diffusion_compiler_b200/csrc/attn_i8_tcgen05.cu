// INT8 attention for sm_100a: INT8 Q.K^T on tcgen05 (kind::i8, INT32 scores in tensor memory),
// fp32 online softmax with a power-of-two running maximum, bf16 P.V on tcgen05 (kind::f16, fp32
// output accumulator in tensor memory), flash-style over 128-key tiles with TMA K/V staging.
// Grouped-query attention and a key-validity mask are supported; non-causal.
//
// Semantics. The op replaced is DiffIR Attention (reference src/runtime/cpu_executor.cpp:
// 1839-1910; GQA head mapping :1853-1863, all-masked-row rule :1881-1887; key mask as produced by
// BooleanMaskToBias with MaskQueries=false, :627-650) in the INT8 lowering that the reference
// only ships for sm_86 (src/runtime/h3_owned_attention.cu:646-929). Numerical contract (per
// query row i of head h, kv head h / (H / KV)):
//   acc_j = sum_d q8[i,d] * k8[j,d]                 INT32, exact
//   u_j   = float(acc_j) * ks'_j                    one fp32 rounding; ks'_j = the key scale rounded
//                                                   (nearest-even) to 22 significant bits;
//                                                   u_j = -inf for masked keys
//   A     = qs_i * (scale * log2(e))
//   m     = an integer >= ceil(max_j u_j * A)       (any such integer gives the same result up
//                                                    to the rounding of the fma below: bf16
//                                                    rounding commutes with powers of two). The
//                                                    kernel takes the Cauchy-Schwarz bound
//                                                    ceil(A * |q8_i| * max_j(|k8_j| * ks'_j)) when
//                                                    that is at most 60 (one pass, no running
//                                                    maximum, no rescaling of the output), else a
//                                                    running maximum
//   p_j   = exp2(fma(u_j, A, -m)),  P_j = bf16(p_j)
//   out   = bf16((sum_j P_j * v_j) / (sum_j p_j))   fp32 accumulation; all keys masked -> 0
// q8/qs and k8/ks are QuantizeInt8Rows(Direct) of the [B,S,H,128] / [B,S,KV,128] tensors.
//
// Structure: one CTA per (batch, head, 256 queries) = two 128-query tiles that share every K/V
// tile. Warpgroup 0: warp 0 = TMA producer, warp 1 = MMA issuer (warps 2-3 idle). Warpgroups 1
// and 2: softmax + epilogue of query tile 0 / 1, one thread per query row (its scores live in
// registers, so no shuffles). K/V arrive in 128-key stages; the score / softmax / P.V pipeline
// works in 64-key steps with the scores of each query tile double-buffered in tensor memory:
// Q.K^T of step g+2 is issued right after P.V of step g, into the buffer that step's P just left,
// so when a softmax warp finishes a step the scores of the next one are already there.
// Tensor memory (512 columns): per query tile two score buffers of 64 columns (INT32; the bf16 P
// of a step overwrites the first 32 columns of its buffer and is the TMEM A operand of P.V),
// then O0 | O1 (fp32, 128 columns each).
//
// Chunked form (the token-sharded block, where keys arrive from other GPUs one slice at a time):
// a launch covers up to two ranges of 128-key tiles and may carry the unnormalised state of every
// query row -- m, l and the fp32 output accumulator -- in from an earlier launch and out to a
// later one. Every m is an integer, so moving a row from one m to a larger one multiplies l, O
// and every p by an exact power of two: a sequence of launches over disjoint key ranges gives the
// single launch's result up to the order of the fp32 sums.
#include "common.cuh"
#include "ops.h"
#include "ptx.cuh"

#include <mutex>

namespace difb200 {
namespace {

constexpr int kTile = 128;          // queries per tile, keys per tile, head dim
constexpr int kStages = 3;          // K/V ring depth
constexpr uint32_t kQBytes = 128 * 128;        // int8 [128 x 128]
constexpr uint32_t kKBytes = 128 * 128;        // int8 [128 keys x 128]
constexpr uint32_t kVBytes = 128 * 128 * 2;    // bf16 [128 keys x 128] as two 64-wide halves
constexpr uint32_t kKsBytes = 128 * 8;         // (key scale, mask bias) per key, as float4 per key pair
constexpr uint32_t kStageBytes = kKBytes + kVBytes + kKsBytes;
constexpr int kThreads = 384;
constexpr size_t kSmemBytes = 1024 + 2 * kQBytes + kStages * kStageBytes + 256;

struct AttnParams {
  const float *qs;       // [B,S,H]
  const float2 *ksmb;    // [B,KV,S_pad/2] x float4 (ks'_j, ks'_j+1, bias_j, bias_j+1)
  const float *tile_bound; // [B,KV,S_pad/128] max over the tile's valid keys of |k8_j| * ks'_j
  uint16_t *out;         // [B,S,H,128] bf16
  uint32_t B, Sq, Sk, H, KV, S_pad; // Sq query tokens, Sk key tokens (S_pad = Sk rounded up to 128)
  float scale_log2e;     // scale * log2(e)
  unsigned long long wait_ns; // limit of every bounded wait
  DeviceStatus *status;
  // key tiles of this launch: [tile_begin[0], +tile_count[0]) then [tile_begin[1], +tile_count[1])
  uint32_t tile_begin[2], tile_count[2];
  float *o_state;        // [B,Sq,H,128] fp32 unnormalised outputs carried between launches
  float2 *ml_state;      // [B,Sq,H] (m, l) carried between launches
  uint32_t carry_in, carry_out;
};

__device__ __forceinline__ void report(DeviceStatus *status, uint32_t role, uint32_t detail) {
  if (atomicExch(&status->flag, 1u) == 0u) {
    status->kernel = 3u;
    status->role = role;
    status->detail = detail;
  }
}

// Builds the per-key table [B,KV,S_pad] of (ks', -C * ks') with C = 1.5 * 2^23: the key scales of
// the [B,S,KV] row order re-laid contiguous along keys, stored per key pair as
// (ks'_j, ks'_j+1, bias_j, bias_j+1) so that one 16-byte load feeds one packed fma. The softmax
// threads turn an INT32 score into fp32 with one integer add, f' = as_float(acc + bits(C)) =
// C + acc exactly, and then u = fma(f', ks', -C * ks') = RN(acc * ks'): rounding ks to 22
// significant bits makes C * ks' exact, so the fused form has the single rounding of a plain
// multiply. Masked and padding keys carry (0, -inf), which yields u = -inf.
// Also writes, per 128-key tile, the largest |k8_j|_2 * ks'_j of its valid keys: with |q8_i|_2 it
// bounds every score of the tile (Cauchy-Schwarz on the integer codes).
// One block of 128 threads per (batch, kv head, key tile), one thread per key.
__global__ void __launch_bounds__(128)
key_table_kernel(const int8_t *k8, const float *ks, const uint8_t *key_valid, float *table,
                 float *tile_bound, uint32_t S, uint32_t KV, uint32_t S_pad, uint32_t begin0, uint32_t count0,
                 uint32_t begin1, uint32_t count1) {
  const uint32_t tiles = S_pad / kTile;     // tiles of the whole key axis (table layout)
  const uint32_t mine = count0 + count1;    // tiles this launch covers
  const uint32_t local = blockIdx.x % mine;
  const uint32_t tile = local < count0 ? begin0 + local : begin1 + (local - count0);
  const uint32_t kvh = (blockIdx.x / mine) % KV;
  const uint32_t b = blockIdx.x / (mine * KV);
  const uint32_t j = tile * kTile + threadIdx.x;
  float k22 = 0.0f, bias = -INFINITY, bound = 0.0f;
  if (j < S && (key_valid == nullptr || key_valid[(uint64_t)b * S + j] != 0)) {
    uint32_t bits = __float_as_uint(ks[((uint64_t)b * S + j) * KV + kvh]);
    bits = (bits + 1u + ((bits >> 2) & 1u)) & ~3u; // nearest-even to 22 significant bits
    k22 = __uint_as_float(bits);
    bias = -12582912.0f * k22;
    const uint4 *row = reinterpret_cast<const uint4 *>(k8 + (((uint64_t)b * S + j) * KV + kvh) * kTile);
    int n2 = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const uint4 w = __ldg(row + c);
      n2 = __dp4a((int)w.x, (int)w.x, n2);
      n2 = __dp4a((int)w.y, (int)w.y, n2);
      n2 = __dp4a((int)w.z, (int)w.z, n2);
      n2 = __dp4a((int)w.w, (int)w.w, n2);
    }
    bound = __fmul_rn(__fsqrt_rn((float)n2), k22);
  }
  float *t = table + (((uint64_t)b * KV + kvh) * S_pad + (j & ~1u)) * 2u + (j & 1u);
  t[0] = k22;
  t[2] = bias;
  __shared__ float warp_max[4];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    bound = fmaxf(bound, __shfl_xor_sync(0xffffffffu, bound, o));
  if ((threadIdx.x & 31) == 0)
    warp_max[threadIdx.x >> 5] = bound;
  __syncthreads();
  if (threadIdx.x == 0)
    tile_bound[((uint64_t)b * KV + kvh) * tiles + tile] =
        fmaxf(fmaxf(warp_max[0], warp_max[1]), fmaxf(warp_max[2], warp_max[3]));
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t packed;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
  return packed;
}

__global__ void __launch_bounds__(kThreads, 1)
attn_i8_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  const uint32_t base = (raw_addr + 1023u) & ~1023u;
  uint8_t *base_ptr = smem_raw + (base - raw_addr);
  const uint32_t q_addr = base;                       // 2 x 16 KB
  const uint32_t stage_addr = base + 2 * kQBytes;     // kStages x (K | V | ksmb)
  const uint32_t bar = stage_addr + kStages * kStageBytes;
  // barriers (8 bytes each)
  const uint32_t q_full = bar;
  const uint32_t k_full = bar + 8, k_empty = k_full + 8 * kStages;
  const uint32_t v_full = k_empty + 8 * kStages, v_empty = v_full + 8 * kStages;
  const uint32_t s_full = v_empty + 8 * kStages;      // [2 tiles][2 buffers]
  const uint32_t p_full = s_full + 32;                // [2][2]
  const uint32_t pv_done = p_full + 32;               // [2] one phase per step (rescaling waits on it)
  const uint32_t o_done = pv_done + 16;               // [2] completes once, after the last P.V
  const uint32_t tmem_slot = o_done + 16;
  volatile uint32_t *slot_ptr = reinterpret_cast<volatile uint32_t *>(base_ptr + (tmem_slot - base));
  volatile uint32_t *abort_ptr = slot_ptr + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned long long wait_ns = p.wait_ns;
  const uint32_t q_blocks = (p.Sq + 255u) / 256u;
  const uint32_t qb = blockIdx.x % q_blocks;
  const uint32_t head = (blockIdx.x / q_blocks) % p.H;
  const uint32_t batch = blockIdx.x / (q_blocks * p.H);
  const uint32_t kvh = head / (p.H / p.KV);
  const uint32_t q0 = qb * 256u;
  const uint32_t n_kv = p.tile_count[0] + p.tile_count[1];
  const uint32_t n_steps = 2u * n_kv;               // 64-key steps
  auto key_tile = [&](uint32_t i) {                 // i-th key tile of this launch -> tile of the key axis
    return i < p.tile_count[0] ? p.tile_begin[0] + i : p.tile_begin[1] + (i - p.tile_count[0]);
  };
  auto score_col = [](uint32_t t, uint32_t b) { return t * 128u + b * 64u; }; // TMEM column of a score buffer

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(k_full + 8 * s, 1);
      ptx::mbar_init(k_empty + 8 * s, 1);
      ptx::mbar_init(v_full + 8 * s, 1);
      ptx::mbar_init(v_empty + 8 * s, 1);
    }
    for (int t = 0; t < 2; ++t) {
      for (int b = 0; b < 2; ++b) {
        ptx::mbar_init(s_full + 16 * t + 8 * b, 1);
        ptx::mbar_init(p_full + 16 * t + 8 * b, 128);
      }
      ptx::mbar_init(pv_done + 8 * t, 1);
      ptx::mbar_init(o_done + 8 * t, 1);
    }
    *abort_ptr = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_q);
    ptx::prefetch_tensormap(&map_k);
    ptx::prefetch_tensormap(&map_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *slot_ptr;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    // The producer and the MMA warp run their loops with all 32 lanes and warp-uniform control
    // flow (every wait ends in a vote); one elected lane issues the asynchronous instructions.
    // Addresses, descriptors and loop state are then warp-uniform values. As single-lane
    // (divergent) loops every TMA / MMA operand was first moved between register files, and
    // issuing the 12 MMAs of one tile step took about twice the 768 clocks they execute in.
    auto give_up = [&](uint32_t role, uint32_t detail) {
      if (lane == 0) {
        if (!*abort_ptr)
          report(p.status, role, detail);
        *abort_ptr = 1;
      }
    };
    if (warp == 0) {
      // ---------------- TMA producer ----------------
      if (ptx::elect_one()) {
        ptx::mbar_expect_tx(q_full, 2 * kQBytes);
        ptx::tma_load_4d(q_addr, &map_q, q_full, 0, (int32_t)head, (int32_t)q0, (int32_t)batch);
        ptx::tma_load_4d(q_addr + kQBytes, &map_q, q_full, 0, (int32_t)head, (int32_t)(q0 + 128u),
                         (int32_t)batch);
      }
      const float2 *table = p.ksmb + ((uint64_t)batch * p.KV + kvh) * p.S_pad;
      uint32_t s = 0, phase = 0;
      for (uint32_t i = 0; i < n_kv; ++i) {
        const uint32_t k_dst = stage_addr + s * kStageBytes, v_dst = k_dst + kKBytes,
                       t_dst = v_dst + kVBytes;
        const uint32_t tile = key_tile(i);
        const int32_t key0 = (int32_t)(tile * kTile);
        if (!ptx::mbar_wait_warp(k_empty + 8 * s, phase ^ 1u, abort_ptr, wait_ns)) {
          give_up(0, i);
          break;
        }
        if (ptx::elect_one()) {
          ptx::mbar_expect_tx(k_full + 8 * s, kKBytes);
          ptx::tma_load_4d(k_dst, &map_k, k_full + 8 * s, 0, (int32_t)kvh, key0, (int32_t)batch);
        }
        if (!ptx::mbar_wait_warp(v_empty + 8 * s, phase ^ 1u, abort_ptr, wait_ns)) {
          give_up(1, i);
          break;
        }
        if (ptx::elect_one()) {
          ptx::mbar_expect_tx(v_full + 8 * s, kVBytes + kKsBytes);
          ptx::tma_load_4d(v_dst, &map_v, v_full + 8 * s, 0, (int32_t)kvh, key0, (int32_t)batch);
          ptx::tma_load_4d(v_dst + kVBytes / 2, &map_v, v_full + 8 * s, 64, (int32_t)kvh, key0,
                           (int32_t)batch);
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
                           "r"(t_dst), "l"(reinterpret_cast<uint64_t>(table + (uint64_t)tile * kTile)),
                       "r"(kKsBytes), "r"(v_full + 8 * s)
                       : "memory");
        }
        if (++s == kStages) {
          s = 0;
          phase ^= 1u;
        }
      }
    } else if (warp == 1) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc_qk = ptx::make_idesc(2 /*S32*/, 1 /*S8*/, 1 /*S8*/, 0, 0, 128, 64);
      constexpr uint32_t idesc_pv = ptx::make_idesc(1 /*F32*/, 1 /*BF16*/, 1 /*BF16*/, 0, 1 /*V is N-major*/, 128, 128);
      const uint64_t q_desc = ptx::smem_desc_sw128(q_addr, 16, 1024);
      const uint64_t k_desc0 = ptx::smem_desc_sw128(stage_addr, 16, 1024);
      // V tile, N-major: 64-wide halves 16 KB apart (leading offset), 8-key groups 1 KB apart.
      const uint64_t v_desc0 = ptx::smem_desc_sw128(stage_addr + kKBytes, kVBytes / 2, 1024);
      bool ok = true;
      // (both are called inside the elected lane's branch) step g covers keys 64 g .. 64 g + 63,
      // i.e. half g & 1 of the 128-key stage (g / 2) % kStages, and score buffer g & 1.
      auto issue_qk = [&](uint32_t t, uint32_t g) {
        const uint32_t h = g & 1u, st = (g >> 1) % kStages;
        const uint64_t a = q_desc + (uint64_t)((t * kQBytes) >> 4);
        const uint64_t b = k_desc0 + (uint64_t)((st * kStageBytes + h * 64u * 128u) >> 4);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          ptx::mma_i8_ss(tmem + score_col(t, h), a + (uint64_t)(2 * k), b + (uint64_t)(2 * k), idesc_qk, k != 0);
        ptx::mma_commit(s_full + 16 * t + 8 * h);
      };
      auto issue_pv = [&](uint32_t t, uint32_t g) {
        // A = P in tensor memory (32 columns of bf16 pairs at the start of the score buffer);
        // B = the 64 keys of the V stage: 16 keys per MMA = 8 TMEM columns, 2048 bytes of V
        const uint32_t h = g & 1u, st = (g >> 1) % kStages;
        const uint64_t b = v_desc0 + (uint64_t)((st * kStageBytes + h * 64u * 128u) >> 4);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          ptx::mma_f16_ts(tmem + 256u + t * 128u, tmem + score_col(t, h) + 8u * k, b + (uint64_t)(128 * k),
                          idesc_pv, k != 0 ? 1u : ((g != 0u || p.carry_in) ? 1u : 0u));
        ptx::mma_commit(pv_done + 8 * t);
      };
      if (!ptx::mbar_wait_warp(q_full, 0, abort_ptr, wait_ns)) {
        give_up(2, 0);
        ok = false;
      }
      if (ok && (!ptx::mbar_wait_warp(k_full, 0, abort_ptr, wait_ns) || !ptx::mbar_wait_warp(v_full, 0, abort_ptr, wait_ns))) {
        give_up(2, 1);
        ok = false;
      }
      if (ok) {
        ptx::tc_fence_after();
        if (ptx::elect_one()) {
          issue_qk(0, 0);
          issue_qk(1, 0);
          issue_qk(0, 1);
          issue_qk(1, 1);
          ptx::mma_commit(k_empty);
        }
      }
      for (uint32_t g = 0; g < n_steps && ok; ++g) {
        const uint32_t h = g & 1u, use = g >> 1;               // use-th time this score buffer is filled
        const uint32_t st = use % kStages;
        const uint32_t use_n = use + 1u, st_n = use_n % kStages, phase_n = (use_n / kStages) & 1u;
        const bool more = g + 2u < n_steps;
        // K, V and the key table of the next stage, before the first Q.K^T on it (the softmax
        // warps take the completion of that Q.K^T as their signal for the table, and this
        // stage's V was awaited the same way one stage earlier)
        if (h == 0u && more &&
            (!ptx::mbar_wait_warp(k_full + 8 * st_n, phase_n, abort_ptr, wait_ns) ||
             !ptx::mbar_wait_warp(v_full + 8 * st_n, phase_n, abort_ptr, wait_ns))) {
          give_up(2, 5);
          break;
        }
#pragma unroll
        for (uint32_t t = 0; t < 2; ++t) {
          if (!ptx::mbar_wait_warp(p_full + 16 * t + 8 * h, use & 1u, abort_ptr, wait_ns)) {
            give_up(2, 3 + t);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          if (ptx::elect_one()) {
            issue_pv(t, g);
            if (g + 1u == n_steps)
              ptx::mma_commit(o_done + 8 * t);
            if (t == 1 && h == 1u)
              ptx::mma_commit(v_empty + 8 * st);
            if (more) {
              issue_qk(t, g + 2u); // into the buffer P of step g is being read from: same pipe, in order
              if (t == 1 && h == 1u)
                ptx::mma_commit(k_empty + 8 * st_n);
            }
          }
        }
      }
    }
  } else {
    // ---------------- softmax + epilogue, one thread per query row ----------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const uint32_t t = (uint32_t)(warp - 4) >> 2;       // query tile 0 / 1
    const uint32_t quarter = (uint32_t)warp & 3u;
    const uint32_t row_in_tile = quarter * 32u + lane;
    const uint32_t qrow = q0 + t * 128u + row_in_tile;
    const bool row_ok = qrow < p.Sq;
    const float A = (row_ok ? __ldg(p.qs + ((uint64_t)batch * p.Sq + qrow) * p.H + head) : 1.0f) *
                    p.scale_log2e;
    const uint32_t lane_base = (quarter * 32u) << 16;
    const uint32_t s_tmem = tmem + lane_base + t * 128u, o_tmem = tmem + lane_base + 256u + t * 128u;
    float m_run = -INFINITY, l = 0.0f;
    bool alive = true;
    // A bound on every score of this row: |q8_i| * max_j(|k8_j| * ks'_j) * A. When it is small
    // for the whole warp, its ceiling is the fixed maximum m of the row and a key tile needs one
    // pass (no maximum, no rescaling); otherwise the warp keeps a running maximum.
    bool fixed_max = false;
    {
      float kmax = 0.0f;
      const float *bounds = p.tile_bound + ((uint64_t)batch * p.KV + kvh) * (p.S_pad / kTile);
      for (uint32_t i = lane; i < n_kv; i += 32)
        kmax = fmaxf(kmax, __ldg(bounds + key_tile(i)));
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        kmax = fmaxf(kmax, __shfl_xor_sync(0xffffffffu, kmax, o));
      if (!ptx::mbar_wait(q_full, 0, wait_ns)) {
        if (lane == 0)
          report(p.status, 9 + t, 0);
        *abort_ptr = 1;
        alive = false;
      }
      // the row's 128 codes: eight 16-byte chunks of one 128-byte row (the swizzle permutes
      // chunks inside the row, and the sum does not care); lanes start at different chunks
      const uint4 *qrow = reinterpret_cast<const uint4 *>(base_ptr + (q_addr - base) + t * kQBytes +
                                                          row_in_tile * 128u);
      int n2 = 0;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 w = qrow[(c + lane) & 7];
        n2 = __dp4a((int)w.x, (int)w.x, n2);
        n2 = __dp4a((int)w.y, (int)w.y, n2);
        n2 = __dp4a((int)w.z, (int)w.z, n2);
        n2 = __dp4a((int)w.w, (int)w.w, n2);
      }
      const float bound = __fmul_rn(__fmul_rn(A, __fsqrt_rn((float)n2)), kmax);
      const float m_fixed = ceilf(__fadd_rn(bound, 0.001f));
      // State carried in from the launch over the previous key ranges. m only ever grows, and
      // the fixed form may use any integer that is at least its bound: the larger of the carried m
      // and this launch's bound serves both, the carried l and O move to it by an exact power of
      // two, and the running form simply goes on from the carried m.
      float m_prev = -INFINITY;
      if (p.carry_in && row_ok) {
        const float2 ml = __ldg(p.ml_state + ((uint64_t)batch * p.Sq + (q0 + t * 128u + row_in_tile)) * p.H + head);
        m_prev = ml.x;
        l = ml.y;
      }
      const float m_both = fmaxf(m_prev, m_fixed);
      fixed_max = __all_sync(0xffffffffu, m_both <= 60.0f);
      m_run = fixed_max ? m_both : m_prev;
      if (p.carry_in) {
        const float factor = (fixed_max && m_prev != -INFINITY) ? ex2(m_prev - m_run) : (fixed_max ? 0.0f : 1.0f);
        l *= factor;
        const float4 *src = reinterpret_cast<const float4 *>(
            p.o_state + (((uint64_t)batch * p.Sq + (q0 + t * 128u + row_in_tile)) * p.H + head) * kTile);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            const float4 x = row_ok ? __ldg(src + 8 * c + v) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            o[4 * v] = __float_as_uint(x.x * factor);
            o[4 * v + 1] = __float_as_uint(x.y * factor);
            o[4 * v + 2] = __float_as_uint(x.z * factor);
            o[4 * v + 3] = __float_as_uint(x.w * factor);
          }
          ptx::tmem_st_32x32(o_tmem + 32u * c, o);
        }
        ptx::tmem_st_wait(); // published to the MMA warp with the arrive behind the first P
      }
    }
    const uint64_t A2 = pack2(A, A);
    for (uint32_t g = 0; g < n_steps && alive; ++g) {
      const uint32_t h = g & 1u, use = g >> 1;
      const uint32_t s = use % kStages;
      // The scores of this step. The stage's key table needs no wait of its own: it arrives on
      // the barrier of the V tile, which the MMA warp has seen complete before it issued the
      // Q.K^T whose completion is awaited here.
      if (!ptx::mbar_wait_abortable(s_full + 16 * t + 8 * h, use & 1u, abort_ptr, wait_ns)) {
        if (!*abort_ptr && lane == 0)
          report(p.status, 3 + t, g);
        *abort_ptr = 1;
        alive = false;
        break;
      }
      ptx::tc_fence_after();
      const uint32_t sc_tmem = s_tmem + h * 64u;
      uint32_t r[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c)
        ptx::tmem_ld_32x32(sc_tmem + 32u * c, r[c]);
      ptx::tmem_ld_wait();
      const float4 *tab = reinterpret_cast<const float4 *>(base_ptr + (stage_addr - base) + s * kStageBytes +
                                                           kKBytes + kVBytes) + h * 32u;
      uint32_t pk[32];
      uint64_t sum2[4] = {0ull, 0ull, 0ull, 0ull}; // 8 partial row sums as packed fp32 pairs
      if (fixed_max) {
        const uint64_t negm2 = pack2(-m_run, -m_run);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float4 kk = tab[(c * 32 + j) >> 1]; // (ks'_j, ks'_j+1, -C ks'_j, -C ks'_j+1)
            const float f0 = __int_as_float((int32_t)r[c][j] + 0x4B400000);     // C + acc, exact
            const float f1 = __int_as_float((int32_t)r[c][j + 1] + 0x4B400000);
            const uint64_t u2 = fma2(pack2(f0, f1), pack2(kk.x, kk.y), pack2(kk.z, kk.w));
            float e0, e1;
            unpack2(fma2(u2, A2, negm2), e0, e1);
            const float p0 = ex2(e0), p1 = ex2(e1);
            sum2[(j >> 1) & 3] = add2(sum2[(j >> 1) & 3], pack2(p0, p1));
            pk[(c * 32 + j) >> 1] = pack_bf16(p0, p1);
          }
        }
      } else {
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float4 kk = tab[(c * 32 + j) >> 1];
            const float f0 = __int_as_float((int32_t)r[c][j] + 0x4B400000);
            const float f1 = __int_as_float((int32_t)r[c][j + 1] + 0x4B400000);
            float u0, u1;
            unpack2(fma2(pack2(f0, f1), pack2(kk.x, kk.y), pack2(kk.z, kk.w)), u0, u1);
            r[c][j] = __float_as_uint(u0);
            r[c][j + 1] = __float_as_uint(u1);
            float &acc_max = mx4[(j >> 1) & 3];
            asm("max.f32 %0, %0, %1, %2;" : "+f"(acc_max) : "f"(u0), "f"(u1));
          }
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        // power-of-two running maximum
        float m_new = m_run;
        if (mx != -INFINITY)
          m_new = fmaxf(m_run, ceilf(mx * A));
        const bool grow = m_new > m_run && m_run != -INFINITY;
        if (__any_sync(0xffffffffu, grow)) {
          // rescale O (and l) by an exact power of two; needs P.V of the previous step finished
          // (grow implies an earlier step with a valid key, so g > 0)
          if (!ptx::mbar_wait(pv_done + 8 * t, (g - 1u) & 1u, wait_ns)) {
            if (lane == 0)
              report(p.status, 5 + t, g);
            *abort_ptr = 1;
            alive = false;
            break;
          }
          ptx::tc_fence_after();
          const float factor = grow ? ex2(m_run - m_new) : 1.0f;
          l *= factor;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t o[32];
            ptx::tmem_ld_32x32(o_tmem + 32u * c, o);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j)
              o[j] = __float_as_uint(__uint_as_float(o[j]) * factor);
            ptx::tmem_st_32x32(o_tmem + 32u * c, o);
          }
          ptx::tmem_st_wait();
        }
        m_run = m_new;
        const float neg_m = (m_run == -INFINITY) ? 0.0f : -m_run;
        const uint64_t negm2 = pack2(neg_m, neg_m);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            float e0, e1;
            unpack2(fma2(pack2(__uint_as_float(r[c][j]), __uint_as_float(r[c][j + 1])), A2, negm2), e0, e1);
            const float p0 = ex2(e0), p1 = ex2(e1);
            sum2[(j >> 1) & 3] = add2(sum2[(j >> 1) & 3], pack2(p0, p1));
            pk[(c * 32 + j) >> 1] = pack_bf16(p0, p1);
          }
        }
      }
      {
        float a0, a1, b0, b1;
        unpack2(add2(sum2[0], sum2[1]), a0, a1);
        unpack2(add2(sum2[2], sum2[3]), b0, b1);
        l += (a0 + a1) + (b0 + b1);
      }
      ptx::tmem_st_32x32(sc_tmem, pk);
      ptx::tmem_st_wait();
      ptx::tc_fence_before();
      ptx::mbar_arrive(p_full + 16 * t + 8 * h);
    }
    if (alive && n_kv > 0) {
      if (!ptx::mbar_wait(o_done + 8 * t, 0, wait_ns)) {
        if (lane == 0)
          report(p.status, 7 + t, 0);
        *abort_ptr = 1;
      } else {
        ptx::tc_fence_after();
        uint16_t *dst = p.out + (((uint64_t)batch * p.Sq + qrow) * p.H + head) * kTile;
        if (p.carry_out && row_ok)
          p.ml_state[((uint64_t)batch * p.Sq + qrow) * p.H + head] = make_float2(m_run, l);
        float4 *carry = reinterpret_cast<float4 *>(p.o_state + (((uint64_t)batch * p.Sq + qrow) * p.H + head) * kTile);
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          ptx::tmem_ld_32x32(o_tmem + 32u * c, o);
          ptx::tmem_ld_wait();
          if (p.carry_out) {
            if (row_ok) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                carry[8 * c + v] = make_float4(__uint_as_float(o[4 * v]), __uint_as_float(o[4 * v + 1]),
                                               __uint_as_float(o[4 * v + 2]), __uint_as_float(o[4 * v + 3]));
            }
          } else if (row_ok) {
            uint32_t w[16];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const float y0 = l > 0.0f ? __fdiv_rn(__uint_as_float(o[j]), l) : 0.0f;
              const float y1 = l > 0.0f ? __fdiv_rn(__uint_as_float(o[j + 1]), l) : 0.0f;
              w[j >> 1] = pack_bf16(y0, y1);
            }
#pragma unroll
            for (int v = 0; v < 4; ++v)
              reinterpret_cast<uint4 *>(dst + 32 * c)[v] =
                  make_uint4(w[4 * v], w[4 * v + 1], w[4 * v + 2], w[4 * v + 3]);
          }
        }
      }
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
}

} // namespace

// Scratch: the key table (8 bytes per padded key and kv head) followed by one bound per key tile.
size_t attention_int8_scratch_bytes(uint64_t B, uint64_t S, uint64_t KV) {
  const uint64_t s_pad = (S + kTile - 1) / kTile * kTile;
  return (size_t)(B * KV * s_pad * sizeof(float2) + ((B * KV * (s_pad / kTile) * sizeof(float) + 15) & ~15ull));
}

size_t attention_int8_state_bytes(uint64_t B, uint64_t Sq, uint64_t H) {
  return (size_t)(B * Sq * H * (kTile * sizeof(float) + sizeof(float2)));
}

int attention_int8(const int8_t *q8, const float *qs, const int8_t *k8, const float *ks, const void *v_bf16,
                   const uint8_t *key_valid, uint64_t B, uint64_t Sq, uint64_t S, uint64_t H, uint64_t KV,
                   uint64_t D, float scale, void *scratch, size_t scratch_bytes, void *out_bf16,
                   cudaStream_t stream, const AttentionChunk *chunk) {
  // S is the number of key/value tokens from here on; Sq the number of query tokens.
  if (!q8 || !qs || !k8 || !ks || !v_bf16 || !out_bf16 || !scratch)
    return fail(kInvalidArgument, "Attention(INT8): null pointer");
  if (D != 128)
    return fail(kUnsupported, "Attention(INT8): head dimension must be 128");
  if (B == 0 || Sq == 0 || H == 0)
    return kOk;
  if (S == 0)
    return fail(kInvalidArgument, "Attention(INT8): no keys");
  if (KV == 0 || H % KV != 0)
    return fail(kInvalidArgument, "Attention(INT8): KvHeads must divide the head count");
  if (B * H * ((Sq + 255) / 256) > 0x7fffffffull || S > 0x7fffff00ull || Sq > 0x7fffff00ull)
    return fail(kUnsupported, "Attention(INT8): problem too large");
  if (scratch_bytes < attention_int8_scratch_bytes(B, S, KV))
    return fail(kInvalidArgument, "Attention(INT8): scratch buffer too small");
  if ((reinterpret_cast<uintptr_t>(q8) | reinterpret_cast<uintptr_t>(k8) |
       reinterpret_cast<uintptr_t>(v_bf16) | reinterpret_cast<uintptr_t>(out_bf16) |
       reinterpret_cast<uintptr_t>(scratch)) & 15)
    return fail(kUnsupported, "Attention(INT8): pointers must be 16-byte aligned");
  DeviceStatus *status = device_status_words();
  if (!status)
    return fail(kOutOfMemory, "Attention(INT8): cannot allocate device status words");
  const uint32_t s_pad = (uint32_t)((S + kTile - 1) / kTile * kTile);
  const uint32_t all_tiles = s_pad / kTile;
  uint32_t begin[2] = {0, 0}, count[2] = {all_tiles, 0};
  if (chunk) {
    for (int i = 0; i < 2; ++i) {
      begin[i] = chunk->tile_begin[i];
      count[i] = chunk->tile_count[i];
      if ((uint64_t)begin[i] + count[i] > all_tiles)
        return fail(kInvalidArgument, "Attention(INT8): key tile range beyond the key axis");
    }
    if (count[0] + count[1] == 0)
      return fail(kInvalidArgument, "Attention(INT8): a launch needs at least one key tile");
    if ((chunk->carry_in || chunk->carry_out) && (!chunk->state || (reinterpret_cast<uintptr_t>(chunk->state) & 15)))
      return fail(kInvalidArgument, "Attention(INT8): carried state needs a 16-byte aligned state buffer");
  }

  CUtensorMap map_q, map_k, map_v;
  {
    const uint64_t dims[4] = {128, H, Sq, B};
    const uint64_t strides[3] = {128, H * 128, Sq * H * 128};
    const uint32_t box[4] = {128, 1, 128, 1};
    if (int rc = encode_tensor_map(&map_q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, q8, dims, strides, box,
                                   CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t dims[4] = {128, KV, S, B};
    const uint64_t strides[3] = {128, KV * 128, S * KV * 128};
    const uint32_t box[4] = {128, 1, 128, 1};
    if (int rc = encode_tensor_map(&map_k, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, k8, dims, strides, box,
                                   CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  {
    const uint64_t dims[4] = {128, KV, S, B};
    const uint64_t strides[3] = {256, KV * 256, S * KV * 256};
    const uint32_t box[4] = {64, 1, 128, 1};
    if (int rc = encode_tensor_map(&map_v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, v_bf16, dims, strides, box,
                                   CU_TENSOR_MAP_SWIZZLE_128B))
      return rc;
  }
  static const char attr_key = 0; // the opt-in belongs to the function in one context: once per device
  if (int rc = current_device_once(&attr_key, [](void *, int *) -> int {
        return check_cuda(cudaFuncSetAttribute(attn_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)kSmemBytes),
                          "cudaFuncSetAttribute(attn_i8_kernel)");
      }, nullptr, nullptr))
    return rc;

  float2 *table = static_cast<float2 *>(scratch);
  float *tile_bound = reinterpret_cast<float *>(table + B * KV * s_pad);
  {
    const uint64_t blocks = B * KV * (count[0] + count[1]);
    if (blocks > 0x7fffffffull)
      return fail(kUnsupported, "Attention(INT8): problem too large");
    key_table_kernel<<<(unsigned)blocks, 128, 0, stream>>>(k8, ks, key_valid, reinterpret_cast<float *>(table),
                                                           tile_bound, (uint32_t)S, (uint32_t)KV, s_pad, begin[0],
                                                           count[0], begin[1], count[1]);
    if (int rc = launched(cudaGetLastError(), "key_table_kernel launch"))
      return rc;
  }
  AttnParams p{};
  p.qs = qs;
  p.ksmb = table;
  p.tile_bound = tile_bound;
  p.out = static_cast<uint16_t *>(out_bf16);
  p.B = (uint32_t)B;
  p.Sq = (uint32_t)Sq;
  p.Sk = (uint32_t)S;
  p.H = (uint32_t)H;
  p.KV = (uint32_t)KV;
  p.S_pad = s_pad;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.wait_ns = wait_limit_ns();
  p.status = status;
  for (int i = 0; i < 2; ++i) {
    p.tile_begin[i] = begin[i];
    p.tile_count[i] = count[i];
  }
  if (chunk && (chunk->carry_in || chunk->carry_out)) {
    // state buffer: fp32 outputs [B,Sq,H,128], then (m, l) per row
    p.o_state = static_cast<float *>(chunk->state);
    p.ml_state = reinterpret_cast<float2 *>(p.o_state + B * Sq * H * kTile);
    p.carry_in = chunk->carry_in ? 1u : 0u;
    p.carry_out = chunk->carry_out ? 1u : 0u;
  }
  const uint64_t grid = B * H * ((Sq + 255) / 256);
  attn_i8_kernel<<<(unsigned)grid, kThreads, kSmemBytes, stream>>>(map_q, map_k, map_v, p);
  return launched(cudaGetLastError(), "attn_i8_kernel launch");
}

} // namespace difb200
