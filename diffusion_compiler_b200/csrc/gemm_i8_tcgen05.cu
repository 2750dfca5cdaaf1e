// LinearInt8Scaled for sm_100a: Y[M,N] = bf16((float(X[M,K] . W[N,K]^T) * xs[m]) * ws[n]),
// optionally followed by the BiasAdd and tanh-Gelu ops that the W8A8 rewrite puts after it.
// Semantics: reference src/runtime/cpu_executor.cpp:309-335 (multiplication order row scale
// first, then column scale), BiasAdd :1288-1296, Gelu :93-113; it replaces the reference's
// Sm80 mma.sync CUTLASS kernel (src/runtime/cutlass_gemm.cu:185-303).
//
// Structure: persistent CTAs, one per SM. Both operands are K-major INT8, brought in by TMA as
// 128-byte-swizzled [rows x 128 B] boxes into a shared-memory ring. One thread issues
// tcgen05.mma kind::i8 into one of two 256-column INT32 accumulators in tensor memory, so the
// epilogue of tile i overlaps the MMAs of tile i+1. Warp roles: 0 = TMA producer, 1 = TMEM owner
// + MMA issuer, 2..9 = epilogue: two warps per TMEM lane quarter (warp_id % 4), one for each
// 128-column half of the tile (four epilogue warps could not keep up with the K = 3072 main
// loop once bias and GELU are fused in).
//
// Two forms of the same kernel (template parameter CTAS):
//   CTAS = 1: 128x256 tile per CTA, cta_group::1, 4 stages of 48 KB.
//   CTAS = 2: a CTA pair (cluster of 2) computes a 256x256 tile with cta_group::2 MMAs: each CTA
//             stages its 128 rows of A and only its 128 rows (half) of the B tile, 5 stages of
//             32 KB. This halves the B bytes every SM moves through shared memory per MAC -- at
//             8192 INT8 MACs/clk/SM the 128x256 single-CTA tile needs 48 KB written plus 48 KB read
//             per 512 clocks, which is what bounds the CTAS = 1 form. The leader CTA (cluster rank
//             0) issues the MMAs; both CTAs load, and both run the epilogue on their own 128 rows.
//             TMA loads never use multicast. The bytes of both CTAs are counted on the leader's
//             mbarrier (the peer issues the cta_group::2 form of the load, whose completion may
//             target the peer CTA's barrier); the leader releases stages and publishes
//             accumulators to both CTAs with one tcgen05.commit that signals the mbarrier of both
//             CTAs. The only remaining software signal across the pair is the epilogue's arrive
//             on the leader's accumulator-empty barrier, with CTA-scope release: a cluster-scope
//             release arrive per k-block costs microseconds while TMA traffic is in flight.
#include "common.cuh"
#include "ptx.cuh"

#include <cstdlib>
#include <mutex>

namespace difb200 {

int encode_tensor_map(CUtensorMap *out, CUtensorMapDataType type, uint32_t rank, const void *base,
                      const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box,
                      CUtensorMapSwizzle swizzle) {
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                               const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                               const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult query;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &query) ==
            cudaSuccess &&
        query == cudaDriverEntryPointSuccess)
      encode = reinterpret_cast<EncodeFn>(fn);
  });
  if (!encode)
    return fail(kInternalError, "cuTensorMapEncodeTiled is unavailable in this driver");
  cuuint32_t elem_strides[5] = {1, 1, 1, 1, 1};
  cuuint64_t gdims[5];
  cuuint64_t gstrides[5];
  cuuint32_t gbox[5];
  for (uint32_t i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    if (i + 1 < rank)
      gstrides[i] = strides_bytes[i];
  }
  const CUresult rc = encode(out, type, rank, const_cast<void *>(base), gdims, gstrides, gbox,
                             elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS)
    return fail(kInvalidArgument, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)rc));
  return kOk;
}

namespace {

constexpr int kBM = 128, kBN = 256, kBK = 128; // per-CTA rows, tile columns, BK in bytes == INT8 elements
constexpr int kUmmaK = 32;
constexpr uint32_t kABytes = kBM * kBK;
constexpr int kThreads = 320;
constexpr int kEpilogueWarps = 8;
template <int CTAS>
struct Cfg {
  static constexpr int kStages = CTAS == 2 ? 5 : 4;
  // staging boxes per epilogue warp (two let a TMA store drain while the next box is filled;
  // the single-CTA form has room for one)
  static constexpr uint32_t kBoxes = CTAS == 2 ? 2 : 1;
  static constexpr uint32_t kStagingBytes = 8 /*epilogue warps*/ * kBoxes * 32 * 64;
  static constexpr uint32_t kBRows = kBN / CTAS;                 // rows of the B tile this CTA stages
  static constexpr uint32_t kBBytes = kBRows * kBK;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr uint32_t kTileM = kBM * CTAS;                 // rows of the (pair's) output tile
};
constexpr uint32_t kTmemCols = 512;
// Epilogue staging: per epilogue warp two [32 rows x 32 bf16] boxes (64-byte rows, 64B TMA
// swizzle); plus, per epilogue warp, 256 column scales and 256 biases (fp32) of the tile.
constexpr uint32_t kStoreBoxBytes = 32 * 64;
constexpr uint32_t kScaleBytes = kEpilogueWarps * 2 * (kBN / 2) * 4; // per warp: scales and biases of its 128 columns
template <int CTAS>
constexpr size_t smem_bytes() {
  return 1024 /*alignment slack*/ + (size_t)Cfg<CTAS>::kStages * Cfg<CTAS>::kStageBytes + Cfg<CTAS>::kStagingBytes +
         kScaleBytes + 256;
}

enum : uint32_t { kEpiBias = 1u, kEpiGeluTanh = 2u };

struct GemmParams {
  const float *row_scales;
  const float *col_scales;
  const uint16_t *bias;
  uint16_t *out;
  int32_t *acc_out;
  uint32_t M, N, K;
  uint32_t epilogue;
  uint32_t tma_store; // 1: outputs leave through TMA stores (needs N % 8 == 0, aligned out)
  uint32_t withhold_kb; // test aid: the loads of this k-block are never issued (0xffffffff = none)
  unsigned long long wait_ns; // limit of every bounded wait
  DeviceStatus *status;
};

__device__ __forceinline__ void report_timeout(DeviceStatus *status, uint32_t role, uint32_t detail) {
  if (atomicExch(&status->flag, 1u) == 0u) {
    status->kernel = 2u;
    status->role = role;
    status->detail = detail;
  }
}

__device__ __forceinline__ float gelu_tanh(float v) {
  // Reference form (cpu_executor.cpp:93-113): 0.5 * v * (1 + tanh(u)), u = 0.79788456 * (v +
  // 0.044715 * v^3). The reference's fp32 sum 1 + tanh(u) cancels for negative v, and that
  // rounding is part of its result, so the same three roundings are kept here and only tanh
  // itself is computed differently: tanh|u| = 1 - 2 / (e^(2|u|) + 1) with two MUFU ops
  // (ex2, rcp), absolute error below one ulp of 1.
  constexpr float kA = 0.7978845608028654f * 2.0f * 1.4426950408889634f;
  constexpr float kB = kA * 0.044715f;
  const float t = fmaf(kB, v * v, kA) * v; // 2u * log2(e), same sign as v
  float e, r;
  asm("ex2.approx.f32 %0, %1;" : "=f"(e) : "f"(fabsf(t)));
  asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(e + 1.0f));
  const float th = copysignf(fmaf(-2.0f, r, 1.0f), v);
  return __fmul_rn(__fmul_rn(0.5f, v), __fadd_rn(1.0f, th));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t packed;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
  return packed;
}

template <int CTAS>
__global__ void __launch_bounds__(kThreads, 1)
gemm_i8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_c, const GemmParams p) {
  constexpr int kStages = Cfg<CTAS>::kStages;
  constexpr uint32_t kStageBytes = Cfg<CTAS>::kStageBytes;
  constexpr uint32_t kTileM = Cfg<CTAS>::kTileM;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t cta_rank = CTAS == 2 ? ptx::cluster_ctarank() : 0u;  // 0 = leader of the pair
  const uint32_t unit = CTAS == 2 ? blockIdx.x >> 1 : blockIdx.x;      // tile-scheduling unit
  const uint32_t units = CTAS == 2 ? gridDim.x >> 1 : gridDim.x;
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t staging_base = smem_base + kStages * kStageBytes;
  const uint32_t scale_base = staging_base + Cfg<CTAS>::kStagingBytes;
  const uint32_t bar_base = scale_base + kScaleBytes;
  // barrier layout (8 bytes each): full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]; then a word
  // for the TMEM base address and a word for the abort flag.
  const uint32_t full_bar = bar_base, empty_bar = bar_base + 8 * kStages;
  const uint32_t tfull_bar = bar_base + 16 * kStages, tempty_bar = tfull_bar + 16;
  const uint32_t tmem_slot = tempty_bar + 16;
  volatile uint32_t *slot_ptr =
      reinterpret_cast<volatile uint32_t *>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
  volatile uint32_t *abort_ptr = slot_ptr + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned long long wait_ns = p.wait_ns;
  const uint32_t tiles_m = (p.M + kTileM - 1) / kTileM, tiles_n = (p.N + kBN - 1) / kBN;
  const uint32_t num_tiles = tiles_m * tiles_n;
  const uint32_t k_blocks = (p.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar + 8 * s, 1);
      ptx::mbar_init(empty_bar + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(tfull_bar + 8 * b, 1);
      ptx::mbar_init(tempty_bar + 8 * b, kEpilogueWarps * CTAS);    // epilogue warps of every CTA of the pair
    }
    *abort_ptr = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
  }
  if (warp == 1) {
    if (CTAS == 2) {
      ptx::tmem_alloc_pair(tmem_slot, kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(tmem_slot, kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (CTAS == 2)
    ptx::cluster_sync(); // the peer's barriers are initialised before anything arrives on them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *slot_ptr;

  // The producer warp and the MMA warp run their loops with all 32 lanes and warp-uniform
  // control flow (every wait ends in a vote) and let one elected lane issue the asynchronous
  // instructions. Loop state, addresses and descriptors are then warp-uniform values; with a
  // single-lane loop (divergent code) every operand of every TMA / MMA instruction is first
  // moved between register files, and that loop needed 640-680 cycles per k-block against the
  // 512 cycles the four MMAs of a k-block take.
  auto give_up = [&](uint32_t role, uint32_t detail) {
    if (lane == 0) {
      if (!*abort_ptr)
        report_timeout(p.status, role, detail);
      *abort_ptr = 1;
    }
  };
  if (warp == 0) {
    uint32_t stage = 0, phase = 0;
    bool ok = true;
    for (uint32_t tile = unit; tile < num_tiles && ok; tile += units) {
      const int32_t m0 = (int32_t)((tile / tiles_n) * kTileM + cta_rank * kBM);
      const int32_t n0 = (int32_t)((tile % tiles_n) * kBN + cta_rank * Cfg<CTAS>::kBRows);
      for (uint32_t kb = 0; kb < k_blocks; ++kb) {
        if (!ptx::mbar_wait_warp(empty_bar + 8 * stage, phase ^ 1u, abort_ptr, wait_ns)) {
          give_up(0, kb);
          ok = false;
          break;
        }
        const uint32_t a_dst = smem_base + stage * kStageBytes, b_dst = a_dst + kABytes;
        const uint32_t bar = full_bar + 8 * stage;
        const int32_t k0 = (int32_t)(kb * kBK);
        if (kb == p.withhold_kb) {
          // test aid: the bytes are announced but never loaded, so the consumer's wait on this
          // stage runs out and the kernel leaves through its give-up path
          if (cta_rank == 0 && ptx::elect_one())
            ptx::mbar_expect_tx(bar, CTAS * kStageBytes);
        } else if (ptx::elect_one()) {
          if (CTAS == 2) {
            // A pair counts the bytes of both CTAs on the leader's barrier: the leader expects
            // them all, the peer's loads complete their bytes there (cta_group::2 form of the
            // load) and the peer itself never arrives.
            if (cta_rank == 0) {
              ptx::mbar_expect_tx(bar, 2 * kStageBytes);
              ptx::tma_load_2d(a_dst, &map_a, bar, k0, m0);
              ptx::tma_load_2d(b_dst, &map_b, bar, k0, n0);
            } else {
              const uint32_t leader_bar = ptx::mapa(bar, 0);
              ptx::tma_load_2d_pair(a_dst, &map_a, leader_bar, k0, m0);
              ptx::tma_load_2d_pair(b_dst, &map_b, leader_bar, k0, n0);
            }
          } else {
            ptx::mbar_expect_tx(bar, kStageBytes);
            ptx::tma_load_2d(a_dst, &map_a, bar, k0, m0);
            ptx::tma_load_2d(b_dst, &map_b, bar, k0, n0);
          }
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (cta_rank == 0) {
      constexpr uint32_t idesc = ptx::make_idesc(2 /*S32*/, 1 /*S8*/, 1 /*S8*/, 0, 0, kTileM, kBN);
      const uint64_t desc0 = ptx::smem_desc_sw128(smem_base, 16, 1024);
      uint32_t stage = 0, phase = 0, local = 0;
      bool ok = true;
      auto commit = [&](uint32_t bar) { // arrives on `bar` of every CTA of the pair
        if (CTAS == 2)
          ptx::mma_commit_pair_both(bar, (uint16_t)3);
        else
          ptx::mma_commit(bar);
      };
      for (uint32_t tile = unit; tile < num_tiles && ok; tile += units, ++local) {
        const uint32_t acc = local & 1u, acc_phase = (local >> 1) & 1u;
        if (!ptx::mbar_wait_warp(tempty_bar + 8 * acc, acc_phase ^ 1u, abort_ptr, wait_ns)) {
          give_up(1, 0xffffu);
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        for (uint32_t kb = 0; kb < k_blocks; ++kb) {
          if (!ptx::mbar_wait_warp(full_bar + 8 * stage, phase, abort_ptr, wait_ns)) {
            give_up(1, kb);
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          // descriptors of this stage: only the 14-bit address field (16-byte units) moves
          const uint64_t a_desc = desc0 + (uint64_t)((stage * kStageBytes) >> 4);
          const uint64_t b_desc = a_desc + (uint64_t)(kABytes >> 4);
          if (ptx::elect_one()) {
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              const uint32_t accumulate = k != 0 ? 1u : (kb != 0u ? 1u : 0u);
              if (CTAS == 2)
                ptx::mma_i8_ss_pair(d_tmem, a_desc + (uint64_t)(k * kUmmaK >> 4), b_desc + (uint64_t)(k * kUmmaK >> 4),
                                    idesc, accumulate);
              else
                ptx::mma_i8_ss(d_tmem, a_desc + (uint64_t)(k * kUmmaK >> 4), b_desc + (uint64_t)(k * kUmmaK >> 4),
                               idesc, accumulate);
            }
            commit(empty_bar + 8 * stage); // frees the smem stage when these MMAs retire
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok && ptx::elect_one())
          commit(tfull_bar + 8 * acc); // accumulator complete
      }
    }
  } else {
    const uint32_t quarter = (uint32_t)warp & 3u;        // TMEM lane quarter of this warp
    const uint32_t ewarp = (uint32_t)warp - 2u;          // 0..7
    const uint32_t col_half = ewarp >> 2;                // columns [128 col_half, 128 col_half + 128)
    uint32_t local = 0, store_buf = 0;
    uint8_t *generic_base = smem_raw + (smem_base - smem_u32(smem_raw));
    float *scale_smem = reinterpret_cast<float *>(generic_base + (scale_base - smem_base));
    const uint32_t my_staging = staging_base + ewarp * Cfg<CTAS>::kBoxes * kStoreBoxBytes;
    uint8_t *my_staging_ptr = generic_base + (my_staging - smem_base);
    for (uint32_t tile = unit; tile < num_tiles; tile += units, ++local) {
      const uint32_t acc = local & 1u, acc_phase = (local >> 1) & 1u;
      const uint32_t m0 = (tile / tiles_n) * kTileM + cta_rank * kBM, n0 = (tile % tiles_n) * kBN;
      // column scales and biases of this tile -> this warp's private shared-memory copy
      // (warp-private so that no cross-warp barrier is needed)
      float *cs = scale_smem + ewarp * kBN, *bs = cs + kBN / 2; // this warp's 128 columns
      __syncwarp();
#pragma unroll
      for (int i = 0; i < kBN / 64; ++i) {
        const uint32_t c = lane + 32u * i, n = n0 + col_half * (kBN / 2) + c;
        cs[c] = n < p.N ? __ldg(p.col_scales + n) : 0.0f;
        bs[c] = ((p.epilogue & kEpiBias) && n < p.N) ? bf16_bits_to_f32(__ldg(p.bias + n)) : 0.0f;
      }
      __syncwarp();
      if (*abort_ptr || !ptx::mbar_wait(tfull_bar + 8 * acc, acc_phase, wait_ns)) {
        if (!*abort_ptr && lane == 0)
          report_timeout(p.status, 2, tile);
        *abort_ptr = 1;
        break;
      }
      ptx::tc_fence_after();
      const uint32_t row = m0 + quarter * 32u + lane;
      const bool row_ok = row < p.M;
      const float rs = row_ok ? __ldg(p.row_scales + row) : 0.0f;
#pragma unroll 1
      for (uint32_t sub = 0; sub < kBN / 64; ++sub) {
        const uint32_t chunk = col_half * (kBN / 64) + sub; // 32-column chunk of the tile
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + ((quarter * 32u) << 16) + acc * kBN + chunk * 32u, r);
        ptx::tmem_ld_wait();
        const uint32_t n_base = n0 + chunk * 32u;
        if (n_base >= p.N)
          continue; // (warp-uniform) whole chunk past the N edge
        if (p.acc_out && row_ok) {
          for (int i = 0; i < 32; ++i)
            if (n_base + i < p.N)
              p.acc_out[(size_t)row * p.N + n_base + i] = (int32_t)r[i];
        }
        uint32_t packed[16];
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const float4 c4 = *reinterpret_cast<const float4 *>(cs + sub * 32 + 4 * g);
          const float4 b4 = *reinterpret_cast<const float4 *>(bs + sub * 32 + 4 * g);
          const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, bb[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int i = 4 * g + 2 * h;
            float y0 = __fmul_rn(__fmul_rn((float)(int32_t)r[i], rs), cc[2 * h]);
            float y1 = __fmul_rn(__fmul_rn((float)(int32_t)r[i + 1], rs), cc[2 * h + 1]);
            uint32_t pk = pack_bf16x2(y0, y1);
            if (p.epilogue & kEpiBias) {
              y0 = __fadd_rn(__uint_as_float(pk << 16), bb[2 * h]);
              y1 = __fadd_rn(__uint_as_float(pk & 0xffff0000u), bb[2 * h + 1]);
              pk = pack_bf16x2(y0, y1);
            }
            if (p.epilogue & kEpiGeluTanh) {
              y0 = gelu_tanh(__uint_as_float(pk << 16));
              y1 = gelu_tanh(__uint_as_float(pk & 0xffff0000u));
              pk = pack_bf16x2(y0, y1);
            }
            packed[i >> 1] = pk;
          }
        }
        if (p.tma_store) {
          // stage this warp's [32 x 32] box (64-byte rows, 16-byte chunk c of row r stored at
          // c ^ ((r >> 1) & 3): the 64B TMA swizzle, conflict-free), then one TMA store.
          if (lane == 0) { // the box about to be filled must have been read by its last store
            if (Cfg<CTAS>::kBoxes == 2)
              asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            else
              asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
          __syncwarp();
          uint8_t *box = my_staging_ptr + store_buf * kStoreBoxBytes;
#pragma unroll
          for (int v = 0; v < 4; ++v)
            *reinterpret_cast<uint4 *>(box + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) =
                make_uint4(packed[4 * v], packed[4 * v + 1], packed[4 * v + 2], packed[4 * v + 3]);
          ptx::fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                             reinterpret_cast<uint64_t>(&map_c)),
                         "r"(my_staging + store_buf * kStoreBoxBytes), "r"((int32_t)n_base),
                         "r"((int32_t)(m0 + quarter * 32u))
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          store_buf = Cfg<CTAS>::kBoxes == 2 ? store_buf ^ 1u : 0u;
        } else if (row_ok) {
          uint16_t *dst = p.out + (size_t)row * p.N + n_base;
          for (int i = 0; i < 32; ++i)
            if (n_base + i < p.N)
              dst[i] = (uint16_t)((packed[i >> 1] >> (16 * (i & 1))) & 0xffffu);
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CTAS == 2)
          ptx::mbar_arrive_remote(ptx::mapa(tempty_bar + 8 * acc, 0)); // the leader issues the MMAs
        else
          ptx::mbar_arrive(tempty_bar + 8 * acc);
      }
    }
    if (lane == 0)
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (CTAS == 2)
    ptx::cluster_sync(); // neither CTA leaves (or frees TMEM) while the peer may still touch it
  if (warp == 1) {
    ptx::tc_fence_after();
    if (CTAS == 2)
      ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    else
      ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
}

} // namespace

int linear_int8_scaled(const int8_t *x, const int8_t *w, const float *row_scales,
                       const float *col_scales, const void *bias_bf16, uint32_t epilogue, uint64_t M,
                       uint64_t N, uint64_t K, void *out_bf16, int32_t *acc_out, cudaStream_t stream,
                       DeviceStatus *status_words) {
  if (!x || !w || !row_scales || !col_scales || !out_bf16)
    return fail(kInvalidArgument, "LinearInt8Scaled: null pointer");
  if ((epilogue & kEpiBias) && !bias_bf16)
    return fail(kInvalidArgument, "LinearInt8Scaled: bias epilogue without a bias pointer");
  if (epilogue & ~(kEpiBias | kEpiGeluTanh))
    return fail(kInvalidArgument, "LinearInt8Scaled: unknown epilogue flags");
  if (M == 0 || N == 0)
    return kOk;
  if (K == 0 || K % 16 != 0)
    return fail(kUnsupported, "LinearInt8Scaled: K must be a positive multiple of 16 (TMA row pitch)");
  if (M > 0x7fffffffull || N > 0x7fffffffull || K > 0x7fffffffull)
    return fail(kUnsupported, "LinearInt8Scaled: dimension too large");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15))
    return fail(kUnsupported, "LinearInt8Scaled: operands must be 16-byte aligned");
  DeviceStatus *status = status_words ? status_words : device_status_words();
  if (!status)
    return fail(kOutOfMemory, "LinearInt8Scaled: cannot allocate device status words");

  // Form: the CTA-pair kernel moves a third less through shared memory per MAC and is the faster
  // one whenever its 256x256 tiles fill the machine as well as 128x256 tiles do; the choice
  // compares the number of tile waves (a pair wave costs about 0.94 of a single-CTA wave).
  // DIFB200_GEMM_CTAS=1|2 forces a form (both give identical bits).
  const uint64_t pair_tiles = ((M + 255) / 256) * ((N + kBN - 1) / kBN);
  const uint64_t single_tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
  const uint64_t sms = (uint64_t)sm_count();
  const uint64_t single_waves = (single_tiles + sms - 1) / sms, pair_waves = (pair_tiles + sms / 2 - 1) / (sms / 2);
  int ctas = (M > (uint64_t)kBM && 94 * pair_waves <= 100 * single_waves) ? 2 : 1;
  if (const char *force = std::getenv("DIFB200_GEMM_CTAS"))
    ctas = force[0] == '2' ? 2 : (force[0] == '1' ? 1 : ctas);
  CUtensorMap map_a, map_b;
  const uint64_t dims_a[2] = {K, M}, dims_b[2] = {K, N};
  const uint64_t strides[1] = {K};
  const uint32_t box_a[2] = {(uint32_t)kBK, (uint32_t)kBM}, box_b[2] = {(uint32_t)kBK, (uint32_t)(kBN / ctas)};
  if (int rc = encode_tensor_map(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, x, dims_a, strides, box_a,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  if (int rc = encode_tensor_map(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w, dims_b, strides, box_b,
                                 CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;

  const bool tma_store = (N % 8 == 0) && ((reinterpret_cast<uintptr_t>(out_bf16) & 15) == 0);
  CUtensorMap map_c = map_a; // placeholder when stores go out directly
  if (tma_store) {
    const uint64_t dims_c[2] = {N, M};
    const uint64_t strides_c[1] = {N * 2};
    const uint32_t box_c[2] = {32, 32};
    if (int rc = encode_tensor_map(&map_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, out_bf16, dims_c,
                                   strides_c, box_c, CU_TENSOR_MAP_SWIZZLE_64B))
      return rc;
  }

  // The dynamic shared-memory opt-in is an attribute of the function in one context, so it is
  // made once per device (a process may hold plugin contexts on several GPUs).
  static const char attr_key = 0;
  if (int rc = current_device_once(&attr_key, [](void *, int *) -> int {
        if (int rc = check_cuda(cudaFuncSetAttribute(gemm_i8_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     (int)smem_bytes<1>()),
                                "cudaFuncSetAttribute(gemm_i8_kernel<1>)"))
          return rc;
        return check_cuda(cudaFuncSetAttribute(gemm_i8_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)smem_bytes<2>()),
                          "cudaFuncSetAttribute(gemm_i8_kernel<2>)");
      }, nullptr, nullptr))
    return rc;

  GemmParams p{};
  p.row_scales = row_scales;
  p.col_scales = col_scales;
  p.bias = static_cast<const uint16_t *>(bias_bf16);
  p.out = static_cast<uint16_t *>(out_bf16);
  p.acc_out = acc_out;
  p.M = (uint32_t)M;
  p.N = (uint32_t)N;
  p.K = (uint32_t)K;
  p.epilogue = epilogue;
  p.tma_store = tma_store ? 1u : 0u;
  p.withhold_kb = take_withheld_gemm_load();
  p.wait_ns = wait_limit_ns();
  p.status = status;
  if (ctas == 2) {
    cudaLaunchConfig_t config{};
    config.gridDim = dim3((unsigned)sm_count());
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = smem_bytes<2>();
    config.stream = stream;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    config.attrs = &attr;
    config.numAttrs = 1;
    // The kernel is persistent: launch exactly as many CTA pairs as can be resident at once
    // (SM pairs are formed inside a GPC, so this can be fewer than SMs / 2); a per-device figure.
    static const char pairs_key = 0;
    int resident_pairs = 0;
    if (int rc = current_device_once(&pairs_key, [](void *arg, int *value) -> int {
          int n = 0;
          if (int rc = check_cuda(cudaOccupancyMaxActiveClusters(&n, gemm_i8_kernel<2>,
                                                                 static_cast<cudaLaunchConfig_t *>(arg)),
                                  "cudaOccupancyMaxActiveClusters"))
            return rc;
          *value = n > 0 ? n : 1;
          return kOk;
        }, &config, &resident_pairs))
      return rc;
    uint64_t pairs = (uint64_t)resident_pairs;
    if (pairs > pair_tiles)
      pairs = pair_tiles;
    config.gridDim = dim3((unsigned)(2 * pairs));
    return launched(cudaLaunchKernelEx(&config, gemm_i8_kernel<2>, map_a, map_b, map_c, p),
                      "gemm_i8_kernel<2> launch");
  }
  const uint64_t tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
  uint64_t grid = (uint64_t)sm_count();
  if (grid > tiles)
    grid = tiles;
  gemm_i8_kernel<1><<<(unsigned)grid, kThreads, smem_bytes<1>(), stream>>>(map_a, map_b, map_c, p);
  return launched(cudaGetLastError(), "gemm_i8_kernel launch");
}

} // namespace difb200
