/*
 * difb200: device-resident C entry points of the B200 (sm_100a) implementation of the
 * quantized DiT hot path of Diffusion Compiler.
 *
 * The drop-in boundary towards the reference project is its backend plugin ABI, restated in
 * difb200/abi.h and exported by the same shared library (dif_backend_get_v2 / _v1). That ABI
 * only moves host buffers, so the entry points below expose the same operators on device
 * pointers for callers that keep tensors resident in HBM (the plugin itself is built on them).
 *
 * Conventions: every function returns a status whose values equal dif_backend_status
 * (0 = OK, 1 = invalid argument, 2 = unsupported, 3 = out of memory, 5 = execution error);
 * difb200_last_error() returns the text of the calling thread's last failure. All pointers
 * are device pointers on the current CUDA device unless stated otherwise. `stream` is a
 * cudaStream_t passed as void* (NULL = default stream). Work is asynchronous: kernels are
 * enqueued and the call returns. There is no CPU fallback.
 */
#ifndef DIFB200_H
#define DIFB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DIFB200_EXPORT __attribute__((visibility("default")))

/* Epilogue ops fused after LinearInt8Scaled (each keeps the bf16 rounding of the separate op). */
#define DIFB200_EPILOGUE_BIAS 1u      /* BiasAdd: y = bf16(y + bias[n]) */
#define DIFB200_EPILOGUE_GELU_TANH 2u /* Gelu, tanh form: y = bf16(gelu(y)) */

DIFB200_EXPORT const char *difb200_last_error(void);
DIFB200_EXPORT int difb200_version(void);
/* Kernels of this library launched by this process so far (every entry point and the plugin count). */
DIFB200_EXPORT uint64_t difb200_launch_count(void);

/*
 * Reads and clears the device-side status words. Kernels with bounded waits (mbarrier spins)
 * record there when a wait ran out instead of hanging; returns 5 with text in that case.
 * Synchronises the device.
 */
DIFB200_EXPORT int difb200_poll_status(void);

/*
 * Limit, in nanoseconds of wall time, after which a bounded device-side wait gives up (default
 * 1.5 s; 0 restores the default). Read at every kernel launch of this process. A kernel whose
 * wait ran out frees what it holds, returns, and leaves status 5 for difb200_poll_status (the
 * plugin's execute reports it as DIF_BACKEND_EXECUTION_ERROR); the context stays usable.
 */
DIFB200_EXPORT void difb200_set_wait_limit_ns(uint64_t nanoseconds);

/*
 * Test aid, not for production use: the next difb200_linear_int8_scaled launch announces but
 * never issues the loads of k-block `k_block` (K / 128 blocks per tile), so that the wait on
 * that stage runs out and the give-up path can be exercised with a short wait limit. The
 * result of that launch is undefined. Disarms itself after one launch.
 */
DIFB200_EXPORT void difb200_test_withhold_gemm_load(uint32_t k_block);

/*
 * Host-only self-check of the library's per-device bookkeeping (one-time set-up keyed by device
 * ordinal, wait-limit state). Touches no GPU; returns 0 when the invariants hold.
 */
DIFB200_EXPORT int difb200_selftest_host(void);

/*
 * Decodes and verifies DIFIR bytes on the host exactly as the plugin's compile does (container:
 * magic, version, trailing SHA-256, counts; program rules: unique ids, operands defined before use,
 * roles; per-operator shape and attribute rules of the operators this backend runs; reference
 * src/ir/codec.cpp:370-476, src/ir/verify.cpp). 0 = compile would accept the program's form,
 * 1 = malformed or invalid, 2 = well-formed but uses an operator or form this backend does not
 * implement; text for difb200_last_error(). Needs no GPU.
 */
DIFB200_EXPORT int difb200_program_check(const uint8_t *diffir, uint64_t size);

/*
 * Opcode QuantizeInt8Rows (67). Replaces the reference CPU op
 * src/runtime/cpu_executor.cpp:124-307 and its generated CUDA kernel
 * src/compiler/compiler.cpp:635-845 (semantics: include/dif/ir/ir.hpp:123-134,285-293;
 * verifier src/ir/verify.cpp:949-1027).
 *   parts / part_widths : HOST arrays of `part_count` (1..8) device pointers to bf16 tensors
 *                         [rows, part_widths[i]] that are concatenated on the last axis.
 *   implementation      : Int8RowQuantization, 1 = Direct .. 7 = H4096F32SignedConvRot.
 *   clip                : static Scale attribute in (0,1]; clip_device, if not NULL, is the
 *                         F32[1] dynamic clip input and wins.
 *   codes [rows, sum(widths)] int8, scales [rows] f32; residual_codes / residual_scales are
 *   the optional second pair (both NULL or both set).
 * ConvRot variants need widths that are multiples of 16 and 16-byte aligned pointers.
 */
DIFB200_EXPORT int difb200_quantize_int8_rows(const void *const *parts, const uint64_t *part_widths,
                                              uint32_t part_count, uint64_t rows,
                                              int32_t implementation, float clip,
                                              const float *clip_device, int8_t *codes,
                                              float *scales, int8_t *residual_codes,
                                              float *residual_scales, void *stream);

/*
 * RmsNormModulate (ExplicitScaleShift layout, src/runtime/cpu_executor.cpp:1241-1264) and
 * QuantizeInt8Rows (a 256-wide ConvRot variant, static clip) in one kernel: the bf16 tensor between
 * the two ops is never written. The reference runs them as two ops on its generic path and has a
 * fused producer of its own for one model (src/runtime/cuda_executor.cpp:5417-5466). x, scale,
 * shift: bf16 [rows, columns]; weight: bf16 [columns] or NULL. The row statistic is summed in
 * parallel, as in difb200_rms_norm_modulate (a different order than there, so the two forms agree
 * to the last bit of the statistic, not beyond).
 */
DIFB200_EXPORT int difb200_rms_norm_modulate_quant(const void *x, const void *weight, const void *scale,
                                                   const void *shift, uint64_t rows, uint64_t columns,
                                                   float epsilon, int32_t implementation, float clip,
                                                   int8_t *codes, float *row_scales, void *stream);

/*
 * LayerNormModulate (src/runtime/cpu_executor.cpp:1108-1148: affine layer norm, then
 * (1 + scale) * h + shift with the reference's intermediate bf16 roundings) and QuantizeInt8Rows
 * (a 256-wide ConvRot variant, static clip) in one kernel. x: bf16 [rows, columns]; weight, bias:
 * bf16 [columns]; scale, shift: bf16 [rows / rows_per_modulation, columns] (one modulation row per
 * batch item). Mean and centred second moment are parallel sums, as in
 * difb200_layer_norm_modulate.
 */
DIFB200_EXPORT int difb200_layer_norm_modulate_quant(const void *x, const void *weight, const void *bias,
                                                     const void *scale, const void *shift, uint64_t rows,
                                                     uint64_t columns, uint64_t rows_per_modulation,
                                                     float epsilon, int32_t implementation, float clip,
                                                     int8_t *codes, float *row_scales, void *stream);

/*
 * Weight-side packing: the bf16 weight matrix [rows = N, columns = K] quantised row by row with
 * the same rotation and quantiser as the activations (clip 1), giving the I8 weight and the
 * per-output-channel scales that LinearInt8Scaled binds as constants. This is the encoder of the
 * reference's offline packer (tools/difflux2sample.cpp:2994-3059; GPU variant
 * tools/difh3convrot.cpp:364-446). mse_scale != 0 selects the row scale by the packer's MSE search
 * over seven clip factors on every fourth rotated element (tools/difflux2sample.cpp:1225-1259;
 * 256-wide ConvRot variants 2, 3, 5, 6 only); the stored scale is then the bf16-rounded one.
 * input_scale (may be NULL) is the packer's input-equalisation vector, bf16 [columns]
 * (:2967-2990: sqrt(column absmax / geometric mean of the column absmaxes), clamped to [0.5, 2]):
 * every weight is divided by its column's entry in fp32 before the rotation (:3005-3014), and the
 * activations are multiplied by the same vector at run time.
 */
DIFB200_EXPORT int difb200_quantize_weight_rows(const void *weight, const void *input_scale, uint64_t rows,
                                                uint64_t columns, int32_t implementation,
                                                int32_t mse_scale, int8_t *codes, float *scales,
                                                void *stream);

/*
 * Opcode LinearInt8Scaled (68), optionally fused with the BiasAdd (10) and Gelu (49, tanh)
 * ops that follow it in a W8A8-rewritten program. Replaces the reference CPU op
 * src/runtime/cpu_executor.cpp:309-335 and the CUTLASS Sm80 kernel
 * src/runtime/cutlass_gemm.cu:185-303,745-778 (BiasAdd: cpu_executor.cpp:1288-1296, Gelu:
 * :93-113).
 *   x [M,K] int8, w [N,K] int8, row_scales [M] f32, col_scales [N] f32, bias [N] bf16 or NULL,
 *   out [M,N] bf16: out = bf16((float(acc) * row_scales[m]) * col_scales[n]) then the epilogue.
 *   acc_out, if not NULL, additionally receives the raw INT32 accumulators [M,N] (checking aid).
 * K must be a multiple of 16; x and w 16-byte aligned.
 */
DIFB200_EXPORT int difb200_linear_int8_scaled(const int8_t *x, const int8_t *w,
                                              const float *row_scales, const float *col_scales,
                                              const void *bias, uint32_t epilogue, uint64_t M,
                                              uint64_t N, uint64_t K, void *out, int32_t *acc_out,
                                              void *stream);

/*
 * INT8 attention on quantised operands. Replaces the reference's sm_86-only INT8 lowering of
 * opcode Attention (8): src/runtime/h3_owned_attention.cu:955-1079 (host entry), kernels
 * :236-295 and :646-929; admission src/runtime/cuda_executor.cpp:3388-3391,10982-10993.
 * Semantics of the op: src/runtime/cpu_executor.cpp:1839-1910 (GQA: query head h reads kv head
 * h / (H / KV); a row whose keys are all masked yields zeros).
 *   q8 [B,Sq,H,128] int8 with qs [B,Sq,H] f32, k8 [B,Sk,KV,128] int8 with ks [B,Sk,KV] f32:
 *   codes and scales of QuantizeInt8Rows(Direct) on the bf16 tensors (one row per token-head);
 *   v [B,Sk,KV,128] bf16; key_valid [B,Sk] bytes or NULL (the Bool mask that
 *   BooleanMaskToBias(MaskQueries=false) would turn into a 0/-inf bias, cpu_executor.cpp:627-650);
 *   scale = AttentionScale (1/sqrt(128) by default); out [B,Sq,H,128] bf16.
 *   Sq == Sk for the DiffIR op; Sq < Sk is the token-sharded form, where a GPU holds the queries
 *   of its token slice and the all-gathered keys/values of the whole sequence.
 *   scratch: device buffer of difb200_attention_int8_scratch_bytes(B,Sk,KV) bytes.
 * Non-causal, head dimension 128 only; everything else returns status 2.
 */
DIFB200_EXPORT uint64_t difb200_attention_int8_scratch_bytes(uint64_t B, uint64_t S, uint64_t KV);
DIFB200_EXPORT int difb200_attention_int8(const int8_t *q8, const float *qs, const int8_t *k8,
                                          const float *ks, const void *v, const uint8_t *key_valid,
                                          uint64_t B, uint64_t Sq, uint64_t Sk, uint64_t H, uint64_t KV,
                                          uint64_t D, float scale, void *scratch,
                                          uint64_t scratch_bytes, void *out, void *stream);

/*
 * One launch of a chunked difb200_attention_int8 (no counterpart in the reference, which runs
 * on one device: include/dif/runtime/executor.hpp:683). It is the form the token-sharded block
 * uses: keys and values arrive from other GPUs one slice at a time, and attention over the
 * slices that are already here runs while the rest is in flight.
 *   tile_ranges = {begin0, count0, begin1, count1}: the launch covers the 128-key tiles
 *   [begin0, begin0 + count0) and [begin1, begin1 + count1) of the key axis (Sk rounded up to 128).
 *   carry_in != 0: start from the state an earlier launch left in `state`; carry_out != 0: leave
 *   the state there instead of writing `out`. state: difb200_attention_int8_state_bytes(B,Sq,H)
 *   bytes, 16-byte aligned (per query row: m, l and 128 unnormalised fp32 outputs).
 * A sequence of launches over disjoint tile ranges -- the first without carry_in, the last
 * without carry_out, all on one stream or ordered by events -- gives the result of the single
 * launch over all tiles up to the order of the fp32 sums (every m is an integer, so moving a row
 * to a larger m is an exact scaling by a power of two).
 */
DIFB200_EXPORT uint64_t difb200_attention_int8_state_bytes(uint64_t B, uint64_t Sq, uint64_t H);
DIFB200_EXPORT int difb200_attention_int8_chunk(const int8_t *q8, const float *qs, const int8_t *k8,
                                                const float *ks, const void *v, const uint8_t *key_valid,
                                                uint64_t B, uint64_t Sq, uint64_t Sk, uint64_t H,
                                                uint64_t KV, uint64_t D, float scale, void *scratch,
                                                uint64_t scratch_bytes, void *out,
                                                const uint32_t *tile_ranges, int32_t carry_in,
                                                int32_t carry_out, void *state, void *stream);

/*
 * The multi-GPU world of the token-sharded block (no counterpart in the reference, which runs one
 * device per executor: include/dif/runtime/executor.hpp:683). One process per GPU; rank r owns a
 * contiguous slice of the tokens; weights are replicated; the only exchange per block is that of
 * the INT8 key codes, their scales and the bf16 values: pushed into the peers' gather blocks by
 * copy-engine copies over NVLink where the blocks can be mapped into each other (CUDA IPC; the
 * default), else sent and received with NCCL, which also bootstraps the mapping (the NCCL library
 * is resolved with dlopen when a world is created: libnccl.so.2 or DIFB200_NCCL_LIBRARY).
 *   difb200_world_unique_id     rank 0 makes the 128-byte communicator id, which the host hands to
 *                               the other ranks by any means it has
 *   difb200_world_rendezvous    optional bounded meeting point in a directory shared by the ranks
 *                               (fresh per job): every rank checks in, rank 0 leaves the id, all wait
 *                               at most timeout_ms and get status 5 if a rank is missing, so that no
 *                               rank enters the unbounded communicator set-up alone
 *   difb200_world_create        communicator + a high-priority communication stream on the current
 *                               device; blocks until every rank has called it
 *   difb200_world_exchange      ring exchange of `count` gather buffers of class `which` (0 = values,
 *                               1 = key codes and scales): buffers[i] holds size * slice_bytes[i] bytes
 *                               and this rank's slice is final once the work enqueued on
 *                               producer_stream so far has run. Step s of size - 1 sends the own slice
 *                               to rank + s and receives that of rank - s; nothing is waited for here
 *   difb200_world_bind          collective: one zeroed device block of payload_bytes per rank for the
 *                               gather buffers (the caller places them at offsets that are the same on
 *                               every rank) and, unless DIFB200_EXCHANGE=nccl or a rank cannot export or
 *                               map, the peers' blocks mapped into this rank; *direct tells which (the
 *                               same on all ranks). difb200_world_unbind, collective too, frees it
 *   difb200_world_push          direct form of difb200_world_exchange for a block with *direct = 1: this
 *                               rank's slice of each buffer (offsets[i] in the block, slice_bytes[i] per
 *                               rank) is copied into every peer's block by the copy engines, in ring
 *                               order, each copy followed by the pass number in the peer's flag area;
 *                               a push of pass n to a peer first waits until that peer's attention of
 *                               pass n - 1 has read the slice it overwrites
 *   difb200_sharded_attention   this rank's queries q8 [Sq,H,128] / qs against the gather buffers k8
 *                               [size * slice_tokens, KV, 128], ks, v (slice_tokens a multiple of 128,
 *                               key_valid [size * slice_tokens] marks real tokens): a few launches of
 *                               difb200_attention_int8_chunk, the own slice first, each ordered behind
 *                               the ring steps it reads (DIFB200_ATTENTION_GROUPS="1,3,4" sets how many
 *                               steps each launch takes): by CUDA events with binding NULL (NCCL), by a
 *                               one-CTA kernel that waits for the pushed slices' flags with a direct
 *                               binding. Those waits are bounded by DIFB200_WORLD_TIMEOUT_MS (worlds
 *                               from the environment; 60 s otherwise): a slice that never arrives ends
 *                               in status 5 at the next difb200_poll_status, not in a hang.
 *                               world may be NULL (one rank)
 *   difb200_world_selftest_flags  the flag kernels on one device: a wait for a flag that is set (set = 1,
 *                               status 0) or that nothing sets (set = 0: gives up after limit_ns,
 *                               status 5), leaving the context usable
 *   difb200_world_plan          the launch plan itself (host only): tile ranges, first ring step and
 *                               number of steps of every launch
 * A rank that is lost while an NCCL exchange is in flight is not detected here (NCCL has no deadline
 * of its own); hosts that need that put a heartbeat in front of every step.
 */
DIFB200_EXPORT int difb200_world_unique_id(uint8_t *id128);
DIFB200_EXPORT int difb200_world_rendezvous(const char *directory, int32_t rank, int32_t size, uint8_t *id128,
                                            uint32_t timeout_ms);
DIFB200_EXPORT int difb200_world_create(const uint8_t *id128, int32_t rank, int32_t size, void **world);
DIFB200_EXPORT int difb200_world_destroy(void *world);
DIFB200_EXPORT int difb200_world_exchange(void *world, int32_t which, void *const *buffers,
                                          const uint64_t *slice_bytes, int32_t count, void *producer_stream);
DIFB200_EXPORT int difb200_world_bind(void *world, uint64_t payload_bytes, void *stream, void **binding, void **block,
                                      int32_t *direct);
DIFB200_EXPORT int difb200_world_unbind(void *world, void *binding);
DIFB200_EXPORT int difb200_world_push(void *world, void *binding, int32_t which, const uint64_t *offsets,
                                      const uint64_t *slice_bytes, int32_t count, void *producer_stream);
DIFB200_EXPORT int difb200_world_selftest_flags(uint64_t limit_ns, int32_t set);
DIFB200_EXPORT int difb200_sharded_attention(void *world, void *binding, const int8_t *q8, const float *qs,
                                             const int8_t *k8, const float *ks, const void *v,
                                             const uint8_t *key_valid, uint64_t Sq, uint64_t slice_tokens, uint64_t H,
                                             uint64_t KV, float scale, void *scratch, uint64_t scratch_bytes,
                                             void *state, void *out, void *stream);
DIFB200_EXPORT int difb200_world_plan(int32_t rank, int32_t size, uint32_t tiles_per_slice,
                                      const int32_t *group_sizes, int32_t group_count, uint32_t *tile_ranges,
                                      int32_t *first_step, int32_t *step_count, int32_t capacity,
                                      int32_t *launches);
/*
 * Host-only check of the exchange schedule: `size` ranks as threads of the calling process run
 * it over a host-memory transport and compare every gathered byte. With missing_rank >= 0 that
 * rank never joins and every other rank must return an execution error within timeout_ms.
 */
DIFB200_EXPORT int difb200_world_selftest_fake(int32_t size, int32_t missing_rank, uint32_t timeout_ms);

/*
 * Opcode Attention (8) on bf16 q [B,S,H,128], k/v [B,S,KV,128] in its INT8 lowering: q and k
 * are quantised per token-head (QuantizeInt8Rows Direct) into scratch, then
 * difb200_attention_int8 runs. scratch: difb200_attention_scratch_bytes(B,S,H,KV) bytes.
 */
DIFB200_EXPORT uint64_t difb200_attention_scratch_bytes(uint64_t B, uint64_t S, uint64_t H, uint64_t KV);
DIFB200_EXPORT int difb200_attention(const void *q, const void *k, const void *v,
                                     const uint8_t *key_valid, uint64_t B, uint64_t S, uint64_t H,
                                     uint64_t KV, uint64_t D, float scale, void *scratch,
                                     uint64_t scratch_bytes, void *out, void *stream);

/*
 * Block glue on device pointers: the row-local, memory-bound ops that sit between the quantized
 * linears and attention in a DiT block. dtype codes are DiffIR's (1 = F32, 2 = BF16, 3 = F16).
 * They follow the reference CPU executor's arithmetic and storage-dtype rounding points:
 *   difb200_rms_norm_modulate    RmsNormModulate, ExplicitScaleShift layout: out = rmsnorm(x) [* weight]
 *                                * (1 + scale) + shift with full-shape scale/shift
 *                                (src/runtime/cpu_executor.cpp:1241-1265); weight may be NULL
 *   difb200_layer_norm_modulate  LayerNormModulate (cpu_executor.cpp:1108-1148); scale/shift have
 *                                modulation_rows rows that broadcast over groups of input rows
 *   difb200_qk_norm_rope         QkNormPartialRope (cpu_executor.cpp:1741-1837); interleaved_v2 != 0
 *                                selects Implementation 2 with the interleaved layout, else half-split
 *   difb200_qk_norm_rope_quant   the same op on bf16 heads of 128 followed by QuantizeInt8Rows(Direct) of
 *                                its result (cpu_executor.cpp:124-307, Direct branch) in one kernel: the
 *                                producer of INT8 attention's q8/qs and k8/ks. out (the bf16 result) and
 *                                codes/scales are each optional. The reference runs these as two ops.
 *   difb200_residual_gate        ResidualGate (cpu_executor.cpp:1703-1719)
 *   difb200_swiglu               SwiGlu (cpu_executor.cpp:1267-1286)
 */
DIFB200_EXPORT int difb200_rms_norm_modulate(const void *x, const void *weight, const void *scale,
                                             const void *shift, void *out, uint32_t dtype, uint64_t rows,
                                             uint64_t cols, float epsilon, void *stream);
DIFB200_EXPORT int difb200_layer_norm_modulate(const void *x, const void *weight, const void *bias,
                                               const void *scale, const void *shift, void *out,
                                               uint32_t dtype, uint64_t rows, uint64_t cols,
                                               uint64_t modulation_rows, float epsilon, void *stream);
DIFB200_EXPORT int difb200_qk_norm_rope(const void *x, const void *weight, const void *cosine,
                                        const void *sine, void *out, uint32_t dtype, uint32_t table_dtype,
                                        uint64_t tokens, uint64_t heads, uint64_t dim, uint64_t rotary,
                                        uint64_t table_width, uint64_t input_sequence,
                                        uint64_t table_sequence, uint64_t table_start, float epsilon,
                                        int32_t interleaved_v2, void *stream);
DIFB200_EXPORT int difb200_qk_norm_rope_quant(const void *x, const void *weight, const void *cosine,
                                              const void *sine, void *out, int8_t *codes, float *scales,
                                              uint32_t table_dtype, uint64_t tokens, uint64_t heads,
                                              uint64_t rotary, uint64_t table_width,
                                              uint64_t input_sequence, uint64_t table_sequence,
                                              uint64_t table_start, float epsilon, int32_t interleaved_v2,
                                              void *stream);
DIFB200_EXPORT int difb200_residual_gate(const void *residual, const void *branch, const void *gate,
                                         void *out, uint32_t dtype, uint64_t rows, uint64_t width,
                                         uint64_t gate_rows, void *stream);
DIFB200_EXPORT int difb200_swiglu(const void *x, void *out, uint32_t dtype, uint64_t rows, uint64_t width,
                                  uint64_t input_width, uint64_t start, int32_t gate_first, void *stream);

/*
 * The W8A8 `int8-convrot` linear as one call: QuantizeInt8Rows(implementation, clip) on the bf16
 * activations x [M,K], then LinearInt8Scaled against w [N,K] / col_scales [N] and the optional
 * epilogue. This is the op pair the reference's W8A8 rewrite puts in place of a Linear
 * (tools/difflux2sample.cpp:2017-2069, 3187-3219) and what its CUDA executor runs as
 * launch() + launch_cutlass_int8_scaled_gemm (src/runtime/cuda_executor.cpp:10940-10960).
 * codes_scratch [M,K] int8 and scales_scratch [M] f32 are scratch buffers supplied by the
 * caller (they hold the activation codes and row scales between the two kernels).
 */
DIFB200_EXPORT int difb200_w8a8_linear(const void *x, const int8_t *w, const float *col_scales,
                                       const void *bias, uint32_t epilogue, int32_t implementation,
                                       float clip, uint64_t M, uint64_t N, uint64_t K,
                                       int8_t *codes_scratch, float *scales_scratch, void *out,
                                       void *stream);

/*
 * difb200_w8a8_linear with no allocation anywhere (no counterpart in the reference).
 * Same computation and arguments as difb200_w8a8_linear, but the activation codes, row scales
 * and the GEMM's status words live in a fixed 40 MiB array inside the library instead of
 * caller scratch, and neither this call nor anything it runs calls cudaMalloc/cudaFree. It is
 * for hosts that planned their device memory up front or must not trigger an allocation while
 * they run a layer. A call needs 256 + roundup(4*M, 256) + M*K bytes; larger problems are
 * rejected with status 2. The first call on a device resolves the array's address (make that
 * first call outside any stream capture); under CUDA's default lazy module loading it is also
 * the moment the 40 MiB are taken on that device, so a host that wants no allocation while it
 * serves calls once with M = 0 per device at start-up (nothing is launched, 0 is returned). The
 * address is cached per device for the life of the process: do not use this entry point after a
 * cudaDeviceReset. All calls share the array: calls that can overlap on the GPU race, so keep
 * them on one stream or order them. check_previous != 0 first synchronises `stream` and returns
 * status 5 (once; the words are cleared) if a bounded wait ran out in the previous call. Those
 * status words live in the static array, not where difb200_poll_status looks: a call with
 * M = 0 and check_previous != 0 is the poll of this entry point.
 */
DIFB200_EXPORT int difb200_w8a8_linear_static(const void *x, const int8_t *w, const float *col_scales,
                                              const void *bias, uint32_t epilogue,
                                              int32_t implementation, float clip, uint64_t M,
                                              uint64_t N, uint64_t K, void *out,
                                              int32_t check_previous, void *stream);

/*
 * ConvRot INT8 weight caches, the files the reference keeps quantised Linear weights in (host side
 * except for the builder). Container: SafeTensors exactly as the reference reads and writes it
 * (src/weights/safetensors.cpp). Forms: per-projection pairs "weight" I8 [N,K] + "scale" F32 [N]
 * (tools/difflux2sample.cpp:3079-3091) and the generic cache "linear.<weight tensor id>.weight" /
 * ".scale" with the identity record "__meta__.convrot_int8" I32[20] = {0x31525643 "CVR1", 1, 256,
 * projection count, 8 words of the program fingerprint, 8 words of the source index digest}
 * (src/runtime/cuda_executor.cpp:4266-4364, tools/difh3convrot.cpp:51,208-231).
 *   difb200_cache_open / _tensor / _close   read a file; `data` points into memory owned by the
 *                                           handle (valid until close); dtype is the DiffIR code
 *                                           (0 for a "__meta__." tensor of another type)
 *   difb200_cache_write                     write tensors (dims8: 8 entries per tensor) under
 *                                           "<path>.building", then rename; refuses to run over an
 *                                           unfinished file of that name
 *   difb200_program_fingerprint             SHA-256 of DIFIR bytes without their trailing digest
 *                                           (src/ir/codec.cpp:494-497)
 *   difb200_cvr1_identity / _check          make the identity record; check magic, version, group,
 *                                           fingerprint (diffir may be NULL) and projection count
 *   difb200_build_convrot_cache             quantise `count` bf16 [rows, columns] HOST weight matrices
 *                                           on the current GPU (H256ConvRot rows, clip 1: the encoder of
 *                                           tools/difh3convrot.cpp:364-446) and write the generic cache
 */
DIFB200_EXPORT int difb200_cache_open(const char *path, void **cache);
DIFB200_EXPORT int difb200_cache_close(void *cache);
DIFB200_EXPORT int difb200_cache_tensor(void *cache, const char *name, uint32_t *dtype, uint32_t *rank,
                                        uint64_t *dims8, const void **data, uint64_t *bytes);
DIFB200_EXPORT int difb200_cache_write(const char *path, uint32_t count, const char *const *names,
                                       const uint32_t *dtypes, const uint32_t *ranks, const uint64_t *dims8,
                                       const void *const *data);
DIFB200_EXPORT int difb200_program_fingerprint(const uint8_t *diffir, uint64_t size, uint8_t *digest32);
DIFB200_EXPORT void difb200_cvr1_identity(uint32_t projections, const uint8_t *program_digest32,
                                          const uint8_t *index_digest32, uint32_t *identity20);
DIFB200_EXPORT int difb200_cvr1_check(const uint32_t *identity20, const uint8_t *diffir, uint64_t size,
                                      uint32_t projections);
DIFB200_EXPORT int difb200_build_convrot_cache(const char *path, const uint8_t *diffir, uint64_t diffir_size,
                                               uint32_t count, const uint32_t *weight_ids,
                                               const void *const *host_weights_bf16, const uint64_t *rows,
                                               const uint64_t *columns, const uint8_t *index_digest32,
                                               void *stream);

/*
 * Measured INT8 tensor-core peak of the current device: one launch in which every SM (form 1) or
 * every resident CTA pair (form 2, cta_group::2) issues `mma_per_issuer` tcgen05.mma kind::i8
 * instructions of M128 (256) x N256 x K32 back to back on operands that stay in shared memory.
 * Best of three timed launches (CUDA events); *tops = 2 * MACs / time. Synchronises `stream`.
 * 8192 MMAs take about half a millisecond.
 */
DIFB200_EXPORT int difb200_measure_i8_mma_peak(int32_t ctas_per_mma, uint32_t mma_per_issuer, double *tops,
                                               double *milliseconds, void *stream);

/*
 * Per-opcode device time of a plugin executable (a dif_backend_executable of this library). With
 * DIFB200_PROFILE=1 in the environment at compile, execute() records a CUDA event on its kernel
 * stream in front of every step of its timed passes; this call returns, per DiffIR opcode, the
 * summed time between consecutive events and the number of steps, and clears the sums. It is how
 * the benchmark times the dominant kernel inside the timed region (the reference reports per-op
 * times from CUDA events the same way: src/runtime/cuda_executor.cpp:11139-11153). A token-sharded
 * executable with the direct exchange adds two entries, opcodes 0xF000 (values) and 0xF001 (keys):
 * the time the copies of its pushes took on the communication stream, and how many pushes
 * (warm-up passes included) that sums.
 */
DIFB200_EXPORT int difb200_executable_profile(void *executable, uint32_t *opcodes, double *milliseconds,
                                              uint64_t *steps, uint32_t capacity, uint32_t *count);

/*
 * How a token-sharded executable of the plugin moves its key / value slices: 0 = it is not sharded
 * (one rank), 1 = NCCL send / receive (difb200_last_error() then holds why the direct form was not
 * set up), 2 = direct pushes into peer-mapped gather blocks.
 */
DIFB200_EXPORT int difb200_executable_exchange(void *executable);

#ifdef __cplusplus
}
#endif

#endif /* DIFB200_H */
