// extern "C" surface of libdifb200.so for device-resident callers (see difb200/difb200.h).
#include "difb200/difb200.h"

#include "common.cuh"
#include "glue.h"
#include "ops.h"
#include "world.h"
#include "diffir.h"

#include <string>
#include <thread>
#include <vector>

using namespace difb200;

namespace difb200 {

int w8a8_linear(const void *x_bf16, const int8_t *w, const float *col_scales, const void *bias_bf16,
                uint32_t epilogue, int implementation, float clip, uint64_t M, uint64_t N, uint64_t K,
                int8_t *codes_scratch, float *scales_scratch, void *out_bf16, cudaStream_t stream,
                DeviceStatus *status_words) {
  if (!x_bf16 || !codes_scratch || !scales_scratch)
    return fail(kInvalidArgument, "w8a8_linear: null input or scratch pointer");
  const void *parts[1] = {x_bf16};
  const uint64_t widths[1] = {K};
  if (int rc = quantize_int8_rows(parts, widths, 1, M, implementation, clip, nullptr, codes_scratch,
                                  scales_scratch, nullptr, nullptr, stream))
    return rc;
  return linear_int8_scaled(codes_scratch, w, scales_scratch, col_scales, bias_bf16, epilogue, M, N, K,
                            out_bf16, nullptr, stream, status_words);
}

namespace {
size_t align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }
} // namespace

size_t attention_scratch_bytes(uint64_t B, uint64_t S, uint64_t H, uint64_t KV) {
  return align256(B * S * H * 128) + align256(B * S * KV * 128) + align256(B * S * H * 4) +
         align256(B * S * KV * 4) + align256(attention_int8_scratch_bytes(B, S, KV));
}

AttentionScratch attention_scratch_layout(void *scratch, uint64_t B, uint64_t S, uint64_t H, uint64_t KV) {
  unsigned char *base = static_cast<unsigned char *>(scratch);
  AttentionScratch l{};
  l.q8 = reinterpret_cast<int8_t *>(base);
  base += align256(B * S * H * 128);
  l.k8 = reinterpret_cast<int8_t *>(base);
  base += align256(B * S * KV * 128);
  l.qs = reinterpret_cast<float *>(base);
  base += align256(B * S * H * 4);
  l.ks = reinterpret_cast<float *>(base);
  base += align256(B * S * KV * 4);
  l.rest = base;
  return l;
}

// q / k null: their codes and scales are already in the scratch buffer (attention_scratch_layout).
int attention_bf16_via_int8(const void *q, const void *k, const void *v, const uint8_t *key_valid, uint64_t B,
                            uint64_t S, uint64_t H, uint64_t KV, uint64_t D, float scale, void *scratch,
                            size_t scratch_bytes, void *out_bf16, cudaStream_t stream) {
  if (D != 128)
    return fail(kUnsupported, "Attention(INT8): head dimension must be 128");
  if (!scratch || scratch_bytes < attention_scratch_bytes(B, S, H, KV))
    return fail(kInvalidArgument, "Attention(INT8): scratch buffer too small");
  const AttentionScratch l = attention_scratch_layout(scratch, B, S, H, KV);
  const void *qp[1] = {q}, *kp[1] = {k};
  const uint64_t w[1] = {128};
  if (q)
    if (int rc = quantize_int8_rows(qp, w, 1, B * S * H, 1, 1.0f, nullptr, l.q8, l.qs, nullptr, nullptr, stream))
      return rc;
  if (k)
    if (int rc = quantize_int8_rows(kp, w, 1, B * S * KV, 1, 1.0f, nullptr, l.k8, l.ks, nullptr, nullptr, stream))
      return rc;
  return attention_int8(l.q8, l.qs, l.k8, l.ks, v, key_valid, B, S, S, H, KV, D, scale, l.rest,
                        attention_int8_scratch_bytes(B, S, KV), out_bf16, stream);
}

} // namespace difb200

extern "C" {

const char *difb200_last_error(void) { return last_error().c_str(); }

int difb200_version(void) { return 3; }

uint64_t difb200_launch_count(void) { return launch_count(); }

int difb200_poll_status(void) {
  if (int rc = check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize"))
    return rc;
  return poll_device_status("difb200_poll_status");
}

void difb200_set_wait_limit_ns(uint64_t nanoseconds) { set_wait_limit_ns(nanoseconds); }

void difb200_test_withhold_gemm_load(uint32_t k_block) { withhold_next_gemm_load(k_block); }

int difb200_program_check(const uint8_t *diffir, uint64_t size) {
  ir::Program program;
  std::string text;
  const int rc = ir::decode(diffir, (size_t)size, program, text);
  return rc ? fail(rc, "DiffIR: " + text) : kOk;
}

int difb200_selftest_host(void) {
  // per_device_once: one initialisation per (key, device ordinal), failures are not cached
  static const char key_a = 0, key_b = 0;
  struct Counter {
    int calls = 0, fail_first = 0;
  };
  auto init = [](void *arg, int *value) -> int {
    Counter *c = static_cast<Counter *>(arg);
    ++c->calls;
    if (c->fail_first && c->calls == 1)
      return kExecutionError;
    *value = 100 + c->calls;
    return kOk;
  };
  Counter a, b;
  int v = 0;
  // ordinals far above any real device, so nothing a real launch cached is touched
  if (per_device_once(&key_a, 1000, init, &a, &v) != kOk || v != 101 || a.calls != 1)
    return fail(kInternalError, "selftest: first use on a device did not initialise");
  if (per_device_once(&key_a, 1000, init, &a, &v) != kOk || v != 101 || a.calls != 1)
    return fail(kInternalError, "selftest: second use on the same device initialised again");
  if (per_device_once(&key_a, 1001, init, &a, &v) != kOk || v != 102 || a.calls != 2)
    return fail(kInternalError, "selftest: another device did not get its own initialisation");
  b.fail_first = 1;
  if (per_device_once(&key_b, 1000, init, &b, &v) == kOk)
    return fail(kInternalError, "selftest: a failing initialisation was reported as success");
  if (per_device_once(&key_b, 1000, init, &b, &v) != kOk || v != 102 || b.calls != 2)
    return fail(kInternalError, "selftest: a failed initialisation was cached");
  // the wait limit and the withheld-load test aid are plain host state
  const unsigned long long before = wait_limit_ns();
  set_wait_limit_ns(12345);
  const bool limit_ok = wait_limit_ns() == 12345;
  set_wait_limit_ns(0);
  const bool default_ok = wait_limit_ns() == 1500ull * 1000ull * 1000ull;
  set_wait_limit_ns(before);
  withhold_next_gemm_load(3);
  const bool armed = take_withheld_gemm_load() == 3u, disarmed = take_withheld_gemm_load() == 0xffffffffu;
  if (!limit_ok || !default_ok || !armed || !disarmed)
    return fail(kInternalError, "selftest: wait limit or withheld-load state misbehaves");
  return kOk;
}

int difb200_quantize_int8_rows(const void *const *parts, const uint64_t *part_widths,
                               uint32_t part_count, uint64_t rows, int32_t implementation,
                               float clip, const float *clip_device, int8_t *codes, float *scales,
                               int8_t *residual_codes, float *residual_scales, void *stream) {
  if (!parts || !part_widths)
    return fail(kInvalidArgument, "difb200_quantize_int8_rows: null part arrays");
  return quantize_int8_rows(parts, part_widths, part_count, rows, implementation, clip, clip_device,
                            codes, scales, residual_codes, residual_scales,
                            static_cast<cudaStream_t>(stream));
}

int difb200_rms_norm_modulate_quant(const void *x, const void *weight, const void *scale, const void *shift,
                                    uint64_t rows, uint64_t columns, float epsilon, int32_t implementation,
                                    float clip, int8_t *codes, float *row_scales, void *stream) {
  if (!x || !scale || !shift)
    return fail(kInvalidArgument, "difb200_rms_norm_modulate_quant: null pointer");
  const void *parts[1] = {x};
  const uint64_t widths[1] = {columns};
  const NormPrologue norm{weight, scale, shift, epsilon};
  return quantize_int8_rows(parts, widths, 1, rows, implementation, clip, nullptr, codes, row_scales, nullptr, nullptr,
                            static_cast<cudaStream_t>(stream), false, nullptr, &norm);
}

int difb200_layer_norm_modulate_quant(const void *x, const void *weight, const void *bias, const void *scale,
                                      const void *shift, uint64_t rows, uint64_t columns, uint64_t rows_per_modulation,
                                      float epsilon, int32_t implementation, float clip, int8_t *codes,
                                      float *row_scales, void *stream) {
  if (!x || !weight || !bias || !scale || !shift)
    return fail(kInvalidArgument, "difb200_layer_norm_modulate_quant: null pointer");
  if (rows_per_modulation == 0 || rows % rows_per_modulation != 0)
    return fail(kInvalidArgument, "difb200_layer_norm_modulate_quant: rows must be a multiple of rows_per_modulation");
  const void *parts[1] = {x};
  const uint64_t widths[1] = {columns};
  const NormPrologue norm{weight, scale, shift, epsilon, bias, rows_per_modulation};
  return quantize_int8_rows(parts, widths, 1, rows, implementation, clip, nullptr, codes, row_scales, nullptr, nullptr,
                            static_cast<cudaStream_t>(stream), false, nullptr, &norm);
}

int difb200_quantize_weight_rows(const void *weight, const void *input_scale, uint64_t rows, uint64_t columns,
                                 int32_t implementation, int32_t mse_scale, int8_t *codes, float *scales,
                                 void *stream) {
  if (!weight)
    return fail(kInvalidArgument, "difb200_quantize_weight_rows: null weight");
  const void *parts[1] = {weight};
  const uint64_t widths[1] = {columns};
  return quantize_int8_rows(parts, widths, 1, rows, implementation, 1.0f, nullptr, codes, scales, nullptr, nullptr,
                            static_cast<cudaStream_t>(stream), mse_scale != 0, input_scale);
}

int difb200_linear_int8_scaled(const int8_t *x, const int8_t *w, const float *row_scales,
                               const float *col_scales, const void *bias, uint32_t epilogue,
                               uint64_t M, uint64_t N, uint64_t K, void *out, int32_t *acc_out,
                               void *stream) {
  return linear_int8_scaled(x, w, row_scales, col_scales, bias, epilogue, M, N, K, out, acc_out,
                            static_cast<cudaStream_t>(stream));
}

uint64_t difb200_attention_int8_scratch_bytes(uint64_t B, uint64_t S, uint64_t KV) {
  return attention_int8_scratch_bytes(B, S, KV);
}

int difb200_attention_int8(const int8_t *q8, const float *qs, const int8_t *k8, const float *ks,
                           const void *v, const uint8_t *key_valid, uint64_t B, uint64_t Sq, uint64_t Sk,
                           uint64_t H, uint64_t KV, uint64_t D, float scale, void *scratch,
                           uint64_t scratch_bytes, void *out, void *stream) {
  return attention_int8(q8, qs, k8, ks, v, key_valid, B, Sq, Sk, H, KV, D, scale, scratch, scratch_bytes, out,
                        static_cast<cudaStream_t>(stream));
}

uint64_t difb200_attention_int8_state_bytes(uint64_t B, uint64_t Sq, uint64_t H) {
  return attention_int8_state_bytes(B, Sq, H);
}

int difb200_attention_int8_chunk(const int8_t *q8, const float *qs, const int8_t *k8, const float *ks,
                                 const void *v, const uint8_t *key_valid, uint64_t B, uint64_t Sq, uint64_t Sk,
                                 uint64_t H, uint64_t KV, uint64_t D, float scale, void *scratch,
                                 uint64_t scratch_bytes, void *out, const uint32_t *tile_ranges,
                                 int32_t carry_in, int32_t carry_out, void *state, void *stream) {
  if (!tile_ranges)
    return fail(kInvalidArgument, "difb200_attention_int8_chunk: null tile ranges");
  AttentionChunk chunk{};
  chunk.tile_begin[0] = tile_ranges[0];
  chunk.tile_count[0] = tile_ranges[1];
  chunk.tile_begin[1] = tile_ranges[2];
  chunk.tile_count[1] = tile_ranges[3];
  chunk.carry_in = carry_in != 0;
  chunk.carry_out = carry_out != 0;
  chunk.state = state;
  return attention_int8(q8, qs, k8, ks, v, key_valid, B, Sq, Sk, H, KV, D, scale, scratch, scratch_bytes, out,
                        static_cast<cudaStream_t>(stream), &chunk);
}

// ---- multi-GPU world ----
int difb200_world_unique_id(uint8_t *id128) {
  if (!id128)
    return fail(kInvalidArgument, "difb200_world_unique_id: null pointer");
  return world_unique_id(id128);
}

int difb200_world_create(const uint8_t *id128, int32_t rank, int32_t size, void **world) {
  if (!world)
    return fail(kInvalidArgument, "difb200_world_create: null pointer");
  World *w = nullptr;
  const int rc = world_create(id128, rank, size, &w);
  *world = w;
  return rc;
}

int difb200_world_destroy(void *world) {
  delete static_cast<World *>(world);
  return kOk;
}

int difb200_world_rendezvous(const char *directory, int32_t rank, int32_t size, uint8_t *id128, uint32_t timeout_ms) {
  if (!directory)
    return fail(kInvalidArgument, "difb200_world_rendezvous: null directory");
  return world_rendezvous(directory, rank, size, id128, timeout_ms);
}

int difb200_world_exchange(void *world, int32_t which, void *const *buffers, const uint64_t *slice_bytes,
                           int32_t count, void *producer_stream) {
  return world_exchange_class(static_cast<World *>(world), which, buffers, slice_bytes, count,
                              static_cast<cudaStream_t>(producer_stream));
}

int difb200_world_bind(void *world, uint64_t payload_bytes, void *stream, void **binding, void **block,
                       int32_t *direct) {
  if (!binding || !block || !direct)
    return fail(kInvalidArgument, "difb200_world_bind: null pointer");
  PeerBinding *b = nullptr;
  const int rc = world_bind(static_cast<World *>(world), (size_t)payload_bytes, static_cast<cudaStream_t>(stream), &b);
  *binding = b;
  *block = b ? b->block : nullptr;
  *direct = b && b->direct ? 1 : 0;
  return rc;
}

int difb200_world_unbind(void *world, void *binding) {
  return world_unbind(static_cast<World *>(world), static_cast<PeerBinding *>(binding));
}

int difb200_world_push(void *world, void *binding, int32_t which, const uint64_t *offsets, const uint64_t *slice_bytes,
                       int32_t count, void *producer_stream) {
  return world_push(static_cast<World *>(world), static_cast<PeerBinding *>(binding), which, offsets, slice_bytes, count,
                    static_cast<cudaStream_t>(producer_stream));
}

int difb200_world_selftest_flags(uint64_t limit_ns, int32_t set) { return world_selftest_flags(limit_ns, set != 0); }

int difb200_sharded_attention(void *world, void *binding, const int8_t *q8, const float *qs, const int8_t *k8,
                              const float *ks, const void *v, const uint8_t *key_valid, uint64_t Sq,
                              uint64_t slice_tokens, uint64_t H, uint64_t KV, float scale, void *scratch,
                              uint64_t scratch_bytes, void *state, void *out, void *stream) {
  return sharded_attention(static_cast<World *>(world), static_cast<PeerBinding *>(binding), q8, qs, k8, ks, v,
                           key_valid, Sq, slice_tokens, H, KV, scale, scratch, scratch_bytes, state, out,
                           static_cast<cudaStream_t>(stream));
}

int difb200_world_plan(int32_t rank, int32_t size, uint32_t tiles_per_slice, const int32_t *group_sizes,
                       int32_t group_count, uint32_t *tile_ranges, int32_t *first_step, int32_t *step_count,
                       int32_t capacity, int32_t *launches) {
  if (!tile_ranges || !first_step || !step_count || !launches || (group_count > 0 && !group_sizes))
    return fail(kInvalidArgument, "difb200_world_plan: null pointer");
  std::vector<int> groups(group_sizes, group_sizes + (group_count > 0 ? group_count : 0));
  std::vector<LaunchPlan> plans;
  if (!plan_launches(rank, size, tiles_per_slice, groups, plans))
    return fail(kInvalidArgument, "difb200_world_plan: the group sizes must be positive and sum to the world size");
  if ((int)plans.size() > capacity)
    return fail(kInvalidArgument, "difb200_world_plan: output arrays are too small");
  *launches = (int32_t)plans.size();
  for (size_t i = 0; i < plans.size(); ++i) {
    tile_ranges[4 * i] = plans[i].tile_begin[0];
    tile_ranges[4 * i + 1] = plans[i].tile_count[0];
    tile_ranges[4 * i + 2] = plans[i].tile_begin[1];
    tile_ranges[4 * i + 3] = plans[i].tile_count[1];
    first_step[i] = plans[i].steps.front();
    step_count[i] = (int32_t)plans[i].steps.size();
  }
  return kOk;
}

int difb200_world_selftest_fake(int32_t size, int32_t missing_rank, uint32_t timeout_ms) {
  // `size` ranks as threads of this process exchange two host buffers (different slice sizes)
  // through the host-memory transport with the schedule the GPUs use. With missing_rank >= 0 that
  // rank never shows up: every other rank must come back with an execution error by the deadline.
  if (size < 1 || size > 64)
    return fail(kInvalidArgument, "selftest: 1..64 ranks");
  FakeFabric *fabric = fake_fabric_create(size, timeout_ms);
  const uint64_t slices[2] = {96, 40};
  std::vector<int> status((size_t)size, -1);
  std::vector<std::string> text((size_t)size);
  std::vector<std::vector<unsigned char>> a((size_t)size), b((size_t)size);
  auto fill = [](int rank, int buffer, uint64_t i) { return (unsigned char)(17 * rank + 5 * buffer + i); };
  std::vector<std::thread> threads;
  for (int r = 0; r < size; ++r) {
    if (r == missing_rank)
      continue;
    threads.emplace_back([&, r] {
      World world;
      world.rank = r;
      world.size = size;
      world.transport = fake_transport(fabric, r);
      a[(size_t)r].assign((size_t)(size * slices[0]), 0);
      b[(size_t)r].assign((size_t)(size * slices[1]), 0);
      for (uint64_t i = 0; i < slices[0]; ++i)
        a[(size_t)r][(size_t)(r * slices[0] + i)] = fill(r, 0, i);
      for (uint64_t i = 0; i < slices[1]; ++i)
        b[(size_t)r][(size_t)(r * slices[1] + i)] = fill(r, 1, i);
      void *buffers[2] = {a[(size_t)r].data(), b[(size_t)r].data()};
      status[(size_t)r] = world_exchange(&world, buffers, slices, 2, nullptr, nullptr);
      text[(size_t)r] = last_error();
    });
  }
  for (auto &t : threads)
    t.join();
  fake_fabric_destroy(fabric);
  for (int r = 0; r < size; ++r) {
    if (r == missing_rank)
      continue;
    if (missing_rank >= 0) {
      if (status[(size_t)r] != kExecutionError)
        return fail(kInternalError, "selftest: rank " + std::to_string(r) + " did not report the missing rank");
      continue;
    }
    if (status[(size_t)r] != kOk)
      return fail(kInternalError, "selftest: rank " + std::to_string(r) + " failed: " + text[(size_t)r]);
    for (int src = 0; src < size; ++src) {
      for (uint64_t i = 0; i < slices[0]; ++i)
        if (a[(size_t)r][(size_t)(src * slices[0] + i)] != fill(src, 0, i))
          return fail(kInternalError, "selftest: wrong bytes in the first buffer");
      for (uint64_t i = 0; i < slices[1]; ++i)
        if (b[(size_t)r][(size_t)(src * slices[1] + i)] != fill(src, 1, i))
          return fail(kInternalError, "selftest: wrong bytes in the second buffer");
    }
  }
  return kOk;
}

uint64_t difb200_attention_scratch_bytes(uint64_t B, uint64_t S, uint64_t H, uint64_t KV) {
  return attention_scratch_bytes(B, S, H, KV);
}

int difb200_attention(const void *q, const void *k, const void *v, const uint8_t *key_valid, uint64_t B,
                      uint64_t S, uint64_t H, uint64_t KV, uint64_t D, float scale, void *scratch,
                      uint64_t scratch_bytes, void *out, void *stream) {
  if (!q || !k)
    return fail(kInvalidArgument, "difb200_attention: null pointer");
  return attention_bf16_via_int8(q, k, v, key_valid, B, S, H, KV, D, scale, scratch, scratch_bytes, out,
                                 static_cast<cudaStream_t>(stream));
}

int difb200_rms_norm_modulate(const void *x, const void *weight, const void *scale, const void *shift, void *out,
                              uint32_t dtype, uint64_t rows, uint64_t cols, float epsilon, void *stream) {
  if (!x || !scale || !shift || !out || dtype < 1 || dtype > 3)
    return fail(kInvalidArgument, "difb200_rms_norm_modulate: bad argument");
  return glue::rms_norm_modulate(x, weight, scale, shift, out, dtype, rows, cols, epsilon, 0.0f, false, 1,
                                 static_cast<cudaStream_t>(stream));
}

int difb200_layer_norm_modulate(const void *x, const void *weight, const void *bias, const void *scale,
                                const void *shift, void *out, uint32_t dtype, uint64_t rows, uint64_t cols,
                                uint64_t modulation_rows, float epsilon, void *stream) {
  if (!x || !weight || !bias || !scale || !shift || !out || dtype < 1 || dtype > 3 || modulation_rows == 0 ||
      rows % modulation_rows != 0)
    return fail(kInvalidArgument, "difb200_layer_norm_modulate: bad argument");
  return glue::layer_norm_modulate(x, weight, bias, scale, shift, out, dtype, rows, cols, rows / modulation_rows,
                                   epsilon, static_cast<cudaStream_t>(stream));
}

int difb200_qk_norm_rope(const void *x, const void *weight, const void *cosine, const void *sine, void *out,
                         uint32_t dtype, uint32_t table_dtype, uint64_t tokens, uint64_t heads, uint64_t dim,
                         uint64_t rotary, uint64_t table_width, uint64_t input_sequence, uint64_t table_sequence,
                         uint64_t table_start, float epsilon, int32_t interleaved_v2, void *stream) {
  if (!x || !weight || !cosine || !sine || !out || dtype < 1 || dtype > 3 || table_dtype < 1 || table_dtype > 3 ||
      rotary > dim || (rotary & 1) || (table_width != rotary && table_width != rotary / 2) || input_sequence == 0 ||
      table_start + input_sequence > table_sequence)
    return fail(kInvalidArgument, "difb200_qk_norm_rope: bad argument");
  return glue::qk_norm_rope(x, weight, cosine, sine, out, dtype, table_dtype, tokens, heads, dim, rotary, table_width,
                            input_sequence, table_sequence, table_start, epsilon, interleaved_v2 != 0,
                            static_cast<cudaStream_t>(stream));
}

int difb200_qk_norm_rope_quant(const void *x, const void *weight, const void *cosine, const void *sine, void *out,
                               int8_t *codes, float *scales, uint32_t table_dtype, uint64_t tokens, uint64_t heads,
                               uint64_t rotary, uint64_t table_width, uint64_t input_sequence,
                               uint64_t table_sequence, uint64_t table_start, float epsilon, int32_t interleaved_v2,
                               void *stream) {
  if (!x || !weight || !cosine || !sine || (!out && !codes) || (codes && !scales) || rotary > 128 || (rotary & 1) ||
      input_sequence == 0 || table_start + input_sequence > table_sequence)
    return fail(kInvalidArgument, "difb200_qk_norm_rope_quant: bad argument");
  int rc = 0;
  if (!glue::qk_norm_rope_fast(x, weight, cosine, sine, out, codes, scales, 2, table_dtype, tokens, heads, 128, rotary,
                               table_width, input_sequence, table_sequence, table_start, epsilon,
                               interleaved_v2 != 0, nullptr, static_cast<cudaStream_t>(stream), &rc))
    return fail(kUnsupported, "difb200_qk_norm_rope_quant: needs bf16 rows of 128, rotary 64 / 96 / 128, bf16 or "
                              "f32 tables whose rows are multiples of 16 bytes, 16-byte aligned pointers");
  return rc;
}

int difb200_residual_gate(const void *residual, const void *branch, const void *gate, void *out, uint32_t dtype,
                          uint64_t rows, uint64_t width, uint64_t gate_rows, void *stream) {
  if (!residual || !branch || !gate || !out || dtype < 1 || dtype > 3 || gate_rows == 0 || rows % gate_rows != 0)
    return fail(kInvalidArgument, "difb200_residual_gate: bad argument");
  return glue::residual_gate(residual, branch, gate, out, dtype, rows * width, width, rows / gate_rows,
                             static_cast<cudaStream_t>(stream));
}

int difb200_swiglu(const void *x, void *out, uint32_t dtype, uint64_t rows, uint64_t width, uint64_t input_width,
                   uint64_t start, int32_t gate_first, void *stream) {
  if (!x || !out || dtype < 1 || dtype > 3 || start + 2 * width > input_width)
    return fail(kInvalidArgument, "difb200_swiglu: bad argument");
  return glue::swiglu(x, out, dtype, rows, width, input_width, start, gate_first != 0,
                      static_cast<cudaStream_t>(stream));
}

int difb200_w8a8_linear(const void *x, const int8_t *w, const float *col_scales, const void *bias,
                        uint32_t epilogue, int32_t implementation, float clip, uint64_t M, uint64_t N,
                        uint64_t K, int8_t *codes_scratch, float *scales_scratch, void *out,
                        void *stream) {
  return w8a8_linear(x, w, col_scales, bias, epilogue, implementation, clip, M, N, K, codes_scratch,
                     scales_scratch, out, static_cast<cudaStream_t>(stream));
}

}
