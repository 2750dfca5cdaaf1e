// TEST INFRASTRUCTURE ONLY. Never linked into, loaded by, or called from the
// product library.
//
// A thin C interface over the reference project's own CPU executor and plugin
// host, compiled against the reference sources where they lie (see Makefile in
// this directory; nothing of the reference is copied into this repository).
// It exists so that parity tests, fixture generation and the CPU baseline leg
// of the benchmark can run the *real* reference arithmetic:
//
//   difref_run          -> dif::ir::decode + dif::runtime::make_cpu_executor()
//                          (src/ir/codec.cpp:407-476, src/runtime/cpu_executor.cpp:2913-3016)
//   difref_run_plugin   -> dif::backend::make_plugin_executor(path)
//                          (src/backend/plugin.cpp:60-117,306-309): the reference's own
//                          dlopen loader driving a backend plugin .so
//   difref_encode_check -> round-trips DIFIR bytes through the reference decoder/encoder
//
// Tensors cross this interface as plain host buffers.
#include "dif/backend/plugin.hpp"
#include "dif/ir/codec.hpp"
#include "dif/ir/ir.hpp"
#include "dif/ir/verify.hpp"
#include "dif/runtime/executor.hpp"
#include "dif/runtime/tensor.hpp"

#include <cstdint>
#include <cstring>
#include <exception>
#include <memory>
#include <span>
#include <string>
#include <vector>

extern "C" {

typedef struct difref_view {
  uint32_t tensor_id;
  void *data;
  uint64_t byte_count;
} difref_view;

}

namespace {

void set_error(char *err, size_t cap, const std::string &text) {
  if (!err || cap == 0U)
    return;
  const auto n = text.size() < cap - 1U ? text.size() : cap - 1U;
  std::memcpy(err, text.data(), n);
  err[n] = '\0';
}

int run_with(dif::runtime::Executor &executor, const uint8_t *diffir, size_t n,
             const difref_view *bound, size_t bound_count, difref_view *outputs,
             size_t output_count, uint32_t warmups, uint32_t iterations,
             double *mean_ms, char *err, size_t errcap) {
  const auto program = dif::ir::decode(std::span<const uint8_t>(diffir, n));
  dif::runtime::TensorMap bindings;
  for (size_t i = 0; i < bound_count; ++i) {
    const auto *desc = program.tensor(bound[i].tensor_id);
    if (!desc)
      throw std::runtime_error("bound tensor id is not in the program");
    if (desc->byte_count() != bound[i].byte_count)
      throw std::runtime_error("bound tensor byte count mismatch for id " +
                               std::to_string(bound[i].tensor_id));
    dif::runtime::Tensor tensor{desc->dtype, desc->dims, {}};
    tensor.bytes.assign(static_cast<const uint8_t *>(bound[i].data),
                        static_cast<const uint8_t *>(bound[i].data) +
                            bound[i].byte_count);
    bindings.emplace(desc->id, std::move(tensor));
  }
  dif::runtime::RunOptions options;
  options.warmups = warmups;
  options.iterations = iterations;
  options.minimum_free_bytes = 0U;
  const auto result = executor.run(program, bindings, options);
  for (size_t i = 0; i < output_count; ++i) {
    const auto it = result.outputs.find(outputs[i].tensor_id);
    if (it == result.outputs.end())
      throw std::runtime_error("requested output is not produced: id " +
                               std::to_string(outputs[i].tensor_id));
    if (it->second.byte_size() != outputs[i].byte_count)
      throw std::runtime_error("output byte count mismatch for id " +
                               std::to_string(outputs[i].tensor_id));
    std::memcpy(outputs[i].data, it->second.data(), outputs[i].byte_count);
  }
  if (mean_ms)
    *mean_ms = result.mean_milliseconds;
  (void)err;
  (void)errcap;
  return 0;
}

} // namespace

extern "C" {

// Runs a DIFIR001-encoded program on the reference CPU executor. `bound` carries every
// Input- and Constant-role tensor. Returns 0 on success, 1 with text in `err` otherwise.
__attribute__((visibility("default"))) int
difref_run(const uint8_t *diffir, size_t n, const difref_view *bound,
           size_t bound_count, difref_view *outputs, size_t output_count,
           uint32_t warmups, uint32_t iterations, double *mean_ms, char *err,
           size_t errcap) {
  try {
    auto executor = dif::runtime::make_cpu_executor();
    return run_with(*executor, diffir, n, bound, bound_count, outputs,
                    output_count, warmups, iterations, mean_ms, err, errcap);
  } catch (const std::exception &e) {
    set_error(err, errcap, e.what());
    return 1;
  }
}

// Same program, but executed by the reference's plugin host on the backend plugin at
// `plugin_path` (the reference's --backend-plugin route).
__attribute__((visibility("default"))) int
difref_run_plugin(const char *plugin_path, int device, const uint8_t *diffir,
                  size_t n, const difref_view *bound, size_t bound_count,
                  difref_view *outputs, size_t output_count, uint32_t warmups,
                  uint32_t iterations, double *mean_ms, char *err,
                  size_t errcap) {
  try {
    auto executor = dif::backend::make_plugin_executor(plugin_path, device);
    return run_with(*executor, diffir, n, bound, bound_count, outputs,
                    output_count, warmups, iterations, mean_ms, err, errcap);
  } catch (const std::exception &e) {
    set_error(err, errcap, e.what());
    return 1;
  }
}

// Decodes (and thereby verifies) DIFIR bytes with the reference decoder and re-encodes
// them; returns 0 when the re-encoding is byte-identical to the input.
__attribute__((visibility("default"))) int
difref_encode_check(const uint8_t *diffir, size_t n, char *err, size_t errcap) {
  try {
    const auto program = dif::ir::decode(std::span<const uint8_t>(diffir, n));
    const auto again = dif::ir::encode(program);
    if (again.size() != n || std::memcmp(again.data(), diffir, n) != 0) {
      set_error(err, errcap, "re-encoded bytes differ");
      return 2;
    }
    return 0;
  } catch (const std::exception &e) {
    set_error(err, errcap, e.what());
    return 1;
  }
}

}

// ---- the reference's own SafeTensors reader / writer and program fingerprint, for the cache
// interoperability tests (src/weights/safetensors.cpp, src/ir/codec.cpp:494-497) ----
#include "dif/weights/safetensors.hpp"

extern "C" {

__attribute__((visibility("default"))) int
difref_fingerprint(const uint8_t *diffir, size_t n, uint8_t *digest32, char *err, size_t errcap) {
  try {
    const auto program = dif::ir::decode(std::span<const uint8_t>(diffir, n));
    const auto digest = dif::ir::fingerprint(program);
    std::memcpy(digest32, digest.data(), 32);
    return 0;
  } catch (const std::exception &e) {
    set_error(err, errcap, e.what());
    return 1;
  }
}

// Writes `count` tensors with the reference's SafeTensorWriter. dims holds 8 entries per tensor.
__attribute__((visibility("default"))) int
difref_write_safetensors(const char *path, size_t count, const char *const *names, const uint32_t *dtypes,
                         const uint32_t *ranks, const uint64_t *dims, const void *const *data,
                         const uint64_t *byte_counts, char *err, size_t errcap) {
  try {
    std::vector<dif::weights::SafeTensorWriteSpec> specs;
    for (size_t i = 0; i < count; ++i)
      specs.push_back({names[i], static_cast<dif::ir::DType>(dtypes[i]),
                       std::vector<std::uint64_t>(dims + 8 * i, dims + 8 * i + ranks[i])});
    dif::weights::SafeTensorWriter writer(path, specs);
    for (size_t i = 0; i < count; ++i)
      writer.append(names[i], std::span<const std::uint8_t>(static_cast<const std::uint8_t *>(data[i]),
                                                            static_cast<size_t>(byte_counts[i])));
    (void)writer.finish();
    return 0;
  } catch (const std::exception &e) {
    set_error(err, errcap, e.what());
    return 1;
  }
}

// Reads one tensor with the reference's reader; returns its description and copies its bytes.
__attribute__((visibility("default"))) int
difref_read_safetensor(const char *path, const char *name, uint32_t *dtype, uint32_t *rank, uint64_t *dims8,
                       void *out, uint64_t capacity, uint64_t *byte_count, char *err, size_t errcap) {
  try {
    const auto file = dif::weights::read_safetensors(path);
    const auto tensor = dif::weights::map_safetensor(file, name);
    *dtype = static_cast<uint32_t>(tensor.dtype);
    *rank = static_cast<uint32_t>(tensor.dims.size());
    for (size_t i = 0; i < tensor.dims.size() && i < 8; ++i)
      dims8[i] = tensor.dims[i];
    *byte_count = tensor.byte_size();
    if (tensor.byte_size() > capacity)
      throw std::runtime_error("output buffer too small");
    std::memcpy(out, tensor.data(), tensor.byte_size());
    return 0;
  } catch (const std::exception &e) {
    set_error(err, errcap, e.what());
    return 1;
  }
}

}
