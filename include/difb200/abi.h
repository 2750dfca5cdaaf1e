/*
 * Backend plugin C-ABI of Diffusion Compiler, versions 1 and 2, as implemented by
 * libdifb200.so. This header restates the interface of the reference's
 * include/dif/backend/abi.h (structure layouts, enum values and symbol names have to be
 * identical for the reference's loader, src/backend/plugin.cpp:60-117, to drive this library);
 * tests/test_abi_and_symbols.py checks every size and offset against the reference header.
 *
 * Contract (reference abi.h:121-126, plugin.cpp:119-283):
 *   create(device_ordinal)            -> context (one CUDA device, one stream)
 *   compile (v2)                      -> decodes + verifies DIFIR001 bytes, copies every
 *                                        Constant-role tensor (passed in program order) to the
 *                                        device, plans buffers and kernels -> executable
 *   compile (v1)                      -> same without constants; they then arrive with every
 *                                        execute call after the Input-role tensors
 *   execute                           -> copies Input-role tensors host->device, runs
 *                                        `warmups` untimed + `iterations` timed passes (CUDA
 *                                        events; copies excluded, like the reference's OpenCL
 *                                        plugin, backends/opencl/opencl_backend.cpp:1369-1389),
 *                                        copies Output-role tensors device->host
 *   errors                            -> status code + NUL-terminated text in error->data
 * All pointers in tensor views are host pointers borrowed for the duration of the call.
 * Lifetimes: destroy every executable before the context it was compiled in (the reference's
 * host does, src/backend/plugin.cpp:96-99,186-191); an executable runs on its context's streams.
 */
#ifndef DIFB200_ABI_H
#define DIFB200_ABI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DIF_BACKEND_ABI_VERSION_V1 1U
#define DIF_BACKEND_ABI_VERSION_V2 2U
#define DIF_BACKEND_EXPORT __attribute__((visibility("default")))

typedef enum dif_backend_status {
  DIF_BACKEND_OK = 0,
  DIF_BACKEND_INVALID_ARGUMENT = 1,
  DIF_BACKEND_UNSUPPORTED = 2,
  DIF_BACKEND_OUT_OF_MEMORY = 3,
  DIF_BACKEND_COMPILE_ERROR = 4,
  DIF_BACKEND_EXECUTION_ERROR = 5,
  DIF_BACKEND_INTERNAL_ERROR = 6
} dif_backend_status;

typedef enum dif_backend_capability {
  DIF_BACKEND_CAP_F32 = 1ULL << 0U,
  DIF_BACKEND_CAP_BF16 = 1ULL << 1U,
  DIF_BACKEND_CAP_F16 = 1ULL << 2U,
  DIF_BACKEND_CAP_I8 = 1ULL << 3U,
  DIF_BACKEND_CAP_TRAINING = 1ULL << 4U,
  DIF_BACKEND_CAP_ASYNC = 1ULL << 5U
} dif_backend_capability;

typedef struct dif_backend_error {
  char *data;
  size_t capacity;
} dif_backend_error;

typedef struct dif_backend_tensor_view {
  uint32_t tensor_id;
  uint32_t dtype;
  uint32_t rank;
  const uint64_t *dims;
  void *host_data;
  uint64_t byte_count;
} dif_backend_tensor_view;

typedef struct dif_backend_run_options {
  uint32_t warmups;
  uint32_t iterations;
  uint64_t minimum_free_bytes;
} dif_backend_run_options;

typedef struct dif_backend_telemetry {
  double mean_milliseconds;
  double minimum_milliseconds;
  double maximum_milliseconds;
  uint64_t free_bytes_before;
  uint64_t free_bytes_after;
  char device_name[256];
} dif_backend_telemetry;

typedef void *dif_backend_context;
typedef void *dif_backend_executable;

typedef struct dif_backend_api_v1 {
  uint32_t struct_size;
  uint32_t abi_version;
  const char *backend_name;
  uint64_t capabilities;
  dif_backend_status (*create)(int32_t device_ordinal, dif_backend_context *context,
                               dif_backend_error *error);
  void (*destroy)(dif_backend_context context);
  dif_backend_status (*compile)(dif_backend_context context, const uint8_t *diffir,
                                size_t diffir_size, dif_backend_executable *executable,
                                dif_backend_error *error);
  void (*destroy_executable)(dif_backend_executable executable);
  dif_backend_status (*execute)(dif_backend_executable executable,
                                const dif_backend_tensor_view *inputs, size_t input_count,
                                dif_backend_tensor_view *outputs, size_t output_count,
                                const dif_backend_run_options *options,
                                dif_backend_telemetry *telemetry, dif_backend_error *error);
} dif_backend_api_v1;

DIF_BACKEND_EXPORT const dif_backend_api_v1 *dif_backend_get_v1(void);

typedef enum dif_backend_compile_flag {
  DIF_BACKEND_COMPILE_COPY_CONSTANTS = 1ULL << 0U
} dif_backend_compile_flag;

typedef struct dif_backend_compile_options_v2 {
  uint64_t minimum_free_bytes;
  uint64_t flags;
} dif_backend_compile_options_v2;

typedef struct dif_backend_compile_telemetry_v2 {
  double preparation_milliseconds;
  uint64_t resident_bytes;
  uint64_t free_bytes_before;
  uint64_t free_bytes_after;
  char device_name[256];
} dif_backend_compile_telemetry_v2;

typedef struct dif_backend_api_v2 {
  uint32_t struct_size;
  uint32_t abi_version;
  const char *backend_name;
  uint64_t capabilities;
  dif_backend_status (*create)(int32_t device_ordinal, dif_backend_context *context,
                               dif_backend_error *error);
  void (*destroy)(dif_backend_context context);
  dif_backend_status (*compile)(dif_backend_context context, const uint8_t *diffir,
                                size_t diffir_size, const dif_backend_tensor_view *constants,
                                size_t constant_count,
                                const dif_backend_compile_options_v2 *options,
                                dif_backend_executable *executable,
                                dif_backend_compile_telemetry_v2 *telemetry,
                                dif_backend_error *error);
  void (*destroy_executable)(dif_backend_executable executable);
  dif_backend_status (*execute)(dif_backend_executable executable,
                                const dif_backend_tensor_view *dynamic_inputs,
                                size_t dynamic_input_count, dif_backend_tensor_view *outputs,
                                size_t output_count, const dif_backend_run_options *options,
                                dif_backend_telemetry *telemetry, dif_backend_error *error);
} dif_backend_api_v2;

DIF_BACKEND_EXPORT const dif_backend_api_v2 *dif_backend_get_v2(void);

#ifdef __cplusplus
}
#endif

#endif /* DIFB200_ABI_H */
