// Host-side helpers shared by the difb200 entry points: error text, CUDA status mapping,
// the per-device status words that kernels with bounded waits report through.
#include "common.cuh"

#include <atomic>
#include <map>
#include <mutex>
#include <unordered_map>
#include <utility>

namespace difb200 {

namespace {
thread_local std::string g_last_error;
std::mutex g_mutex;
std::unordered_map<int, DeviceStatus *> g_status_words;
std::unordered_map<int, int> g_sm_counts;
std::mutex g_once_mutex;
std::map<std::pair<const void *, int>, int> g_once_values;
} // namespace

namespace {
std::atomic<unsigned long long> g_wait_limit_ns{1500ull * 1000ull * 1000ull};
std::atomic<uint32_t> g_withhold_kb{0xffffffffu};
} // namespace

unsigned long long wait_limit_ns() { return g_wait_limit_ns.load(); }
void set_wait_limit_ns(unsigned long long ns) { g_wait_limit_ns.store(ns ? ns : 1500ull * 1000ull * 1000ull); }
void withhold_next_gemm_load(uint32_t k_block) { g_withhold_kb.store(k_block); }
uint32_t take_withheld_gemm_load() { return g_withhold_kb.exchange(0xffffffffu); }

int per_device_once(const void *key, int device, int (*init)(void *arg, int *value), void *arg, int *value) {
  std::lock_guard<std::mutex> lock(g_once_mutex);
  const auto it = g_once_values.find({key, device});
  if (it != g_once_values.end()) {
    if (value)
      *value = it->second;
    return kOk;
  }
  int v = 0;
  if (int rc = init(arg, &v))
    return rc;
  g_once_values[{key, device}] = v;
  if (value)
    *value = v;
  return kOk;
}

int current_device_once(const void *key, int (*init)(void *arg, int *value), void *arg, int *value) {
  int device = 0;
  if (int rc = check_cuda(cudaGetDevice(&device), "cudaGetDevice"))
    return rc;
  return per_device_once(key, device, init, arg, value);
}

void set_last_error(const std::string &text) { g_last_error = text; }
const std::string &last_error() { return g_last_error; }

int fail(int status, const std::string &text) {
  g_last_error = text;
  return status;
}

int check_cuda(cudaError_t code, const char *what) {
  if (code == cudaSuccess)
    return kOk;
  std::string text = std::string(what) + ": " + cudaGetErrorName(code) + " (" +
                     cudaGetErrorString(code) + ")";
  return fail(code == cudaErrorMemoryAllocation ? kOutOfMemory : kExecutionError, text);
}

namespace {
std::atomic<unsigned long long> g_launches{0};
}
int launched(cudaError_t code, const char *what) {
  if (code == cudaSuccess)
    g_launches.fetch_add(1, std::memory_order_relaxed);
  return check_cuda(code, what);
}
unsigned long long launch_count() { return g_launches.load(); }

int sm_count() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess)
    return 148;
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = g_sm_counts.find(device);
  if (it != g_sm_counts.end())
    return it->second;
  int count = 148;
  cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
  g_sm_counts[device] = count;
  return count;
}

void *device_scratch(size_t bytes) {
  static std::unordered_map<int, std::pair<void *, size_t>> areas;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess)
    return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  auto &area = areas[device];
  if (area.second >= bytes && area.first)
    return area.first;
  if (area.first)
    cudaFree(area.first); // waits for everything that may still read the old area
  area = {nullptr, 0};
  const size_t rounded = (bytes + (1u << 20) - 1) & ~(size_t)((1u << 20) - 1);
  if (cudaMalloc(&area.first, rounded) != cudaSuccess) {
    area.first = nullptr;
    return nullptr;
  }
  area.second = rounded;
  return area.first;
}

DeviceStatus *device_status_words() {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess)
    return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  auto it = g_status_words.find(device);
  if (it != g_status_words.end())
    return it->second;
  DeviceStatus *words = nullptr;
  if (cudaMalloc(&words, sizeof(DeviceStatus)) != cudaSuccess)
    return nullptr;
  cudaMemset(words, 0, sizeof(DeviceStatus));
  g_status_words[device] = words;
  return words;
}

int poll_device_status(const char *what) {
  DeviceStatus *words = device_status_words();
  if (!words)
    return fail(kInternalError, "device status words are unavailable");
  DeviceStatus host{};
  if (int rc = check_cuda(cudaMemcpy(&host, words, sizeof(host), cudaMemcpyDeviceToHost), what))
    return rc;
  if (host.flag == 0)
    return kOk;
  cudaMemset(words, 0, sizeof(DeviceStatus));
  return fail(kExecutionError, std::string(what) + ": a bounded device-side wait ran out (kernel " +
                                   std::to_string(host.kernel) + ", role " + std::to_string(host.role) +
                                   ", detail " + std::to_string(host.detail) + ")");
}

} // namespace difb200
