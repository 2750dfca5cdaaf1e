// Multi-GPU world: NCCL communicator (the library is resolved at run time, so a single-GPU host
// needs no NCCL), the ring exchange of the key / value slices, the launch plan of the chunked
// attention, a bounded rendezvous, and a host-memory transport for CPU tests. See world.h.
#include "world.h"

#include "common.cuh"
#include "ops.h"

#include <dlfcn.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <thread>

namespace difb200 {

// ---- launch plan ------------------------------------------------------------------------------
std::vector<int> default_groups(int size, bool direct) {
  // Measured on 8 B200s (video block, 33272 tokens): every further launch costs more than the
  // overlap it buys. NCCL: {1, 7} 2.49 ms, {1, 3, 4} 2.82 ms, {1, 1, 2, 4} 3.22 ms. Direct pushes
  // arrive one after another, so one split of the remote slices pays: {1, 2, 5} 2.58 ms, {1, 7} 2.70 ms.
  std::vector<int> groups{1};
  if (size > 1 && (size <= 4 || !direct)) {
    groups.push_back(size - 1);
  } else if (size > 4) {
    groups.push_back(2);
    groups.push_back(size - 3);
  }
  return groups;
}

std::vector<int> launch_groups(int size, bool direct) {
  // DIFB200_ATTENTION_GROUPS="1,3,4": how many ring steps (the own slice is step 0) each attention
  // launch covers; a list that is malformed or does not sum to the world size is ignored
  std::vector<int> groups;
  if (const char *text = std::getenv("DIFB200_ATTENTION_GROUPS")) {
    int value = 0, total = 0;
    bool digits = false, ok = true;
    for (const char *c = text;; ++c) {
      if (*c >= '0' && *c <= '9') {
        value = value * 10 + (*c - '0');
        digits = true;
      } else {
        if (digits) {
          groups.push_back(value);
          total += value;
          ok = ok && value > 0;
        }
        value = 0;
        digits = false;
        if (!*c)
          break;
      }
    }
    if (!ok || total != size)
      groups.clear();
  }
  return groups.empty() ? default_groups(size, direct) : groups;
}

bool plan_launches(int rank, int size, uint32_t tiles_per_slice, std::vector<int> group_sizes,
                   std::vector<LaunchPlan> &out) {
  out.clear();
  if (size < 1 || rank < 0 || rank >= size)
    return false;
  if (group_sizes.empty())
    group_sizes = default_groups(size, false);
  int total = 0;
  for (int g : group_sizes) {
    if (g <= 0)
      return false;
    total += g;
  }
  if (total != size)
    return false;
  int first = 0; // first ring step of the group
  for (int g : group_sizes) {
    LaunchPlan plan{};
    for (int s = first; s < first + g; ++s)
      plan.steps.push_back(s);
    // steps first .. first + g - 1 bring the slices of ranks rank - first, rank - first - 1, ...:
    // the slices [rank - first - g + 1, rank - first] modulo size, i.e. one or two runs of tiles
    const int low = ((rank - first - g + 1) % size + size) % size;
    const int run0 = low + g <= size ? g : size - low; // slices before the wrap
    plan.tile_begin[0] = (uint32_t)low * tiles_per_slice;
    plan.tile_count[0] = (uint32_t)run0 * tiles_per_slice;
    plan.tile_begin[1] = 0;
    plan.tile_count[1] = (uint32_t)(g - run0) * tiles_per_slice;
    out.push_back(plan);
    first += g;
  }
  return true;
}

// ---- NCCL, resolved with dlopen ---------------------------------------------------------------
namespace {

struct NcclUniqueId {
  char internal[128];
};
typedef struct ncclComm *NcclComm;

struct NcclApi {
  int (*GetUniqueId)(NcclUniqueId *) = nullptr;
  int (*CommInitRank)(NcclComm *, int, NcclUniqueId, int) = nullptr;
  int (*CommDestroy)(NcclComm) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  int (*Send)(const void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  int (*Recv)(void *, size_t, int, int, NcclComm, cudaStream_t) = nullptr;
  const char *(*GetErrorString)(int) = nullptr;
  bool ok = false;
  std::string error;
};

const NcclApi &nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    const char *name = std::getenv("DIFB200_NCCL_LIBRARY");
    void *handle = dlopen(name && name[0] ? name : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!handle) {
      api.error = std::string("cannot load NCCL (libnccl.so.2; set DIFB200_NCCL_LIBRARY): ") + dlerror();
      return;
    }
    auto sym = [&](const char *symbol) { return dlsym(handle, symbol); };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
    api.Send = reinterpret_cast<decltype(api.Send)>(sym("ncclSend"));
    api.Recv = reinterpret_cast<decltype(api.Recv)>(sym("ncclRecv"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.GroupStart && api.GroupEnd && api.Send &&
             api.Recv && api.GetErrorString;
    if (!api.ok)
      api.error = "the NCCL library lacks a required symbol";
  });
  return api;
}

int check_nccl(int rc, const char *what) {
  if (rc == 0)
    return kOk;
  return fail(kExecutionError, std::string(what) + ": NCCL error " + std::to_string(rc) + " (" +
                                   nccl().GetErrorString(rc) + ")");
}

class NcclTransport : public Transport {
public:
  NcclComm comm = nullptr;
  ~NcclTransport() override {
    if (comm)
      nccl().CommDestroy(comm);
  }
  int group_start() override { return check_nccl(nccl().GroupStart(), "ncclGroupStart"); }
  int send(const void *data, size_t bytes, int peer, cudaStream_t stream) override {
    return check_nccl(nccl().Send(data, bytes, 0 /* ncclInt8 */, peer, comm, stream), "ncclSend");
  }
  int recv(void *data, size_t bytes, int peer, cudaStream_t stream) override {
    return check_nccl(nccl().Recv(data, bytes, 0 /* ncclInt8 */, peer, comm, stream), "ncclRecv");
  }
  int group_end() override { return check_nccl(nccl().GroupEnd(), "ncclGroupEnd"); }
  bool on_device() const override { return true; }
};

} // namespace

World::~World() {
  delete transport;
  for (auto &events : landed)
    for (cudaEvent_t e : events)
      if (e)
        cudaEventDestroy(e);
  for (cudaEvent_t e : push_done)
    cudaEventDestroy(e);
  for (cudaStream_t st : push_streams)
    cudaStreamDestroy(st);
  if (push_fork)
    cudaEventDestroy(push_fork);
  if (ready)
    cudaEventDestroy(ready);
  if (comm_stream)
    cudaStreamDestroy(comm_stream);
}

int world_unique_id(uint8_t id[128]) {
  if (!nccl().ok)
    return fail(kUnsupported, nccl().error);
  NcclUniqueId uid;
  if (int rc = check_nccl(nccl().GetUniqueId(&uid), "ncclGetUniqueId"))
    return rc;
  std::memcpy(id, uid.internal, 128);
  return kOk;
}

int world_create(const uint8_t id[128], int rank, int size, World **out) {
  if (!out || !id || size < 1 || rank < 0 || rank >= size)
    return fail(kInvalidArgument, "world: bad rank or size");
  *out = nullptr;
  if (!nccl().ok)
    return fail(kUnsupported, nccl().error);
  World *world = new World();
  world->rank = rank;
  world->size = size;
  if (int rc = check_cuda(cudaGetDevice(&world->device), "cudaGetDevice")) {
    delete world;
    return rc;
  }
  int least = 0, greatest = 0;
  cudaDeviceGetStreamPriorityRange(&least, &greatest);
  int rc = check_cuda(cudaStreamCreateWithPriority(&world->comm_stream, cudaStreamNonBlocking, greatest),
                      "cudaStreamCreateWithPriority");
  if (!rc)
    rc = check_cuda(cudaEventCreateWithFlags(&world->ready, cudaEventDisableTiming), "cudaEventCreate");
  if (!rc) {
    NcclTransport *transport = new NcclTransport();
    world->transport = transport;
    NcclUniqueId uid;
    std::memcpy(uid.internal, id, 128);
    rc = check_nccl(nccl().CommInitRank(&transport->comm, size, uid, rank), "ncclCommInitRank");
  }
  if (rc) {
    delete world;
    return rc;
  }
  *out = world;
  return kOk;
}

// ---- rendezvous -------------------------------------------------------------------------------
int world_rendezvous(const std::string &directory, int rank, int size, uint8_t id[128], uint32_t timeout_ms,
                     uint32_t generation) {
  if (directory.empty() || size < 1 || rank < 0 || rank >= size || !id)
    return fail(kInvalidArgument, "world rendezvous: bad arguments");
  auto path = [&](int r) {
    return directory + "/world_" + std::to_string(generation) + "_rank_" + std::to_string(r);
  };
  {
    const std::string temp = path(rank) + ".writing";
    FILE *f = std::fopen(temp.c_str(), "wb");
    if (!f)
      return fail(kExecutionError, "world rendezvous: cannot write into " + directory);
    const size_t written = std::fwrite(id, 1, 128, f); // only rank 0's content is read
    std::fclose(f);
    if (written != 128 || std::rename(temp.c_str(), path(rank).c_str()) != 0)
      return fail(kExecutionError, "world rendezvous: cannot publish " + path(rank));
  }
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (;;) {
    int missing = -1;
    for (int r = 0; r < size; ++r) {
      struct stat st;
      if (stat(path(r).c_str(), &st) != 0 || st.st_size != 128) {
        missing = r;
        break;
      }
    }
    if (missing < 0)
      break;
    if (std::chrono::steady_clock::now() >= deadline)
      return fail(kExecutionError, "world rendezvous: rank " + std::to_string(missing) + " of " +
                                       std::to_string(size) + " did not arrive within " +
                                       std::to_string(timeout_ms) + " ms; not entering the communicator set-up");
    std::this_thread::sleep_for(std::chrono::milliseconds(2));
  }
  if (rank != 0) {
    FILE *f = std::fopen(path(0).c_str(), "rb");
    if (!f || std::fread(id, 1, 128, f) != 128) {
      if (f)
        std::fclose(f);
      return fail(kExecutionError, "world rendezvous: cannot read the communicator id");
    }
    std::fclose(f);
  }
  return kOk;
}

int world_from_environment(World **out) {
  *out = nullptr;
  const char *size_text = std::getenv("DIFB200_WORLD_SIZE");
  const int size = size_text ? std::atoi(size_text) : 1;
  if (size <= 1)
    return kOk;
  const char *rank_text = std::getenv("DIFB200_WORLD_RANK"), *dir = std::getenv("DIFB200_WORLD_DIR");
  if (!rank_text || !dir)
    return fail(kInvalidArgument, "DIFB200_WORLD_SIZE > 1 needs DIFB200_WORLD_RANK and DIFB200_WORLD_DIR");
  const int rank = std::atoi(rank_text);
  const char *timeout_text = std::getenv("DIFB200_WORLD_TIMEOUT_MS");
  const uint32_t timeout_ms = timeout_text ? (uint32_t)std::strtoul(timeout_text, nullptr, 10) : 60000u;
  uint8_t id[128] = {0};
  if (rank == 0)
    if (int rc = world_unique_id(id))
      return rc;
  // A process may join several worlds one after another (one per plugin context): the n-th world
  // of every rank meets under the n-th name, so the files of an earlier world are never mistaken
  // for this one's. Every rank has to create its worlds in the same order.
  static std::atomic<uint32_t> generation{0};
  if (int rc = world_rendezvous(dir, rank, size, id, timeout_ms, generation.fetch_add(1)))
    return rc;
  if (int rc = world_create(id, rank, size, out))
    return rc;
  (*out)->wait_ns = (unsigned long long)(timeout_ms ? timeout_ms : 1u) * 1000ull * 1000ull;
  return kOk;
}

// ---- exchange ---------------------------------------------------------------------------------
int world_exchange(World *world, void *const *buffers, const uint64_t *slice_bytes, int count,
                   cudaStream_t producer, cudaEvent_t *events) {
  if (!world || !world->transport || count < 1 || !buffers || !slice_bytes)
    return fail(kInvalidArgument, "world exchange: bad arguments");
  if (world->size == 1)
    return kOk;
  Transport &t = *world->transport;
  cudaStream_t stream = world->comm_stream;
  if (t.on_device()) {
    if (int rc = check_cuda(cudaEventRecord(world->ready, producer), "cudaEventRecord(slice ready)"))
      return rc;
    if (int rc = check_cuda(cudaStreamWaitEvent(stream, world->ready, 0), "cudaStreamWaitEvent(slice ready)"))
      return rc;
  }
  // The ring steps go out in the groups in which the attention launches consume them (one
  // grouped NCCL call per launch: its peers are served concurrently); all steps of a group share
  // the moment they are marked as landed.
  const std::vector<int> groups = launch_groups(world->size, false);
  int first = 0;
  for (int g : groups) {
    const int begin = first == 0 ? 1 : first, end = first + g; // step 0 is the own slice
    first = end;
    if (begin >= end)
      continue;
    if (int rc = t.group_start())
      return rc;
    for (int s = begin; s < end; ++s) {
      const RingStep step = ring_step(world->rank, world->size, s);
      for (int i = 0; i < count; ++i) {
        char *base = static_cast<char *>(buffers[i]);
        if (int rc = t.send(base + (uint64_t)world->rank * slice_bytes[i], (size_t)slice_bytes[i], step.send_to, stream))
          return rc;
        if (int rc = t.recv(base + (uint64_t)step.recv_from * slice_bytes[i], (size_t)slice_bytes[i], step.recv_from,
                            stream))
          return rc;
      }
    }
    if (int rc = t.group_end())
      return rc;
    for (int s = begin; s < end; ++s)
      if (events && events[s - 1] && t.on_device())
        if (int rc = check_cuda(cudaEventRecord(events[s - 1], stream), "cudaEventRecord(step landed)"))
          return rc;
  }
  return kOk;
}

int world_exchange_class(World *world, int which, void *const *buffers, const uint64_t *slice_bytes, int count,
                         cudaStream_t producer) {
  if (!world || which < 0 || which > 1)
    return fail(kInvalidArgument, "world exchange: bad class");
  auto &events = world->landed[which];
  while ((int)events.size() < world->size - 1) {
    cudaEvent_t e = nullptr;
    if (int rc = check_cuda(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate"))
      return rc;
    events.push_back(e);
  }
  return world_exchange(world, buffers, slice_bytes, count, producer, events.data());
}

// ---- direct exchange: peer-mapped gather blocks, copy-engine pushes, sequence flags -------------
namespace {

struct FlagList {
  uint32_t *flag[2 * kMaxDirectWorld];
  uint32_t value[2 * kMaxDirectWorld];
  int count;
};

// One thread per flag: waits until the word has reached its value (the words only grow; the
// comparison is wrap-safe) or `limit_ns` has passed, which is reported in the device status words
// (kernel 5; role = index in the list, detail = the value seen last) and ends the wait.
__global__ void wait_flags_kernel(FlagList list, unsigned long long limit_ns, DeviceStatus *status) {
  const int i = (int)threadIdx.x;
  if (i >= list.count)
    return;
  const uint32_t *flag = list.flag[i];
  const uint32_t want = list.value[i];
  unsigned long long start = 0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
  for (;;) {
    uint32_t seen;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
    if ((int32_t)(seen - want) >= 0)
      break;
    unsigned long long now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (now - start > limit_ns) {
      if (atomicExch(&status->flag, 1u) == 0u) {
        status->kernel = 5u;
        status->role = (unsigned)i;
        status->detail = seen;
      }
      break;
    }
    __nanosleep(200);
  }
  __threadfence_system();
}

// Opens a pass of pushes: waits like wait_flags_kernel (the peers have read the slices of the
// previous pass), then sets the word that the flag copies of this pass take their value from.
__global__ void open_pass_kernel(FlagList list, uint32_t *stamp, uint32_t pass, unsigned long long limit_ns,
                                 DeviceStatus *status) {
  const int i = (int)threadIdx.x;
  if (i < list.count) {
    const uint32_t *flag = list.flag[i];
    const uint32_t want = list.value[i];
    unsigned long long start = 0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(start));
    for (;;) {
      uint32_t seen;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(flag) : "memory");
      if ((int32_t)(seen - want) >= 0)
        break;
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (now - start > limit_ns) {
        if (atomicExch(&status->flag, 1u) == 0u) {
          status->kernel = 6u;
          status->role = (unsigned)i;
          status->detail = seen;
        }
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  if (i == 0) {
    *stamp = pass;
    __threadfence_system();
  }
}

// One thread per flag: everything this stream did before is visible before the word is.
__global__ void set_flags_kernel(FlagList list) {
  const int i = (int)threadIdx.x;
  if (i >= list.count)
    return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(list.flag[i]), "r"(list.value[i]) : "memory");
}

int wait_flags(const FlagList &list, unsigned long long limit_ns, cudaStream_t stream) {
  if (list.count == 0)
    return kOk;
  DeviceStatus *status = device_status_words();
  if (!status)
    return fail(kInternalError, "device status words are unavailable");
  wait_flags_kernel<<<1, 2 * kMaxDirectWorld, 0, stream>>>(list, limit_ns, status);
  return launched(cudaGetLastError(), "wait_flags_kernel");
}

int set_flags(const FlagList &list, cudaStream_t stream) {
  if (list.count == 0)
    return kOk;
  set_flags_kernel<<<1, 2 * kMaxDirectWorld, 0, stream>>>(list);
  return launched(cudaGetLastError(), "set_flags_kernel");
}

struct BindRecord {
  cudaIpcMemHandle_t handle;
  int32_t ok;
  char gpu[16]; // the device's UUID: two ranks on one GPU must not wait for each other's kernels
};

// before an attention launch: the slices of its ring steps, both classes, carry this pass's number
int await_slices(World *world, PeerBinding *binding, const LaunchPlan &plan, cudaStream_t stream) {
  FlagList list{};
  ExchangeFlags *own = binding->flags(world->rank);
  for (int step : plan.steps) {
    if (step == 0)
      continue;
    const int source = ring_step(world->rank, world->size, step).recv_from;
    for (int which = 0; which < 2; ++which) {
      if (binding->pushes[which] == 0)
        return fail(kInvalidArgument, "sharded attention: the exchange of the gather buffers was not enqueued");
      list.flag[list.count] = &own->arrived[which][source];
      list.value[list.count] = binding->pushes[which];
      ++list.count;
    }
  }
  return wait_flags(list, world->wait_ns, stream);
}

// behind the last attention launch of a pass: the own slice may be overwritten once the pushes
// have read it, and every peer learns that its slice here has been read
int release_slices(World *world, PeerBinding *binding, cudaStream_t stream) {
  if (int rc = check_cuda(cudaStreamWaitEvent(stream, binding->pushed, 0), "cudaStreamWaitEvent(slices pushed)"))
    return rc;
  ++binding->passes;
  FlagList list{};
  for (int r = 0; r < world->size; ++r) {
    if (r == world->rank)
      continue;
    list.flag[list.count] = &binding->flags(r)->consumed[world->rank];
    list.value[list.count] = binding->passes;
    ++list.count;
  }
  return set_flags(list, stream);
}

} // namespace

int world_all_gather_host(World *world, const void *mine, void *all, size_t bytes, cudaStream_t stream) {
  if (!world || !mine || !all || bytes == 0)
    return fail(kInvalidArgument, "world all-gather: bad arguments");
  const size_t size = (size_t)world->size;
  if (!world->transport->on_device()) { // host transport (tests): the buffers are host memory
    std::memcpy(static_cast<char *>(all) + (size_t)world->rank * bytes, mine, bytes);
    void *buffers[1] = {all};
    const uint64_t slice[1] = {bytes};
    return world_exchange(world, buffers, slice, 1, stream, nullptr);
  }
  char *device = nullptr;
  if (int rc = check_cuda(cudaMalloc(&device, size * bytes), "cudaMalloc(all-gather)"))
    return rc;
  int rc = check_cuda(cudaMemcpyAsync(device + (size_t)world->rank * bytes, mine, bytes, cudaMemcpyHostToDevice, stream),
                      "cudaMemcpyAsync(all-gather)");
  void *buffers[1] = {device};
  const uint64_t slice[1] = {bytes};
  if (!rc)
    rc = world_exchange(world, buffers, slice, 1, stream, nullptr);
  if (!rc)
    rc = check_cuda(cudaStreamSynchronize(world->comm_stream), "cudaStreamSynchronize(all-gather)");
  if (!rc)
    rc = check_cuda(cudaMemcpy(all, device, size * bytes, cudaMemcpyDeviceToHost), "cudaMemcpy(all-gather)");
  cudaFree(device);
  return rc;
}

int world_bind(World *world, size_t payload_bytes, cudaStream_t stream, PeerBinding **out) {
  if (!world || !out)
    return fail(kInvalidArgument, "world bind: bad arguments");
  *out = nullptr;
  PeerBinding *b = new PeerBinding();
  b->payload_bytes = (payload_bytes + 255) / 256 * 256;
  // a block of its own mapping granule, so that the exported handle covers exactly this block
  const size_t granule = 2u << 20;
  b->block_bytes = (b->payload_bytes + sizeof(ExchangeFlags) + granule - 1) / granule * granule;
  b->peer.assign((size_t)world->size, nullptr);
  int rc = check_cuda(cudaMalloc(&b->block, b->block_bytes), "cudaMalloc(gather block)");
  if (!rc)
    rc = check_cuda(cudaMemsetAsync(b->block, 0, b->block_bytes, stream), "cudaMemsetAsync(gather block)");
  if (!rc) // zero before any peer can learn the handle: a push must never be wiped
    rc = check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize(gather block)");
  if (!rc)
    rc = check_cuda(cudaEventCreateWithFlags(&b->pushed, cudaEventDisableTiming), "cudaEventCreate");
  if (rc) {
    if (b->block)
      cudaFree(b->block);
    delete b;
    return rc;
  }
  b->peer[(size_t)world->rank] = static_cast<char *>(b->block);
  *out = b;
  if (world->size == 1)
    return kOk;
  // DIFB200_EXCHANGE=direct | nccl; unset: direct up to 4 ranks, NCCL beyond. Measured on B200s (video
  // block, 33272 tokens, ms per pass direct / NCCL): 2 ranks 8.01 / 8.11, 4 ranks 4.27 / 4.39, 8 ranks
  // 2.58 / 2.49 -- with 7 peers the copy engines reach about 420 GB/s per GPU in the all-to-all
  // pattern where NCCL's SM copies reach more, and that outweighs the SMs NCCL takes.
  const char *mode = std::getenv("DIFB200_EXCHANGE");
  const bool chosen = mode && mode[0] ? std::strcmp(mode, "nccl") != 0 : world->size <= 4;
  const bool wanted = chosen && world->size <= kMaxDirectWorld && world->transport->on_device();
  // first gather: every rank's handle; second gather: whether every rank could map every handle
  std::vector<BindRecord> records((size_t)world->size);
  BindRecord mine{};
  {
    cudaDeviceProp prop{};
    if (cudaGetDeviceProperties(&prop, world->device) == cudaSuccess)
      std::memcpy(mine.gpu, prop.uuid.bytes, 16);
    else
      cudaGetLastError();
  }
  if (wanted) {
    mine.ok = cudaIpcGetMemHandle(&mine.handle, b->block) == cudaSuccess ? 1 : 0;
    if (!mine.ok)
      cudaGetLastError();
  }
  if (int rc2 = world_all_gather_host(world, &mine, records.data(), sizeof(BindRecord), stream))
    return rc2;
  bool all_exported = true, shared_gpu = false;
  for (size_t r = 0; r < records.size(); ++r) {
    all_exported = all_exported && records[r].ok == 1;
    for (size_t o = 0; o < r; ++o)
      shared_gpu = shared_gpu || std::memcmp(records[r].gpu, records[o].gpu, 16) == 0;
  }
  all_exported = all_exported && !shared_gpu;
  int32_t mapped = all_exported ? 1 : 0;
  if (all_exported) {
    for (int r = 0; r < world->size && mapped; ++r) {
      if (r == world->rank)
        continue;
      void *ptr = nullptr;
      if (cudaIpcOpenMemHandle(&ptr, records[(size_t)r].handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        mapped = 0;
      } else {
        b->peer[(size_t)r] = static_cast<char *>(ptr);
      }
    }
  }
  std::vector<int32_t> everyone((size_t)world->size, 0);
  if (int rc2 = world_all_gather_host(world, &mapped, everyone.data(), sizeof(int32_t), stream))
    return rc2;
  bool all_mapped = true;
  for (int32_t m : everyone)
    all_mapped = all_mapped && m == 1;
  if (all_mapped) {
    b->direct = true;
    return kOk;
  }
  for (int r = 0; r < world->size; ++r)
    if (r != world->rank && b->peer[(size_t)r]) {
      cudaIpcCloseMemHandle(b->peer[(size_t)r]);
      b->peer[(size_t)r] = nullptr;
    }
  b->note = !wanted ? "direct exchange not requested or not possible for this world"
                    : (shared_gpu ? "two ranks share a GPU"
                       : !all_exported ? "a rank could not export its gather block (CUDA IPC)"
                                     : "a rank could not map a peer's gather block (CUDA IPC, peer access)");
  return kOk;
}

int world_unbind(World *world, PeerBinding *b) {
  if (!b)
    return kOk;
  int rc = kOk;
  if (b->direct) {
    // own pushes and flag stores are done; then nobody touches a block that is about to go
    rc = check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize(unbind)");
    for (char *mapped : b->peer)
      if (mapped && mapped != b->block)
        cudaIpcCloseMemHandle(mapped);
    if (world) { // (a world that is gone already: the caller broke the order of destruction; no barrier then)
      int32_t here = 1;
      std::vector<int32_t> everyone((size_t)world->size, 0);
      const int rc2 = world_all_gather_host(world, &here, everyone.data(), sizeof(int32_t), world->comm_stream);
      rc = rc ? rc : rc2;
    }
  }
  for (auto &spans : b->spans)
    for (cudaEvent_t e : spans)
      cudaEventDestroy(e);
  if (b->pushed)
    cudaEventDestroy(b->pushed);
  if (b->block)
    cudaFree(b->block);
  delete b;
  return rc;
}

namespace {
// the push streams of a world, made on first use
int push_streams_of(World *world) {
  if (!world->push_streams.empty())
    return kOk;
  int lanes = 4;
  if (const char *text = std::getenv("DIFB200_PUSH_STREAMS")) {
    const int value = std::atoi(text);
    if (value >= 1 && value <= kMaxDirectWorld)
      lanes = value;
  }
  int least = 0, greatest = 0;
  cudaDeviceGetStreamPriorityRange(&least, &greatest);
  if (int rc = check_cuda(cudaEventCreateWithFlags(&world->push_fork, cudaEventDisableTiming), "cudaEventCreate"))
    return rc;
  for (int k = 0; k < lanes; ++k) {
    cudaStream_t st = nullptr;
    cudaEvent_t e = nullptr;
    if (int rc = check_cuda(cudaStreamCreateWithPriority(&st, cudaStreamNonBlocking, greatest),
                            "cudaStreamCreateWithPriority(push)"))
      return rc;
    world->push_streams.push_back(st);
    if (int rc = check_cuda(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate"))
      return rc;
    world->push_done.push_back(e);
  }
  return kOk;
}
} // namespace

int world_push(World *world, PeerBinding *b, int which, const uint64_t *offsets, const uint64_t *slice_bytes, int count,
               cudaStream_t producer) {
  if (!world || !b || !b->direct || which < 0 || which > 1 || count < 1 || !offsets || !slice_bytes)
    return fail(kInvalidArgument, "world push: bad arguments");
  for (int i = 0; i < count; ++i)
    if (offsets[i] + (uint64_t)world->size * slice_bytes[i] > b->payload_bytes)
      return fail(kInvalidArgument, "world push: a buffer does not fit the gather block");
  cudaStream_t stream = world->comm_stream;
  const uint32_t pass = ++b->pushes[which];
  ExchangeFlags *own = b->flags(world->rank);
  if (b->begun < pass) {
    // first push of this pass: on the producer's stream (kernel after kernel), so that the
    // communication stream carries nothing but copies
    b->begun = pass;
    FlagList list{};
    if (pass > 1)
      for (int r = 0; r < world->size; ++r)
        if (r != world->rank) {
          list.flag[list.count] = &own->consumed[r];
          list.value[list.count] = pass - 1;
          ++list.count;
        }
    DeviceStatus *status = device_status_words();
    if (!status)
      return fail(kInternalError, "device status words are unavailable");
    open_pass_kernel<<<1, 2 * kMaxDirectWorld, 0, producer>>>(list, &own->stamp, pass, world->wait_ns, status);
    if (int rc = launched(cudaGetLastError(), "open_pass_kernel"))
      return rc;
  }
  if (int rc = check_cuda(cudaEventRecord(world->ready, producer), "cudaEventRecord(slice ready)"))
    return rc;
  if (int rc = check_cuda(cudaStreamWaitEvent(stream, world->ready, 0), "cudaStreamWaitEvent(slice ready)"))
    return rc;
  if (b->timed) {
    for (int k = 0; k < 2; ++k) {
      cudaEvent_t e = nullptr;
      if (int rc = check_cuda(cudaEventCreate(&e), "cudaEventCreate(push span)"))
        return rc;
      b->spans[which].push_back(e);
    }
    cudaEventRecord(b->spans[which][b->spans[which].size() - 2], stream);
  }
  if (int rc = push_streams_of(world))
    return rc;
  const int lanes = (int)world->push_streams.size();
  if (int rc = check_cuda(cudaEventRecord(world->push_fork, stream), "cudaEventRecord(push fork)"))
    return rc;
  for (int k = 0; k < lanes && k < world->size - 1; ++k)
    if (int rc = check_cuda(cudaStreamWaitEvent(world->push_streams[(size_t)k], world->push_fork, 0),
                            "cudaStreamWaitEvent(push fork)"))
      return rc;
  for (int s = 1; s < world->size; ++s) {
    const int peer = ring_step(world->rank, world->size, s).send_to;
    cudaStream_t lane = world->push_streams[(size_t)((s - 1) % lanes)]; // ring order within and across the lanes
    for (int i = 0; i < count; ++i) {
      const uint64_t at = offsets[i] + (uint64_t)world->rank * slice_bytes[i];
      if (int rc = check_cuda(cudaMemcpyAsync(b->peer[(size_t)peer] + at, static_cast<char *>(b->block) + at,
                                              (size_t)slice_bytes[i], cudaMemcpyDeviceToDevice, lane),
                              "cudaMemcpyAsync(slice to peer)"))
        return rc;
    }
    // the pass number behind the data, by the same engine: in stream order, so it lands after them
    if (int rc = check_cuda(cudaMemcpyAsync(&b->flags(peer)->arrived[which][world->rank], &own->stamp, sizeof(uint32_t),
                                            cudaMemcpyDeviceToDevice, lane),
                            "cudaMemcpyAsync(flag to peer)"))
      return rc;
  }
  for (int k = 0; k < lanes && k < world->size - 1; ++k) {
    if (int rc = check_cuda(cudaEventRecord(world->push_done[(size_t)k], world->push_streams[(size_t)k]),
                            "cudaEventRecord(push lane)"))
      return rc;
    if (int rc = check_cuda(cudaStreamWaitEvent(stream, world->push_done[(size_t)k], 0), "cudaStreamWaitEvent(push lane)"))
      return rc;
  }
  if (b->timed)
    cudaEventRecord(b->spans[which].back(), stream);
  return check_cuda(cudaEventRecord(b->pushed, stream), "cudaEventRecord(slices pushed)");
}

void world_push_times(PeerBinding *b, int which, double *milliseconds, uint64_t *pushes) {
  *milliseconds = 0.0;
  *pushes = 0;
  if (!b || which < 0 || which > 1)
    return;
  auto &spans = b->spans[which];
  for (size_t i = 0; i + 1 < spans.size(); i += 2) {
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, spans[i], spans[i + 1]) == cudaSuccess) {
      *milliseconds += ms;
      *pushes += 1;
    } else {
      cudaGetLastError();
    }
  }
  for (cudaEvent_t e : spans)
    cudaEventDestroy(e);
  spans.clear();
}

int world_selftest_flags(unsigned long long limit_ns, bool set) {
  uint32_t *word = nullptr;
  if (int rc = check_cuda(cudaMalloc(&word, 256), "cudaMalloc(flag)"))
    return rc;
  int rc = check_cuda(cudaMemset(word, 0, 256), "cudaMemset(flag)");
  FlagList list{};
  list.flag[0] = word;
  list.value[0] = 7;
  list.count = 1;
  if (!rc && set)
    rc = set_flags(list, nullptr);
  if (!rc)
    rc = wait_flags(list, limit_ns, nullptr);
  if (!rc)
    rc = poll_device_status("flag self-test");
  else
    cudaDeviceSynchronize();
  cudaFree(word);
  return rc;
}

int sharded_attention(World *world, PeerBinding *binding, const int8_t *q8, const float *qs, const int8_t *k8, const float *ks,
                      const void *v_bf16, const uint8_t *key_valid, uint64_t Sq, uint64_t slice_tokens, uint64_t H,
                      uint64_t KV, float scale, void *scratch, size_t scratch_bytes, void *state, void *out_bf16,
                      cudaStream_t stream) {
  const int size = world ? world->size : 1, rank = world ? world->rank : 0;
  if (slice_tokens == 0 || slice_tokens % 128 != 0)
    return fail(kInvalidArgument, "sharded attention: the slice length must be a positive multiple of 128");
  std::vector<LaunchPlan> launches;
  if (!plan_launches(rank, size, (uint32_t)(slice_tokens / 128), launch_groups(size, binding && binding->direct), launches))
    return fail(kInternalError, "sharded attention: no launch plan");
  if (launches.size() > 1 && !state)
    return fail(kInvalidArgument, "sharded attention: several launches need a state buffer");
  const uint64_t keys = (uint64_t)size * slice_tokens;
  const bool direct = binding && binding->direct && size > 1;
  for (size_t i = 0; i < launches.size(); ++i) {
    const LaunchPlan &plan = launches[i];
    if (direct) {
      if (int rc = await_slices(world, binding, plan, stream))
        return rc;
    }
    for (int step : plan.steps) {
      if (step == 0 || direct)
        continue; // the own slice: written on `stream` itself
      for (int which = 0; which < 2; ++which) {
        if ((int)world->landed[which].size() < step)
          return fail(kInvalidArgument, "sharded attention: the exchange of the gather buffers was not enqueued");
        if (int rc = check_cuda(cudaStreamWaitEvent(stream, world->landed[which][(size_t)step - 1], 0),
                                "cudaStreamWaitEvent(slice landed)"))
          return rc;
      }
    }
    AttentionChunk chunk{};
    for (int r = 0; r < 2; ++r) {
      chunk.tile_begin[r] = plan.tile_begin[r];
      chunk.tile_count[r] = plan.tile_count[r];
    }
    chunk.carry_in = i > 0;
    chunk.carry_out = i + 1 < launches.size();
    chunk.state = state;
    if (int rc = attention_int8(q8, qs, k8, ks, v_bf16, key_valid, 1, Sq, keys, H, KV, 128, scale, scratch,
                                scratch_bytes, out_bf16, stream, &chunk))
      return rc;
  }
  if (direct)
    return release_slices(world, binding, stream);
  return kOk;
}

// ---- host-memory transport for tests ----------------------------------------------------------
struct FakeFabric {
  int size;
  uint32_t timeout_ms;
  std::mutex mutex;
  std::condition_variable arrived;
  std::map<std::pair<int, int>, std::deque<std::vector<char>>> mail; // (from, to) -> messages in order
};

namespace {
class FakeTransport : public Transport {
public:
  FakeFabric *fabric;
  int rank;
  FakeTransport(FakeFabric *f, int r) : fabric(f), rank(r) {}
  int group_start() override { return kOk; }
  int group_end() override { return kOk; }
  bool on_device() const override { return false; }
  int send(const void *data, size_t bytes, int peer, cudaStream_t) override {
    if (peer < 0 || peer >= fabric->size)
      return fail(kInvalidArgument, "fake transport: bad peer");
    std::lock_guard<std::mutex> lock(fabric->mutex);
    const char *p = static_cast<const char *>(data);
    fabric->mail[{rank, peer}].emplace_back(p, p + bytes);
    fabric->arrived.notify_all();
    return kOk;
  }
  int recv(void *data, size_t bytes, int peer, cudaStream_t) override {
    std::unique_lock<std::mutex> lock(fabric->mutex);
    auto &queue = fabric->mail[{peer, rank}];
    if (!fabric->arrived.wait_for(lock, std::chrono::milliseconds(fabric->timeout_ms), [&] { return !queue.empty(); }))
      return fail(kExecutionError, "fake transport: rank " + std::to_string(peer) + " sent nothing to rank " +
                                       std::to_string(rank) + " within the deadline");
    if (queue.front().size() != bytes)
      return fail(kExecutionError, "fake transport: message size mismatch");
    std::memcpy(data, queue.front().data(), bytes);
    queue.pop_front();
    return kOk;
  }
};
} // namespace

FakeFabric *fake_fabric_create(int size, uint32_t timeout_ms) {
  FakeFabric *f = new FakeFabric();
  f->size = size;
  f->timeout_ms = timeout_ms;
  return f;
}
void fake_fabric_destroy(FakeFabric *fabric) { delete fabric; }
Transport *fake_transport(FakeFabric *fabric, int rank) { return new FakeTransport(fabric, rank); }

} // namespace difb200
