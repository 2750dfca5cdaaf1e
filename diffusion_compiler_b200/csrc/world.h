// The multi-GPU world of the token-sharded block: one process per GPU, one NCCL communicator,
// and the schedule by which the key / value slices of all ranks reach every rank.
//
// The reference runs on one device per executor (reference include/dif/runtime/executor.hpp:683)
// and has no communication layer; this is the sequence-partitioned form of its video block
// (graph: reference tools/difc.cpp:261-345). Rank r owns a contiguous slice of the tokens.
// Everything but attention is row-local. Before attention every rank needs the INT8 key codes,
// their per-token-head scales and the bf16 values of all tokens: each rank keeps full-length
// gather buffers whose own slice its producer kernels write directly, and the slices travel in
// size - 1 ring-shifted steps (step s: send the own slice to rank + s, receive the slice of
// rank - s; every GPU sends and receives one slice per step, which NVSwitch serves at full
// bandwidth). Attention starts on the own slice while the others are in flight and takes the
// arrived slices in a few launches that carry the softmax state (attention_int8 with an
// AttentionChunk).
//
// Two ways to move the slices. (1) Direct: the gather block
// of every rank is mapped into every other rank (CUDA IPC over NVLink), and a rank PUSHES its
// slice into the peers' blocks with copy-engine copies on its communication stream, each followed
// by a four-byte copy of the pass number into the peer's flag area (the communication stream
// carries copies only, so it never changes engines); an attention launch is preceded by a one-CTA
// kernel that waits (bounded, see World::wait_ns) until the flags of the slices it reads carry the
// number of this pass. No SM and no rendezvous between the two sides is involved in a transfer, so
// transfers neither compete with the attention and GEMM CTAs for SMs nor couple the ranks' kernel
// schedules. (2) NCCL send / receive pairs, one grouped call per launch group, ordered by CUDA
// events; this is also what bootstraps (1). Which one a world uses by default follows the
// measurements quoted in world_bind (direct up to 4 ranks, NCCL beyond).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

namespace difb200 {

// Point-to-point transport of one rank. The schedule above is written against this interface so
// that it also runs among CPU threads over a host-memory transport (how it is tested without GPUs).
class Transport {
public:
  virtual ~Transport() {}
  virtual int group_start() = 0;
  virtual int send(const void *data, size_t bytes, int peer, cudaStream_t stream) = 0;
  virtual int recv(void *data, size_t bytes, int peer, cudaStream_t stream) = 0;
  virtual int group_end() = 0;
  virtual bool on_device() const = 0; // false: host memory, calls complete before they return
};

struct RingStep {
  int send_to, recv_from;
};
inline RingStep ring_step(int rank, int size, int step) {
  return RingStep{(rank + step) % size, ((rank - step) % size + size) % size};
}

// One attention launch of the chunked form: which ring steps must have landed before it, and the
// (at most two) ranges of 128-key tiles it covers. Step 0 is the rank's own slice.
struct LaunchPlan {
  std::vector<int> steps;
  uint32_t tile_begin[2], tile_count[2];
};
// `group_sizes` partitions the steps 0 .. size - 1 in order (e.g. {1, 3, 4} at 8 ranks); an empty
// vector selects the default (own slice first, the rest in one launch; with the direct exchange and
// more than 4 ranks the rest in two launches, the two nearest ring steps first).
// Returns false when the sizes do not sum to `size` or contain a zero.
bool plan_launches(int rank, int size, uint32_t tiles_per_slice, std::vector<int> group_sizes,
                   std::vector<LaunchPlan> &out);
std::vector<int> default_groups(int size, bool direct = false);
// The grouping in force: DIFB200_ATTENTION_GROUPS when it is well-formed for `size`, else the default.
std::vector<int> launch_groups(int size, bool direct = false);

class World {
public:
  int rank = 0, size = 1, device = 0;
  Transport *transport = nullptr;       // owned
  cudaStream_t comm_stream = nullptr;   // the exchange runs here, at the highest priority
  cudaEvent_t ready = nullptr;          // producer stream -> communication stream
  // direct exchange: the pushes to different peers go out on several streams (DIFB200_PUSH_STREAMS,
  // default 4), so that the set-up time of one copy hides behind the transfer of another
  std::vector<cudaStream_t> push_streams;
  std::vector<cudaEvent_t> push_done;   // one per push stream: its copies of the current push are enqueued
  cudaEvent_t push_fork = nullptr;      // communication stream -> push streams
  // landed[c][s - 1]: slice of rank - s has arrived in the buffers of exchange class c
  // (0 = values, 1 = key codes and scales); recorded by world_exchange_class
  std::vector<cudaEvent_t> landed[2];
  // limit of the waits for another rank's flag (direct exchange), DIFB200_WORLD_TIMEOUT_MS
  unsigned long long wait_ns = 60ull * 1000ull * 1000ull * 1000ull;
  ~World();
};

// Every rank's `bytes` bytes, in rank order, into `all` (host memory; blocks until they are there).
int world_all_gather_host(World *world, const void *mine, void *all, size_t bytes, cudaStream_t stream);

// ---- direct exchange --------------------------------------------------------------------------
constexpr int kMaxDirectWorld = 16;
// Flag area at the end of every gather block; all words count passes (1, 2, ...) and only grow.
struct ExchangeFlags {
  uint32_t arrived[2][kMaxDirectWorld]; // [class][source rank]: that rank's slice of pass n is here
  uint32_t consumed[kMaxDirectWorld];   // [reader rank]: that rank's attention of pass n has read MY slice there
  uint32_t stamp;                       // the number of the pass being pushed: the source of the flag copies
  uint32_t reserved[15];
};
// One gather block (the buffers of one sharded attention, at the same offsets on every rank).
struct PeerBinding {
  bool direct = false;       // false: the block is plain device memory and the slices travel by NCCL
  std::string note;          // why not direct
  void *block = nullptr;     // own block: payload, then ExchangeFlags
  size_t payload_bytes = 0, block_bytes = 0;
  std::vector<char *> peer;  // peer[r]: the block of rank r as mapped here ([rank] = block)
  uint32_t pushes[2] = {0, 0}; // exchanges enqueued so far, per class
  uint32_t passes = 0;         // attention passes enqueued so far
  uint32_t begun = 0;          // passes whose opening kernel (wait for `consumed`, set `stamp`) is enqueued
  cudaEvent_t pushed = nullptr;  // communication stream: every push enqueued so far has read the own slice
  bool timed = false;            // record an event pair around the copies of every push (world_push_times)
  std::vector<cudaEvent_t> spans[2]; // per class: begin, end, begin, end, ...
  ExchangeFlags *flags(int r) const { return reinterpret_cast<ExchangeFlags *>(peer[(size_t)r] + payload_bytes); }
};
// Collective: allocates a zeroed block of `payload_bytes` (+ flags) on every rank and, unless
// DIFB200_EXCHANGE=nccl, maps the peers' blocks; `direct` is the same on all ranks (one rank that
// cannot export or map makes all of them use NCCL, `note` says why).
int world_bind(World *world, size_t payload_bytes, cudaStream_t stream, PeerBinding **out);
// Collective: waits for this device's work, unmaps the peers, waits for all ranks, frees the block.
int world_unbind(World *world, PeerBinding *binding);
// Direct form of world_exchange_class: pushes this rank's slice of `count` buffers (at `offsets`
// in the block, `slice_bytes` per rank) to every peer, in ring order, once `producer` has run what
// is enqueued so far. The first push of a pass puts a one-CTA kernel on `producer` in front of
// that: it waits (bounded) until every peer's attention of the previous pass has read the slices
// about to be overwritten there, and sets the pass number the flag copies carry.
int world_push(World *world, PeerBinding *binding, int which, const uint64_t *offsets, const uint64_t *slice_bytes,
               int count, cudaStream_t producer);
// With binding->timed: the device time the copies of class `which` took on the communication stream,
// summed over the pushes since the last call, and their number (call after the streams have drained).
void world_push_times(PeerBinding *binding, int which, double *milliseconds, uint64_t *pushes);
// Test of the flag kernels on one device: a wait for a flag that is set beforehand (`set` true:
// returns kOk) or that nothing sets (`set` false: the wait gives up after `limit_ns` and the
// status poll returns kExecutionError); the context stays usable either way.
int world_selftest_flags(unsigned long long limit_ns, bool set);

// Rendezvous of `size` processes through a directory all of them can reach, bounded by
// `timeout_ms`: every rank leaves a file, rank 0 also the 128-byte communicator id (`id` in for
// rank 0, out for the others), and every rank waits until all files are there. Returns
// kExecutionError with text when a rank is missing at the deadline, so that no rank enters the
// (unbounded) communicator set-up alone. `generation` tells apart the worlds that meet in one
// directory one after another (the file names carry it).
int world_rendezvous(const std::string &directory, int rank, int size, uint8_t id[128], uint32_t timeout_ms,
                     uint32_t generation = 0);

int world_unique_id(uint8_t id[128]);
// Communicator on the current device (blocks until all ranks have called it).
int world_create(const uint8_t id[128], int rank, int size, World **out);
// World from the environment of this process: DIFB200_WORLD_SIZE (absent or 1: *out = nullptr),
// DIFB200_WORLD_RANK, DIFB200_WORLD_DIR (rendezvous directory), DIFB200_WORLD_TIMEOUT_MS (60000).
int world_from_environment(World **out);

// Ring exchange of gather buffers. buffers[i] holds size * slice_bytes[i] bytes; this rank's slice
// is final once everything enqueued on `producer` so far has run. The size - 1 steps are enqueued
// on the communication stream, one grouped transport call per attention launch group
// (launch_groups); events[s - 1] (caller-owned, may be null) is recorded when the group of step s,
// and with it the slice of rank - s, has landed in every buffer of this call.
int world_exchange(World *world, void *const *buffers, const uint64_t *slice_bytes, int count,
                   cudaStream_t producer, cudaEvent_t *events);

// The same exchange with the world's own events of class `which` (0 = values, 1 = keys).
int world_exchange_class(World *world, int which, void *const *buffers, const uint64_t *slice_bytes, int count,
                         cudaStream_t producer);

// Attention of this rank's queries over the keys and values of all ranks, as the launches of
// `plan_launches` on `stream`: each launch first waits (CUDA events) for the ring steps whose
// slices it reads. Gather buffers: k8 [size * slice_tokens, KV, 128] int8, ks [size * slice_tokens,
// KV] f32, v [size * slice_tokens, KV, 128] bf16 with slice_tokens a multiple of 128; key_valid
// [size * slice_tokens] marks real tokens (slice padding is 0); the exchanges of both classes must
// have been enqueued. `world` may be null (one rank: a single launch over the own slice).
// scratch: attention_int8_scratch_bytes(1, size * slice_tokens, KV); state:
// attention_int8_state_bytes(1, Sq, H) (unused with one launch).
// `binding` (may be null: NCCL events) selects the direct exchange's flags as the ordering.
int sharded_attention(World *world, PeerBinding *binding, const int8_t *q8, const float *qs, const int8_t *k8, const float *ks,
                      const void *v_bf16, const uint8_t *key_valid, uint64_t Sq, uint64_t slice_tokens, uint64_t H,
                      uint64_t KV, float scale, void *scratch, size_t scratch_bytes, void *state, void *out_bf16,
                      cudaStream_t stream);

// Host-memory transport among the threads of one process, for tests: `size` mailboxes, every
// recv waits at most timeout_ms for its matching send.
struct FakeFabric;
FakeFabric *fake_fabric_create(int size, uint32_t timeout_ms);
void fake_fabric_destroy(FakeFabric *fabric);
Transport *fake_transport(FakeFabric *fabric, int rank);

} // namespace difb200
