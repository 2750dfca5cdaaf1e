// Backend plugin entry points dif_backend_get_v2 / dif_backend_get_v1 (difb200/abi.h): the
// reference's drop-in boundary (reference include/dif/backend/abi.h; host side
// src/backend/plugin.cpp:60-283). compile() decodes + verifies the DIFIR001 bytes, keeps every
// tensor resident on the device, uploads constants, and plans one step per operation, fusing
//   LinearInt8Scaled -> BiasAdd -> Gelu(tanh)       into the GEMM epilogue, and
//   BooleanMaskToBias(MaskQueries=false) -> Attention into the attention kernel's key mask
// (the [B,1,S,S] bias is then never materialised). execute() copies inputs in, runs the steps
// `warmups` + `iterations` times (CUDA events around each timed pass), copies outputs out.
//
// Attention runs in its INT8 lowering when it is bf16, head dimension 128, non-causal,
// Implementation == 2 and either unbiased or biased by a fusable key mask -- the admission rule
// of the reference's INT8 route (src/runtime/cuda_executor.cpp:8422-8423, 3388-3391). The
// environment variable DIFB200_INT8_ATTENTION=0 turns the lowering off; an Attention that is not
// admitted is reported as unsupported (there is no exact-attention kernel and no CPU path here).
//
// Token-sharded execution. With DIFB200_WORLD_SIZE > 1 in the environment (plus DIFB200_WORLD_RANK
// and DIFB200_WORLD_DIR, see world.h) create() joins an NCCL world of one process per GPU. Every
// rank then compiles and executes the SAME program on ITS slice of the tokens (the program's token
// count is the slice length; weights are replicated as constants), and an Attention op attends from
// the local queries to the keys and values of all ranks: K codes, K scales and V are produced
// straight into this rank's slice of a full-length gather block, pushed into the peers' blocks by
// the copy engines or sent with NCCL (world.h) as soon as their producers are enqueued (the steps in
// front of the attention are reordered so that the V and K chains run before the Q chain), and
// attention runs as a few launches, the own slice first, each behind the slices it reads. The reference has no such
// mode (one device per executor, include/dif/runtime/executor.hpp:683); a single-process host
// drives one rank exactly as before.
#include "difb200/abi.h"
#include "difb200/difb200.h"

#include "common.cuh"
#include "diffir.h"
#include "glue.h"
#include "ops.h"
#include "world.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <limits>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace difb200 {
namespace {

struct Context {
  int device = 0;
  World *world = nullptr;           // token-sharded mode: the NCCL world this context is a rank of
  std::shared_ptr<bool> world_alive = std::make_shared<bool>(false); // read by executables that outlive the context
  cudaStream_t stream = nullptr;    // kernels
  cudaStream_t h2d = nullptr;       // uploads of an overlapped execute
  cudaStream_t d2h = nullptr;       // downloads of an overlapped execute
  char device_name[256] = {0};
};

struct Step {
  const ir::Op *op = nullptr;
  uint32_t epilogue = 0;            // LinearInt8Scaled: fused bias / gelu
  int bias_tensor = -1;             // index of the fused bias tensor
  int out_tensor = -1;              // index of the tensor the (fused) step writes
  int mask_tensor = -1;             // Attention: index of the fused Bool key mask
  bool skip = false;                // op absorbed by a neighbour, or a Reshape served by aliasing
  bool alias = false;               // Reshape: the output shares the input's buffer
  // QkNormPartialRope fused with its neighbours
  int rope_source = -1;             // tensor read in place (an absorbed last-axis Slice), else in[0]
  uint64_t rope_in_stride = 0, rope_in_offset = 0;
  int rope_attention = -1;          // step of the Attention whose INT8 q / k this op writes directly
  int rope_role = 0;                // 0 = q, 1 = k
  uint64_t rope_out_seq = 0, rope_out_start = 0;
  // Attention whose q / k arrive already quantised in the scratch buffer
  bool q_quantised = false, k_quantised = false;
  // QuantizeInt8Rows that also runs the RmsNormModulate (explicit scale / shift) producing its input
  int norm_step = -1;
  // token-sharded mode: Attention over the gathered keys / values (index into Executable::sharded);
  // steps after which this rank's V / K slice is final and its ring exchange starts
  int sharded = -1, exchange_v_for = -1, exchange_k_for = -1;
};

// Gather buffers and geometry of one token-sharded Attention.
struct Sharded {
  size_t step = 0;
  uint64_t tokens = 0, slice_tokens = 0, heads = 0, kv_heads = 0;
  int8_t *k8 = nullptr, *q8 = nullptr;   // k8 [size * slice_tokens, KV, 128]; q8 [tokens, H, 128]
  float *ks = nullptr, *qs = nullptr;
  void *v = nullptr;                     // bf16 [size * slice_tokens, KV, 128]
  uint8_t *valid = nullptr;              // [size * slice_tokens]
  void *scratch = nullptr, *state = nullptr;
  size_t scratch_bytes = 0;
  int v_root = -1;                       // tensor whose buffer IS this rank's V slice (-1: V is copied in)
  PeerBinding *binding = nullptr;        // the gather block holding v, k8, ks (mapped into the peers when direct)
  uint64_t at_v = 0, at_k8 = 0, at_ks = 0; // their offsets in the block
};

struct Executable {
  Context *ctx = nullptr;
  int device = 0;                   // ordinal of ctx's device (kept here: the destructor must not read ctx)
  ir::Program program;
  std::vector<void *> dev;          // device buffer per tensor (nullptr when never materialised)
  std::vector<uint8_t> owned;       // 0 where dev[i] aliases another tensor's buffer (Reshape)
  std::vector<Step> steps;
  std::vector<size_t> order;        // execution order of the steps (program order unless token-sharded)
  std::vector<Sharded> sharded;
  World *world = nullptr;           // ctx->world, valid while *world_alive
  std::shared_ptr<bool> world_alive;
  std::vector<void *> world_buffers; // device allocations beyond one per tensor (shared blocks, token-sharded mode)
  void *attn_scratch = nullptr;
  size_t attn_scratch_bytes = 0;
  unsigned int *flag = nullptr;     // device flag for data-dependent argument errors
  uint64_t resident_bytes = 0;
  bool constants_bound = false;     // v2: uploaded at compile
  std::vector<cudaEvent_t> uploaded, produced; // per tensor, made on first use by an overlapped execute
  // DIFB200_PROFILE=1: CUDA events in front of every step of the timed passes; the time between two
  // of them on the kernel stream is summed per opcode (difb200_executable_profile reads and clears)
  bool profile = false, profile_pass = false;
  std::vector<cudaEvent_t> profile_events;
  std::vector<uint32_t> profile_opcodes;        // opcode of the step that follows event i of this pass
  std::map<uint32_t, std::pair<double, uint64_t>> profile_sum;
  ~Executable() {
    cudaSetDevice(device);
    for (cudaEvent_t e : profile_events)
      cudaEventDestroy(e);
    for (cudaEvent_t e : uploaded)
      if (e)
        cudaEventDestroy(e);
    for (cudaEvent_t e : produced)
      if (e)
        cudaEventDestroy(e);
    for (size_t i = 0; i < dev.size(); ++i)
      if (dev[i] && (i >= owned.size() || owned[i]))
        cudaFree(dev[i]);
    for (Sharded &sh : sharded) // collective among the ranks while the world lives
      if (sh.binding)
        world_unbind(world_alive && *world_alive ? world : nullptr, sh.binding);
    for (void *b : world_buffers)
      cudaFree(b);
    if (attn_scratch)
      cudaFree(attn_scratch);
    if (flag)
      cudaFree(flag);
  }
};

struct EventPair { // two CUDA events that do not outlive their scope
  cudaEvent_t a = nullptr, b = nullptr;
  ~EventPair() {
    if (a)
      cudaEventDestroy(a);
    if (b)
      cudaEventDestroy(b);
  }
};

struct EventList { // CUDA events that do not outlive their scope
  std::vector<cudaEvent_t> events;
  ~EventList() {
    for (cudaEvent_t e : events)
      cudaEventDestroy(e);
  }
};

void write_error(dif_backend_error *error, const std::string &text) {
  if (!error || !error->data || error->capacity == 0)
    return;
  const size_t n = text.size() < error->capacity - 1 ? text.size() : error->capacity - 1;
  std::memcpy(error->data, text.data(), n);
  error->data[n] = '\0';
}

dif_backend_status status_of(int rc) {
  return rc >= 0 && rc <= 6 ? static_cast<dif_backend_status>(rc) : DIF_BACKEND_INTERNAL_ERROR;
}

struct PluginError {
  int status;
  std::string text;
};
void require(int rc) {
  if (rc != 0)
    throw PluginError{rc, last_error()};
}
void require_cuda(cudaError_t code, const char *what) { require(check_cuda(code, what)); }

bool int8_attention_enabled() {
  const char *v = std::getenv("DIFB200_INT8_ATTENTION");
  return !(v && v[0] == '0');
}

// ---- planning -------------------------------------------------------------------------------
void plan(Executable &exe) {
  const ir::Program &p = exe.program;
  std::map<uint32_t, int> consumers;
  std::map<uint32_t, size_t> consumer_op;
  for (size_t i = 0; i < p.ops.size(); ++i)
    for (auto id : p.ops[i].in) {
      consumers[id]++;
      consumer_op[id] = i;
    }
  exe.steps.assign(p.ops.size(), Step{});
  std::map<uint32_t, size_t> producer;
  for (size_t i = 0; i < p.ops.size(); ++i) {
    exe.steps[i].op = &p.ops[i];
    exe.steps[i].out_tensor = p.ops[i].out.empty() ? -1 : p.index_of(p.ops[i].out[0]);
    for (auto id : p.ops[i].out)
      producer[id] = i;
  }
  auto sole_consumer = [&](uint32_t id, uint32_t opcode, size_t &idx) {
    const ir::Tensor *t = p.tensor(id);
    if (!t || t->has(ir::Output) || consumers[id] != 1)
      return false;
    idx = consumer_op[id];
    return p.ops[idx].opcode == opcode && p.ops[idx].in[0] == id;
  };
  for (size_t i = 0; i < p.ops.size(); ++i) {
    const ir::Op &op = p.ops[i];
    Step &st = exe.steps[i];
    if (op.opcode == ir::LinearInt8Scaled) {
      size_t b = 0, g = 0;
      if (sole_consumer(op.out[0], ir::BiasAdd, b) && p.tensor(p.ops[b].in[1])->dtype == ir::BF16) {
        st.epilogue |= 1u;
        st.bias_tensor = p.index_of(p.ops[b].in[1]);
        st.out_tensor = p.index_of(p.ops[b].out[0]);
        exe.steps[b].skip = true;
        if (sole_consumer(p.ops[b].out[0], ir::Gelu, g) && p.ops[g].u64(ir::Approximation, 0) == 1) {
          st.epilogue |= 2u;
          st.out_tensor = p.index_of(p.ops[g].out[0]);
          exe.steps[g].skip = true;
        }
      }
    } else if (op.opcode == ir::Attention) {
      const ir::Tensor &q = *p.tensor(op.in[0]);
      const bool admitted = q.dtype == ir::BF16 && q.last() == 128 && !op.boolean(ir::Causal, false) &&
                            op.u64(ir::Implementation, 1) == 2 && int8_attention_enabled();
      if (!admitted)
        throw PluginError{2, "Attention (op " + std::to_string(op.id) +
                                 "): only the INT8 lowering exists here (bf16, head dim 128, non-causal, "
                                 "Implementation 2, DIFB200_INT8_ATTENTION not 0)"};
      if (op.in.size() == 4) {
        const auto it = producer.find(op.in[3]);
        const ir::Tensor *bias = p.tensor(op.in[3]);
        const bool fusable = it != producer.end() && p.ops[it->second].opcode == ir::BooleanMaskToBias &&
                             !p.ops[it->second].boolean(ir::MaskQueries, true) &&
                             p.tensor(p.ops[it->second].in[0])->dims.size() == 2 && consumers[op.in[3]] == 1 &&
                             !bias->has(ir::Output);
        if (!fusable)
          throw PluginError{2, "Attention (op " + std::to_string(op.id) +
                                   "): an additive bias is supported only as a key mask from "
                                   "BooleanMaskToBias(MaskQueries=false) consumed by this op alone"};
        st.mask_tensor = p.index_of(p.ops[it->second].in[0]);
        exe.steps[it->second].skip = true;
      }
    } else if (op.opcode == ir::Reshape) {
      // same bytes in the same order (cpu_executor.cpp:496-502 copies them): share the buffer
      st.alias = true;
      st.skip = true;
    } else if (op.opcode == ir::Linear) {
      const ir::Tensor &x = *p.tensor(op.in[0]), &w = *p.tensor(op.in[1]);
      if (2.0 * (double)x.dims[0] * (double)w.dims[0] * (double)w.dims[1] > 2.0e11)
        throw PluginError{2, "Linear (op " + std::to_string(op.id) +
                                 "): plain float Linear of this size is outside the quantized path; bind it "
                                 "as QuantizeInt8Rows + LinearInt8Scaled"};
    }
  }

  // ---- RmsNormModulate (explicit scale / shift) or LayerNormModulate -> QuantizeInt8Rows (256-wide ConvRot) ----
  // One kernel normalises, modulates, rotates and quantises; the normalised tensor is not
  // materialised. The row statistic is summed in another order than by the separate norm kernel
  // (both are parallel sums; the reference sums sequentially, cpu_executor.cpp:1241-1264), so a
  // few codes in 10^5 can move by one. DIFB200_NORM_FUSION=0 keeps the two kernels.
  const char *norm_fusion = std::getenv("DIFB200_NORM_FUSION");
  if (!(norm_fusion && norm_fusion[0] == '0'))
    for (size_t n = 0; n < p.ops.size(); ++n) {
      const ir::Op &norm = p.ops[n];
      size_t qi = 0;
      const bool rms = norm.opcode == ir::RmsNormModulate && norm.u64(ir::ModulationLayout, 1) != 2;
      // LayerNormModulate has two row reductions and three more roundings per element: in the
      // instruction-bound quantiser that costs more than the saved tensor above a few thousand
      // rows (measured at 3072 columns: 45 -> 29 us at 1024 rows, 78 -> 85 us at 8192), so only
      // short tensors are fused.
      const bool layer = norm.opcode == ir::LayerNormModulate && norm.in.size() == 5 &&
                         p.tensor(norm.in[0])->rows() <= 2048;
      if (!(rms || layer) || !sole_consumer(norm.out[0], ir::QuantizeInt8Rows, qi))
        continue;
      const ir::Op &quant = p.ops[qi];
      const ir::Tensor &x = *p.tensor(norm.in[0]);
      const uint64_t impl = quant.u64(ir::Implementation, 1);
      bool all_bf16 = true;
      for (auto id : norm.in)
        all_bf16 = all_bf16 && p.tensor(id)->dtype == ir::BF16;
      if (quant.in.size() != 1 || quant.out.size() != 2 || !all_bf16 || (rms && x.dims.size() != 2) ||
          x.last() % 256 != 0 || !(impl == 2 || impl == 3 || impl == 5 || impl == 6))
        continue;
      exe.steps[qi].norm_step = (int)n;
      exe.steps[n].skip = true;
    }

  // ---- QkNormPartialRope and its neighbours (all on 128-wide bf16 heads) ----
  // DIFB200_ROPE_FUSION=0 keeps the ops separate (same bits, more traffic): a test aid.
  if (const char *v = std::getenv("DIFB200_ROPE_FUSION"))
    if (v[0] == '0')
      return;
  auto private_to = [&](uint32_t id, size_t consumer) { // one reader, not an output of the program
    const ir::Tensor *t = p.tensor(id);
    return t && !t->has(ir::Output) && consumers[id] == 1 && consumer_op[id] == consumer;
  };
  auto rope_kernel_covers = [&](const ir::Op &op) {
    const ir::Tensor &x = *p.tensor(op.in[0]), &c = *p.tensor(op.in[2]);
    const uint64_t rotary = op.u64(ir::RotaryDim, x.last());
    const bool v2 = op.u64(ir::Implementation, 1) == 2 && op.u64(ir::RotaryLayout, 2) == 1;
    const uint64_t entry = c.dtype == ir::F32 ? 4 : 2;
    return x.dtype == ir::BF16 && x.last() == 128 && (c.dtype == ir::F32 || c.dtype == ir::BF16) &&
           (rotary == 64 || rotary == 96 || rotary == 128) && (c.last() * entry) % 16 == 0 &&
           (v2 ? c.last() == rotary / 2 : (c.last() == rotary || c.last() == rotary / 2));
  };
  for (size_t r = 0; r < p.ops.size(); ++r) {
    const ir::Op &rope = p.ops[r];
    if (rope.opcode != ir::QkNormPartialRope || !rope_kernel_covers(rope))
      continue;
    // (1) Slice on the last axis [-> Reshape] -> this op: read the slice in place
    auto it = producer.find(rope.in[0]);
    if (it == producer.end())
      continue;
    size_t reshape = p.ops.size(), slice = it->second;
    if (p.ops[slice].opcode == ir::Reshape && private_to(rope.in[0], r)) {
      reshape = slice;
      const auto up = producer.find(p.ops[reshape].in[0]);
      if (up == producer.end())
        continue;
      slice = up->second;
    }
    const ir::Op &sl = p.ops[slice];
    if (sl.opcode != ir::Slice)
      continue;
    const ir::Tensor &z = *p.tensor(sl.in[0]), &y = *p.tensor(sl.out[0]), &x = *p.tensor(rope.in[0]);
    const uint64_t heads = x.dims[x.dims.size() - 2];
    if (sl.u64(ir::Axis, 0) + 1 != z.dims.size() || y.last() != heads * 128 || z.last() % 8 != 0 ||
        sl.u64(ir::Start, 0) % 8 != 0 || !private_to(sl.out[0], reshape < p.ops.size() ? reshape : r) ||
        exe.steps[slice].skip)
      continue;
    Step &st = exe.steps[r];
    st.rope_source = p.index_of(sl.in[0]);
    st.rope_in_stride = z.last();
    st.rope_in_offset = sl.u64(ir::Start, 0);
    exe.steps[slice].skip = true;
    if (reshape < p.ops.size()) {
      exe.steps[reshape].alias = false; // nothing left to alias: neither tensor is materialised
      exe.steps[reshape].skip = true;
    }
  }
  // (2) this op [-> Concat along tokens] -> Attention q / k: write the INT8 codes the attention
  // kernel reads, straight into its scratch buffer
  size_t previous_attention = 0;
  bool seen_attention = false;
  for (size_t a = 0; a < p.ops.size(); ++a) {
    const ir::Op &att = p.ops[a];
    if (att.opcode != ir::Attention)
      continue;
    const size_t fence = seen_attention ? previous_attention : 0; // the scratch buffer is shared
    const bool has_fence = seen_attention;
    previous_attention = a;
    seen_attention = true;
    const ir::Tensor &q = *p.tensor(att.in[0]);
    const size_t token_axis = q.dims.size() - 3;
    for (int role = 0; role < 2; ++role) {
      const uint32_t id = att.in[(size_t)role];
      const auto it = producer.find(id);
      if (it == producer.end() || !private_to(id, a))
        continue;
      std::vector<std::pair<size_t, uint64_t>> parts; // rope step, first output token
      size_t concat = p.ops.size();
      const ir::Op &src = p.ops[it->second];
      if (src.opcode == ir::QkNormPartialRope) {
        parts.push_back({it->second, 0});
      } else if (src.opcode == ir::Concat && src.u64(ir::Axis, 0) == token_axis) {
        concat = it->second;
        uint64_t start = 0;
        bool ok = true;
        for (auto part : src.in) {
          const auto pr = producer.find(part);
          if (pr == producer.end() || p.ops[pr->second].opcode != ir::QkNormPartialRope ||
              !private_to(part, concat)) {
            ok = false;
            break;
          }
          parts.push_back({pr->second, start});
          start += p.tensor(part)->dims[token_axis];
        }
        if (!ok)
          continue;
      } else {
        continue;
      }
      bool ok = !parts.empty();
      for (const auto &part : parts)
        ok = ok && rope_kernel_covers(p.ops[part.first]) && exe.steps[part.first].rope_attention < 0 &&
             (!has_fence || part.first > fence) && part.first < a;
      if (!ok)
        continue;
      for (const auto &part : parts) {
        Step &st = exe.steps[part.first];
        st.rope_attention = (int)a;
        st.rope_role = role;
        st.rope_out_seq = q.dims[token_axis];
        st.rope_out_start = part.second;
      }
      if (concat < p.ops.size())
        exe.steps[concat].skip = true;
      (role == 0 ? exe.steps[a].q_quantised : exe.steps[a].k_quantised) = true;
    }
  }
}


// ---- token-sharded mode: which Attention ops gather their keys / values over the world, when the
// ring exchanges start, and the order in which the steps in front of an attention run ----
void plan_world(Executable &exe) {
  const ir::Program &p = exe.program;
  exe.order.resize(exe.steps.size());
  for (size_t i = 0; i < exe.order.size(); ++i)
    exe.order[i] = i;
  World *world = exe.ctx->world;
  if (!world || world->size <= 1)
    return;
  std::map<uint32_t, size_t> producer;
  for (size_t i = 0; i < p.ops.size(); ++i)
    for (auto id : p.ops[i].out)
      producer[id] = i;
  size_t window_begin = 0; // steps before this index keep their place (they belong to an earlier attention)
  for (size_t a = 0; a < p.ops.size(); ++a) {
    const ir::Op &att = p.ops[a];
    Step &st = exe.steps[a];
    if (att.opcode != ir::Attention || st.skip)
      continue;
    const ir::Tensor &q = *p.tensor(att.in[0]);
    const bool batched = q.dims.size() == 4;
    if ((batched && q.dims[0] != 1) || st.mask_tensor >= 0 || att.in.size() != 3)
      throw PluginError{2, "Attention (op " + std::to_string(att.id) + "): the token-sharded mode covers one "
                               "sequence per program (no batch axis above 1) without a key mask"};
    Sharded sh;
    sh.step = a;
    sh.tokens = q.dims[batched ? 1 : 0];
    sh.heads = q.dims[batched ? 2 : 1];
    sh.kv_heads = att.u64(ir::KvHeads, sh.heads);
    const int index = (int)exe.sharded.size();
    st.sharded = index;
    // K: final after the last QkNormPartialRope part that writes its codes; else at the attention itself
    if (st.k_quantised) {
      int last = -1;
      for (size_t r = 0; r < a; ++r)
        if (exe.steps[r].rope_attention == (int)a && exe.steps[r].rope_role == 1)
          last = (int)r;
      if (last >= 0)
        exe.steps[(size_t)last].exchange_k_for = index;
    }
    // V: the buffer of the tensor behind the chain of aliasing Reshapes becomes this rank's slice
    uint32_t v_id = att.in[2];
    for (;;) {
      const auto it = producer.find(v_id);
      if (it == producer.end() || !exe.steps[it->second].alias)
        break;
      v_id = p.ops[it->second].in[0];
    }
    const ir::Tensor &v_root = *p.tensor(v_id);
    if (!v_root.has(ir::Input) && !v_root.has(ir::Constant) && producer.count(v_id)) {
      const int root = p.index_of(v_id);
      for (size_t k = 0; k < a; ++k) {
        const Step &cand = exe.steps[k];
        const bool writes = !cand.skip && (cand.out_tensor == root ||
                                           std::find(cand.op->out.begin(), cand.op->out.end(), v_id) != cand.op->out.end());
        if (writes) {
          sh.v_root = root;
          exe.steps[k].exchange_v_for = index;
        }
      }
    }
    exe.sharded.push_back(sh);

    // Order of the steps in [window_begin, a): whatever several operands need first, then the V
    // chain, the K chain, the Q chain, then steps the attention does not depend on. Each class
    // keeps its program order, so every step still runs after the steps it reads from.
    std::vector<unsigned> klass(a, 0u);
    for (unsigned operand = 0; operand < 3; ++operand) {
      std::vector<uint32_t> todo{att.in[operand]};
      while (!todo.empty()) {
        const uint32_t id = todo.back();
        todo.pop_back();
        const auto it = producer.find(id);
        if (it == producer.end() || it->second >= a || (klass[it->second] & (1u << operand)))
          continue;
        klass[it->second] |= 1u << operand;
        for (auto in : p.ops[it->second].in)
          todo.push_back(in);
      }
    }
    auto rank_of = [&](size_t i) {
      switch (klass[i]) {
      case 4u: return 1; // V only (operand index 2)
      case 2u: return 2; // K only
      case 1u: return 3; // Q only
      case 0u: return 4; // not needed by this attention
      default: return 0; // shared by several operands
      }
    };
    std::stable_sort(exe.order.begin() + (long)window_begin, exe.order.begin() + (long)a,
                     [&](size_t x, size_t y) { return rank_of(x) < rank_of(y); });
    window_begin = a + 1;
  }
}

// Token-sharded mode: the ranks agree on a common padded slice length, then every sharded
// Attention gets its gather buffers (zeroed once: padding rows must stay finite, a masked key still
// multiplies its value row by zero), the validity mask of the gathered key axis, the local query
// codes, the key table scratch and the state carried between attention launches.
void allocate_world(Executable &exe) {
  World *world = exe.ctx->world;
  if (exe.sharded.empty() || !world)
    return;
  const uint64_t size = (uint64_t)world->size;
  auto device_alloc = [&](size_t bytes, bool zero) {
    void *ptr = nullptr;
    require_cuda(cudaMalloc(&ptr, bytes ? bytes : 16), "cudaMalloc(token-sharded attention)");
    exe.world_buffers.push_back(ptr);
    exe.resident_bytes += bytes;
    if (zero)
      require_cuda(cudaMemsetAsync(ptr, 0, bytes ? bytes : 16, exe.ctx->stream), "cudaMemsetAsync");
    return ptr;
  };
  for (Sharded &sh : exe.sharded) {
    // every rank's token count, through the world's own exchange
    std::vector<uint64_t> tokens(size);
    require(world_all_gather_host(world, &sh.tokens, tokens.data(), sizeof(uint64_t), exe.ctx->stream));
    uint64_t longest = 0;
    for (uint64_t t : tokens)
      longest = t > longest ? t : longest;
    sh.slice_tokens = (longest + 127) / 128 * 128;
    const uint64_t keys = size * sh.slice_tokens, KV = sh.kv_heads;
    // one block for the three gather buffers: with the direct exchange the peers map it as a whole
    auto aligned = [](uint64_t bytes) { return (bytes + 255) / 256 * 256; };
    sh.at_v = 0;
    sh.at_k8 = sh.at_v + aligned(keys * KV * 256);
    sh.at_ks = sh.at_k8 + aligned(keys * KV * 128);
    require(world_bind(world, (size_t)(sh.at_ks + aligned(keys * KV * sizeof(float))), exe.ctx->stream, &sh.binding));
    exe.resident_bytes += sh.binding->block_bytes;
    sh.binding->timed = exe.profile;
    char *block = static_cast<char *>(sh.binding->block);
    sh.v = block + sh.at_v;
    sh.k8 = reinterpret_cast<int8_t *>(block + sh.at_k8);
    sh.ks = reinterpret_cast<float *>(block + sh.at_ks);
    sh.q8 = static_cast<int8_t *>(device_alloc(sh.tokens * sh.heads * 128, false));
    sh.qs = static_cast<float *>(device_alloc(sh.tokens * sh.heads * sizeof(float), false));
    sh.scratch_bytes = attention_int8_scratch_bytes(1, keys, KV);
    sh.scratch = device_alloc(sh.scratch_bytes, false);
    sh.state = device_alloc(attention_int8_state_bytes(1, sh.tokens, sh.heads), false);
    std::vector<uint8_t> valid(keys, 0);
    for (uint64_t r = 0; r < size; ++r)
      for (uint64_t t = 0; t < tokens[r]; ++t)
        valid[r * sh.slice_tokens + t] = 1;
    sh.valid = static_cast<uint8_t *>(device_alloc(keys, false));
    require_cuda(cudaMemcpyAsync(sh.valid, valid.data(), keys, cudaMemcpyHostToDevice, exe.ctx->stream),
                 "cudaMemcpyAsync(key validity)");
    require_cuda(cudaStreamSynchronize(exe.ctx->stream), "cudaStreamSynchronize");
    if (sh.v_root >= 0) {
      exe.dev[(size_t)sh.v_root] = static_cast<char *>(sh.v) + (uint64_t)world->rank * sh.slice_tokens * KV * 256;
      exe.owned[(size_t)sh.v_root] = 0;
    }
  }
}

void allocate(Executable &exe) {
  const ir::Program &p = exe.program;
  const size_t n = p.tensors.size();
  exe.dev.assign(n, nullptr);
  // Reshape outputs share the buffer of their input: every tensor belongs to the group of its root
  std::vector<size_t> root(n);
  for (size_t i = 0; i < n; ++i)
    root[i] = i;
  for (const Step &st : exe.steps)
    if (st.alias)
      root[(size_t)p.index_of(st.op->out[0])] = root[(size_t)p.index_of(st.op->in[0])];
  std::vector<size_t> position(exe.steps.size(), 0); // when a step runs (exe.order)
  for (size_t k = 0; k < exe.order.size(); ++k)
    position[exe.order[k]] = k;
  // tensors produced only by skipped ops are never materialised; for the others, the first and
  // the last step that touches their buffer
  const size_t never = ~(size_t)0;
  std::vector<bool> needed(n, false);
  std::vector<size_t> first(n, never), last(n, 0);
  for (size_t i = 0; i < n; ++i)
    if (p.tensors[i].has(ir::Input) || p.tensors[i].has(ir::Constant) || p.tensors[i].has(ir::Output))
      needed[i] = true;
  for (size_t step = 0; step < exe.steps.size(); ++step) {
    const Step &st = exe.steps[step];
    auto touch = [&](int tensor) {
      needed[(size_t)tensor] = true;
      const size_t r = root[(size_t)tensor], at = position[step];
      first[r] = first[r] == never || at < first[r] ? at : first[r];
      last[r] = at > last[r] ? at : last[r];
    };
    if (st.alias)
      needed[(size_t)p.index_of(st.op->in[0])] = true;
    if (st.skip)
      continue;
    for (size_t k = 0; k < st.op->in.size(); ++k) {
      const uint32_t id = st.op->in[k];
      // inputs that a fused step does not read: the materialised attention bias, q / k that
      // arrive as INT8 codes in the scratch buffer, the slice a rope op reads in place
      if (st.op->opcode == ir::Attention && ((st.mask_tensor >= 0 && k == 3) || (st.q_quantised && k == 0) ||
                                             (st.k_quantised && k == 1)))
        continue;
      if (st.op->opcode == ir::QkNormPartialRope && st.rope_source >= 0 && k == 0) {
        touch(st.rope_source);
        continue;
      }
      if (st.op->opcode == ir::QuantizeInt8Rows && st.norm_step >= 0) { // reads the norm's inputs instead
        for (auto nid : exe.steps[(size_t)st.norm_step].op->in)
          touch(p.index_of(nid));
        continue;
      }
      touch(p.index_of(id));
    }
    if (st.op->opcode == ir::LinearInt8Scaled) {
      touch(st.out_tensor);
      if (st.bias_tensor >= 0)
        touch(st.bias_tensor);
    } else if (st.op->opcode == ir::QkNormPartialRope && st.rope_attention >= 0) {
      // writes INT8 codes into the attention scratch buffer, no bf16 tensor
    } else {
      for (auto id : st.op->out)
        touch(p.index_of(id));
    }
    if (st.mask_tensor >= 0)
      touch(st.mask_tensor);
  }
  std::vector<bool> aliased(n, false);
  for (const Step &st : exe.steps)
    if (st.alias)
      aliased[(size_t)p.index_of(st.op->out[0])] = true;
  exe.owned.assign(n, 1);
  for (const Sharded &sh : exe.sharded) // lives inside the gather buffer (allocate_world)
    if (sh.v_root >= 0)
      aliased[(size_t)sh.v_root] = true;
  // Internal tensors whose lifetimes do not overlap share device memory: a sweep over the step
  // positions takes a block for every tensor at its first step (the smallest free block that holds
  // it without wasting more than its size again, else a new allocation) and returns the blocks of
  // the tensors whose last step this was. A block freed by a step is never handed to an output of
  // the same step, so no kernel runs in place. Inputs, Outputs, Constants and every group with such
  // a member keep buffers of their own (copies on other streams touch them).
  // DIFB200_BUFFER_REUSE=0 gives every tensor its own allocation.
  const char *reuse_env = std::getenv("DIFB200_BUFFER_REUSE");
  const bool reuse = !(reuse_env && reuse_env[0] == '0');
  std::vector<bool> pinned(n, false);
  for (size_t i = 0; i < n; ++i)
    if (p.tensors[i].has(ir::Input) || p.tensors[i].has(ir::Constant) || p.tensors[i].has(ir::Output))
      pinned[root[i]] = true;
  std::vector<std::vector<size_t>> born(exe.order.size()), dying(exe.order.size());
  for (size_t i = 0; i < n; ++i) {
    if (!needed[i] || aliased[i])
      continue;
    const size_t bytes = (size_t)p.tensors[i].bytes();
    if (!reuse || pinned[i] || first[i] == never) {
      require_cuda(cudaMalloc(&exe.dev[i], bytes ? bytes : 16), "cudaMalloc(tensor)");
      exe.resident_bytes += bytes;
    } else {
      born[first[i]].push_back(i);
      dying[last[i]].push_back(i);
    }
  }
  struct Block {
    void *ptr;
    size_t bytes;
  };
  std::vector<Block> free_blocks;
  std::vector<Block> block_of(n, Block{nullptr, 0});
  for (size_t k = 0; k < exe.order.size(); ++k) {
    for (size_t i : born[k]) {
      const size_t bytes = (size_t)p.tensors[i].bytes() ? (size_t)p.tensors[i].bytes() : 16;
      size_t best = free_blocks.size();
      for (size_t b = 0; b < free_blocks.size(); ++b)
        if (free_blocks[b].bytes >= bytes && free_blocks[b].bytes <= 2 * bytes &&
            (best == free_blocks.size() || free_blocks[b].bytes < free_blocks[best].bytes))
          best = b;
      if (best < free_blocks.size()) {
        block_of[i] = free_blocks[best];
        free_blocks.erase(free_blocks.begin() + (long)best);
      } else {
        void *ptr = nullptr;
        require_cuda(cudaMalloc(&ptr, bytes), "cudaMalloc(tensor)");
        exe.world_buffers.push_back(ptr); // freed with the executable
        exe.resident_bytes += bytes;
        block_of[i] = Block{ptr, bytes};
      }
      exe.dev[i] = block_of[i].ptr;
      exe.owned[i] = 0;
    }
    for (size_t i : dying[k])
      free_blocks.push_back(block_of[i]);
  }
  allocate_world(exe);
  for (const Step &st : exe.steps) // program order: a chain of reshapes resolves front to back
    if (st.alias) {
      const size_t out = (size_t)p.index_of(st.op->out[0]);
      exe.dev[out] = exe.dev[(size_t)p.index_of(st.op->in[0])];
      exe.owned[out] = 0;
    }
  size_t scratch = 0;
  for (const Step &st : exe.steps) {
    if (st.skip || st.op->opcode != ir::Attention || st.sharded >= 0)
      continue;
    const ir::Tensor &q = *p.tensor(st.op->in[0]);
    const bool batched = q.dims.size() == 4;
    const uint64_t B = batched ? q.dims[0] : 1, S = q.dims[batched ? 1 : 0], H = q.dims[batched ? 2 : 1];
    const uint64_t KV = st.op->u64(ir::KvHeads, H);
    const size_t need = attention_scratch_bytes(B, S, H, KV);
    scratch = need > scratch ? need : scratch;
  }
  if (scratch) {
    require_cuda(cudaMalloc(&exe.attn_scratch, scratch), "cudaMalloc(attention scratch)");
    exe.attn_scratch_bytes = scratch;
    exe.resident_bytes += scratch;
  }
  require_cuda(cudaMalloc(&exe.flag, sizeof(unsigned int)), "cudaMalloc(flag)");
  require_cuda(cudaMemset(exe.flag, 0, sizeof(unsigned int)), "cudaMemset(flag)");
}

// State of an overlapped execute (one pass, copies on their own streams): which Input tensors'
// uploads the kernel stream has not yet waited for, and the order in which Output tensors
// became final.
struct Overlap {
  std::vector<uint8_t> upload_pending;
  std::vector<int> finished_outputs;
};

// DIFB200_PROFILE: an event on the kernel stream in front of the next step (opcode 0 closes a pass).
void profile_mark(Executable &exe, uint32_t opcode) {
  const size_t at = exe.profile_opcodes.size();
  if (at >= exe.profile_events.size()) {
    cudaEvent_t e = nullptr;
    require_cuda(cudaEventCreate(&e), "cudaEventCreate(profile)");
    exe.profile_events.push_back(e);
  }
  require_cuda(cudaEventRecord(exe.profile_events[at], exe.ctx->stream), "cudaEventRecord(profile)");
  exe.profile_opcodes.push_back(opcode);
}
// After the pass has finished on the device: add the spans to the per-opcode sums.
void profile_collect(Executable &exe) {
  for (size_t i = 0; i + 1 < exe.profile_opcodes.size(); ++i) {
    float ms = 0.0f;
    if (exe.profile_opcodes[i] == 0)
      continue; // the mark that closes a pass: what follows it belongs to no step
    if (cudaEventElapsedTime(&ms, exe.profile_events[i], exe.profile_events[i + 1]) == cudaSuccess) {
      auto &sum = exe.profile_sum[exe.profile_opcodes[i]];
      sum.first += ms;
      sum.second += 1;
    }
  }
  exe.profile_opcodes.clear();
}

// ---- one pass over the program ---------------------------------------------------------------
void run_steps(Executable &exe, Overlap *overlap = nullptr) {
  const ir::Program &p = exe.program;
  cudaStream_t s = exe.ctx->stream;
  auto D = [&](uint32_t id) -> void * { return exe.dev[(size_t)p.index_of(id)]; };
  auto T = [&](uint32_t id) -> const ir::Tensor & { return *p.tensor(id); };
  auto await_upload = [&](int idx) {
    if (idx >= 0 && overlap->upload_pending[(size_t)idx]) {
      require_cuda(cudaStreamWaitEvent(s, exe.uploaded[(size_t)idx], 0), "cudaStreamWaitEvent(upload)");
      overlap->upload_pending[(size_t)idx] = 0;
    }
  };
  World *world = exe.ctx->world;
  // token-sharded mode: this rank's slice of a gather buffer is final, its ring exchange starts
  auto exchange = [&](const Sharded &sh, int which) {
    const uint64_t KV = sh.kv_heads, rows = sh.slice_tokens;
    const bool direct = sh.binding && sh.binding->direct;
    if (which == 0) {
      void *buffers[1] = {sh.v};
      const uint64_t bytes[1] = {rows * KV * 256}, at[1] = {sh.at_v};
      require(direct ? world_push(world, sh.binding, 0, at, bytes, 1, s)
                     : world_exchange_class(world, 0, buffers, bytes, 1, s));
    } else {
      void *buffers[2] = {sh.k8, sh.ks};
      const uint64_t bytes[2] = {rows * KV * 128, rows * KV * sizeof(float)}, at[2] = {sh.at_k8, sh.at_ks};
      require(direct ? world_push(world, sh.binding, 1, at, bytes, 2, s)
                     : world_exchange_class(world, 1, buffers, bytes, 2, s));
    }
  };
  // where the INT8 operands of an Attention live: its scratch buffer, or (token-sharded) the local
  // query buffers and this rank's slice of the gathered key buffers
  auto operands_of = [&](size_t attention_step) {
    const Step &at = exe.steps[attention_step];
    const ir::Tensor &q = T(at.op->in[0]);
    const bool batched = q.dims.size() == 4;
    const uint64_t B = batched ? q.dims[0] : 1, S = q.dims[batched ? 1 : 0], H = q.dims[batched ? 2 : 1];
    if (at.sharded < 0)
      return attention_scratch_layout(exe.attn_scratch, B, S, H, at.op->u64(ir::KvHeads, H));
    const Sharded &sh = exe.sharded[(size_t)at.sharded];
    const uint64_t first = (uint64_t)world->rank * sh.slice_tokens * sh.kv_heads;
    AttentionScratch l{};
    l.q8 = sh.q8;
    l.qs = sh.qs;
    l.k8 = sh.k8 + first * 128;
    l.ks = sh.ks + first;
    l.rest = sh.scratch;
    return l;
  };
  for (size_t position = 0; position <= exe.order.size(); ++position) {
    if (overlap && position > 0) {
      // every Output tensor the previous op (run, fused away or skipped) lists is final now
      for (auto id : exe.steps[exe.order[position - 1]].op->out) {
        const int idx = p.index_of(id);
        if (idx >= 0 && p.tensors[(size_t)idx].has(ir::Output) && exe.dev[(size_t)idx]) {
          require_cuda(cudaEventRecord(exe.produced[(size_t)idx], s), "cudaEventRecord(output)");
          overlap->finished_outputs.push_back(idx);
        }
      }
    }
    if (position == exe.order.size())
      break;
    const Step &st = exe.steps[exe.order[position]];
    if (overlap) {
      for (auto id : st.op->in)
        await_upload(p.index_of(id));
      await_upload(st.bias_tensor);
      await_upload(st.mask_tensor);
    }
    if (st.skip)
      continue;
    const ir::Op &op = *st.op;
    if (exe.profile_pass)
      profile_mark(exe, op.opcode);
    switch (op.opcode) {
    case ir::QuantizeInt8Rows: {
      if (st.norm_step >= 0) {
        const ir::Op &norm = *exe.steps[(size_t)st.norm_step].op;
        const bool weighted = norm.in.size() == 4;
        NormPrologue prologue{weighted ? D(norm.in[1]) : nullptr, D(norm.in[weighted ? 2 : 1]),
                              D(norm.in[weighted ? 3 : 2]), (float)norm.f64(ir::Epsilon, 1.0e-5)};
        if (norm.opcode == ir::LayerNormModulate)
          prologue = NormPrologue{D(norm.in[1]), D(norm.in[3]), D(norm.in[4]), (float)norm.f64(ir::Epsilon, 1.0e-5),
                                  D(norm.in[2]), T(norm.in[0]).rows() / T(norm.in[3]).rows()};
        const void *part = D(norm.in[0]);
        const uint64_t width = T(norm.in[0]).last();
        require(quantize_int8_rows(&part, &width, 1, T(norm.in[0]).rows(), (int)op.u64(ir::Implementation, 1),
                                   (float)op.f64(ir::Scale, 1.0), nullptr, static_cast<int8_t *>(D(op.out[0])),
                                   static_cast<float *>(D(op.out[1])), nullptr, nullptr, s, false, nullptr,
                                   &prologue));
        break;
      }
      const bool dynamic = T(op.in.back()).dtype == ir::F32;
      const size_t n_data = op.in.size() - (dynamic ? 1 : 0);
      const void *parts[8];
      uint64_t widths[8];
      for (size_t k = 0; k < n_data; ++k) {
        parts[k] = D(op.in[k]);
        widths[k] = T(op.in[k]).last();
      }
      const bool residual = op.out.size() == 4;
      require(quantize_int8_rows(parts, widths, (uint32_t)n_data, T(op.in[0]).rows(),
                                 (int)op.u64(ir::Implementation, 1), (float)op.f64(ir::Scale, 1.0),
                                 dynamic ? static_cast<const float *>(D(op.in.back())) : nullptr,
                                 static_cast<int8_t *>(D(op.out[0])), static_cast<float *>(D(op.out[1])),
                                 residual ? static_cast<int8_t *>(D(op.out[2])) : nullptr,
                                 residual ? static_cast<float *>(D(op.out[3])) : nullptr, s));
      break;
    }
    case ir::LinearInt8Scaled: {
      const ir::Tensor &x = T(op.in[0]), &w = T(op.in[1]);
      require(linear_int8_scaled(static_cast<const int8_t *>(D(op.in[0])), static_cast<const int8_t *>(D(op.in[1])),
                                 static_cast<const float *>(D(op.in[2])), static_cast<const float *>(D(op.in[3])),
                                 st.bias_tensor >= 0 ? exe.dev[(size_t)st.bias_tensor] : nullptr, st.epilogue,
                                 x.rows(), w.dims[0], w.dims[1], exe.dev[(size_t)st.out_tensor], nullptr, s));
      break;
    }
    case ir::Attention: {
      const ir::Tensor &q = T(op.in[0]);
      const bool batched = q.dims.size() == 4;
      const uint64_t B = batched ? q.dims[0] : 1, S = q.dims[batched ? 1 : 0], H = q.dims[batched ? 2 : 1];
      const uint64_t KV = op.u64(ir::KvHeads, H);
      const float scale = (float)op.f64(ir::AttentionScale, 1.0 / std::sqrt((double)q.last()));
      if (st.sharded >= 0) {
        const Sharded &sh = exe.sharded[(size_t)st.sharded];
        const AttentionScratch l = operands_of(exe.order[position]);
        const uint64_t width[1] = {128};
        if (!st.q_quantised) {
          const void *part[1] = {D(op.in[0])};
          require(quantize_int8_rows(part, width, 1, S * H, 1, 1.0f, nullptr, l.q8, l.qs, nullptr, nullptr, s));
        }
        if (!st.k_quantised) {
          const void *part[1] = {D(op.in[1])};
          require(quantize_int8_rows(part, width, 1, S * KV, 1, 1.0f, nullptr, l.k8, l.ks, nullptr, nullptr, s));
        }
        if (sh.v_root < 0) // V was not produced in place: copy this rank's rows into its slice
          require_cuda(cudaMemcpyAsync(static_cast<char *>(sh.v) + (uint64_t)world->rank * sh.slice_tokens * KV * 256,
                                       D(op.in[2]), (size_t)(S * KV * 256), cudaMemcpyDeviceToDevice, s),
                       "cudaMemcpyAsync(values into the gather buffer)");
        bool v_started = false, k_started = false; // exchanges a producer step has already started
        for (const Step &other : exe.steps) {
          v_started = v_started || other.exchange_v_for == st.sharded;
          k_started = k_started || other.exchange_k_for == st.sharded;
        }
        if (!v_started)
          exchange(sh, 0);
        if (!k_started)
          exchange(sh, 1);
        require(sharded_attention(world, sh.binding, l.q8, l.qs, sh.k8, sh.ks, sh.v, sh.valid, S, sh.slice_tokens, H, KV, scale,
                                  sh.scratch, sh.scratch_bytes, sh.state, D(op.out[0]), s));
        break;
      }
      require(attention_bf16_via_int8(st.q_quantised ? nullptr : D(op.in[0]), st.k_quantised ? nullptr : D(op.in[1]),
                                      D(op.in[2]),
                                      st.mask_tensor >= 0 ? static_cast<const uint8_t *>(exe.dev[(size_t)st.mask_tensor])
                                                          : nullptr,
                                      B, S, H, KV, q.last(), scale, exe.attn_scratch, exe.attn_scratch_bytes,
                                      D(op.out[0]), s));
      break;
    }
    case ir::Add:
    case ir::Multiply:
      require(glue::binary(D(op.in[0]), D(op.in[1]), D(op.out[0]), T(op.in[0]).dtype, T(op.in[0]).elements(),
                           op.opcode == ir::Multiply, s));
      break;
    case ir::Gelu:
      require(glue::unary(D(op.in[0]), D(op.out[0]), T(op.in[0]).dtype, T(op.out[0]).dtype, T(op.in[0]).elements(),
                          op.u64(ir::Approximation, 1) == 2 ? 2 : 1, s));
      break;
    case ir::SiLU:
    case ir::Sigmoid:
    case ir::Cast:
      require(glue::unary(D(op.in[0]), D(op.out[0]), T(op.in[0]).dtype, T(op.out[0]).dtype, T(op.in[0]).elements(),
                          op.opcode == ir::SiLU ? 3 : (op.opcode == ir::Sigmoid ? 4 : 0), s));
      break;
    case ir::BiasAdd:
      require(glue::bias_add(D(op.in[0]), D(op.in[1]), D(op.out[0]), T(op.in[0]).dtype, T(op.in[0]).elements(),
                             T(op.in[0]).last(), s));
      break;
    case ir::AffineLastDim:
      require(glue::affine_last_dim(D(op.in[0]), D(op.in[1]), op.in.size() == 3 ? D(op.in[2]) : nullptr, D(op.out[0]),
                                    T(op.in[0]).dtype, T(op.in[0]).elements(), T(op.in[0]).last(), s));
      break;
    case ir::Fill:
      require(glue::fill(D(op.out[0]), T(op.out[0]).dtype, T(op.out[0]).elements(), (float)op.f64(ir::Value, 0.0), s));
      break;
    case ir::RmsNorm:
      require(glue::rms_norm(D(op.in[0]), D(op.in[1]), D(op.out[0]), T(op.in[0]).dtype, T(op.in[0]).rows(),
                             T(op.in[0]).last(), (float)op.f64(ir::Epsilon, 1.0e-5),
                             (float)op.f64(ir::WeightOffset, 0.0), s));
      break;
    case ir::LayerNormModulate:
      require(glue::layer_norm_modulate(D(op.in[0]), D(op.in[1]), D(op.in[2]), D(op.in[3]), D(op.in[4]), D(op.out[0]),
                                        T(op.in[0]).dtype, T(op.in[0]).rows(), T(op.in[0]).last(),
                                        T(op.in[0]).rows() / T(op.in[3]).rows(), (float)op.f64(ir::Epsilon, 1.0e-5), s));
      break;
    case ir::RmsNormModulate: {
      const ir::Tensor &x = T(op.in[0]);
      const float eps = (float)op.f64(ir::Epsilon, 1.0e-5);
      if (op.u64(ir::ModulationLayout, 1) == 2) {
        require(glue::rms_norm_modulate(D(op.in[0]), D(op.in[1]), D(op.in[2]), D(op.in[3]), D(op.out[0]), x.dtype,
                                        x.dims[0], x.dims[1], eps, (float)op.f64(ir::WeightOffset, 0.0), true,
                                        x.dims[0] / T(op.in[2]).dims[0], s));
      } else {
        const bool weighted = op.in.size() == 4;
        require(glue::rms_norm_modulate(D(op.in[0]), weighted ? D(op.in[1]) : nullptr, D(op.in[weighted ? 2 : 1]),
                                        D(op.in[weighted ? 3 : 2]), D(op.out[0]), x.dtype, x.dims[0], x.dims[1], eps,
                                        0.0f, false, 1, s));
      }
      break;
    }
    case ir::QkNormPartialRope: {
      const ir::Tensor &x = T(op.in[0]), &c = T(op.in[2]);
      const uint64_t dim = x.last(), heads = x.dims[x.dims.size() - 2];
      const uint64_t tokens = x.elements() / (heads * dim);
      const uint64_t input_seq = x.dims.size() == 4 ? x.dims[1] : x.dims[0];
      const uint64_t table_seq = c.dims.size() == 3 ? c.dims[1] : c.dims[0];
      const bool v2 = op.u64(ir::Implementation, 1) == 2 && op.u64(ir::RotaryLayout, 2) == 1;
      const uint64_t rotary = op.u64(ir::RotaryDim, dim), start = op.u64(ir::Start, 0);
      const float eps = (float)op.f64(ir::Epsilon, 1.0e-5);
      if (st.rope_source < 0 && st.rope_attention < 0) {
        require(glue::qk_norm_rope(D(op.in[0]), D(op.in[1]), D(op.in[2]), D(op.in[3]), D(op.out[0]), x.dtype, c.dtype,
                                   tokens, heads, dim, rotary, c.last(), input_seq, table_seq, start, eps, v2, s));
        break;
      }
      // fused with a Slice before it and / or the Attention after it (see plan())
      glue::RopeLayout layout{heads * dim, 0, input_seq, 0};
      const void *source = D(op.in[0]);
      if (st.rope_source >= 0) {
        source = exe.dev[(size_t)st.rope_source];
        layout.in_token_stride = st.rope_in_stride;
        layout.in_offset = st.rope_in_offset;
      }
      void *out = nullptr;
      int8_t *codes = nullptr;
      float *scales = nullptr;
      if (st.rope_attention >= 0) {
        const AttentionScratch l = operands_of((size_t)st.rope_attention);
        codes = st.rope_role == 0 ? l.q8 : l.k8;
        scales = st.rope_role == 0 ? l.qs : l.ks;
        layout.out_seq = st.rope_out_seq;
        layout.out_start = st.rope_out_start;
      } else {
        out = D(op.out[0]);
      }
      int rc = 0;
      if (!glue::qk_norm_rope_fast(source, D(op.in[1]), D(op.in[2]), D(op.in[3]), out, codes, scales, x.dtype, c.dtype,
                                   tokens, heads, dim, rotary, c.last(), input_seq, table_seq, start, eps, v2, &layout,
                                   s, &rc))
        throw PluginError{6, "QkNormPartialRope (op " + std::to_string(op.id) + "): fused form not applicable"};
      require(rc);
      break;
    }
    case ir::RotaryFrequency: {
      const ir::Tensor &pos = T(op.in[0]);
      require(glue::rotary_frequency(static_cast<const float *>(D(op.in[0])), static_cast<const int32_t *>(D(op.in[1])),
                                     static_cast<const int32_t *>(D(op.in[2])), static_cast<const int32_t *>(D(op.in[3])),
                                     static_cast<float *>(D(op.out[0])), static_cast<float *>(D(op.out[1])),
                                     pos.dims[0] * pos.dims[1], pos.dims[2], T(op.in[1]).dims[0],
                                     op.f64(ir::Theta, 10000.0) * op.f64(ir::Ntk, 1.0), exe.flag, s));
      break;
    }
    case ir::RotaryApply: {
      const ir::Tensor &x = T(op.in[0]);
      require(glue::rotary_apply(D(op.in[0]), static_cast<const float *>(D(op.in[1])),
                                 static_cast<const float *>(D(op.in[2])), D(op.out[0]), x.dtype,
                                 x.dims[0] * x.dims[1], x.dims[2], x.dims[3], T(op.in[1]).dims[2], s));
      break;
    }
    case ir::ResidualGate: {
      const ir::Tensor &r = T(op.in[0]);
      require(glue::residual_gate(D(op.in[0]), D(op.in[1]), D(op.in[2]), D(op.out[0]), r.dtype, r.elements(), r.last(),
                                  r.rows() / T(op.in[2]).rows(), s));
      break;
    }
    case ir::SwiGlu: {
      const ir::Tensor &o = T(op.out[0]);
      require(glue::swiglu(D(op.in[0]), D(op.out[0]), o.dtype, o.rows(), o.last(), T(op.in[0]).last(),
                           op.u64(ir::Start, 0), op.boolean(ir::GateFirst, false), s));
      break;
    }
    case ir::Reshape:
      require_cuda(cudaMemcpyAsync(D(op.out[0]), D(op.in[0]), (size_t)T(op.out[0]).bytes(), cudaMemcpyDeviceToDevice, s),
                   "cudaMemcpyAsync(reshape)");
      break;
    case ir::Slice: {
      // one axis of a contiguous tensor: `outer` runs of `run` bytes, `pitch` bytes apart in the source
      const ir::Tensor &x = T(op.in[0]), &o = T(op.out[0]);
      const uint64_t axis = op.u64(ir::Axis, 0), elem = ir::dtype_size(o.dtype);
      uint64_t outer = 1, inner = elem;
      for (size_t a = 0; a < axis; ++a)
        outer *= o.dims[a];
      for (size_t a = axis + 1; a < o.dims.size(); ++a)
        inner *= o.dims[a];
      const uint64_t run = o.dims[axis] * inner, pitch = x.dims[axis] * inner;
      const char *src = static_cast<const char *>(D(op.in[0])) + op.u64(ir::Start, 0) * inner;
      if (run && outer)
        require_cuda(cudaMemcpy2DAsync(D(op.out[0]), (size_t)run, src, (size_t)pitch, (size_t)run, (size_t)outer,
                                       cudaMemcpyDeviceToDevice, s),
                     "cudaMemcpy2DAsync(slice)");
      break;
    }
    case ir::BroadcastTo: {
      const ir::Tensor &x = T(op.in[0]), &o = T(op.out[0]);
      uint64_t in_strides[8] = {0}, full[8] = {0};
      const size_t rank = o.dims.size(), pad = rank - x.dims.size();
      uint64_t stride = 1;
      for (size_t a = x.dims.size(); a-- > 0;) {
        full[a] = stride;
        stride *= x.dims[a];
      }
      for (size_t a = 0; a < rank; ++a)
        in_strides[a] = (a < pad || x.dims[a - pad] == 1) ? 0 : full[a - pad];
      require(glue::gather(D(op.in[0]), D(op.out[0]), (uint32_t)ir::dtype_size(o.dtype), (uint32_t)rank,
                           o.dims.data(), in_strides, 0, s));
      break;
    }
    case ir::Concat: {
      const ir::Tensor &o = T(op.out[0]);
      const uint64_t axis = op.u64(ir::Axis, 0), elem = ir::dtype_size(o.dtype);
      uint64_t outer = 1, inner = elem;
      for (size_t a = 0; a < axis; ++a)
        outer *= o.dims[a];
      for (size_t a = axis + 1; a < o.dims.size(); ++a)
        inner *= o.dims[a];
      const uint64_t pitch = o.dims[axis] * inner;
      uint64_t offset = 0;
      for (auto id : op.in) {
        const uint64_t chunk = T(id).dims[axis] * inner;
        if (chunk && outer)
          require_cuda(cudaMemcpy2DAsync(static_cast<char *>(D(op.out[0])) + offset, (size_t)pitch, D(id),
                                         (size_t)chunk, (size_t)chunk, (size_t)outer, cudaMemcpyDeviceToDevice, s),
                       "cudaMemcpy2DAsync(concat)");
        offset += chunk;
      }
      break;
    }
    case ir::BooleanMaskToBias: {
      const ir::Tensor &m = T(op.in[0]), &o = T(op.out[0]);
      require(glue::mask_to_bias(static_cast<const uint8_t *>(D(op.in[0])), D(op.out[0]), o.dtype, o.dims[0], o.dims[2],
                                 m.dims.size() == 2, op.boolean(ir::MaskQueries, true), s));
      break;
    }
    case ir::Linear: {
      const ir::Tensor &x = T(op.in[0]), &w = T(op.in[1]);
      require(glue::linear(D(op.in[0]), D(op.in[1]), op.in.size() == 3 ? D(op.in[2]) : nullptr, D(op.out[0]), x.dtype,
                           x.dims[0], w.dims[0], w.dims[1], s));
      break;
    }
    default:
      throw PluginError{2, std::string("unsupported opcode ") + ir::opcode_name(op.opcode)};
    }
    if (st.exchange_v_for >= 0)
      exchange(exe.sharded[(size_t)st.exchange_v_for], 0);
    if (st.exchange_k_for >= 0)
      exchange(exe.sharded[(size_t)st.exchange_k_for], 1);
  }
}

// ---- ABI functions ----------------------------------------------------------------------------
template <typename F>
dif_backend_status guarded(dif_backend_error *error, F &&body) {
  try {
    body();
    return DIF_BACKEND_OK;
  } catch (const PluginError &e) {
    write_error(error, e.text);
    return status_of(e.status);
  } catch (const std::bad_alloc &) {
    write_error(error, "host allocation failed");
    return DIF_BACKEND_OUT_OF_MEMORY;
  } catch (const std::exception &e) {
    write_error(error, std::string("internal error: ") + e.what());
    return DIF_BACKEND_INTERNAL_ERROR;
  } catch (...) {
    write_error(error, "internal error");
    return DIF_BACKEND_INTERNAL_ERROR;
  }
}

dif_backend_status create(int32_t device_ordinal, dif_backend_context *context, dif_backend_error *error) {
  return guarded(error, [&] {
    if (!context)
      throw PluginError{1, "create: null context pointer"};
    *context = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
      throw PluginError{2, "no CUDA device is available (this backend has no CPU path)"};
    if (device_ordinal < 0 || device_ordinal >= count)
      throw PluginError{1, "create: device ordinal out of range"};
    cudaDeviceProp prop{};
    require_cuda(cudaGetDeviceProperties(&prop, device_ordinal), "cudaGetDeviceProperties");
    if (prop.major != 10)
      throw PluginError{2, std::string("device '") + prop.name + "' is not sm_100 (B200); this backend is sm_100a only"};
    auto ctx = std::make_unique<Context>();
    ctx->device = device_ordinal;
    require_cuda(cudaSetDevice(device_ordinal), "cudaSetDevice");
    require_cuda(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking), "cudaStreamCreate");
    require_cuda(cudaStreamCreateWithFlags(&ctx->h2d, cudaStreamNonBlocking), "cudaStreamCreate");
    require_cuda(cudaStreamCreateWithFlags(&ctx->d2h, cudaStreamNonBlocking), "cudaStreamCreate");
    // token-sharded mode: join the world the environment describes (bounded rendezvous, then NCCL)
    World *world = nullptr;
    require(world_from_environment(&world));
    ctx->world = world;
    *ctx->world_alive = world != nullptr;
    if (world)
      std::snprintf(ctx->device_name, sizeof(ctx->device_name),
                    "%.180s (difb200 sm_100a, int8-attention %s, token-sharded rank %d of %d)", prop.name,
                    int8_attention_enabled() ? "on" : "off", world->rank, world->size);
    else
      std::snprintf(ctx->device_name, sizeof(ctx->device_name), "%.200s (difb200 sm_100a, int8-attention %s)",
                    prop.name, int8_attention_enabled() ? "on" : "off");
    *context = ctx.release();
  });
}

void destroy(dif_backend_context context) {
  Context *ctx = static_cast<Context *>(context);
  if (!ctx)
    return;
  cudaSetDevice(ctx->device);
  *ctx->world_alive = false;
  delete ctx->world; // the communicator and its stream go first
  if (ctx->stream)
    cudaStreamDestroy(ctx->stream);
  if (ctx->h2d)
    cudaStreamDestroy(ctx->h2d);
  if (ctx->d2h)
    cudaStreamDestroy(ctx->d2h);
  delete ctx;
}

// Returns the tensor's index. The copy goes to `stream` (default: the kernel stream).
int upload(Executable &exe, const dif_backend_tensor_view &view, uint32_t role, const char *what,
           cudaStream_t stream = nullptr) {
  const int idx = exe.program.index_of(view.tensor_id);
  if (idx < 0)
    throw PluginError{1, std::string(what) + ": unknown tensor id " + std::to_string(view.tensor_id)};
  const ir::Tensor &t = exe.program.tensors[(size_t)idx];
  if (!t.has(role) || view.dtype != t.dtype || view.byte_count != t.bytes() || (!view.host_data && t.bytes()))
    throw PluginError{1, std::string(what) + ": tensor " + std::to_string(view.tensor_id) +
                             " does not match the program (role, dtype or byte count)"};
  if (exe.dev[(size_t)idx] && t.bytes())
    require_cuda(cudaMemcpyAsync(exe.dev[(size_t)idx], view.host_data, (size_t)t.bytes(), cudaMemcpyHostToDevice,
                                 stream ? stream : exe.ctx->stream),
                 "cudaMemcpyAsync(host to device)");
  return idx;
}

dif_backend_status compile_common(dif_backend_context context, const uint8_t *diffir, size_t size,
                                  const dif_backend_tensor_view *constants, size_t constant_count, bool v2,
                                  uint64_t minimum_free, dif_backend_executable *executable,
                                  dif_backend_compile_telemetry_v2 *telemetry, dif_backend_error *error) {
  return guarded(error, [&] {
    Context *ctx = static_cast<Context *>(context);
    if (!ctx || !diffir || !executable)
      throw PluginError{1, "compile: null argument"};
    *executable = nullptr;
    require_cuda(cudaSetDevice(ctx->device), "cudaSetDevice");
    EventPair events; // destroyed on every way out, a failed compile included
    require_cuda(cudaEventCreate(&events.a), "cudaEventCreate");
    require_cuda(cudaEventCreate(&events.b), "cudaEventCreate");
    const cudaEvent_t e0 = events.a, e1 = events.b;
    cudaEventRecord(e0, ctx->stream);
    size_t free_before = 0, total = 0;
    cudaMemGetInfo(&free_before, &total);
    auto exe = std::make_unique<Executable>();
    exe->ctx = ctx;
    exe->device = ctx->device;
    exe->world = ctx->world;
    exe->world_alive = ctx->world_alive;
    if (const char *v = std::getenv("DIFB200_PROFILE"))
      exe->profile = v[0] == '1';
    std::string text;
    if (int rc = ir::decode(diffir, size, exe->program, text))
      throw PluginError{rc == 2 ? 2 : 4, "DiffIR: " + text};
    plan(*exe);
    plan_world(*exe);
    allocate(*exe);
    if (v2) {
      size_t expected = 0;
      for (const auto &t : exe->program.tensors)
        expected += t.has(ir::Constant) ? 1 : 0;
      if (constant_count != expected || (expected && !constants))
        throw PluginError{1, "compile: expected " + std::to_string(expected) + " constant views, got " +
                                 std::to_string(constant_count)};
      for (size_t i = 0; i < constant_count; ++i)
        upload(*exe, constants[i], ir::Constant, "compile");
      exe->constants_bound = true;
    }
    require_cuda(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
    size_t free_after = 0;
    cudaMemGetInfo(&free_after, &total);
    if (free_after < minimum_free)
      throw PluginError{3, "compile: free device memory fell below minimum_free_bytes"};
    cudaEventRecord(e1, ctx->stream);
    cudaEventSynchronize(e1);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    if (telemetry) {
      telemetry->preparation_milliseconds = ms;
      telemetry->resident_bytes = exe->resident_bytes;
      telemetry->free_bytes_before = free_before;
      telemetry->free_bytes_after = free_after;
      std::memcpy(telemetry->device_name, ctx->device_name, sizeof(telemetry->device_name));
    }
    *executable = exe.release();
  });
}

dif_backend_status compile_v2(dif_backend_context context, const uint8_t *diffir, size_t size,
                              const dif_backend_tensor_view *constants, size_t constant_count,
                              const dif_backend_compile_options_v2 *options, dif_backend_executable *executable,
                              dif_backend_compile_telemetry_v2 *telemetry, dif_backend_error *error) {
  return compile_common(context, diffir, size, constants, constant_count, true,
                        options ? options->minimum_free_bytes : 0, executable, telemetry, error);
}
dif_backend_status compile_v1(dif_backend_context context, const uint8_t *diffir, size_t size,
                              dif_backend_executable *executable, dif_backend_error *error) {
  return compile_common(context, diffir, size, nullptr, 0, false, 0, executable, nullptr, error);
}

void destroy_executable(dif_backend_executable executable) { delete static_cast<Executable *>(executable); }

dif_backend_status execute(dif_backend_executable executable, const dif_backend_tensor_view *inputs,
                           size_t input_count, dif_backend_tensor_view *outputs, size_t output_count,
                           const dif_backend_run_options *options, dif_backend_telemetry *telemetry,
                           dif_backend_error *error) {
  return guarded(error, [&] {
    Executable *exe = static_cast<Executable *>(executable);
    if (!exe || !options || (input_count && !inputs) || (output_count && !outputs))
      throw PluginError{1, "execute: null argument"};
    if (options->iterations == 0)
      throw PluginError{1, "execute: iterations must be positive"};
    Context *ctx = exe->ctx;
    require_cuda(cudaSetDevice(ctx->device), "cudaSetDevice");
    size_t free_before = 0, total = 0;
    cudaMemGetInfo(&free_before, &total);
    if (free_before < options->minimum_free_bytes)
      throw PluginError{3, "execute: free device memory is below minimum_free_bytes"};
    // v2: exactly the Input-role tensors; v1: Inputs followed by Constants
    size_t n_in = 0, n_const = 0, n_out = 0;
    for (const auto &t : exe->program.tensors) {
      n_in += t.has(ir::Input) ? 1 : 0;
      n_const += t.has(ir::Constant) ? 1 : 0;
      n_out += t.has(ir::Output) ? 1 : 0;
    }
    const size_t expected = exe->constants_bound ? n_in : n_in + n_const;
    if (input_count != expected)
      throw PluginError{1, "execute: expected " + std::to_string(expected) + " input views, got " +
                               std::to_string(input_count)};
    if (output_count > n_out)
      throw PluginError{1, "execute: more output views than Output-role tensors"};
    std::vector<int> out_view_of(exe->program.tensors.size(), -1);
    for (size_t i = 0; i < output_count; ++i) {
      const int idx = exe->program.index_of(outputs[i].tensor_id);
      if (idx < 0 || !exe->program.tensors[(size_t)idx].has(ir::Output) ||
          outputs[i].byte_count != exe->program.tensors[(size_t)idx].bytes() ||
          (!outputs[i].host_data && outputs[i].byte_count))
        throw PluginError{1, "execute: output view " + std::to_string(outputs[i].tensor_id) +
                                 " does not match an Output-role tensor"};
      out_view_of[(size_t)idx] = (int)i;
    }
    auto download = [&](size_t view, int idx, cudaStream_t stream) {
      if (outputs[view].byte_count)
        require_cuda(cudaMemcpyAsync(outputs[view].host_data, exe->dev[(size_t)idx], (size_t)outputs[view].byte_count,
                                     cudaMemcpyDeviceToHost, stream),
                     "cudaMemcpyAsync(device to host)");
    };
    EventPair events; // timing pair, destroyed on every way out
    require_cuda(cudaEventCreate(&events.a), "cudaEventCreate");
    require_cuda(cudaEventCreate(&events.b), "cudaEventCreate");
    const cudaEvent_t e0 = events.a, e1 = events.b;
    struct Drain { // on an error, nothing may still be reading or writing the caller's buffers
      Context *ctx;
      bool armed = true;
      ~Drain() {
        if (armed) {
          cudaStreamSynchronize(ctx->h2d);
          cudaStreamSynchronize(ctx->stream);
          cudaStreamSynchronize(ctx->d2h);
        }
      }
    } drain{ctx};
    double sum = 0.0, lo = std::numeric_limits<double>::max(), hi = 0.0;
    // A single pass (no warm-ups, one iteration -- what the host's run() asks for) overlaps the
    // three phases: uploads go to their own stream in view order, every op waits only for the
    // uploads it reads, and each Output tensor starts its way back as soon as the op that
    // completes it has been enqueued. With page-locked host buffers the two copy directions and
    // the kernels then run concurrently; with pageable buffers the copies block the calling
    // thread as they always do and the result is the same. The telemetry time of such a pass is
    // the span of the kernel stream, upload waits included.
    const char *overlap_env = std::getenv("DIFB200_EXECUTE_OVERLAP"); // "0": one stream, the three phases in turn
    const bool overlapped = options->warmups == 0 && options->iterations == 1 && !(overlap_env && overlap_env[0] == '0');
    if (overlapped) {
      const size_t n = exe->program.tensors.size();
      if (exe->uploaded.empty()) {
        exe->uploaded.assign(n, nullptr);
        exe->produced.assign(n, nullptr);
        for (size_t i = 0; i < n; ++i) {
          const ir::Tensor &t = exe->program.tensors[i];
          if (t.has(ir::Input) || (!exe->constants_bound && t.has(ir::Constant)))
            require_cuda(cudaEventCreateWithFlags(&exe->uploaded[i], cudaEventDisableTiming), "cudaEventCreate");
          if (t.has(ir::Output))
            require_cuda(cudaEventCreateWithFlags(&exe->produced[i], cudaEventDisableTiming), "cudaEventCreate");
        }
      }
      Overlap overlap;
      overlap.upload_pending.assign(n, 0);
      // the upload stream starts after whatever the kernel stream still holds of an earlier call
      require_cuda(cudaEventRecord(e0, ctx->stream), "cudaEventRecord");
      require_cuda(cudaStreamWaitEvent(ctx->h2d, e0, 0), "cudaStreamWaitEvent");
      for (size_t i = 0; i < input_count; ++i) {
        const int idx = exe->program.index_of(inputs[i].tensor_id);
        const bool is_const = idx >= 0 && exe->program.tensors[(size_t)idx].has(ir::Constant);
        const int at = upload(*exe, inputs[i], is_const ? ir::Constant : ir::Input, "execute", ctx->h2d);
        if (exe->uploaded[(size_t)at]) {
          require_cuda(cudaEventRecord(exe->uploaded[(size_t)at], ctx->h2d), "cudaEventRecord(upload)");
          overlap.upload_pending[(size_t)at] = 1;
        }
      }
      run_steps(*exe, &overlap);
      // an upload nothing waited for (an Input no op reads) still has to land before the call ends
      for (size_t i = 0; i < n; ++i)
        if (overlap.upload_pending[i])
          require_cuda(cudaStreamWaitEvent(ctx->stream, exe->uploaded[i], 0), "cudaStreamWaitEvent(upload)");
      require_cuda(cudaEventRecord(e1, ctx->stream), "cudaEventRecord");
      std::vector<uint8_t> sent(output_count, 0);
      for (int idx : overlap.finished_outputs) {
        const int view = out_view_of[(size_t)idx];
        if (view < 0 || sent[(size_t)view])
          continue;
        require_cuda(cudaStreamWaitEvent(ctx->d2h, exe->produced[(size_t)idx], 0), "cudaStreamWaitEvent(output)");
        download((size_t)view, idx, ctx->d2h);
        sent[(size_t)view] = 1;
      }
      // outputs no op produces (an Output that is also an Input or a Constant) go last
      require_cuda(cudaStreamWaitEvent(ctx->d2h, e1, 0), "cudaStreamWaitEvent");
      for (size_t i = 0; i < output_count; ++i)
        if (!sent[i])
          download(i, exe->program.index_of(outputs[i].tensor_id), ctx->d2h);
      require_cuda(cudaStreamSynchronize(ctx->d2h), "cudaStreamSynchronize(download)");
      require_cuda(cudaEventSynchronize(e1), "cudaEventSynchronize");
      float ms = 0.0f;
      cudaEventElapsedTime(&ms, e0, e1);
      sum = lo = hi = ms;
    } else {
      for (size_t i = 0; i < input_count; ++i) {
        const int idx = exe->program.index_of(inputs[i].tensor_id);
        const bool is_const = idx >= 0 && exe->program.tensors[(size_t)idx].has(ir::Constant);
        upload(*exe, inputs[i], is_const ? ir::Constant : ir::Input, "execute");
      }
      for (uint32_t w = 0; w < options->warmups; ++w)
        run_steps(*exe);
      // The timed passes are enqueued back to back, an event between every two, and waited for
      // once: the host stays ahead of the device, so no pass starts with an empty queue.
      EventList marks;
      for (uint32_t it = 0; it <= options->iterations; ++it) {
        cudaEvent_t e = nullptr;
        require_cuda(cudaEventCreate(&e), "cudaEventCreate");
        marks.events.push_back(e);
      }
      require_cuda(cudaEventRecord(marks.events[0], ctx->stream), "cudaEventRecord");
      for (uint32_t it = 0; it < options->iterations; ++it) {
        exe->profile_pass = exe->profile;
        run_steps(*exe);
        if (exe->profile_pass)
          profile_mark(*exe, 0);
        exe->profile_pass = false;
        require_cuda(cudaEventRecord(marks.events[(size_t)it + 1], ctx->stream), "cudaEventRecord");
      }
      require_cuda(cudaEventSynchronize(marks.events.back()), "cudaEventSynchronize");
      profile_collect(*exe);
      for (uint32_t it = 0; it < options->iterations; ++it) {
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, marks.events[it], marks.events[(size_t)it + 1]);
        sum += ms;
        lo = ms < lo ? ms : lo;
        hi = ms > hi ? ms : hi;
      }
      for (size_t i = 0; i < output_count; ++i)
        download(i, exe->program.index_of(outputs[i].tensor_id), ctx->stream);
    }
    unsigned int flag = 0;
    require_cuda(cudaMemcpyAsync(&flag, exe->flag, sizeof(flag), cudaMemcpyDeviceToHost, ctx->stream),
                 "cudaMemcpyAsync(flag)");
    require_cuda(cudaStreamSynchronize(ctx->stream), "cudaStreamSynchronize");
    drain.armed = false;
    if (flag) {
      cudaMemset(exe->flag, 0, sizeof(flag));
      throw PluginError{5, "RotaryFrequency pair map is outside its declared axis"};
    }
    require(poll_device_status("execute"));
    if (telemetry) {
      size_t free_after = 0;
      cudaMemGetInfo(&free_after, &total);
      telemetry->mean_milliseconds = sum / options->iterations;
      telemetry->minimum_milliseconds = lo;
      telemetry->maximum_milliseconds = hi;
      telemetry->free_bytes_before = free_before;
      telemetry->free_bytes_after = free_after;
      std::memcpy(telemetry->device_name, ctx->device_name, sizeof(telemetry->device_name));
    }
  });
}

const uint64_t kCapabilities = DIF_BACKEND_CAP_F32 | DIF_BACKEND_CAP_BF16 | DIF_BACKEND_CAP_F16 | DIF_BACKEND_CAP_I8;

const dif_backend_api_v1 kApiV1 = {sizeof(dif_backend_api_v1), DIF_BACKEND_ABI_VERSION_V1, "difb200", kCapabilities,
                                   create, destroy, compile_v1, destroy_executable, execute};
const dif_backend_api_v2 kApiV2 = {sizeof(dif_backend_api_v2), DIF_BACKEND_ABI_VERSION_V2, "difb200", kCapabilities,
                                   create, destroy, compile_v2, destroy_executable, execute};

} // namespace
} // namespace difb200

extern "C" int difb200_executable_profile(void *executable, uint32_t *opcodes, double *milliseconds, uint64_t *steps,
                                          uint32_t capacity, uint32_t *count) {
  using namespace difb200;
  Executable *exe = static_cast<Executable *>(executable);
  if (!exe || !opcodes || !milliseconds || !steps || !count)
    return fail(kInvalidArgument, "difb200_executable_profile: null pointer");
  uint32_t n = 0;
  for (const auto &entry : exe->profile_sum) {
    if (n == capacity)
      break;
    opcodes[n] = entry.first;
    milliseconds[n] = entry.second.first;
    steps[n] = entry.second.second;
    ++n;
  }
  // token-sharded, direct exchange: the copies of the value / key pushes on the communication stream
  for (int which = 0; which < 2; ++which) {
    double ms = 0.0;
    uint64_t pushes = 0;
    for (const Sharded &sh : exe->sharded) {
      double one = 0.0;
      uint64_t k = 0;
      world_push_times(sh.binding, which, &one, &k);
      ms += one;
      pushes += k;
    }
    if (pushes && n < capacity) {
      opcodes[n] = 0xF000u + (uint32_t)which;
      milliseconds[n] = ms;
      steps[n] = pushes;
      ++n;
    }
  }
  *count = n;
  exe->profile_sum.clear();
  return kOk;
}

extern "C" int difb200_executable_exchange(void *executable) {
  using namespace difb200;
  const Executable *exe = static_cast<const Executable *>(executable);
  if (!exe || exe->sharded.empty())
    return 0;
  for (const Sharded &sh : exe->sharded)
    if (!sh.binding || !sh.binding->direct) {
      if (sh.binding && !sh.binding->note.empty())
        fail(kOk, sh.binding->note); // the reason, for difb200_last_error()
      return 1;
    }
  return 2;
}

extern "C" {
const dif_backend_api_v1 *dif_backend_get_v1(void) { return &difb200::kApiV1; }
const dif_backend_api_v2 *dif_backend_get_v2(void) { return &difb200::kApiV2; }
}
