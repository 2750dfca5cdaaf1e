// DIFIR001 decoder, SHA-256 and the subset verifier of the difb200 plugin (see diffir.h).
#include "diffir.h"

#include <cmath>
#include <cstring>
#include <set>

namespace difb200 {
namespace ir {

// ---------------------------------------------------------------------------------------
// SHA-256 (FIPS 180-4)
// ---------------------------------------------------------------------------------------
namespace {
inline uint32_t rotr(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }

const uint32_t kRound[64] = {
    0x428a2f98, 0x71374491, 0xb5c0fbcf, 0xe9b5dba5, 0x3956c25b, 0x59f111f1, 0x923f82a4, 0xab1c5ed5,
    0xd807aa98, 0x12835b01, 0x243185be, 0x550c7dc3, 0x72be5d74, 0x80deb1fe, 0x9bdc06a7, 0xc19bf174,
    0xe49b69c1, 0xefbe4786, 0x0fc19dc6, 0x240ca1cc, 0x2de92c6f, 0x4a7484aa, 0x5cb0a9dc, 0x76f988da,
    0x983e5152, 0xa831c66d, 0xb00327c8, 0xbf597fc7, 0xc6e00bf3, 0xd5a79147, 0x06ca6351, 0x14292967,
    0x27b70a85, 0x2e1b2138, 0x4d2c6dfc, 0x53380d13, 0x650a7354, 0x766a0abb, 0x81c2c92e, 0x92722c85,
    0xa2bfe8a1, 0xa81a664b, 0xc24b8b70, 0xc76c51a3, 0xd192e819, 0xd6990624, 0xf40e3585, 0x106aa070,
    0x19a4c116, 0x1e376c08, 0x2748774c, 0x34b0bcb5, 0x391c0cb3, 0x4ed8aa4a, 0x5b9cca4f, 0x682e6ff3,
    0x748f82ee, 0x78a5636f, 0x84c87814, 0x8cc70208, 0x90befffa, 0xa4506ceb, 0xbef9a3f7, 0xc67178f2};

void compress(uint32_t state[8], const uint8_t block[64]) {
  uint32_t w[64];
  for (int i = 0; i < 16; ++i)
    w[i] = (uint32_t)block[4 * i] << 24 | (uint32_t)block[4 * i + 1] << 16 |
           (uint32_t)block[4 * i + 2] << 8 | (uint32_t)block[4 * i + 3];
  for (int i = 16; i < 64; ++i) {
    const uint32_t s0 = rotr(w[i - 15], 7) ^ rotr(w[i - 15], 18) ^ (w[i - 15] >> 3);
    const uint32_t s1 = rotr(w[i - 2], 17) ^ rotr(w[i - 2], 19) ^ (w[i - 2] >> 10);
    w[i] = w[i - 16] + s0 + w[i - 7] + s1;
  }
  uint32_t a = state[0], b = state[1], c = state[2], d = state[3], e = state[4], f = state[5],
           g = state[6], h = state[7];
  for (int i = 0; i < 64; ++i) {
    const uint32_t S1 = rotr(e, 6) ^ rotr(e, 11) ^ rotr(e, 25);
    const uint32_t ch = (e & f) ^ (~e & g);
    const uint32_t t1 = h + S1 + ch + kRound[i] + w[i];
    const uint32_t S0 = rotr(a, 2) ^ rotr(a, 13) ^ rotr(a, 22);
    const uint32_t maj = (a & b) ^ (a & c) ^ (b & c);
    const uint32_t t2 = S0 + maj;
    h = g; g = f; f = e; e = d + t1; d = c; c = b; b = a; a = t1 + t2;
  }
  state[0] += a; state[1] += b; state[2] += c; state[3] += d;
  state[4] += e; state[5] += f; state[6] += g; state[7] += h;
}
} // namespace

void sha256(const uint8_t *data, size_t size, uint8_t digest[32]) {
  uint32_t state[8] = {0x6a09e667, 0xbb67ae85, 0x3c6ef372, 0xa54ff53a,
                       0x510e527f, 0x9b05688c, 0x1f83d9ab, 0x5be0cd19};
  size_t offset = 0;
  for (; offset + 64 <= size; offset += 64)
    compress(state, data + offset);
  uint8_t tail[128] = {0};
  const size_t rest = size - offset;
  std::memcpy(tail, data + offset, rest);
  tail[rest] = 0x80;
  const size_t padded = rest + 9 <= 64 ? 64 : 128;
  const uint64_t bits = (uint64_t)size * 8;
  for (int i = 0; i < 8; ++i)
    tail[padded - 1 - i] = (uint8_t)(bits >> (8 * i));
  compress(state, tail);
  if (padded == 128)
    compress(state, tail + 64);
  for (int i = 0; i < 8; ++i) {
    digest[4 * i] = (uint8_t)(state[i] >> 24);
    digest[4 * i + 1] = (uint8_t)(state[i] >> 16);
    digest[4 * i + 2] = (uint8_t)(state[i] >> 8);
    digest[4 * i + 3] = (uint8_t)state[i];
  }
}

// ---------------------------------------------------------------------------------------
// model helpers
// ---------------------------------------------------------------------------------------
size_t dtype_size(uint32_t dtype) {
  switch (dtype) {
  case F32: case I32: return 4;
  case BF16: case F16: return 2;
  case I8: case Bool: case FP8E4M3: case FP8E8M0: return 1;
  default: return 0;
  }
}

uint64_t Tensor::elements() const {
  uint64_t n = 1;
  for (auto d : dims)
    n *= d;
  return n;
}
uint64_t Tensor::bytes() const { return elements() * dtype_size(dtype); }

const Attr *Op::find(uint32_t key) const {
  for (const auto &a : attrs)
    if (a.key == key)
      return &a;
  return nullptr;
}
uint64_t Op::u64(uint32_t key, uint64_t fallback) const {
  const Attr *a = find(key);
  return a ? a->bits : fallback;
}
double Op::f64(uint32_t key, double fallback) const {
  const Attr *a = find(key);
  if (!a)
    return fallback;
  double v;
  std::memcpy(&v, &a->bits, 8);
  return v;
}
bool Op::boolean(uint32_t key, bool fallback) const {
  const Attr *a = find(key);
  return a ? a->bits != 0 : fallback;
}

const Tensor *Program::tensor(uint32_t id) const {
  const int i = index_of(id);
  return i < 0 ? nullptr : &tensors[(size_t)i];
}
int Program::index_of(uint32_t id) const {
  for (size_t i = 0; i < tensors.size(); ++i)
    if (tensors[i].id == id)
      return (int)i;
  return -1;
}

const char *opcode_name(uint32_t opcode) {
  switch (opcode) {
  case Add: return "Add"; case Multiply: return "Multiply"; case RmsNormModulate: return "RmsNormModulate";
  case SwiGlu: return "SwiGlu"; case ResidualGate: return "ResidualGate"; case Linear: return "Linear";
  case QkNormPartialRope: return "QkNormPartialRope"; case Attention: return "Attention";
  case BiasAdd: return "BiasAdd"; case SiLU: return "SiLU"; case RmsNorm: return "RmsNorm";
  case Fill: return "Fill"; case Cast: return "Cast"; case AffineLastDim: return "AffineLastDim";
  case Gelu: return "Gelu"; case Sigmoid: return "Sigmoid"; case Reshape: return "Reshape";
  case BroadcastTo: return "BroadcastTo"; case Slice: return "Slice";
  case RotaryFrequency: return "RotaryFrequency"; case RotaryApply: return "RotaryApply";
  case BooleanMaskToBias: return "BooleanMaskToBias"; case Concat: return "Concat";
  case QuantizeInt8Rows: return "QuantizeInt8Rows"; case LinearInt8Scaled: return "LinearInt8Scaled";
  case LayerNormModulate: return "LayerNormModulate";
  default: return "opcode outside the quantized DiT hot path";
  }
}

// ---------------------------------------------------------------------------------------
// decoder
// ---------------------------------------------------------------------------------------
namespace {
struct Reader {
  const uint8_t *p;
  size_t n, pos = 0;
  bool ok = true;
  uint32_t u32() {
    if (pos + 4 > n) { ok = false; return 0; }
    uint32_t v;
    std::memcpy(&v, p + pos, 4);
    pos += 4;
    return v;
  }
  uint64_t u64() {
    if (pos + 8 > n) { ok = false; return 0; }
    uint64_t v;
    std::memcpy(&v, p + pos, 8);
    pos += 8;
    return v;
  }
};
constexpr uint32_t kMaxCount = 1u << 20;
} // namespace

int decode(const uint8_t *bytes, size_t size, Program &program, std::string &error) {
  static const char magic[8] = {'D', 'I', 'F', 'I', 'R', '0', '0', '1'};
  if (!bytes || size < 8 + 12 + 32) {
    error = "DiffIR buffer is too small";
    return 1;
  }
  uint8_t digest[32];
  sha256(bytes, size - 32, digest);
  if (std::memcmp(digest, bytes + size - 32, 32) != 0) {
    error = "DiffIR SHA-256 mismatch";
    return 1;
  }
  if (std::memcmp(bytes, magic, 8) != 0) {
    error = "invalid DiffIR magic";
    return 1;
  }
  Reader r{bytes + 8, size - 40};
  const uint32_t version = r.u32(), n_tensors = r.u32(), n_ops = r.u32();
  if (version != 1) {
    error = "unsupported DiffIR version";
    return 1;
  }
  if (n_tensors > kMaxCount || n_ops > kMaxCount) {
    error = "DiffIR tensor/operation count is too large";
    return 1;
  }
  program.tensors.clear();
  program.ops.clear();
  for (uint32_t i = 0; i < n_tensors && r.ok; ++i) {
    Tensor t;
    t.id = r.u32();
    t.dtype = r.u32();
    t.roles = r.u32();
    const uint32_t rank = r.u32();
    if (rank == 0 || rank > 8) {
      error = "invalid DiffIR tensor rank";
      return 1;
    }
    for (uint32_t a = 0; a < rank; ++a)
      t.dims.push_back(r.u64());
    program.tensors.push_back(std::move(t));
  }
  for (uint32_t i = 0; i < n_ops && r.ok; ++i) {
    Op op;
    op.id = r.u32();
    op.opcode = r.u32();
    const uint32_t n_in = r.u32(), n_out = r.u32(), n_attr = r.u32();
    if (n_in > kMaxCount || n_out > kMaxCount || n_attr > kMaxCount) {
      error = "DiffIR operand count is too large";
      return 1;
    }
    for (uint32_t k = 0; k < n_in && r.ok; ++k)
      op.in.push_back(r.u32());
    for (uint32_t k = 0; k < n_out && r.ok; ++k)
      op.out.push_back(r.u32());
    for (uint32_t k = 0; k < n_attr && r.ok; ++k) {
      Attr a;
      a.key = r.u32();
      a.kind = r.u32();
      a.bits = r.u64();
      op.attrs.push_back(a);
    }
    program.ops.push_back(std::move(op));
  }
  if (!r.ok) {
    error = "truncated DiffIR payload";
    return 1;
  }
  if (r.pos != r.n) {
    error = "trailing bytes in DiffIR payload";
    return 1;
  }
  return verify(program, error);
}

// ---------------------------------------------------------------------------------------
// verifier: program-level rules for every program, per-op shape rules for the supported subset
// ---------------------------------------------------------------------------------------
namespace {

struct Fail {
  int status;
  std::string text;
};

[[noreturn]] void bad(const Op &op, const std::string &text, int status = 1) {
  throw Fail{status, std::string(opcode_name(op.opcode)) + " (op " + std::to_string(op.id) + "): " + text};
}

const Tensor &T(const Program &p, const Op &op, uint32_t id) {
  const Tensor *t = p.tensor(id);
  if (!t)
    bad(op, "unknown tensor id " + std::to_string(id));
  return *t;
}

void counts(const Op &op, size_t n_in, size_t n_out) {
  if (op.in.size() != n_in || op.out.size() != n_out)
    bad(op, "expects " + std::to_string(n_in) + " inputs and " + std::to_string(n_out) + " outputs");
}
void same(const Op &op, const Tensor &a, const Tensor &b) {
  if (a.dtype != b.dtype || a.dims != b.dims)
    bad(op, "operands must share shape and dtype");
}
void need(const Op &op, bool cond, const char *text) {
  if (!cond)
    bad(op, text);
}

// Attribute reads of the verifier: an attribute that is present must have the kind it is read as
// (reference src/ir/codec.cpp:104-127, the accessors every rule below goes through).
struct AttrReader {
  const Op &op;
  const Attr *kind(uint32_t key, uint32_t want, const char *name) const {
    const Attr *a = op.find(key);
    if (a && a->kind != want)
      bad(op, std::string("attribute ") + std::to_string(key) + " must be " + name);
    return a;
  }
  uint64_t u64(uint32_t key, uint64_t fallback) const {
    const Attr *a = kind(key, 1, "u64");
    return a ? a->bits : fallback;
  }
  double f64(uint32_t key, double fallback) const {
    const Attr *a = kind(key, 3, "f64");
    if (!a)
      return fallback;
    double v;
    std::memcpy(&v, &a->bits, 8);
    return v;
  }
  bool boolean(uint32_t key, bool fallback) const {
    const Attr *a = kind(key, 4, "bool");
    return a ? a->bits != 0 : fallback;
  }
  bool has(uint32_t key) const { return op.find(key) != nullptr; }
};

bool power_of_two_in(uint64_t v, uint64_t low, uint64_t high) { return v >= low && v <= high && (v & (v - 1)) == 0; }

// Shape, dtype and attribute rules per operator, restated from the reference verifier (reference
// src/ir/verify.cpp:89-1338, the cases of the operators this backend runs): what it rejects is
// rejected here with status 1. A form it admits but this backend cannot run is status 2, given
// here or by the planner.
void verify_op(const Program &p, const Op &op) {
  auto in = [&](size_t i) -> const Tensor & { return T(p, op, op.in.at(i)); };
  auto out = [&](size_t i) -> const Tensor & { return T(p, op, op.out.at(i)); };
  const AttrReader attr{op};
  switch (op.opcode) {
  case Add:
  case Multiply:
    counts(op, 2, 1);
    same(op, in(0), in(1));
    same(op, in(0), out(0));
    need(op, in(0).is_float(), "needs f32/bf16/f16");
    return;
  case Gelu: {
    counts(op, 1, 1);
    same(op, in(0), out(0));
    need(op, in(0).is_float(), "needs f32/bf16/f16");
    need(op, attr.has(Approximation), "needs an explicit Approximation (1 = tanh, 2 = erf)");
    const uint64_t a = attr.u64(Approximation, 0);
    need(op, a == 1 || a == 2, "needs an explicit Approximation (1 = tanh, 2 = erf)");
    return;
  }
  case SiLU:
  case Sigmoid:
    counts(op, 1, 1);
    same(op, in(0), out(0));
    need(op, in(0).is_float(), "needs f32/bf16/f16");
    return;
  case BiasAdd:
    counts(op, 2, 1);
    same(op, in(0), out(0));
    need(op, in(0).is_float() && in(1).dtype == in(0).dtype && in(1).dims.size() == 1 &&
                 in(1).dims[0] == in(0).last(),
         "bias must be [last dim] in the input dtype");
    return;
  case AffineLastDim:
    need(op, (op.in.size() == 2 || op.in.size() == 3) && op.out.size() == 1, "expects input, scale, optional bias");
    same(op, in(0), out(0));
    need(op, in(0).is_float() && in(1).dtype == in(0).dtype && in(1).dims.size() == 1 &&
                 in(1).dims[0] == in(0).last(),
         "scale must be [last dim]");
    if (op.in.size() == 3)
      need(op, in(2).dtype == in(0).dtype && in(2).dims == in(1).dims, "bias must match the scale");
    return;
  case RmsNorm: {
    counts(op, 2, 1);
    same(op, in(0), out(0));
    need(op, in(0).is_float() && in(1).dtype == in(0).dtype && in(1).dims.size() == 1 &&
                 in(1).dims[0] == in(0).last(),
         "weight must be [last dim]");
    need(op, attr.f64(Epsilon, 1.0e-5) > 0.0, "Epsilon must be positive");
    (void)attr.f64(WeightOffset, 0.0); // finite like every f64 attribute
    const uint64_t block = attr.u64(BlockSize, 256);
    need(op, power_of_two_in(block, 32, 1024), "BlockSize must be a power of two in [32,1024]");
    const uint64_t impl = attr.u64(Implementation, 1);
    need(op, impl == 1 || impl == 2, "Implementation must be 1 or 2");
    if (impl == 2)
      need(op, in(0).dtype == BF16 && in(0).last() == 128 && block == 128,
           "Implementation 2 needs bf16, width 128 and BlockSize 128");
    const uint64_t tile = attr.u64(ReductionTileSize, 0);
    need(op, tile == 0 || tile == 2048 || tile == 8192, "ReductionTileSize must be 0, 2048 or 8192");
    if (tile != 0)
      need(op, block == 512 && in(0).last() == 6144, "a reduction tile needs BlockSize 512 and width 6144");
    return;
  }
  case Fill:
    counts(op, 0, 1);
    need(op, out(0).is_float(), "needs a float output");
    return;
  case Cast:
    counts(op, 1, 1);
    need(op, in(0).is_float() && out(0).is_float() && in(0).dtype != out(0).dtype && in(0).dims == out(0).dims,
         "needs equal-shaped tensors of two different float dtypes");
    return;
  case Reshape:
    counts(op, 1, 1);
    need(op, in(0).is_float() && in(0).dtype == out(0).dtype && in(0).elements() == out(0).elements(),
         "needs equal element counts and dtypes");
    return;
  case BroadcastTo: {
    counts(op, 1, 1);
    const Tensor &a = in(0), &o = out(0);
    need(op, a.is_float() && a.dtype == o.dtype && a.dims.size() <= o.dims.size(), "rank/dtype mismatch");
    const size_t pad = o.dims.size() - a.dims.size();
    for (size_t i = 0; i < a.dims.size(); ++i)
      need(op, a.dims[i] == 1 || a.dims[i] == o.dims[pad + i], "dimension is not broadcastable");
    return;
  }
  case Slice: {
    counts(op, 1, 1);
    const Tensor &a = in(0), &o = out(0);
    need(op, a.is_float() && a.dtype == o.dtype && a.dims.size() == o.dims.size() && attr.has(Axis) && attr.has(Start),
         "needs equal-rank float tensors and Axis / Start");
    const uint64_t axis = attr.u64(Axis, 0), start = attr.u64(Start, 0);
    need(op, axis < a.dims.size() && start <= a.dims[axis] && o.dims[axis] <= a.dims[axis] - start,
         "axis or window is outside the input");
    for (size_t i = 0; i < a.dims.size(); ++i)
      need(op, i == axis || o.dims[i] == a.dims[i], "only the sliced axis may change");
    return;
  }
  case Concat: {
    need(op, op.in.size() >= 2 && op.out.size() == 1, "expects at least two inputs and one output");
    const Tensor &first = in(0), &o = out(0);
    need(op, attr.has(Axis), "needs an Axis");
    const uint64_t axis = attr.u64(Axis, 0);
    need(op, axis < first.dims.size() && first.is_float() && o.dtype == first.dtype &&
                 o.dims.size() == first.dims.size(),
         "axis/dtype/rank mismatch");
    uint64_t total = 0;
    for (size_t k = 0; k < op.in.size(); ++k) {
      const Tensor &a = in(k);
      need(op, a.dtype == first.dtype && a.dims.size() == first.dims.size(), "inputs must share rank and dtype");
      for (size_t i = 0; i < a.dims.size(); ++i)
        need(op, i == axis || a.dims[i] == first.dims[i], "inputs must agree off the axis");
      need(op, total <= UINT64_MAX - a.dims[axis], "axis extent overflows");
      total += a.dims[axis];
    }
    for (size_t i = 0; i < first.dims.size(); ++i)
      need(op, o.dims[i] == (i == axis ? total : first.dims[i]), "output shape is not the joined inputs");
    return;
  }
  case RotaryFrequency: {
    counts(op, 4, 2);
    const Tensor &pos = in(0), &axes = in(1), &idx = in(2), &adims = in(3);
    need(op, pos.dtype == F32 && pos.dims.size() == 3 && axes.dtype == I32 && idx.dtype == I32 &&
                 adims.dtype == I32 && axes.dims.size() == 1 && idx.dims == axes.dims &&
                 adims.dims.size() == 1 && adims.dims[0] == pos.dims[2],
         "positions F32 [B,L,A] and I32 pair maps expected");
    for (int k = 0; k < 2; ++k)
      need(op, out(k).dtype == F32 && out(k).dims.size() == 3 && out(k).dims[0] == pos.dims[0] &&
                   out(k).dims[1] == pos.dims[1] && out(k).dims[2] == axes.dims[0],
           "tables must be F32 [B,L,P]");
    need(op, attr.f64(Theta, 10000.0) > 0.0 && attr.f64(Ntk, 1.0) > 0.0, "Theta and Ntk must be positive");
    return;
  }
  case RotaryApply: {
    counts(op, 3, 1);
    const Tensor &x = in(0), &c = in(1), &s = in(2);
    same(op, x, out(0));
    need(op, x.is_float() && x.dims.size() == 4 && c.dtype == F32 && c.dims.size() == 3 && s.dims == c.dims &&
                 s.dtype == F32 && c.dims[0] == x.dims[0] && c.dims[1] == x.dims[1] && c.dims[2] <= x.dims[3] / 2,
         "input [B,S,H,D] with F32 [B,S,P] tables expected");
    need(op, attr.u64(RotaryLayout, 0) == 1, "needs an explicit interleaved RotaryLayout");
    return;
  }
  case BooleanMaskToBias: {
    counts(op, 1, 1);
    const Tensor &m = in(0), &o = out(0);
    need(op, m.dtype == Bool && o.is_float() && o.dims.size() == 4 && o.dims[1] == 1 && o.dims[2] == o.dims[3] &&
                 (m.dims.size() == 2 || m.dims.size() == 3) && o.dims[0] == m.dims[0] &&
                 ((m.dims.size() == 2 && m.dims[1] == o.dims[2]) ||
                  (m.dims.size() == 3 && m.dims[1] == o.dims[2] && m.dims[2] == o.dims[2])),
         "Bool [B,L] or [B,L,L] -> float [B,1,L,L] expected");
    (void)attr.boolean(MaskQueries, true);
    return;
  }
  case QkNormPartialRope: {
    counts(op, 4, 1);
    const Tensor &x = in(0), &w = in(1), &c = in(2), &s = in(3);
    same(op, x, out(0));
    need(op, x.is_float() && (x.dims.size() == 3 || x.dims.size() == 4), "input [S,H,D] or [B,S,H,D] expected");
    const bool table_rank_fits = x.dims.size() == 4 ? c.dims.size() == 3
                                                    : (c.dims.size() == 2 || (c.dims.size() == 3 && c.dims[0] == 1));
    need(op, w.dtype == x.dtype && w.dims.size() == 1 && (c.dtype == x.dtype || c.dtype == F32) &&
                 s.dtype == c.dtype && c.dims == s.dims && table_rank_fits,
         "weight [D] and matching cos/sin tables expected");
    const size_t head_axis = x.dims.size() - 2;
    const uint64_t D = x.last(), width = c.last();
    const uint64_t heads = attr.u64(Heads, x.dims[head_axis]), head_dim = attr.u64(HeadDim, D);
    need(op, width <= UINT64_MAX / 2, "table width overflows");
    const uint64_t rotary = attr.u64(RotaryDim, width * 2);
    const uint64_t in_batch = x.dims.size() == 4 ? x.dims[0] : 1, in_seq = x.dims.size() == 4 ? x.dims[1] : x.dims[0];
    const uint64_t tab_batch = c.dims.size() == 3 ? c.dims[0] : 1, tab_seq = c.dims.size() == 3 ? c.dims[1] : c.dims[0];
    const uint64_t start = attr.u64(Start, 0);
    need(op, heads == x.dims[head_axis] && head_dim == D && w.dims[0] == D && tab_batch == in_batch &&
                 start <= tab_seq && in_seq <= tab_seq - start && rotary != 0 && rotary <= D && rotary % 2 == 0 &&
                 (width == rotary || width * 2 == rotary),
         "Heads / HeadDim / RotaryDim / Start do not fit the shapes");
    need(op, power_of_two_in(attr.u64(BlockSize, 256), 32, 1024), "BlockSize must be a power of two in [32,1024]");
    return;
  }
  case RmsNormModulate: {
    need(op, (op.in.size() == 3 || op.in.size() == 4) && op.out.size() == 1, "expects x, [weight], scale, shift");
    const Tensor &x = in(0);
    const uint64_t layout = attr.u64(ModulationLayout, 1);
    if (layout == 2) {
      counts(op, 4, 1);
      same(op, x, out(0));
      need(op, x.is_float() && x.dims.size() == 2, "rank-2 float input expected");
      const uint64_t cols = x.dims[1];
      need(op, in(1).dtype == x.dtype && in(1).dims.size() == 1 && in(1).dims[0] == cols &&
                   in(2).dtype == x.dtype && in(2).dims.size() == 2 && in(2).dims[1] == cols && in(2).dims[0] > 0 &&
                   x.dims[0] % in(2).dims[0] == 0 && in(3).dtype == x.dtype && in(3).dims.size() == 2 &&
                   in(3).dims[0] == 2 && in(3).dims[1] == cols,
           "weight [H], vector [V,H], delta [2,H] expected");
      need(op, attr.f64(Epsilon, 1.0e-5) > 0.0, "Epsilon must be positive");
      (void)attr.f64(WeightOffset, 0.0);
      const uint64_t block = attr.u64(BlockSize, 256), tile = attr.u64(ReductionTileSize, 0);
      need(op, power_of_two_in(block, 32, 1024) && (tile == 0 || tile == 2048 || tile == 8192) &&
                   (tile == 0 || (block == 512 && cols == 6144)),
           "BlockSize / ReductionTileSize do not fit");
      return;
    }
    need(op, layout == 1, "unknown ModulationLayout");
    const bool weighted = op.in.size() == 4;
    same(op, x, in(weighted ? 2 : 1));
    same(op, x, in(weighted ? 3 : 2));
    same(op, x, out(0));
    need(op, x.is_float() && x.dims.size() == 2, "rank-2 float input expected");
    if (weighted)
      need(op, in(1).dtype == x.dtype && in(1).dims.size() == 1 && in(1).dims[0] == x.dims[1], "weight must be [H]");
    need(op, attr.f64(Epsilon, 1.0e-5) > 0.0, "Epsilon must be positive");
    need(op, power_of_two_in(attr.u64(BlockSize, 256), 32, 1024), "BlockSize must be a power of two in [32,1024]");
    return;
  }
  case LayerNormModulate: {
    counts(op, 5, 1);
    const Tensor &x = in(0);
    same(op, x, out(0));
    need(op, x.is_float() && in(1).dims.size() == 1 && in(1).dims[0] == x.last() && in(2).dims == in(1).dims &&
                 in(3).dims == in(4).dims && !in(3).dims.empty() && in(3).last() == x.last() &&
                 in(1).dtype == x.dtype && in(2).dtype == x.dtype && in(3).dtype == x.dtype && in(4).dtype == x.dtype,
         "[hidden] weight/bias and compatible scale/shift rows expected");
    need(op, in(3).rows() > 0 && x.rows() % in(3).rows() == 0, "scale/shift rows must divide the input rows");
    need(op, power_of_two_in(attr.u64(BlockSize, 256), 32, 1024) && attr.f64(Epsilon, 1.0e-5) > 0.0,
         "BlockSize must be a power of two in [32,1024] and Epsilon positive");
    return;
  }
  case ResidualGate: {
    counts(op, 3, 1);
    same(op, in(0), in(1));
    same(op, in(0), out(0));
    need(op, in(0).is_float() && in(2).dtype == in(0).dtype && !in(2).dims.empty() && in(2).last() == in(0).last() &&
                 in(2).rows() > 0 && in(0).rows() % in(2).rows() == 0,
         "gate rows must divide the residual rows");
    return;
  }
  case SwiGlu: {
    counts(op, 1, 1);
    const Tensor &x = in(0), &o = out(0);
    need(op, x.is_float() && o.dtype == x.dtype && x.dims.size() == o.dims.size(), "compatible float tensors expected");
    for (size_t i = 0; i + 1 < x.dims.size(); ++i)
      need(op, x.dims[i] == o.dims[i], "prefix dimensions must match");
    const uint64_t start = attr.u64(Start, 0);
    need(op, o.last() <= (UINT64_MAX - start) / 2 && start + 2 * o.last() <= x.last(),
         "packed window is outside the input");
    (void)attr.boolean(GateFirst, false);
    return;
  }
  case Linear: {
    need(op, (op.in.size() == 2 || op.in.size() == 3) && op.out.size() == 1, "expects input, weight, optional bias");
    const Tensor &x = in(0), &w = in(1), &o = out(0);
    need(op, x.is_float() && w.dtype == x.dtype && o.dtype == x.dtype && w.dims.size() == 2, "uniform float dtype, rank-2 weight");
    const uint64_t rows = x.dims[0];
    need(op, x.elements() / rows == w.dims[1] && o.dims[0] == rows && o.elements() / o.dims[0] == w.dims[0],
         "shapes must flatten as [M,K] x [N,K] -> [M,N]");
    if (op.in.size() == 3)
      need(op, in(2).dtype == x.dtype && in(2).dims.size() == 1 && in(2).dims[0] == w.dims[0], "bias must be [N]");
    const uint64_t bias_mode = attr.u64(LinearBiasMode, 1);
    need(op, bias_mode == 1 || (bias_mode == 2 && op.in.size() == 3), "LinearBiasMode must be 1, or 2 with a bias");
    if (attr.has(WorkspaceLimitBytes))
      need(op, attr.u64(WorkspaceLimitBytes, 0) != 0, "WorkspaceLimitBytes must be positive");
    const uint64_t impl = attr.u64(Implementation, 1);
    need(op, impl >= 1 && impl <= 3 && (impl != 2 || x.dtype == F32), "Implementation must be 1..3 (2 needs f32)");
    return;
  }
  case QuantizeInt8Rows: {
    need(op, !op.in.empty() && (op.out.size() == 2 || op.out.size() == 4), "expects BF16 inputs and 2 or 4 outputs");
    const bool dynamic = in(op.in.size() - 1).dtype == F32;
    const size_t n_data = op.in.size() - (dynamic ? 1 : 0);
    need(op, n_data >= 1, "needs at least one data input in front of the clip");
    if (dynamic)
      need(op, in(op.in.size() - 1).dims == std::vector<uint64_t>{1}, "dynamic clip must be F32[1]");
    const uint64_t rows = in(0).rows();
    uint64_t width = 0;
    for (size_t k = 0; k < n_data; ++k) {
      need(op, in(k).dtype == BF16 && in(k).rows() == rows, "data inputs must be BF16 with equal row counts");
      need(op, width <= UINT64_MAX - in(k).last(), "combined width overflows");
      width += in(k).last();
    }
    need(op, out(0).dtype == I8 && out(0).last() == width && out(0).elements() / width == rows &&
                 out(1).dtype == F32 && out(1).dims == std::vector<uint64_t>{rows},
         "outputs must be I8 [.., width] and F32 [rows]");
    if (op.out.size() == 4)
      need(op, out(2).dtype == I8 && out(2).dims == out(0).dims && out(3).dtype == F32 && out(3).dims == out(1).dims,
           "residual outputs must mirror the primary ones");
    need(op, attr.u64(BlockSize, 256) == 256, "BlockSize must be 256");
    const double clip = attr.f64(Scale, 1.0);
    need(op, clip > 0.0 && clip <= 1.0, "Scale must be in (0,1]");
    const uint64_t impl = attr.u64(Implementation, 1);
    need(op, impl >= 1 && impl <= 7, "unknown Implementation");
    if (impl == 4 || impl == 7)
      need(op, width % 4096 == 0, "H4096 variants need a width divisible by 4096");
    else if (impl != 1)
      need(op, width % 256 == 0, "H256 variants need a width divisible by 256");
    if (n_data > 8)
      bad(op, "more than 8 concatenated data inputs are not implemented", 2);
    return;
  }
  case LinearInt8Scaled: {
    counts(op, 4, 1);
    const Tensor &x = in(0), &w = in(1), &rs = in(2), &cs = in(3), &o = out(0);
    need(op, x.dtype == I8 && w.dtype == I8 && rs.dtype == F32 && cs.dtype == F32 && o.dtype == BF16 &&
                 w.dims.size() == 2,
         "I8 input/weight, F32 scales, BF16 output expected");
    const uint64_t rows = x.rows();
    need(op, w.dims[1] == x.last() && rs.dims == std::vector<uint64_t>{rows} &&
                 cs.dims == std::vector<uint64_t>{w.dims[0]} && w.dims[0] <= UINT64_MAX / rows &&
                 o.elements() == rows * w.dims[0] && o.last() == w.dims[0],
         "shapes must flatten as [M,K] x [N,K] with row [M], column [N], BF16 [M,N]");
    need(op, w.has(Constant) && cs.has(Constant), "weight and column scales must be constants");
    return;
  }
  case Attention: {
    need(op, (op.in.size() == 3 || op.in.size() == 4) && op.out.size() == 1, "expects q, k, v, optional bias");
    const Tensor &q = in(0), &k = in(1), &v = in(2);
    same(op, k, v);
    same(op, q, out(0));
    need(op, q.is_float() && (q.dims.size() == 3 || q.dims.size() == 4), "float [S,H,D] or [B,S,H,D] expected");
    const size_t ha = q.dims.size() - 2, sa = q.dims.size() - 3;
    const uint64_t H = q.dims[ha], S = q.dims[sa];
    const uint64_t kv = attr.u64(KvHeads, H);
    need(op, kv != 0 && H % kv == 0, "KvHeads must divide the head count");
    auto expect = q.dims;
    expect[ha] = kv;
    need(op, k.dtype == q.dtype && k.dims == expect, "k/v must carry KvHeads heads");
    const bool biased = op.in.size() == 4, batched = q.dims.size() == 4;
    if (biased) {
      const Tensor &b = in(3);
      need(op, batched && b.dtype == q.dtype && b.dims == std::vector<uint64_t>{q.dims[0], 1, S, S},
           "bias must be [B,1,S,S] in the query dtype");
    }
    const uint64_t impl = attr.u64(Implementation, 1);
    need(op, impl >= 1 && impl <= 5, "Implementation must be 1..5");
    // what each implementation admits (reference src/ir/verify.cpp:1293-1320)
    if (impl == 2)
      need(op, q.dtype == BF16 || q.dtype == F16, "Implementation 2 needs bf16 or f16");
    if (impl == 1)
      need(op, !batched && !biased && S <= 4096, "Implementation 1 is unbatched, unbiased and S <= 4096");
    const bool causal = (impl >= 3) ? attr.boolean(Causal, false) : false;
    if (impl == 3)
      need(op, q.dtype == F32 && !batched && H == 1 && kv == 1 && !biased && !causal,
           "Implementation 3 is noncausal unbatched f32 [S,1,D] without bias");
    if (impl == 4)
      need(op, q.dtype == BF16 && q.last() == 128 && !biased && !causal,
           "Implementation 4 is noncausal bf16 head dimension 128 without bias");
    if (impl == 5)
      need(op, q.dtype == BF16 && q.last() == 128 && kv == H && !biased && !causal,
           "Implementation 5 is noncausal bf16 head dimension 128, full heads, no bias");
    need(op, power_of_two_in(attr.u64(BlockSize, 64), 32, 256), "BlockSize must be a power of two in [32,256]");
    return;
  }
  default:
    bad(op, "this backend implements only the quantized DiT hot path opcodes", 2);
  }
}

} // namespace

int verify(const Program &program, std::string &error) {
  try {
    if (program.tensors.empty())
      throw Fail{1, "program has no tensors"};
    std::set<uint32_t> ids;
    for (const auto &t : program.tensors) {
      if (t.id == 0 || !ids.insert(t.id).second)
        throw Fail{1, "tensor ids must be unique and non-zero"};
      if (t.dtype < F32 || t.dtype > FP8E8M0)
        throw Fail{1, "unknown tensor dtype"};
      if (t.dims.empty() || t.dims.size() > 8)
        throw Fail{1, "tensor rank must be 1..8"};
      if ((t.roles & ~63u) != 0 || (t.has(Streamed) && !t.has(Constant)))
        throw Fail{1, "invalid tensor role mask"};
      // training roles (reference src/ir/verify.cpp:2073-2085): parameters and optimizer state are
      // inputs or outputs and never constants
      const bool trained = t.has(Parameter) || t.has(OptimizerState);
      if (trained && ((!t.has(Input) && !t.has(Output)) || t.has(Constant)))
        throw Fail{1, "a parameter or optimizer state must be an input or output and not a constant"};
      uint64_t n = 1;
      for (auto d : t.dims) {
        if (d == 0 || n > UINT64_MAX / d)
          throw Fail{1, "tensor has a zero dimension or its element count overflows"};
        n *= d;
      }
      if (n > UINT64_MAX / dtype_size(t.dtype))
        throw Fail{1, "tensor byte count overflows"};
    }
    std::set<uint32_t> available, written, op_ids;
    for (const auto &t : program.tensors)
      if (t.has(Input) || t.has(Constant))
        available.insert(t.id);
    for (const auto &op : program.ops) {
      if (op.id == 0 || !op_ids.insert(op.id).second)
        throw Fail{1, "operation ids must be unique and non-zero"};
      if (op.opcode < kFirstOpcode || op.opcode > kLastOpcode)
        throw Fail{1, "opcode out of range"};
      std::set<uint32_t> keys;
      for (const auto &a : op.attrs) {
        if (a.key < kFirstAttr || a.key > kLastAttr || a.kind < 1 || a.kind > 4 || !keys.insert(a.key).second)
          bad(op, "invalid or duplicate attribute");
        if (a.kind == 4 && a.bits > 1)
          bad(op, "boolean attribute out of range");
        if (a.kind == 3) {
          double v;
          std::memcpy(&v, &a.bits, 8);
          if (!std::isfinite(v))
            bad(op, "non-finite attribute");
        }
      }
      for (auto id : op.in)
        if (!available.count(id))
          bad(op, "input " + std::to_string(id) + " is not available before this operation");
      for (auto id : op.out) {
        const Tensor *t = program.tensor(id);
        if (!t)
          bad(op, "unknown output tensor");
        if (t->has(Input) || t->has(Constant) || !written.insert(id).second)
          bad(op, "outputs must be written once and may not be inputs or constants");
      }
      verify_op(program, op);
      for (auto id : op.out)
        available.insert(id);
    }
    for (const auto &t : program.tensors)
      if (t.has(Output) && !available.count(t.id))
        throw Fail{1, "output tensor " + std::to_string(t.id) + " is never produced"};
  } catch (const Fail &f) {
    error = f.text;
    return f.status;
  } catch (const std::exception &e) {
    error = std::string("malformed program: ") + e.what();
    return 1;
  }
  return 0;
}

} // namespace ir
} // namespace difb200
