// Native DiffIR model, DIFIR001 decoder and the subset verifier of the difb200 plugin.
// Wire format and rules follow the reference (src/ir/codec.cpp:370-476 for the byte layout,
// src/ir/verify.cpp:2051-2122 for the program-level rules); written from those descriptions,
// with its own SHA-256 (FIPS 180-4).
#pragma once

#include <stdint.h>

#include <string>
#include <vector>

namespace difb200 {
namespace ir {

enum DType : uint32_t { F32 = 1, BF16 = 2, F16 = 3, I8 = 4, I32 = 5, Bool = 6, FP8E4M3 = 7, FP8E8M0 = 8 };
enum Role : uint32_t { Input = 1, Output = 2, Constant = 4, Streamed = 8, Parameter = 16, OptimizerState = 32 };

enum Opcode : uint32_t {
  Add = 1, Multiply = 2, RmsNormModulate = 3, SwiGlu = 4, ResidualGate = 5, Linear = 6,
  QkNormPartialRope = 7, Attention = 8, BiasAdd = 10, SiLU = 16, RmsNorm = 17, Fill = 18, Cast = 21,
  AffineLastDim = 29, Gelu = 49, Sigmoid = 50, Reshape = 51, BroadcastTo = 52, Slice = 53,
  RotaryFrequency = 54, RotaryApply = 55, BooleanMaskToBias = 56, Concat = 59,
  QuantizeInt8Rows = 67, LinearInt8Scaled = 68, LayerNormModulate = 75,
  kFirstOpcode = 1, kLastOpcode = 75,
};

enum AttrKey : uint32_t {
  Epsilon = 1, BlockSize = 2, Heads = 3, HeadDim = 4, RotaryDim = 5, AttentionScale = 6, Causal = 7,
  Implementation = 9, GateFirst = 13, Value = 15, Scale = 18, KvHeads = 39, Approximation = 40, Axis = 41,
  Start = 42, Theta = 43, Ntk = 44, WeightOffset = 45, RotaryLayout = 46, LinearBiasMode = 55,
  ReductionTileSize = 56, ModulationLayout = 57, WorkspaceLimitBytes = 58, MaskQueries = 73,
  kFirstAttr = 1, kLastAttr = 74,
};

struct Attr {
  uint32_t key, kind;
  uint64_t bits;
};

struct Tensor {
  uint32_t id = 0, dtype = 0, roles = 0;
  std::vector<uint64_t> dims;
  uint64_t elements() const;
  uint64_t bytes() const;
  uint64_t last() const { return dims.back(); }
  uint64_t rows() const { return elements() / dims.back(); }
  bool has(uint32_t role) const { return (roles & role) != 0; }
  bool is_float() const { return dtype == F32 || dtype == BF16 || dtype == F16; }
};

struct Op {
  uint32_t id = 0, opcode = 0;
  std::vector<uint32_t> in, out;
  std::vector<Attr> attrs;
  const Attr *find(uint32_t key) const;
  uint64_t u64(uint32_t key, uint64_t fallback) const;
  double f64(uint32_t key, double fallback) const;
  bool boolean(uint32_t key, bool fallback) const;
};

struct Program {
  std::vector<Tensor> tensors;
  std::vector<Op> ops;
  const Tensor *tensor(uint32_t id) const;
  int index_of(uint32_t id) const;
};

size_t dtype_size(uint32_t dtype);
const char *opcode_name(uint32_t opcode);

void sha256(const uint8_t *data, size_t size, uint8_t digest[32]);

// Both return 0 on success; otherwise a dif_backend_status value (1 = malformed / invalid,
// 2 = an opcode or form this backend does not implement) and text in `error`.
int decode(const uint8_t *bytes, size_t size, Program &program, std::string &error);
int verify(const Program &program, std::string &error);

} // namespace ir
} // namespace difb200
