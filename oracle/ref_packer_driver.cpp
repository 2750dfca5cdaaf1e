// TEST INFRASTRUCTURE ONLY. A command-line probe of the reference's offline weight packer
// (reference tools/difflux2sample.cpp): that tool keeps its functions in an unnamed namespace, so
// this file includes the tool's source where it lies (nothing is copied), renames its main(), and
// calls the two pieces of the packer that the INT8 weight path depends on:
//
//   difpacker_scale <rows.f32> <rows> <columns>
//       choose_mse_int8_weight_scale (tools/difflux2sample.cpp:1225-1259) on fp32 rows; prints one
//       scale per row as 8 hex digits
//   difpacker_scale pack <weight.bf16> <rows> <columns> <quantization 1..7> <equalise 0|1> <mse 0|1> <directory>
//       rewrite_named_linear_w8a8 (tools/difflux2sample.cpp:1607-2096) on a one-Linear program whose
//       weight is the given bf16 matrix: the tool computes the input-equalisation vector, rotates and
//       encodes the rows and writes its cache file (weight, scale, input_scale) into the directory;
//       prints the file's path
//
// The rest of the tool (frontends, tokenizer, PNG, sampling) is never called; the link leaves those
// references unresolved (oracle/Makefile).
#define main difflux2sample_tool_main
#include "tools/difflux2sample.cpp"
#undef main

#include <cstdio>
#include <cstdlib>

namespace {
int pack(int argc, char **argv) {
  if (argc != 9) {
    std::fprintf(stderr, "usage: difpacker_scale pack <weight.bf16> <rows> <columns> <quantization> <equalise> <mse> <directory>\n");
    return 2;
  }
  const std::uint64_t rows = std::strtoull(argv[3], nullptr, 10), columns = std::strtoull(argv[4], nullptr, 10);
  const auto quantization = static_cast<dif::ir::Int8RowQuantization>(std::strtoull(argv[5], nullptr, 10));
  const bool equalise = std::atoi(argv[6]) != 0, mse = std::atoi(argv[7]) != 0;
  std::vector<std::uint8_t> bytes(static_cast<std::size_t>(rows * columns * 2U));
  std::FILE *f = std::fopen(argv[2], "rb");
  if (!f || std::fread(bytes.data(), 1U, bytes.size(), f) != bytes.size()) {
    std::fprintf(stderr, "difpacker_scale: cannot read %zu bytes from %s\n", bytes.size(), argv[2]);
    return 1;
  }
  std::fclose(f);
  // x [4, columns] -> Linear(x, w) -> y [4, rows]; the weight is checkpoint tensor "blk.0.weight"
  constexpr std::uint32_t input_role = static_cast<std::uint32_t>(dif::ir::TensorRole::Input);
  constexpr std::uint32_t output_role = static_cast<std::uint32_t>(dif::ir::TensorRole::Output);
  constexpr std::uint32_t constant_role = static_cast<std::uint32_t>(dif::ir::TensorRole::Constant);
  dif::ir::Program program;
  program.tensors.push_back({1U, dif::ir::DType::BF16, input_role, {4U, columns}});
  program.tensors.push_back({2U, dif::ir::DType::BF16, constant_role, {rows, columns}});
  program.tensors.push_back({3U, dif::ir::DType::BF16, output_role, {4U, rows}});
  program.operations.push_back({1U, dif::ir::Opcode::Linear, {1U, 2U}, {3U}, {}});
  dif::runtime::TensorMap bindings;
  bindings.emplace(2U, dif::runtime::Tensor{dif::ir::DType::BF16, {rows, columns}, std::move(bytes)});
  dif::frontend::Flux2KleinTransformerBuild transformer;
  transformer.checkpoint_tensors = {2U};
  transformer.checkpoint_names = {"blk.0.weight"};
  const std::uint32_t blocks[1] = {0U};
  try {
    const auto result = rewrite_named_linear_w8a8(program, bindings, transformer, blocks, quantization, "blk.",
                                                  ".weight", "probe", fs::path(argv[8]), equalise, mse, false);
    if (result.linear_count != 1U) {
      std::fprintf(stderr, "difpacker_scale: the packer rewrote %llu Linear ops\n",
                   static_cast<unsigned long long>(result.linear_count));
      return 1;
    }
  } catch (const std::exception &error) {
    std::fprintf(stderr, "difpacker_scale: %s\n", error.what());
    return 1;
  }
  for (const auto &entry : fs::directory_iterator(argv[8]))
    std::printf("%s\n", entry.path().c_str());
  return 0;
}
} // namespace

int main(int argc, char **argv) {
  if (argc >= 2 && std::strcmp(argv[1], "pack") == 0)
    return pack(argc, argv);
  if (argc != 4) {
    std::fprintf(stderr, "usage: difpacker_scale <rows.f32> <rows> <columns>\n");
    return 2;
  }
  const std::size_t rows = std::strtoull(argv[2], nullptr, 10), columns = std::strtoull(argv[3], nullptr, 10);
  std::vector<float> values(rows * columns);
  std::FILE *f = std::fopen(argv[1], "rb");
  if (!f || std::fread(values.data(), sizeof(float), values.size(), f) != values.size()) {
    std::fprintf(stderr, "difpacker_scale: cannot read %zu floats from %s\n", values.size(), argv[1]);
    return 1;
  }
  std::fclose(f);
  for (std::size_t r = 0; r < rows; ++r) {
    const float scale = choose_mse_int8_weight_scale(std::span<const float>(values.data() + r * columns, columns));
    std::uint32_t bits;
    std::memcpy(&bits, &scale, sizeof(bits));
    std::printf("%08x\n", bits);
  }
  return 0;
}
