// TEST INFRASTRUCTURE ONLY. A command-line probe of the reference's offline weight packer
// (reference tools/difflux2sample.cpp): that tool keeps its functions in an unnamed namespace, so
// this file includes the tool's source where it lies (nothing is copied), renames its main(), and
// exposes the one self-contained piece of the packer that the INT8 weight path depends on: the
// MSE-optimal row scale search, choose_mse_int8_weight_scale (tools/difflux2sample.cpp:1225-1259).
// The rest of the tool (frontends, tokenizer, PNG, sampling) is never called; the link leaves
// those references unresolved (oracle/Makefile).
//
//   difpacker_scale <rows.f32> <rows> <columns>     prints one scale per row as 8 hex digits
#define main difflux2sample_tool_main
#include "tools/difflux2sample.cpp"
#undef main

#include <cstdio>
#include <cstdlib>

int main(int argc, char **argv) {
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
