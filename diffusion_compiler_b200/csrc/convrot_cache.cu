// ConvRot INT8 weight caches: reading and writing the files the reference keeps its quantised
// Linear weights in, and building one on the GPU.
//
// Container: SafeTensors as the reference reads and writes it (src/weights/safetensors.cpp:
// an 8-byte little-endian header length, a JSON object {name: {"dtype", "shape",
// "data_offsets": [begin, end]}} padded with spaces to a multiple of 8, then the tensor bytes in
// header order; dtype names F32 BF16 F16 I8 I32 BOOL F8_E4M3 F8_E8M0; names starting with
// "__meta__." may carry other dtypes). Two cache forms use it:
//   * per-Linear pairs "weight" I8 [N,K] + "scale" F32 [N] (+ "input_scale" [K]) in one file per
//     projection, written behind a ".building" name and renamed when complete
//     (tools/difflux2sample.cpp:3074-3097);
//   * the generic cache: "linear.<weight tensor id>.weight" / ".scale" for every eligible Linear
//     of a program plus the identity record "__meta__.convrot_int8" I32[20] = {magic 0x31525643
//     "CVR1", version 1, rotation group 256, projection count, 8 words of the program's
//     fingerprint (SHA-256 of its DIFIR bytes without the trailing digest), 8 words of the source
//     index digest} (src/runtime/cuda_executor.cpp:4266-4364, tools/difh3convrot.cpp:51,208-231).
// The encoder of the weights is the weight-side quantiser (quantize_int8_rows on the [N,K] rows).
#include "difb200/difb200.h"

#include "common.cuh"
#include "diffir.h"
#include "ops.h"

#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include <sys/stat.h>

namespace difb200 {
namespace {

constexpr uint32_t kCvr1Magic = 0x31525643u, kCvr1Version = 1u, kCvr1Group = 256u;

struct CacheTensor {
  uint32_t dtype = 0; // DiffIR code; 0 for a metadata tensor of another dtype
  std::vector<uint64_t> dims;
  uint64_t offset = 0, bytes = 0;
};

struct Cache {
  std::vector<uint8_t> file;
  std::map<std::string, CacheTensor> tensors;
};

const char *dtype_name(uint32_t dtype) {
  switch (dtype) {
  case ir::F32: return "F32";
  case ir::BF16: return "BF16";
  case ir::F16: return "F16";
  case ir::I8: return "I8";
  case ir::I32: return "I32";
  case ir::Bool: return "BOOL";
  case ir::FP8E4M3: return "F8_E4M3";
  case ir::FP8E8M0: return "F8_E8M0";
  default: return nullptr;
  }
}
uint32_t dtype_code(const std::string &name) {
  for (uint32_t code = 1; code <= 8; ++code)
    if (name == dtype_name(code))
      return code;
  return 0;
}
uint64_t width_of(const std::string &name) {
  if (name == "F64" || name == "I64" || name == "U64")
    return 8;
  if (name == "F32" || name == "I32" || name == "U32")
    return 4;
  if (name == "BF16" || name == "F16" || name == "I16" || name == "U16")
    return 2;
  if (name == "I8" || name == "U8" || name == "BOOL" || name == "F8_E4M3" || name == "F8_E8M0" || name == "F8_E5M2")
    return 1;
  return 0;
}

// ---- the little JSON a SafeTensors header is made of ----
struct Json {
  const char *p, *end;
  std::string error;
  void skip() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r'))
      ++p;
  }
  bool take(char c) {
    skip();
    if (p < end && *p == c) {
      ++p;
      return true;
    }
    return false;
  }
  bool string(std::string &out) {
    skip();
    if (p >= end || *p != '"')
      return false;
    ++p;
    out.clear();
    while (p < end && *p != '"') {
      if (*p == '\\') {
        if (p + 1 >= end)
          return false;
        ++p;
        if (*p == 'u') { // \u00XX as the reference's writer emits for control bytes
          if (p + 4 >= end)
            return false;
          out.push_back((char)std::strtoul(std::string(p + 1, p + 5).c_str(), nullptr, 16));
          p += 5;
          continue;
        }
        out.push_back(*p == 'n' ? '\n' : (*p == 't' ? '\t' : *p));
        ++p;
        continue;
      }
      out.push_back(*p++);
    }
    return p < end && *p++ == '"';
  }
  bool number(uint64_t &out) {
    skip();
    if (p >= end || *p < '0' || *p > '9')
      return false;
    out = 0;
    while (p < end && *p >= '0' && *p <= '9') {
      if (out > (0xffffffffffffffffull - 9) / 10)
        return false;
      out = out * 10 + (uint64_t)(*p++ - '0');
    }
    return true;
  }
  bool skip_value() { // anything (used for "__metadata__")
    skip();
    if (p >= end)
      return false;
    if (*p == '"') {
      std::string s;
      return string(s);
    }
    if (*p == '{' || *p == '[') {
      const char open = *p, close = open == '{' ? '}' : ']';
      ++p;
      if (take(close))
        return true;
      for (;;) {
        if (open == '{') {
          std::string key;
          if (!string(key) || !take(':'))
            return false;
        }
        if (!skip_value())
          return false;
        if (take(close))
          return true;
        if (!take(','))
          return false;
      }
    }
    while (p < end && *p != ',' && *p != '}' && *p != ']')
      ++p;
    return true;
  }
};

int parse(Cache &cache, std::string &error) {
  const std::vector<uint8_t> &f = cache.file;
  if (f.size() < 8)
    return error = "file is shorter than a SafeTensors header length", 1;
  uint64_t header = 0;
  for (int i = 7; i >= 0; --i)
    header = (header << 8) | f[(size_t)i];
  if (header == 0 || header > f.size() - 8)
    return error = "invalid SafeTensors header length", 1;
  const uint64_t data_offset = 8 + header;
  Json j{reinterpret_cast<const char *>(f.data()) + 8, reinterpret_cast<const char *>(f.data()) + data_offset, {}};
  if (!j.take('{'))
    return error = "SafeTensors header root must be an object", 1;
  if (j.take('}'))
    return error = "SafeTensors file has no tensors", 1;
  for (;;) {
    std::string name;
    if (!j.string(name) || !j.take(':'))
      return error = "malformed SafeTensors header", 1;
    if (name == "__metadata__") {
      if (!j.skip_value())
        return error = "malformed __metadata__", 1;
    } else {
      if (!j.take('{'))
        return error = "invalid SafeTensors tensor record: " + name, 1;
      std::string dtype;
      CacheTensor t;
      uint64_t begin = 0, finish = 0;
      bool have_dtype = false, have_shape = false, have_offsets = false;
      for (;;) {
        std::string key;
        if (!j.string(key) || !j.take(':'))
          return error = "invalid SafeTensors tensor record: " + name, 1;
        if (key == "dtype") {
          have_dtype = j.string(dtype);
        } else if (key == "shape") {
          if (!j.take('['))
            return error = "invalid shape of " + name, 1;
          if (!j.take(']'))
            for (;;) {
              uint64_t d = 0;
              if (!j.number(d))
                return error = "invalid shape of " + name, 1;
              t.dims.push_back(d);
              if (j.take(']'))
                break;
              if (!j.take(','))
                return error = "invalid shape of " + name, 1;
            }
          have_shape = true;
        } else if (key == "data_offsets") {
          have_offsets = j.take('[') && j.number(begin) && j.take(',') && j.number(finish) && j.take(']');
        } else if (!j.skip_value()) {
          return error = "invalid SafeTensors tensor record: " + name, 1;
        }
        if (j.take('}'))
          break;
        if (!j.take(','))
          return error = "invalid SafeTensors tensor record: " + name, 1;
      }
      if (!have_dtype || !have_shape || !have_offsets)
        return error = "invalid SafeTensors tensor record: " + name, 1;
      if (finish < begin || finish > f.size() - data_offset)
        return error = "SafeTensors tensor offset is out of bounds: " + name, 1;
      uint64_t elements = 1;
      for (uint64_t d : t.dims) {
        if (d == 0 || elements > 0xffffffffffffffffull / d)
          return error = "SafeTensors tensor shape overflow: " + name, 1;
        elements *= d;
      }
      const uint64_t width = width_of(dtype);
      if (width == 0 || t.dims.size() > 8 || elements * width != finish - begin)
        return error = "SafeTensors tensor byte count mismatch: " + name, 1;
      t.dtype = dtype_code(dtype);
      if (t.dtype == 0 && name.rfind("__meta__.", 0) != 0 && !t.dims.empty())
        return error = "unsupported non-metadata SafeTensors dtype " + dtype + " for tensor " + name, 1;
      t.offset = data_offset + begin;
      t.bytes = finish - begin;
      cache.tensors[name] = t;
    }
    if (j.take('}'))
      break;
    if (!j.take(','))
      return error = "malformed SafeTensors header", 1;
  }
  if (cache.tensors.empty())
    return error = "SafeTensors file has no tensors", 1;
  return 0;
}

std::string json_string(const std::string &value) {
  std::string out = "\"";
  for (char c : value) {
    if (c == '"' || c == '\\') {
      out.push_back('\\');
      out.push_back(c);
    } else if ((unsigned char)c < 0x20) {
      char buf[8];
      std::snprintf(buf, sizeof(buf), "\\u%04x", (unsigned)(unsigned char)c);
      out += buf;
    } else {
      out.push_back(c);
    }
  }
  return out + "\"";
}

} // namespace
} // namespace difb200

using namespace difb200;

extern "C" {

int difb200_cache_open(const char *path, void **cache) {
  if (!path || !cache)
    return fail(kInvalidArgument, "difb200_cache_open: null argument");
  *cache = nullptr;
  FILE *f = std::fopen(path, "rb");
  if (!f)
    return fail(kInvalidArgument, std::string("cannot open ConvRot cache: ") + path);
  Cache *c = new Cache();
  std::fseek(f, 0, SEEK_END);
  const long size = std::ftell(f);
  std::fseek(f, 0, SEEK_SET);
  c->file.resize(size > 0 ? (size_t)size : 0);
  const size_t got = c->file.empty() ? 0 : std::fread(c->file.data(), 1, c->file.size(), f);
  std::fclose(f);
  std::string error;
  if (got != c->file.size() || parse(*c, error)) {
    delete c;
    return fail(kInvalidArgument, std::string(path) + ": " + (error.empty() ? "cannot read the file" : error));
  }
  *cache = c;
  return kOk;
}

int difb200_cache_close(void *cache) {
  delete static_cast<Cache *>(cache);
  return kOk;
}

int difb200_cache_tensor(void *cache, const char *name, uint32_t *dtype, uint32_t *rank, uint64_t *dims8,
                         const void **data, uint64_t *bytes) {
  Cache *c = static_cast<Cache *>(cache);
  if (!c || !name)
    return fail(kInvalidArgument, "difb200_cache_tensor: null argument");
  const auto it = c->tensors.find(name);
  if (it == c->tensors.end())
    return fail(kInvalidArgument, std::string("the cache holds no tensor named ") + name);
  if (dtype)
    *dtype = it->second.dtype;
  if (rank)
    *rank = (uint32_t)it->second.dims.size();
  if (dims8)
    for (size_t i = 0; i < it->second.dims.size(); ++i)
      dims8[i] = it->second.dims[i];
  if (data)
    *data = c->file.data() + it->second.offset;
  if (bytes)
    *bytes = it->second.bytes;
  return kOk;
}

int difb200_cache_write(const char *path, uint32_t count, const char *const *names, const uint32_t *dtypes,
                        const uint32_t *ranks, const uint64_t *dims8, const void *const *data) {
  if (!path || !names || !dtypes || !ranks || !dims8 || !data || count == 0)
    return fail(kInvalidArgument, "difb200_cache_write: null argument or no tensors");
  std::string header = "{";
  std::vector<uint64_t> sizes;
  uint64_t offset = 0;
  std::map<std::string, bool> seen;
  for (uint32_t i = 0; i < count; ++i) {
    const char *dtype = dtype_name(dtypes[i]);
    if (!names[i] || !names[i][0] || !dtype || ranks[i] == 0 || ranks[i] > 8 || !seen.emplace(names[i], true).second)
      return fail(kInvalidArgument, "difb200_cache_write: invalid tensor specification");
    uint64_t elements = 1;
    for (uint32_t a = 0; a < ranks[i]; ++a) {
      if (dims8[8 * i + a] == 0)
        return fail(kInvalidArgument, "difb200_cache_write: zero dimension");
      elements *= dims8[8 * i + a];
    }
    const uint64_t bytes = elements * ir::dtype_size(dtypes[i]);
    sizes.push_back(bytes);
    header += (i ? "," : "") + json_string(names[i]) + ":{\"dtype\":" + json_string(dtype) + ",\"shape\":[";
    for (uint32_t a = 0; a < ranks[i]; ++a)
      header += (a ? "," : "") + std::to_string(dims8[8 * i + a]);
    header += "],\"data_offsets\":[" + std::to_string(offset) + "," + std::to_string(offset + bytes) + "]}";
    offset += bytes;
  }
  header += "}";
  while (header.size() % 8 != 0)
    header.push_back(' ');
  // an unfinished file never carries the final name (tools/difflux2sample.cpp:3074-3097)
  const std::string building = std::string(path) + ".building";
  struct stat st;
  if (stat(building.c_str(), &st) == 0)
    return fail(kExecutionError, "refusing to overwrite an incomplete cache: " + building);
  FILE *f = std::fopen(building.c_str(), "wb");
  if (!f)
    return fail(kExecutionError, "cannot create " + building);
  unsigned char length[8];
  for (int i = 0; i < 8; ++i)
    length[i] = (unsigned char)((uint64_t)header.size() >> (8 * i));
  bool ok = std::fwrite(length, 1, 8, f) == 8 && std::fwrite(header.data(), 1, header.size(), f) == header.size();
  for (uint32_t i = 0; i < count && ok; ++i)
    ok = sizes[i] == 0 || std::fwrite(data[i], 1, (size_t)sizes[i], f) == sizes[i];
  ok = std::fclose(f) == 0 && ok;
  if (!ok || std::rename(building.c_str(), path) != 0) {
    std::remove(building.c_str());
    return fail(kExecutionError, std::string("cannot write ") + path);
  }
  return kOk;
}

int difb200_program_fingerprint(const uint8_t *diffir, uint64_t size, uint8_t *digest32) {
  if (!diffir || !digest32 || size <= 32)
    return fail(kInvalidArgument, "difb200_program_fingerprint: not DIFIR bytes");
  ir::sha256(diffir, (size_t)size - 32, digest32); // the trailing 32 bytes are this very digest
  return kOk;
}

void difb200_cvr1_identity(uint32_t projections, const uint8_t *program_digest32, const uint8_t *index_digest32,
                           uint32_t *identity20) {
  std::memset(identity20, 0, 20 * sizeof(uint32_t));
  identity20[0] = kCvr1Magic;
  identity20[1] = kCvr1Version;
  identity20[2] = kCvr1Group;
  identity20[3] = projections;
  for (int w = 0; w < 8; ++w) {
    if (program_digest32)
      identity20[4 + w] = (uint32_t)program_digest32[4 * w] | ((uint32_t)program_digest32[4 * w + 1] << 8) |
                          ((uint32_t)program_digest32[4 * w + 2] << 16) | ((uint32_t)program_digest32[4 * w + 3] << 24);
    if (index_digest32)
      identity20[12 + w] = (uint32_t)index_digest32[4 * w] | ((uint32_t)index_digest32[4 * w + 1] << 8) |
                           ((uint32_t)index_digest32[4 * w + 2] << 16) | ((uint32_t)index_digest32[4 * w + 3] << 24);
  }
}

int difb200_cvr1_check(const uint32_t *identity20, const uint8_t *diffir, uint64_t size, uint32_t projections) {
  if (!identity20)
    return fail(kInvalidArgument, "difb200_cvr1_check: null identity");
  if (identity20[0] != kCvr1Magic || identity20[1] != kCvr1Version || identity20[2] != kCvr1Group)
    return fail(kInvalidArgument, "generic ConvRot cache has unsupported format metadata");
  if (diffir) {
    uint8_t digest[32];
    if (int rc = difb200_program_fingerprint(diffir, size, digest))
      return rc;
    uint32_t expect[20];
    difb200_cvr1_identity(projections, digest, nullptr, expect);
    for (int w = 0; w < 8; ++w)
      if (identity20[4 + w] != expect[4 + w])
        return fail(kInvalidArgument, "generic ConvRot cache DiffIR fingerprint mismatch");
  }
  if (identity20[3] != projections)
    return fail(kInvalidArgument, "generic ConvRot cache projection count does not match the program");
  return kOk;
}

int difb200_build_convrot_cache(const char *path, const uint8_t *diffir, uint64_t diffir_size, uint32_t count,
                                const uint32_t *weight_ids, const void *const *host_weights_bf16,
                                const uint64_t *rows, const uint64_t *columns, const uint8_t *index_digest32,
                                void *stream) {
  if (!path || !diffir || !weight_ids || !host_weights_bf16 || !rows || !columns || count == 0)
    return fail(kInvalidArgument, "difb200_build_convrot_cache: null argument");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  std::vector<std::vector<int8_t>> codes(count);
  std::vector<std::vector<float>> scales(count);
  for (uint32_t i = 0; i < count; ++i) {
    const uint64_t N = rows[i], K = columns[i];
    if (N == 0 || K == 0 || K % kCvr1Group != 0)
      return fail(kInvalidArgument, "difb200_build_convrot_cache: widths must be multiples of the rotation group 256");
    void *w = nullptr;
    int8_t *c = nullptr;
    float *sc = nullptr;
    int rc = check_cuda(cudaMalloc(&w, N * K * 2), "cudaMalloc(weight)");
    if (!rc)
      rc = check_cuda(cudaMalloc(reinterpret_cast<void **>(&c), N * K), "cudaMalloc(codes)");
    if (!rc)
      rc = check_cuda(cudaMalloc(reinterpret_cast<void **>(&sc), N * sizeof(float)), "cudaMalloc(scales)");
    if (!rc)
      rc = check_cuda(cudaMemcpyAsync(w, host_weights_bf16[i], N * K * 2, cudaMemcpyHostToDevice, s), "cudaMemcpyAsync");
    const void *part[1] = {w};
    if (!rc)
      rc = quantize_int8_rows(part, &K, 1, N, 2 /* H256ConvRot */, 1.0f, nullptr, c, sc, nullptr, nullptr, s);
    codes[i].resize(N * K);
    scales[i].resize(N);
    if (!rc)
      rc = check_cuda(cudaMemcpyAsync(codes[i].data(), c, N * K, cudaMemcpyDeviceToHost, s), "cudaMemcpyAsync");
    if (!rc)
      rc = check_cuda(cudaMemcpyAsync(scales[i].data(), sc, N * sizeof(float), cudaMemcpyDeviceToHost, s),
                      "cudaMemcpyAsync");
    if (!rc)
      rc = check_cuda(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    cudaFree(w);
    cudaFree(c);
    cudaFree(sc);
    if (rc)
      return rc;
  }
  uint8_t digest[32];
  if (int rc = difb200_program_fingerprint(diffir, diffir_size, digest))
    return rc;
  uint32_t identity[20];
  difb200_cvr1_identity(count, digest, index_digest32, identity);
  std::vector<std::string> names;
  std::vector<uint32_t> dtypes, ranks;
  std::vector<uint64_t> dims;
  std::vector<const void *> data;
  auto add = [&](const std::string &name, uint32_t dtype, std::vector<uint64_t> shape, const void *bytes) {
    names.push_back(name);
    dtypes.push_back(dtype);
    ranks.push_back((uint32_t)shape.size());
    shape.resize(8, 0);
    dims.insert(dims.end(), shape.begin(), shape.end());
    data.push_back(bytes);
  };
  add("__meta__.convrot_int8", ir::I32, {20}, identity);
  for (uint32_t i = 0; i < count; ++i) {
    add("linear." + std::to_string(weight_ids[i]) + ".weight", ir::I8, {rows[i], columns[i]}, codes[i].data());
    add("linear." + std::to_string(weight_ids[i]) + ".scale", ir::F32, {rows[i]}, scales[i].data());
  }
  std::vector<const char *> c_names;
  for (const auto &n : names)
    c_names.push_back(n.c_str());
  return difb200_cache_write(path, (uint32_t)names.size(), c_names.data(), dtypes.data(), ranks.data(), dims.data(),
                             data.data());
}

} // extern "C"
