// llmcp-benchmark for AOT ABI v2 libraries: the driver of tools/llmcp-benchmark/llmcp-benchmark.cpp
// (same options, same protocol, same seven output lines) on top of this repository's container
// reader, so that libllmcp_b200.so can be timed the way the reference times its compiled models.
//
//   llmcp-benchmark --weights weights.bin --aot libllmcp_b200.so [--prefill-tokens 32]
//                   [--decode-tokens 8] [--token 9419] [--verbose] [--synthetic SEED]
//
// --synthetic writes a random-init Qwen3.5-4B-shaped container to --weights first if the file does
// not exist.  The timer covers the entry-point calls and the host argmax, not mapping or set-up.

#include <dlfcn.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../format.h"

using namespace llmcp_b200;

namespace {

// Strided memref descriptor of the MLIR C interface (include/llmcp/Runtime/AotRuntime.h:52-58).
template <typename T, int N> struct MemRef {
  T *base;
  T *data;
  int64_t offset;
  int64_t sizes[N];
  int64_t strides[N];
};

using EntryFn = void (*)(void *, void *, void *, void *, void *, void *, void *, void *, void *, void *);

struct Arena {
  const uint8_t *base = nullptr;
  uint64_t mapped = 0, size = 0;
  Manifest manifest;

  std::string load(const std::string &path) {
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0)
      return "cannot open " + path;
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < static_cast<off_t>(kHeaderBytes)) {
      close(fd);
      return "packed weights file is too small";
    }
    void *mapping = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (mapping == MAP_FAILED)
      return "mmap failed";
    Manifest parsed;
    const std::string error = parse_container(static_cast<const uint8_t *>(mapping), static_cast<uint64_t>(st.st_size), &parsed);
    if (!error.empty()) {
      munmap(mapping, static_cast<size_t>(st.st_size));
      return error;
    }
    base = static_cast<const uint8_t *>(mapping);
    mapped = static_cast<uint64_t>(st.st_size);
    size = parsed.total_bytes;
    manifest = std::move(parsed);
    return "";
  }
};

// lib/Runtime/AotRuntime.cpp:39-120 with the model constants of :41-43.
struct Runtime {
  ModelDims dims;
  void *handle = nullptr;
  EntryFn prefill = nullptr, decode = nullptr;
  int64_t capacity = 0;
  std::vector<uint16_t> kv, conv;
  std::vector<float> delta;

  bool init(const std::string &path, int64_t max_sequence) {
    capacity = max_sequence;
    kv.assign(static_cast<size_t>(dims.full_layers() * 2 * dims.kv_heads * capacity * dims.head_dim), 0);
    delta.assign(static_cast<size_t>(dims.linear_layers() * dims.lin_v_heads * dims.lin_k_dim * dims.lin_v_dim), 0.0f);
    conv.assign(static_cast<size_t>(dims.linear_layers() * (dims.conv_kernel - 1) * dims.qkv_dim()), 0);
    handle = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!handle) {
      std::fprintf(stderr, "AotRuntime: dlopen: %s\n", dlerror());
      return false;
    }
    auto version = reinterpret_cast<int32_t (*)()>(dlsym(handle, "llmcp_model_abi_version"));
    if (!version || version() != 2) {
      std::fprintf(stderr, "AotRuntime: incompatible AOT ABI\n");
      return false;
    }
    prefill = reinterpret_cast<EntryFn>(dlsym(handle, "_mlir_ciface_llmcp_model_prefill"));
    decode = reinterpret_cast<EntryFn>(dlsym(handle, "_mlir_ciface_llmcp_model_decode"));
    if (!prefill || !decode) {
      std::fprintf(stderr, "AotRuntime: missing prefill/decode entry points\n");
      return false;
    }
    return true;
  }

  bool forward(const Arena &arena, const std::vector<int64_t> &tokens, int64_t start, int64_t cache_length,
               std::vector<float> &logits) {
    const int64_t sequence = static_cast<int64_t>(tokens.size());
    if (sequence == 0 || start < 0 || start > capacity || sequence > capacity - start)
      return false;
    std::vector<int64_t> ids = tokens;
    const int64_t rot = dims.rotary;
    std::vector<float> cos(static_cast<size_t>(sequence * rot)), sin(cos.size());
    for (int64_t t = 0; t < sequence; ++t)
      make_cos_sin(start + t, rot, dims.rope_theta, cos.data() + t * rot, sin.data() + t * rot);
    logits.assign(static_cast<size_t>(dims.vocab), 0.0f);
    MemRef<int64_t, 1> rt{ids.data(), ids.data(), 0, {sequence}, {1}};
    MemRef<float, 2> rc{cos.data(), cos.data(), 0, {sequence, rot}, {rot, 1}};
    MemRef<float, 2> rs{sin.data(), sin.data(), 0, {sequence, rot}, {rot, 1}};
    int8_t *bytes = const_cast<int8_t *>(reinterpret_cast<const int8_t *>(arena.base));
    MemRef<int8_t, 1> ra{bytes, bytes, 0, {static_cast<int64_t>(arena.size)}, {1}};
    MemRef<uint16_t, 5> rk{kv.data(), kv.data(), 0, {dims.full_layers(), 2, dims.kv_heads, capacity, dims.head_dim},
                           {2 * dims.kv_heads * capacity * dims.head_dim, dims.kv_heads * capacity * dims.head_dim,
                            capacity * dims.head_dim, dims.head_dim, 1}};
    MemRef<float, 4> rd{delta.data(), delta.data(), 0, {dims.linear_layers(), dims.lin_v_heads, dims.lin_k_dim, dims.lin_v_dim},
                        {dims.lin_v_heads * dims.lin_k_dim * dims.lin_v_dim, dims.lin_k_dim * dims.lin_v_dim, dims.lin_v_dim, 1}};
    MemRef<uint16_t, 3> rv{conv.data(), conv.data(), 0, {dims.linear_layers(), dims.conv_kernel - 1, dims.qkv_dim()},
                           {(dims.conv_kernel - 1) * dims.qkv_dim(), dims.qkv_dim(), 1}};
    MemRef<float, 2> ro{logits.data(), logits.data(), 0, {1, dims.vocab}, {dims.vocab, 1}};
    EntryFn fn = sequence > 1 ? prefill : decode;
    fn(&rt, &rc, &rs, reinterpret_cast<void *>(start), reinterpret_cast<void *>(cache_length), &ra, &rk, &rd, &rv, &ro);
    return true;
  }
};

int64_t argmax(const std::vector<float> &values) {
  return static_cast<int64_t>(std::max_element(values.begin(), values.end()) - values.begin());
}

} // namespace

int main(int argc, char **argv) {
  std::string weights = "build/weights.bin", aot;
  int64_t prefill_tokens = 32, decode_tokens = 8, token = 9419;
  bool verbose = false, synthetic = false;
  uint64_t seed = 0;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto value = [&](const char *name) -> const char * {
      const std::string eq = std::string(name) + "=";
      if (a.rfind(eq, 0) == 0)
        return argv[i] + eq.size();
      if (a == name && i + 1 < argc)
        return argv[++i];
      return nullptr;
    };
    if (const char *v = value("--weights")) weights = v;
    else if (const char *v = value("--aot")) aot = v;
    else if (const char *v = value("--prefill-tokens")) prefill_tokens = std::atoll(v);
    else if (const char *v = value("--decode-tokens")) decode_tokens = std::atoll(v);
    else if (const char *v = value("--token")) token = std::atoll(v);
    else if (const char *v = value("--synthetic")) { synthetic = true; seed = std::strtoull(v, nullptr, 10); }
    else if (a == "--verbose") verbose = true;
    else { std::fprintf(stderr, "llmcp-benchmark: unknown option %s\n", a.c_str()); return 1; }
  }
  if (aot.empty()) {
    std::fprintf(stderr, "llmcp-benchmark: --aot is required\n");
    return 1;
  }
  if (prefill_tokens <= 0 || decode_tokens < 0) {
    std::fprintf(stderr, "llmcp-benchmark: prefill-tokens must be > 0 and decode-tokens >= 0\n");
    return 1;
  }
  Runtime runtime;
  if (synthetic && access(weights.c_str(), R_OK) != 0) {
    const uint64_t bytes = synthetic_container_bytes(runtime.dims, nullptr);
    std::vector<uint8_t> file(bytes);
    const std::string error = fill_synthetic_container(runtime.dims, seed, file.data(), bytes);
    FILE *out = error.empty() ? std::fopen(weights.c_str(), "wb") : nullptr;
    if (!out || std::fwrite(file.data(), 1, bytes, out) != bytes) {
      std::fprintf(stderr, "llmcp-benchmark: cannot write %s %s\n", weights.c_str(), error.c_str());
      return 1;
    }
    std::fclose(out);
  }
  Arena arena;
  if (const std::string error = arena.load(weights); !error.empty()) {
    std::fprintf(stderr, "llmcp-benchmark: %s\n", error.c_str());
    return 1;
  }
  if (!runtime.init(aot, prefill_tokens + decode_tokens + 8))
    return 1;

  std::vector<int64_t> prompt(static_cast<size_t>(prefill_tokens), token);
  std::vector<float> logits;
  auto seconds = [](auto a, auto b) { return std::chrono::duration<double>(b - a).count(); };
  const auto prefill_begin = std::chrono::steady_clock::now();
  if (!runtime.forward(arena, prompt, 0, prefill_tokens, logits))
    return 1;
  const auto prefill_end = std::chrono::steady_clock::now();
  std::vector<int64_t> generated;
  const auto decode_begin = std::chrono::steady_clock::now();
  for (int64_t i = 0; i < decode_tokens; ++i) {
    const int64_t next = argmax(logits);
    generated.push_back(next);
    const int64_t position = prefill_tokens + i;
    if (!runtime.forward(arena, {next}, position, position + 1, logits))
      return 1;
  }
  const auto decode_end = std::chrono::steady_clock::now();
  const double p = seconds(prefill_begin, prefill_end), d = seconds(decode_begin, decode_end);
  std::printf("prefill_tokens: %lld\n", static_cast<long long>(prefill_tokens));
  std::printf("decode_tokens: %lld\n", static_cast<long long>(decode_tokens));
  std::printf("prefill_seconds: %.4f\n", p);
  std::printf("decode_seconds: %.4f\n", d);
  std::printf("total_seconds: %.4f\n", p + d);
  std::printf("prefill_tokens_per_second: %.4f\n", prefill_tokens / p);
  std::printf("decode_tokens_per_second: %.4f\n", d > 0 ? decode_tokens / d : 0.0);
  if (verbose) {
    std::printf("generated_tokens:");
    for (int64_t id : generated)
      std::printf(" %lld", static_cast<long long>(id));
    std::printf("\n");
  }
  return 0;
}
