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

#include "aot_host.h"

using namespace llmcp_b200;
using namespace llmcp_b200::host;

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
