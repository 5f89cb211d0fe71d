// llmcp-pack: packs a Qwen3.5 text checkpoint (config.json + safetensors shards) into the
// single-file weight container, with the options and the summary line of
// tools/llmcp-pack/llmcp-pack.cpp:
//
//   llmcp-pack --model DIR [--out weights.bin] [--quant none|q8_0] [--dry-run] [--verbose]
//
// Both `--name value` and `--name=value` are accepted, with one or two dashes.
//
// Additive (not in the reference's tool): `llmcp-pack --synthetic SEED --out weights.bin` writes
// the q8_0 container of a random-init model with the Qwen3.5-4B text dimensions, the stand-in
// for the real checkpoint that benchmarks and tests use.  Host code only.

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "../checkpoint.h"
#include "../format.h"

using namespace llmcp_b200;

int main(int argc, char **argv) {
  std::string model, out, quant = "none", synthetic;
  bool dry_run = false, verbose = false;
  for (int i = 1; i < argc; ++i) {
    std::string arg = argv[i];
    while (!arg.empty() && arg[0] == '-')
      arg.erase(0, 1);
    std::string value;
    bool has_value = false;
    const size_t eq = arg.find('=');
    if (eq != std::string::npos) {
      value = arg.substr(eq + 1);
      arg.erase(eq);
      has_value = true;
    }
    auto take = [&](std::string *dst) {
      if (!has_value) {
        if (i + 1 >= argc) {
          std::fprintf(stderr, "llmcp-pack: --%s needs a value\n", arg.c_str());
          return false;
        }
        value = argv[++i];
      }
      *dst = value;
      return true;
    };
    if (arg == "model") {
      if (!take(&model))
        return 1;
    } else if (arg == "out") {
      if (!take(&out))
        return 1;
    } else if (arg == "synthetic") {
      if (!take(&synthetic))
        return 1;
    } else if (arg == "quant") {
      if (!take(&quant))
        return 1;
    } else if (arg == "dry-run") {
      dry_run = !has_value || value != "false";
    } else if (arg == "verbose") {
      verbose = !has_value || value != "false";
    } else {
      std::fprintf(stderr, "llmcp-pack: unknown option '%s'\n", argv[i]);
      return 1;
    }
  }
  if (!synthetic.empty()) {
    if (out.empty()) {
      std::fprintf(stderr, "llmcp-pack: --synthetic needs --out\n");
      return 1;
    }
    const ModelDims dims;
    const uint64_t bytes = synthetic_container_bytes(dims, nullptr);
    std::vector<uint8_t> file(bytes);
    const std::string error = fill_synthetic_container(dims, std::strtoull(synthetic.c_str(), nullptr, 10), file.data(), bytes);
    if (!error.empty()) {
      std::fprintf(stderr, "llmcp-pack: %s\n", error.c_str());
      return 1;
    }
    const std::string tmp = out + ".tmp";
    FILE *f = std::fopen(tmp.c_str(), "wb");
    if (!f || std::fwrite(file.data(), 1, bytes, f) != bytes || std::fclose(f) != 0 || std::rename(tmp.c_str(), out.c_str()) != 0) {
      std::fprintf(stderr, "llmcp-pack: cannot write %s\n", out.c_str());
      return 1;
    }
    std::printf("synthetic container, seed %s, %llu bytes -> %s\n", synthetic.c_str(), static_cast<unsigned long long>(bytes),
                out.c_str());
    return 0;
  }
  if (model.empty()) {
    std::fprintf(stderr, "llmcp-pack: --model is required\n");
    return 1;
  }
  if (!dry_run && out.empty()) {
    std::fprintf(stderr, "llmcp-pack: --out is required unless --dry-run is set\n");
    return 1;
  }
  PackSummary summary;
  const std::string error = pack_checkpoint(model, out, quant, dry_run, verbose, &summary);
  if (!error.empty()) {
    std::fprintf(stderr, "llmcp-pack: %s\n", error.c_str());
    return 1;
  }
  std::printf("%s %llu tensors, %llu source bytes, arena %llu bytes, quant %s", dry_run ? "validated" : "packed",
              static_cast<unsigned long long>(summary.tensors), static_cast<unsigned long long>(summary.source_bytes),
              static_cast<unsigned long long>(summary.arena_bytes), quant.c_str());
  if (!dry_run)
    std::printf(" -> %s", out.c_str());
  std::printf("\n");
  return 0;
}
