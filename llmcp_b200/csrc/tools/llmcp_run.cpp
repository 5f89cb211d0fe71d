// llmcp-run, AOT half: the generation driver of tools/llmcp-run/llmcp-run.cpp:626-704 for AOT ABI v2
// libraries (prefill, greedy decode until --max-new-tokens or the end-of-turn token, text streamed
// through the ByteLevel streaming decoder, then the `tokens:` line; without new tokens the
// `aot logits: N next T` line), on top of this repository's container reader.
//
//   llmcp-run --weights weights.bin --aot libllmcp_b200.so --tokenizer tokenizer.json
//             [--text 'Hello' [--chat] [--system S] [--no-thinking] | --tokens ID | --token-ids a,b,c]
//             [--max-new-tokens N] [--eos-token ID] [--dump-logits] [--synthetic SEED]
//   llmcp-run --tokenizer tokenizer.json --text 'Hello' --tokenize-only [--expect-token ID]
//   llmcp-run --text 'Hello' [--chat] [--system S] [--no-thinking] --print-prompt
//
// --text is encoded with the tokenizer's own pre-tokeniser, normaliser and merges (text.h); with
// --chat the Qwen chat template goes around it first (llmcp-run.cpp:608-624).  --tokenize-only
// prints the ids, comma-separated, and exits (llmcp-run.cpp:646-653).  --print-prompt writes the text
// that would be encoded and exits.  The reference's interpreter half (no --aot) is not here.

#include <cstdlib>
#include <cstring>
#include <fstream>
#include <sstream>

#include "../text.h"
#include "aot_host.h"

using namespace llmcp_b200;
using namespace llmcp_b200::host;

int main(int argc, char **argv) {
  std::string weights = "build/weights.bin", aot, tokenizer_path, text, system_prompt, ids_text;
  int64_t token = 9419, max_new_tokens = 0, eos_override = -2, expect_token = -1;
  bool chat = false, no_thinking = false, dump_logits = false, print_prompt = false, synthetic = false, tokenize_only = false;
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
    else if (const char *v = value("--tokenizer")) tokenizer_path = v;
    else if (const char *v = value("--tokens")) token = std::atoll(v);
    else if (const char *v = value("--token-ids")) ids_text = v;
    else if (const char *v = value("--text")) text = v;
    else if (const char *v = value("--system")) system_prompt = v;
    else if (const char *v = value("--max-new-tokens")) max_new_tokens = std::atoll(v);
    else if (const char *v = value("--eos-token")) eos_override = std::atoll(v);
    else if (const char *v = value("--synthetic")) { synthetic = true; seed = std::strtoull(v, nullptr, 10); }
    else if (a == "--chat") chat = true;
    else if (a == "--no-thinking") no_thinking = true;
    else if (a == "--dump-logits") dump_logits = true;
    else if (const char *v = value("--expect-token")) expect_token = std::atoll(v);
    else if (a == "--print-prompt") print_prompt = true;
    else if (a == "--tokenize-only") tokenize_only = true;
    else { std::fprintf(stderr, "llmcp-run: unknown option %s\n", a.c_str()); return 1; }
  }
  if (print_prompt) {
    const std::string prompt = chat ? make_chat_prompt(text, system_prompt, !no_thinking) : text;
    std::fwrite(prompt.data(), 1, prompt.size(), stdout);
    return 0;
  }
  if (max_new_tokens < 0) {
    std::fprintf(stderr, "llmcp-run: max-new-tokens must be >= 0\n");
    return 1;
  }

  ByteLevelVocab vocab;
  bool have_vocab = false;
  int64_t eos = -1;
  if (!tokenizer_path.empty()) {
    std::ifstream file(tokenizer_path, std::ios::binary);
    std::stringstream blob;
    blob << file.rdbuf();
    if (!file) {
      std::fprintf(stderr, "llmcp-run: cannot read %s\n", tokenizer_path.c_str());
      return 1;
    }
    const std::string json = blob.str();
    if (const std::string error = vocab.load(json.data(), json.size()); !error.empty()) {
      std::fprintf(stderr, "llmcp-run: %s\n", error.c_str());
      return 1;
    }
    have_vocab = true;
    eos = vocab.token_to_id("<|im_end|>");
  }
  if (eos_override != -2)
    eos = eos_override;

  std::vector<int64_t> tokens;
  if (!text.empty()) {
    if (!have_vocab) {
      std::fprintf(stderr, "llmcp-run: --text needs --tokenizer\n");
      return 1;
    }
    std::vector<int32_t> ids;
    const std::string prompt = chat ? make_chat_prompt(text, system_prompt, !no_thinking) : text;
    if (const std::string error = vocab.encode(prompt, &ids); !error.empty()) {
      std::fprintf(stderr, "llmcp-run: %s\n", error.c_str());
      return 1;
    }
    tokens.assign(ids.begin(), ids.end());
  } else if (!ids_text.empty()) {
    std::stringstream stream(ids_text);
    std::string item;
    while (std::getline(stream, item, ',')) {
      char *end = nullptr;
      const long long id = std::strtoll(item.c_str(), &end, 10);
      if (item.empty() || *end) {
        std::fprintf(stderr, "llmcp-run: --token-ids wants comma-separated integers\n");
        return 1;
      }
      tokens.push_back(id);
    }
  } else {
    tokens.push_back(token);
  }
  if (tokenize_only) {
    for (size_t i = 0; i < tokens.size(); ++i)
      std::printf("%s%lld", i ? "," : "", static_cast<long long>(tokens[i]));
    std::printf("\n");
    return expect_token >= 0 && (tokens.empty() || tokens[0] != expect_token) ? 1 : 0;
  }
  if (tokens.empty()) {
    std::fprintf(stderr, "llmcp-run: the prompt has no tokens\n");
    return 1;
  }
  if (aot.empty()) {
    std::fprintf(stderr, "llmcp-run: --aot is required (the interpreter half is not part of this build)\n");
    return 1;
  }

  Runtime runtime;
  if (synthetic && access(weights.c_str(), R_OK) != 0) {
    const uint64_t bytes = synthetic_container_bytes(runtime.dims, nullptr);
    std::vector<uint8_t> file(bytes);
    const std::string error = fill_synthetic_container(runtime.dims, seed, file.data(), bytes);
    FILE *out = error.empty() ? std::fopen(weights.c_str(), "wb") : nullptr;
    if (!out || std::fwrite(file.data(), 1, bytes, out) != bytes) {
      std::fprintf(stderr, "llmcp-run: cannot write %s %s\n", weights.c_str(), error.c_str());
      return 1;
    }
    std::fclose(out);
  }
  Arena arena;
  if (const std::string error = arena.load(weights); !error.empty()) {
    std::fprintf(stderr, "llmcp-run: %s\n", error.c_str());
    return 1;
  }
  const int64_t prompt_tokens = static_cast<int64_t>(tokens.size());
  if (!runtime.init(aot, prompt_tokens + max_new_tokens + 16))
    return 1;
  std::vector<float> logits;
  if (!runtime.forward(arena, tokens, 0, prompt_tokens, logits))
    return 1;
  std::vector<int64_t> generated;
  ByteLevelStreamingDecoder decoder(vocab);
  auto emit = [&](const std::string &chunk) {
    std::fwrite(chunk.data(), 1, chunk.size(), stdout);
    std::fflush(stdout);
  };
  if (max_new_tokens > 0)
    emit("output: ");
  for (int64_t i = 0; i < max_new_tokens; ++i) {
    const int64_t next = argmax(logits);
    if (next == eos)
      break;
    generated.push_back(next);
    if (have_vocab)
      emit(decoder.append(static_cast<int32_t>(next)));
    const int64_t position = prompt_tokens + static_cast<int64_t>(generated.size()) - 1;
    if (!runtime.forward(arena, {next}, position, position + 1, logits))
      return 1;
  }
  if (have_vocab)
    emit(decoder.finish());
  if (!generated.empty()) {
    std::printf("\ntokens:");
    for (int64_t id : generated)
      std::printf(" %lld", static_cast<long long>(id));
    std::printf("\n");
  } else {
    std::printf("aot logits: %zu next %lld\n", logits.size(), static_cast<long long>(argmax(logits)));
  }
  if (dump_logits)
    for (float v : logits)
      std::printf("%g\n", v);
  return 0;
}
