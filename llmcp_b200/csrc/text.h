// Token ids -> text for the interactive driver: the ByteLevel decoding that the reference gets from
// its tokenizer dependency (tokenizers-cpp, a wrapper of the HuggingFace `tokenizers` crate, pinned
// as the submodule third_party/tokenizers-cpp and absent from the reference tree), restated from
// the published algorithm, the streaming decoder of tools/llmcp-run/StreamingDecoder.{h,cpp} and
// the chat template of tools/llmcp-run/llmcp-run.cpp:608-624.  Host-only C++.
//
// What is not here: text -> ids (the BPE merges and the Unicode-class pre-tokeniser regex);
// prompts reach the driver as ids.
#pragma once

#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

namespace llmcp_b200 {

// Bytes -> UTF-8 text with every maximal ill-formed subsequence replaced by U+FFFD (the lossy
// conversion the ByteLevel decoder ends with).
std::string utf8_lossy(const std::string &bytes);

class ByteLevelVocab {
public:
  // json: either a tokenizer.json (model.vocab, added_tokens) or a bare {"token": id, ...} object
  // (what the reference's tests hand to Tokenizer::FromBlobByteLevelBPE).  Returns an error text or "".
  std::string load(const char *json, size_t bytes);

  int64_t size() const { return static_cast<int64_t>(tokens_.size()); }
  // -1 when the text is no token.
  int32_t token_to_id(const std::string &token) const;
  // Decode of the tokenizer: ids without a token are skipped, each token's characters are mapped
  // back to bytes through the GPT-2 byte alphabet (a token with a character outside it contributes
  // its own UTF-8 bytes), then the lossy conversion over all bytes together.
  std::string decode(const int32_t *ids, size_t count) const;

private:
  std::vector<std::string> tokens_; // id -> token text ("" + present_[id] == 0: no such id)
  std::vector<uint8_t> present_;
  std::unordered_map<std::string, int32_t> ids_;
};

// tools/llmcp-run/StreamingDecoder.cpp:13-29: text is held back while the decoded tail is U+FFFD
// (the bytes of a character may be completed by the next token).
class ByteLevelStreamingDecoder {
public:
  explicit ByteLevelStreamingDecoder(const ByteLevelVocab &vocab) : vocab_(vocab) {}
  std::string append(int32_t token);
  std::string finish();

private:
  const ByteLevelVocab &vocab_;
  std::vector<int32_t> pending_;
};

// tools/llmcp-run/llmcp-run.cpp:608-624.
std::string make_chat_prompt(const std::string &user, const std::string &system, bool thinking);

} // namespace llmcp_b200
