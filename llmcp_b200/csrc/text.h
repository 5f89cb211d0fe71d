// Text <-> token ids for the interactive driver: the ByteLevel decoding that the reference gets from
// its tokenizer dependency (tokenizers-cpp, a wrapper of the HuggingFace `tokenizers` crate, pinned
// as the submodule third_party/tokenizers-cpp and absent from the reference tree), restated from
// the published algorithm, the streaming decoder of tools/llmcp-run/StreamingDecoder.{h,cpp} and
// the chat template of tools/llmcp-run/llmcp-run.cpp:608-624.  Host-only C++.
//
// Text -> ids (Tokenizer::Encode) is restated for byte-level BPE tokenizers: added tokens are cut out
// first; where the tokenizer normalises to NFC, the text between them is normalised (UAX #15 on
// generated tables that hold what that library's own normaliser knows); the pre_tokenizer's Split
// steps and ByteLevel's own pattern run on the matcher of text_regex.h (the Qwen pattern on a
// hand-written scanner over the same character classes); then the ByteLevel alphabet and the
// byte-pair merges by rank.  A tokenizer.json with any other pre-tokeniser step, a pattern outside
// the matcher's subset, another normaliser or an added-token matching option loads for decoding
// and refuses to encode, with the reason.
#pragma once

#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

#include "text_regex.h"

namespace llmcp_b200 {

namespace detail {
struct Json;
}

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

  // Encode of the tokenizer (no special tokens are added around the text).  Needs a tokenizer.json
  // with merges and the supported pre-tokeniser; returns an error text or "".
  std::string encode(const std::string &text, std::vector<int32_t> *ids) const;
  bool can_encode() const { return encoder_ready_; }
  const std::string &encode_refusal() const { return encode_refusal_; }

private:
  // One splitting step of the pre_tokenizer (a Split, or the pattern ByteLevel applies itself).
  struct PreStep {
    detail::Regex regex;
    detail::SplitBehavior behavior = detail::SplitBehavior::kIsolated;
    bool invert = false;
    bool scanner = false; // the Qwen pattern, isolated: pretokenize() below does the same without backtracking
  };
  std::string parse_pre_tokenizer(const detail::Json *pre); // "" or why encode() will refuse
  std::string split_pieces(const std::string &segment, std::vector<std::string> *pieces) const;
  void encode_piece(const std::string &piece, std::vector<int32_t> *ids) const;

  std::vector<PreStep> steps_;
  bool prefix_space_ = false; // ByteLevel's add_prefix_space

  std::vector<std::string> tokens_; // id -> token text ("" + present_[id] == 0: no such id)
  std::vector<uint8_t> present_;
  std::unordered_map<std::string, int32_t> ids_;
  struct Merge {
    int32_t rank, id; // position in the merges list; id of the joined token
  };
  static uint64_t pair_key(int32_t left, int32_t right) {
    return (static_cast<uint64_t>(static_cast<uint32_t>(left)) << 32) | static_cast<uint32_t>(right);
  }
  std::unordered_map<uint64_t, Merge> merge_rank_; // (left id, right id) -> merge
  std::vector<std::string> added_;                       // added tokens, longest first
  bool ignore_merges_ = false;
  bool encoder_ready_ = false;
  bool nfc_ = false;           // the tokenizer normalises to NFC: encode() normalises what lies between added tokens
  bool added_normalized_ = false; // an added token with normalized = true (matched after normalisation)
  bool added_options_ = false; // an added token with lstrip / rstrip / single_word: not restated, encode() refuses
  std::string encode_refusal_ = "the tokenizer has no merges";
};

// Unicode Normalization Form C of a UTF-8 text (canonical decomposition, canonical ordering,
// canonical composition; Hangul by arithmetic), with the tokenizer library's view of which code
// points combine or decompose.
std::string normalize_nfc(const std::string &text);

// The pieces the pre-tokenisation pattern
//   (?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+
// cuts a text into (byte ranges, in order; ill-formed bytes count as one character each).
std::vector<std::string> pretokenize(const std::string &text);

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
