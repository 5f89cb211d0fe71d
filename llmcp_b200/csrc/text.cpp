#include "text.h"

#include "json.h"

namespace llmcp_b200 {

namespace {

// Code point -> byte of the GPT-2 byte alphabet: printable Latin-1 bytes stand for themselves, the
// other 68 bytes are numbered from U+0100 in byte order.  -1: not in the alphabet.
struct ByteAlphabet {
  int16_t byte_of[512];
  ByteAlphabet() {
    for (int i = 0; i < 512; ++i)
      byte_of[i] = -1;
    int next = 256;
    for (int byte = 0; byte < 256; ++byte) {
      const bool direct = (byte >= 33 && byte <= 126) || (byte >= 161 && byte <= 172) || byte >= 174;
      byte_of[direct ? byte : next++] = static_cast<int16_t>(byte);
    }
  }
};

const ByteAlphabet &alphabet() {
  static const ByteAlphabet table;
  return table;
}

// Length of the well-formed UTF-8 sequence at p (0 if ill-formed); *valid_prefix: how many bytes
// form the maximal prefix of a well-formed sequence (at least 1).  Unicode Table 3-7.
int well_formed(const unsigned char *p, size_t left, int *valid_prefix) {
  const unsigned char b0 = p[0];
  *valid_prefix = 1;
  if (b0 < 0x80)
    return 1;
  int length;
  unsigned char lo = 0x80, hi = 0xbf;
  if (b0 >= 0xc2 && b0 <= 0xdf) {
    length = 2;
  } else if (b0 >= 0xe0 && b0 <= 0xef) {
    length = 3;
    if (b0 == 0xe0)
      lo = 0xa0;
    if (b0 == 0xed)
      hi = 0x9f;
  } else if (b0 >= 0xf0 && b0 <= 0xf4) {
    length = 4;
    if (b0 == 0xf0)
      lo = 0x90;
    if (b0 == 0xf4)
      hi = 0x8f;
  } else {
    return 0;
  }
  for (int i = 1; i < length; ++i) {
    if (static_cast<size_t>(i) >= left)
      return 0;
    const unsigned char b = p[i];
    const unsigned char low = i == 1 ? lo : 0x80, high = i == 1 ? hi : 0xbf;
    if (b < low || b > high)
      return 0;
    *valid_prefix = i + 1;
  }
  return length;
}

} // namespace

std::string utf8_lossy(const std::string &bytes) {
  std::string out;
  out.reserve(bytes.size());
  const unsigned char *p = reinterpret_cast<const unsigned char *>(bytes.data());
  size_t i = 0;
  while (i < bytes.size()) {
    int prefix = 1;
    const int length = well_formed(p + i, bytes.size() - i, &prefix);
    if (length > 0) {
      out.append(bytes, i, static_cast<size_t>(length));
      i += static_cast<size_t>(length);
    } else {
      out += "\xef\xbf\xbd";
      i += static_cast<size_t>(prefix);
    }
  }
  return out;
}

std::string ByteLevelVocab::load(const char *json, size_t bytes) {
  detail::JsonReader reader{json, json + bytes};
  const detail::Json root = reader.value();
  if (!reader.ok || root.kind != detail::Json::Object)
    return "tokenizer: not a JSON object";
  const detail::Json *vocab = &root;
  const detail::Json *added = nullptr;
  if (const detail::Json *model = root.get("model")) {
    vocab = model->get("vocab");
    if (!vocab || vocab->kind != detail::Json::Object)
      return "tokenizer: model.vocab is missing";
    if (const detail::Json *decoder = root.get("decoder")) {
      const detail::Json *type = decoder->get("type");
      if (type && type->kind == detail::Json::String && type->text != "ByteLevel")
        return "tokenizer: decoder type " + type->text + " is not supported (ByteLevel only)";
    }
    added = root.get("added_tokens");
  }
  tokens_.clear();
  present_.clear();
  ids_.clear();
  auto put = [&](const std::string &token, int64_t id) -> bool {
    if (id < 0 || id > (1 << 24))
      return false;
    if (static_cast<size_t>(id) >= tokens_.size()) {
      tokens_.resize(static_cast<size_t>(id) + 1);
      present_.resize(static_cast<size_t>(id) + 1, 0);
    }
    tokens_[static_cast<size_t>(id)] = token;
    present_[static_cast<size_t>(id)] = 1;
    ids_[token] = static_cast<int32_t>(id);
    return true;
  };
  for (const auto &member : vocab->members) {
    int64_t id = 0;
    if (!detail::as_integer(&member.second, &id) || !put(member.first, id))
      return "tokenizer: vocab entry '" + member.first + "' has no valid id";
  }
  if (added && added->kind == detail::Json::Array) {
    for (const detail::Json &entry : added->items) {
      int64_t id = 0;
      const detail::Json *content = entry.get("content");
      if (!detail::as_integer(entry.get("id"), &id) || !content || content->kind != detail::Json::String || !put(content->text, id))
        return "tokenizer: malformed added_tokens entry";
    }
  }
  if (tokens_.empty())
    return "tokenizer: empty vocabulary";
  return "";
}

int32_t ByteLevelVocab::token_to_id(const std::string &token) const {
  const auto it = ids_.find(token);
  return it == ids_.end() ? -1 : it->second;
}

std::string ByteLevelVocab::decode(const int32_t *ids, size_t count) const {
  std::string bytes;
  const ByteAlphabet &table = alphabet();
  for (size_t n = 0; n < count; ++n) {
    const int32_t id = ids[n];
    if (id < 0 || static_cast<size_t>(id) >= tokens_.size() || !present_[static_cast<size_t>(id)])
      continue;
    const std::string &token = tokens_[static_cast<size_t>(id)];
    // every character through the alphabet, or the token's own bytes if one of them is outside it
    std::string mapped;
    bool inside = true;
    const unsigned char *p = reinterpret_cast<const unsigned char *>(token.data());
    for (size_t i = 0; i < token.size() && inside;) {
      int prefix = 1;
      const int length = well_formed(p + i, token.size() - i, &prefix);
      uint32_t code = 0;
      if (length == 1)
        code = p[i];
      else if (length == 2)
        code = (static_cast<uint32_t>(p[i] & 0x1f) << 6) | (p[i + 1] & 0x3f);
      else
        inside = false;
      if (inside && code < 512 && table.byte_of[code] >= 0)
        mapped += static_cast<char>(table.byte_of[code]);
      else
        inside = false;
      i += static_cast<size_t>(length > 0 ? length : prefix);
    }
    bytes += inside ? mapped : token;
  }
  return utf8_lossy(bytes);
}

std::string ByteLevelStreamingDecoder::append(int32_t token) {
  pending_.push_back(token);
  std::string text = vocab_.decode(pending_.data(), pending_.size());
  if (text.size() >= 3 && text.compare(text.size() - 3, 3, "\xef\xbf\xbd") == 0)
    return {};
  pending_.clear();
  return text;
}

std::string ByteLevelStreamingDecoder::finish() {
  if (pending_.empty())
    return {};
  std::string text = vocab_.decode(pending_.data(), pending_.size());
  pending_.clear();
  return text;
}

std::string make_chat_prompt(const std::string &user, const std::string &system, bool thinking) {
  std::string prompt;
  if (!system.empty())
    prompt += "<|im_start|>system\n" + system + "<|im_end|>\n";
  prompt += "<|im_start|>user\n" + user + "<|im_end|>\n<|im_start|>assistant\n";
  prompt += thinking ? "<think>\n" : "<think>\n\n</think>\n\n";
  return prompt;
}

} // namespace llmcp_b200
