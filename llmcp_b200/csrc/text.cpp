#include "text.h"

#include <algorithm>
#include <climits>
#include <functional>
#include <queue>
#include <cstddef>
#include <cstdio>

#include "json.h"
#include "unicode_tables.h"

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

bool in_ranges(const detail::CodeRange *ranges, size_t count, uint32_t cp) {
  size_t lo = 0, hi = count;
  while (lo < hi) {
    const size_t mid = (lo + hi) / 2;
    if (cp > ranges[mid].last)
      lo = mid + 1;
    else if (cp < ranges[mid].first)
      hi = mid;
    else
      return true;
  }
  return false;
}
bool is_letter(uint32_t cp) { return in_ranges(detail::kLetterRanges, sizeof(detail::kLetterRanges) / sizeof(detail::CodeRange), cp); }
bool is_number(uint32_t cp) { return in_ranges(detail::kNumberRanges, sizeof(detail::kNumberRanges) / sizeof(detail::CodeRange), cp); }
// \s of a Unicode-aware pattern: the White_Space property.
bool is_space(uint32_t cp) {
  return (cp >= 9 && cp <= 13) || cp == 0x20 || cp == 0x85 || cp == 0xa0 || cp == 0x1680 || (cp >= 0x2000 && cp <= 0x200a) ||
         cp == 0x2028 || cp == 0x2029 || cp == 0x202f || cp == 0x205f || cp == 0x3000;
}
bool is_newline(uint32_t cp) { return cp == '\r' || cp == '\n'; }

// Code points of a text with the byte offset of each (one more offset at the end); an ill-formed
// byte stands for itself as a character outside every category.
void decode_points(const std::string &text, std::vector<uint32_t> *points, std::vector<size_t> *offsets) {
  const unsigned char *p = reinterpret_cast<const unsigned char *>(text.data());
  size_t i = 0;
  while (i < text.size()) {
    int prefix = 1;
    const int length = well_formed(p + i, text.size() - i, &prefix);
    uint32_t cp;
    if (length == 1)
      cp = p[i];
    else if (length == 2)
      cp = (static_cast<uint32_t>(p[i] & 0x1f) << 6) | (p[i + 1] & 0x3f);
    else if (length == 3)
      cp = (static_cast<uint32_t>(p[i] & 0x0f) << 12) | (static_cast<uint32_t>(p[i + 1] & 0x3f) << 6) | (p[i + 2] & 0x3f);
    else if (length == 4)
      cp = (static_cast<uint32_t>(p[i] & 0x07) << 18) | (static_cast<uint32_t>(p[i + 1] & 0x3f) << 12) |
           (static_cast<uint32_t>(p[i + 2] & 0x3f) << 6) | (p[i + 3] & 0x3f);
    else
      cp = 0xfffd;
    points->push_back(cp);
    offsets->push_back(i);
    i += static_cast<size_t>(length > 0 ? length : 1);
  }
  offsets->push_back(text.size());
}

void append_utf8(uint32_t cp, std::string *out) {
  if (cp < 0x80) {
    *out += static_cast<char>(cp);
  } else if (cp < 0x800) {
    *out += static_cast<char>(0xc0 | (cp >> 6));
    *out += static_cast<char>(0x80 | (cp & 0x3f));
  } else if (cp < 0x10000) {
    *out += static_cast<char>(0xe0 | (cp >> 12));
    *out += static_cast<char>(0x80 | ((cp >> 6) & 0x3f));
    *out += static_cast<char>(0x80 | (cp & 0x3f));
  } else {
    *out += static_cast<char>(0xf0 | (cp >> 18));
    *out += static_cast<char>(0x80 | ((cp >> 12) & 0x3f));
    *out += static_cast<char>(0x80 | ((cp >> 6) & 0x3f));
    *out += static_cast<char>(0x80 | (cp & 0x3f));
  }
}

// ---- Unicode Normalization Form C (UAX #15), on the tables of unicode_tables.h ------------------
constexpr uint32_t kHangulS = 0xac00, kHangulL = 0x1100, kHangulV = 0x1161, kHangulT = 0x11a7;
constexpr uint32_t kHangulLCount = 19, kHangulVCount = 21, kHangulTCount = 28;
constexpr uint32_t kHangulNCount = kHangulVCount * kHangulTCount, kHangulSCount = kHangulLCount * kHangulNCount;

uint32_t combining_class(uint32_t cp) {
  constexpr size_t count = sizeof(detail::kCombiningClasses) / sizeof(detail::kCombiningClasses[0]);
  const detail::CombiningClass *end = detail::kCombiningClasses + count;
  const detail::CombiningClass *it =
      std::upper_bound(detail::kCombiningClasses, end, cp, [](uint32_t v, const detail::CombiningClass &r) { return v < r.first; });
  if (it == detail::kCombiningClasses)
    return 0;
  --it;
  return cp <= it->last ? it->value : 0;
}

const detail::Decomposition *find_decomposition(uint32_t cp) {
  constexpr size_t count = sizeof(detail::kDecompositions) / sizeof(detail::kDecompositions[0]);
  const detail::Decomposition *end = detail::kDecompositions + count;
  const detail::Decomposition *it =
      std::lower_bound(detail::kDecompositions, end, cp, [](const detail::Decomposition &r, uint32_t v) { return r.point < v; });
  return it != end && it->point == cp ? it : nullptr;
}

// Full canonical decomposition of one code point, appended to out.
void decompose(uint32_t cp, std::vector<uint32_t> *out) {
  if (cp >= kHangulS && cp < kHangulS + kHangulSCount) {
    const uint32_t s = cp - kHangulS;
    out->push_back(kHangulL + s / kHangulNCount);
    out->push_back(kHangulV + (s % kHangulNCount) / kHangulTCount);
    if (s % kHangulTCount)
      out->push_back(kHangulT + s % kHangulTCount);
    return;
  }
  const detail::Decomposition *d = cp < 0xc0 ? nullptr : find_decomposition(cp);
  if (!d) {
    out->push_back(cp);
    return;
  }
  decompose(d->first, out);
  if (d->second)
    decompose(d->second, out);
}

// The primary composite of a pair, or 0.
uint32_t compose(uint32_t a, uint32_t b) {
  if (a >= kHangulL && a < kHangulL + kHangulLCount && b >= kHangulV && b < kHangulV + kHangulVCount)
    return kHangulS + ((a - kHangulL) * kHangulVCount + (b - kHangulV)) * kHangulTCount;
  if (a >= kHangulS && a < kHangulS + kHangulSCount && (a - kHangulS) % kHangulTCount == 0 && b > kHangulT && b < kHangulT + kHangulTCount)
    return a + (b - kHangulT);
  static const std::unordered_map<uint64_t, uint32_t> pairs = [] {
    std::unordered_map<uint64_t, uint32_t> map;
    for (const detail::Decomposition &d : detail::kDecompositions)
      if (d.composes)
        map.emplace((static_cast<uint64_t>(d.first) << 32) | d.second, d.point);
    return map;
  }();
  const auto it = pairs.find((static_cast<uint64_t>(a) << 32) | b);
  return it == pairs.end() ? 0 : it->second;
}

// Byte -> the UTF-8 text of its character in the GPT-2 byte alphabet.
struct ByteText {
  std::string text[256];
  ByteText() {
    int next = 256;
    for (int byte = 0; byte < 256; ++byte) {
      const bool direct = (byte >= 33 && byte <= 126) || (byte >= 161 && byte <= 172) || byte >= 174;
      const int cp = direct ? byte : next++;
      if (cp < 128) {
        text[byte] = std::string(1, static_cast<char>(cp));
      } else {
        text[byte] += static_cast<char>(0xc0 | (cp >> 6));
        text[byte] += static_cast<char>(0x80 | (cp & 0x3f));
      }
    }
  }
};
const ByteText &byte_text() {
  static const ByteText table;
  return table;
}

const char *const kSupportedPattern =
    "(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\\r\\n\\p{L}\\p{N}]?\\p{L}+|\\p{N}| ?[^\\s\\p{L}\\p{N}]+[\\r\\n]*|\\s*[\\r\\n]+|\\s+(?!\\S)|\\s+";

} // namespace

namespace detail {
void utf8_points(const std::string &text, std::vector<uint32_t> *points, std::vector<size_t> *offsets) {
  decode_points(text, points, offsets);
}
} // namespace detail

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
  // text -> ids: merges by rank, added tokens, and the one pre-tokeniser this code restates
  merge_rank_.clear();
  added_.clear();
  encoder_ready_ = nfc_ = added_options_ = added_normalized_ = ignore_merges_ = false;
  encode_refusal_ = "the tokenizer has no merges";
  const detail::Json *model = root.get("model");
  const detail::Json *merges = model ? model->get("merges") : nullptr;
  if (merges && merges->kind == detail::Json::Array) {
    int32_t rank = 0;
    bool outside = false;
    for (const detail::Json &m : merges->items) {
      std::string left, right;
      if (m.kind == detail::Json::String && m.text.find(' ') != std::string::npos) {
        left = m.text.substr(0, m.text.find(' '));
        right = m.text.substr(m.text.find(' ') + 1);
      } else if (m.kind == detail::Json::Array && m.items.size() == 2 && m.items[0].kind == detail::Json::String &&
                 m.items[1].kind == detail::Json::String) {
        left = m.items[0].text;
        right = m.items[1].text;
      } else {
        return "tokenizer: malformed merges entry";
      }
      const auto a = ids_.find(left), b = ids_.find(right), joined = ids_.find(left + right);
      if (a == ids_.end() || b == ids_.end() || joined == ids_.end())
        outside = true;
      else
        merge_rank_.emplace(pair_key(a->second, b->second), Merge{rank, joined->second});
      ++rank;
    }
    if (const detail::Json *flag = model->get("ignore_merges"))
      ignore_merges_ = flag->kind == detail::Json::Bool && flag->boolean;
    if (added && added->kind == detail::Json::Array)
      for (const detail::Json &entry : added->items) {
        if (!entry.get("content")->text.empty())
          added_.push_back(entry.get("content")->text);
        if (const detail::Json *flag = entry.get("normalized"))
          if (flag->kind == detail::Json::Bool && flag->boolean)
            added_normalized_ = true;
        for (const char *option : {"lstrip", "rstrip", "single_word"})
          if (const detail::Json *flag = entry.get(option))
            if (flag->kind == detail::Json::Bool && flag->boolean)
              added_options_ = true;
      }
    std::sort(added_.begin(), added_.end(), [](const std::string &a, const std::string &b) { return a.size() > b.size(); });
    // pre_tokenizer: ByteLevel, or a Sequence of Split steps that ends in ByteLevel
    steps_.clear();
    prefix_space_ = false;
    encode_refusal_ = parse_pre_tokenizer(root.get("pre_tokenizer"));
    encoder_ready_ = encode_refusal_.empty();
    if (encoder_ready_ && outside) {
      encoder_ready_ = false;
      encode_refusal_ = "a merge names a token outside the vocabulary";
    }
    if (encoder_ready_) { // model options that change what Encode returns
      auto refuse = [&](const char *why) {
        encoder_ready_ = false;
        encode_refusal_ = why;
      };
      const detail::Json *kind = model->get("type"), *dropout = model->get("dropout"), *fallback = model->get("byte_fallback");
      const detail::Json *prefix = model->get("continuing_subword_prefix"), *suffix = model->get("end_of_word_suffix");
      if (kind && kind->kind == detail::Json::String && kind->text != "BPE")
        refuse("its model is not BPE");
      else if (dropout && dropout->kind == detail::Json::Number && dropout->number > 0)
        refuse("its model drops merges at random (dropout)");
      else if (fallback && fallback->kind == detail::Json::Bool && fallback->boolean)
        refuse("its model falls back to byte tokens (byte_fallback)");
      else if ((prefix && !prefix->text.empty()) || (suffix && !suffix->text.empty()))
        refuse("its model has a subword prefix or an end-of-word suffix");
      else
        for (int byte = 0; byte < 256; ++byte)
          if (ids_.find(byte_text().text[byte]) == ids_.end()) {
            refuse("its vocabulary lacks a symbol of the byte alphabet");
            break;
          }
    }
    if (encoder_ready_ && added_options_) {
      encoder_ready_ = false;
      encode_refusal_ = "an added token asks for lstrip, rstrip or single_word matching";
    }
    if (encoder_ready_)
      if (const detail::Json *normalizer = root.get("normalizer"))
        if (normalizer->kind == detail::Json::Object) {
          const detail::Json *type = normalizer->get("type");
          const detail::Json *members = normalizer->get("normalizers");
          if (type && type->text == "Sequence" && members && members->kind == detail::Json::Array && members->items.size() == 1)
            type = members->items[0].get("type"); // a Sequence of one normaliser is that normaliser
          if (type && type->text == "NFC" && !added_normalized_) {
            nfc_ = true;
          } else if (type && type->text == "NFC") {
            encoder_ready_ = false;
            encode_refusal_ = "an added token is matched in normalised text (normalized = true) under the NFC normaliser";
          } else {
            encoder_ready_ = false;
            encode_refusal_ = "its normalizer is neither absent nor NFC";
          }
        }
  }
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

// The pre-tokenisation pattern the ByteLevel pre-tokeniser applies when it is asked to (use_regex).
static const char *const kByteLevelPattern =
    "'s|'t|'re|'ve|'m|'ll|'d| ?\\p{L}+| ?\\p{N}+| ?[^\\s\\p{L}\\p{N}]+|\\s+(?!\\S)|\\s+";

std::string ByteLevelVocab::parse_pre_tokenizer(const detail::Json *pre) {
  if (!pre || pre->kind != detail::Json::Object)
    return "it has no pre_tokenizer (a byte-level vocabulary needs the ByteLevel step)";
  std::vector<const detail::Json *> list;
  const detail::Json *type = pre->get("type");
  if (type && type->text == "Sequence") {
    const detail::Json *items = pre->get("pretokenizers");
    if (!items || items->kind != detail::Json::Array)
      return "its pre_tokenizer Sequence has no list";
    for (const detail::Json &item : items->items)
      list.push_back(&item);
  } else {
    list.push_back(pre);
  }
  bool byte_level = false;
  for (size_t i = 0; i < list.size(); ++i) {
    const detail::Json *kind = list[i]->get("type");
    const std::string name = kind ? kind->text : "";
    if (byte_level)
      return "its pre_tokenizer has a step behind ByteLevel";
    PreStep step;
    std::string pattern;
    if (name == "Split") {
      const detail::Json *p = list[i]->get("pattern");
      const detail::Json *regex = p ? p->get("Regex") : nullptr, *literal = p ? p->get("String") : nullptr;
      if (regex && regex->kind == detail::Json::String) {
        pattern = regex->text;
      } else if (literal && literal->kind == detail::Json::String && !literal->text.empty()) {
        for (unsigned char c : literal->text) { // the literal as a pattern: punctuation escaped
          if (c < 0x80 && !((c >= '0' && c <= '9') || (c >= 'a' && c <= 'z') || (c >= 'A' && c <= 'Z') || c == ' '))
            pattern += '\\';
          pattern += static_cast<char>(c);
        }
      } else {
        return "a Split step of its pre_tokenizer has neither a Regex nor a String pattern";
      }
      const detail::Json *behavior = list[i]->get("behavior"), *invert = list[i]->get("invert");
      if (const std::string error = detail::parse_split_behavior(behavior ? behavior->text : "", &step.behavior); !error.empty())
        return "a Split step of its pre_tokenizer: " + error;
      step.invert = invert && invert->kind == detail::Json::Bool && invert->boolean;
    } else if (name == "ByteLevel") {
      byte_level = true;
      const detail::Json *use_regex = list[i]->get("use_regex"), *prefix = list[i]->get("add_prefix_space");
      if (prefix && prefix->kind == detail::Json::Bool && prefix->boolean) {
        if (i != 0)
          return "its ByteLevel step adds a prefix space behind other steps";
        prefix_space_ = true;
      }
      if (use_regex && use_regex->kind == detail::Json::Bool && !use_regex->boolean)
        continue; // only the byte mapping
      pattern = kByteLevelPattern;
      step.behavior = detail::SplitBehavior::kIsolated;
    } else {
      return "its pre_tokenizer has a step of type '" + name + "' (Split and ByteLevel are restated)";
    }
    step.scanner = pattern == kSupportedPattern && step.behavior == detail::SplitBehavior::kIsolated && !step.invert;
    if (const std::string error = step.regex.compile(pattern); !error.empty())
      return "a pattern of its pre_tokenizer is outside what is restated: " + error;
    steps_.push_back(std::move(step));
  }
  if (!byte_level)
    return "its pre_tokenizer does not end in ByteLevel";
  return "";
}

std::string ByteLevelVocab::split_pieces(const std::string &segment, std::vector<std::string> *pieces) const {
  std::vector<std::string> current;
  if (!segment.empty())
    current.push_back(prefix_space_ && segment[0] != ' ' ? " " + segment : segment);
  for (const PreStep &step : steps_) {
    std::vector<std::string> next;
    for (const std::string &piece : current) {
      if (step.scanner) {
        for (std::string &part : pretokenize(piece))
          next.push_back(std::move(part));
      } else if (const std::string error = detail::regex_split(step.regex, piece, step.behavior, step.invert, &next); !error.empty()) {
        return "tokenizer: cannot encode text: " + error;
      }
    }
    current.swap(next);
  }
  pieces->swap(current);
  return "";
}

std::string normalize_nfc(const std::string &text) {
  bool ascii = true;
  for (unsigned char c : text)
    ascii = ascii && c < 0x80;
  if (ascii)
    return text;
  std::vector<uint32_t> points, parts;
  std::vector<size_t> offsets;
  decode_points(text, &points, &offsets);
  for (uint32_t cp : points)
    decompose(cp, &parts);
  // canonical ordering: marks of a run between starters, by class, order among equals kept
  std::vector<uint32_t> classes(parts.size());
  for (size_t i = 0; i < parts.size(); ++i)
    classes[i] = combining_class(parts[i]);
  for (size_t i = 1; i < parts.size(); ++i)
    for (size_t j = i; j > 0 && classes[j] != 0 && classes[j - 1] > classes[j]; --j) {
      std::swap(parts[j], parts[j - 1]);
      std::swap(classes[j], classes[j - 1]);
    }
  // canonical composition: a character joins the last starter unless something between them has
  // its class or a higher one (or is a starter itself)
  std::vector<uint32_t> out;
  size_t starter = SIZE_MAX;
  int64_t between = -1; // class of the last character kept after the starter; -1: none
  for (size_t i = 0; i < parts.size(); ++i) {
    const int64_t cc = classes[i];
    if (starter != SIZE_MAX && (between < 0 || between < cc)) {
      if (const uint32_t joined = compose(out[starter], parts[i])) {
        out[starter] = joined;
        continue;
      }
    }
    if (cc == 0) {
      starter = out.size();
      between = -1;
    } else {
      between = cc;
    }
    out.push_back(parts[i]);
  }
  std::string result;
  for (uint32_t cp : out)
    append_utf8(cp, &result);
  return result;
}

std::vector<std::string> pretokenize(const std::string &text) {
  std::vector<uint32_t> cp;
  std::vector<size_t> at;
  decode_points(text, &cp, &at);
  const size_t n = cp.size();
  std::vector<std::string> pieces;
  auto fold = [](uint32_t c) { return c == 0x17f ? uint32_t('s') : c == 0x212a ? uint32_t('k') : (c >= 'A' && c <= 'Z') ? c + 32 : c; };
  auto punct = [](uint32_t c) { return !is_space(c) && !is_letter(c) && !is_number(c); };
  size_t p = 0;
  while (p < n) {
    size_t end = 0;
    // 1. contractions, case-insensitive, in the pattern's order
    if (cp[p] == '\'' && p + 1 < n) {
      const uint32_t a = fold(cp[p + 1]), b = p + 2 < n ? fold(cp[p + 2]) : 0;
      if (a == 's' || a == 't')
        end = p + 2;
      else if ((a == 'r' && b == 'e') || (a == 'v' && b == 'e'))
        end = p + 3;
      else if (a == 'm')
        end = p + 2;
      else if (a == 'l' && b == 'l')
        end = p + 3;
      else if (a == 'd')
        end = p + 2;
    }
    // 2. an optional character that is no letter, number, CR or LF, then letters
    if (!end) {
      size_t q = p;
      if (!is_letter(cp[q]) && !is_number(cp[q]) && !is_newline(cp[q]) && q + 1 < n && is_letter(cp[q + 1]))
        ++q;
      if (is_letter(cp[q])) {
        while (q < n && is_letter(cp[q]))
          ++q;
        end = q;
      }
    }
    // 3. one number character
    if (!end && is_number(cp[p]))
      end = p + 1;
    // 4. an optional space, characters that are no space, letter or number, then CRs and LFs
    if (!end) {
      size_t q = p;
      if (cp[q] == ' ' && q + 1 < n && punct(cp[q + 1]))
        ++q;
      if (punct(cp[q])) {
        while (q < n && punct(cp[q]))
          ++q;
        while (q < n && is_newline(cp[q]))
          ++q;
        end = q;
      }
    }
    if (!end && is_space(cp[p])) {
      size_t run = p;
      while (run < n && is_space(cp[run]))
        ++run;
      // 5. white space up to and including its last CR or LF
      size_t last_newline = n;
      for (size_t i = p; i < run; ++i)
        if (is_newline(cp[i]))
          last_newline = i;
      if (last_newline != n)
        end = last_newline + 1;
      else if (run == n)      // 6. white space not followed by anything else ...
        end = run;
      else if (run - p >= 2)  //    ... or all of it but the last character
        end = run - 1;
      else                    // 7. white space
        end = run;
    }
    if (!end)
      end = p + 1; // not reachable: every character is a letter, a number, white space or none of them
    pieces.emplace_back(text, at[p], at[end] - at[p]);
    p = end;
  }
  return pieces;
}

void ByteLevelVocab::encode_piece(const std::string &piece, std::vector<int32_t> *ids) const {
  const ByteText &alphabet = byte_text();
  if (ignore_merges_) {
    std::string whole;
    for (unsigned char byte : piece)
      whole += alphabet.text[byte];
    const auto it = ids_.find(whole);
    if (it != ids_.end()) {
      ids->push_back(it->second);
      return;
    }
  }
  // One symbol per byte, in a doubly linked list; candidates in a heap ordered by (rank, position):
  // the adjacent pair of lowest rank, leftmost among equals, is merged until none is left.
  struct Symbol {
    int32_t id, prev, next;
  };
  struct Candidate {
    int32_t rank, at;
    bool operator>(const Candidate &o) const { return rank != o.rank ? rank > o.rank : at > o.at; }
  };
  const int32_t n = static_cast<int32_t>(piece.size());
  std::vector<Symbol> symbols(piece.size());
  for (int32_t i = 0; i < n; ++i) {
    const auto it = ids_.find(alphabet.text[static_cast<unsigned char>(piece[static_cast<size_t>(i)])]);
    symbols[static_cast<size_t>(i)] = {it == ids_.end() ? -1 : it->second, i - 1, i + 1 < n ? i + 1 : -1};
  }
  std::priority_queue<Candidate, std::vector<Candidate>, std::greater<Candidate>> heap;
  auto offer = [&](int32_t at) {
    if (at < 0 || symbols[static_cast<size_t>(at)].next < 0)
      return;
    const Symbol &l = symbols[static_cast<size_t>(at)], &r = symbols[static_cast<size_t>(l.next)];
    if (l.id < 0 || r.id < 0)
      return;
    const auto it = merge_rank_.find(pair_key(l.id, r.id));
    if (it != merge_rank_.end())
      heap.push({it->second.rank, at});
  };
  for (int32_t i = 0; i + 1 < n; ++i)
    offer(i);
  while (!heap.empty()) {
    const Candidate top = heap.top();
    heap.pop();
    Symbol &l = symbols[static_cast<size_t>(top.at)];
    if (l.id < 0 || l.next < 0)
      continue; // the left symbol was merged away, or lost its neighbour
    Symbol &r = symbols[static_cast<size_t>(l.next)];
    const auto it = merge_rank_.find(pair_key(l.id, r.id));
    if (it == merge_rank_.end() || it->second.rank != top.rank)
      continue; // the pair at this position is no longer the one that was offered
    l.id = it->second.id;
    r.id = -2; // gone
    l.next = r.next;
    if (l.next >= 0)
      symbols[static_cast<size_t>(l.next)].prev = top.at;
    offer(l.prev);
    offer(top.at);
  }
  for (int32_t i = n ? 0 : -1; i >= 0; i = symbols[static_cast<size_t>(i)].next)
    if (symbols[static_cast<size_t>(i)].id >= 0)
      ids->push_back(symbols[static_cast<size_t>(i)].id);
}

std::string ByteLevelVocab::encode(const std::string &text, std::vector<int32_t> *ids) const {
  if (!encoder_ready_)
    return "tokenizer: cannot encode text: " + encode_refusal_;
  {
    // Ill-formed UTF-8 has no encoding (the reference hands the text to a library that takes UTF-8 only).
    std::vector<uint32_t> points;
    std::vector<size_t> offsets;
    decode_points(text, &points, &offsets);
    for (size_t i = 0; i < points.size(); ++i)
      if (points[i] == 0xfffd && offsets[i + 1] - offsets[i] == 1)
        return "tokenizer: cannot encode text: ill-formed UTF-8 at byte " + std::to_string(offsets[i]);
  }
  size_t p = 0;
  std::vector<size_t> next(added_.size(), 0); // where each added token occurs next (searched again once passed)
  std::vector<uint8_t> searched(added_.size(), 0);
  while (p < text.size()) {
    // the leftmost added token; the longest of those that start there (added_ is sorted by length)
    size_t where = std::string::npos;
    const std::string *which = nullptr;
    for (size_t t = 0; t < added_.size(); ++t) {
      if (!searched[t] || (next[t] != std::string::npos && next[t] < p)) {
        next[t] = text.find(added_[t], p);
        searched[t] = 1;
      }
      if (next[t] != std::string::npos && next[t] < where) {
        where = next[t];
        which = &added_[t];
      }
    }
    const size_t stop = which ? where : text.size();
    if (stop > p) {
      const std::string segment = text.substr(p, stop - p);
      std::vector<std::string> pieces;
      if (const std::string error = split_pieces(nfc_ ? normalize_nfc(segment) : segment, &pieces); !error.empty())
        return error;
      for (const std::string &piece : pieces)
        encode_piece(piece, ids);
    }
    if (!which)
      break;
    ids->push_back(ids_.at(*which));
    p = where + which->size();
  }
  return "";
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
