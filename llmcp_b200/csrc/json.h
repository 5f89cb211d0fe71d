// A small JSON reader for the container manifest, config.json and safetensors headers:
// objects, arrays, strings, numbers, true/false/null.  Internal to the host-side format code.
#pragma once

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <string>
#include <utility>
#include <vector>

namespace llmcp_b200 {
namespace detail {

struct Json {
  enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
  bool boolean = false;
  double number = 0;
  bool integral = false;
  int64_t integer = 0;
  std::string text;
  std::vector<Json> items;
  std::vector<std::pair<std::string, Json>> members;

  const Json *get(const char *key) const {
    for (const auto &m : members)
      if (m.first == key)
        return &m.second;
    return nullptr;
  }
};

struct JsonReader {
  const char *p, *end;
  bool ok = true;

  void skip() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r'))
      ++p;
  }
  bool eat(char c) {
    skip();
    if (p < end && *p == c) {
      ++p;
      return true;
    }
    return false;
  }
  std::string string() {
    std::string out;
    if (!eat('"')) {
      ok = false;
      return out;
    }
    while (p < end && *p != '"') {
      if (*p == '\\' && p + 1 < end) {
        ++p;
        switch (*p) {
        case 'n': out += '\n'; break;
        case 't': out += '\t'; break;
        case 'r': out += '\r'; break;
        case 'b': out += '\b'; break;
        case 'f': out += '\f'; break;
        case 'u': {
          // \uXXXX, a surrogate pair included, as UTF-8
          auto hex4 = [&](const char *q, unsigned *code) {
            *code = 0;
            for (int i = 0; i < 4; ++i) {
              const char c = q[i];
              const int digit = c >= '0' && c <= '9' ? c - '0' : (c | 32) >= 'a' && (c | 32) <= 'f' ? (c | 32) - 'a' + 10 : -1;
              if (digit < 0)
                return false;
              *code = *code * 16 + static_cast<unsigned>(digit);
            }
            return true;
          };
          unsigned code = 0;
          if (p + 4 >= end || !hex4(p + 1, &code)) {
            ok = false;
            break;
          }
          p += 4;
          if (code >= 0xd800 && code <= 0xdbff && p + 6 < end && p[1] == '\\' && p[2] == 'u') {
            unsigned low = 0;
            if (hex4(p + 3, &low) && low >= 0xdc00 && low <= 0xdfff) {
              code = 0x10000 + ((code - 0xd800) << 10) + (low - 0xdc00);
              p += 6;
            }
          }
          if (code < 0x80) {
            out += static_cast<char>(code);
          } else if (code < 0x800) {
            out += static_cast<char>(0xc0 | (code >> 6));
            out += static_cast<char>(0x80 | (code & 0x3f));
          } else if (code < 0x10000) {
            out += static_cast<char>(0xe0 | (code >> 12));
            out += static_cast<char>(0x80 | ((code >> 6) & 0x3f));
            out += static_cast<char>(0x80 | (code & 0x3f));
          } else {
            out += static_cast<char>(0xf0 | (code >> 18));
            out += static_cast<char>(0x80 | ((code >> 12) & 0x3f));
            out += static_cast<char>(0x80 | ((code >> 6) & 0x3f));
            out += static_cast<char>(0x80 | (code & 0x3f));
          }
          break;
        }
        default: out += *p;
        }
        ++p;
      } else {
        out += *p++;
      }
    }
    if (p >= end)
      ok = false;
    else
      ++p;
    return out;
  }
  Json value(int depth = 0) {
    Json v;
    skip();
    if (p >= end || depth > 32) {
      ok = false;
      return v;
    }
    if (*p == '{') {
      ++p;
      v.kind = Json::Object;
      if (eat('}'))
        return v;
      do {
        std::string key = string();
        if (!ok || !eat(':')) {
          ok = false;
          return v;
        }
        v.members.emplace_back(std::move(key), value(depth + 1));
      } while (ok && eat(','));
      if (!eat('}'))
        ok = false;
    } else if (*p == '[') {
      ++p;
      v.kind = Json::Array;
      if (eat(']'))
        return v;
      do {
        v.items.push_back(value(depth + 1));
      } while (ok && eat(','));
      if (!eat(']'))
        ok = false;
    } else if (*p == '"') {
      v.kind = Json::String;
      v.text = string();
    } else if (end - p >= 4 && !std::strncmp(p, "true", 4)) {
      v.kind = Json::Bool;
      v.boolean = true;
      p += 4;
    } else if (end - p >= 5 && !std::strncmp(p, "false", 5)) {
      v.kind = Json::Bool;
      p += 5;
    } else if (end - p >= 4 && !std::strncmp(p, "null", 4)) {
      p += 4;
    } else {
      const char *start = p;
      bool integral = true;
      if (p < end && (*p == '-' || *p == '+'))
        ++p;
      while (p < end && ((*p >= '0' && *p <= '9') || *p == '.' || *p == 'e' || *p == 'E' || *p == '-' || *p == '+')) {
        if (*p == '.' || *p == 'e' || *p == 'E')
          integral = false;
        ++p;
      }
      if (p == start) {
        ok = false;
        return v;
      }
      std::string text(start, p);
      v.kind = Json::Number;
      v.number = std::strtod(text.c_str(), nullptr);
      v.integral = integral && text.size() < 19;
      if (v.integral)
        v.integer = std::strtoll(text.c_str(), nullptr, 10);
    }
    return v;
  }
};

inline bool as_integer(const Json *j, int64_t *out) {
  if (!j || j->kind != Json::Number || !j->integral)
    return false;
  *out = j->integer;
  return true;
}

inline void append_escaped(std::string &out, const std::string &s) {
  out += '"';
  for (char c : s) {
    if (c == '"' || c == '\\') {
      out += '\\';
      out += c;
    } else if (c == '\n') {
      out += "\\n";
    } else {
      out += c;
    }
  }
  out += '"';
}

} // namespace detail
} // namespace llmcp_b200
