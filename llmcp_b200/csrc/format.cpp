#include "format.h"
#include "json.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <sstream>

namespace llmcp_b200 {

// ------------------------------------------------------------------------------
// scalar conversions
// ------------------------------------------------------------------------------
static uint32_t float_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}
static float bits_float(uint32_t u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

uint16_t f32_to_bf16_bits(float value) {
  uint32_t bits = float_bits(value);
  if ((bits & 0x7fffffffu) > 0x7f800000u)
    return static_cast<uint16_t>((bits >> 16) | 0x40);
  bits += 0x7fffu + ((bits >> 16) & 1u);
  return static_cast<uint16_t>(bits >> 16);
}

float bf16_bits_to_f32_host(uint16_t bits) { return bits_float(static_cast<uint32_t>(bits) << 16); }

// IEEE binary32 -> binary16, round to nearest even, with subnormals and overflow to inf.
uint16_t f32_to_f16_bits(float value) {
  const uint32_t bits = float_bits(value);
  const uint16_t sign = static_cast<uint16_t>((bits >> 16) & 0x8000u);
  const uint32_t mag = bits & 0x7fffffffu;
  if (mag >= 0x7f800000u)
    return static_cast<uint16_t>(sign | 0x7c00u | (mag > 0x7f800000u ? 0x200u : 0u));
  if (mag >= 0x477ff000u) // rounds to >= 65520 -> inf
    return static_cast<uint16_t>(sign | 0x7c00u);
  if (mag < 0x33000001u) // below half of the smallest subnormal (2^-25) or exactly it: 0
    return sign;
  int exponent = static_cast<int>(mag >> 23) - 127;
  uint32_t mantissa = (mag & 0x7fffffu) | 0x800000u; // 24 bits
  int shift;
  uint32_t base;
  if (exponent < -14) {
    shift = 13 + (-14 - exponent); // subnormal half
    base = 0;
  } else {
    shift = 13;
    base = static_cast<uint32_t>(exponent + 15) << 10;
    mantissa &= 0x7fffffu;
  }
  uint32_t kept = mantissa >> shift;
  const uint32_t rest = mantissa & ((1u << shift) - 1u);
  const uint32_t halfway = 1u << (shift - 1);
  if (rest > halfway || (rest == halfway && (kept & 1u)))
    ++kept; // a carry out of the mantissa correctly bumps the exponent
  return static_cast<uint16_t>(sign | (base + kept));
}

float f16_bits_to_f32_host(uint16_t bits) {
  const uint32_t sign = static_cast<uint32_t>(bits & 0x8000u) << 16;
  const uint32_t exponent = (bits >> 10) & 0x1fu;
  const uint32_t mantissa = bits & 0x3ffu;
  if (exponent == 0x1f)
    return bits_float(sign | 0x7f800000u | (mantissa << 13));
  if (exponent == 0) {
    if (mantissa == 0)
      return bits_float(sign);
    const float magnitude = std::ldexp(static_cast<float>(mantissa), -24);
    return (sign ? -magnitude : magnitude);
  }
  return bits_float(sign | ((exponent + 112u) << 23) | (mantissa << 13));
}

// ------------------------------------------------------------------------------
// header
// ------------------------------------------------------------------------------
static void put32(uint8_t *p, uint32_t v) {
  for (int i = 0; i < 4; ++i)
    p[i] = static_cast<uint8_t>(v >> (8 * i));
}
static void put64(uint8_t *p, uint64_t v) {
  for (int i = 0; i < 8; ++i)
    p[i] = static_cast<uint8_t>(v >> (8 * i));
}
static uint32_t get32(const uint8_t *p) {
  uint32_t v = 0;
  for (int i = 0; i < 4; ++i)
    v |= static_cast<uint32_t>(p[i]) << (8 * i);
  return v;
}
static uint64_t get64(const uint8_t *p) {
  uint64_t v = 0;
  for (int i = 0; i < 8; ++i)
    v |= static_cast<uint64_t>(p[i]) << (8 * i);
  return v;
}

void write_header(uint8_t *data, uint64_t arena_bytes, uint64_t manifest_bytes) {
  std::memset(data, 0, kHeaderBytes);
  std::memcpy(data, "LLMCPWGT", 8);
  put32(data + 8, 1);
  put32(data + 12, static_cast<uint32_t>(kHeaderBytes));
  put64(data + 16, arena_bytes);
  put64(data + 24, arena_bytes); // the manifest starts where the arena ends
  put64(data + 32, manifest_bytes);
}

std::string read_header(const uint8_t *data, uint64_t file_bytes, uint64_t *arena_bytes,
                        uint64_t *manifest_offset, uint64_t *manifest_bytes) {
  if ((file_bytes != 0 && file_bytes < kHeaderBytes) || std::memcmp(data, "LLMCPWGT", 8) != 0)
    return "invalid packed weights header";
  if (get32(data + 8) != 1 || get32(data + 12) != kHeaderBytes)
    return "unsupported packed weights format version or header size";
  *arena_bytes = get64(data + 16);
  *manifest_offset = get64(data + 24);
  *manifest_bytes = get64(data + 32);
  if (*arena_bytes < kHeaderBytes || *manifest_offset != *arena_bytes || *manifest_bytes == 0)
    return "invalid packed weights arena or manifest bounds";
  if (file_bytes != 0 &&
      (*manifest_offset > file_bytes || *manifest_bytes != file_bytes - *manifest_offset))
    return "invalid packed weights arena or manifest bounds";
  return "";
}

using namespace detail;

const TensorEntry *Manifest::find(const std::string &name) const {
  for (const auto &t : tensors)
    if (t.name == name)
      return &t;
  return nullptr;
}

std::string Manifest::to_json() const {
  // block_size and quant_layout accompany a quantised arena only (WeightPacker.cpp:126-137).
  const bool quantised = quantization != "none";
  std::string out = std::string("{\"alignment\":64,") + (quantised ? "\"block_size\":32," : "") +
                    "\"group_stride\":" + std::to_string(group_stride) +
                    ",\"header_bytes\":" + std::to_string(header_bytes) + ",\"model\":";
  append_escaped(out, model);
  out += ",\"num_groups\":" + std::to_string(num_groups) + (quantised ? ",\"quant_layout\":\"q8_0_p4\"" : "") +
         ",\"quantization\":";
  append_escaped(out, quantization);
  out += ",\"tensors\":[";
  for (size_t i = 0; i < tensors.size(); ++i) {
    const TensorEntry &t = tensors[i];
    if (i)
      out += ',';
    out += "{\"dtype\":";
    append_escaped(out, t.dtype);
    out += ",\"name\":";
    append_escaped(out, t.name);
    out += ",\"offset\":" + std::to_string(t.offset) + ",\"shape\":[";
    for (size_t d = 0; d < t.shape.size(); ++d)
      out += (d ? "," : "") + std::to_string(t.shape[d]);
    out += "],\"size\":" + std::to_string(t.size) + ",\"source_size\":" + std::to_string(t.source_size) + "}";
  }
  out += "],\"total_bytes\":" + std::to_string(total_bytes) + "}\n";
  return out;
}

std::string parse_manifest(const char *text, uint64_t length, uint64_t arena_bytes, Manifest *out) {
  JsonReader reader{text, text + length};
  Json root = reader.value();
  const std::string invalid = "invalid embedded weight manifest";
  if (!reader.ok || root.kind != Json::Object)
    return invalid;
  int64_t total = 0, header = 0;
  const Json *mode = root.get("quantization");
  const Json *tensors = root.get("tensors");
  if (!as_integer(root.get("total_bytes"), &total) || total < 0 ||
      static_cast<uint64_t>(total) != arena_bytes || !as_integer(root.get("header_bytes"), &header) ||
      header != static_cast<int64_t>(kHeaderBytes) || !mode || mode->kind != Json::String ||
      (mode->text != "none" && mode->text != "q8_0") || !tensors || tensors->kind != Json::Array ||
      tensors->items.empty())
    return invalid;
  Manifest m;
  m.total_bytes = static_cast<uint64_t>(total);
  m.quantization = mode->text;
  if (const Json *model = root.get("model"))
    m.model = model->text;
  int64_t tmp = 0;
  if (as_integer(root.get("group_stride"), &tmp))
    m.group_stride = static_cast<uint64_t>(tmp);
  if (as_integer(root.get("num_groups"), &tmp))
    m.num_groups = tmp;
  if (mode->text == "q8_0") {
    int64_t block = 0;
    const Json *layout = root.get("quant_layout");
    if (!as_integer(root.get("block_size"), &block) || block != 32 || !layout || layout->text != "q8_0_p4")
      return invalid;
  }
  std::map<std::string, bool> seen;
  for (const Json &item : tensors->items) {
    if (item.kind != Json::Object)
      return invalid;
    const Json *name = item.get("name"), *dtype = item.get("dtype"), *shape = item.get("shape");
    int64_t offset = 0, bytes = 0;
    if (!name || name->kind != Json::String || name->text.empty() || !as_integer(item.get("offset"), &offset) ||
        offset < 64 || offset % 64 != 0 || !as_integer(item.get("size"), &bytes) || bytes <= 0 || !dtype ||
        dtype->kind != Json::String || !shape || shape->kind != Json::Array || shape->items.empty())
      return invalid;
    const uint64_t begin = static_cast<uint64_t>(offset), len = static_cast<uint64_t>(bytes);
    if (begin > arena_bytes || len > arena_bytes - begin)
      return "tensor outside arena: " + name->text;
    TensorEntry entry;
    entry.name = name->text;
    entry.offset = begin;
    entry.size = len;
    entry.dtype = dtype->text;
    if (as_integer(item.get("source_size"), &tmp))
      entry.source_size = static_cast<uint64_t>(tmp);
    uint64_t elements = 1;
    for (const Json &dim : shape->items) {
      int64_t extent = 0;
      if (!as_integer(&dim, &extent) || extent <= 0 || elements > UINT64_MAX / static_cast<uint64_t>(extent))
        return invalid;
      elements *= static_cast<uint64_t>(extent);
      entry.shape.push_back(extent);
    }
    uint64_t unit;
    if (entry.dtype == "Q8_0") {
      if (mode->text != "q8_0" || entry.shape.size() != 2 || entry.shape[1] % 32 != 0)
        return invalid;
      elements /= 32;
      unit = 34;
    } else if (entry.dtype == "BF16") {
      unit = 2;
    } else if (entry.dtype == "F32") {
      unit = 4;
    } else {
      return invalid;
    }
    if (elements > UINT64_MAX / unit || elements * unit != len)
      return invalid;
    if (seen.count(entry.name))
      return invalid;
    seen[entry.name] = true;
    m.tensors.push_back(std::move(entry));
  }
  *out = std::move(m);
  return "";
}

std::string parse_container(const uint8_t *base, uint64_t file_bytes, Manifest *out) {
  uint64_t arena = 0, offset = 0, bytes = 0;
  std::string error = read_header(base, file_bytes, &arena, &offset, &bytes);
  if (!error.empty())
    return error;
  return parse_manifest(reinterpret_cast<const char *>(base + offset), bytes, arena, out);
}

// ------------------------------------------------------------------------------
// layout
// ------------------------------------------------------------------------------
namespace {

uint64_t align_up(uint64_t v) { return (v + kTensorAlignment - 1) & ~(kTensorAlignment - 1); }

struct LayoutBuilder {
  Manifest m;
  uint64_t cursor = kHeaderBytes;
  const SourceTensors *source = nullptr; // checkpoint headers, or null for the synthetic model
  bool quantize = true;
  std::string error;

  // `element_bytes` 2 = bf16 source, 4 = f32 source (used when there is no checkpoint; with
  // one, dtype and byte size come from its header and the shape must match).  2-D bf16/f32
  // tensors with rows % 8 == 0 and cols % 32 == 0 are stored as Q8_0 (WeightLayout.cpp:72-82).
  void add(const std::string &name, std::vector<int64_t> shape, int element_bytes) {
    if (!error.empty())
      return;
    TensorEntry e;
    e.name = name;
    e.offset = align_up(cursor);
    uint64_t elements = 1;
    for (int64_t d : shape)
      elements *= static_cast<uint64_t>(d);
    e.source_size = elements * element_bytes;
    e.dtype = element_bytes == 2 ? "BF16" : "F32";
    if (source) {
      auto it = source->find(name);
      if (it == source->end()) {
        error = "missing tensor '" + name + "'";
        return;
      }
      const SourceTensor &t = it->second;
      if (t.shape.size() != shape.size()) {
        error = "tensor '" + name + "' has rank " + std::to_string(t.shape.size()) + ", expected " +
                std::to_string(shape.size());
        return;
      }
      for (size_t i = 0; i < shape.size(); ++i)
        if (t.shape[i] != shape[i]) {
          error = "tensor '" + name + "' dimension " + std::to_string(i) + " is " + std::to_string(t.shape[i]) +
                  ", expected " + std::to_string(shape[i]);
          return;
        }
      e.source_size = t.data_size;
      e.dtype = t.dtype;
    }
    e.size = e.source_size;
    if (quantize && shape.size() == 2 && shape[0] > 0 && shape[1] > 0 && shape[0] % 8 == 0 && shape[1] % 32 == 0 &&
        (e.dtype == "BF16" || e.dtype == "F32")) {
      e.size = static_cast<uint64_t>(shape[0]) * (shape[1] / 32) * 34;
      e.dtype = "Q8_0";
    }
    e.shape = std::move(shape);
    cursor = e.offset + e.size;
    m.tensors.push_back(std::move(e));
  }
};

void lay_out_model(const ModelDims &c, LayoutBuilder &b);

} // namespace

Manifest build_layout(const ModelDims &c) {
  LayoutBuilder b;
  lay_out_model(c, b);
  b.m.model = "synthetic";
  return b.m;
}

std::string plan_layout(const ModelDims &c, const SourceTensors &tensors, bool q8, Manifest *out) {
  if (c.full_interval <= 0 || c.layers <= 0 || c.layers % c.full_interval != 0)
    return "num_hidden_layers must be divisible by full_attention_interval";
  LayoutBuilder b;
  b.source = &tensors;
  b.quantize = q8;
  b.m.quantization = q8 ? "q8_0" : "none";
  lay_out_model(c, b);
  if (!b.error.empty())
    return b.error;
  *out = std::move(b.m);
  return "";
}

namespace {

// Tensor order of the arena (WeightLayout.cpp:96-268): the embedding table, then per group of
// `full_interval` layers the layer tensors (every group padded to the first one's size), then
// the final norm.
void lay_out_model(const ModelDims &c, LayoutBuilder &b) {
  const std::string root = "model.language_model.";
  b.add(root + "embed_tokens.weight", {c.vocab, c.hidden}, 2);
  const int64_t groups = c.layers / c.full_interval;
  for (int64_t g = 0; g < groups; ++g) {
    const uint64_t group_start = b.cursor;
    for (int64_t i = 0; i < c.full_interval; ++i) {
      const int64_t layer = g * c.full_interval + i;
      const std::string p = root + "layers." + std::to_string(layer) + ".";
      b.add(p + "input_layernorm.weight", {c.hidden}, 2);
      b.add(p + "post_attention_layernorm.weight", {c.hidden}, 2);
      if (!c.is_full(layer)) {
        b.add(p + "linear_attn.in_proj_qkv.weight", {c.qkv_dim(), c.hidden}, 2);
        b.add(p + "linear_attn.in_proj_z.weight", {c.value_dim(), c.hidden}, 2);
        b.add(p + "linear_attn.in_proj_a.weight", {c.lin_v_heads, c.hidden}, 2);
        b.add(p + "linear_attn.in_proj_b.weight", {c.lin_v_heads, c.hidden}, 2);
        b.add(p + "linear_attn.conv1d.weight", {c.qkv_dim(), 1, c.conv_kernel}, 2);
        b.add(p + "linear_attn.dt_bias", {c.lin_v_heads}, 2);
        b.add(p + "linear_attn.A_log", {c.lin_v_heads}, 4);
        b.add(p + "linear_attn.norm.weight", {c.lin_v_dim}, 4);
        b.add(p + "linear_attn.out_proj.weight", {c.hidden, c.value_dim()}, 2);
      } else {
        b.add(p + "self_attn.q_proj.weight", {c.q_out(), c.hidden}, 2);
        b.add(p + "self_attn.k_proj.weight", {c.kv_dim(), c.hidden}, 2);
        b.add(p + "self_attn.v_proj.weight", {c.kv_dim(), c.hidden}, 2);
        b.add(p + "self_attn.o_proj.weight", {c.hidden, c.attn_dim()}, 2);
        b.add(p + "self_attn.q_norm.weight", {c.head_dim}, 2);
        b.add(p + "self_attn.k_norm.weight", {c.head_dim}, 2);
      }
      b.add(p + "mlp.gate_proj.weight", {c.intermediate, c.hidden}, 2);
      b.add(p + "mlp.up_proj.weight", {c.intermediate, c.hidden}, 2);
      b.add(p + "mlp.down_proj.weight", {c.hidden, c.intermediate}, 2);
    }
    const uint64_t group_bytes = align_up(b.cursor - group_start);
    if (g == 0)
      b.m.group_stride = group_bytes;
    else if (b.m.group_stride != group_bytes && b.error.empty())
      b.error = "layer groups have different weight sizes";
    b.cursor = group_start + b.m.group_stride;
  }
  b.add(root + "norm.weight", {c.hidden}, 2);
  b.m.total_bytes = align_up(b.cursor);
  b.m.num_groups = groups;
}

} // namespace

// ------------------------------------------------------------------------------
// Q8_0 quantisation and lane packing
// ------------------------------------------------------------------------------
void quantize_row_q8_0(const float *values, int64_t cols, uint16_t *d, int8_t *qs) {
  for (int64_t b = 0; b < cols / 32; ++b) {
    const float *v = values + b * 32;
    float amax = 0.0f;
    for (int i = 0; i < 32; ++i)
      amax = std::max(amax, std::fabs(v[i]));
    if (amax == 0.0f) {
      d[b] = 0;
      std::memset(qs + b * 32, 0, 32);
      continue;
    }
    const float scale = amax / 127.0f;
    d[b] = f32_to_f16_bits(scale);
    for (int i = 0; i < 32; ++i) {
      long q = std::lround(v[i] / scale);
      qs[b * 32 + i] = static_cast<int8_t>(std::min(127L, std::max(-127L, q)));
    }
  }
}

bool pack_q8_0_p4(const float *values, int64_t rows, int64_t cols, uint8_t *dst) {
  if (rows <= 0 || cols <= 0 || rows % 8 != 0 || cols % 32 != 0)
    return false;
  const int64_t blocks = cols / 32;
#pragma omp parallel for schedule(static)
  for (int64_t g = 0; g < rows / 4; ++g) {
    std::vector<uint16_t> d(static_cast<size_t>(blocks));
    std::vector<int8_t> qs(static_cast<size_t>(cols));
    for (int lane = 0; lane < 4; ++lane) {
      quantize_row_q8_0(values + (g * 4 + lane) * cols, cols, d.data(), qs.data());
      for (int64_t b = 0; b < blocks; ++b) {
        uint8_t *rec = dst + (g * blocks + b) * 136;
        rec[lane * 2] = static_cast<uint8_t>(d[b] & 0xff);
        rec[lane * 2 + 1] = static_cast<uint8_t>(d[b] >> 8);
        for (int word = 0; word < 8; ++word)
          std::memcpy(rec + 8 + word * 16 + lane * 4, qs.data() + b * 32 + word * 4, 4);
      }
    }
  }
  return true;
}

// ------------------------------------------------------------------------------
// synthetic checkpoint
// ------------------------------------------------------------------------------
static uint64_t mix64(uint64_t x) {
  x += 0x9e3779b97f4a7c15ull;
  x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull;
  x = (x ^ (x >> 27)) * 0x94d049bb133111ebull;
  return x ^ (x >> 31);
}

float synthetic_normal(uint64_t seed, uint64_t tensor, uint64_t index) {
  const uint64_t key = mix64(seed * 0x2545f4914f6cdd1dull + tensor);
  int32_t sum = 0;
  for (uint64_t part = 0; part < 3; ++part) {
    uint64_t r = mix64(key ^ (index * 3 + part));
    sum += static_cast<int32_t>(r & 0xffff) + static_cast<int32_t>((r >> 16) & 0xffff) +
           static_cast<int32_t>((r >> 32) & 0xffff) + static_cast<int32_t>(r >> 48);
  }
  return static_cast<float>(sum - 6 * 65535) * (1.0f / 65536.0f);
}

uint64_t synthetic_container_bytes(const ModelDims &dims, Manifest *layout) {
  Manifest m = build_layout(dims);
  const uint64_t bytes = m.total_bytes + m.to_json().size();
  if (layout)
    *layout = std::move(m);
  return bytes;
}

static bool ends_with(const std::string &s, const char *suffix) {
  const size_t n = std::strlen(suffix);
  return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}

std::string fill_synthetic_container(const ModelDims &dims, uint64_t seed, uint8_t *file, uint64_t file_bytes) {
  Manifest m = build_layout(dims);
  const std::string json = m.to_json();
  if (file_bytes != m.total_bytes + json.size())
    return "buffer size does not match synthetic_container_bytes";
  std::memset(file, 0, kHeaderBytes);
  // Alignment gaps are zeroed so that equal seeds give equal files.
  uint64_t covered = kHeaderBytes;
  for (const TensorEntry &t : m.tensors) {
    if (t.offset > covered)
      std::memset(file + covered, 0, t.offset - covered);
    covered = t.offset + t.size;
  }
  if (m.total_bytes > covered)
    std::memset(file + covered, 0, m.total_bytes - covered);
  for (size_t index = 0; index < m.tensors.size(); ++index) {
    const TensorEntry &t = m.tensors[index];
    uint8_t *dst = file + t.offset;
    if (t.dtype == "Q8_0") {
      const int64_t rows = t.shape[0], cols = t.shape[1], blocks = cols / 32;
      // Generated and packed four rows at a time so the bf16 checkpoint never exists whole.
#pragma omp parallel for schedule(static)
      for (int64_t g = 0; g < rows / 4; ++g) {
        std::vector<float> values(static_cast<size_t>(cols));
        std::vector<uint16_t> d(static_cast<size_t>(blocks));
        std::vector<int8_t> qs(static_cast<size_t>(cols));
        for (int lane = 0; lane < 4; ++lane) {
          const uint64_t row = static_cast<uint64_t>(g) * 4 + lane;
          for (int64_t c = 0; c < cols; ++c) {
            const float w = 0.02f * synthetic_normal(seed, index, row * cols + c);
            values[c] = bf16_bits_to_f32_host(f32_to_bf16_bits(w));
          }
          quantize_row_q8_0(values.data(), cols, d.data(), qs.data());
          for (int64_t b = 0; b < blocks; ++b) {
            uint8_t *rec = dst + (g * blocks + b) * 136;
            rec[lane * 2] = static_cast<uint8_t>(d[b] & 0xff);
            rec[lane * 2 + 1] = static_cast<uint8_t>(d[b] >> 8);
            for (int word = 0; word < 8; ++word)
              std::memcpy(rec + 8 + word * 16 + lane * 4, qs.data() + b * 32 + word * 4, 4);
          }
        }
      }
    } else if (ends_with(t.name, "conv1d.weight")) {
      uint16_t *out = reinterpret_cast<uint16_t *>(dst);
      for (uint64_t i = 0; i < t.size / 2; ++i)
        out[i] = f32_to_bf16_bits(0.5f * synthetic_normal(seed, index, i));
    } else if (ends_with(t.name, "linear_attn.norm.weight")) {
      float *out = reinterpret_cast<float *>(dst);
      for (uint64_t i = 0; i < t.size / 4; ++i)
        out[i] = 1.0f;
    } else {
      std::memset(dst, 0, t.size); // zero-centred gains, A_log, dt_bias
    }
  }
  std::memcpy(file + m.total_bytes, json.data(), json.size());
  write_header(file, m.total_bytes, json.size()); // the header is the commit marker
  return "";
}

void make_cos_sin(int64_t position, int64_t rotary, float theta, float *cos_out, float *sin_out) {
  for (int64_t d = 0; d < rotary / 2; ++d) {
    const float inv_freq = 1.0f / std::pow(theta, static_cast<float>(2 * d) / static_cast<float>(rotary));
    const float angle = static_cast<float>(position) * inv_freq;
    cos_out[d] = cos_out[d + rotary / 2] = std::cos(angle);
    sin_out[d] = sin_out[d + rotary / 2] = std::sin(angle);
  }
}

} // namespace llmcp_b200
