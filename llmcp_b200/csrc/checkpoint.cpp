#include "checkpoint.h"
#include "json.h"

#include <algorithm>
#include <cerrno>
#include <cstdio>
#include <cstring>
#include <dirent.h>
#include <fcntl.h>
#include <memory>
#include <set>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

namespace llmcp_b200 {

using namespace detail;

namespace {

constexpr uint64_t kMaxHeaderBytes = 64ull << 20; // a safetensors header larger than this is refused

const Json *member(const Json &object, const char *key, Json::Kind kind) {
  const Json *j = object.get(key);
  return j && j->kind == kind ? j : nullptr;
}

bool required_integer(const Json &object, const char *key, int64_t *out, std::string *error) {
  if (as_integer(object.get(key), out))
    return true;
  *error = std::string("missing or invalid integer field '") + key + "'";
  return false;
}

int64_t integer_or(const Json &object, const char *key, int64_t fallback) {
  int64_t v = 0;
  return as_integer(object.get(key), &v) ? v : fallback;
}

double number_or(const Json &object, const char *key, double fallback) {
  const Json *j = member(object, key, Json::Number);
  return j ? j->number : fallback;
}

bool read_whole_file(const std::string &path, std::string *out) {
  FILE *f = std::fopen(path.c_str(), "rb");
  if (!f)
    return false;
  char buffer[1 << 16];
  size_t n;
  out->clear();
  while ((n = std::fread(buffer, 1, sizeof buffer, f)) > 0)
    out->append(buffer, n);
  std::fclose(f);
  return true;
}

bool file_exists(const std::string &path) {
  struct stat st;
  return ::stat(path.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

bool has_suffix(const std::string &s, const char *suffix) {
  const size_t n = std::strlen(suffix);
  return s.size() >= n && s.compare(s.size() - n, n, suffix) == 0;
}

} // namespace

uint64_t safetensors_dtype_bytes(const std::string &dtype) {
  if (dtype == "BF16" || dtype == "F16" || dtype == "I16" || dtype == "U16")
    return 2;
  if (dtype == "F32" || dtype == "I32" || dtype == "U32")
    return 4;
  if (dtype == "F64" || dtype == "I64" || dtype == "U64")
    return 8;
  if (dtype == "I8" || dtype == "U8" || dtype == "BOOL" || dtype == "F8_E4M3" || dtype == "F8_E5M2")
    return 1;
  return 0;
}

std::string parse_model_config(const char *text, uint64_t length, ModelDims *dims) {
  JsonReader reader{text, text + length};
  const Json root = reader.value();
  if (!reader.ok)
    return "config.json is not valid JSON";
  if (root.kind != Json::Object)
    return "config.json must contain a top-level object";
  const Json *tc = member(root, "text_config", Json::Object);
  if (!tc)
    return "config.json must contain a 'text_config' object";

  ModelDims d;
  std::string error;
  if (!required_integer(*tc, "hidden_size", &d.hidden, &error) ||
      !required_integer(*tc, "intermediate_size", &d.intermediate, &error) ||
      !required_integer(*tc, "num_hidden_layers", &d.layers, &error) ||
      !required_integer(*tc, "num_attention_heads", &d.heads, &error) ||
      !required_integer(*tc, "num_key_value_heads", &d.kv_heads, &error) ||
      !required_integer(*tc, "vocab_size", &d.vocab, &error))
    return error;
  d.head_dim = integer_or(*tc, "head_dim", 0);
  if (d.head_dim == 0 && d.heads != 0)
    d.head_dim = d.hidden / d.heads;
  d.full_interval = integer_or(*tc, "full_attention_interval", 4);
  if (!required_integer(*tc, "linear_num_key_heads", &d.lin_k_heads, &error) ||
      !required_integer(*tc, "linear_num_value_heads", &d.lin_v_heads, &error) ||
      !required_integer(*tc, "linear_key_head_dim", &d.lin_k_dim, &error) ||
      !required_integer(*tc, "linear_value_head_dim", &d.lin_v_dim, &error))
    return error;
  d.conv_kernel = integer_or(*tc, "linear_conv_kernel_dim", 4);
  const Json *act = member(*tc, "hidden_act", Json::String);
  if (!act)
    return "missing or invalid string field 'hidden_act'";
  d.eps = static_cast<float>(number_or(*tc, "rms_norm_eps", 1.0e-6));
  double theta = 1.0e7, rotary_factor = 0.25;
  if (const Json *rope = member(*tc, "rope_parameters", Json::Object)) {
    theta = number_or(*rope, "rope_theta", theta);
    rotary_factor = number_or(*rope, "partial_rotary_factor", rotary_factor);
  }
  d.rope_theta = static_cast<float>(theta);

  // The checks of ModelConfig::verify (lib/Model/ModelConfig.cpp:228-283), in its order.
  if (d.layers <= 0)
    return "num_hidden_layers must be positive";
  if (d.full_interval <= 0)
    return "full_attention_interval must be positive";
  if (const Json *types = member(*tc, "layer_types", Json::Array)) {
    if (static_cast<int64_t>(types->items.size()) != d.layers)
      return "layer_types has " + std::to_string(types->items.size()) + " entries, expected " +
             std::to_string(d.layers);
    for (int64_t i = 0; i < d.layers; ++i) {
      const Json &t = types->items[static_cast<size_t>(i)];
      if (t.kind != Json::String)
        return "layer_types must contain strings";
      if (t.text != "linear_attention" && t.text != "full_attention")
        return "unknown layer type '" + t.text + "'";
      // The engine runs one mixer pattern: every `full_interval`-th layer is full attention.
      if ((t.text == "full_attention") != d.is_full(i))
        return "unsupported layer pattern: layer " + std::to_string(i) + " is " + t.text;
    }
  }
  if (d.hidden <= 0 || d.intermediate <= 0 || d.vocab <= 0)
    return "hidden/intermediate/vocab sizes must be positive";
  if (d.heads <= 0 || d.kv_heads <= 0 || d.head_dim <= 0)
    return "attention head configuration must be positive";
  if (d.heads % d.kv_heads != 0)
    return "num_attention_heads must be divisible by num_key_value_heads";
  if (d.lin_k_heads <= 0 || d.lin_v_heads <= 0 || d.lin_k_dim <= 0 || d.lin_v_dim <= 0)
    return "linear attention head configuration must be positive";
  if (d.lin_v_heads % d.lin_k_heads != 0)
    return "linear_num_value_heads must be divisible by linear_num_key_heads";
  if (d.conv_kernel <= 0)
    return "linear_conv_kernel_dim must be positive";
  if (!(rotary_factor > 0.0 && rotary_factor <= 1.0))
    return "partial_rotary_factor must be in (0, 1]";
  if (!(d.eps > 0.0f))
    return "rms_norm_eps must be positive";
  if (act->text != "silu")
    return "unsupported hidden_act '" + act->text + "' (only 'silu' is supported)";
  if (d.layers % d.full_interval != 0)
    return "num_hidden_layers must be divisible by full_attention_interval";
  d.rotary = static_cast<int64_t>(static_cast<double>(d.head_dim) * rotary_factor);
  if (d.rotary <= 0 || d.rotary % 2 != 0)
    return "rotary dimension must be positive and even";
  if (d.full_interval < 2)
    return "model must contain at least one linear attention layer";
  bool tied = true;
  if (const Json *t = member(root, "tie_word_embeddings", Json::Bool))
    tied = t->boolean;
  else if (const Json *t2 = member(*tc, "tie_word_embeddings", Json::Bool))
    tied = t2->boolean;
  if (!tied)
    return "untied lm_head is not supported yet";
  *dims = d;
  return "";
}

std::string parse_safetensors_header(const char *json, uint64_t length, uint64_t data_start, uint64_t file_size,
                                     const std::string &shard, SourceTensors *out) {
  if (data_start > file_size)
    return "safetensors header extends past end of file";
  JsonReader reader{json, json + length};
  const Json root = reader.value();
  if (!reader.ok)
    return "safetensors header is not valid JSON";
  if (root.kind != Json::Object)
    return "safetensors header must be a JSON object";
  SourceTensors found;
  for (const auto &entry : root.members) {
    const std::string &name = entry.first;
    if (name == "__metadata__")
      continue;
    const Json &info = entry.second;
    if (info.kind != Json::Object)
      return "tensor '" + name + "' metadata must be an object";
    const Json *dtype = member(info, "dtype", Json::String);
    if (!dtype)
      return "tensor '" + name + "' is missing dtype";
    const uint64_t element_bytes = safetensors_dtype_bytes(dtype->text);
    if (element_bytes == 0)
      return "unsupported safetensors dtype '" + dtype->text + "'";
    const Json *shape = member(info, "shape", Json::Array);
    if (!shape)
      return "tensor '" + name + "' is missing shape";
    SourceTensor t;
    t.name = name;
    t.dtype = dtype->text;
    t.shard = shard;
    uint64_t elements = 1;
    for (const Json &dim : shape->items) {
      int64_t extent = 0;
      if (!as_integer(&dim, &extent) || extent < 0)
        return "tensor '" + name + "' has an invalid shape";
      t.shape.push_back(extent);
      elements *= static_cast<uint64_t>(extent);
    }
    const Json *offsets = member(info, "data_offsets", Json::Array);
    int64_t begin = 0, end = 0;
    if (!offsets || offsets->items.size() != 2)
      return "tensor '" + name + "' is missing data_offsets";
    if (!as_integer(&offsets->items[0], &begin) || !as_integer(&offsets->items[1], &end) || begin < 0 || end < begin)
      return "tensor '" + name + "' has invalid data_offsets";
    if (static_cast<uint64_t>(end) > file_size - data_start)
      return "tensor '" + name + "' extends past end of file";
    if (static_cast<uint64_t>(end - begin) != elements * element_bytes)
      return "tensor '" + name + "' data size does not match dtype and shape";
    t.data_offset = data_start + static_cast<uint64_t>(begin);
    t.data_size = static_cast<uint64_t>(end - begin);
    if (!found.emplace(name, std::move(t)).second)
      return "duplicate tensor '" + name + "'";
  }
  for (auto &item : found)
    if (!out->emplace(item.first, std::move(item.second)).second)
      return "duplicate tensor '" + item.first + "'";
  return "";
}

std::string read_safetensors_file(const std::string &path, const std::string &shard, SourceTensors *out) {
  FILE *f = std::fopen(path.c_str(), "rb");
  if (!f)
    return "cannot open safetensors file '" + path + "'";
  std::unique_ptr<FILE, int (*)(FILE *)> closer(f, std::fclose);
  struct stat st;
  if (::fstat(fileno(f), &st) != 0 || st.st_size < 8)
    return "safetensors file '" + path + "' is too small";
  const uint64_t file_size = static_cast<uint64_t>(st.st_size);
  unsigned char size_bytes[8];
  if (std::fread(size_bytes, 1, 8, f) != 8)
    return "cannot read header size from '" + path + "'";
  uint64_t header_bytes = 0;
  for (int i = 0; i < 8; ++i)
    header_bytes |= static_cast<uint64_t>(size_bytes[i]) << (8 * i);
  if (header_bytes > kMaxHeaderBytes || header_bytes > file_size - 8)
    return "invalid safetensors header size in '" + path + "'";
  std::string header(header_bytes, '\0');
  if (header_bytes && std::fread(&header[0], 1, header_bytes, f) != header_bytes)
    return "cannot read header from '" + path + "'";
  return parse_safetensors_header(header.data(), header.size(), 8 + header_bytes, file_size, shard, out);
}

std::string read_checkpoint_tensors(const std::string &model_dir, SourceTensors *out) {
  std::vector<std::string> shards;
  std::string index_text;
  if (read_whole_file(model_dir + "/model.safetensors.index.json", &index_text)) {
    JsonReader reader{index_text.data(), index_text.data() + index_text.size()};
    const Json root = reader.value();
    if (!reader.ok || root.kind != Json::Object)
      return "safetensors index must be a JSON object";
    const Json *map = member(root, "weight_map", Json::Object);
    if (!map)
      return "safetensors index is missing weight_map";
    std::set<std::string> seen;
    for (const auto &entry : map->members) {
      if (entry.second.kind != Json::String)
        return "weight_map entry '" + entry.first + "' must be a string";
      if (seen.insert(entry.second.text).second)
        shards.push_back(entry.second.text);
    }
  } else {
    DIR *dir = ::opendir(model_dir.c_str());
    if (!dir)
      return "cannot scan model directory '" + model_dir + "'";
    while (const dirent *e = ::readdir(dir)) {
      const std::string name = e->d_name;
      if (has_suffix(name, ".safetensors") && file_exists(model_dir + "/" + name))
        shards.push_back(name);
    }
    ::closedir(dir);
  }
  std::sort(shards.begin(), shards.end());
  if (shards.empty())
    return "no safetensors shards found";
  SourceTensors tensors;
  for (const std::string &shard : shards) {
    std::string error = read_safetensors_file(model_dir + "/" + shard, shard, &tensors);
    if (!error.empty())
      return error;
  }
  *out = std::move(tensors);
  return "";
}

// ------------------------------------------------------------------------------
// synthetic checkpoint
// ------------------------------------------------------------------------------
namespace {

std::string format_double(double v) {
  char text[40];
  std::snprintf(text, sizeof text, "%.17g", v);
  return text;
}

std::string config_json(const ModelDims &d) {
  std::string layer_types;
  for (int64_t i = 0; i < d.layers; ++i)
    layer_types += std::string(i ? "," : "") + (d.is_full(i) ? "\"full_attention\"" : "\"linear_attention\"");
  std::string out = "{\"architectures\":[\"Qwen3_5ForConditionalGeneration\"],\"tie_word_embeddings\":true,\"text_config\":{";
  auto integer = [&](const char *key, int64_t v) { out += std::string("\"") + key + "\":" + std::to_string(v) + ","; };
  out += "\"attention_bias\":false,\"attn_output_gate\":true,\"hidden_act\":\"silu\",";
  integer("head_dim", d.head_dim);
  integer("hidden_size", d.hidden);
  integer("intermediate_size", d.intermediate);
  integer("full_attention_interval", d.full_interval);
  out += "\"layer_types\":[" + layer_types + "],";
  integer("linear_conv_kernel_dim", d.conv_kernel);
  integer("linear_key_head_dim", d.lin_k_dim);
  integer("linear_num_key_heads", d.lin_k_heads);
  integer("linear_num_value_heads", d.lin_v_heads);
  integer("linear_value_head_dim", d.lin_v_dim);
  integer("num_attention_heads", d.heads);
  integer("num_hidden_layers", d.layers);
  integer("num_key_value_heads", d.kv_heads);
  out += "\"rms_norm_eps\":" + format_double(static_cast<double>(d.eps)) + ",";
  out += "\"rope_parameters\":{\"partial_rotary_factor\":" +
         format_double(static_cast<double>(d.rotary) / static_cast<double>(d.head_dim)) +
         ",\"rope_theta\":" + format_double(static_cast<double>(d.rope_theta)) + ",\"rope_type\":\"default\"},";
  out += "\"tie_word_embeddings\":true,\"vocab_size\":" + std::to_string(d.vocab) + "}}\n";
  return out;
}

bool write_text(const std::string &path, const std::string &text) {
  FILE *f = std::fopen(path.c_str(), "wb");
  if (!f)
    return false;
  const bool ok = std::fwrite(text.data(), 1, text.size(), f) == text.size();
  return std::fclose(f) == 0 && ok;
}

} // namespace

std::string write_synthetic_checkpoint(const ModelDims &dims, uint64_t seed, const std::string &model_dir) {
  // The tensors, their order and their value streams are those of fill_synthetic_container, so
  // that packing this checkpoint reproduces that container byte for byte.
  const Manifest layout = build_layout(dims);
  struct Source {
    const TensorEntry *entry;
    bool f32;
    uint64_t elements, begin;
  };
  std::vector<Source> sources;
  uint64_t cursor = 0;
  std::string header = "{\"__metadata__\":{\"format\":\"pt\"}";
  std::string weight_map;
  for (const TensorEntry &t : layout.tensors) {
    uint64_t elements = 1;
    for (int64_t dim : t.shape)
      elements *= static_cast<uint64_t>(dim);
    const bool f32 = t.source_size == elements * 4;
    sources.push_back({&t, f32, elements, cursor});
    std::string shape;
    for (size_t i = 0; i < t.shape.size(); ++i)
      shape += (i ? "," : "") + std::to_string(t.shape[i]);
    header += ",\"" + t.name + "\":{\"dtype\":\"" + (f32 ? "F32" : "BF16") + "\",\"shape\":[" + shape +
              "],\"data_offsets\":[" + std::to_string(cursor) + "," + std::to_string(cursor + t.source_size) + "]}";
    weight_map += std::string(weight_map.empty() ? "" : ",") + "\"" + t.name + "\":\"model.safetensors\"";
    cursor += t.source_size;
  }
  header += "}";
  while (header.size() % 8 != 0) // the data section starts 8-byte aligned, as writers of the format do
    header += ' ';

  FILE *f = std::fopen((model_dir + "/model.safetensors").c_str(), "wb");
  if (!f)
    return "cannot create '" + model_dir + "/model.safetensors'";
  std::unique_ptr<FILE, int (*)(FILE *)> closer(f, std::fclose);
  unsigned char size_bytes[8];
  for (int i = 0; i < 8; ++i)
    size_bytes[i] = static_cast<unsigned char>(static_cast<uint64_t>(header.size()) >> (8 * i));
  if (std::fwrite(size_bytes, 1, 8, f) != 8 || std::fwrite(header.data(), 1, header.size(), f) != header.size())
    return "cannot write the safetensors header";
  for (size_t index = 0; index < sources.size(); ++index) {
    const Source &src = sources[index];
    const TensorEntry &t = *src.entry;
    const uint64_t chunk = 1u << 20;
    std::vector<uint8_t> buffer;
    for (uint64_t first = 0; first < src.elements; first += chunk) {
      const uint64_t count = std::min(chunk, src.elements - first);
      buffer.assign(count * (src.f32 ? 4 : 2), 0);
      if (t.dtype == "Q8_0" || has_suffix(t.name, "conv1d.weight")) {
        const float gain = t.dtype == "Q8_0" ? 0.02f : 0.5f;
        uint16_t *out = reinterpret_cast<uint16_t *>(buffer.data());
#pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < static_cast<int64_t>(count); ++i)
          out[i] = f32_to_bf16_bits(gain * synthetic_normal(seed, index, first + static_cast<uint64_t>(i)));
      } else if (has_suffix(t.name, "linear_attn.norm.weight")) {
        float *out = reinterpret_cast<float *>(buffer.data());
        for (uint64_t i = 0; i < count; ++i)
          out[i] = 1.0f;
      } // zero-centred gains, A_log and dt_bias stay zero
      if (std::fwrite(buffer.data(), 1, buffer.size(), f) != buffer.size())
        return "cannot write tensor data of " + t.name;
    }
  }
  closer.reset();
  if (!write_text(model_dir + "/model.safetensors.index.json",
                  "{\"metadata\":{\"total_size\":" + std::to_string(cursor) + "},\"weight_map\":{" + weight_map + "}}\n") ||
      !write_text(model_dir + "/config.json", config_json(dims)))
    return "cannot write config.json / model.safetensors.index.json in '" + model_dir + "'";
  return "";
}

// ------------------------------------------------------------------------------
// packing
// ------------------------------------------------------------------------------
namespace {

// A whole file mapped into memory: shards read-only, the output read-write at its final size.
class MappedFile {
public:
  MappedFile() = default;
  MappedFile(const MappedFile &) = delete;
  MappedFile &operator=(const MappedFile &) = delete;
  ~MappedFile() {
    if (base_)
      ::munmap(base_, size_);
    if (fd_ >= 0)
      ::close(fd_);
  }

  std::string open_read(const std::string &path) {
    fd_ = ::open(path.c_str(), O_RDONLY);
    struct stat st;
    if (fd_ < 0 || ::fstat(fd_, &st) != 0)
      return "cannot open '" + path + "': " + std::strerror(errno);
    size_ = static_cast<uint64_t>(st.st_size);
    return map(path, PROT_READ);
  }

  std::string create(const std::string &path, uint64_t size) {
    fd_ = ::open(path.c_str(), O_RDWR | O_CREAT | O_TRUNC, 0644);
    if (fd_ < 0 || ::ftruncate(fd_, static_cast<off_t>(size)) != 0)
      return "cannot create '" + path + "': " + std::strerror(errno);
    size_ = size;
    return map(path, PROT_READ | PROT_WRITE);
  }

  uint8_t *data() const { return static_cast<uint8_t *>(base_); }
  uint64_t size() const { return size_; }

private:
  std::string map(const std::string &path, int protection) {
    if (size_ == 0)
      return "'" + path + "' is empty";
    void *p = ::mmap(nullptr, size_, protection, MAP_SHARED, fd_, 0);
    if (p == MAP_FAILED)
      return "cannot map '" + path + "': " + std::strerror(errno);
    base_ = p;
    return "";
  }

  int fd_ = -1;
  void *base_ = nullptr;
  uint64_t size_ = 0;
};

// Q8_0 with the four-row lane packing straight from checkpoint bytes
// (lib/Model/Quantization.cpp:165-214).  Eight rows at a time, so that the f32 copy of a
// 248320-row table never exists whole; the chunks are independent and run on all host threads.
void quantise_tensor(const uint8_t *source, bool bf16, int64_t rows, int64_t cols, uint8_t *destination) {
  const int64_t blocks = cols / 32;
#pragma omp parallel
  {
    std::vector<float> values(static_cast<size_t>(8 * cols));
#pragma omp for schedule(static)
    for (int64_t chunk = 0; chunk < rows / 8; ++chunk) {
      const uint64_t first = static_cast<uint64_t>(chunk) * 8 * cols;
      if (bf16) {
        const uint8_t *src = source + first * 2;
        for (int64_t i = 0; i < 8 * cols; ++i) {
          uint16_t bits;
          std::memcpy(&bits, src + i * 2, 2);
          values[i] = bf16_bits_to_f32_host(bits);
        }
      } else {
        std::memcpy(values.data(), source + first * 4, static_cast<size_t>(8 * cols) * 4);
      }
      pack_q8_0_p4(values.data(), 8, cols, destination + static_cast<uint64_t>(chunk) * 2 * blocks * 136);
    }
  }
}

} // namespace

std::string pack_checkpoint(const std::string &model_dir, const std::string &output_path, const std::string &quant,
                            bool dry_run, bool verbose, PackSummary *summary) {
  if (quant != "none" && quant != "q8_0")
    return "unknown quantization mode '" + quant + "' (expected none or q8_0)";
  if (!dry_run && output_path.empty())
    return "an output path is required unless this is a dry run";

  std::string config_text;
  if (!read_whole_file(model_dir + "/config.json", &config_text))
    return "cannot read '" + model_dir + "/config.json'";
  ModelDims dims;
  std::string error = parse_model_config(config_text.data(), config_text.size(), &dims);
  if (!error.empty())
    return error;
  SourceTensors tensors;
  error = read_checkpoint_tensors(model_dir, &tensors);
  if (!error.empty())
    return error;
  Manifest layout;
  error = plan_layout(dims, tensors, quant == "q8_0", &layout);
  if (!error.empty())
    return error;
  layout.model = model_dir;

  PackSummary s;
  s.tensors = layout.tensors.size();
  s.arena_bytes = layout.total_bytes;
  for (const TensorEntry &t : layout.tensors)
    s.source_bytes += t.source_size;
  if (summary)
    *summary = s;
  if (dry_run) {
    if (verbose)
      std::printf("validated %zu tensors\n", layout.tensors.size());
    return "";
  }

  const std::string manifest = layout.to_json();
  MappedFile output;
  error = output.create(output_path, layout.total_bytes + manifest.size());
  if (!error.empty())
    return error;
  // A new file reads as zeros, so the alignment gaps need no clearing; the header stays zero
  // (not a valid container) until everything else is in place.
  std::memset(output.data(), 0, kHeaderBytes);

  std::map<std::string, std::unique_ptr<MappedFile>> shards;
  for (const TensorEntry &entry : layout.tensors) {
    const SourceTensor &source = tensors.at(entry.name);
    std::unique_ptr<MappedFile> &shard = shards[source.shard];
    if (!shard) {
      shard.reset(new MappedFile);
      error = shard->open_read(model_dir + "/" + source.shard);
      if (!error.empty())
        return error;
    }
    if (source.data_offset > shard->size() || source.data_size > shard->size() - source.data_offset)
      return "tensor extends past shard: " + entry.name;
    const uint8_t *bytes = shard->data() + source.data_offset;
    if (entry.dtype == "Q8_0")
      quantise_tensor(bytes, source.dtype == "BF16", entry.shape[0], entry.shape[1], output.data() + entry.offset);
    else
      std::memcpy(output.data() + entry.offset, bytes, entry.size);
    if (verbose)
      std::printf("  %llu +%llu %s\n", static_cast<unsigned long long>(entry.offset),
                  static_cast<unsigned long long>(entry.size), entry.name.c_str());
  }
  std::memcpy(output.data() + layout.total_bytes, manifest.data(), manifest.size());
  write_header(output.data(), layout.total_bytes, manifest.size()); // published last
  return "";
}

} // namespace llmcp_b200
