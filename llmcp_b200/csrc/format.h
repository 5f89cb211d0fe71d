// Host-side formats of the llmcp weight container: the 64-byte "LLMCPWGT" header, the JSON
// manifest that follows the arena, the deterministic tensor layout, Q8_0 quantisation with
// the four-row lane packing, and a seeded synthetic checkpoint generator.
//
// Format references (paths inside the llmcp project):
//   header      include/llmcp/Support/PackedWeights.h:21-58
//   manifest    lib/Model/WeightPacker.cpp:126-160, checks lib/Runtime/WeightArena.cpp:51-123
//   layout      lib/Model/WeightLayout.cpp:96-268
//   Q8_0 + p4   lib/Model/Quantization.cpp:92-116,165-214, Support/Q8PackedLayout.h:17-42
#pragma once

#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace llmcp_b200 {

struct ModelDims {
  int64_t hidden = 2560, intermediate = 9216, vocab = 248320, layers = 32, full_interval = 4;
  int64_t heads = 16, kv_heads = 4, head_dim = 256, rotary = 64;
  int64_t lin_k_heads = 16, lin_v_heads = 32, lin_k_dim = 128, lin_v_dim = 128, conv_kernel = 4;
  float eps = 1.0e-6f;
  float rope_theta = 1.0e7f;

  int64_t qkv_dim() const { return 2 * lin_k_heads * lin_k_dim + lin_v_heads * lin_v_dim; }
  int64_t value_dim() const { return lin_v_heads * lin_v_dim; }
  int64_t q_out() const { return heads * head_dim * 2; }
  int64_t kv_dim() const { return kv_heads * head_dim; }
  int64_t attn_dim() const { return heads * head_dim; }
  int64_t full_layers() const { return layers / full_interval; }
  int64_t linear_layers() const { return layers - full_layers(); }
  bool is_full(int64_t layer) const { return layer % full_interval == full_interval - 1; }
};

struct TensorEntry {
  std::string name;
  uint64_t offset = 0;
  uint64_t size = 0;        // bytes in the arena
  uint64_t source_size = 0; // bytes in the checkpoint
  std::string dtype;        // "Q8_0", "BF16", "F32"
  std::vector<int64_t> shape;
};

struct Manifest {
  std::string model;
  uint64_t total_bytes = 0, header_bytes = 64, group_stride = 0;
  int64_t num_groups = 0;
  std::string quantization = "q8_0";
  std::vector<TensorEntry> tensors;

  const TensorEntry *find(const std::string &name) const;
  std::string to_json() const;
};

constexpr uint64_t kHeaderBytes = 64;
constexpr uint64_t kTensorAlignment = 64;

// Writes / reads the file header.  read_header returns an empty string on success, else
// the reason the header is rejected.
void write_header(uint8_t *data, uint64_t arena_bytes, uint64_t manifest_bytes);
std::string read_header(const uint8_t *data, uint64_t file_bytes, uint64_t *arena_bytes,
                        uint64_t *manifest_offset, uint64_t *manifest_bytes);

// Parses and validates the manifest text against the arena size.  Returns "" on success.
std::string parse_manifest(const char *text, uint64_t length, uint64_t arena_bytes, Manifest *out);

// Header + manifest of a mapped container whose first byte is `base`.  `file_bytes` may be 0
// when only the arena length is known (the AOT entry points): the manifest is then located
// through the header fields alone.
std::string parse_container(const uint8_t *base, uint64_t file_bytes, Manifest *out);

// Tensor order, shapes, dtypes and offsets of a Qwen3.5-style model packed with --quant q8_0.
Manifest build_layout(const ModelDims &dims);

// One tensor of a checkpoint as a safetensors header describes it: `data_offset` is the
// absolute position of its first byte in the shard file `shard`
// (include/llmcp/Model/Safetensors.h:24-33).
struct SourceTensor {
  std::string name, dtype, shard;
  std::vector<int64_t> shape;
  uint64_t data_offset = 0, data_size = 0;
};
using SourceTensors = std::map<std::string, SourceTensor>;

// The same layout for a real checkpoint: every tensor must be present with the expected
// shape; dtype and byte size come from the checkpoint; with `q8` the 2-D bf16/f32 tensors
// whose shape allows it become Q8_0.  Returns "" or the reason (lib/Model/WeightLayout.cpp:54-268).
std::string plan_layout(const ModelDims &dims, const SourceTensors &tensors, bool q8, Manifest *out);

// Q8_0: per 32 values d = f16(amax / 127), q = clamp(lround(x / (amax / 127)), -127, 127).
void quantize_row_q8_0(const float *values, int64_t cols, uint16_t *d, int8_t *qs);
// Four-row lane packing of a [rows, cols] f32 matrix; dst holds rows/4 * cols/32 records of
// 136 bytes.  Returns false when rows % 8 or cols % 32 is non-zero.
bool pack_q8_0_p4(const float *values, int64_t rows, int64_t cols, uint8_t *dst);

uint16_t f32_to_f16_bits(float value);
float f16_bits_to_f32_host(uint16_t bits);
uint16_t f32_to_bf16_bits(float value);
float bf16_bits_to_f32_host(uint16_t bits);

// Deterministic pseudo-normal value number `index` of stream (`seed`, `tensor`): the sum of
// twelve 16-bit uniforms, centred and scaled to unit variance.  Integer arithmetic plus one
// exact scaling, so every platform produces the same bits.
float synthetic_normal(uint64_t seed, uint64_t tensor, uint64_t index);

// Fills `file` (arena + manifest, size synthetic_container_bytes) with a random-init model:
// 2-D weights 0.02 * N(0,1) rounded to bf16 then packed to q8_0_p4, zero-centred norm gains 0,
// linear_attn.norm.weight 1.0 (f32), A_log 0 (f32), dt_bias 0 (bf16), conv weights
// 0.5 * N(0,1) (bf16).  Returns "" on success.
uint64_t synthetic_container_bytes(const ModelDims &dims, Manifest *layout);
std::string fill_synthetic_container(const ModelDims &dims, uint64_t seed, uint8_t *file, uint64_t file_bytes);

// cos/sin rows of the rotary embedding for one position (lib/Runtime/AotRuntime.cpp:22-32).
void make_cos_sin(int64_t position, int64_t rotary, float theta, float *cos_out, float *sin_out);

} // namespace llmcp_b200
