// Reading a Qwen3.5 checkpoint directory (config.json + safetensors shards) and packing it
// into the llmcp weight container, i.e. what `llmcp-pack --model DIR --out FILE --quant q8_0`
// does in the llmcp project:
//   config      lib/Model/ModelConfig.cpp:70-283
//   safetensors lib/Model/Safetensors.cpp:47-253
//   packing     lib/Model/WeightPacker.cpp:163-274, tools/llmcp-pack/llmcp-pack.cpp:44-89
// Every function returns "" on success, else the reason.
#pragma once

#include "format.h"

#include <cstdint>
#include <string>

namespace llmcp_b200 {

// Bytes per element of a safetensors dtype name, 0 for an unknown one.
uint64_t safetensors_dtype_bytes(const std::string &dtype);

// Model dimensions from the text of config.json (the `text_config` object).
std::string parse_model_config(const char *text, uint64_t length, ModelDims *dims);

// Tensors named by one safetensors JSON header.  `data_start` is the file position of the
// first data byte, `file_size` the size of the shard; offsets in `out` are absolute.
std::string parse_safetensors_header(const char *json, uint64_t length, uint64_t data_start, uint64_t file_size,
                                     const std::string &shard, SourceTensors *out);

// Header of one shard file (no tensor data is read).
std::string read_safetensors_file(const std::string &path, const std::string &shard, SourceTensors *out);

// All shard headers of a model directory: the shards model.safetensors.index.json names, or,
// without an index, every *.safetensors file of the directory in name order.
std::string read_checkpoint_tensors(const std::string &model_dir, SourceTensors *out);

// Writes a random-init checkpoint directory (config.json, model.safetensors,
// model.safetensors.index.json) whose tensors are the values fill_synthetic_container draws for
// (`dims`, `seed`): packing it with --quant q8_0 gives that container byte for byte, apart from
// the manifest's model field.  The 4B-shaped model is 8.4 GB of bf16.
std::string write_synthetic_checkpoint(const ModelDims &dims, uint64_t seed, const std::string &model_dir);

struct PackSummary {
  uint64_t tensors = 0, source_bytes = 0, arena_bytes = 0;
};

// Packs the checkpoint in `model_dir` into the single-file container `output_path`
// (arena, manifest, header written last).  `quant` is "none" or "q8_0".  With `dry_run` the
// checkpoint is only validated against the layout and nothing is written.
std::string pack_checkpoint(const std::string &model_dir, const std::string &output_path, const std::string &quant,
                            bool dry_run, bool verbose, PackSummary *summary);

} // namespace llmcp_b200
