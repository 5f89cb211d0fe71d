// What the reference's drivers share, on top of this repository's container reader: the mapped
// weights file (lib/Runtime/WeightArena.cpp:39-123) and the AOT ABI v2 runtime that owns the
// generation state and calls the two entry points (lib/Runtime/AotRuntime.cpp:39-120).
#pragma once

#include <dlfcn.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../format.h"

namespace llmcp_b200 {
namespace host {

// Strided memref descriptor of the MLIR C interface (include/llmcp/Runtime/AotRuntime.h:52-58).
template <typename T, int N> struct MemRef {
  T *base;
  T *data;
  int64_t offset;
  int64_t sizes[N];
  int64_t strides[N];
};

using EntryFn = void (*)(void *, void *, void *, void *, void *, void *, void *, void *, void *, void *);

struct Arena {
  const uint8_t *base = nullptr;
  uint64_t mapped = 0, size = 0;
  Manifest manifest;

  std::string load(const std::string &path) {
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0)
      return "cannot open " + path;
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < static_cast<off_t>(kHeaderBytes)) {
      close(fd);
      return "packed weights file is too small";
    }
    void *mapping = mmap(nullptr, static_cast<size_t>(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (mapping == MAP_FAILED)
      return "mmap failed";
    Manifest parsed;
    const std::string error = parse_container(static_cast<const uint8_t *>(mapping), static_cast<uint64_t>(st.st_size), &parsed);
    if (!error.empty()) {
      munmap(mapping, static_cast<size_t>(st.st_size));
      return error;
    }
    base = static_cast<const uint8_t *>(mapping);
    mapped = static_cast<uint64_t>(st.st_size);
    size = parsed.total_bytes;
    manifest = std::move(parsed);
    return "";
  }
};

// lib/Runtime/AotRuntime.cpp:39-120 with the model constants of :41-43.
struct Runtime {
  ModelDims dims;
  void *handle = nullptr;
  EntryFn prefill = nullptr, decode = nullptr;
  int64_t capacity = 0;
  std::vector<uint16_t> kv, conv;
  std::vector<float> delta;

  bool init(const std::string &path, int64_t max_sequence) {
    capacity = max_sequence;
    kv.assign(static_cast<size_t>(dims.full_layers() * 2 * dims.kv_heads * capacity * dims.head_dim), 0);
    delta.assign(static_cast<size_t>(dims.linear_layers() * dims.lin_v_heads * dims.lin_k_dim * dims.lin_v_dim), 0.0f);
    conv.assign(static_cast<size_t>(dims.linear_layers() * (dims.conv_kernel - 1) * dims.qkv_dim()), 0);
    handle = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!handle) {
      std::fprintf(stderr, "AotRuntime: dlopen: %s\n", dlerror());
      return false;
    }
    auto version = reinterpret_cast<int32_t (*)()>(dlsym(handle, "llmcp_model_abi_version"));
    if (!version || version() != 2) {
      std::fprintf(stderr, "AotRuntime: incompatible AOT ABI\n");
      return false;
    }
    prefill = reinterpret_cast<EntryFn>(dlsym(handle, "_mlir_ciface_llmcp_model_prefill"));
    decode = reinterpret_cast<EntryFn>(dlsym(handle, "_mlir_ciface_llmcp_model_decode"));
    if (!prefill || !decode) {
      std::fprintf(stderr, "AotRuntime: missing prefill/decode entry points\n");
      return false;
    }
    return true;
  }

  bool forward(const Arena &arena, const std::vector<int64_t> &tokens, int64_t start, int64_t cache_length,
               std::vector<float> &logits) {
    const int64_t sequence = static_cast<int64_t>(tokens.size());
    if (sequence == 0 || start < 0 || start > capacity || sequence > capacity - start)
      return false;
    std::vector<int64_t> ids = tokens;
    const int64_t rot = dims.rotary;
    std::vector<float> cos(static_cast<size_t>(sequence * rot)), sin(cos.size());
    for (int64_t t = 0; t < sequence; ++t)
      make_cos_sin(start + t, rot, dims.rope_theta, cos.data() + t * rot, sin.data() + t * rot);
    logits.assign(static_cast<size_t>(dims.vocab), 0.0f);
    MemRef<int64_t, 1> rt{ids.data(), ids.data(), 0, {sequence}, {1}};
    MemRef<float, 2> rc{cos.data(), cos.data(), 0, {sequence, rot}, {rot, 1}};
    MemRef<float, 2> rs{sin.data(), sin.data(), 0, {sequence, rot}, {rot, 1}};
    int8_t *bytes = const_cast<int8_t *>(reinterpret_cast<const int8_t *>(arena.base));
    MemRef<int8_t, 1> ra{bytes, bytes, 0, {static_cast<int64_t>(arena.size)}, {1}};
    MemRef<uint16_t, 5> rk{kv.data(), kv.data(), 0, {dims.full_layers(), 2, dims.kv_heads, capacity, dims.head_dim},
                           {2 * dims.kv_heads * capacity * dims.head_dim, dims.kv_heads * capacity * dims.head_dim,
                            capacity * dims.head_dim, dims.head_dim, 1}};
    MemRef<float, 4> rd{delta.data(), delta.data(), 0, {dims.linear_layers(), dims.lin_v_heads, dims.lin_k_dim, dims.lin_v_dim},
                        {dims.lin_v_heads * dims.lin_k_dim * dims.lin_v_dim, dims.lin_k_dim * dims.lin_v_dim, dims.lin_v_dim, 1}};
    MemRef<uint16_t, 3> rv{conv.data(), conv.data(), 0, {dims.linear_layers(), dims.conv_kernel - 1, dims.qkv_dim()},
                           {(dims.conv_kernel - 1) * dims.qkv_dim(), dims.qkv_dim(), 1}};
    MemRef<float, 2> ro{logits.data(), logits.data(), 0, {1, dims.vocab}, {dims.vocab, 1}};
    EntryFn fn = sequence > 1 ? prefill : decode;
    fn(&rt, &rc, &rs, reinterpret_cast<void *>(start), reinterpret_cast<void *>(cache_length), &ra, &rk, &rd, &rv, &ro);
    return true;
  }
};

inline int64_t argmax(const std::vector<float> &values) {
  return static_cast<int64_t>(std::max_element(values.begin(), values.end()) - values.begin());
}

} // namespace host
} // namespace llmcp_b200
