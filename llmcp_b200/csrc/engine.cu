#include "engine.h"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>

#include "kernels.h"
#include "tp_comm.h"

namespace llmcp_b200 {

namespace {

size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// After a decode step of the device-resident loop: record the token, make it the next input,
// advance the position and stage the rotary rows of the new position.
__global__ void advance_kernel(const int64_t *__restrict__ next_token, int64_t *__restrict__ tokens,
                               int64_t *__restrict__ generated, int64_t *__restrict__ step,
                               int64_t *__restrict__ position, const float *__restrict__ cos_table,
                               const float *__restrict__ sin_table, float *__restrict__ cos_row,
                               float *__restrict__ sin_row, int rotary, int64_t capacity) {
  grid_dependency_sync();
  const int64_t p = *position + 1;
  const int i = threadIdx.x;
  if (p < capacity && i < rotary) {
    cos_row[i] = cos_table[p * rotary + i];
    sin_row[i] = sin_table[p * rotary + i];
  }
  __syncthreads();
  if (i == 0) {
    generated[*step] = *next_token;
    tokens[0] = *next_token;
    *step += 1;
    *position = p;
  }
}

int dtype_of(const TensorEntry &t) {
  if (t.dtype == "BF16")
    return kBF16;
  if (t.dtype == "F32")
    return kF32;
  throw std::runtime_error("tensor " + t.name + " has dtype " + t.dtype + ", expected BF16 or F32");
}

std::atomic<int> g_default_mode{-1};

} // namespace

// Names of the prefill GEMM forms (LLMCP_B200_GEMM): the value is 0 for the CUDA-core kernel, 1 for
// the cp.async-fed tcgen05 kernel, 2 + GemmForm for the TMA-fed ones.
int gemm_kind_from_name(const char *name) {
  const std::string kind = name ? name : "";
  if (kind == "dp4a")
    return 0;
  if (kind == "i8-cpasync")
    return 1;
  if (kind == "i8")
    return 2 + kGemmI8;
  if (kind == "i8x2")
    return 2 + kGemmI8Packed;
  if (kind == "f16")
    return 2 + kGemmF16;
  if (kind == "f16x2")
    return 2 + kGemmF16Packed;
  return kDefaultGemmKind;
}

int default_mode() {
  const int stored = g_default_mode.load();
  if (stored >= 0)
    return stored;
  if (const char *flag = std::getenv("LLMCP_B200_MODE"))
    return (std::string(flag) == "fast" || std::string(flag) == "1") ? kModeFast : kModeExact;
  return kModeExact;
}

void set_default_mode(int mode) { g_default_mode.store(mode == kModeFast ? kModeFast : kModeExact); }

void Engine::check(cudaError_t e, const char *what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

std::string Engine::tp_unsupported(const ModelDims &d, int size) {
  if (size < 1 || size > kTpMaxRanks)
    return "tensor parallel group size must be 1 .. 8";
  if (size == 1)
    return "";
  if (d.lin_k_heads % size || d.lin_v_heads % size || d.heads % size)
    return "head counts do not divide by the group size";
  if (d.kv_heads % size && size % d.kv_heads)
    return "KV heads neither divide by the group size nor divide it";
  if (d.hidden % (size * 8) || d.vocab % (size * 8))
    return "hidden / vocabulary rows do not split into whole groups of 8 rows";
  if (d.intermediate % (size * 128) || (d.lin_v_heads / size * d.lin_v_dim) % 128 || (d.heads / size * d.head_dim) % 128)
    return "a rank's share of intermediate / value / attention width must be a multiple of 128";
  return "";
}

size_t Engine::tp_slot_bytes(const ModelDims &d, int64_t max_tokens) {
  const size_t rows = static_cast<size_t>(std::max<int64_t>(1, max_tokens));
  const size_t widest = static_cast<size_t>(std::max({d.intermediate, d.value_dim(), d.attn_dim()}));
  const size_t quant = round_up(rows * widest, 256) + round_up(rows * (widest / 32) * 4, 256);
  const size_t rows_bf16 = round_up(rows * static_cast<size_t>(d.hidden) * 2, 256);
  const size_t logits = round_up(static_cast<size_t>(d.vocab) * 4, 256);
  return std::max({quant, rows_bf16, logits}) + 256;
}

Engine::Engine(const uint8_t *base, uint64_t file_bytes, const ModelDims &dims, int64_t capacity, int device, int mode,
               TpComm *tp, int64_t max_tokens, int batch)
    : dims_(dims), local_(dims), tp_(tp), max_tokens_(max_tokens), batch_(batch), capacity_(capacity), device_(device),
      mode_(mode < 0 ? default_mode() : (mode == kModeFast ? kModeFast : kModeExact)) {
  if (capacity <= 0)
    throw std::runtime_error("capacity must be positive");
  if (batch < 1 || batch > kArgmaxParts)
    throw std::runtime_error("batch must be 1 .. " + std::to_string(kArgmaxParts));
  if (batch > 1 && tp && tp->size() > 1)
    throw std::runtime_error("a batch of sequences and tensor parallelism are not offered together");
  if (tp && tp->size() > 1) {
    tp_rank_ = tp->rank();
    tp_size_ = tp->size();
    const std::string why = tp_unsupported(dims, tp_size_);
    if (!why.empty())
      throw std::runtime_error("tensor parallel: " + why);
    if (tp->slot_bytes() < tp_slot_bytes(dims, max_tokens))
      throw std::runtime_error("tensor parallel: the exchange slots are smaller than Engine::tp_slot_bytes()");
    local_.lin_k_heads = dims.lin_k_heads / tp_size_;
    local_.lin_v_heads = dims.lin_v_heads / tp_size_;
    local_.heads = dims.heads / tp_size_;
    if (dims.kv_heads >= tp_size_) {
      local_.kv_heads = dims.kv_heads / tp_size_;
      kv_head0_ = tp_rank_ * local_.kv_heads;
    } else { // more ranks than KV heads: every KV head lives on size / kv_heads ranks
      local_.kv_heads = 1;
      kv_head0_ = tp_rank_ / (tp_size_ / dims.kv_heads);
    }
  } else {
    tp_ = nullptr;
  }
  hidden_rows_ = dims.hidden / tp_size_;
  inter_rows_ = dims.intermediate / tp_size_;
  vocab_rows_ = dims.vocab / tp_size_;
  vocab_row0_ = tp_rank_ * vocab_rows_;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
    throw std::runtime_error("no CUDA device: this library has no CPU path");
  check(cudaSetDevice(device), "cudaSetDevice");
  // A constructor that throws does not run the destructor: everything acquired so far is released
  // here, so that a failed create leaves no device or pinned memory behind.
  try {
  check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
  // On for engines that hold a batch of sequences (their steps are GEMMs of a few tiles each), off
  // for a single sequence (see engine.h); the switch overrides both.
  concurrent_gemms_ = batch_ > 1;
  if (const char *flag = std::getenv("LLMCP_B200_CONCURRENT_GEMMS"))
    concurrent_gemms_ = std::atoi(flag) != 0;

  // Prefill GEMM form: decides which weight planes load_weights() builds.
  if (const char *flag = std::getenv("LLMCP_B200_GEMM")) {
    gemm_kind_ = gemm_kind_from_name(flag);
    use_tensor_cores_ = gemm_kind_ != 0;
  }
  Manifest manifest;
  const std::string error = parse_container(base, file_bytes, &manifest);
  if (!error.empty())
    throw std::runtime_error(error);
  if (manifest.quantization == "none")
    bf16_weights_ = true; // bf16 matrices (llmcp-pack --quant none): MatmulLoweringCommon.cpp:509-527
  else if (manifest.quantization != "q8_0")
    throw std::runtime_error("only q8_0 and unquantised arenas are supported (quantization = " + manifest.quantization + ")");
  if (bf16_weights_ && (tp_ || batch_ > 1))
    throw std::runtime_error("an unquantised (bf16) arena runs one sequence on one GPU");
  load_weights(base, manifest);

  const ModelDims &c = local_; // state is per rank: this rank's heads
  const size_t kv_bytes = static_cast<size_t>(c.full_layers()) * 2 * c.kv_heads * capacity_ * c.head_dim * 2;
  const size_t delta_bytes = static_cast<size_t>(c.linear_layers()) * c.lin_v_heads * c.lin_k_dim * c.lin_v_dim * 4;
  const size_t conv_bytes = static_cast<size_t>(c.linear_layers()) * (c.conv_kernel - 1) * c.qkv_dim() * 2;
  auto alloc = [&](size_t bytes) {
    void *p = nullptr;
    check(cudaMalloc(&p, std::max<size_t>(bytes, 256)), "cudaMalloc");
    allocations_.push_back(p);
    return p;
  };
  kv_seq_ = kv_bytes / 2, delta_seq_ = delta_bytes / 4, conv_seq_ = conv_bytes / 2;
  kv_ = static_cast<uint16_t *>(alloc(kv_bytes * batch_));
  delta_ = static_cast<float *>(alloc(delta_bytes * batch_));
  conv_ = static_cast<uint16_t *>(alloc(conv_bytes * batch_));
  if (batch_ > 1) {
    batch_logits_ = static_cast<float *>(alloc(static_cast<size_t>(batch_) * dims_.vocab * 4));
    batch_tokens_ = static_cast<int64_t *>(alloc(static_cast<size_t>(batch_) * 8));
  }
  cos_table_ = static_cast<float *>(alloc(static_cast<size_t>(capacity_) * c.rotary * 4));
  sin_table_ = static_cast<float *>(alloc(static_cast<size_t>(capacity_) * c.rotary * 4));
  {
    std::vector<float> cos_host(static_cast<size_t>(capacity_) * c.rotary), sin_host(cos_host.size());
    for (int64_t p = 0; p < capacity_; ++p)
      make_cos_sin(p, c.rotary, c.rope_theta, cos_host.data() + p * c.rotary, sin_host.data() + p * c.rotary);
    check(cudaMemcpy(cos_table_, cos_host.data(), cos_host.size() * 4, cudaMemcpyHostToDevice), "cos table");
    check(cudaMemcpy(sin_table_, sin_host.data(), sin_host.size() * 4, cudaMemcpyHostToDevice), "sin table");
  }
  final_hidden_ = static_cast<uint16_t *>(alloc(static_cast<size_t>(c.hidden) * 2));
  logits_ = static_cast<float *>(alloc(static_cast<size_t>(c.vocab) * 4));
  argmax_v_ = static_cast<float *>(alloc(kArgmaxParts * 4));
  argmax_i_ = static_cast<int64_t *>(alloc(kArgmaxParts * 8));
  argmax_pair_ = static_cast<uint8_t *>(alloc(16));
  // [next token (8 bytes) | GEMM status word (4)]: one copy brings both back after a call.
  uint8_t *results = static_cast<uint8_t *>(alloc(16));
  next_token_ = reinterpret_cast<int64_t *>(results);
  gemm_error_ = reinterpret_cast<int *>(results + 8);
  // The inputs of a one-token step, [position | token | cos row | sin row], in one block so
  // that one copy from the pinned packet of the same layout delivers them all.
  step_block_bytes_ = 16 + 2 * static_cast<size_t>(c.rotary) * 4;
  uint8_t *block = static_cast<uint8_t *>(alloc(step_block_bytes_));
  position_dev_ = reinterpret_cast<int64_t *>(block);
  dec_tokens_ = reinterpret_cast<int64_t *>(block + 8);
  dec_cos_ = reinterpret_cast<float *>(block + 16);
  dec_sin_ = dec_cos_ + c.rotary;
  step_dev_ = static_cast<int64_t *>(alloc(8));
  check(cudaMallocHost(&position_pinned_, step_block_bytes_), "cudaMallocHost");
  if (const char *flag = std::getenv("LLMCP_B200_NO_GRAPH"))
    use_graph_ = std::atoi(flag) == 0;
  if (const char *flag = std::getenv("LLMCP_B200_GEMV_FLAGS"))
    gemv_flags_ = std::atoi(flag);
  if (const char *flag = std::getenv("LLMCP_B200_FUSE_MIXER"))
    fuse_decode_mixer_ = std::atoi(flag);
  if (const char *flag = std::getenv("LLMCP_B200_TC_ATTENTION"))
    tc_prefill_attention_ = std::atoi(flag) != 0;
  if (const char *flag = std::getenv("LLMCP_B200_FUSE_SWIGLU"))
    fuse_swiglu_ = std::atoi(flag) != 0;
  if (const char *flag = std::getenv("LLMCP_B200_PREFETCH_NEXT"))
    prefetch_next_ = std::atoi(flag) != 0;
  check(cudaMemsetAsync(gemm_error_, 0, 4, stream_), "memset");
  generated_ = static_cast<int64_t *>(alloc(static_cast<size_t>(capacity_) * 8));
  check(cudaMallocHost(&logits_pinned_, static_cast<size_t>(c.vocab) * 4), "cudaMallocHost");
  check(cudaMallocHost(&token_pinned_, 16), "cudaMallocHost");
  reset_state();
  ensure_workspace(1, capacity_ - 1);
  // One throw-away decode step loads every kernel and applies its launch attributes, so that
  // nothing of that kind happens later while a graph is being captured.
  check(cudaMemsetAsync(tokens_, 0, 8, stream_), "warm-up");
  set_position(0);
  run(tokens_, 1, capacity_ - 1, cos_table_, sin_table_, 1);
  reset_state();
  check(cudaStreamSynchronize(stream_), "engine setup");
  } catch (...) {
    release();
    throw;
  }
}

Engine::~Engine() { release(); }

void Engine::release() noexcept {
  cudaSetDevice(device_);
  if (stream_)
    cudaStreamSynchronize(stream_);
  if (decode_graph_)
    cudaGraphExecDestroy(decode_graph_);
  decode_graph_ = nullptr;
  for (void *p : ws_allocations_)
    cudaFree(p);
  ws_allocations_.clear();
  for (void *p : allocations_)
    cudaFree(p);
  allocations_.clear();
  if (logits_pinned_)
    cudaFreeHost(logits_pinned_);
  if (token_pinned_)
    cudaFreeHost(token_pinned_);
  if (position_pinned_)
    cudaFreeHost(position_pinned_);
  logits_pinned_ = nullptr;
  token_pinned_ = nullptr;
  position_pinned_ = nullptr;
  drop_side_streams();
  if (stream_)
    cudaStreamDestroy(stream_);
  stream_ = nullptr;
  cudaGetLastError();
}

// The side streams exist only while a call of more than one token runs.
void Engine::make_side_streams() {
  for (int i = 0; i < kSideStreams; ++i) {
    if (!side_streams_[i])
      check(cudaStreamCreateWithFlags(&side_streams_[i], cudaStreamNonBlocking), "cudaStreamCreate");
    if (!join_events_[i])
      check(cudaEventCreateWithFlags(&join_events_[i], cudaEventDisableTiming), "cudaEventCreate");
  }
  if (!fork_event_)
    check(cudaEventCreateWithFlags(&fork_event_, cudaEventDisableTiming), "cudaEventCreate");
}

void Engine::drop_side_streams() noexcept {
  for (int i = 0; i < kSideStreams; ++i) {
    if (side_streams_[i])
      cudaStreamDestroy(side_streams_[i]); // returns at once; the stream goes when its work is done
    if (join_events_[i])
      cudaEventDestroy(join_events_[i]);
    side_streams_[i] = nullptr;
    join_events_[i] = nullptr;
  }
  if (fork_event_)
    cudaEventDestroy(fork_event_);
  fork_event_ = nullptr;
}

void Engine::validate_tokens(const int64_t *tokens, int64_t S) const {
  for (int64_t i = 0; i < S; ++i)
    if (tokens[i] < 0 || tokens[i] >= dims_.vocab)
      throw std::runtime_error("token id " + std::to_string(tokens[i]) + " at index " + std::to_string(i) +
                               " is outside the vocabulary [0, " + std::to_string(dims_.vocab) + ")");
}

void Engine::check_status() {
  const int status = *reinterpret_cast<const int *>(token_pinned_ + 1);
  if (status == 0)
    return;
  cudaMemsetAsync(gemm_error_, 0, 4, stream_);
  if (status & 2)
    throw std::runtime_error("a token id outside the vocabulary reached the embedding kernel");
  throw std::runtime_error("tensor-core GEMM: a bounded wait ran out (pipeline protocol error)");
}

// rms_norm of the forward (zero-centred weight, fused residual add and quantisation); the fast
// mode takes the tree-reduced kernel where the row length allows.
void Engine::rms_norm(const uint16_t *a, const uint16_t *b, int64_t S, const SmallTensor &w, uint16_t *sum_out, uint16_t *y) {
  const int H = static_cast<int>(dims_.hidden);
  // bf16 arena: the next linear reads the normalised rows themselves, not a quantised copy
  int8_t *q = bf16_weights_ ? nullptr : aq_;
  float *qs = bf16_weights_ ? nullptr : as_;
  if (bf16_weights_ && !y)
    y = xb_;
  if (mode_ == kModeFast) {
    const cudaError_t e = launch_rms_norm_fast(a, b, S, H, w.data, w.dtype, dims_.eps, 1, sum_out, y, q, qs, stream_);
    if (e == cudaSuccess)
      return;
    if (e != cudaErrorNotSupported)
      check(e, "rms_norm (fast)");
  }
  check(launch_rms_norm(a, b, S, H, w.data, w.dtype, dims_.eps, 1, sum_out, y, q, qs, stream_), "rms_norm");
}

void Engine::load_weights(const uint8_t *base, const Manifest &manifest) {
  const ModelDims &c = dims_;
  const ModelDims &m = local_;
  const std::string root = "model.language_model.";
  struct Rows { // rows [row0, row0 + rows) of a tensor's first dimension
    int64_t row0, rows;
  };
  const int G = tp_size_, r = tp_rank_;
  // One pool for all device weights; a staging buffer for the largest packed tensor.  A rank of a
  // tensor-parallel group keeps 1 / size of every projection (the tied table and the 2 x heads rows of
  // a / b stay whole), so the pool is sized by the rows actually taken.
  size_t pool_bytes = 0, staging_bytes = 0;
  auto q8_bytes = [&](size_t n, size_t k) {
    size_t bytes = round_up(n * k, 256) + round_up(n * (k / 32) * 2, 256);
    if (gemm_kind_ >= 1)
      bytes += round_up(n * (k / 32) * 4, 256); // f32 scales, row-major or block-major
    if (gemm_kind_ >= 2 + kGemmF16)
      bytes += round_up(n * k * 2, 256);
    return bytes;
  };
  for (const TensorEntry &t : manifest.tensors) {
    if (t.dtype == "Q8_0") {
      const size_t n = static_cast<size_t>(t.shape[0]), k = static_cast<size_t>(t.shape[1]);
      const bool whole = G == 1 || t.name.find("embed_tokens") != std::string::npos ||
                         t.name.find("in_proj_a") != std::string::npos || t.name.find("in_proj_b") != std::string::npos;
      size_t rows = whole ? n : n / G + 8;
      if (!whole && (t.name.find("k_proj") != std::string::npos || t.name.find("v_proj") != std::string::npos))
        rows = static_cast<size_t>(m.kv_dim()); // KV heads are duplicated when the group is larger than their number
      pool_bytes += q8_bytes(rows, k);
      staging_bytes = std::max<size_t>(staging_bytes, t.size);
    } else {
      pool_bytes += round_up(t.size, 256);
    }
  }
  uint8_t *pool = nullptr, *staging = nullptr;
  check(cudaMalloc(&pool, pool_bytes), "cudaMalloc(weights)");
  allocations_.push_back(pool);
  check(cudaMalloc(&staging, std::max<size_t>(staging_bytes, 256)), "cudaMalloc(staging)");
  allocations_.push_back(staging); // released with the rest if loading throws
  size_t cursor = 0;
  auto take = [&](size_t bytes) {
    uint8_t *p = pool + cursor;
    cursor += round_up(bytes, 256);
    if (cursor > pool_bytes)
      throw std::runtime_error("weight pool overflow");
    return p;
  };

  // A Q8 tensor [rows, cols] of which this rank keeps the given row ranges (whole 8-row groups), in
  // that order.  A range is a contiguous byte range of the packed records (group-major layout).
  auto q8 = [&](const std::string &name, int64_t rows, int64_t cols, std::vector<Rows> keep = {}) {
    const TensorEntry *t = manifest.find(name);
    if (!t)
      throw std::runtime_error("missing tensor " + name);
    if (bf16_weights_) { // the matrix as it is in the arena
      if (t->dtype != "BF16" || t->shape.size() != 2 || t->shape[0] != rows || t->shape[1] != cols)
        throw std::runtime_error("tensor " + name + " is not BF16 [" + std::to_string(rows) + ", " + std::to_string(cols) + "]");
      Q8Weight w;
      w.N = static_cast<int>(rows);
      w.K = static_cast<int>(cols);
      uint8_t *dst = take(static_cast<size_t>(rows) * cols * 2);
      check(cudaMemcpyAsync(dst, base + t->offset, static_cast<size_t>(rows) * cols * 2, cudaMemcpyHostToDevice, stream_), "upload weights");
      w.bf = reinterpret_cast<const uint16_t *>(dst);
      return w;
    }
    if (t->dtype != "Q8_0" || t->shape.size() != 2 || t->shape[0] != rows || t->shape[1] != cols)
      throw std::runtime_error("tensor " + name + " is not Q8_0 [" + std::to_string(rows) + ", " +
                               std::to_string(cols) + "]");
    if (keep.empty())
      keep.push_back({0, rows});
    int64_t kept = 0;
    for (const Rows &range : keep) {
      if (range.row0 % 8 || range.rows % 8 || range.row0 + range.rows > rows)
        throw std::runtime_error("tensor " + name + ": a rank's rows must be whole groups of 8");
      kept += range.rows;
    }
    const int64_t nb = cols / 32;
    Q8Weight w;
    w.N = static_cast<int>(kept);
    w.K = static_cast<int>(cols);
    w.q = reinterpret_cast<int8_t *>(take(static_cast<size_t>(kept) * cols));
    w.d = reinterpret_cast<uint16_t *>(take(static_cast<size_t>(kept) * nb * 2));
    if (gemm_kind_ == 1)
      w.d32 = reinterpret_cast<float *>(take(static_cast<size_t>(kept) * nb * 4));
    int64_t at = 0;
    size_t staged = 0;
    for (const Rows &range : keep) {
      const size_t offset = static_cast<size_t>(range.row0 / 4) * nb * kRecordBytes;
      const size_t bytes = static_cast<size_t>(range.rows / 4) * nb * kRecordBytes;
      check(cudaMemcpyAsync(staging + staged, base + t->offset + offset, bytes, cudaMemcpyHostToDevice, stream_), "upload weights");
      launch_repack_p4(staging + staged, range.rows, cols, w.q + at * cols, w.d + at * nb, w.d32 ? w.d32 + at * nb : nullptr, stream_);
      check(cudaGetLastError(), "repack");
      at += range.rows;
      staged += bytes;
    }
    if (gemm_kind_ >= 2) { // TMA-fed forms: block-major scales, and for the f16 forms the f16-valued plane
      w.d32t = reinterpret_cast<float *>(take(static_cast<size_t>(kept) * nb * 4));
      if (gemm_kind_ >= 2 + kGemmF16) {
        w.h = take(static_cast<size_t>(kept) * cols * 2);
        launch_weights_to_f16(w.q, w.d, kept, static_cast<int>(cols), w.h, w.d32t, stream_);
      } else {
        launch_scales_block_major(w.d, 1, kept, static_cast<int>(cols), kept, w.d32t, stream_);
      }
      check(cudaGetLastError(), "GEMM planes");
    }
    return w;
  };
  // A BF16 / F32 tensor of which the given ranges of its first dimension are kept (`inner`
  // elements per index of that dimension).
  auto small = [&](const std::string &name, int64_t elements, std::vector<Rows> keep = {}, int64_t inner = 1) {
    const TensorEntry *t = manifest.find(name);
    if (!t)
      throw std::runtime_error("missing tensor " + name);
    SmallTensor st;
    st.dtype = dtype_of(*t);
    uint64_t count = 1;
    for (int64_t d : t->shape)
      count *= static_cast<uint64_t>(d);
    if (static_cast<int64_t>(count) != elements)
      throw std::runtime_error("tensor " + name + " has " + std::to_string(count) + " elements, expected " +
                               std::to_string(elements));
    const size_t width = st.dtype == kBF16 ? 2 : 4;
    if (keep.empty())
      keep.push_back({0, elements / inner});
    size_t kept = 0;
    for (const Rows &range : keep)
      kept += static_cast<size_t>(range.rows) * inner * width;
    st.data = take(kept);
    size_t at = 0;
    for (const Rows &range : keep) {
      const size_t bytes = static_cast<size_t>(range.rows) * inner * width;
      check(cudaMemcpyAsync(static_cast<uint8_t *>(st.data) + at, base + t->offset + static_cast<size_t>(range.row0) * inner * width,
                            bytes, cudaMemcpyHostToDevice, stream_), "upload tensor");
      at += bytes;
    }
    return st;
  };

  embed_ = q8(root + "embed_tokens.weight", c.vocab, c.hidden);
  lm_head_ = embed_; // the tied table's rows [vocab_row0_, + vocab_rows_) for the vocabulary projection
  lm_head_.N = static_cast<int>(vocab_rows_);
  if (!bf16_weights_) {
    lm_head_.q = embed_.q + vocab_row0_ * c.hidden;
    lm_head_.d = embed_.d + vocab_row0_ * (c.hidden / 32);
  }
  if (embed_.d32)
    lm_head_.d32 = embed_.d32 + vocab_row0_ * (c.hidden / 32);
  if (G > 1)
    lm_head_.h = nullptr, lm_head_.d32t = nullptr; // block-major planes cannot be sliced by rows
  // This rank's rows of the fused q | k | v projection, of the convolution over them and of the
  // per-head parameters: its key heads' q and k channels, then its value heads' channels.
  const int64_t qk = m.lin_k_heads * c.lin_k_dim, vd = m.lin_v_heads * c.lin_v_dim;
  const std::vector<Rows> qkv_rows = {{r * qk, qk}, {c.lin_k_heads * c.lin_k_dim + r * qk, qk},
                                      {2 * c.lin_k_heads * c.lin_k_dim + r * vd, vd}};
  const std::vector<Rows> v_heads = {{r * m.lin_v_heads, m.lin_v_heads}};
  layers_.resize(static_cast<size_t>(c.layers));
  for (int64_t l = 0; l < c.layers; ++l) {
    LayerWeights &L = layers_[static_cast<size_t>(l)];
    const std::string p = root + "layers." + std::to_string(l) + ".";
    L.full = c.is_full(l);
    L.input_norm = small(p + "input_layernorm.weight", c.hidden);
    L.post_norm = small(p + "post_attention_layernorm.weight", c.hidden);
    if (!L.full) {
      L.qkv = q8(p + "linear_attn.in_proj_qkv.weight", c.qkv_dim(), c.hidden, qkv_rows);
      L.z = q8(p + "linear_attn.in_proj_z.weight", c.value_dim(), c.hidden, {{r * vd, vd}});
      L.a = q8(p + "linear_attn.in_proj_a.weight", c.lin_v_heads, c.hidden);
      L.b = q8(p + "linear_attn.in_proj_b.weight", c.lin_v_heads, c.hidden);
      L.conv = small(p + "linear_attn.conv1d.weight", c.qkv_dim() * c.conv_kernel, qkv_rows, c.conv_kernel);
      if (L.conv.dtype != kBF16)
        throw std::runtime_error("conv1d.weight must be BF16");
      L.dt_bias = small(p + "linear_attn.dt_bias", c.lin_v_heads, v_heads);
      L.a_log = small(p + "linear_attn.A_log", c.lin_v_heads, v_heads);
      L.lin_norm = small(p + "linear_attn.norm.weight", c.lin_v_dim);
      L.out_proj = q8(p + "linear_attn.out_proj.weight", c.hidden, c.value_dim(), {{r * hidden_rows_, hidden_rows_}});
    } else {
      L.q_proj = q8(p + "self_attn.q_proj.weight", c.q_out(), c.hidden, {{r * m.q_out(), m.q_out()}});
      L.k_proj = q8(p + "self_attn.k_proj.weight", c.kv_dim(), c.hidden, {{kv_head0_ * c.head_dim, m.kv_dim()}});
      L.v_proj = q8(p + "self_attn.v_proj.weight", c.kv_dim(), c.hidden, {{kv_head0_ * c.head_dim, m.kv_dim()}});
      L.o_proj = q8(p + "self_attn.o_proj.weight", c.hidden, c.attn_dim(), {{r * hidden_rows_, hidden_rows_}});
      L.q_norm = small(p + "self_attn.q_norm.weight", c.head_dim);
      L.k_norm = small(p + "self_attn.k_norm.weight", c.head_dim);
      if (L.q_norm.dtype != kBF16 || L.k_norm.dtype != kBF16)
        throw std::runtime_error("q_norm / k_norm must be BF16");
    }
    L.gate = q8(p + "mlp.gate_proj.weight", c.intermediate, c.hidden, {{r * inter_rows_, inter_rows_}});
    L.up = q8(p + "mlp.up_proj.weight", c.intermediate, c.hidden, {{r * inter_rows_, inter_rows_}});
    L.down = q8(p + "mlp.down_proj.weight", c.hidden, c.intermediate, {{r * hidden_rows_, hidden_rows_}});
  }
  final_norm_ = small(root + "norm.weight", c.hidden);
  check(cudaStreamSynchronize(stream_), "weight upload");
  allocations_.pop_back();
  cudaFree(staging);
}

void Engine::select_sequence(int sequence) {
  if (sequence < 0 || sequence >= batch_)
    throw std::runtime_error("sequence " + std::to_string(sequence) + " outside the batch of " + std::to_string(batch_));
  sequence_ = sequence;
}

// Clears the state of every sequence.
void Engine::reset_state() {
  check(cudaMemsetAsync(kv_, 0, kv_seq_ * 2 * batch_, stream_), "memset");
  check(cudaMemsetAsync(delta_, 0, delta_seq_ * 4 * batch_, stream_), "memset");
  check(cudaMemsetAsync(conv_, 0, conv_seq_ * 2 * batch_, stream_), "memset");
}

void Engine::upload_state(const uint16_t *kv, const float *delta, const uint16_t *conv) {
  check(cudaMemcpyAsync(kv_ + sequence_ * kv_seq_, kv, kv_seq_ * 2, cudaMemcpyHostToDevice, stream_), "upload kv");
  check(cudaMemcpyAsync(delta_ + sequence_ * delta_seq_, delta, delta_seq_ * 4, cudaMemcpyHostToDevice, stream_), "upload delta");
  check(cudaMemcpyAsync(conv_ + sequence_ * conv_seq_, conv, conv_seq_ * 2, cudaMemcpyHostToDevice, stream_), "upload conv");
  check(cudaStreamSynchronize(stream_), "upload state");
}

void Engine::download_state(uint16_t *kv, float *delta, uint16_t *conv) {
  if (kv)
    check(cudaMemcpyAsync(kv, kv_ + sequence_ * kv_seq_, kv_seq_ * 2, cudaMemcpyDeviceToHost, stream_), "download kv");
  if (delta)
    check(cudaMemcpyAsync(delta, delta_ + sequence_ * delta_seq_, delta_seq_ * 4, cudaMemcpyDeviceToHost, stream_), "download delta");
  if (conv)
    check(cudaMemcpyAsync(conv, conv_ + sequence_ * conv_seq_, conv_seq_ * 2, cudaMemcpyDeviceToHost, stream_), "download conv");
  check(cudaStreamSynchronize(stream_), "download state");
}

void Engine::ensure_workspace(int64_t S, int64_t position) {
  const ModelDims &c = dims_;
  const ModelDims &m = local_;
  // sized for tokens of one sequence and for one token each of S sequences (a batched step)
  size_t need_attn =
      std::max(attn_scratch_bytes(S, static_cast<int>(m.heads), static_cast<int>(m.head_dim), position),
               attn_fast_scratch_bytes(static_cast<int>(m.heads), static_cast<int>(m.head_dim), position + S - 1,
                                       static_cast<int>(std::min<int64_t>(S, batch_))));
  if (attention_prefill_tc_supported(static_cast<int>(m.heads), static_cast<int>(m.kv_heads), static_cast<int>(m.head_dim)))
    need_attn = std::max(need_attn, attention_prefill_tc_scratch_bytes(S, static_cast<int>(m.heads), static_cast<int>(m.kv_heads), capacity_));
  if (S <= ws_tokens_ && need_attn <= attn_scratch_bytes_)
    return;
  if (tp_ && S > max_tokens_)
    throw std::runtime_error("tensor parallel: a call of " + std::to_string(S) + " tokens exceeds the " +
                             std::to_string(max_tokens_) + " the exchange slots were sized for");
  check(cudaStreamSynchronize(stream_), "workspace resize");
  if (decode_graph_) { // the captured step points into the buffers that are about to move
    cudaGraphExecDestroy(decode_graph_);
    decode_graph_ = nullptr;
  }
  for (void *p : ws_allocations_)
    cudaFree(p);
  ws_allocations_.clear();
  const int64_t rows = std::max(S, ws_tokens_);
  auto alloc = [&](size_t bytes) {
    void *p = nullptr;
    check(cudaMalloc(&p, std::max<size_t>(bytes, 256)), "cudaMalloc(workspace)");
    ws_allocations_.push_back(p);
    return p;
  };
  const size_t r = static_cast<size_t>(rows);
  const size_t max_k = static_cast<size_t>(std::max({c.hidden, c.intermediate, c.value_dim(), c.attn_dim()}));
  tokens_ = static_cast<int64_t *>(alloc(r * 8));
  cos_ = static_cast<float *>(alloc(r * c.rotary * 4));
  sin_ = static_cast<float *>(alloc(r * c.rotary * 4));
  hidden_[0] = static_cast<uint16_t *>(alloc(r * c.hidden * 2));
  hidden_[1] = static_cast<uint16_t *>(alloc(r * c.hidden * 2));
  branch_ = static_cast<uint16_t *>(alloc(r * c.hidden * 2));
  mlp_out_ = static_cast<uint16_t *>(alloc(r * c.hidden * 2));
  xb_ = bf16_weights_ ? static_cast<uint16_t *>(alloc(r * max_k * 2)) : nullptr;
  aq_ = static_cast<int8_t *>(alloc(r * max_k));
  as_ = static_cast<float *>(alloc(r * (max_k / 32) * 4));
  ah_ = nullptr;
  ast_ = nullptr;
  if (gemm_kind_ >= 2 && rows > 1) {
    if (gemm_kind_ >= 2 + kGemmF16)
      ah_ = alloc(r * max_k * 2);
    ast_ = static_cast<float *>(alloc(static_cast<size_t>(gemm_tc16_scale_pitch(rows)) * (max_k / 32) * 4));
  }
  // Mixer and MLP intermediates hold this rank's heads / rows only; a and b are whole.
  qkv_ = static_cast<uint16_t *>(alloc(r * m.qkv_dim() * 2));
  z_ = static_cast<uint16_t *>(alloc(r * m.value_dim() * 2));
  a_ = static_cast<uint16_t *>(alloc(r * c.lin_v_heads * 2));
  b_ = static_cast<uint16_t *>(alloc(r * c.lin_v_heads * 2));
  convd_ = static_cast<uint16_t *>(alloc(r * m.qkv_dim() * 2));
  gdn_ = static_cast<uint16_t *>(alloc(r * m.value_dim() * 2));
  qg_ = static_cast<uint16_t *>(alloc(r * m.q_out() * 2));
  k_ = static_cast<uint16_t *>(alloc(r * m.kv_dim() * 2));
  v_ = static_cast<uint16_t *>(alloc(r * m.kv_dim() * 2));
  attn_ = static_cast<uint16_t *>(alloc(r * m.attn_dim() * 2));
  gate_ = static_cast<uint16_t *>(alloc(r * inter_rows_ * 2));
  up_ = static_cast<uint16_t *>(alloc(r * inter_rows_ * 2));
  gdn_scratch_ = static_cast<float *>(alloc(
      gdn_scratch_floats(rows, static_cast<int>(m.lin_k_heads), static_cast<int>(m.lin_v_heads), static_cast<int>(m.lin_k_dim)) * 4));
  attn_scratch_bytes_ = std::max(need_attn, attn_scratch_bytes_);
  attn_scratch_ = alloc(attn_scratch_bytes_);
  ws_tokens_ = rows;
}

// Tensor parallel: the rows left in aq_ / as_ hold this rank's k_local columns; every rank gets all of
// them (in a slot of the exchange buffer).  With one rank the local buffers are the result.
void Engine::gather_quant(int64_t S, int64_t k_local, const int8_t **q, const float **s, const int8_t *src_q,
                          const float *src_s) {
  if (!src_q)
    src_q = aq_, src_s = as_;
  if (!tp_) {
    *q = src_q;
    *s = src_s;
    return;
  }
  const int slot = exchange_++ & 1;
  const size_t q_bytes = round_up(static_cast<size_t>(S) * k_local * tp_size_, 256);
  const TpSegment segments[2] = {{src_q, static_cast<size_t>(k_local), static_cast<size_t>(S), 0},
                                 {src_s, static_cast<size_t>(k_local / 32 * 4), static_cast<size_t>(S), q_bytes}};
  check(tp_->all_gather(segments, 2, slot, gemm_error_, stream_), "all-gather (quantised rows)");
  launches_ += 1;
  *q = reinterpret_cast<const int8_t *>(tp_->slot(slot));
  *s = reinterpret_cast<const float *>(tp_->slot(slot) + q_bytes);
}

// The same for bf16 rows of n_local columns per rank.
const uint16_t *Engine::gather_rows(const uint16_t *src, int64_t S, int64_t n_local) {
  if (!tp_)
    return src;
  const int slot = exchange_++ & 1;
  const TpSegment segment = {src, static_cast<size_t>(n_local) * 2, static_cast<size_t>(S), 0};
  check(tp_->all_gather(&segment, 1, slot, gemm_error_, stream_), "all-gather (rows)");
  launches_ += 1;
  return reinterpret_cast<const uint16_t *>(tp_->slot(slot));
}

// Streams and events for independent GEMMs that share an input (Engine::side_streams_).
struct SideStreams {
  cudaStream_t *streams;
  cudaEvent_t fork, *joins;
  int count;
};

struct LinearJob {
  const Q8Weight *w;
  void *y;
  int y_dtype;
  int activation;
};

// Buffers of the f16-form GEMM input (null: not in use).
struct F16Planes {
  void *ah;
  float *ast;
  int form; // GemmForm, or -1: not a TMA-fed form
};

// The matrix and the scales of a projection, as ranges for the GEMV in front of it to ask for in L2.
static void add_weight(PrefetchList *list, const Q8Weight &w) {
  auto add = [&](const void *p, uint64_t bytes) {
    if (p && bytes && bytes <= 0xffffffffull && bytes % 16 == 0 && reinterpret_cast<uintptr_t>(p) % 16 == 0 &&
        list->count < kMaxPrefetchRanges) {
      list->ptr[list->count] = p;
      list->bytes[list->count] = static_cast<uint32_t>(bytes);
      ++list->count;
    }
  };
  add(w.q, static_cast<uint64_t>(w.N) * static_cast<uint64_t>(w.K));
  add(w.d, static_cast<uint64_t>(w.N) * static_cast<uint64_t>(w.K / 32) * 2);
}

static void run_linears(const F16Planes &planes, const int8_t *aq, const float *as, int64_t S, const LinearJob *jobs, int count,
                        cudaStream_t stream, uint64_t *launches, int flags, int *gemm_error = nullptr,
                        const uint16_t *xb = nullptr, int *status = nullptr, const SideStreams *side = nullptr,
                        const PrefetchList *next = nullptr) {
  if (jobs[0].w->bf) { // bf16 matrices: the input rows are bf16 (xb), one launch per matrix
    for (int i = 0; i < count; ++i) {
      const Q8Weight &w = *jobs[i].w;
      const cudaError_t e = S == 1 ? launch_gemv_bf16(xb, w.K, w.bf, w.N, jobs[i].y, jobs[i].y_dtype, jobs[i].activation, stream)
                                   : launch_gemm_bf16_tc(xb, static_cast<int>(S), w.K, w.bf, w.N, jobs[i].y, jobs[i].y_dtype,
                                                         jobs[i].activation, status, stream);
      if (e != cudaSuccess)
        throw std::runtime_error(std::string("bf16 linear: ") + cudaGetErrorString(e));
      *launches += 1;
    }
    return;
  }
  if (S == 1) {
    GemvJobs g{};
    g.count = count;
    g.flags = flags;
    g.error_flag = gemm_error;
    for (int i = 0; i < count; ++i) {
      g.job[i].wq = jobs[i].w->q;
      g.job[i].wd = jobs[i].w->d;
      g.job[i].y = jobs[i].y;
      g.job[i].N = jobs[i].w->N;
      g.job[i].activation = jobs[i].activation;
      g.job[i].y_dtype = jobs[i].y_dtype;
    }
    if (next)
      g.next = *next;
    cudaError_t e = launch_gemv_q8(aq, as, jobs[0].w->K, g, nullptr, stream);
    if (e != cudaSuccess)
      throw std::runtime_error(std::string("gemv: ") + cudaGetErrorString(e));
    *launches += 1;
    return;
  }
  const bool tma = gemm_error && planes.form >= 0 && planes.ast && jobs[0].w->d32t;
  const bool f16 = tma && planes.form >= kGemmF16;
  if (tma) { // the shared input once: scales block-major, and for the f16 forms the int8 values as f16
    if (f16)
      launch_act_to_f16(aq, as, S, jobs[0].w->K, planes.ah, planes.ast, stream);
    else
      launch_scales_block_major(as, 0, S, jobs[0].w->K, gemm_tc16_scale_pitch(S), planes.ast, stream);
    *launches += 1;
  }
  // Matrices that share the input are independent: the first stays on the stream, the others go to
  // side streams behind a fork event, and the stream waits for all of them afterwards.  Their tiles
  // then fill the SMs together instead of ending in a partly empty wave each.
  const bool fork = side && count > 1 && tma;
  if (fork && cudaEventRecord(side->fork, stream) != cudaSuccess)
    throw std::runtime_error("gemm: cudaEventRecord");
  for (int i = 0; i < count; ++i) {
    cudaStream_t stream_i = stream;
    if (fork && i > 0) {
      stream_i = side->streams[(i - 1) % side->count];
      if (i - 1 < side->count && cudaStreamWaitEvent(stream_i, side->fork, 0) != cudaSuccess)
        throw std::runtime_error("gemm: cudaStreamWaitEvent");
    }
    cudaError_t e =
        tma ? launch_gemm_q8_tma(planes.form, f16 ? planes.ah : static_cast<const void *>(aq), planes.ast, static_cast<int>(S),
                                 jobs[i].w->K, f16 ? jobs[i].w->h : static_cast<const void *>(jobs[i].w->q), jobs[i].w->d32t,
                                 jobs[i].w->N, jobs[i].y, jobs[i].y_dtype, jobs[i].activation, nullptr, gemm_error, stream_i)
        : gemm_error ? launch_gemm_q8_tc(aq, as, static_cast<int>(S), jobs[i].w->K, jobs[i].w->q, jobs[i].w->d32,
                                         jobs[i].w->N, jobs[i].y, jobs[i].y_dtype, jobs[i].activation, nullptr, gemm_error,
                                         stream)
                     : launch_gemm_q8_dp4a(aq, as, static_cast<int>(S), jobs[i].w->K, jobs[i].w->q, jobs[i].w->d,
                                           jobs[i].w->N, jobs[i].y, jobs[i].y_dtype, jobs[i].activation, nullptr, stream);
    if (e != cudaSuccess)
      throw std::runtime_error(std::string("gemm: ") + cudaGetErrorString(e));
    *launches += 1;
  }
  if (fork) {
    const int used = std::min(count - 1, side->count);
    for (int i = 0; i < used; ++i)
      if (cudaEventRecord(side->joins[i], side->streams[i]) != cudaSuccess || cudaStreamWaitEvent(stream, side->joins[i], 0) != cudaSuccess)
        throw std::runtime_error("gemm: joining the side streams failed");
  }
}

void Engine::set_position(int64_t position) {
  // The pinned word is reused: wait until an earlier copy has been consumed.
  check(cudaStreamSynchronize(stream_), "set_position");
  *position_pinned_ = position;
  check(cudaMemcpyAsync(position_dev_, position_pinned_, 8, cudaMemcpyHostToDevice, stream_), "position");
}

void Engine::decode_step() {
  if (!use_graph_) {
    run(dec_tokens_, 1, capacity_ - 1, dec_cos_, dec_sin_, 0);
    return;
  }
  if (!decode_graph_) {
    cudaGraph_t graph = nullptr;
    const uint64_t before = launches_;
    check(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeRelaxed), "begin capture");
    try {
      run(dec_tokens_, 1, capacity_ - 1, dec_cos_, dec_sin_, 0);
    } catch (...) {
      cudaStreamEndCapture(stream_, &graph);
      if (graph)
        cudaGraphDestroy(graph);
      throw;
    }
    check(cudaStreamEndCapture(stream_, &graph), "end capture");
    decode_graph_launches_ = launches_ - before;
    launches_ = before;
    check(cudaGraphInstantiate(&decode_graph_, graph, 0), "graph instantiate");
    cudaGraphDestroy(graph);
  }
  check(cudaGraphLaunch(decode_graph_, stream_), "graph launch");
  launches_ += decode_graph_launches_;
}

// First maximum over the ranks' {maximum, index} pairs: the largest value, the lowest index among
// equal values (what the host argmax of llmcp-benchmark.cpp:51-54 picks over the whole row).
__global__ void tp_argmax_merge_kernel(const uint8_t *__restrict__ pairs, int size, int64_t *__restrict__ out_index) {
  grid_dependency_sync();
  if (threadIdx.x != 0)
    return;
  float best = -INFINITY;
  int64_t index = INT64_MAX;
  for (int r = 0; r < size; ++r) {
    const float v = *reinterpret_cast<const float *>(pairs + 16 * r);
    const int64_t i = *reinterpret_cast<const int64_t *>(pairs + 16 * r + 8);
    if (v > best || (v == best && i < index)) {
      best = v;
      index = i;
    }
  }
  *out_index = index;
}

void Engine::run(const int64_t *tokens_dev, int64_t S, int64_t position, const float *cos_dev, const float *sin_dev,
                 int rows_from_position, bool rows_are_sequences) {
  const ModelDims &c = dims_;
  const ModelDims &m = local_; // this rank's heads
  const int H = static_cast<int>(c.hidden);
  if (rows_are_sequences && (S != batch_ || all_logits_ || tp_))
    throw std::runtime_error("a batched step takes one token of each of the engine's sequences");
  // One-token kernels serve a single token and a batch of single tokens; state of the selected
  // sequence, or of all of them side by side.
  const bool one_token = S == 1 || rows_are_sequences;
  const int sequences = rows_are_sequences ? static_cast<int>(S) : 1;
  uint16_t *kv_base = kv_ + (rows_are_sequences ? 0 : sequence_ * kv_seq_);
  float *delta_base = delta_ + (rows_are_sequences ? 0 : sequence_ * delta_seq_);
  uint16_t *conv_base = conv_ + (rows_are_sequences ? 0 : sequence_ * conv_seq_);
  if (S <= 0 || position < 0 || position + (rows_are_sequences ? 1 : S) > capacity_)
    throw std::runtime_error("sequence does not fit the cache: position " + std::to_string(position) + " + " +
                             std::to_string(rows_are_sequences ? 1 : S) + " > capacity " + std::to_string(capacity_));
  if (tp_ && all_logits_)
    throw std::runtime_error("all-position logits are not offered under tensor parallelism");
  ensure_workspace(S, position);
  exchange_ = 0;
  // bf16 arena: operators hand bf16 rows to the next linear (act_y) instead of int8 blocks (act_q, act_s)
  const bool bf = bf16_weights_;
  int8_t *act_q = bf ? nullptr : aq_;
  float *act_s = bf ? nullptr : as_;
  uint16_t *act_y = bf ? xb_ : nullptr;
  if (bf)
    check(launch_embedding_bf16(tokens_dev, S, H, c.vocab, embed_.bf, hidden_[0], gemm_error_, stream_), "embedding");
  else
    launch_embedding_q8(tokens_dev, S, H, c.vocab, embed_.q, embed_.d, hidden_[0], gemm_error_, stream_);
  launches_ += 1;
  const int gemv_flags = gemv_flags_ | (mode_ == kModeFast ? kGemvFast : 0);
  const F16Planes planes = {ah_, ast_, gemm_kind_ >= 2 ? gemm_kind_ - 2 : -1};
  int *gemm_status = use_tensor_cores_ ? gemm_error_ : nullptr;
  const bool use_side_streams = concurrent_gemms_ && S > 1 && !bf16_weights_;
  if (use_side_streams)
    make_side_streams();
  SideStreams side_streams = {side_streams_, fork_event_, join_events_, kSideStreams};
  const SideStreams *side = use_side_streams ? &side_streams : nullptr;
  // One token: every GEMV asks for the next GEMV's weights in L2 while it runs (PrefetchList in kernels.h).
  const bool prefetch_next = prefetch_next_ && S == 1 && !rows_are_sequences && !bf && !tp_;
  auto input_weights = [&](const LayerWeights &L, PrefetchList *list) {
    if (L.full) {
      add_weight(list, L.q_proj), add_weight(list, L.k_proj), add_weight(list, L.v_proj);
    } else {
      add_weight(list, L.qkv), add_weight(list, L.z), add_weight(list, L.a), add_weight(list, L.b);
    }
  };
  int cur = 0;
  const uint16_t *pending = nullptr; // the MLP output still to be added to the residual stream
  int64_t lin_index = 0, full_index = 0;
  for (int64_t l = 0; l < c.layers; ++l) {
    const LayerWeights &L = layers_[static_cast<size_t>(l)];
    if (pending) {
      rms_norm(hidden_[cur], pending, S, L.input_norm, hidden_[cur ^ 1], nullptr);
      cur ^= 1;
    } else {
      rms_norm(hidden_[cur], nullptr, S, L.input_norm, nullptr, nullptr);
    }
    launches_ += 1;
    const int8_t *mixer_q = nullptr; // the mixer's quantised output, all columns
    const float *mixer_s = nullptr;
    PrefetchList after_input{}, after_out{}, after_mlp{}, after_down{};
    if (prefetch_next) {
      add_weight(&after_input, L.full ? L.o_proj : L.out_proj);
      add_weight(&after_out, L.gate), add_weight(&after_out, L.up);
      add_weight(&after_mlp, L.down);
      if (l + 1 < c.layers)
        input_weights(layers_[static_cast<size_t>(l + 1)], &after_down);
    }
    if (!L.full) {
      const LinearJob jobs[4] = {{&L.qkv, qkv_, kBF16, kNone},
                                 {&L.z, z_, kBF16, kSilu},
                                 {&L.a, a_, kBF16, kNone},
                                 {&L.b, b_, kBF16, kSigmoid}};
      run_linears(planes, aq_, as_, S, jobs, 4, stream_, &launches_, gemv_flags, gemm_status, xb_, gemm_error_, side, &after_input);
      const int C = static_cast<int>(m.qkv_dim());
      uint16_t *conv_state = conv_base + lin_index * (c.conv_kernel - 1) * C;
      float *delta_state = delta_base + lin_index * m.lin_v_heads * c.lin_k_dim * c.lin_v_dim;
      const int nk = static_cast<int>(m.lin_k_heads), nv = static_cast<int>(m.lin_v_heads);
      const int dk = static_cast<int>(c.lin_k_dim), dv = static_cast<int>(c.lin_v_dim);
      // a and b are computed for all heads on every rank; this rank's heads start at head0.
      const int nv_all = static_cast<int>(c.lin_v_heads), head0 = tp_rank_ * nv;
      const GdnBatch strides = {static_cast<int64_t>(conv_seq_), nv_all, static_cast<int64_t>(delta_seq_)};
      if (one_token && fuse_decode_mixer_ && gdn_decode_supported(static_cast<int>(c.conv_kernel), nk, nv, dk, dv)) {
        const int single = fuse_decode_mixer_ >= 2 && gdn_decode_single_kernel_supported(static_cast<int>(c.conv_kernel), nk, nv, dk, dv);
        check(launch_gdn_decode(qkv_, static_cast<const uint16_t *>(L.conv.data), conv_state, static_cast<int>(c.conv_kernel),
                                a_ + head0, b_ + head0, L.a_log.data, L.a_log.dtype, L.dt_bias.data, L.dt_bias.dtype, delta_state,
                                nk, nv, dk, dv, 1, z_, L.lin_norm.data, L.lin_norm.dtype, c.eps, 1, gdn_scratch_, convd_, act_y,
                                act_q, act_s, stream_, sequences, &strides, single, mode_ == kModeFast ? 1 : 0), "gated_delta_net (decode)");
        launches_ += single ? 1 : 2;
      } else if (rows_are_sequences) {
        // Shapes the fused one-token kernels do not take: the general kernels, sequence by sequence.
        const int64_t V = m.value_dim();
        for (int64_t b = 0; b < S; ++b) {
          check(launch_causal_conv1d(qkv_ + b * C, static_cast<const uint16_t *>(L.conv.data), conv_state + b * conv_seq_, 1, C,
                                     static_cast<int>(c.conv_kernel), convd_ + b * C, stream_), "causal_conv1d");
          check(launch_gated_delta_net(convd_ + b * C, a_ + b * nv_all + head0, b_ + b * nv_all + head0, L.a_log.data, L.a_log.dtype,
                                       L.dt_bias.data, L.dt_bias.dtype, delta_state + b * delta_seq_, 1, nk, nv, dk, dv, 1,
                                       gdn_scratch_, gdn_ + b * V, stream_, nv_all), "gated_delta_net");
          launches_ += 4;
        }
        check(launch_gated_rms_norm(gdn_, z_, L.lin_norm.data, L.lin_norm.dtype, S, static_cast<int>(V), dv, c.eps, 1, nullptr, aq_,
                                    as_, stream_), "gated_rms_norm");
        launches_ += 1;
      } else {
        check(launch_causal_conv1d(qkv_, static_cast<const uint16_t *>(L.conv.data), conv_state, S, C,
                                   static_cast<int>(c.conv_kernel), convd_, stream_), "causal_conv1d");
        check(launch_gated_delta_net(convd_, a_ + head0, b_ + head0, L.a_log.data, L.a_log.dtype, L.dt_bias.data, L.dt_bias.dtype,
                                     delta_state, S, nk, nv, dk, dv, 1, gdn_scratch_, gdn_, stream_, nv_all, mode_ == kModeFast ? 1 : 0),
              "gated_delta_net");
        check(launch_gated_rms_norm(gdn_, z_, L.lin_norm.data, L.lin_norm.dtype, S, static_cast<int>(m.value_dim()), dv,
                                    c.eps, 1, act_y, act_q, act_s, stream_), "gated_rms_norm");
        launches_ += 5;
      }
      if (!bf)
        gather_quant(S, m.value_dim(), &mixer_q, &mixer_s);
      ++lin_index;
    } else {
      const LinearJob jobs[3] = {{&L.q_proj, qg_, kBF16, kNone}, {&L.k_proj, k_, kBF16, kNone}, {&L.v_proj, v_, kBF16, kNone}};
      run_linears(planes, aq_, as_, S, jobs, 3, stream_, &launches_, gemv_flags, gemm_status, xb_, gemm_error_, side, &after_input);
      uint16_t *cache = kv_base + full_index * 2 * m.kv_heads * capacity_ * c.head_dim;
      const int nh = static_cast<int>(m.heads), nkv = static_cast<int>(m.kv_heads), hd = static_cast<int>(c.head_dim);
      const int64_t cache_stride = rows_are_sequences ? static_cast<int64_t>(kv_seq_) : 0;
      if (mode_ == kModeFast && one_token && attention_decode_fast_supported(nh, nkv, hd)) {
        check(launch_attention_decode_fast(qg_, k_, v_, static_cast<const uint16_t *>(L.q_norm.data),
                                           static_cast<const uint16_t *>(L.k_norm.data), cos_dev, sin_dev, rows_from_position,
                                           cache, position_dev_, position, nh, nkv, hd, static_cast<int>(c.rotary), capacity_,
                                           attn_scratch_, attn_, act_q, act_s, stream_, sequences, cache_stride), "attention (fast)");
      } else if (mode_ == kModeFast && S > 1 && !rows_are_sequences && tc_prefill_attention_ &&
                 attention_prefill_tc_supported(nh, nkv, hd)) {
        check(launch_attention_prefill_tc(qg_, k_, v_, static_cast<const uint16_t *>(L.q_norm.data),
                                          static_cast<const uint16_t *>(L.k_norm.data), cos_dev, sin_dev, rows_from_position, cache,
                                          position_dev_, position, S, nh, nkv, hd, static_cast<int>(c.rotary), capacity_,
                                          attn_scratch_, attn_, act_q, act_s, gemm_error_, stream_), "attention (tensor cores)");
      } else {
        check(launch_attention(qg_, k_, v_, static_cast<const uint16_t *>(L.q_norm.data),
                               static_cast<const uint16_t *>(L.k_norm.data), cos_dev, sin_dev, rows_from_position, cache,
                               position_dev_, position, S, nh, nkv, hd, static_cast<int>(c.rotary), capacity_, attn_scratch_,
                               attn_, act_q, act_s, stream_, cache_stride), "attention");
      }
      launches_ += 3;
      if (!bf)
        gather_quant(S, m.attn_dim(), &mixer_q, &mixer_s);
      ++full_index;
    }
    // Output projection of the mixer: this rank's rows of the hidden vector, then all of them.
    const LinearJob out = {L.full ? &L.o_proj : &L.out_proj, branch_, kBF16, kNone};
    run_linears(planes, mixer_q, mixer_s, S, &out, 1, stream_, &launches_, gemv_flags, gemm_status, L.full ? attn_ : xb_, gemm_error_,
                nullptr, &after_out);
    const uint16_t *branch = gather_rows(branch_, S, hidden_rows_);
    rms_norm(hidden_[cur], branch, S, L.post_norm, hidden_[cur ^ 1], nullptr);
    cur ^= 1;
    const int8_t *mlp_q = nullptr;
    const float *mlp_s = nullptr;
    if (!bf && S == 1 && fuse_swiglu_ && L.gate.K == L.up.K && L.gate.N == L.up.N && gemv_swiglu_supported(L.gate.K, L.gate.N)) {
      // One token: both projections, the product and its quantisation in one launch.  The launch
      // reads the quantised input while it writes the quantised product, so the product goes to
      // the (otherwise unused) rows of the separate projections' outputs.
      int8_t *product_q = reinterpret_cast<int8_t *>(gate_);
      float *product_s = reinterpret_cast<float *>(up_);
      check(launch_gemv_q8_swiglu(aq_, as_, L.gate.K, L.gate.q, L.gate.d, L.up.q, L.up.d, L.gate.N, nullptr, product_q, product_s,
                                  gemv_flags, stream_, &after_mlp), "gate/up (one launch)");
      launches_ += 1;
      gather_quant(S, inter_rows_, &mlp_q, &mlp_s, product_q, product_s);
    } else {
      const LinearJob mlp[2] = {{&L.gate, gate_, kBF16, kSilu}, {&L.up, up_, kBF16, kNone}};
      run_linears(planes, aq_, as_, S, mlp, 2, stream_, &launches_, gemv_flags, gemm_status, xb_, gemm_error_, side);
      check(launch_pointwise(gate_, up_, S * inter_rows_, 1, act_y, act_q, act_s, stream_), "mul");
      launches_ += 2;
      if (!bf)
        gather_quant(S, inter_rows_, &mlp_q, &mlp_s);
    }
    const LinearJob down = {&L.down, mlp_out_, kBF16, kNone};
    run_linears(planes, mlp_q, mlp_s, S, &down, 1, stream_, &launches_, gemv_flags, gemm_status, xb_, gemm_error_, nullptr, &after_down);
    pending = gather_rows(mlp_out_, S, hidden_rows_);
  }
  if (all_logits_) {
    // Every position's logits, what the tensor-returning `llmcp_model` function computes
    // (ModelBuilder.cpp:406-438): final norm over all rows, then one S x vocab x hidden contraction.
    rms_norm(hidden_[cur], pending, S, final_norm_, nullptr, branch_);
    const LinearJob all = {&embed_, all_logits_, kF32, kNone};
    run_linears(planes, aq_, as_, S, &all, 1, stream_, &launches_, gemv_flags & kGemvOverlapPrevious,
                S > 1 ? gemm_status : nullptr, branch_, gemm_error_);
    launches_ += 1;
  }
  if (rows_are_sequences) {
    // Every row is a sequence's last position: final norm and vocabulary projection of all rows,
    // then one first maximum per row.
    rms_norm(hidden_[cur], pending, S, final_norm_, nullptr, nullptr);
    const LinearJob heads = {&embed_, batch_logits_, kF32, kNone};
    run_linears(planes, aq_, as_, S, &heads, 1, stream_, &launches_, gemv_flags & kGemvOverlapPrevious, gemm_status);
    launch_argmax(batch_logits_, c.vocab, argmax_v_, argmax_i_, 0, batch_tokens_, nullptr, stream_, static_cast<int>(S));
    launches_ += 3;
    check(cudaGetLastError(), "forward");
    if (use_side_streams)
      drop_side_streams();
    return;
  }
  // Final norm and vocabulary projection of the last position only (ModelBuilder.cpp:489-512).
  const uint16_t *last = hidden_[cur] + (S - 1) * H;
  rms_norm(last, pending ? pending + (S - 1) * H : nullptr, 1, final_norm_, nullptr, final_hidden_);
  float *logits_rows = logits_ + vocab_row0_; // this rank's rows of the logits
  const LinearJob head = {&lm_head_, logits_rows, kF32, kNone};
  run_linears(planes, aq_, as_, 1, &head, 1, stream_, &launches_, gemv_flags_ & kGemvOverlapPrevious, nullptr, final_hidden_, gemm_error_);
  if (!tp_) {
    launch_argmax(logits_, c.vocab, argmax_v_, argmax_i_, 0, next_token_, nullptr, stream_);
    launches_ += 3;
  } else {
    // The whole row for the host only when it is asked for (1 / size of it comes from each rank).
    if (gather_logits_) {
      const int slot = exchange_++ & 1;
      const TpSegment segment = {logits_rows, static_cast<size_t>(vocab_rows_) * 4, 1, 0};
      check(tp_->all_gather(&segment, 1, slot, gemm_error_, stream_), "all-gather (logits)");
      check(cudaMemcpyAsync(logits_, tp_->slot(slot), static_cast<size_t>(c.vocab) * 4, cudaMemcpyDeviceToDevice, stream_), "logits");
      launches_ += 1;
    }
    // This rank's first maximum with its global index, then the first maximum over the ranks.  The
    // step's last exchange has a slot of its own, so that the next step's first one never follows
    // it into the same slot.
    launch_argmax(logits_rows, vocab_rows_, argmax_v_, argmax_i_, vocab_row0_, reinterpret_cast<int64_t *>(argmax_pair_ + 8),
                  reinterpret_cast<float *>(argmax_pair_), stream_);
    const TpSegment pair = {argmax_pair_, 16, 1, 0};
    check(tp_->all_gather(&pair, 1, 2, gemm_error_, stream_), "all-gather (argmax)");
    launch_chained(tp_argmax_merge_kernel, dim3(1), dim3(32), 0, stream_, tp_->slot(2), tp_size_, next_token_);
    launches_ += 6;
  }
  check(cudaGetLastError(), "forward");
  if (use_side_streams)
    drop_side_streams();
}

int64_t Engine::forward_host(const int64_t *tokens, int64_t S, int64_t position, const float *cos, const float *sin,
                             float *logits_host) {
  const ModelDims &c = dims_;
  check(cudaSetDevice(device_), "cudaSetDevice");
  if (S <= 0 || position < 0 || position + S > capacity_)
    throw std::runtime_error("sequence does not fit the cache");
  validate_tokens(tokens, S); // before any copy or launch
  if (tp_ && gather_logits_ != (logits_host != nullptr)) {
    // Whether the whole logits row is assembled is part of the captured step.
    gather_logits_ = logits_host != nullptr;
    check(cudaStreamSynchronize(stream_), "forward");
    if (decode_graph_)
      cudaGraphExecDestroy(decode_graph_);
    decode_graph_ = nullptr;
  }
  ensure_workspace(S, position);
  const size_t row_bytes = static_cast<size_t>(c.rotary) * 4;
  if (S == 1) {
    // One packet, one copy: position, token and the two rotary rows.
    check(cudaStreamSynchronize(stream_), "forward"); // the pinned packet is reused
    uint8_t *packet = reinterpret_cast<uint8_t *>(position_pinned_);
    std::memcpy(packet, &position, 8);
    std::memcpy(packet + 8, tokens, 8);
    size_t bytes = 16;
    if (cos && sin) {
      std::memcpy(packet + 16, cos, row_bytes);
      std::memcpy(packet + 16 + row_bytes, sin, row_bytes);
      bytes = step_block_bytes_;
    }
    check(cudaMemcpyAsync(position_dev_, packet, bytes, cudaMemcpyHostToDevice, stream_), "step inputs");
    if (!(cos && sin)) {
      check(cudaMemcpyAsync(dec_cos_, cos_table_ + position * c.rotary, row_bytes, cudaMemcpyDeviceToDevice, stream_), "cos");
      check(cudaMemcpyAsync(dec_sin_, sin_table_ + position * c.rotary, row_bytes, cudaMemcpyDeviceToDevice, stream_), "sin");
    }
    decode_step();
  } else {
    set_position(position);
    check(cudaMemcpyAsync(tokens_, tokens, static_cast<size_t>(S) * 8, cudaMemcpyHostToDevice, stream_), "tokens");
    if (cos && sin) {
      check(cudaMemcpyAsync(cos_, cos, static_cast<size_t>(S) * row_bytes, cudaMemcpyHostToDevice, stream_), "cos");
      check(cudaMemcpyAsync(sin_, sin, static_cast<size_t>(S) * row_bytes, cudaMemcpyHostToDevice, stream_), "sin");
    } else {
      check(cudaMemcpyAsync(cos_, cos_table_ + position * c.rotary, static_cast<size_t>(S) * row_bytes, cudaMemcpyDeviceToDevice, stream_), "cos");
      check(cudaMemcpyAsync(sin_, sin_table_ + position * c.rotary, static_cast<size_t>(S) * row_bytes, cudaMemcpyDeviceToDevice, stream_), "sin");
    }
    run(tokens_, S, position, cos_, sin_, 0);
  }
  if (logits_host)
    check(cudaMemcpyAsync(logits_pinned_, logits_, static_cast<size_t>(c.vocab) * 4, cudaMemcpyDeviceToHost, stream_), "logits");
  check(cudaMemcpyAsync(token_pinned_, next_token_, 16, cudaMemcpyDeviceToHost, stream_), "argmax and GEMM status");
  check(cudaStreamSynchronize(stream_), "forward");
  check_status();
  if (logits_host)
    std::memcpy(logits_host, logits_pinned_, static_cast<size_t>(c.vocab) * 4);
  return *token_pinned_;
}

void Engine::forward_all_host(const int64_t *tokens, int64_t S, int64_t position, float *logits_host) {
  const ModelDims &c = dims_;
  check(cudaSetDevice(device_), "cudaSetDevice");
  if (S <= 0 || position < 0 || position + S > capacity_)
    throw std::runtime_error("sequence does not fit the cache");
  if (!logits_host)
    throw std::runtime_error("forward_all needs a logits buffer of S x vocab floats");
  validate_tokens(tokens, S);
  ensure_workspace(S, position);
  const size_t bytes = static_cast<size_t>(S) * c.vocab * sizeof(float);
  float *device_rows = nullptr;
  check(cudaMalloc(&device_rows, bytes), "cudaMalloc(all-position logits)");
  try {
    set_position(position);
    check(cudaMemcpyAsync(tokens_, tokens, static_cast<size_t>(S) * 8, cudaMemcpyHostToDevice, stream_), "tokens");
    const size_t row_bytes = static_cast<size_t>(c.rotary) * 4;
    check(cudaMemcpyAsync(cos_, cos_table_ + position * c.rotary, static_cast<size_t>(S) * row_bytes, cudaMemcpyDeviceToDevice, stream_), "cos");
    check(cudaMemcpyAsync(sin_, sin_table_ + position * c.rotary, static_cast<size_t>(S) * row_bytes, cudaMemcpyDeviceToDevice, stream_), "sin");
    all_logits_ = device_rows;
    run(tokens_, S, position, cos_, sin_, 0);
    all_logits_ = nullptr;
    check(cudaMemcpyAsync(logits_host, device_rows, bytes, cudaMemcpyDeviceToHost, stream_), "all-position logits");
    check(cudaMemcpyAsync(token_pinned_, next_token_, 16, cudaMemcpyDeviceToHost, stream_), "argmax and GEMM status");
    check(cudaStreamSynchronize(stream_), "forward_all");
  } catch (...) {
    all_logits_ = nullptr;
    cudaStreamSynchronize(stream_);
    cudaFree(device_rows);
    throw;
  }
  cudaFree(device_rows);
  check_status();
}

namespace {

// After a batched step: every sequence's argmax becomes its next input, is recorded, and the
// common position advances.
__global__ void advance_batch_kernel(const int64_t *__restrict__ next, int64_t *__restrict__ tokens, int64_t *__restrict__ generated,
                                     int64_t *__restrict__ step, int64_t *__restrict__ position, int batch) {
  grid_dependency_sync();
  const int b = threadIdx.x;
  const int64_t at = *step;
  if (b < batch) {
    tokens[b] = next[b];
    generated[at * batch + b] = next[b];
  }
  __syncthreads();
  if (b == 0) {
    *step = at + 1;
    *position += 1;
  }
}

} // namespace

void Engine::decode_batch(const int64_t *tokens_host, int64_t position, float *logits_host, int64_t *argmax_host) {
  check(cudaSetDevice(device_), "cudaSetDevice");
  if (batch_ < 2)
    throw std::runtime_error("decode_batch needs an engine created with a batch of sequences");
  if (position < 0 || position + 1 > capacity_)
    throw std::runtime_error("position does not fit the cache");
  validate_tokens(tokens_host, batch_);
  ensure_workspace(batch_, position);
  set_position(position);
  check(cudaMemcpyAsync(tokens_, tokens_host, static_cast<size_t>(batch_) * 8, cudaMemcpyHostToDevice, stream_), "tokens");
  run(tokens_, batch_, position, cos_table_, sin_table_, 1, true);
  if (logits_host)
    check(cudaMemcpyAsync(logits_host, batch_logits_, static_cast<size_t>(batch_) * dims_.vocab * 4, cudaMemcpyDeviceToHost, stream_),
          "logits");
  if (argmax_host)
    check(cudaMemcpyAsync(argmax_host, batch_tokens_, static_cast<size_t>(batch_) * 8, cudaMemcpyDeviceToHost, stream_), "argmax");
  check(cudaMemcpyAsync(token_pinned_, next_token_, 16, cudaMemcpyDeviceToHost, stream_), "status");
  check(cudaStreamSynchronize(stream_), "decode_batch");
  check_status();
}

void Engine::generate_batch(const int64_t *first_tokens_host, int64_t position, int64_t steps, int64_t *out_tokens_host,
                            float *device_ms) {
  check(cudaSetDevice(device_), "cudaSetDevice");
  if (batch_ < 2)
    throw std::runtime_error("generate_batch needs an engine created with a batch of sequences");
  if (steps <= 0 || position < 0 || position + steps > capacity_)
    throw std::runtime_error("generation does not fit the cache");
  validate_tokens(first_tokens_host, batch_);
  ensure_workspace(batch_, position + steps - 1);
  set_position(position);
  check(cudaMemcpyAsync(tokens_, first_tokens_host, static_cast<size_t>(batch_) * 8, cudaMemcpyHostToDevice, stream_), "tokens");
  check(cudaMemsetAsync(step_dev_, 0, 8, stream_), "step counter");
  int64_t *generated = nullptr;
  check(cudaMalloc(&generated, static_cast<size_t>(steps) * batch_ * 8), "cudaMalloc(generated tokens)");
  cudaEvent_t begin = nullptr, end = nullptr;
  try {
    check(cudaEventCreate(&begin), "event");
    check(cudaEventCreate(&end), "event");
    check(cudaEventRecord(begin, stream_), "event");
    for (int64_t i = 0; i < steps; ++i) {
      run(tokens_, batch_, position + i, cos_table_, sin_table_, 1, true);
      launch_chained(advance_batch_kernel, dim3(1), dim3((batch_ + 31) / 32 * 32), 0, stream_, batch_tokens_, tokens_, generated,
                     step_dev_, position_dev_, batch_);
      launches_ += 1;
    }
    check(cudaEventRecord(end, stream_), "event");
    check(cudaMemcpyAsync(token_pinned_, next_token_, 16, cudaMemcpyDeviceToHost, stream_), "status");
    check(cudaStreamSynchronize(stream_), "generate_batch");
    if (device_ms)
      check(cudaEventElapsedTime(device_ms, begin, end), "event");
    if (out_tokens_host)
      check(cudaMemcpy(out_tokens_host, generated, static_cast<size_t>(steps) * batch_ * 8, cudaMemcpyDeviceToHost), "tokens");
  } catch (...) {
    if (begin)
      cudaEventDestroy(begin);
    if (end)
      cudaEventDestroy(end);
    cudaStreamSynchronize(stream_);
    cudaFree(generated);
    throw;
  }
  cudaEventDestroy(begin);
  cudaEventDestroy(end);
  cudaFree(generated);
  check_status();
}

void Engine::generate(int64_t first_token, int64_t position, int64_t steps, int64_t *out_tokens_host, float *device_ms) {
  const ModelDims &c = dims_;
  check(cudaSetDevice(device_), "cudaSetDevice");
  if (steps <= 0 || position < 0 || position + steps > capacity_)
    throw std::runtime_error("generation does not fit the cache");
  if (c.rotary > 1024)
    throw std::runtime_error("rotary dimension too large");
  validate_tokens(&first_token, 1);
  if (tp_ && gather_logits_) { // the loop keeps tokens on the device: no rank needs the whole logits row
    gather_logits_ = false;
    check(cudaStreamSynchronize(stream_), "generate");
    if (decode_graph_)
      cudaGraphExecDestroy(decode_graph_);
    decode_graph_ = nullptr;
  }
  set_position(position);
  *token_pinned_ = first_token;
  check(cudaMemcpyAsync(dec_tokens_, token_pinned_, 8, cudaMemcpyHostToDevice, stream_), "first token");
  check(cudaMemsetAsync(step_dev_, 0, 8, stream_), "step counter");
  const size_t row_bytes = static_cast<size_t>(c.rotary) * 4;
  check(cudaMemcpyAsync(dec_cos_, cos_table_ + position * c.rotary, row_bytes, cudaMemcpyDeviceToDevice, stream_), "cos");
  check(cudaMemcpyAsync(dec_sin_, sin_table_ + position * c.rotary, row_bytes, cudaMemcpyDeviceToDevice, stream_), "sin");
  cudaEvent_t begin = nullptr, end = nullptr;
  try {
    check(cudaEventCreate(&begin), "event");
    check(cudaEventCreate(&end), "event");
    check(cudaEventRecord(begin, stream_), "event");
    const int threads = static_cast<int>((c.rotary + 31) / 32 * 32);
    for (int64_t i = 0; i < steps; ++i) {
      decode_step();
      launch_chained(advance_kernel, dim3(1), dim3(threads), 0, stream_, next_token_, dec_tokens_, generated_, step_dev_,
                     position_dev_, cos_table_, sin_table_, dec_cos_, dec_sin_, static_cast<int>(c.rotary), capacity_);
      launches_ += 1;
    }
    check(cudaEventRecord(end, stream_), "event");
    check(cudaStreamSynchronize(stream_), "generate");
    if (device_ms)
      check(cudaEventElapsedTime(device_ms, begin, end), "event");
  } catch (...) {
    if (begin)
      cudaEventDestroy(begin);
    if (end)
      cudaEventDestroy(end);
    throw;
  }
  cudaEventDestroy(begin);
  cudaEventDestroy(end);
  if (out_tokens_host)
    check(cudaMemcpy(out_tokens_host, generated_, static_cast<size_t>(steps) * 8, cudaMemcpyDeviceToHost), "tokens");
}

} // namespace llmcp_b200
