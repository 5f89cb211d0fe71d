// extern "C" surface of libllmcp_b200.so (see include/llmcp_b200.h).

#include "../../include/llmcp_b200.h"

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "checkpoint.h"
#include "engine.h"
#include "kernels.h"
#include "text.h"
#include "text_regex.h"
#include "tp_comm.h"

using namespace llmcp_b200;

namespace {

std::mutex g_mutex;
std::string g_error;
int g_device = -1; // -1: whatever device is current
std::atomic<uint64_t> g_launches{0};

void set_error(const std::string &message) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_error = message;
  std::fprintf(stderr, "llmcp_b200: %s\n", message.c_str());
}

void require_device() {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    cudaGetLastError();
    throw std::runtime_error("no CUDA device: this library has no CPU path");
  }
  if (g_device >= 0 && cudaSetDevice(g_device) != cudaSuccess)
    throw std::runtime_error("cudaSetDevice failed");
}

void cuda_check(cudaError_t e, const char *what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// Device buffer that optionally starts as a copy of host data.
struct Buf {
  void *p = nullptr;
  size_t bytes = 0;
  Buf() = default;
  explicit Buf(size_t n, const void *host = nullptr) : bytes(n) {
    cuda_check(cudaMalloc(&p, n ? n : 1), "cudaMalloc");
    if (host && n)
      cuda_check(cudaMemcpy(p, host, n, cudaMemcpyHostToDevice), "cudaMemcpy H2D");
  }
  Buf(const Buf &) = delete;
  Buf &operator=(const Buf &) = delete;
  ~Buf() {
    if (p)
      cudaFree(p);
  }
  template <typename T> T *as() const { return static_cast<T *>(p); }
  void to_host(void *host, size_t n) const {
    if (n)
      cuda_check(cudaMemcpy(host, p, n, cudaMemcpyDeviceToHost), "cudaMemcpy D2H");
  }
};

size_t elem(int dtype) { return dtype == kBF16 ? 2 : 4; }

} // namespace

namespace llmcp_b200 {
void report_error(const std::string &message) { set_error(message); }
} // namespace llmcp_b200

namespace {

template <typename F> int guarded(F &&body) {
  try {
    body();
    cuda_check(cudaDeviceSynchronize(), "kernel execution");
    return 0;
  } catch (const std::exception &e) {
    set_error(e.what());
    return 1;
  }
}

template <typename F> int guarded_async(F &&body) {
  try {
    body();
    return 0;
  } catch (const std::exception &e) {
    set_error(e.what());
    return 1;
  }
}

void check_q8_shape(int64_t N, int64_t K) {
  if (N <= 0 || K <= 0 || N % 8 != 0 || K % 32 != 0)
    throw std::runtime_error("packed Q8_0 needs rows % 8 == 0 and cols % 32 == 0"); // Q8PackedLayout.h:38-42
}

// Uploads packed records and re-lays them out: returns q and d planes.
int gemm_kind() {
  const char *flag = std::getenv("LLMCP_B200_GEMM");
  return flag ? gemm_kind_from_name(flag) : kDefaultGemmKind;
}

bool tensor_core_gemm_enabled() { return gemm_kind() != 0; }

struct DeviceQ8 {
  Buf q, d, d32;
  std::unique_ptr<Buf> h, d32t; // planes of the f16-form GEMM, made on demand
  int64_t N, K;
  DeviceQ8(const uint8_t *records, int64_t N, int64_t K)
      : q(static_cast<size_t>(N) * K), d(static_cast<size_t>(N) * (K / 32) * 2), d32(static_cast<size_t>(N) * (K / 32) * 4), N(N),
        K(K) {
    Buf staging(static_cast<size_t>(N) * (K / 32) * 34, records);
    launch_repack_p4(staging.as<uint8_t>(), N, K, q.as<int8_t>(), d.as<uint16_t>(), d32.as<float>(), nullptr);
    cuda_check(cudaDeviceSynchronize(), "repack");
    g_launches += 1;
  }
  // Planes of the TMA-fed GEMM forms: block-major f32 scales, and for the f16 forms the f16-valued integers.
  void make_tma_planes(bool f16) {
    if (!d32t) {
      d32t = std::make_unique<Buf>(static_cast<size_t>(N) * (K / 32) * 4);
      launch_scales_block_major(d.as<uint16_t>(), 1, N, static_cast<int>(K), N, d32t->as<float>(), nullptr);
      g_launches += 1;
    }
    if (f16 && !h) {
      h = std::make_unique<Buf>(static_cast<size_t>(N) * K * 2);
      launch_weights_to_f16(q.as<int8_t>(), d.as<uint16_t>(), N, static_cast<int>(K), h->p, d32t->as<float>(), nullptr);
      g_launches += 1;
    }
    cuda_check(cudaDeviceSynchronize(), "GEMM planes");
  }
};

// Tensor-core GEMM with its status word checked after completion (synchronises).
void run_gemm_tc(const int8_t *aq, const float *as, int64_t M, int64_t K, DeviceQ8 &w, int64_t N, void *y, int y_dtype,
                 int activation, int32_t *dots) {
  int zero = 0;
  Buf status(4, &zero);
  if (gemm_kind() >= 2) {
    const int form = gemm_kind() - 2;
    const bool f16 = form >= kGemmF16;
    w.make_tma_planes(f16);
    Buf ah(f16 ? static_cast<size_t>(M) * K * 2 : 0), ast(static_cast<size_t>(gemm_tc16_scale_pitch(M)) * (K / 32) * 4);
    if (f16)
      launch_act_to_f16(aq, as, M, static_cast<int>(K), ah.p, ast.as<float>(), nullptr);
    else
      launch_scales_block_major(as, 0, M, static_cast<int>(K), gemm_tc16_scale_pitch(M), ast.as<float>(), nullptr);
    g_launches += 1;
    cuda_check(launch_gemm_q8_tma(form, f16 ? ah.p : static_cast<const void *>(aq), ast.as<float>(), static_cast<int>(M),
                                  static_cast<int>(K), f16 ? w.h->p : w.q.p, w.d32t->as<float>(), static_cast<int>(N), y, y_dtype,
                                  activation, dots, status.as<int>(), nullptr), "gemm");
    g_launches += 1;
    cuda_check(cudaDeviceSynchronize(), "gemm");
    int raised = 0;
    status.to_host(&raised, 4);
    if (raised)
      throw std::runtime_error("tensor-core GEMM: a bounded wait ran out (pipeline protocol error)");
    return;
  }
  cuda_check(launch_gemm_q8_tc(aq, as, static_cast<int>(M), static_cast<int>(K), w.q.as<int8_t>(), w.d32.as<float>(),
                               static_cast<int>(N), y, y_dtype, activation, dots, status.as<int>(), nullptr), "gemm");
  g_launches += 1;
  cuda_check(cudaDeviceSynchronize(), "gemm");
  int raised = 0;
  status.to_host(&raised, 4);
  if (raised)
    throw std::runtime_error("tensor-core GEMM: a bounded wait ran out (pipeline protocol error)");
}

void run_linear(const int8_t *aq, const float *as, int64_t M, int64_t K, const int8_t *wq, const uint16_t *wd,
                int64_t N, void *y, int y_dtype, int activation, int32_t *dots, int rows_per_warp,
                cudaStream_t stream, int flags = 0) {
  if (M == 1) {
    GemvJobs jobs{};
    jobs.count = 1;
    jobs.flags = flags;
    jobs.job[0].wq = wq;
    jobs.job[0].wd = wd;
    jobs.job[0].y = y;
    jobs.job[0].N = static_cast<int>(N);
    jobs.job[0].activation = activation;
    jobs.job[0].y_dtype = y_dtype;
    cuda_check(launch_gemv_q8(aq, as, static_cast<int>(K), jobs, dots, stream, rows_per_warp), "gemv");
  } else {
    cuda_check(launch_gemm_q8_dp4a(aq, as, static_cast<int>(M), static_cast<int>(K), wq, wd, static_cast<int>(N), y,
                                   y_dtype, activation, dots, stream), "gemm");
  }
  g_launches += 1;
}

// ---- AOT entry plumbing -------------------------------------------------------------
template <typename T, int N> struct MemRef {
  T *base;
  T *data;
  int64_t offset;
  int64_t sizes[N];
  int64_t strides[N];
};

struct Session {
  const uint8_t *arena = nullptr;
  uint64_t arena_bytes = 0;
  const void *kv = nullptr, *delta = nullptr, *conv = nullptr;
  int64_t capacity = 0;
  uint64_t last_use = 0;
  std::unique_ptr<Engine> engine;
};

// Sessions are keyed by the caller's arena and state buffers, so a caller that reallocates its state
// vectors (AotRuntime::init does, AotRuntime.cpp:41-43) makes a new one each time while the old one
// still holds a copy of the weights.  The list is therefore bounded: beyond
// LLMCP_B200_MAX_SESSIONS (default 4) the least recently used session is released.
std::vector<std::unique_ptr<Session>> g_sessions;
uint64_t g_session_clock = 0;

size_t max_sessions() {
  const char *flag = std::getenv("LLMCP_B200_MAX_SESSIONS");
  const long v = flag ? std::atol(flag) : 4;
  return static_cast<size_t>(v < 1 ? 1 : v);
}

bool contiguous(const int64_t *sizes, const int64_t *strides, int rank) {
  int64_t expect = 1;
  for (int i = rank - 1; i >= 0; --i) {
    if (sizes[i] != 1 && strides[i] != expect)
      return false;
    expect *= sizes[i];
  }
  return true;
}

void aot_entry(void *tokens_p, void *cos_p, void *sin_p, void *start_pos, void *cache_length, void *arena_p,
               void *kv_p, void *delta_p, void *conv_p, void *logits_p) {
  auto *logits = static_cast<MemRef<float, 2> *>(logits_p);
  float *row = logits->data + logits->offset;
  const int64_t vocab = logits->sizes[1];
  try {
    require_device();
    auto *tokens = static_cast<MemRef<int64_t, 1> *>(tokens_p);
    auto *cos = static_cast<MemRef<float, 2> *>(cos_p);
    auto *sin = static_cast<MemRef<float, 2> *>(sin_p);
    auto *arena = static_cast<MemRef<uint8_t, 1> *>(arena_p);
    auto *kv = static_cast<MemRef<uint16_t, 5> *>(kv_p);
    auto *delta = static_cast<MemRef<float, 4> *>(delta_p);
    auto *conv = static_cast<MemRef<uint16_t, 3> *>(conv_p);
    const int64_t position = reinterpret_cast<int64_t>(start_pos);
    (void)cache_length; // accepted and unused, as in LowerAttention.cpp:408-412
    const int64_t S = tokens->sizes[0];
    if (tokens->strides[0] != 1 && S > 1)
      throw std::runtime_error("tokens must be contiguous");
    if (!contiguous(cos->sizes, cos->strides, 2) || !contiguous(sin->sizes, sin->strides, 2) ||
        !contiguous(kv->sizes, kv->strides, 5) || !contiguous(delta->sizes, delta->strides, 4) ||
        !contiguous(conv->sizes, conv->strides, 3))
      throw std::runtime_error("cos/sin/kv/delta/conv must be contiguous row-major buffers");

    const uint8_t *base = arena->data + arena->offset;
    Session *session = nullptr;
    {
      std::lock_guard<std::mutex> lock(g_mutex);
      for (auto &s : g_sessions)
        if (s->arena == base && s->arena_bytes == static_cast<uint64_t>(arena->sizes[0]) &&
            s->kv == kv->data && s->delta == delta->data && s->conv == conv->data && s->capacity == kv->sizes[3])
          session = s.get();
      if (session)
        session->last_use = ++g_session_clock;
    }
    if (!session) {
      // Dimensions the generated code has baked in come from the descriptors and the
      // manifest here (AotRuntime.cpp:41-43,87-114).
      Manifest manifest;
      const std::string error = parse_container(base, 0, &manifest);
      if (!error.empty())
        throw std::runtime_error(error);
      if (manifest.total_bytes != static_cast<uint64_t>(arena->sizes[0]))
        throw std::runtime_error("arena descriptor length differs from the container header");
      const std::string root = "model.language_model.";
      const TensorEntry *embed = manifest.find(root + "embed_tokens.weight");
      const TensorEntry *gate = manifest.find(root + "layers.0.mlp.gate_proj.weight");
      if (!embed || !gate)
        throw std::runtime_error("manifest lacks embed_tokens / layers.0.mlp.gate_proj");
      ModelDims d;
      d.vocab = embed->shape[0];
      d.hidden = embed->shape[1];
      d.intermediate = gate->shape[0];
      int64_t layers = 0;
      while (manifest.find(root + "layers." + std::to_string(layers) + ".input_layernorm.weight"))
        ++layers;
      d.layers = layers;
      const int64_t full = kv->sizes[0], linear = delta->sizes[0];
      if (full <= 0 || full + linear != layers || layers % full != 0)
        throw std::runtime_error("state descriptors do not match the layer count of the manifest");
      d.full_interval = layers / full;
      d.kv_heads = kv->sizes[2];
      d.head_dim = kv->sizes[4];
      d.rotary = cos->sizes[1];
      d.lin_v_heads = delta->sizes[1];
      d.lin_k_dim = delta->sizes[2];
      d.lin_v_dim = delta->sizes[3];
      d.conv_kernel = conv->sizes[1] + 1;
      const int64_t qkv_dim = conv->sizes[2];
      d.lin_k_heads = (qkv_dim - d.lin_v_heads * d.lin_v_dim) / (2 * d.lin_k_dim);
      const TensorEntry *q_proj = nullptr;
      for (int64_t l = 0; l < layers && !q_proj; ++l)
        q_proj = manifest.find(root + "layers." + std::to_string(l) + ".self_attn.q_proj.weight");
      if (!q_proj)
        throw std::runtime_error("manifest lacks a self_attn.q_proj.weight");
      d.heads = q_proj->shape[0] / (2 * d.head_dim);
      if (vocab != d.vocab)
        throw std::runtime_error("logits descriptor width differs from the vocabulary of the arena");
      int device = g_device;
      if (device < 0)
        cuda_check(cudaGetDevice(&device), "cudaGetDevice");
      auto fresh = std::make_unique<Session>();
      fresh->arena = base;
      fresh->arena_bytes = static_cast<uint64_t>(arena->sizes[0]);
      fresh->kv = kv->data;
      fresh->delta = delta->data;
      fresh->conv = conv->data;
      fresh->capacity = kv->sizes[3];
      fresh->engine = std::make_unique<Engine>(base, 0, d, kv->sizes[3], device);
      std::lock_guard<std::mutex> lock(g_mutex);
      while (g_sessions.size() >= max_sessions()) { // the engine's destructor waits for its stream and frees its memory
        size_t oldest = 0;
        for (size_t i = 1; i < g_sessions.size(); ++i)
          if (g_sessions[i]->last_use < g_sessions[oldest]->last_use)
            oldest = i;
        g_sessions.erase(g_sessions.begin() + static_cast<std::ptrdiff_t>(oldest));
      }
      fresh->last_use = ++g_session_clock;
      g_sessions.push_back(std::move(fresh));
      session = g_sessions.back().get();
    }
    Engine &engine = *session->engine;
    static const bool sync_state = std::getenv("LLMCP_B200_SYNC_STATE") && std::atoi(std::getenv("LLMCP_B200_SYNC_STATE")) != 0;
    if (sync_state)
      engine.upload_state(kv->data + kv->offset, delta->data + delta->offset, conv->data + conv->offset);
    else if (position == 0)
      engine.reset_state();
    const uint64_t before = engine.launches();
    engine.forward_host(tokens->data + tokens->offset, S, position, cos->data + cos->offset, sin->data + sin->offset, row);
    g_launches += engine.launches() - before;
    if (sync_state)
      engine.download_state(kv->data + kv->offset, delta->data + delta->offset, conv->data + conv->offset);
  } catch (const std::exception &e) {
    set_error(e.what());
    for (int64_t i = 0; i < vocab; ++i)
      row[i] = NAN;
  }
}

ModelDims to_dims(const llmcp_b200_dims *d) {
  ModelDims m;
  if (!d)
    return m;
  m.hidden = d->hidden;
  m.intermediate = d->intermediate;
  m.vocab = d->vocab;
  m.layers = d->layers;
  m.full_interval = d->full_interval;
  m.heads = d->heads;
  m.kv_heads = d->kv_heads;
  m.head_dim = d->head_dim;
  m.rotary = d->rotary;
  m.lin_k_heads = d->lin_k_heads;
  m.lin_v_heads = d->lin_v_heads;
  m.lin_k_dim = d->lin_k_dim;
  m.lin_v_dim = d->lin_v_dim;
  m.conv_kernel = d->conv_kernel;
  m.eps = d->eps;
  m.rope_theta = d->rope_theta;
  return m;
}

void check_dims(const ModelDims &d) {
  if (d.hidden <= 0 || d.hidden % 32 || d.intermediate <= 0 || d.intermediate % 32 || d.vocab % 8 || d.layers <= 0 ||
      d.full_interval <= 0 || d.layers % d.full_interval || d.heads <= 0 || d.kv_heads <= 0 || d.heads % d.kv_heads ||
      d.head_dim <= 0 || d.rotary % 2 || d.rotary > d.head_dim || d.lin_k_heads <= 0 || d.lin_v_heads % d.lin_k_heads ||
      d.lin_v_heads % 8 || d.lin_v_dim % 32 || d.value_dim() % 32 || d.attn_dim() % 32 || d.qkv_dim() % 8 ||
      d.kv_dim() % 8 || d.q_out() % 8 || d.conv_kernel < 2)
    throw std::runtime_error("unsupported model dimensions");
}

} // namespace

extern "C" {

int32_t llmcp_model_abi_version(void) { return 2; }

void _mlir_ciface_llmcp_model_prefill(void *tokens, void *cos, void *sin, void *start_pos, void *cache_length,
                                      void *arena, void *kv, void *delta, void *conv, void *logits) {
  aot_entry(tokens, cos, sin, start_pos, cache_length, arena, kv, delta, conv, logits);
}

void _mlir_ciface_llmcp_model_decode(void *tokens, void *cos, void *sin, void *start_pos, void *cache_length,
                                     void *arena, void *kv, void *delta, void *conv, void *logits) {
  aot_entry(tokens, cos, sin, start_pos, cache_length, arena, kv, delta, conv, logits);
}

size_t llmcp_b200_last_error(char *buffer, size_t capacity) {
  std::lock_guard<std::mutex> lock(g_mutex);
  if (buffer && capacity) {
    const size_t n = std::min(capacity - 1, g_error.size());
    std::memcpy(buffer, g_error.data(), n);
    buffer[n] = 0;
  }
  return g_error.size();
}

void llmcp_b200_clear_error(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_error.clear();
}

int llmcp_b200_device_count(void) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return count;
}

int llmcp_b200_set_device(int device) {
  return guarded_async([&] {
    if (device < 0 || device >= llmcp_b200_device_count())
      throw std::runtime_error("no such CUDA device");
    g_device = device;
    cuda_check(cudaSetDevice(device), "cudaSetDevice");
  });
}

void llmcp_b200_release_all(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_sessions.clear();
}

int llmcp_b200_session_count(void) {
  std::lock_guard<std::mutex> lock(g_mutex);
  return static_cast<int>(g_sessions.size());
}

uint64_t llmcp_b200_launch_count(void) { return g_launches.load(); }

int llmcp_b200_set_mode(int mode) {
  if (mode != kModeExact && mode != kModeFast) {
    set_error("mode must be 0 (exact) or 1 (fast)");
    return 1;
  }
  set_default_mode(mode);
  return 0;
}

int llmcp_b200_get_mode(void) { return default_mode(); }

// ---- operators on host pointers ------------------------------------------------------
int llmcp_op_act_quant(const void *x, int x_dtype, int64_t M, int64_t K, int8_t *q, float *scales) {
  return guarded([&] {
    require_device();
    if (K % 32 != 0 || M < 0)
      throw std::runtime_error("K must be a multiple of 32");
    Buf dx(static_cast<size_t>(M) * K * elem(x_dtype), x), dq(static_cast<size_t>(M) * K), ds(static_cast<size_t>(M) * (K / 32) * 4);
    launch_act_quant(dx.p, x_dtype, M, K, dq.as<int8_t>(), ds.as<float>(), nullptr);
    g_launches += 1;
    cuda_check(cudaDeviceSynchronize(), "act_quant");
    dq.to_host(q, dq.bytes);
    ds.to_host(scales, ds.bytes);
  });
}

int llmcp_op_linear_q8(const void *x, int x_dtype, int64_t M, int64_t K, const uint8_t *weight, int64_t N, void *y,
                       int y_dtype, int activation, int32_t *block_dots) {
  return guarded([&] {
    require_device();
    check_q8_shape(N, K);
    if (M <= 0)
      return; // an empty input produces an empty output
    DeviceQ8 w(weight, N, K);
    Buf dx(static_cast<size_t>(M) * K * elem(x_dtype), x), dq(static_cast<size_t>(M) * K), ds(static_cast<size_t>(M) * (K / 32) * 4);
    Buf dy(static_cast<size_t>(M) * N * elem(y_dtype));
    Buf dots(block_dots ? static_cast<size_t>(M) * N * (K / 32) * 4 : 0);
    launch_act_quant(dx.p, x_dtype, M, K, dq.as<int8_t>(), ds.as<float>(), nullptr);
    g_launches += 1;
    if (M > 1 && tensor_core_gemm_enabled())
      run_gemm_tc(dq.as<int8_t>(), ds.as<float>(), M, K, w, N, dy.p, y_dtype, activation,
                  block_dots ? dots.as<int32_t>() : nullptr);
    else
      run_linear(dq.as<int8_t>(), ds.as<float>(), M, K, w.q.as<int8_t>(), w.d.as<uint16_t>(), N, dy.p, y_dtype, activation,
                 block_dots ? dots.as<int32_t>() : nullptr, 0, nullptr,
                 default_mode() == kModeFast && !block_dots ? kGemvFast : 0);
    cuda_check(cudaDeviceSynchronize(), "linear");
    dy.to_host(y, dy.bytes);
    if (block_dots)
      dots.to_host(block_dots, dots.bytes);
  });
}

int llmcp_op_linear_bf16(const uint16_t *x, int64_t M, int64_t K, const uint16_t *weight, int64_t N, void *y, int y_dtype,
                         int activation) {
  return guarded([&] {
    require_device();
    if (N <= 0 || K <= 0 || K % 16 != 0 || (M > 1 && N % 8 != 0))
      throw std::runtime_error("bf16 linear: K must be a multiple of 16 (and N of 8 for more than one row)");
    if (M <= 0)
      return;
    Buf dx(static_cast<size_t>(M) * K * 2, x), dw(static_cast<size_t>(N) * K * 2, weight), dy(static_cast<size_t>(M) * N * elem(y_dtype)),
        dstatus(4);
    cuda_check(cudaMemset(dstatus.p, 0, 4), "memset");
    if (M == 1)
      cuda_check(launch_gemv_bf16(dx.as<uint16_t>(), static_cast<int>(K), dw.as<uint16_t>(), N, dy.p, y_dtype, activation, nullptr),
                 "bf16 GEMV");
    else
      cuda_check(launch_gemm_bf16_tc(dx.as<uint16_t>(), static_cast<int>(M), static_cast<int>(K), dw.as<uint16_t>(),
                                     static_cast<int>(N), dy.p, y_dtype, activation, dstatus.as<int>(), nullptr), "bf16 GEMM");
    g_launches += 1;
    cuda_check(cudaDeviceSynchronize(), "bf16 linear");
    int status = 0;
    dstatus.to_host(&status, 4);
    if (status)
      throw std::runtime_error("bf16 linear: a bounded wait inside the tensor-core kernel ran out");
    dy.to_host(y, dy.bytes);
  });
}

int llmcp_op_lm_head_q8(const uint16_t *hidden, int64_t M, int64_t K, const uint8_t *table, int64_t vocab,
                        float *logits, int64_t *argmax) {
  return guarded([&] {
    require_device();
    check_q8_shape(vocab, K);
    if (M <= 0)
      return;
    DeviceQ8 w(table, vocab, K);
    Buf dx(static_cast<size_t>(M) * K * 2, hidden), dq(static_cast<size_t>(M) * K), ds(static_cast<size_t>(M) * (K / 32) * 4);
    Buf dy(static_cast<size_t>(M) * vocab * 4), sv(kArgmaxParts * 4), si(kArgmaxParts * 8), out(static_cast<size_t>(M) * 8);
    launch_act_quant(dx.p, kBF16, M, K, dq.as<int8_t>(), ds.as<float>(), nullptr);
    g_launches += 1;
    if (M > 1 && tensor_core_gemm_enabled())
      run_gemm_tc(dq.as<int8_t>(), ds.as<float>(), M, K, w, vocab, dy.p, kF32, kNone, nullptr);
    else
      run_linear(dq.as<int8_t>(), ds.as<float>(), M, K, w.q.as<int8_t>(), w.d.as<uint16_t>(), vocab, dy.p, kF32, kNone,
                 nullptr, 0, nullptr);
    for (int64_t m = 0; m < M; ++m) {
      launch_argmax(dy.as<float>() + m * vocab, vocab, sv.as<float>(), si.as<int64_t>(), 0, out.as<int64_t>() + m,
                    nullptr, nullptr);
      g_launches += 2;
    }
    cuda_check(cudaDeviceSynchronize(), "lm_head");
    if (logits)
      dy.to_host(logits, dy.bytes);
    if (argmax)
      out.to_host(argmax, out.bytes);
  });
}

int llmcp_op_embedding_q8(const int64_t *tokens, int64_t S, const uint8_t *table, int64_t vocab, int64_t hidden,
                          uint16_t *out) {
  return guarded([&] {
    require_device();
    check_q8_shape(vocab, hidden);
    for (int64_t i = 0; i < S; ++i)
      if (tokens[i] < 0 || tokens[i] >= vocab)
        throw std::runtime_error("token id outside the table");
    if (S <= 0)
      return;
    DeviceQ8 w(table, vocab, hidden);
    Buf dt(static_cast<size_t>(S) * 8, tokens), dy(static_cast<size_t>(S) * hidden * 2);
    launch_embedding_q8(dt.as<int64_t>(), S, hidden, vocab, w.q.as<int8_t>(), w.d.as<uint16_t>(), dy.as<uint16_t>(), nullptr,
                        nullptr);
    g_launches += 1;
    cuda_check(cudaDeviceSynchronize(), "embedding");
    dy.to_host(out, dy.bytes);
  });
}

int llmcp_op_rms_norm(const uint16_t *x, int64_t M, int64_t H, const void *weight, int w_dtype, float eps,
                      int zero_centered, uint16_t *y) {
  return guarded([&] {
    require_device();
    if (M <= 0 || H <= 0)
      return;
    Buf dx(static_cast<size_t>(M) * H * 2, x), dw(static_cast<size_t>(H) * elem(w_dtype), weight), dy(static_cast<size_t>(M) * H * 2);
    cudaError_t e = cudaErrorNotSupported;
    if (default_mode() == kModeFast)
      e = launch_rms_norm_fast(dx.as<uint16_t>(), nullptr, M, static_cast<int>(H), dw.p, w_dtype, eps, zero_centered, nullptr,
                               dy.as<uint16_t>(), nullptr, nullptr, nullptr);
    if (e == cudaErrorNotSupported)
      e = launch_rms_norm(dx.as<uint16_t>(), nullptr, M, static_cast<int>(H), dw.p, w_dtype, eps, zero_centered, nullptr,
                          dy.as<uint16_t>(), nullptr, nullptr, nullptr);
    cuda_check(e, "rms_norm");
    g_launches += 1;
    cuda_check(cudaDeviceSynchronize(), "rms_norm");
    dy.to_host(y, dy.bytes);
  });
}

int llmcp_op_pointwise(const uint16_t *a, const uint16_t *b, int64_t count, int op, uint16_t *y) {
  return guarded([&] {
    require_device();
    if (op < 0 || op > 2)
      throw std::runtime_error("op must be 0 (add), 1 (mul) or 2 (silu_mul)");
    if (count <= 0)
      return;
    Buf da(static_cast<size_t>(count) * 2, a), db(static_cast<size_t>(count) * 2, b), dy(static_cast<size_t>(count) * 2);
    cuda_check(launch_pointwise(da.as<uint16_t>(), db.as<uint16_t>(), count, op, dy.as<uint16_t>(), nullptr, nullptr, nullptr), "pointwise");
    g_launches += 1;
    cuda_check(cudaDeviceSynchronize(), "pointwise");
    dy.to_host(y, dy.bytes);
  });
}

int llmcp_op_gated_rms_norm(const uint16_t *x, const uint16_t *gate, const void *weight, int w_dtype, int64_t M,
                            int64_t H, int64_t group, float eps, int gate_activated, uint16_t *y) {
  return guarded([&] {
    require_device();
    if (group <= 0 || H % group != 0)
      throw std::runtime_error("hidden must be a multiple of group_size");
    if (M <= 0)
      return;
    Buf dx(static_cast<size_t>(M) * H * 2, x), dg(static_cast<size_t>(M) * H * 2, gate), dw(static_cast<size_t>(group) * elem(w_dtype), weight),
        dy(static_cast<size_t>(M) * H * 2);
    cuda_check(launch_gated_rms_norm(dx.as<uint16_t>(), dg.as<uint16_t>(), dw.p, w_dtype, M, static_cast<int>(H),
                                     static_cast<int>(group), eps, gate_activated, dy.as<uint16_t>(), nullptr, nullptr, nullptr),
               "gated_rms_norm");
    g_launches += 1;
    cuda_check(cudaDeviceSynchronize(), "gated_rms_norm");
    dy.to_host(y, dy.bytes);
  });
}

int llmcp_op_causal_conv1d(const uint16_t *x, const uint16_t *weight, uint16_t *state, int64_t S, int64_t C,
                           int64_t kernel, uint16_t *y) {
  return guarded([&] {
    require_device();
    if (kernel <= 1 || C <= 0)
      throw std::runtime_error("kernel_size must exceed 1");
    if (S <= 0)
      return;
    Buf dx(static_cast<size_t>(S) * C * 2, x), dw(static_cast<size_t>(C) * kernel * 2, weight), ds(static_cast<size_t>(kernel - 1) * C * 2, state),
        dy(static_cast<size_t>(S) * C * 2);
    cuda_check(launch_causal_conv1d(dx.as<uint16_t>(), dw.as<uint16_t>(), ds.as<uint16_t>(), S, static_cast<int>(C),
                                    static_cast<int>(kernel), dy.as<uint16_t>(), nullptr), "causal_conv1d");
    g_launches += 2;
    cuda_check(cudaDeviceSynchronize(), "causal_conv1d");
    dy.to_host(y, dy.bytes);
    ds.to_host(state, ds.bytes);
  });
}

int llmcp_op_gated_delta_net(const uint16_t *conv, const uint16_t *a, const uint16_t *b, const float *a_log,
                             const uint16_t *dt_bias, float *state, int64_t S, int64_t nk, int64_t nv, int64_t dk,
                             int64_t dv, int b_activated, uint16_t *out) {
  return guarded([&] {
    require_device();
    if (nk <= 0 || nv <= 0 || dk <= 0 || dv <= 0 || nv % nk != 0)
      throw std::runtime_error("num_v_heads must be a positive multiple of num_k_heads");
    if (S <= 0)
      return;
    const size_t channels = static_cast<size_t>(2 * nk * dk + nv * dv);
    Buf dc(static_cast<size_t>(S) * channels * 2, conv), da(static_cast<size_t>(S) * nv * 2, a), db(static_cast<size_t>(S) * nv * 2, b),
        dl(static_cast<size_t>(nv) * 4, a_log), dt(static_cast<size_t>(nv) * 2, dt_bias), ds(static_cast<size_t>(nv) * dk * dv * 4, state),
        dout(static_cast<size_t>(S) * nv * dv * 2),
        scratch(gdn_scratch_floats(S, static_cast<int>(nk), static_cast<int>(nv), static_cast<int>(dk)) * 4);
    cuda_check(launch_gated_delta_net(dc.as<uint16_t>(), da.as<uint16_t>(), db.as<uint16_t>(), dl.p, kF32, dt.p, kBF16,
                                      ds.as<float>(), S, static_cast<int>(nk), static_cast<int>(nv), static_cast<int>(dk),
                                      static_cast<int>(dv), b_activated, scratch.as<float>(), dout.as<uint16_t>(), nullptr, 0,
                                      default_mode() == kModeFast ? 1 : 0),
               "gated_delta_net");
    g_launches += 2;
    cuda_check(cudaDeviceSynchronize(), "gated_delta_net");
    dout.to_host(out, dout.bytes);
    ds.to_host(state, ds.bytes);
  });
}

int llmcp_op_attention(const uint16_t *qg, const uint16_t *k, const uint16_t *v, const uint16_t *q_norm,
                       const uint16_t *k_norm, const float *cos, const float *sin, uint16_t *cache, int64_t position,
                       int64_t S, int64_t nh, int64_t nkv, int64_t hd, int64_t rot, int64_t cap, uint16_t *out) {
  return guarded([&] {
    require_device();
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || rot < 0 || rot > hd || rot % 2 != 0)
      throw std::runtime_error("invalid head configuration");
    if (position < 0 || position + S > cap)
      throw std::runtime_error("tokens do not fit the KV cache");
    if (S <= 0)
      return;
    Buf dqg(static_cast<size_t>(S) * nh * 2 * hd * 2, qg), dk(static_cast<size_t>(S) * nkv * hd * 2, k), dv(static_cast<size_t>(S) * nkv * hd * 2, v),
        dqn(static_cast<size_t>(hd) * 2, q_norm), dkn(static_cast<size_t>(hd) * 2, k_norm), dcos(static_cast<size_t>(S) * rot * 4, cos),
        dsin(static_cast<size_t>(S) * rot * 4, sin), dcache(static_cast<size_t>(2) * nkv * cap * hd * 2, cache),
        dout(static_cast<size_t>(S) * nh * hd * 2),
        scratch(std::max({attn_scratch_bytes(S, static_cast<int>(nh), static_cast<int>(hd), position),
                          attn_fast_scratch_bytes(static_cast<int>(nh), static_cast<int>(hd), position + S - 1),
                          attention_prefill_tc_scratch_bytes(S, static_cast<int>(nh), static_cast<int>(nkv), cap)})),
        dpos(8, &position), dstatus(4);
    const bool tensor_cores = default_mode() == kModeFast && S > 1 &&
                              attention_prefill_tc_supported(static_cast<int>(nh), static_cast<int>(nkv), static_cast<int>(hd));
    if (tensor_cores) {
      cuda_check(cudaMemset(dstatus.p, 0, 4), "memset");
      cuda_check(launch_attention_prefill_tc(dqg.as<uint16_t>(), dk.as<uint16_t>(), dv.as<uint16_t>(), dqn.as<uint16_t>(),
                                             dkn.as<uint16_t>(), dcos.as<float>(), dsin.as<float>(), 0, dcache.as<uint16_t>(),
                                             dpos.as<int64_t>(), position, S, static_cast<int>(nh), static_cast<int>(nkv),
                                             static_cast<int>(hd), static_cast<int>(rot), cap, scratch.p, dout.as<uint16_t>(),
                                             nullptr, nullptr, dstatus.as<int>(), nullptr), "attention (tensor cores)");
    } else
    if (default_mode() == kModeFast && S == 1 &&
        attention_decode_fast_supported(static_cast<int>(nh), static_cast<int>(nkv), static_cast<int>(hd))) {
      cuda_check(launch_attention_decode_fast(dqg.as<uint16_t>(), dk.as<uint16_t>(), dv.as<uint16_t>(), dqn.as<uint16_t>(),
                                              dkn.as<uint16_t>(), dcos.as<float>(), dsin.as<float>(), 0, dcache.as<uint16_t>(),
                                              dpos.as<int64_t>(), position, static_cast<int>(nh), static_cast<int>(nkv),
                                              static_cast<int>(hd), static_cast<int>(rot), cap, scratch.p, dout.as<uint16_t>(),
                                              nullptr, nullptr, nullptr), "attention (fast)");
    } else
    cuda_check(launch_attention(dqg.as<uint16_t>(), dk.as<uint16_t>(), dv.as<uint16_t>(), dqn.as<uint16_t>(),
                                dkn.as<uint16_t>(), dcos.as<float>(), dsin.as<float>(), 0, dcache.as<uint16_t>(),
                                dpos.as<int64_t>(), position, S,
                                static_cast<int>(nh), static_cast<int>(nkv), static_cast<int>(hd), static_cast<int>(rot), cap,
                                scratch.p, dout.as<uint16_t>(), nullptr, nullptr, nullptr), "attention");
    g_launches += 3;
    cuda_check(cudaDeviceSynchronize(), "attention");
    if (tensor_cores) {
      int status = 0;
      dstatus.to_host(&status, 4);
      if (status)
        throw std::runtime_error("attention: a bounded wait inside the tensor-core kernel ran out");
    }
    dout.to_host(out, dout.bytes);
    dcache.to_host(cache, dcache.bytes);
  });
}

// ---- operators on device pointers ------------------------------------------------------
int llmcp_dev_repack_q8(const uint8_t *records, int64_t N, int64_t K, int8_t *q, uint16_t *d, void *stream) {
  return guarded_async([&] {
    check_q8_shape(N, K);
    launch_repack_p4(records, N, K, q, d, nullptr, static_cast<cudaStream_t>(stream));
    g_launches += 1;
    cuda_check(cudaGetLastError(), "repack");
  });
}

int llmcp_dev_act_quant(const void *x, int x_dtype, int64_t M, int64_t K, int8_t *q, float *scales, void *stream) {
  return guarded_async([&] {
    if (K % 32 != 0)
      throw std::runtime_error("K must be a multiple of 32");
    launch_act_quant(x, x_dtype, M, K, q, scales, static_cast<cudaStream_t>(stream));
    g_launches += 1;
    cuda_check(cudaGetLastError(), "act_quant");
  });
}

int llmcp_dev_gemv_q8(const int8_t *aq, const float *as, int64_t K, const int8_t *wq, const uint16_t *wd, int64_t N,
                      void *y, int y_dtype, int activation, int rows_per_warp, int flags, void *stream) {
  return guarded_async([&] {
    check_q8_shape(N, K);
    run_linear(aq, as, 1, K, wq, wd, N, y, y_dtype, activation, nullptr, rows_per_warp, static_cast<cudaStream_t>(stream), flags);
  });
}

int llmcp_dev_gemv_q8_swiglu(const int8_t *aq, const float *as, int64_t K, const int8_t *gate_q, const uint16_t *gate_d,
                             const int8_t *up_q, const uint16_t *up_d, int64_t N, uint16_t *product, int8_t *q_out,
                             float *s_out, int flags, void *stream) {
  return guarded_async([&] {
    check_q8_shape(N, K);
    if (!gemv_swiglu_supported(static_cast<int>(K), N))
      throw std::runtime_error("llmcp_dev_gemv_q8_swiglu takes K = 2560 and N % 32 == 0");
    if (static_cast<const void *>(aq) == q_out || static_cast<const void *>(as) == s_out)
      throw std::runtime_error("llmcp_dev_gemv_q8_swiglu: the quantised product must not overwrite the quantised input");
    cuda_check(launch_gemv_q8_swiglu(aq, as, static_cast<int>(K), gate_q, gate_d, up_q, up_d, N, product, q_out, s_out, flags,
                                     static_cast<cudaStream_t>(stream)), "gate/up GEMV");
    g_launches += 1;
  });
}

int llmcp_dev_gemm_q8(const int8_t *aq, const float *as, int64_t M, int64_t K, const int8_t *wq, const uint16_t *wd,
                      int64_t N, void *y, int y_dtype, int activation, void *stream) {
  return guarded_async([&] {
    check_q8_shape(N, K);
    if (M < 2)
      throw std::runtime_error("llmcp_dev_gemm_q8 needs M > 1; use llmcp_dev_gemv_q8 for one row");
    run_linear(aq, as, M, K, wq, wd, N, y, y_dtype, activation, nullptr, 0, static_cast<cudaStream_t>(stream));
  });
}

int llmcp_dev_gemm_q8_tc(const int8_t *aq, const float *as, int64_t M, int64_t K, const int8_t *wq, const float *wd32,
                         int64_t N, void *y, int y_dtype, int activation, int *status, void *stream) {
  return guarded_async([&] {
    check_q8_shape(N, K);
    if (M < 1)
      throw std::runtime_error("llmcp_dev_gemm_q8_tc needs M >= 1");
    cuda_check(launch_gemm_q8_tc(aq, as, static_cast<int>(M), static_cast<int>(K), wq, wd32, static_cast<int>(N), y, y_dtype,
                                 activation, nullptr, status, static_cast<cudaStream_t>(stream)), "gemm");
    g_launches += 1;
  });
}

int llmcp_dev_q8_gemm_planes(const int8_t *q, const void *scales, int scales_are_f16, int64_t rows, int64_t K, void *values_f16,
                             float *scales_block_major, void *stream) {
  return guarded_async([&] {
    if (rows <= 0 || K <= 0 || K % 32 != 0 || !scales_block_major)
      throw std::runtime_error("rows > 0, K % 32 == 0 and a scale plane are required");
    const int64_t pitch = scales_are_f16 ? rows : gemm_tc16_scale_pitch(rows);
    if (!values_f16)
      launch_scales_block_major(scales, scales_are_f16, rows, static_cast<int>(K), pitch, scales_block_major,
                                static_cast<cudaStream_t>(stream));
    else if (scales_are_f16)
      launch_weights_to_f16(q, static_cast<const uint16_t *>(scales), rows, static_cast<int>(K), values_f16, scales_block_major,
                            static_cast<cudaStream_t>(stream));
    else
      launch_act_to_f16(q, static_cast<const float *>(scales), rows, static_cast<int>(K), values_f16, scales_block_major,
                        static_cast<cudaStream_t>(stream));
    g_launches += 1;
    cuda_check(cudaGetLastError(), "GEMM planes");
  });
}

int64_t llmcp_dev_gemm_q8_tma_scale_pitch(int64_t M) { return gemm_tc16_scale_pitch(M); }

int llmcp_dev_gemm_q8_tma(int form, const void *a, const float *a_scales, int64_t M, int64_t K, const void *w,
                          const float *w_scales, int64_t N, void *y, int y_dtype, int activation, int *status,
                          uint32_t spin_limit, int fault, void *stream) {
  return guarded_async([&] {
    check_q8_shape(N, K);
    if (M < 1)
      throw std::runtime_error("llmcp_dev_gemm_q8_tma needs M >= 1");
    cuda_check(launch_gemm_q8_tma(form, a, a_scales, static_cast<int>(M), static_cast<int>(K), w, w_scales, static_cast<int>(N), y,
                                  y_dtype, activation, nullptr, status, static_cast<cudaStream_t>(stream), spin_limit, fault),
               "gemm");
    g_launches += 1;
  });
}

int llmcp_dev_argmax(const float *x, int64_t n, float *scratch_values, int64_t *scratch_indices, int64_t *out_index,
                     void *stream) {
  return guarded_async([&] {
    if (n <= 0)
      throw std::runtime_error("argmax of an empty vector");
    launch_argmax(x, n, scratch_values, scratch_indices, 0, out_index, nullptr, static_cast<cudaStream_t>(stream));
    g_launches += 2;
    cuda_check(cudaGetLastError(), "argmax");
  });
}

// ---- container helpers and engine --------------------------------------------------------
static void from_dims(const ModelDims &m, llmcp_b200_dims *d);

void llmcp_b200_default_dims(llmcp_b200_dims *d) { from_dims(ModelDims(), d); }

static void from_dims(const ModelDims &m, llmcp_b200_dims *d) {
  d->hidden = m.hidden;
  d->intermediate = m.intermediate;
  d->vocab = m.vocab;
  d->layers = m.layers;
  d->full_interval = m.full_interval;
  d->heads = m.heads;
  d->kv_heads = m.kv_heads;
  d->head_dim = m.head_dim;
  d->rotary = m.rotary;
  d->lin_k_heads = m.lin_k_heads;
  d->lin_v_heads = m.lin_v_heads;
  d->lin_k_dim = m.lin_k_dim;
  d->lin_v_dim = m.lin_v_dim;
  d->conv_kernel = m.conv_kernel;
  d->eps = m.eps;
  d->rope_theta = m.rope_theta;
}

uint64_t llmcp_b200_synthetic_bytes(const llmcp_b200_dims *dims) {
  try {
    const ModelDims d = to_dims(dims);
    check_dims(d);
    return synthetic_container_bytes(d, nullptr);
  } catch (const std::exception &e) {
    set_error(e.what());
    return 0;
  }
}

int llmcp_b200_synthetic_fill(const llmcp_b200_dims *dims, uint64_t seed, uint8_t *file, uint64_t file_bytes) {
  return guarded_async([&] {
    const ModelDims d = to_dims(dims);
    check_dims(d);
    const std::string error = fill_synthetic_container(d, seed, file, file_bytes);
    if (!error.empty())
      throw std::runtime_error(error);
  });
}

int llmcp_b200_pack_q8_0_p4(const float *values, int64_t rows, int64_t cols, uint8_t *dst) {
  return guarded_async([&] {
    if (!pack_q8_0_p4(values, rows, cols, dst))
      throw std::runtime_error("packed Q8_0 needs rows % 8 == 0 and cols % 32 == 0");
  });
}

int llmcp_b200_validate(const uint8_t *file, uint64_t file_bytes) {
  return guarded_async([&] {
    if (file_bytes < kHeaderBytes)
      throw std::runtime_error("packed weights file is too small");
    Manifest m;
    const std::string error = parse_container(file, file_bytes, &m);
    if (!error.empty())
      throw std::runtime_error(error);
  });
}

// ---- token ids -> text (text.h) ----------------------------------------------------------------
namespace {
uint64_t copy_text(const std::string &text, char *out, uint64_t capacity) {
  if (out && capacity) {
    const uint64_t n = std::min<uint64_t>(text.size(), capacity - 1);
    std::memcpy(out, text.data(), n);
    out[n] = 0;
  }
  return text.size();
}
} // namespace

void *llmcp_b200_vocab_create(const char *json, uint64_t length) {
  auto *vocab = new ByteLevelVocab();
  const std::string error = vocab->load(json, length);
  if (!error.empty()) {
    set_error(error);
    delete vocab;
    return nullptr;
  }
  return vocab;
}

void llmcp_b200_vocab_destroy(void *vocab) { delete static_cast<ByteLevelVocab *>(vocab); }

int64_t llmcp_b200_vocab_size(const void *vocab) { return static_cast<const ByteLevelVocab *>(vocab)->size(); }

int32_t llmcp_b200_vocab_token_to_id(const void *vocab, const char *token) {
  return static_cast<const ByteLevelVocab *>(vocab)->token_to_id(token ? token : "");
}

uint64_t llmcp_b200_vocab_decode(const void *vocab, const int32_t *ids, uint64_t count, char *out, uint64_t capacity) {
  return copy_text(static_cast<const ByteLevelVocab *>(vocab)->decode(ids, count), out, capacity);
}

int64_t llmcp_b200_vocab_encode(const void *vocab, const char *text, uint64_t length, int32_t *ids, uint64_t capacity) {
  std::vector<int32_t> out;
  const std::string error = static_cast<const ByteLevelVocab *>(vocab)->encode(std::string(text ? text : "", text ? length : 0), &out);
  if (!error.empty()) {
    set_error(error);
    return -1;
  }
  if (ids)
    std::memcpy(ids, out.data(), std::min<uint64_t>(out.size(), capacity) * sizeof(int32_t));
  return static_cast<int64_t>(out.size());
}

int64_t llmcp_b200_pretokenize(const char *text, uint64_t length, int64_t *ends, uint64_t capacity) {
  const std::vector<std::string> pieces = pretokenize(std::string(text ? text : "", text ? length : 0));
  int64_t end = 0;
  for (size_t i = 0; i < pieces.size(); ++i) {
    end += static_cast<int64_t>(pieces[i].size());
    if (ends && i < capacity)
      ends[i] = end;
  }
  return static_cast<int64_t>(pieces.size());
}

int64_t llmcp_b200_regex_split(const char *pattern, const char *text, uint64_t length, const char *behavior, int invert,
                               char *out, uint64_t out_capacity, int64_t *lengths, uint64_t capacity) {
  detail::Regex regex;
  detail::SplitBehavior how = detail::SplitBehavior::kIsolated;
  std::string error = regex.compile(pattern ? pattern : "");
  if (error.empty())
    error = detail::parse_split_behavior(behavior ? behavior : "isolated", &how);
  std::vector<std::string> pieces;
  if (error.empty())
    error = detail::regex_split(regex, std::string(text ? text : "", text ? length : 0), how, invert != 0, &pieces);
  if (!error.empty()) {
    set_error(error);
    return -1;
  }
  uint64_t at = 0;
  for (size_t i = 0; i < pieces.size(); ++i) {
    if (out && at + pieces[i].size() <= out_capacity)
      std::memcpy(out + at, pieces[i].data(), pieces[i].size());
    at += pieces[i].size();
    if (lengths && i < capacity)
      lengths[i] = static_cast<int64_t>(pieces[i].size());
  }
  return static_cast<int64_t>(pieces.size());
}

uint64_t llmcp_b200_normalize_nfc(const char *text, uint64_t length, char *out, uint64_t capacity) {
  return copy_text(normalize_nfc(std::string(text ? text : "", text ? length : 0)), out, capacity);
}

void *llmcp_b200_stream_create(const void *vocab) {
  return new ByteLevelStreamingDecoder(*static_cast<const ByteLevelVocab *>(vocab));
}

void llmcp_b200_stream_destroy(void *stream) { delete static_cast<ByteLevelStreamingDecoder *>(stream); }

uint64_t llmcp_b200_stream_append(void *stream, int32_t token, char *out, uint64_t capacity) {
  return copy_text(static_cast<ByteLevelStreamingDecoder *>(stream)->append(token), out, capacity);
}

uint64_t llmcp_b200_stream_finish(void *stream, char *out, uint64_t capacity) {
  return copy_text(static_cast<ByteLevelStreamingDecoder *>(stream)->finish(), out, capacity);
}

uint64_t llmcp_b200_chat_prompt(const char *user, const char *system, int thinking, char *out, uint64_t capacity) {
  return copy_text(make_chat_prompt(user ? user : "", system ? system : "", thinking != 0), out, capacity);
}

int llmcp_b200_parse_config(const char *json, uint64_t length, llmcp_b200_dims *dims) {
  return guarded_async([&] {
    ModelDims d;
    const std::string error = parse_model_config(json, length, &d);
    if (!error.empty())
      throw std::runtime_error(error);
    from_dims(d, dims);
  });
}

uint64_t llmcp_b200_read_safetensors(const char *path, char *buffer, uint64_t capacity) {
  SourceTensors tensors;
  const std::string error = read_safetensors_file(path, path, &tensors);
  if (!error.empty()) {
    set_error(error);
    return 0;
  }
  std::string text;
  for (const auto &item : tensors) {
    const SourceTensor &t = item.second;
    text += t.name + "\t" + t.dtype + "\t" + std::to_string(t.data_offset) + "\t" + std::to_string(t.data_size) + "\t";
    for (size_t i = 0; i < t.shape.size(); ++i)
      text += (i ? "," : "") + std::to_string(t.shape[i]);
    text += "\n";
  }
  if (buffer && capacity) {
    const uint64_t n = std::min<uint64_t>(capacity - 1, text.size());
    std::memcpy(buffer, text.data(), n);
    buffer[n] = 0;
  }
  return text.size();
}

int llmcp_b200_synthetic_checkpoint(const llmcp_b200_dims *dims, uint64_t seed, const char *model_dir) {
  return guarded_async([&] {
    const ModelDims d = to_dims(dims);
    check_dims(d);
    const std::string error = write_synthetic_checkpoint(d, seed, model_dir ? model_dir : "");
    if (!error.empty())
      throw std::runtime_error(error);
  });
}

int llmcp_b200_pack_checkpoint(const char *model_dir, const char *output_path, const char *quant, int dry_run,
                               int verbose, uint64_t *tensors, uint64_t *source_bytes, uint64_t *arena_bytes) {
  return guarded_async([&] {
    PackSummary summary;
    const std::string error = pack_checkpoint(model_dir ? model_dir : "", output_path ? output_path : "",
                                              quant ? quant : "none", dry_run != 0, verbose != 0, &summary);
    if (!error.empty())
      throw std::runtime_error(error);
    if (tensors)
      *tensors = summary.tensors;
    if (source_bytes)
      *source_bytes = summary.source_bytes;
    if (arena_bytes)
      *arena_bytes = summary.arena_bytes;
  });
}

void llmcp_b200_make_cos_sin(int64_t position, int64_t rotary, float theta, float *cos_out, float *sin_out) {
  make_cos_sin(position, rotary, theta, cos_out, sin_out);
}

uint64_t llmcp_b200_manifest(const uint8_t *file, uint64_t file_bytes, char *buffer, uint64_t capacity) {
  uint64_t arena = 0, offset = 0, bytes = 0;
  const std::string error = read_header(file, file_bytes, &arena, &offset, &bytes);
  if (!error.empty()) {
    set_error(error);
    return 0;
  }
  if (buffer && capacity) {
    const uint64_t n = std::min<uint64_t>(capacity - 1, bytes);
    std::memcpy(buffer, file + offset, n);
    buffer[n] = 0;
  }
  return bytes;
}

void *llmcp_b200_engine_create(const uint8_t *file, uint64_t file_bytes, const llmcp_b200_dims *dims, int64_t capacity,
                               int device) {
  try {
    const ModelDims d = to_dims(dims);
    check_dims(d);
    return new Engine(file, file_bytes, d, capacity, device);
  } catch (const std::exception &e) {
    set_error(e.what());
    return nullptr;
  }
}

void *llmcp_b200_engine_create_mode(const uint8_t *file, uint64_t file_bytes, const llmcp_b200_dims *dims, int64_t capacity,
                                    int device, int mode) {
  try {
    const ModelDims d = to_dims(dims);
    check_dims(d);
    if (mode != kModeExact && mode != kModeFast)
      throw std::runtime_error("mode must be 0 (exact) or 1 (fast)");
    return new Engine(file, file_bytes, d, capacity, device, mode);
  } catch (const std::exception &e) {
    set_error(e.what());
    return nullptr;
  }
}

uint64_t llmcp_b200_tp_slot_bytes(const llmcp_b200_dims *dims, int64_t max_tokens) {
  return Engine::tp_slot_bytes(to_dims(dims), max_tokens);
}

void *llmcp_b200_tp_create(int rank, int size, uint64_t slot_bytes, int device, uint8_t *handle_out) {
  try {
    cuda_check(cudaSetDevice(device), "cudaSetDevice");
    return new TpComm(rank, size, slot_bytes, handle_out);
  } catch (const std::exception &e) {
    set_error(e.what());
    return nullptr;
  }
}

int llmcp_b200_tp_attach(void *tp, const uint8_t *handles) {
  return guarded_async([&] { static_cast<TpComm *>(tp)->attach(handles); });
}

void llmcp_b200_tp_destroy(void *tp) { delete static_cast<TpComm *>(tp); }

int llmcp_b200_tp_all_gather(void *tp, const void *src, uint64_t row_bytes, uint64_t rows, int slot, void *dst, int *status,
                             void *stream) {
  return guarded_async([&] {
    TpComm &comm = *static_cast<TpComm *>(tp);
    const TpSegment segment = {src, static_cast<size_t>(row_bytes), static_cast<size_t>(rows), 0};
    cuda_check(comm.all_gather(&segment, 1, slot, status, static_cast<cudaStream_t>(stream)), "all-gather");
    g_launches += 1;
    if (dst)
      cuda_check(cudaMemcpyAsync(dst, comm.slot(slot), static_cast<size_t>(row_bytes) * rows * comm.size(), cudaMemcpyDeviceToDevice,
                                 static_cast<cudaStream_t>(stream)), "copy out of the slot");
  });
}

void *llmcp_b200_engine_create_tp(const uint8_t *file, uint64_t file_bytes, const llmcp_b200_dims *dims, int64_t capacity,
                                  int device, int mode, void *tp, int64_t max_tokens) {
  try {
    const ModelDims d = to_dims(dims);
    check_dims(d);
    if (mode != kModeExact && mode != kModeFast)
      throw std::runtime_error("mode must be 0 (exact) or 1 (fast)");
    return new Engine(file, file_bytes, d, capacity, device, mode, static_cast<TpComm *>(tp), max_tokens);
  } catch (const std::exception &e) {
    set_error(e.what());
    return nullptr;
  }
}

void *llmcp_b200_engine_create_batch(const uint8_t *file, uint64_t file_bytes, const llmcp_b200_dims *dims, int64_t capacity,
                                     int device, int mode, int batch) {
  try {
    const ModelDims d = to_dims(dims);
    check_dims(d);
    if (mode != kModeExact && mode != kModeFast)
      throw std::runtime_error("mode must be 0 (exact) or 1 (fast)");
    return new Engine(file, file_bytes, d, capacity, device, mode, nullptr, 1024, batch);
  } catch (const std::exception &e) {
    set_error(e.what());
    return nullptr;
  }
}

int llmcp_b200_engine_select_sequence(void *engine, int sequence) {
  return guarded_async([&] { static_cast<Engine *>(engine)->select_sequence(sequence); });
}

int llmcp_b200_engine_decode_batch(void *engine, const int64_t *tokens, int64_t position, float *logits, int64_t *argmax) {
  return guarded_async([&] {
    Engine &e = *static_cast<Engine *>(engine);
    const uint64_t before = e.launches();
    e.decode_batch(tokens, position, logits, argmax);
    g_launches += e.launches() - before;
  });
}

int llmcp_b200_engine_generate_batch(void *engine, const int64_t *first_tokens, int64_t position, int64_t steps,
                                     int64_t *out_tokens, float *device_ms) {
  return guarded_async([&] {
    Engine &e = *static_cast<Engine *>(engine);
    const uint64_t before = e.launches();
    e.generate_batch(first_tokens, position, steps, out_tokens, device_ms);
    g_launches += e.launches() - before;
  });
}

int llmcp_b200_engine_local_dims(void *engine, llmcp_b200_dims *dims, int64_t *kv_head0) {
  return guarded_async([&] {
    Engine &e = *static_cast<Engine *>(engine);
    from_dims(e.local_dims(), dims);
    if (kv_head0)
      *kv_head0 = e.kv_head0();
  });
}

void llmcp_b200_engine_destroy(void *engine) { delete static_cast<Engine *>(engine); }

int llmcp_b200_engine_reset(void *engine) {
  return guarded_async([&] { static_cast<Engine *>(engine)->reset_state(); });
}

int llmcp_b200_engine_forward(void *engine, const int64_t *tokens, int64_t S, int64_t position, float *logits,
                              int64_t *argmax) {
  return guarded_async([&] {
    Engine &e = *static_cast<Engine *>(engine);
    const uint64_t before = e.launches();
    const int64_t token = e.forward_host(tokens, S, position, nullptr, nullptr, logits);
    g_launches += e.launches() - before;
    if (argmax)
      *argmax = token;
  });
}

int llmcp_b200_engine_forward_all(void *engine, const int64_t *tokens, int64_t S, int64_t position, float *logits) {
  return guarded_async([&] {
    Engine &e = *static_cast<Engine *>(engine);
    const uint64_t before = e.launches();
    e.forward_all_host(tokens, S, position, logits);
    g_launches += e.launches() - before;
  });
}

int llmcp_b200_engine_generate(void *engine, int64_t first_token, int64_t position, int64_t steps, int64_t *out_tokens,
                               float *device_ms) {
  return guarded_async([&] {
    Engine &e = *static_cast<Engine *>(engine);
    const uint64_t before = e.launches();
    e.generate(first_token, position, steps, out_tokens, device_ms);
    g_launches += e.launches() - before;
  });
}

int llmcp_b200_engine_read_state(void *engine, uint16_t *kv, float *delta, uint16_t *conv) {
  return guarded_async([&] { static_cast<Engine *>(engine)->download_state(kv, delta, conv); });
}

int llmcp_b200_engine_read_hidden(void *engine, uint16_t *hidden) {
  return guarded_async([&] {
    Engine &e = *static_cast<Engine *>(engine);
    cuda_check(cudaMemcpy(hidden, e.final_hidden_device(), static_cast<size_t>(e.dims().hidden) * 2, cudaMemcpyDeviceToHost),
               "read hidden");
  });
}

} // extern "C"
