// llmcp_dev_gated_delta_net_noalloc: the gated_delta_net operator for callers that must not
// allocate device memory.
//
// The operator needs a little working memory beyond its inputs and outputs: the normalised
// query and key vectors of every token and each head's beta and decay factors.  The regular
// entry points obtain it from cudaMalloc.  Some hosts cannot do that: a serving process that
// handed every byte of the GPU to its own pool at start-up (a cudaMalloc from a plugin then
// fails or eats into memory promised elsewhere), or a decode loop with a latency budget that
// cannot afford the device-wide synchronisation an allocation may imply.  For them the
// working memory lives in a fixed array that is part of the library image itself.
//
// Costs and rules that follow from that choice:
//   * the array (256 KiB) is resident on every GPU that loads the library, until exit;
//   * a call whose working set does not fit is rejected, nothing is truncated;
//   * all calls on a device share the one array.  It still holds whatever the previous call
//     left there; the kernels write every element they later read, so nothing has to be
//     cleared first.  Two calls that are in flight on the same GPU at the same time (two
//     streams, two threads) would overwrite each other's vectors: keep them ordered;
//   * the first call on each device looks up the array's device address.  Make that first
//     call during start-up, before any stream capture is begun.

#include <mutex>
#include <string>

#include "../../include/llmcp_b200.h"
#include "kernels.h"

namespace llmcp_b200 {
void report_error(const std::string &message); // api.cu
}

namespace {

constexpr size_t kScratchFloats = 64 * 1024; // 256 KiB
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_gdn_scratch[kScratchFloats];

std::mutex g_setup_mutex;
float *g_scratch_address[kMaxDevices] = {};

// In host code `g_gdn_scratch` only names the symbol; the address a kernel can use has to be
// asked for, once per device, with that device current.
float *scratch_for_current_device(std::string *error) {
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
    *error = std::string("cudaGetDevice: ") + (e != cudaSuccess ? cudaGetErrorString(e) : "device index out of range");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_address[device]) {
    void *address = nullptr;
    e = cudaGetSymbolAddress(&address, g_gdn_scratch);
    if (e != cudaSuccess || !address) {
      *error = std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e);
      return nullptr;
    }
    g_scratch_address[device] = static_cast<float *>(address);
  }
  return g_scratch_address[device];
}

} // namespace

extern "C" int llmcp_dev_gated_delta_net_noalloc(const uint16_t *conv, const uint16_t *a, const uint16_t *b,
                                                 const float *a_log, const uint16_t *dt_bias, float *state,
                                                 int64_t S, int64_t nk, int64_t nv, int64_t dk, int64_t dv,
                                                 int b_activated, uint16_t *out, void *stream) {
  using namespace llmcp_b200;
  if (S < 0 || nk <= 0 || nv <= 0 || dk <= 0 || dv <= 0 || nv % nk != 0) {
    report_error("gated_delta_net: num_v_heads must be a positive multiple of num_k_heads");
    return 1;
  }
  if (S == 0)
    return 0;
  const size_t needed = gdn_scratch_floats(S, static_cast<int>(nk), static_cast<int>(nv), static_cast<int>(dk));
  if (needed > kScratchFloats) {
    report_error("llmcp_dev_gated_delta_net_noalloc: this call needs " + std::to_string(needed) +
                 " floats of working memory, the built-in array holds " + std::to_string(kScratchFloats) +
                 "; split the tokens into smaller calls or use llmcp_op_gated_delta_net");
    return 2;
  }
  std::string error;
  float *scratch = scratch_for_current_device(&error);
  if (!scratch) {
    report_error(error);
    return 3;
  }
  const cudaError_t e = launch_gated_delta_net(conv, a, b, a_log, kF32, dt_bias, kBF16, state, S, static_cast<int>(nk),
                                               static_cast<int>(nv), static_cast<int>(dk), static_cast<int>(dv),
                                               b_activated, scratch, out, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    report_error(std::string("gated_delta_net: ") + cudaGetErrorString(e));
    return 4;
  }
  return 0;
}
