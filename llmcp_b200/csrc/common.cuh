// Shared device helpers for the llmcp Q8 operator kernels (sm_100a).
//
// Numerical contract of every kernel in this library: each f32 multiply, add and
// divide is a separate IEEE round-to-nearest operation unless __fmaf_rn is written
// (the library is compiled with -fmad=false), reductions run in the order the
// reference's lowering runs them, and exp/log are the f32 rounding of the
// double-precision function.  With that contract the kernels reproduce the
// reference's f32 results bit for bit, not only within a tolerance.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>
#include <set>
#include <utility>

namespace llmcp_b200 {

constexpr int kBlock = 32;          // weights per Q8_0 block (Q8PackedLayout.h:21)
constexpr int kRecordBytes = 136;   // 4 f16 scales + 8 x 16 B (Q8PackedLayout.h:24-35)

enum DType : int { kF32 = 0, kBF16 = 1 };
enum Activation : int { kNone = 0, kSilu = 1, kSigmoid = 2, kSoftplus = 3 };

__host__ __device__ inline float bf16_to_f32(uint16_t v) {
#ifdef __CUDA_ARCH__
  return __uint_as_float(static_cast<uint32_t>(v) << 16);
#else
  union { uint32_t u; float f; } c;
  c.u = static_cast<uint32_t>(v) << 16;
  return c.f;
#endif
}

// arith.truncf f32 -> bf16: round to nearest, ties to even.
__host__ __device__ inline uint16_t f32_to_bf16(float f) {
#ifdef __CUDA_ARCH__
  uint32_t bits = __float_as_uint(f);
#else
  union { uint32_t u; float f; } c;
  c.f = f;
  uint32_t bits = c.u;
#endif
  if ((bits & 0x7fffffffu) > 0x7f800000u)
    return static_cast<uint16_t>((bits >> 16) | 0x40);
  bits += 0x7fffu + ((bits >> 16) & 1u);
  return static_cast<uint16_t>(bits >> 16);
}

// The same rounding by the conversion instruction (finite values give the same bits; used by the
// fast-mode kernels, where it replaces about eight integer instructions per value).
__device__ __forceinline__ uint16_t f32_to_bf16_hw(float f) {
  uint16_t r;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(r) : "f"(f));
  return r;
}
// {lo, hi} -> one 32-bit word holding two bf16 values, lo in the low half.
__device__ __forceinline__ uint32_t f32x2_to_bf16x2_hw(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

__device__ inline float f16_bits_to_f32(uint16_t v) {
  float f;
  asm("{ .reg .b16 h; mov.b16 h, %1; cvt.f32.f16 %0, h; }" : "=f"(f) : "h"(v));
  return f;
}

__device__ inline float load_as_f32(const void *p, int dtype, int64_t i) {
  return dtype == kBF16 ? bf16_to_f32(static_cast<const uint16_t *>(p)[i])
                        : static_cast<const float *>(p)[i];
}

__device__ inline void store_from_f32(void *p, int dtype, int64_t i, float v) {
  if (dtype == kBF16)
    static_cast<uint16_t *>(p)[i] = f32_to_bf16(v);
  else
    static_cast<float *>(p)[i] = v;
}

// exp / log as the f32 rounding of the double-precision function.
__device__ inline float d_exp(float x) { return static_cast<float>(exp(static_cast<double>(x))); }
__device__ inline float d_log(float x) { return static_cast<float>(log(static_cast<double>(x))); }
// math.rsqrt lowers to 1 / sqrt(x).
__device__ inline float d_rsqrt(float x) { return __fdiv_rn(1.0f, __fsqrt_rn(x)); }
__device__ inline float d_sigmoid(float v) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, d_exp(-v))); }

// MatmulLoweringCommon.cpp:78-103
__device__ inline float apply_activation(float v, int activation) {
  switch (activation) {
  case kSilu:
    return __fmul_rn(v, d_sigmoid(v));
  case kSigmoid:
    return d_sigmoid(v);
  case kSoftplus:
    return d_log(__fadd_rn(1.0f, d_exp(v)));
  default:
    return v;
  }
}

__device__ inline int dp4a(int a, int b, int c) { return __dp4a(a, b, c); }

// Quantises 32 consecutive values held one per lane of a full warp (Q8Decode.cpp:83-120).
__device__ inline void warp_quant_block(float v, int8_t *q, float *s, int64_t element, int64_t block,
                                        int lane) {
  float amax = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = __fdiv_rn(amax, 127.0f);
  const float inv = amax == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
  q[element] = static_cast<int8_t>(__float2int_rn(__fmul_rn(v, inv)));
  if (lane == 0)
    s[block] = scale;
}

// Every kernel of the forward is launched as a programmatic dependent of the kernel in front of
// it on the stream: its CTAs may be placed once that kernel's CTAs have exited or released their
// dependents, and this call, the first statement of the kernel, holds them until that kernel
// has finished and its writes are visible.  release_early lets the kernel behind this one be
// placed right away; the kernels in front of a GEMV do that, so that the GEMV requests its
// weights while they run.  The others release at exit, which bounds the look-ahead to one kernel.
__device__ __forceinline__ void grid_dependency_sync(bool release_early = false) {
  if (release_early)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Barrier over all threads of the thread-block cluster; shared-memory stores made before it (to
// any CTA of the cluster) are visible after it.
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Stores v at the place of `local` (an address in this CTA's shared memory) in the shared memory
// of CTA `rank` of the cluster.
__device__ __forceinline__ void store_shared_cluster(float *local, int rank, float v) {
  const uint32_t mine = static_cast<uint32_t>(__cvta_generic_to_shared(local));
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(mine), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

// Raises a kernel's dynamic shared-memory limit once per (kernel, device).  The attribute belongs
// to the device that is current when it is set, so a process that drives several GPUs has to make
// the opt-in on each of them; the record of what has been done is guarded by a mutex.
inline cudaError_t opt_in_shared_memory(const void *kernel, size_t bytes) {
  static std::mutex mutex;
  static std::set<std::pair<const void *, int>> done;
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess)
    return e;
  std::lock_guard<std::mutex> lock(mutex);
  if (done.count({kernel, device}))
    return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
  if (e == cudaSuccess)
    done.insert({kernel, device});
  return e;
}

// Number of SMs of the current device.
inline cudaError_t current_sm_count(int *sms) {
  int device = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e == cudaSuccess)
    e = cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, device);
  return e;
}

// false when LLMCP_B200_PDL=0: kernels are then launched fully serialised.
bool overlap_launches_enabled();

// Launch with programmatic stream serialisation (see grid_dependency_sync).
template <typename... Params, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = overlap_launches_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// The same with thread-block clusters of cluster_x CTAs along x (grid.x a multiple of it).
template <typename... Params, typename... Args>
inline cudaError_t launch_chained_cluster(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                          int cluster_x, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = static_cast<unsigned>(cluster_x);
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = overlap_launches_enabled() ? 2 : 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

} // namespace llmcp_b200
