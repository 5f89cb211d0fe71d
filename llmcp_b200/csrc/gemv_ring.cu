// Decode GEMV (Q8Decode.cpp:131-225) fed through shared memory by bulk asynchronous copies.
//
// What bounds a small decode GEMV is not bandwidth but how much of the matrix is in flight at
// once: a warp that loads a few rows, waits, computes and loads again pays the memory latency once
// per round.  Here every warp owns a ring of D shared-memory stages, one group of RC consecutive
// rows (weights, then scales: one contiguous run of each in the row-major device layout) per
// stage, filled by cp.async.bulk with completion on an mbarrier.  All D copies are issued before
// the kernel waits for the kernel in front of it (the weights do not depend on it, only the
// input row does), so a matrix that fits in the rings of all SMs is on chip when its input
// arrives, and a larger one keeps ~170 KB per SM in flight for as long as it streams.
//
// Per group: a lane takes whole 32-byte blocks from the stage, eight dp4a against the activation
// block give the exact int32 dot, (float(dot), a_scale * w_scale) are kept in registers until the
// warp has read all weights of the group, then written over them (the slab) and RC lanes walk
// their row's pairs in ascending block order:  acc = fma(float(dot), factor, acc)  -- the
// accumulation order that fixes the f32 result bit for bit.  Lane 0 then refills the stage.
//
// Every wait on a copy is bounded; if the limit runs out the kernel raises the error flag and
// reads that group from global memory instead, so the result stays correct.

#include "kernels.h"

namespace llmcp_b200 {

namespace {

constexpr uint32_t kRingSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ bool ring_wait(uint64_t *bar, uint32_t parity) {
  const uint32_t addr = smem_addr(bar);
  for (uint32_t spin = 0; spin < kRingSpinLimit; ++spin) {
    uint32_t done;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(done)
                 : "r"(addr), "r"(parity)
                 : "memory");
    if (done)
      return true;
  }
  return false;
}

template <int NB, int RC> __host__ __device__ constexpr int ring_stage_bytes() { return RC * NB * 32 + RC * NB * 2; }

template <int NB, int RC, int D> constexpr size_t ring_smem_bytes(int warps) {
  return static_cast<size_t>(NB) * 32 + NB * 4 + static_cast<size_t>(warps) * D * ring_stage_bytes<NB, RC>() +
         static_cast<size_t>(warps) * D * sizeof(uint64_t);
}

// NB: blocks per row (K/32).  RC: rows per group.  D: stages per warp.  THREADS: CTA size.
template <int NB, int RC, int D, int THREADS, bool DOTS>
__global__ void __launch_bounds__(THREADS)
gemv_q8_ring_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as, const GemvJobs jobs, int total_groups,
                    int32_t *__restrict__ dots_out, int *__restrict__ error_flag) {
  constexpr int K = NB * 32;
  constexpr int NL = (NB + 31) / 32; // blocks per lane per row
  constexpr int kWarps = THREADS / 32;
  constexpr int kStage = ring_stage_bytes<NB, RC>();
  extern __shared__ __align__(16) unsigned char smem[];
  uint4 *a_lo = reinterpret_cast<uint4 *>(smem);           // bytes 0..15 of every activation block
  uint4 *a_hi = reinterpret_cast<uint4 *>(smem + NB * 16); // bytes 16..31
  float *as_sm = reinterpret_cast<float *>(smem + K);
  const int lane = threadIdx.x & 31;
  const int warp_in_cta = threadIdx.x >> 5;
  unsigned char *ring = smem + K + NB * 4 + static_cast<size_t>(warp_in_cta) * D * kStage;
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + K + NB * 4 + static_cast<size_t>(kWarps) * D * kStage) + warp_in_cta * D;
  const int total_warps = gridDim.x * kWarps;
  const int first_group = blockIdx.x * kWarps + warp_in_cta;
  const int my_groups = first_group < total_groups ? (total_groups - first_group + total_warps - 1) / total_warps : 0;

  struct Rows {
    const int8_t *wq;
    const uint16_t *wd;
    void *y;
    int row0, activation, y_dtype, dots_offset;
  };
  auto resolve = [&](int g) {
    Rows c{jobs.job[0].wq, jobs.job[0].wd, jobs.job[0].y, 0, jobs.job[0].activation, jobs.job[0].y_dtype, 0};
    int begin = 0;
#pragma unroll
    for (int t = 1; t < kMaxGemvJobs; ++t)
      if (t < jobs.count && g >= jobs.job[t].warp_begin) {
        c.wq = jobs.job[t].wq;
        c.wd = jobs.job[t].wd;
        c.y = jobs.job[t].y;
        begin = jobs.job[t].warp_begin;
        c.activation = jobs.job[t].activation;
        c.y_dtype = jobs.job[t].y_dtype;
        c.dots_offset = jobs.job[t].dots_offset;
      }
    c.row0 = (g - begin) * RC;
    return c;
  };
  // lane 0 only: request group j of this warp into its stage
  auto request = [&](int j) {
    const Rows c = resolve(first_group + j * total_warps);
    unsigned char *stage = ring + (j % D) * kStage;
    const uint32_t bar = smem_addr(bars + (j % D));
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(static_cast<uint32_t>(kStage)) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(stage)),
                 "l"(c.wq + static_cast<size_t>(c.row0) * K), "r"(RC * K), "r"(bar)
                 : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(stage + RC * K)),
                 "l"(c.wd + static_cast<size_t>(c.row0) * NB), "r"(RC * NB * 2), "r"(bar)
                 : "memory");
  };

  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < D; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(bars + s)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    for (int j = 0; j < D && j < my_groups; ++j)
      request(j);
  }
  // The kernel behind this one is placed when this one's CTAs exit (no early release): a GEMV
  // needs the whole shared memory of an SM for its rings.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  for (int i = threadIdx.x; i < 2 * NB; i += THREADS) {
    const uint4 v = reinterpret_cast<const uint4 *>(aq)[i];
    if (i & 1)
      a_hi[i >> 1] = v;
    else
      a_lo[i >> 1] = v;
  }
  for (int i = threadIdx.x; i < NB; i += THREADS)
    as_sm[i] = as[i];
  __syncthreads();

  for (int j = 0; j < my_groups; ++j) {
    const Rows c = resolve(first_group + j * total_warps);
    unsigned char *stage = ring + (j % D) * kStage;
    const bool landed = __all_sync(0xffffffffu, ring_wait(bars + (j % D), (j / D) & 1));
    if (!landed && lane == 0 && error_flag)
      atomicExch(error_flag, 1);
    float2 pair[RC][NL];
#pragma unroll
    for (int r = 0; r < RC; ++r) {
#pragma unroll
      for (int i = 0; i < NL; ++i) {
        pair[r][i] = make_float2(0.0f, 0.0f);
        if (32 * i + 32 <= NB || lane < NB - 32 * i) {
          const int kb = 32 * i + lane;
          uint4 lo, hi;
          uint16_t scale_bits;
          if (landed) {
            const unsigned char *wrow = stage + r * K + kb * 32;
            lo = *reinterpret_cast<const uint4 *>(wrow);
            hi = *reinterpret_cast<const uint4 *>(wrow + 16);
            scale_bits = reinterpret_cast<const uint16_t *>(stage + RC * K)[r * NB + kb];
          } else { // the copy never completed: read the rows from global memory
            const int8_t *wrow = c.wq + static_cast<size_t>(c.row0 + r) * K + kb * 32;
            lo = __ldg(reinterpret_cast<const uint4 *>(wrow));
            hi = __ldg(reinterpret_cast<const uint4 *>(wrow + 16));
            scale_bits = __ldg(c.wd + static_cast<size_t>(c.row0 + r) * NB + kb);
          }
          const uint4 xl = a_lo[kb], xh = a_hi[kb];
          int dot = dp4a(static_cast<int>(lo.x), static_cast<int>(xl.x), 0);
          dot = dp4a(static_cast<int>(lo.y), static_cast<int>(xl.y), dot);
          dot = dp4a(static_cast<int>(lo.z), static_cast<int>(xl.z), dot);
          dot = dp4a(static_cast<int>(lo.w), static_cast<int>(xl.w), dot);
          dot = dp4a(static_cast<int>(hi.x), static_cast<int>(xh.x), dot);
          dot = dp4a(static_cast<int>(hi.y), static_cast<int>(xh.y), dot);
          dot = dp4a(static_cast<int>(hi.z), static_cast<int>(xh.z), dot);
          dot = dp4a(static_cast<int>(hi.w), static_cast<int>(xh.w), dot);
          pair[r][i] = make_float2(static_cast<float>(dot), __fmul_rn(as_sm[kb], f16_bits_to_f32(scale_bits)));
          if (DOTS)
            dots_out[static_cast<size_t>(c.dots_offset + c.row0 + r) * NB + kb] = dot;
        }
      }
    }
    // The weights of the group have been read by every lane: the pairs go where they were.
    // Row r's slab starts 16 bytes further per row so that the chain lanes hit distinct banks.
    __syncwarp();
#pragma unroll
    for (int r = 0; r < RC; ++r) {
      float2 *slab = reinterpret_cast<float2 *>(stage + r * K + r * 16);
#pragma unroll
      for (int i = 0; i < NL; ++i)
        if (32 * i + 32 <= NB || lane < NB - 32 * i)
          slab[32 * i + lane] = pair[r][i];
    }
    __syncwarp();
    if (lane < RC) {
      const float4 *mine = reinterpret_cast<const float4 *>(stage + lane * K + lane * 16);
      float acc = 0.0f;
      for (int p = 0; p < NB / 2; p += 8) {
        float4 t[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          t[u] = mine[p + u];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          acc = __fmaf_rn(t[u].x, t[u].y, acc);
          acc = __fmaf_rn(t[u].z, t[u].w, acc);
        }
      }
      store_from_f32(c.y, c.y_dtype, c.row0 + lane, apply_activation(acc, c.activation));
    }
    __syncwarp();
    // The stage is free: request the group that will use it next (the generic-proxy accesses
    // above are ordered before the asynchronous write by the fence).
    if (lane == 0 && j + D < my_groups) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      request(j + D);
    }
  }
}

template <int NB, int RC, int D, int THREADS>
cudaError_t launch_ring(const int8_t *aq, const float *as, GemvJobs jobs, int32_t *dots_out, int *error_flag,
                        cudaStream_t stream) {
  int groups = 0, rows = 0;
  for (int t = 0; t < jobs.count; ++t) {
    jobs.job[t].warp_begin = groups;
    jobs.job[t].dots_offset = rows;
    groups += jobs.job[t].N / RC;
    rows += jobs.job[t].N;
  }
  constexpr int warps = THREADS / 32;
  const size_t smem = ring_smem_bytes<NB, RC, D>(warps);
  static int sms = 0, ctas_per_sm = 0;
  if (sms == 0) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e == cudaSuccess)
      e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemv_q8_ring_kernel<NB, RC, D, THREADS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemv_q8_ring_kernel<NB, RC, D, THREADS, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem));
    if (e == cudaSuccess)
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas_per_sm, gemv_q8_ring_kernel<NB, RC, D, THREADS, false>, THREADS,
                                                        smem);
    if (e == cudaSuccess && ctas_per_sm < 1)
      e = cudaErrorInvalidConfiguration;
    if (e != cudaSuccess) {
      sms = 0;
      return e;
    }
  }
  const int ctas = std::min((groups + warps - 1) / warps, sms * ctas_per_sm);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(ctas);
  config.blockDim = dim3(THREADS);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = (jobs.flags & kGemvOverlapPrevious) ? 1 : 0;
  if (dots_out)
    return cudaLaunchKernelEx(&config, gemv_q8_ring_kernel<NB, RC, D, THREADS, true>, aq, as, jobs, groups, dots_out, error_flag);
  int32_t *no_dots = nullptr;
  return cudaLaunchKernelEx(&config, gemv_q8_ring_kernel<NB, RC, D, THREADS, false>, aq, as, jobs, groups, no_dots, error_flag);
}

} // namespace

bool gemv_ring_supported(int K, const GemvJobs &jobs) {
  if (K != 2560 && K != 4096 && K != 9216)
    return false;
  for (int t = 0; t < jobs.count; ++t) {
    if (jobs.job[t].N % 8 != 0)
      return false;
    // bulk copies need 16-byte aligned sources
    if ((reinterpret_cast<uintptr_t>(jobs.job[t].wq) | reinterpret_cast<uintptr_t>(jobs.job[t].wd)) & 15)
      return false;
  }
  return true;
}

cudaError_t launch_gemv_q8_ring(const int8_t *aq, const float *as, int K, const GemvJobs &jobs, int32_t *dots_out,
                                int *error_flag, cudaStream_t stream) {
  if (!gemv_ring_supported(K, jobs))
    return cudaErrorInvalidValue;
  switch (K) {
  case 2560: // 2 rows per group, 2 stages, 8 warps: 90 KB per CTA, two CTAs per SM
    return launch_ring<80, 2, 2, 256>(aq, as, jobs, dots_out, error_flag, stream);
  case 4096: // 1 row per group, 2 stages: 75 KB per CTA
    return launch_ring<128, 1, 2, 256>(aq, as, jobs, dots_out, error_flag, stream);
  default: // 9216: 1 row per group, 1 stage, 9 warps so that 2 x 9 x 148 warps cover 2560 rows at once
    return launch_ring<288, 1, 1, 288>(aq, as, jobs, dots_out, error_flag, stream);
  }
}

} // namespace llmcp_b200
