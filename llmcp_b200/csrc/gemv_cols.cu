// Decode GEMV for the long rows (K = 4096, 9216) of a single matrix.  Q8Decode.cpp:131-225.
//
// A CTA takes R consecutive rows and has one thread per quantisation block of a row (K/32
// threads).  Thread t meets the same input block in every row, so it keeps that block and its
// scale in registers; its R weight blocks (32 bytes each, one 256-bit streaming load per row,
// a warp reads 1 KB of a row at a time) are all requested before the kernel waits for the kernel
// in front of it, which makes the whole matrix one round of loads with nothing in shared memory
// but the (float(dot), a_scale * w_scale) pairs.  After one barrier the first R lanes walk the
// pairs of their rows in ascending block order,  acc = fma(float(dot), factor, acc)  -- the
// accumulation order that fixes the f32 result bit for bit -- R chains per instruction instead
// of one.  R is chosen so that all CTAs of the 2560-row projections are resident at once.

#include "kernels.h"

namespace llmcp_b200 {

namespace {

struct ColsBlock {
  uint32_t v[8];
};

__device__ inline ColsBlock ld_cols_block(const void *p) {
  ColsBlock r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7])
      : "l"(p));
  return r;
}

// Asks for the ranges of `next` in L2, 2 KB per request; request c of the concatenated ranges goes to
// thread c of the grid (most threads issue one request or none).  The ranges are indexed with
// constants only, so the list stays in the kernel's parameter space.
__device__ __forceinline__ void prefetch_next_weights(const PrefetchList &next, unsigned thread, unsigned threads) {
  constexpr uint32_t kShift = 11, kChunk = 1u << kShift;
  if (next.count == 0)
    return;
  uint32_t total = 0;
#pragma unroll
  for (int r = 0; r < kMaxPrefetchRanges; ++r)
    total += r < next.count ? (next.bytes[r] + kChunk - 1) >> kShift : 0u;
  for (uint32_t c = thread; c < total; c += threads) {
    uint32_t local = c, bytes = 0;
    const char *base = nullptr;
#pragma unroll
    for (int r = 0; r < kMaxPrefetchRanges; ++r) {
      const uint32_t chunks = r < next.count ? (next.bytes[r] + kChunk - 1) >> kShift : 0u;
      if (base == nullptr && local < chunks) {
        base = static_cast<const char *>(next.ptr[r]);
        bytes = next.bytes[r];
      } else if (base == nullptr) {
        local -= chunks;
      }
    }
    if (base != nullptr) {
      const uint32_t offset = local << kShift;
      const uint32_t size = min(kChunk, bytes - offset);
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + offset), "r"(size) : "memory");
    }
  }
}

// FAST: the row's block products  float(dot) * (a_scale * w_scale)  are added by a warp (lane-strided
// partial sums, then shuffles) instead of the ascending fma chain.
template <int NB, int R, bool DOTS, bool FAST>
__global__ void __launch_bounds__(NB, NB == 288 ? 2 : 5) // resident CTAs per SM that gemv_cols_supported counts on
gemv_q8_cols_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as, const int8_t *__restrict__ wq,
                    const uint16_t *__restrict__ wd, void *__restrict__ y, int N, int activation, int y_dtype,
                    int32_t *__restrict__ dots_out, const PrefetchList next) {
  constexpr int K = NB * 32;
  constexpr int kStride = NB + 2; // float2 units: rows start 16-byte aligned on distinct banks
  __shared__ __align__(16) float2 slab[R * kStride];
  const int t = threadIdx.x;
  const int row0 = blockIdx.x * R;
  const int rows = min(R, N - row0);

  ColsBlock w[R];
  uint16_t scale_bits[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    if (i < rows) {
      w[i] = ld_cols_block(wq + static_cast<size_t>(row0 + i) * K + t * 32);
      scale_bits[i] = __ldg(wd + static_cast<size_t>(row0 + i) * NB + t);
    }
  }
  prefetch_next_weights(next, blockIdx.x * NB + t, gridDim.x * NB);
  // The weights are on their way; the input row belongs to the kernel in front.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint4 lo = reinterpret_cast<const uint4 *>(aq)[2 * t];
  const uint4 hi = reinterpret_cast<const uint4 *>(aq)[2 * t + 1];
  const float a_scale = as[t];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    if (i < rows) {
      int dot = dp4a(static_cast<int>(w[i].v[0]), static_cast<int>(lo.x), 0);
      dot = dp4a(static_cast<int>(w[i].v[1]), static_cast<int>(lo.y), dot);
      dot = dp4a(static_cast<int>(w[i].v[2]), static_cast<int>(lo.z), dot);
      dot = dp4a(static_cast<int>(w[i].v[3]), static_cast<int>(lo.w), dot);
      dot = dp4a(static_cast<int>(w[i].v[4]), static_cast<int>(hi.x), dot);
      dot = dp4a(static_cast<int>(w[i].v[5]), static_cast<int>(hi.y), dot);
      dot = dp4a(static_cast<int>(w[i].v[6]), static_cast<int>(hi.z), dot);
      dot = dp4a(static_cast<int>(w[i].v[7]), static_cast<int>(hi.w), dot);
      if (FAST)
        reinterpret_cast<float *>(slab)[i * (NB + 1) + t] =
            __fmul_rn(static_cast<float>(dot), __fmul_rn(a_scale, f16_bits_to_f32(scale_bits[i])));
      else
        slab[i * kStride + t] = make_float2(static_cast<float>(dot), __fmul_rn(a_scale, f16_bits_to_f32(scale_bits[i])));
      if (DOTS)
        dots_out[static_cast<size_t>(row0 + i) * NB + t] = dot;
    }
  }
  __syncthreads();
  if (FAST) {
    const int lane = t & 31;
    for (int r = t >> 5; r < rows; r += NB / 32) {
      const float *mine = reinterpret_cast<const float *>(slab) + r * (NB + 1);
      float acc = 0.0f;
#pragma unroll
      for (int p = 0; p < NB / 32; ++p)
        acc = __fadd_rn(acc, mine[lane + 32 * p]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o));
      if (lane == 0)
        store_from_f32(y, y_dtype, row0 + r, apply_activation(acc, activation));
    }
    return;
  }
  if (t < rows) {
    const float4 *mine = reinterpret_cast<const float4 *>(slab + t * kStride);
    float acc = 0.0f;
    for (int p = 0; p < NB / 2; p += 8) {
      float4 pairs[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        pairs[u] = mine[p + u];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        acc = __fmaf_rn(pairs[u].x, pairs[u].y, acc);
        acc = __fmaf_rn(pairs[u].z, pairs[u].w, acc);
      }
    }
    store_from_f32(y, y_dtype, row0 + t, apply_activation(acc, activation));
  }
}

template <int NB, int R>
cudaError_t launch_cols(const int8_t *aq, const float *as, const GemvJob &job, int flags, int32_t *dots_out,
                        cudaStream_t stream, const PrefetchList &next) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3((job.N + R - 1) / R);
  config.blockDim = dim3(NB);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = (flags & kGemvOverlapPrevious) ? 1 : 0;
  if (dots_out)
    return cudaLaunchKernelEx(&config, gemv_q8_cols_kernel<NB, R, true, false>, aq, as, job.wq, job.wd, job.y, job.N,
                              job.activation, job.y_dtype, dots_out, next);
  int32_t *no_dots = nullptr;
  if (flags & kGemvFast)
    return cudaLaunchKernelEx(&config, gemv_q8_cols_kernel<NB, R, false, true>, aq, as, job.wq, job.wd, job.y, job.N,
                              job.activation, job.y_dtype, no_dots, next);
  return cudaLaunchKernelEx(&config, gemv_q8_cols_kernel<NB, R, false, false>, aq, as, job.wq, job.wd, job.y, job.N,
                            job.activation, job.y_dtype, no_dots, next);
}

// K = 2560 (80 blocks per row), up to four matrices that share the input row.  160 threads: thread
// t meets block t % 80 of every row it handles, and handles rows (t / 80) * 8 .. + 7 of the CTA's
// set of 16 rows, all requested at once.  CTAs are persistent: the loads of the next set are
// issued before the 16 chains of the current one run.
constexpr int kSetRows = 16;

// FAST: eight threads per row add ten block products each, then three shuffles, instead of the chain.
template <bool DOTS, bool FAST>
__global__ void __launch_bounds__(160, 4)
gemv_q8_cols80_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as, const GemvJobs jobs, int total_sets,
                      int32_t *__restrict__ dots_out) {
  constexpr int NB = 80, K = 2560, kHalf = kSetRows / 2;
  constexpr int kStride = NB + 2;
  constexpr int kFastStride = 88; // floats: the four rows a warp sums start on banks 0, 24, 16, 8
  __shared__ __align__(16) float2 slab[kSetRows * kStride];
  const int t = threadIdx.x;
  const int kb = t % NB, half = t / NB;

  struct Set {
    const int8_t *wq;
    const uint16_t *wd;
    void *y;
    int row0, activation, y_dtype, dots_offset;
  };
  // warp_begin holds each matrix's first set
  auto resolve = [&](int s) {
    Set c{jobs.job[0].wq, jobs.job[0].wd, jobs.job[0].y, 0, jobs.job[0].activation, jobs.job[0].y_dtype, 0};
    int begin = 0;
#pragma unroll
    for (int j = 1; j < kMaxGemvJobs; ++j)
      if (j < jobs.count && s >= jobs.job[j].warp_begin) {
        c.wq = jobs.job[j].wq;
        c.wd = jobs.job[j].wd;
        c.y = jobs.job[j].y;
        begin = jobs.job[j].warp_begin;
        c.activation = jobs.job[j].activation;
        c.y_dtype = jobs.job[j].y_dtype;
        c.dots_offset = jobs.job[j].dots_offset;
      }
    c.row0 = (s - begin) * kSetRows;
    return c;
  };
  ColsBlock w[kHalf];
  uint16_t scale_bits[kHalf];
  auto load = [&](const Set &c) {
#pragma unroll
    for (int i = 0; i < kHalf; ++i) {
      const size_t row = static_cast<size_t>(c.row0 + half * kHalf + i);
      w[i] = ld_cols_block(c.wq + row * K + kb * 32);
      scale_bits[i] = __ldg(c.wd + row * NB + kb);
    }
  };

  int s = blockIdx.x;
  if (s < total_sets)
    load(resolve(s));
  // Later sets of this CTA: ask for them in L2 while the kernel in front still runs.
  if ((jobs.flags & kGemvPrefetchL2) && t < kSetRows) {
    for (int later = s + gridDim.x; later < total_sets; later += gridDim.x) {
      const Set c = resolve(later);
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(c.wq + static_cast<size_t>(c.row0 + t) * K), "r"(K) : "memory");
      if (t == 0)
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(c.wd + static_cast<size_t>(c.row0) * NB),
                     "r"(kSetRows * NB * 2)
                     : "memory");
    }
  }
  prefetch_next_weights(jobs.next, blockIdx.x * 160 + t, gridDim.x * 160);
  // The weights are on their way; the input row belongs to the kernel in front.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint4 lo = reinterpret_cast<const uint4 *>(aq)[2 * kb];
  const uint4 hi = reinterpret_cast<const uint4 *>(aq)[2 * kb + 1];
  const float a_scale = as[kb];
  for (; s < total_sets; s += gridDim.x) {
    const Set c = resolve(s);
#pragma unroll
    for (int i = 0; i < kHalf; ++i) {
      int dot = dp4a(static_cast<int>(w[i].v[0]), static_cast<int>(lo.x), 0);
      dot = dp4a(static_cast<int>(w[i].v[1]), static_cast<int>(lo.y), dot);
      dot = dp4a(static_cast<int>(w[i].v[2]), static_cast<int>(lo.z), dot);
      dot = dp4a(static_cast<int>(w[i].v[3]), static_cast<int>(lo.w), dot);
      dot = dp4a(static_cast<int>(w[i].v[4]), static_cast<int>(hi.x), dot);
      dot = dp4a(static_cast<int>(w[i].v[5]), static_cast<int>(hi.y), dot);
      dot = dp4a(static_cast<int>(w[i].v[6]), static_cast<int>(hi.z), dot);
      dot = dp4a(static_cast<int>(w[i].v[7]), static_cast<int>(hi.w), dot);
      const int row = half * kHalf + i;
      if (FAST)
        reinterpret_cast<float *>(slab)[row * kFastStride + kb] =
            __fmul_rn(static_cast<float>(dot), __fmul_rn(a_scale, f16_bits_to_f32(scale_bits[i])));
      else
        slab[row * kStride + kb] = make_float2(static_cast<float>(dot), __fmul_rn(a_scale, f16_bits_to_f32(scale_bits[i])));
      if (DOTS)
        dots_out[static_cast<size_t>(c.dots_offset + c.row0 + row) * NB + kb] = dot;
    }
    __syncthreads();
    if (s + gridDim.x < total_sets)
      load(resolve(s + gridDim.x)); // travels while the sums below run
    if (FAST) {
      if (t < kSetRows * 8) {
        const int row = t >> 3, j = t & 7;
        const float *mine = reinterpret_cast<const float *>(slab) + row * kFastStride + j;
        float acc = 0.0f;
#pragma unroll
        for (int p = 0; p < NB / 8; ++p)
          acc = __fadd_rn(acc, mine[8 * p]);
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
        if (j == 0)
          store_from_f32(c.y, c.y_dtype, c.row0 + row, apply_activation(acc, c.activation));
      }
    } else if (t < kSetRows) {
      const float4 *mine = reinterpret_cast<const float4 *>(slab + t * kStride);
      float acc = 0.0f;
      for (int p = 0; p < NB / 2; p += 8) {
        float4 pairs[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          pairs[u] = mine[p + u];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          acc = __fmaf_rn(pairs[u].x, pairs[u].y, acc);
          acc = __fmaf_rn(pairs[u].z, pairs[u].w, acc);
        }
      }
      store_from_f32(c.y, c.y_dtype, c.row0 + t, apply_activation(acc, c.activation));
    }
    __syncthreads(); // the slab is free again
  }
}

cudaError_t launch_cols80(const int8_t *aq, const float *as, GemvJobs jobs, int32_t *dots_out, cudaStream_t stream) {
  int sets = 0, rows = 0;
  for (int j = 0; j < jobs.count; ++j) {
    jobs.job[j].warp_begin = sets;
    jobs.job[j].dots_offset = rows;
    sets += jobs.job[j].N / kSetRows;
    rows += jobs.job[j].N;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(std::min(sets, 148 * 4));
  config.blockDim = dim3(160);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = (jobs.flags & kGemvOverlapPrevious) ? 1 : 0;
  if (dots_out)
    return cudaLaunchKernelEx(&config, gemv_q8_cols80_kernel<true, false>, aq, as, jobs, sets, dots_out);
  int32_t *no_dots = nullptr;
  if (jobs.flags & kGemvFast)
    return cudaLaunchKernelEx(&config, gemv_q8_cols80_kernel<false, true>, aq, as, jobs, sets, no_dots);
  return cudaLaunchKernelEx(&config, gemv_q8_cols80_kernel<false, false>, aq, as, jobs, sets, no_dots);
}

// gate and up projections of the MLP with their product in one launch (K = 2560):
//   h = bf16(bf16(silu(gate . x)) * bf16(up . x)),  then the int8 quantisation of h that the down
// projection reads (Q8Decode.cpp:83-120).  A cluster of two CTAs owns one quantisation block of h:
// CTA 0 takes rows [32 u, 32 u + 32) of the gate matrix, CTA 1 the same rows of the up matrix, each
// as two sets of 16 rows through the registers -> shared memory -> row sums path of
// gemv_q8_cols80_kernel (so the launch streams like that kernel: 4 CTAs per SM, one set in flight
// per CTA).  CTA 1 then stores its 32 results into CTA 0's shared memory, and CTA 0's first warp
// forms the 32 products, their maximum and the int8 values.  Every value has the arithmetic of the
// separate linear, linear, multiply launches (FuseLinearActivations.cpp:27-77,
// LowerToLinalg.cpp:312-427).
template <bool FAST>
__global__ void __launch_bounds__(160, 4)
gemv_q8_swiglu80_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as, const int8_t *__restrict__ gate_q,
                        const uint16_t *__restrict__ gate_d, const int8_t *__restrict__ up_q,
                        const uint16_t *__restrict__ up_d, uint16_t *__restrict__ product, int8_t *__restrict__ q_out,
                        float *__restrict__ s_out, const PrefetchList next) {
  constexpr int NB = 80, K = 2560, kHalf = kSetRows / 2;
  constexpr int kStride = NB + 2;
  constexpr int kFastStride = 88;
  __shared__ __align__(16) float2 slab[kSetRows * kStride];
  __shared__ float results[4 * kSetRows]; // silu(gate) rows 0..31, then up rows 0..31, each rounded to bf16
  const int t = threadIdx.x;
  const int kb = t % NB, half = t / NB;
  const int rank = blockIdx.x & 1, unit = blockIdx.x >> 1; // clusters of two along x
  const int row_base = unit * 32;
  const int8_t *wq = rank ? up_q : gate_q;
  const uint16_t *wd = rank ? up_d : gate_d;
  const int activation = rank ? kNone : kSilu;

  ColsBlock w[kHalf];
  uint16_t scale_bits[kHalf];
  auto load = [&](int set) {
#pragma unroll
    for (int i = 0; i < kHalf; ++i) {
      const size_t row = static_cast<size_t>(row_base + set * kSetRows + half * kHalf + i);
      w[i] = ld_cols_block(wq + row * K + kb * 32);
      scale_bits[i] = __ldg(wd + row * NB + kb);
    }
  };
  load(0);
  prefetch_next_weights(next, blockIdx.x * 160 + t, gridDim.x * 160);
  // first half of a cluster barrier: by the time CTA 1 stores into CTA 0's shared memory both have started
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  // The weights are on their way; the input row belongs to the kernel in front.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const uint4 lo = reinterpret_cast<const uint4 *>(aq)[2 * kb];
  const uint4 hi = reinterpret_cast<const uint4 *>(aq)[2 * kb + 1];
  const float a_scale = as[kb];
#pragma unroll
  for (int set = 0; set < 2; ++set) {
#pragma unroll
    for (int i = 0; i < kHalf; ++i) {
      int dot = dp4a(static_cast<int>(w[i].v[0]), static_cast<int>(lo.x), 0);
      dot = dp4a(static_cast<int>(w[i].v[1]), static_cast<int>(lo.y), dot);
      dot = dp4a(static_cast<int>(w[i].v[2]), static_cast<int>(lo.z), dot);
      dot = dp4a(static_cast<int>(w[i].v[3]), static_cast<int>(lo.w), dot);
      dot = dp4a(static_cast<int>(w[i].v[4]), static_cast<int>(hi.x), dot);
      dot = dp4a(static_cast<int>(w[i].v[5]), static_cast<int>(hi.y), dot);
      dot = dp4a(static_cast<int>(w[i].v[6]), static_cast<int>(hi.z), dot);
      dot = dp4a(static_cast<int>(w[i].v[7]), static_cast<int>(hi.w), dot);
      const int row = half * kHalf + i;
      const float factor = __fmul_rn(a_scale, f16_bits_to_f32(scale_bits[i]));
      if (FAST)
        reinterpret_cast<float *>(slab)[row * kFastStride + kb] = __fmul_rn(static_cast<float>(dot), factor);
      else
        slab[row * kStride + kb] = make_float2(static_cast<float>(dot), factor);
    }
    __syncthreads();
    if (set == 0)
      load(1); // travels while the sums below run
    float *mine_out = results + rank * 2 * kSetRows + set * kSetRows;
    if (FAST) {
      if (t < kSetRows * 8) {
        const int row = t >> 3, j = t & 7;
        const float *mine = reinterpret_cast<const float *>(slab) + row * kFastStride + j;
        float acc = 0.0f;
#pragma unroll
        for (int p = 0; p < NB / 8; ++p)
          acc = __fadd_rn(acc, mine[8 * p]);
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 4));
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
        if (j == 0)
          mine_out[row] = bf16_to_f32(f32_to_bf16(apply_activation(acc, activation)));
      }
    } else if (t < kSetRows) {
      const float4 *mine = reinterpret_cast<const float4 *>(slab + t * kStride);
      float acc = 0.0f;
      for (int p = 0; p < NB / 2; p += 8) {
        float4 pairs[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          pairs[u] = mine[p + u];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          acc = __fmaf_rn(pairs[u].x, pairs[u].y, acc);
          acc = __fmaf_rn(pairs[u].z, pairs[u].w, acc);
        }
      }
      mine_out[t] = bf16_to_f32(f32_to_bf16(apply_activation(acc, activation)));
    }
    __syncthreads(); // the slab is free again; after the second set this CTA's 32 results are complete
  }
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  if (rank == 1 && t < 2 * kSetRows)
    store_shared_cluster(results + 2 * kSetRows + t, 0, results[2 * kSetRows + t]);
  cluster_sync_all();
  if (rank == 0 && t < 32) {
    const uint16_t bits = f32_to_bf16(__fmul_rn(results[t], results[2 * kSetRows + t]));
    if (product)
      product[row_base + t] = bits;
    warp_quant_block(bf16_to_f32(bits), q_out, s_out, row_base + t, unit, t);
  }
}

} // namespace

// K = 2560: up to four matrices of the layer.  K = 4096 or 9216: one matrix with few enough rows
// that one wave of CTAs covers them.
bool gemv_cols_supported(int K, const GemvJobs &jobs) {
  if (K == 2560) { // the layer projections; the vocabulary projection stays with the row kernel
    int rows = 0;
    for (int j = 0; j < jobs.count; ++j) {
      if (jobs.job[j].N % kSetRows != 0)
        return false;
      rows += jobs.job[j].N;
    }
    return rows <= 32768;
  }
  if (jobs.count != 1 || (K != 4096 && K != 9216))
    return false;
  // resident CTAs per SM by registers: 5 of 128 threads, 2 of 288 threads
  const int rows_per_cta = K == 4096 ? 8 : 9, resident = K == 4096 ? 148 * 5 : 148 * 2;
  return (jobs.job[0].N + rows_per_cta - 1) / rows_per_cta <= resident;
}

cudaError_t launch_gemv_q8_cols(const int8_t *aq, const float *as, int K, const GemvJobs &jobs, int32_t *dots_out,
                                cudaStream_t stream) {
  if (!gemv_cols_supported(K, jobs))
    return cudaErrorInvalidValue;
  if (K == 2560)
    return launch_cols80(aq, as, jobs, dots_out, stream);
  if (K == 4096)
    return launch_cols<128, 8>(aq, as, jobs.job[0], jobs.flags, dots_out, stream, jobs.next);
  return launch_cols<288, 9>(aq, as, jobs.job[0], jobs.flags, dots_out, stream, jobs.next);
}

bool gemv_swiglu_supported(int K, int64_t N) { return K == 2560 && N > 0 && N % 32 == 0; }

cudaError_t launch_gemv_q8_swiglu(const int8_t *aq, const float *as, int K, const int8_t *gate_q, const uint16_t *gate_d,
                                  const int8_t *up_q, const uint16_t *up_d, int64_t N, uint16_t *product, int8_t *q_out,
                                  float *s_out, int flags, cudaStream_t stream, const PrefetchList *next) {
  if (!gemv_swiglu_supported(K, N) || !q_out || !s_out)
    return cudaErrorInvalidValue;
  const PrefetchList ranges = next ? *next : PrefetchList{};
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(N / 32 * 2));
  config.blockDim = dim3(160);
  config.dynamicSmemBytes = 0;
  config.stream = stream;
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = 2;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = (flags & kGemvOverlapPrevious) ? 2 : 1;
  if (flags & kGemvFast)
    return cudaLaunchKernelEx(&config, gemv_q8_swiglu80_kernel<true>, aq, as, gate_q, gate_d, up_q, up_d, product, q_out, s_out, ranges);
  return cudaLaunchKernelEx(&config, gemv_q8_swiglu80_kernel<false>, aq, as, gate_q, gate_d, up_q, up_d, product, q_out, s_out, ranges);
}

} // namespace llmcp_b200
