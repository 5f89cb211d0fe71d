// Decode GEMV for the reduction sizes of the model (K = 2560, 4096, 9216).  Q8Decode.cpp:131-225.
//
// Work split: a warp takes groups of RC consecutive rows.  A lane owns whole quantisation
// blocks: for row r and load i it fetches the 32 bytes of block 32*i + lane with one 256-bit
// streaming load (sm_100: ld.global.v8.b32, no L1 allocation, L2 evict-first, so the weights
// that are read once per token do not push the activations, KV cache and recurrent state out
// of L2).  Eight dp4a against the activation block (staged once per CTA in shared memory, the
// two 16-byte halves in separate planes so that the reads are conflict-free) give the exact
// int32 block dot.  The lane converts it, forms factor = a_scale * w_scale and parks the pair in
// the warp's shared-memory slab.  After RC rows, RC lanes walk their row's pairs in ascending
// block order:  acc = fma(float(dot), factor, acc)  -- the accumulation order that fixes the f32
// result bit for bit -- apply the activation and store.  CTAs are persistent: a warp strides
// over the groups of all matrices of the launch (up to four that share the input row).
//
// The weights do not depend on the kernel in front, only the input row does.  Launched as a
// programmatic dependent, a warp requests the first rows of its first group (registers) and
// prefetches the rest of its share into L2 before it waits for that kernel; inside the loop the
// first rows of the next group are requested before the accumulation chain of the current one.

#include "kernels.h"

namespace llmcp_b200 {

namespace {

struct Block32 {
  uint32_t v[8];
};

__device__ inline Block32 ld_block(const void *p) {
  Block32 r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7])
      : "l"(p));
  return r;
}

template <int NB, int RC> constexpr size_t rows_smem_bytes(int warps) {
  return static_cast<size_t>(NB) * 32 + NB * 4 + static_cast<size_t>(warps) * RC * (NB + 2) * sizeof(float2);
}
// NB: blocks per row (K/32).  RC: rows per group (one chain lane each).  RL: rows whose loads
// are issued together (RC % RL == 0).
template <int NB, int RC, int RL, bool DOTS>
__global__ void __launch_bounds__(256)
gemv_q8_rows_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as, const GemvJobs jobs,
                    int total_groups, int32_t *__restrict__ dots_out) {
  constexpr int K = NB * 32;
  constexpr int NL = (NB + 31) / 32; // loads per lane per row
  constexpr bool kInputInRegisters = NB <= 80;
  extern __shared__ __align__(16) unsigned char smem[];
  uint4 *a_lo = reinterpret_cast<uint4 *>(smem);           // bytes 0..15 of every activation block
  uint4 *a_hi = reinterpret_cast<uint4 *>(smem + NB * 16); // bytes 16..31
  float *as_sm = reinterpret_cast<float *>(smem + K);
  float2 *slabs = reinterpret_cast<float2 *>(smem + K + NB * 4);

  const int kWarps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int warp_in_cta = threadIdx.x >> 5;
  constexpr int kSlabStride = NB + 2; // float2 units: rows start 16-byte aligned on distinct banks
  float2 *slab = slabs + warp_in_cta * RC * kSlabStride;
  const int total_warps = gridDim.x * kWarps;
  const int first_group = blockIdx.x * kWarps + warp_in_cta;

  struct Rows {
    const int8_t *wq;
    const uint16_t *wd;
    void *y;
    int row0, activation, y_dtype, dots_offset;
  };
  // Which matrix and which rows a group stands for; warp_begin holds each matrix's first group.
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
  Block32 w[RL][NL];
  uint16_t dbits[RL][NL];
  auto load = [&](const Rows &c, int r0) {
#pragma unroll
    for (int r = 0; r < RL; ++r) {
      const int8_t *wrow = c.wq + static_cast<size_t>(c.row0 + r0 + r) * K + lane * 32;
      const uint16_t *drow = c.wd + static_cast<size_t>(c.row0 + r0 + r) * NB + lane;
#pragma unroll
      for (int i = 0; i < NL; ++i) {
        if (32 * i + 32 <= NB || lane < NB - 32 * i) {
          w[r][i] = ld_block(wrow + i * 1024);
          dbits[r][i] = __ldg(drow + 32 * i);
        }
      }
    }
  };

  // The weights do not depend on the kernel in front of this one: the first rows are requested
  // (and the rest of the warp's share prefetched into L2) before waiting for it.
  int preloaded_group = -1; // the group whose first RL rows sit in w / dbits
  if (first_group < total_groups) {
    load(resolve(first_group), 0);
    preloaded_group = first_group;
    if ((jobs.flags & kGemvPrefetchL2) && lane == 0) {
      for (int g = first_group; g < total_groups; g += total_warps) {
        const Rows p = resolve(g);
        const int skip = g == first_group ? RL : 0;
        if (RC - skip > 0) {
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.wq + static_cast<size_t>(p.row0 + skip) * K),
                       "r"((RC - skip) * K)
                       : "memory");
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p.wd + static_cast<size_t>(p.row0 + skip) * NB),
                       "r"((RC - skip) * NB * 2)
                       : "memory");
        }
      }
    }
  }
  // No early release here: the kernel behind a GEMV is placed when the GEMV's CTAs exit, which
  // keeps the look-ahead at one kernel (several matrices prefetching at once thrash L2).
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // The input row: for the short rows every lane keeps its own blocks (those it meets in every
  // row) in registers, read straight from global memory; for longer rows that costs residency,
  // so the row is staged once per CTA in shared memory instead.
  uint4 x_lo[kInputInRegisters ? NL : 1], x_hi[kInputInRegisters ? NL : 1];
  float x_scale[kInputInRegisters ? NL : 1];
  if (kInputInRegisters) {
#pragma unroll
    for (int i = 0; i < NL; ++i) {
      if (32 * i + 32 <= NB || lane < NB - 32 * i) {
        const int kb = 32 * i + lane;
        x_lo[i] = reinterpret_cast<const uint4 *>(aq)[2 * kb];
        x_hi[i] = reinterpret_cast<const uint4 *>(aq)[2 * kb + 1];
        x_scale[i] = as[kb];
      }
    }
  } else {
    for (int i = threadIdx.x; i < 2 * NB; i += blockDim.x) {
      const uint4 v = reinterpret_cast<const uint4 *>(aq)[i];
      if (i & 1)
        a_hi[i >> 1] = v;
      else
        a_lo[i >> 1] = v;
    }
    for (int i = threadIdx.x; i < NB; i += blockDim.x)
      as_sm[i] = as[i];
    __syncthreads();
  }

  // One block of one row: exact int32 dot, then (float(dot), a_scale * w_scale) into the slab.
  auto block_dot = [&](const Rows &c, int row, int i, const uint32_t (&wv)[8], uint16_t scale_bits) {
    const int kb = 32 * i + lane;
    uint4 lo, hi;
    float a_scale;
    if (kInputInRegisters) {
      lo = x_lo[i];
      hi = x_hi[i];
      a_scale = x_scale[i];
    } else {
      lo = a_lo[kb];
      hi = a_hi[kb];
      a_scale = as_sm[kb];
    }
    int dot = dp4a(static_cast<int>(wv[0]), static_cast<int>(lo.x), 0);
    dot = dp4a(static_cast<int>(wv[1]), static_cast<int>(lo.y), dot);
    dot = dp4a(static_cast<int>(wv[2]), static_cast<int>(lo.z), dot);
    dot = dp4a(static_cast<int>(wv[3]), static_cast<int>(lo.w), dot);
    dot = dp4a(static_cast<int>(wv[4]), static_cast<int>(hi.x), dot);
    dot = dp4a(static_cast<int>(wv[5]), static_cast<int>(hi.y), dot);
    dot = dp4a(static_cast<int>(wv[6]), static_cast<int>(hi.z), dot);
    dot = dp4a(static_cast<int>(wv[7]), static_cast<int>(hi.w), dot);
    const float factor = __fmul_rn(a_scale, f16_bits_to_f32(scale_bits));
    slab[row * kSlabStride + kb] = make_float2(static_cast<float>(dot), factor);
    if (DOTS)
      dots_out[static_cast<size_t>(c.dots_offset + c.row0 + row) * NB + kb] = dot;
  };
  // RC lanes walk their row's pairs in ascending block order: the reference's accumulation.
  // Sixteen pairs are fetched (eight 16-byte reads), then folded in.
  auto chain = [&](const Rows &c) {
    __syncwarp();
    if (lane < RC) {
      const float4 *mine = reinterpret_cast<const float4 *>(slab + lane * kSlabStride);
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
  };

  for (int g = first_group; g < total_groups; g += total_warps) {
    const Rows c = resolve(g);
#pragma unroll
    for (int r0 = 0; r0 < RC; r0 += RL) {
      if (!(r0 == 0 && g == preloaded_group))
        load(c, r0);
#pragma unroll
      for (int r = 0; r < RL; ++r) {
#pragma unroll
        for (int i = 0; i < NL; ++i) {
          if (32 * i + 32 <= NB || lane < NB - 32 * i)
            block_dot(c, r0 + r, i, w[r][i].v, dbits[r][i]);
        }
      }
    }
    // The registers are free: the first rows of the next group are requested now and travel
    // while the chain below runs.
    if (g + total_warps < total_groups) {
      load(resolve(g + total_warps), 0);
      preloaded_group = g + total_warps;
    }
    chain(c);
  }
}

template <int NB, int RC>
cudaError_t launch_rows(const int8_t *aq, const float *as, GemvJobs jobs, int32_t *dots_out, cudaStream_t stream) {
  // Rows loaded together: enough bytes in flight per warp without running out of registers.
  constexpr int RL = (NB <= 128 && RC >= 2) ? 2 : 1;
  int groups = 0, rows = 0;
  for (int t = 0; t < jobs.count; ++t) {
    jobs.job[t].warp_begin = groups;
    jobs.job[t].dots_offset = rows;
    groups += jobs.job[t].N / RC;
    rows += jobs.job[t].N;
  }
  int sms = 0;
  cudaError_t e = current_sm_count(&sms);
  if (e == cudaSuccess)
    e = opt_in_shared_memory(reinterpret_cast<const void *>(gemv_q8_rows_kernel<NB, RC, RL, false>), 200 * 1024);
  if (e == cudaSuccess)
    e = opt_in_shared_memory(reinterpret_cast<const void *>(gemv_q8_rows_kernel<NB, RC, RL, true>), 200 * 1024);
  if (e != cudaSuccess)
    return e;
  // Eight-warp CTAs, several per SM; with about one group per resident warp every weight byte
  // of a small matrix is requested in the first microsecond.  More groups than resident warps
  // (the vocabulary projection) are walked with a grid stride.
  constexpr int warps = 8;
  const size_t smem = rows_smem_bytes<NB, RC>(warps);
  static int ctas_per_sm = 0;
  if (ctas_per_sm == 0) {
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas_per_sm, gemv_q8_rows_kernel<NB, RC, RL, false>, warps * 32,
                                                      smem);
    if (e != cudaSuccess || ctas_per_sm < 1) {
      ctas_per_sm = 0;
      return e != cudaSuccess ? e : cudaErrorInvalidConfiguration;
    }
  }
  const int ctas = std::min((groups + warps - 1) / warps, sms * ctas_per_sm);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(ctas);
  config.blockDim = dim3(warps * 32);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = (jobs.flags & kGemvOverlapPrevious) ? 1 : 0;
  int32_t *no_dots = nullptr;
  if (dots_out)
    return cudaLaunchKernelEx(&config, gemv_q8_rows_kernel<NB, RC, RL, true>, aq, as, jobs, groups, dots_out);
  return cudaLaunchKernelEx(&config, gemv_q8_rows_kernel<NB, RC, RL, false>, aq, as, jobs, groups, no_dots);
}

template <int NI>
cudaError_t launch_rows_ni(const int8_t *aq, const float *as, const GemvJobs &jobs, int rc, int32_t *dots_out,
                           cudaStream_t stream) {
  switch (rc) {
  case 1:
    return launch_rows<NI, 1>(aq, as, jobs, dots_out, stream);
  case 2:
    return launch_rows<NI, 2>(aq, as, jobs, dots_out, stream);
  case 4:
    return launch_rows<NI, 4>(aq, as, jobs, dots_out, stream);
  default:
    return launch_rows<NI, 8>(aq, as, jobs, dots_out, stream);
  }
}

} // namespace

bool gemv_rows_supported(int K) { return K == 2560 || K == 4096 || K == 9216; }

cudaError_t launch_gemv_q8_rows(const int8_t *aq, const float *as, int K, const GemvJobs &jobs, int32_t *dots_out,
                                cudaStream_t stream, int rows_per_group) {
  int total_rows = 0;
  for (int t = 0; t < jobs.count; ++t) {
    if (jobs.job[t].N % 8 != 0)
      return cudaErrorInvalidValue;
    total_rows += jobs.job[t].N;
  }
  int rc = rows_per_group;
  if (rc != 1 && rc != 2 && rc != 4 && rc != 8) {
    // About one group per resident warp for the small matrices, eight rows once there are plenty.
    rc = 8;
    while (rc > 1 && total_rows / rc < 148 * 16)
      rc >>= 1;
    if (K == 9216 && rc > 4)
      rc = 4; // keeps the slabs of a CTA under 80 KB
  }
  switch (K) {
  case 2560:
    return launch_rows_ni<80>(aq, as, jobs, rc, dots_out, stream);
  case 4096:
    return launch_rows_ni<128>(aq, as, jobs, rc, dots_out, stream);
  case 9216:
    return launch_rows_ni<288>(aq, as, jobs, std::min(rc, 4), dots_out, stream);
  default:
    return cudaErrorInvalidValue;
  }
}

} // namespace llmcp_b200
