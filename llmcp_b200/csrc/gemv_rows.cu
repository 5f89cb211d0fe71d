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

constexpr int kWarps = 8;

template <int NB, int RC> constexpr size_t rows_smem_bytes() {
  return static_cast<size_t>(NB) * 32 + NB * 4 + static_cast<size_t>(kWarps) * RC * (NB + 1) * sizeof(float2);
}

// NB: blocks per row (K/32).  RC: rows per group (one chain lane each).  RL: rows whose loads
// are issued together (RC % RL == 0).
template <int NB, int RC, int RL, bool DOTS>
__global__ void __launch_bounds__(kWarps * 32)
gemv_q8_rows_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as, const GemvJobs jobs,
                    int total_groups, int32_t *__restrict__ dots_out) {
  constexpr int K = NB * 32;
  constexpr int NL = (NB + 31) / 32; // loads per lane per row
  extern __shared__ __align__(16) unsigned char smem[];
  uint4 *a_lo = reinterpret_cast<uint4 *>(smem);           // bytes 0..15 of every activation block
  uint4 *a_hi = reinterpret_cast<uint4 *>(smem + NB * 16); // bytes 16..31
  float *as_sm = reinterpret_cast<float *>(smem + K);
  float2 *slabs = reinterpret_cast<float2 *>(smem + K + NB * 4);

  for (int i = threadIdx.x; i < 2 * NB; i += kWarps * 32) {
    const uint4 v = reinterpret_cast<const uint4 *>(aq)[i];
    if (i & 1)
      a_hi[i >> 1] = v;
    else
      a_lo[i >> 1] = v;
  }
  for (int i = threadIdx.x; i < NB; i += kWarps * 32)
    as_sm[i] = as[i];
  __syncthreads();

  const int lane = threadIdx.x & 31;
  const int warp_in_cta = threadIdx.x >> 5;
  float2 *slab = slabs + warp_in_cta * RC * (NB + 1);
  const int total_warps = gridDim.x * kWarps;

  for (int g = blockIdx.x * kWarps + warp_in_cta; g < total_groups; g += total_warps) {
    // Which matrix, which rows.  warp_begin holds the first group of each matrix.
    const int8_t *wq = jobs.job[0].wq;
    const uint16_t *wd = jobs.job[0].wd;
    void *y = jobs.job[0].y;
    int begin = 0, activation = jobs.job[0].activation, y_dtype = jobs.job[0].y_dtype, dots_offset = 0;
#pragma unroll
    for (int t = 1; t < kMaxGemvJobs; ++t)
      if (t < jobs.count && g >= jobs.job[t].warp_begin) {
        wq = jobs.job[t].wq;
        wd = jobs.job[t].wd;
        y = jobs.job[t].y;
        begin = jobs.job[t].warp_begin;
        activation = jobs.job[t].activation;
        y_dtype = jobs.job[t].y_dtype;
        dots_offset = jobs.job[t].dots_offset;
      }
    const int row0 = (g - begin) * RC;

#pragma unroll
    for (int r0 = 0; r0 < RC; r0 += RL) {
      Block32 w[RL][NL];
      uint16_t dbits[RL][NL];
#pragma unroll
      for (int r = 0; r < RL; ++r) {
        const int8_t *wrow = wq + static_cast<size_t>(row0 + r0 + r) * K + lane * 32;
        const uint16_t *drow = wd + static_cast<size_t>(row0 + r0 + r) * NB + lane;
#pragma unroll
        for (int i = 0; i < NL; ++i) {
          if (32 * i + 32 <= NB || lane < NB - 32 * i) {
            w[r][i] = ld_block(wrow + i * 1024);
            dbits[r][i] = __ldg(drow + 32 * i);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < RL; ++r) {
#pragma unroll
        for (int i = 0; i < NL; ++i) {
          if (32 * i + 32 <= NB || lane < NB - 32 * i) {
            const int kb = 32 * i + lane;
            const uint4 lo = a_lo[kb], hi = a_hi[kb];
            int dot = dp4a(static_cast<int>(w[r][i].v[0]), static_cast<int>(lo.x), 0);
            dot = dp4a(static_cast<int>(w[r][i].v[1]), static_cast<int>(lo.y), dot);
            dot = dp4a(static_cast<int>(w[r][i].v[2]), static_cast<int>(lo.z), dot);
            dot = dp4a(static_cast<int>(w[r][i].v[3]), static_cast<int>(lo.w), dot);
            dot = dp4a(static_cast<int>(w[r][i].v[4]), static_cast<int>(hi.x), dot);
            dot = dp4a(static_cast<int>(w[r][i].v[5]), static_cast<int>(hi.y), dot);
            dot = dp4a(static_cast<int>(w[r][i].v[6]), static_cast<int>(hi.z), dot);
            dot = dp4a(static_cast<int>(w[r][i].v[7]), static_cast<int>(hi.w), dot);
            const float factor = __fmul_rn(as_sm[kb], f16_bits_to_f32(dbits[r][i]));
            slab[(r0 + r) * (NB + 1) + kb] = make_float2(static_cast<float>(dot), factor);
            if (DOTS)
              dots_out[static_cast<size_t>(dots_offset + row0 + r0 + r) * NB + kb] = dot;
          }
        }
      }
    }
    __syncwarp();
    if (lane < RC) {
      const float2 *mine = slab + lane * (NB + 1);
      float acc = 0.0f;
#pragma unroll 16
      for (int kb = 0; kb < NB; ++kb) {
        const float2 v = mine[kb];
        acc = __fmaf_rn(v.x, v.y, acc);
      }
      store_from_f32(y, y_dtype, row0 + lane, apply_activation(acc, activation));
    }
    __syncwarp();
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
  constexpr size_t smem = rows_smem_bytes<NB, RC>();
  static int ctas_per_sm = 0;
  if (ctas_per_sm == 0) {
    cudaError_t e = cudaFuncSetAttribute(gemv_q8_rows_kernel<NB, RC, RL, false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemv_q8_rows_kernel<NB, RC, RL, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(smem));
    if (e == cudaSuccess)
      e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas_per_sm, gemv_q8_rows_kernel<NB, RC, RL, false>,
                                                        kWarps * 32, smem);
    if (e != cudaSuccess)
      return e;
    if (ctas_per_sm < 1)
      return cudaErrorInvalidConfiguration;
  }
  int sms = 148;
  int device = 0;
  if (cudaGetDevice(&device) == cudaSuccess)
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const int ctas = std::min((groups + kWarps - 1) / kWarps, sms * ctas_per_sm);
  if (dots_out)
    gemv_q8_rows_kernel<NB, RC, RL, true><<<ctas, kWarps * 32, smem, stream>>>(aq, as, jobs, groups, dots_out);
  else
    gemv_q8_rows_kernel<NB, RC, RL, false><<<ctas, kWarps * 32, smem, stream>>>(aq, as, jobs, groups, nullptr);
  return cudaGetLastError();
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
