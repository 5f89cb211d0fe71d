// Q8_0-weight x int8-activation contraction for sm_100a: weight re-layout, activation
// quantisation, the decode GEMV, a CUDA-core GEMM, the embedding gather and argmax.
//
// Device weight layout ("rows"): the packed q8_0_p4 records of the arena
// (lib/Model/Quantization.cpp:165-214) are re-arranged once at load time into
//   q : int8  [N][K]      row-major, the same integers
//   d : f16   [N][K/32]   row-major, the same scale bits
// The four-row lane interleave of the arena format only serves a 4-lane SDOT; on the
// GPU a row-major plane gives 16-byte coalesced loads and is what TMA tiles for the
// tensor-core path.

#include <cstdlib>

#include "kernels.h"

namespace llmcp_b200 {

bool overlap_launches_enabled() {
  static const bool enabled = [] {
    const char *flag = std::getenv("LLMCP_B200_PDL");
    return !(flag && flag[0] == '0');
  }();
  return enabled;
}

// ---------------------------------------------------------------------------------
// Weight re-layout (one-time, at load)
// ---------------------------------------------------------------------------------
__global__ void repack_p4_kernel(const uint8_t *__restrict__ src, int64_t N, int64_t K,
                                 int8_t *__restrict__ q, uint16_t *__restrict__ d, float *__restrict__ d32) {
  grid_dependency_sync();
  const int64_t nb = K / kBlock;
  const int64_t words = N * (K / 4);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < words; i += stride) {
    const int64_t row = i / (K / 4);
    const int64_t w = i % (K / 4);
    const int64_t b = w / 8, c = w % 8;
    const uint8_t *rec = src + ((row / 4) * nb + b) * kRecordBytes;
    const uint32_t v = *reinterpret_cast<const uint32_t *>(rec + 8 + c * 16 + (row % 4) * 4);
    reinterpret_cast<uint32_t *>(q)[i] = v;
    if (c == 0) {
      const uint16_t bits = *reinterpret_cast<const uint16_t *>(rec + (row % 4) * 2);
      d[row * nb + b] = bits;
      if (d32)
        d32[row * nb + b] = f16_bits_to_f32(bits);
    }
  }
}

void launch_repack_p4(const uint8_t *src, int64_t N, int64_t K, int8_t *q, uint16_t *d, float *d32,
                      cudaStream_t stream) {
  const int64_t words = N * (K / 4);
  const int blocks = static_cast<int>(std::min<int64_t>((words + 255) / 256, 148 * 16));
  launch_chained(repack_p4_kernel, dim3(blocks), dim3(256), 0, stream, src, N, K, q, d, d32);
}

// ---------------------------------------------------------------------------------
// Activation quantisation (Q8Decode.cpp:83-120, Q8Matmul.cpp:93-141): one warp per
// 32-wide block.  scale = amax / 127 (f32, kept), q = int8(roundeven(x * (1 / scale))).
// ---------------------------------------------------------------------------------
__global__ void act_quant_kernel(const void *__restrict__ x, int x_dtype, int64_t blocks_total,
                                 int8_t *__restrict__ q, float *__restrict__ s) {
  grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int64_t warp = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  if (warp >= blocks_total)
    return;
  const int64_t i = warp * kBlock + lane;
  const float v = load_as_f32(x, x_dtype, i);
  float amax = fabsf(v);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = __fdiv_rn(amax, 127.0f);
  const float inv = amax == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
  q[i] = static_cast<int8_t>(__float2int_rn(__fmul_rn(v, inv)));
  if (lane == 0)
    s[warp] = scale;
}

void launch_act_quant(const void *x, int x_dtype, int64_t M, int64_t K, int8_t *q, float *s,
                      cudaStream_t stream) {
  const int64_t blocks_total = M * (K / kBlock);
  if (blocks_total == 0)
    return;
  const int64_t ctas = (blocks_total + 7) / 8;
  launch_chained(act_quant_kernel, dim3(static_cast<unsigned>(ctas)), dim3(256), 0, stream, x, x_dtype, blocks_total, q, s);
}

// ---------------------------------------------------------------------------------
// Decode GEMV (M = 1).  Q8Decode.cpp:131-225.
//
// A warp owns RW consecutive output rows; their int8 weights are one contiguous run of
// RW*K bytes which the 32 lanes stream with 16-byte loads.  A lane's 16 bytes are half a
// quantisation block: 4 dp4a against the matching activation words, then one shuffle with
// the neighbouring lane gives the exact int32 block dot.  The f32 accumulation
//   acc = fma(float(dot[kb]), a_scale[kb] * w_scale[kb], acc),  kb = 0 .. K/32-1
// must run in ascending kb per output (that is what fixes the result bit for bit), so the
// (float(dot), factor) pairs are staged in a per-warp slab of shared memory and RW lanes
// then run the RW chains side by side.  Up to four weight matrices that share the input
// row are served by one launch (qkv | z | a | b, gate | up, q | k | v).
// ---------------------------------------------------------------------------------
__device__ inline uint4 ld_stream_u4(const uint4 *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

template <int RW>
__global__ void __launch_bounds__(256)
gemv_q8_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as, int K,
               const GemvJobs jobs, int32_t *__restrict__ dots_out) {
  extern __shared__ __align__(16) unsigned char smem[];
  grid_dependency_sync();
  const int nb = K / kBlock;
  int8_t *a_sm = reinterpret_cast<int8_t *>(smem);
  float *as_sm = reinterpret_cast<float *>(smem + K);
  float2 *slabs = reinterpret_cast<float2 *>(smem + K + nb * 4 + ((nb & 1) ? 4 : 0));

  for (int i = threadIdx.x; i < K / 16; i += blockDim.x)
    reinterpret_cast<uint4 *>(a_sm)[i] = reinterpret_cast<const uint4 *>(aq)[i];
  for (int i = threadIdx.x; i < nb; i += blockDim.x)
    as_sm[i] = as[i];
  __syncthreads();

  const int lane = threadIdx.x & 31;
  const int warp_in_cta = threadIdx.x >> 5;
  const int warp = blockIdx.x * (blockDim.x >> 5) + warp_in_cta;

  // Which matrix does this warp work on?
  int j = 0;
#pragma unroll
  for (int t = 1; t < kMaxGemvJobs; ++t)
    if (t < jobs.count && warp >= jobs.job[t].warp_begin)
      j = t;
  const GemvJob &job = jobs.job[j];
  const int row0 = (warp - job.warp_begin) * RW;
  if (row0 >= job.N)
    return;

  float2 *slab = slabs + static_cast<size_t>(warp_in_cta) * RW * (nb + 1);
  const int pieces = K / 16; // 16-byte pieces per row
  const int total = RW * pieces;
  const uint4 *wbase = reinterpret_cast<const uint4 *>(job.wq + static_cast<size_t>(row0) * K);
  const uint16_t *dbase = job.wd + static_cast<size_t>(row0) * nb;

  constexpr int U = 8;
  for (int base = 0; base < total; base += 32 * U) {
    uint4 w[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int f = base + u * 32 + lane;
      w[u] = f < total ? ld_stream_u4(wbase + f) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int f = base + u * 32 + lane;
      const int r = f / pieces;
      const int p = f - r * pieces;
      const bool valid = f < total;
      const uint4 a = valid ? *reinterpret_cast<const uint4 *>(a_sm + p * 16) : make_uint4(0, 0, 0, 0);
      int dot = dp4a(static_cast<int>(w[u].x), static_cast<int>(a.x), 0);
      dot = dp4a(static_cast<int>(w[u].y), static_cast<int>(a.y), dot);
      dot = dp4a(static_cast<int>(w[u].z), static_cast<int>(a.z), dot);
      dot = dp4a(static_cast<int>(w[u].w), static_cast<int>(a.w), dot);
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      if (valid && !(lane & 1)) {
        const int kb = p >> 1;
        const float factor = __fmul_rn(as_sm[kb], f16_bits_to_f32(dbase[r * nb + kb]));
        slab[r * (nb + 1) + kb] = make_float2(static_cast<float>(dot), factor);
        if (dots_out)
          dots_out[static_cast<size_t>(job.dots_offset + row0 + r) * nb + kb] = dot;
      }
    }
  }
  __syncwarp();
  if (lane < RW) {
    const float2 *mine = slab + lane * (nb + 1);
    float acc = 0.0f;
#pragma unroll 8
    for (int kb = 0; kb < nb; ++kb) {
      const float2 v = mine[kb];
      acc = __fmaf_rn(v.x, v.y, acc);
    }
    const float out = apply_activation(acc, job.activation);
    store_from_f32(job.y, job.y_dtype, row0 + lane, out);
  }
}

static size_t gemv_smem_bytes(int K, int rw, int warps) {
  const int nb = K / kBlock;
  return static_cast<size_t>(K) + nb * 4 + ((nb & 1) ? 4 : 0) +
         static_cast<size_t>(warps) * rw * (nb + 1) * sizeof(float2);
}

template <int RW>
static cudaError_t gemv_launch(const int8_t *aq, const float *as, int K, GemvJobs jobs,
                               int32_t *dots_out, cudaStream_t stream) {
  constexpr int kWarps = 8;
  int warp = 0;
  int dots_rows = 0;
  for (int t = 0; t < jobs.count; ++t) {
    jobs.job[t].warp_begin = warp;
    jobs.job[t].dots_offset = dots_rows;
    warp += (jobs.job[t].N + RW - 1) / RW;
    dots_rows += jobs.job[t].N;
  }
  const int ctas = (warp + kWarps - 1) / kWarps;
  const size_t smem = gemv_smem_bytes(K, RW, kWarps);
  if (cudaError_t e = opt_in_shared_memory(reinterpret_cast<const void *>(gemv_q8_kernel<RW>), 200 * 1024); e != cudaSuccess)
    return e;
  if (smem > 200 * 1024)
    return cudaErrorInvalidValue;
  launch_chained(gemv_q8_kernel<RW>, dim3(ctas), dim3(kWarps * 32), smem, stream, aq, as, K, jobs, dots_out);
  return cudaGetLastError();
}

cudaError_t launch_gemv_q8(const int8_t *aq, const float *as, int K, const GemvJobs &jobs,
                           int32_t *dots_out, cudaStream_t stream, int rows_per_warp) {
  if (jobs.count < 1 || jobs.count > kMaxGemvJobs || K % kBlock != 0)
    return cudaErrorInvalidValue;
  if (!(jobs.flags & kGemvNoCols) && rows_per_warp == 0 && gemv_cols_supported(K, jobs))
    return launch_gemv_q8_cols(aq, as, K, jobs, dots_out, stream);
  if (gemv_rows_supported(K) && rows_per_warp >= 0)
    return launch_gemv_q8_rows(aq, as, K, jobs, dots_out, stream, rows_per_warp);
  if (rows_per_warp < 0)
    rows_per_warp = 0; // negative: force the general kernel
  int total_rows = 0;
  for (int t = 0; t < jobs.count; ++t)
    total_rows += jobs.job[t].N;
  int rw = rows_per_warp;
  if (rw <= 0) {
    // Enough warps to keep ~24 per SM streaming; more rows per warp once there are plenty.
    rw = 8;
    while (rw > 1 && total_rows / rw < 148 * 24)
      rw >>= 1;
    while (rw > 1 && gemv_smem_bytes(K, rw, 8) > 64 * 1024)
      rw >>= 1;
  }
  switch (rw) {
  case 1:
    return gemv_launch<1>(aq, as, K, jobs, dots_out, stream);
  case 2:
    return gemv_launch<2>(aq, as, K, jobs, dots_out, stream);
  case 4:
    return gemv_launch<4>(aq, as, K, jobs, dots_out, stream);
  case 8:
    return gemv_launch<8>(aq, as, K, jobs, dots_out, stream);
  default:
    return cudaErrorInvalidValue;
  }
}

// ---------------------------------------------------------------------------------
// GEMM on CUDA cores (M > 1).  Q8Matmul.cpp:143-289.  64 x 64 output tile per CTA,
// 4 x 4 outputs per thread, one quantisation block of K per step; every output keeps its
// own ascending-kb fma chain, so results equal the GEMV's bit for bit.
// ---------------------------------------------------------------------------------
constexpr int kTile = 64;

__global__ void __launch_bounds__(256)
gemm_q8_dp4a_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as, int M, int K,
                    const int8_t *__restrict__ wq, const uint16_t *__restrict__ wd, int N,
                    void *__restrict__ y, int y_dtype, int activation, int32_t *__restrict__ dots_out) {
  __shared__ __align__(16) uint32_t a_sm[kTile][9]; // 8 words per row + 1 pad
  __shared__ __align__(16) uint32_t w_sm[kTile][9];
  __shared__ float as_sm[kTile];
  __shared__ float wd_sm[kTile];
  grid_dependency_sync();
  const int nb = K / kBlock;
  const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4; // tx -> columns, ty -> rows
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int jx = 0; jx < 4; ++jx)
      acc[i][jx] = 0.0f;

  for (int kb = 0; kb < nb; ++kb) {
    // 64 rows x 8 words for each operand: 512 words, 2 per thread.
    for (int i = threadIdx.x; i < kTile * 8; i += 256) {
      const int r = i >> 3, c = i & 7;
      const int m = m0 + r, n = n0 + r;
      a_sm[r][c] = m < M ? reinterpret_cast<const uint32_t *>(aq + static_cast<size_t>(m) * K + kb * kBlock)[c] : 0u;
      w_sm[r][c] = n < N ? reinterpret_cast<const uint32_t *>(wq + static_cast<size_t>(n) * K + kb * kBlock)[c] : 0u;
    }
    if (threadIdx.x < kTile) {
      const int m = m0 + threadIdx.x;
      as_sm[threadIdx.x] = m < M ? as[static_cast<size_t>(m) * nb + kb] : 0.0f;
    } else if (threadIdx.x < 2 * kTile) {
      const int n = n0 + threadIdx.x - kTile;
      wd_sm[threadIdx.x - kTile] = n < N ? f16_bits_to_f32(wd[static_cast<size_t>(n) * nb + kb]) : 0.0f;
    }
    __syncthreads();
    int dot[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int jx = 0; jx < 4; ++jx)
        dot[i][jx] = 0;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      int a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[i] = static_cast<int>(a_sm[ty * 4 + i][c]);
        w[i] = static_cast<int>(w_sm[tx * 4 + i][c]);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int jx = 0; jx < 4; ++jx)
          dot[i][jx] = dp4a(a[i], w[jx], dot[i][jx]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float sa = as_sm[ty * 4 + i];
#pragma unroll
      for (int jx = 0; jx < 4; ++jx) {
        const float factor = __fmul_rn(sa, wd_sm[tx * 4 + jx]);
        acc[i][jx] = __fmaf_rn(static_cast<float>(dot[i][jx]), factor, acc[i][jx]);
        if (dots_out) {
          const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + jx;
          if (m < M && n < N)
            dots_out[(static_cast<size_t>(m) * N + n) * nb + kb] = dot[i][jx];
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M)
      continue;
#pragma unroll
    for (int jx = 0; jx < 4; ++jx) {
      const int n = n0 + tx * 4 + jx;
      if (n < N)
        store_from_f32(y, y_dtype, static_cast<int64_t>(m) * N + n, apply_activation(acc[i][jx], activation));
    }
  }
}

cudaError_t launch_gemm_q8_dp4a(const int8_t *aq, const float *as, int M, int K, const int8_t *wq,
                                const uint16_t *wd, int N, void *y, int y_dtype, int activation,
                                int32_t *dots_out, cudaStream_t stream) {
  dim3 grid((N + kTile - 1) / kTile, (M + kTile - 1) / kTile);
  launch_chained(gemm_q8_dp4a_kernel, dim3(grid), dim3(256), 0, stream, aq, as, M, K, wq, wd, N, y, y_dtype, activation, dots_out);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------
// Embedding gather (LowerToLinalg.cpp:435-531): bf16(float(q) * float(f16 scale)).
// ---------------------------------------------------------------------------------
// A token id outside [0, vocab) reads nothing: its row is written as zeros and bit 1 of *status
// (optional) is raised, which the host turns into an error after the call.
__global__ void embedding_q8_kernel(const int64_t *__restrict__ tokens, int64_t S, int64_t hidden, int64_t vocab,
                                    const int8_t *__restrict__ wq, const uint16_t *__restrict__ wd,
                                    uint16_t *__restrict__ out, int *__restrict__ status) {
  grid_dependency_sync();
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i >= S * hidden)
    return;
  const int64_t r = i / hidden, c = i % hidden;
  const int64_t token = tokens[r];
  if (token < 0 || token >= vocab) {
    out[i] = 0;
    if (status && c == 0)
      atomicOr(status, 2);
    return;
  }
  const float scale = f16_bits_to_f32(wd[token * (hidden / kBlock) + c / kBlock]);
  out[i] = f32_to_bf16(__fmul_rn(static_cast<float>(wq[token * hidden + c]), scale));
}

void launch_embedding_q8(const int64_t *tokens, int64_t S, int64_t hidden, int64_t vocab, const int8_t *wq,
                         const uint16_t *wd, uint16_t *out, int *status, cudaStream_t stream) {
  const int64_t total = S * hidden;
  launch_chained(embedding_q8_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, stream, tokens, S, hidden,
                 vocab, wq, wd, out, status);
}

// ---------------------------------------------------------------------------------
// argmax with std::max_element semantics (first maximum; llmcp-benchmark.cpp:51-54).
// ---------------------------------------------------------------------------------
__device__ inline void argmax_merge(float &bv, int64_t &bi, float v, int64_t i) {
  if (v > bv || (v == bv && i < bi)) {
    bv = v;
    bi = i;
  }
}

// blockIdx.y: row of a [rows, n] matrix (one argmax per row).
__global__ void argmax_partial_kernel(const float *__restrict__ x, int64_t n, float *__restrict__ pv,
                                      int64_t *__restrict__ pi) {
  __shared__ float sv[32];
  __shared__ int64_t si[32];
  grid_dependency_sync();
  x += static_cast<int64_t>(blockIdx.y) * n;
  pv += blockIdx.y * gridDim.x;
  pi += blockIdx.y * gridDim.x;
  float bv = -INFINITY;
  int64_t bi = INT64_MAX;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n; i += stride)
    argmax_merge(bv, bi, x[i], i);
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_merge(bv, bi, ov, oi);
  }
  if ((threadIdx.x & 31) == 0) {
    sv[threadIdx.x >> 5] = bv;
    si[threadIdx.x >> 5] = bi;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int warps = blockDim.x >> 5;
    bv = threadIdx.x < warps ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < warps ? si[threadIdx.x] : INT64_MAX;
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
      argmax_merge(bv, bi, ov, oi);
    }
    if (threadIdx.x == 0) {
      pv[blockIdx.x] = bv;
      pi[blockIdx.x] = bi;
    }
  }
}

__global__ void argmax_final_kernel(const float *__restrict__ pv, const int64_t *__restrict__ pi, int parts,
                                    int64_t index_base, int64_t *__restrict__ out_index,
                                    float *__restrict__ out_value) {
  grid_dependency_sync();
  pv += blockIdx.x * parts; // blockIdx.x: row
  pi += blockIdx.x * parts;
  out_index += blockIdx.x;
  if (out_value)
    out_value += blockIdx.x;
  float bv = -INFINITY;
  int64_t bi = INT64_MAX;
  for (int i = threadIdx.x; i < parts; i += 32)
    argmax_merge(bv, bi, pv[i], pi[i]);
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int64_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
    argmax_merge(bv, bi, ov, oi);
  }
  if (threadIdx.x == 0) {
    *out_index = bi + index_base;
    if (out_value)
      *out_value = bv;
  }
}

void launch_argmax(const float *x, int64_t n, float *scratch_v, int64_t *scratch_i, int64_t index_base,
                   int64_t *out_index, float *out_value, cudaStream_t stream, int rows) {
  const int parts = static_cast<int>(std::min<int64_t>((n + 1023) / 1024, kArgmaxParts / std::max(1, rows)));
  launch_chained(argmax_partial_kernel, dim3(std::max(parts, 1), rows), dim3(256), 0, stream, x, n, scratch_v, scratch_i);
  launch_chained(argmax_final_kernel, dim3(rows), dim3(32), 0, stream, scratch_v, scratch_i, std::max(parts, 1), index_base, out_index,
                 out_value);
}

} // namespace llmcp_b200
