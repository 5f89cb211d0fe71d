// rms_norm, gated_rms_norm and the bf16 pointwise ops, each optionally emitting the int8
// activation quantisation that the following Q8 linear needs (so that the linear reads
// int8 + f32 block scales and no separate quantisation pass runs).
//
// Reduction order: the reference sums the squares of a row sequentially in f32
// (LowerToLinalg.cpp:251-262, DecodeNormalization.cpp:96-105).  In the default, exact
// mode one thread adds the squares in that order; every other step is elementwise.

#include <cstdlib>

#include "kernels.h"
#include "ordered_sum.cuh"

namespace llmcp_b200 {

// One CTA per row.  x = bf(a + b) when b is given (the residual add of the layer,
// LowerToLinalg.cpp:359-374), else x = a.  Outputs (each optional): sum_out = x,
// y = bf((x * rstd) * (w [+ 1])), and the block quantisation of y.
__global__ void __launch_bounds__(256)
rms_norm_kernel(const uint16_t *__restrict__ a, const uint16_t *__restrict__ b, int H,
                const void *__restrict__ w, int w_dtype, float eps, int zero_centered,
                uint16_t *__restrict__ sum_out, uint16_t *__restrict__ y, int8_t *__restrict__ q,
                float *__restrict__ s) {
  extern __shared__ float row_sm[]; // x values, then their squares
  grid_dependency_sync();
  float *sq_sm = row_sm + H;
  __shared__ float rstd_sm;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * H;
  for (int d = threadIdx.x; d < H; d += blockDim.x) {
    float v = bf16_to_f32(a[base + d]);
    if (b) {
      const uint16_t r = f32_to_bf16(__fadd_rn(v, bf16_to_f32(b[base + d])));
      if (sum_out)
        sum_out[base + d] = r;
      v = bf16_to_f32(r);
    }
    row_sm[d] = v;
    sq_sm[d] = __fmul_rn(v, v);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float sum = 0.0f;
    int d = 0;
    // Loads run ahead of the dependent adds: 32 values are fetched, then added in order.
    for (; (H & 3) == 0 && d + 32 <= H; d += 32) {
      float4 t[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        t[u] = *reinterpret_cast<const float4 *>(sq_sm + d + 4 * u);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        sum = __fadd_rn(sum, t[u].x);
        sum = __fadd_rn(sum, t[u].y);
        sum = __fadd_rn(sum, t[u].z);
        sum = __fadd_rn(sum, t[u].w);
      }
    }
    for (; d < H; ++d)
      sum = __fadd_rn(sum, sq_sm[d]);
    const float mean = __fdiv_rn(sum, static_cast<float>(H));
    rstd_sm = d_rsqrt(__fadd_rn(mean, eps));
  }
  __syncthreads();
  const float rstd = rstd_sm;
  const int lane = threadIdx.x & 31;
  const int64_t nb = H / kBlock;
  // Whole warps walk consecutive 32-element groups so that a quantisation block sits in
  // one warp; a ragged tail (H % 32) is only reachable without quantised output.
  for (int d0 = (threadIdx.x >> 5) * 32; d0 < H; d0 += blockDim.x) {
    const int d = d0 + lane;
    float out = 0.0f;
    if (d < H) {
      float wt = load_as_f32(w, w_dtype, d);
      if (zero_centered)
        wt = __fadd_rn(wt, 1.0f);
      out = bf16_to_f32(f32_to_bf16(__fmul_rn(__fmul_rn(row_sm[d], rstd), wt)));
      if (y)
        y[base + d] = f32_to_bf16(out);
    }
    if (q)
      warp_quant_block(out, q, s, base + d, blockIdx.x * nb + d0 / kBlock, lane);
  }
}

// The same operator for H % 32 == 0 with four consecutive elements per thread (8-byte loads
// and stores, all of a row's loads in flight at once); eight neighbouring lanes hold one
// quantisation block.
__global__ void __launch_bounds__(1024)
rms_norm_vec4_kernel(const uint16_t *__restrict__ a, const uint16_t *__restrict__ b, int H,
                     const void *__restrict__ w, int w_dtype, float eps, int zero_centered,
                     uint16_t *__restrict__ sum_out, uint16_t *__restrict__ y, int8_t *__restrict__ q,
                     float *__restrict__ s, int block_sum) {
  extern __shared__ __align__(16) float vrow_sm[]; // squares
  __shared__ float rstd_sm;
  __shared__ OrderedSumScratch sum_scratch;
  const int64_t base = static_cast<int64_t>(blockIdx.x) * H;
  const int quads = H >> 2;
  const int per_thread = (quads + blockDim.x - 1) / blockDim.x; // 1 for H <= 4096
  // The norm weights do not depend on the kernel in front: they are fetched before waiting for it.
  float wt[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int i = r * blockDim.x + threadIdx.x;
    if (r < per_thread && i < quads) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        wt[r][u] = load_as_f32(w, w_dtype, 4 * i + u);
        if (zero_centered)
          wt[r][u] = __fadd_rn(wt[r][u], 1.0f);
      }
    }
  }
  grid_dependency_sync(true);
  float x[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int i = r * blockDim.x + threadIdx.x;
    if (r < per_thread && i < quads) {
      const uint2 ra = reinterpret_cast<const uint2 *>(a + base)[i];
      uint32_t words[2] = {ra.x, ra.y};
      if (b) {
        const uint2 rb = reinterpret_cast<const uint2 *>(b + base)[i];
        const uint32_t wb[2] = {rb.x, rb.y};
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const uint16_t lo = f32_to_bf16(__fadd_rn(__uint_as_float(words[u] << 16), __uint_as_float(wb[u] << 16)));
          const uint16_t hi = f32_to_bf16(__fadd_rn(__uint_as_float(words[u] & 0xffff0000u), __uint_as_float(wb[u] & 0xffff0000u)));
          words[u] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
        }
        if (sum_out)
          reinterpret_cast<uint2 *>(sum_out + base)[i] = make_uint2(words[0], words[1]);
      }
      x[r][0] = __uint_as_float(words[0] << 16);
      x[r][1] = __uint_as_float(words[0] & 0xffff0000u);
      x[r][2] = __uint_as_float(words[1] << 16);
      x[r][3] = __uint_as_float(words[1] & 0xffff0000u);
      reinterpret_cast<float4 *>(vrow_sm)[i] = make_float4(__fmul_rn(x[r][0], x[r][0]), __fmul_rn(x[r][1], x[r][1]),
                                                            __fmul_rn(x[r][2], x[r][2]), __fmul_rn(x[r][3], x[r][3]));
    }
  }
  __syncthreads();
  float rstd;
  if (block_sum && per_thread == 1) {
    // The serial sum of the squares (the reference's order), evaluated by the whole block: the
    // same value bit for bit, in fewer dependent steps than the chain below.
    float sq[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    bool bad = false;
    if (static_cast<int>(threadIdx.x) < quads) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        sq[u] = __fmul_rn(x[0][u], x[0][u]);
        bad |= !(sq[u] <= 3.402823466e38f); // infinity or NaN
      }
    }
    const float mean_over = static_cast<float>(H);
    rstd = block_ordered_sum(sq, vrow_sm, H, bad, sum_scratch, [mean_over, eps](float sum) {
      return d_rsqrt(__fadd_rn(__fdiv_rn(sum, mean_over), eps));
    });
  } else {
    if (threadIdx.x == 0) {
      // One dependent chain of H adds (the reference's order); 32 squares are fetched, then added.
      float sum = 0.0f;
      for (int d = 0; d < H; d += 32) {
        float4 t[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          t[u] = *reinterpret_cast<const float4 *>(vrow_sm + d + 4 * u);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          sum = __fadd_rn(sum, t[u].x);
          sum = __fadd_rn(sum, t[u].y);
          sum = __fadd_rn(sum, t[u].z);
          sum = __fadd_rn(sum, t[u].w);
        }
      }
      rstd_sm = d_rsqrt(__fadd_rn(__fdiv_rn(sum, static_cast<float>(H)), eps));
    }
    __syncthreads();
    rstd = rstd_sm;
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    if (r >= per_thread)
      break;
    const int i = r * blockDim.x + threadIdx.x;
    const bool live = i < quads;
    float o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (live) {
#pragma unroll
      for (int u = 0; u < 4; ++u)
        o[u] = bf16_to_f32(f32_to_bf16(__fmul_rn(__fmul_rn(x[r][u], rstd), wt[r][u])));
      if (y)
        reinterpret_cast<uint2 *>(y + base)[i] =
            make_uint2(static_cast<uint32_t>(f32_to_bf16(o[0])) | (static_cast<uint32_t>(f32_to_bf16(o[1])) << 16),
                       static_cast<uint32_t>(f32_to_bf16(o[2])) | (static_cast<uint32_t>(f32_to_bf16(o[3])) << 16));
    }
    if (q) {
      float amax = fmaxf(fmaxf(fabsf(o[0]), fabsf(o[1])), fmaxf(fabsf(o[2]), fabsf(o[3])));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      if (live) {
        const float scale = __fdiv_rn(amax, 127.0f);
        const float inv = amax == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
        uint32_t packed = 0;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          packed |= (static_cast<uint32_t>(__float2int_rn(__fmul_rn(o[u], inv))) & 0xffu) << (8 * u);
        reinterpret_cast<uint32_t *>(q + base)[i] = packed;
        if ((i & 7) == 0)
          s[(base >> 5) + (i >> 3)] = scale;
      }
    }
  }
}

cudaError_t launch_rms_norm(const uint16_t *a, const uint16_t *b, int64_t M, int H, const void *w,
                            int w_dtype, float eps, int zero_centered, uint16_t *sum_out, uint16_t *y,
                            int8_t *q, float *s, cudaStream_t stream) {
  if (M == 0)
    return cudaSuccess;
  if (q && H % kBlock != 0)
    return cudaErrorInvalidValue;
  if (H % kBlock == 0 && H <= 16384) {
    // One row: a thread per four elements.  Many rows (prefill): 256-thread CTAs, so that eight
    // rows per SM run their serial sums side by side.
    // (a thread holds at most four quads, so long rows still get more threads).  Few rows get one
    // warp more where 1024 threads allow: it holds no elements and adds the head of the sum of
    // squares while the others scan (block_ordered_sum).
    const int quads = H / 4;
    const int threads = M >= 64 ? std::min(1024, std::max(256, ((quads + 3) / 4 + 31) / 32 * 32))
                                : std::min(1024, (quads + 31) / 32 * 32 + 32);
    // Few rows: the sum of squares is evaluated by the whole block (LLMCP_B200_ORDERED_SUM=0: by
    // one thread).  Many rows keep the one-thread chain: eight rows per SM hide its latency.
    static const bool block_sum_enabled = [] {
      const char *flag = std::getenv("LLMCP_B200_ORDERED_SUM");
      return !(flag && flag[0] == '0');
    }();
    const int block_sum = block_sum_enabled && M < 64 && threads * 4 >= H ? 1 : 0;
    launch_chained(rms_norm_vec4_kernel, dim3(static_cast<unsigned>(M)), dim3(threads), H * sizeof(float), stream, 
        a, b, H, w, w_dtype, eps, zero_centered, sum_out, y, q, s, block_sum);
    return cudaGetLastError();
  }
  launch_chained(rms_norm_kernel, dim3(static_cast<unsigned>(M)), dim3(256), 2 * H * sizeof(float), stream, 
      a, b, H, w, w_dtype, eps, zero_centered, sum_out, y, q, s);
  return cudaGetLastError();
}

// Fast mode.  The same operator with EPT (4 or 8) consecutive elements per thread and the sum of
// squares reduced by warp shuffles and one shared-memory table, i.e. in another order than the
// reference's serial sum: rstd can differ in its last bit, every other step is unchanged.
// Four elements per thread for rows up to 4096 (more warps, shorter dependent chains: the kernel
// is a chain of latencies, not of throughput), eight beyond; 32 / EPT neighbouring lanes hold a
// quantisation block.  bf16 roundings use the conversion instruction.
template <int EPT>
__global__ void __launch_bounds__(1024)
rms_norm_fast_kernel(const uint16_t *__restrict__ a, const uint16_t *__restrict__ b, int H,
                     const void *__restrict__ w, int w_dtype, float eps, int zero_centered,
                     uint16_t *__restrict__ sum_out, uint16_t *__restrict__ y, int8_t *__restrict__ q,
                     float *__restrict__ s) {
  constexpr int W = EPT / 2; // 32-bit words of bf16 pairs per thread
  __shared__ float warp_sums[32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * H;
  const int i = threadIdx.x;
  const bool live = i < H / EPT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  auto load_words = [&](const uint16_t *p, uint32_t *dst) {
    if (EPT == 8) {
      const uint4 r = reinterpret_cast<const uint4 *>(p)[i];
      dst[0] = r.x, dst[1] = r.y, dst[W - 2] = r.z, dst[W - 1] = r.w;
    } else {
      const uint2 r = reinterpret_cast<const uint2 *>(p)[i];
      dst[0] = r.x, dst[1] = r.y;
    }
  };
  auto store_words = [&](uint16_t *p, const uint32_t *src) {
    if (EPT == 8)
      reinterpret_cast<uint4 *>(p)[i] = make_uint4(src[0], src[1], src[W - 2], src[W - 1]);
    else
      reinterpret_cast<uint2 *>(p)[i] = make_uint2(src[0], src[1]);
  };
  // The norm weights do not depend on the kernel in front: they are fetched before waiting for it.
  float wt[EPT];
#pragma unroll
  for (int u = 0; u < EPT; ++u)
    wt[u] = 0.0f;
  if (live) {
    if (w_dtype == kBF16) {
      uint32_t ww[W];
      load_words(static_cast<const uint16_t *>(w), ww);
#pragma unroll
      for (int u = 0; u < W; ++u) {
        wt[2 * u] = __uint_as_float(ww[u] << 16);
        wt[2 * u + 1] = __uint_as_float(ww[u] & 0xffff0000u);
      }
    } else {
#pragma unroll
      for (int v = 0; v < EPT / 4; ++v) {
        const float4 w4 = reinterpret_cast<const float4 *>(w)[(EPT / 4) * i + v];
        wt[4 * v] = w4.x, wt[4 * v + 1] = w4.y, wt[4 * v + 2] = w4.z, wt[4 * v + 3] = w4.w;
      }
    }
    if (zero_centered) {
#pragma unroll
      for (int u = 0; u < EPT; ++u)
        wt[u] = __fadd_rn(wt[u], 1.0f);
    }
  }
  grid_dependency_sync(true);
  float x[EPT];
#pragma unroll
  for (int u = 0; u < EPT; ++u)
    x[u] = 0.0f;
  if (live) {
    uint32_t words[W];
    load_words(a + base, words);
    if (b) {
      uint32_t wb[W];
      load_words(b + base, wb);
#pragma unroll
      for (int u = 0; u < W; ++u)
        words[u] = f32x2_to_bf16x2_hw(__fadd_rn(__uint_as_float(words[u] << 16), __uint_as_float(wb[u] << 16)),
                                      __fadd_rn(__uint_as_float(words[u] & 0xffff0000u), __uint_as_float(wb[u] & 0xffff0000u)));
      if (sum_out)
        store_words(sum_out + base, words);
    }
#pragma unroll
    for (int u = 0; u < W; ++u) {
      x[2 * u] = __uint_as_float(words[u] << 16);
      x[2 * u + 1] = __uint_as_float(words[u] & 0xffff0000u);
    }
  }
  float part = 0.0f;
#pragma unroll
  for (int u = 0; u < EPT; ++u)
    part = __fmaf_rn(x[u], x[u], part);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, o));
  if (lane == 0)
    warp_sums[warp] = part;
  __syncthreads();
  // Every thread adds the table in the same order: lane k takes entry k, then one shuffle tree.
  float sum = lane < warps ? warp_sums[lane] : 0.0f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
  const float rstd = d_rsqrt(__fadd_rn(__fdiv_rn(sum, static_cast<float>(H)), eps));
  uint32_t wo[W];
  float o[EPT];
#pragma unroll
  for (int u = 0; u < W; ++u) {
    wo[u] = f32x2_to_bf16x2_hw(__fmul_rn(__fmul_rn(x[2 * u], rstd), wt[2 * u]), __fmul_rn(__fmul_rn(x[2 * u + 1], rstd), wt[2 * u + 1]));
    o[2 * u] = __uint_as_float(wo[u] << 16);
    o[2 * u + 1] = __uint_as_float(wo[u] & 0xffff0000u);
  }
  if (live && y)
    store_words(y + base, wo);
  if (q) { // H % 32 == 0: whole groups of 32 / EPT lanes are live or not
    float amax = 0.0f;
#pragma unroll
    for (int u = 0; u < EPT; ++u)
      amax = fmaxf(amax, fabsf(o[u]));
    if (EPT == 4)
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    if (live) {
      const float scale = __fdiv_rn(amax, 127.0f);
      const float inv = amax == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
      uint32_t packed[EPT / 4];
#pragma unroll
      for (int v = 0; v < EPT / 4; ++v) {
        packed[v] = 0u;
#pragma unroll
        for (int u = 0; u < 4; ++u)
          packed[v] |= (static_cast<uint32_t>(__float2int_rn(__fmul_rn(o[4 * v + u], inv))) & 0xffu) << (8 * u);
      }
      if (EPT == 8)
        reinterpret_cast<uint2 *>(q + base)[i] = make_uint2(packed[0], packed[EPT / 4 - 1]);
      else
        reinterpret_cast<uint32_t *>(q + base)[i] = packed[0];
      if ((i & (32 / EPT - 1)) == 0)
        s[(base >> 5) + i / (32 / EPT)] = scale;
    }
  }
}

cudaError_t launch_rms_norm_fast(const uint16_t *a, const uint16_t *b, int64_t M, int H, const void *w, int w_dtype,
                                 float eps, int zero_centered, uint16_t *sum_out, uint16_t *y, int8_t *q, float *s,
                                 cudaStream_t stream) {
  if (M == 0)
    return cudaSuccess;
  if (H % 8 != 0 || H > 8192 || (q && H % kBlock != 0))
    return cudaErrorNotSupported;
  static const int wide = [] { // LLMCP_B200_NORM_EPT=8: eight elements per thread for every row length
    const char *flag = std::getenv("LLMCP_B200_NORM_EPT");
    return flag && std::atoi(flag) == 8 ? 1 : 0;
  }();
  if (H <= 4096 && !wide) {
    const int threads = (H / 4 + 31) / 32 * 32;
    launch_chained(rms_norm_fast_kernel<4>, dim3(static_cast<unsigned>(M)), dim3(threads), 0, stream, a, b, H, w, w_dtype, eps,
                   zero_centered, sum_out, y, q, s);
  } else {
    const int threads = (H / 8 + 31) / 32 * 32;
    launch_chained(rms_norm_fast_kernel<8>, dim3(static_cast<unsigned>(M)), dim3(threads), 0, stream, a, b, H, w, w_dtype, eps,
                   zero_centered, sum_out, y, q, s);
  }
  return cudaGetLastError();
}

// One warp per (row, group).  y = bf(((x * silu(g)) * w) * rstd); with gate_activated the
// gate already holds silu(g) (LowerToLinalg.cpp:655-718, DecodeNormalization.cpp:118-131).
__global__ void __launch_bounds__(128)
gated_rms_norm_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ gate,
                      const void *__restrict__ w, int w_dtype, int64_t groups_total, int group,
                      float eps, int gate_activated, uint16_t *__restrict__ y, int8_t *__restrict__ q,
                      float *__restrict__ s) {
  extern __shared__ float sq_all[];
  grid_dependency_sync(true);
  const int lane = threadIdx.x & 31;
  const int warp_in_cta = threadIdx.x >> 5;
  const int64_t g = blockIdx.x * static_cast<int64_t>(blockDim.x >> 5) + warp_in_cta;
  if (g >= groups_total)
    return;
  float *sq = sq_all + warp_in_cta * group;
  const int64_t base = g * group;
  for (int d = lane; d < group; d += 32) {
    const float v = bf16_to_f32(x[base + d]);
    sq[d] = __fmul_rn(v, v);
  }
  __syncwarp();
  float rstd = 0.0f;
  if (lane == 0) {
    float sum = 0.0f;
    for (int d = 0; d < group; ++d)
      sum = __fadd_rn(sum, sq[d]);
    rstd = d_rsqrt(__fadd_rn(__fdiv_rn(sum, static_cast<float>(group)), eps));
  }
  rstd = __shfl_sync(0xffffffffu, rstd, 0);
  for (int d0 = 0; d0 < group; d0 += 32) {
    const int d = d0 + lane;
    float out = 0.0f;
    if (d < group) {
      const float v = bf16_to_f32(x[base + d]);
      const float gv = bf16_to_f32(gate[base + d]);
      const float silu = gate_activated ? gv : __fmul_rn(gv, d_sigmoid(gv));
      float t = __fmul_rn(v, silu);
      t = __fmul_rn(t, load_as_f32(w, w_dtype, d));
      t = __fmul_rn(t, rstd);
      const uint16_t r = f32_to_bf16(t);
      out = bf16_to_f32(r);
      if (y)
        y[base + d] = r;
    }
    if (q)
      warp_quant_block(out, q, s, base + d, (base + d0) / kBlock, lane);
  }
}

cudaError_t launch_gated_rms_norm(const uint16_t *x, const uint16_t *gate, const void *w, int w_dtype,
                                  int64_t M, int H, int group, float eps, int gate_activated,
                                  uint16_t *y, int8_t *q, float *s, cudaStream_t stream) {
  if (M == 0)
    return cudaSuccess;
  if (group <= 0 || H % group != 0 || (q && group % kBlock != 0))
    return cudaErrorInvalidValue;
  const int64_t groups_total = M * (H / group);
  const unsigned ctas = static_cast<unsigned>((groups_total + 3) / 4);
  launch_chained(gated_rms_norm_kernel, dim3(ctas), dim3(128), 4 * group * sizeof(float), stream, 
      x, gate, w, w_dtype, groups_total, group, eps, gate_activated, y, q, s);
  return cudaGetLastError();
}

// add / mul / silu_mul on bf16 operands (LowerToLinalg.cpp:312-427).  count is padded to a
// multiple of 32 by the launcher's grid; quantised output needs count % 32 == 0.
__global__ void pointwise_kernel(const uint16_t *__restrict__ a, const uint16_t *__restrict__ b,
                                 int64_t count, int op, uint16_t *__restrict__ y, int8_t *__restrict__ q,
                                 float *__restrict__ s) {
  grid_dependency_sync(true);
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  float out = 0.0f;
  if (i < count) {
    const float x = bf16_to_f32(a[i]), z = bf16_to_f32(b[i]);
    float r;
    if (op == 0)
      r = __fadd_rn(x, z);
    else if (op == 1)
      r = __fmul_rn(x, z);
    else
      r = __fmul_rn(__fmul_rn(x, d_sigmoid(x)), z);
    const uint16_t rb = f32_to_bf16(r);
    out = bf16_to_f32(rb);
    if (y)
      y[i] = rb;
  }
  if (q && (i - (threadIdx.x & 31)) < count)
    warp_quant_block(out, q, s, i, i / kBlock, threadIdx.x & 31);
}

// The same for many rows at once (count % 32 == 0, 16-byte aligned rows): eight elements per thread,
// one 16-byte load per operand, the four threads of a 32-block share the maximum with two shuffles.
// Every element goes through the operations of pointwise_kernel in the same order.
__global__ void __launch_bounds__(256)
pointwise8_kernel(const uint16_t *__restrict__ a, const uint16_t *__restrict__ b, int64_t count, int op,
                  uint16_t *__restrict__ y, int8_t *__restrict__ q, float *__restrict__ s) {
  grid_dependency_sync(true);
  const int64_t i = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) * 8;
  const bool live = i < count; // whole 32-blocks are live or not: count % 32 == 0
  float out[8];
  uint32_t words[4] = {0, 0, 0, 0};
  if (live) {
    const uint4 av = *reinterpret_cast<const uint4 *>(a + i), bv = *reinterpret_cast<const uint4 *>(b + i);
    const uint32_t aw[4] = {av.x, av.y, av.z, av.w}, bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const uint32_t ax = u & 1 ? aw[u >> 1] & 0xffff0000u : aw[u >> 1] << 16;
      const uint32_t bx = u & 1 ? bw[u >> 1] & 0xffff0000u : bw[u >> 1] << 16;
      const float x = __uint_as_float(ax), z = __uint_as_float(bx);
      float r;
      if (op == 0)
        r = __fadd_rn(x, z);
      else if (op == 1)
        r = __fmul_rn(x, z);
      else
        r = __fmul_rn(__fmul_rn(x, d_sigmoid(x)), z);
      const uint16_t rb = f32_to_bf16(r);
      out[u] = bf16_to_f32(rb);
      words[u >> 1] |= static_cast<uint32_t>(rb) << (16 * (u & 1));
    }
    if (y)
      *reinterpret_cast<uint4 *>(y + i) = make_uint4(words[0], words[1], words[2], words[3]);
  } else {
#pragma unroll
    for (int u = 0; u < 8; ++u)
      out[u] = 0.0f;
  }
  if (q) { // Q8Decode.cpp:83-120 on the 32-block these four threads hold
    float amax = 0.0f;
#pragma unroll
    for (int u = 0; u < 8; ++u)
      amax = fmaxf(amax, fabsf(out[u]));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    if (live) {
      const float scale = __fdiv_rn(amax, 127.0f);
      const float inv = amax == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
      uint32_t packed[2] = {0, 0};
#pragma unroll
      for (int u = 0; u < 8; ++u)
        packed[u >> 2] |= (static_cast<uint32_t>(__float2int_rn(__fmul_rn(out[u], inv))) & 0xffu) << (8 * (u & 3));
      *reinterpret_cast<uint2 *>(q + i) = make_uint2(packed[0], packed[1]);
      if ((threadIdx.x & 3) == 0)
        s[i >> 5] = scale;
    }
  }
}

cudaError_t launch_pointwise(const uint16_t *a, const uint16_t *b, int64_t count, int op, uint16_t *y,
                             int8_t *q, float *s, cudaStream_t stream) {
  if (count == 0)
    return cudaSuccess;
  if (q && count % kBlock != 0)
    return cudaErrorInvalidValue;
  const auto aligned = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (count % kBlock == 0 && count >= 4096 && aligned(a) && aligned(b) && aligned(y) && aligned(q)) {
    launch_chained(pointwise8_kernel, dim3(static_cast<unsigned>((count / 8 + 255) / 256)), dim3(256), 0, stream, a, b, count, op, y, q, s);
    return cudaGetLastError();
  }
  launch_chained(pointwise_kernel, dim3(static_cast<unsigned>((count + 255) / 256)), dim3(256), 0, stream, a, b, count, op, y, q, s);
  return cudaGetLastError();
}

} // namespace llmcp_b200
