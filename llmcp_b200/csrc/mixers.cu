// Token mixers of the Qwen3.5 layers: causal_conv1d, the gated_delta_net recurrence and
// the gated GQA attention.  Every reduction keeps the reference's order (see common.cuh),
// and parallelism comes only from dimensions the reference treats as independent:
// channels and time for the convolution, value columns and heads for the recurrence,
// keys (scores) and head-dim lanes (weighted sum) for attention.

#include <cstdlib>

#include "kernels.h"

namespace llmcp_b200 {

// ---------------------------------------------------------------------------------
// causal_conv1d + SiLU (LowerCausalConv1d.cpp:74-182).  state: [kernel-1, C] bf16.
// ---------------------------------------------------------------------------------
__global__ void causal_conv1d_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ w,
                                     const uint16_t *__restrict__ state, int64_t S, int C, int kernel,
                                     uint16_t *__restrict__ y) {
  grid_dependency_sync();
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  if (i >= S * C)
    return;
  const int64_t t = i / C;
  const int c = static_cast<int>(i % C);
  const int state_len = kernel - 1;
  float acc = 0.0f;
  for (int k = 0; k < kernel; ++k) {
    const int64_t src = t + k - state_len;
    const uint16_t raw = src < 0 ? state[(src + state_len) * C + c] : x[src * C + c];
    acc = __fadd_rn(acc, __fmul_rn(bf16_to_f32(raw), bf16_to_f32(w[c * kernel + k])));
  }
  y[i] = f32_to_bf16(__fmul_rn(acc, d_sigmoid(acc)));
}

// The same with eight channels per thread (C % 8 == 0, kernel == 4): 16-byte loads of the four input
// rows and of the channels' 32 taps; every output goes through the operations above in the same order.
__global__ void __launch_bounds__(256)
causal_conv1d8_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ w, const uint16_t *__restrict__ state,
                      int64_t S, int C, uint16_t *__restrict__ y) {
  constexpr int kernel = 4, state_len = 3;
  grid_dependency_sync();
  const int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int groups = C / 8;
  if (i >= S * groups)
    return;
  const int64_t t = i / groups;
  const int c0 = static_cast<int>(i % groups) * 8;
  uint4 rows[kernel];
#pragma unroll
  for (int k = 0; k < kernel; ++k) {
    const int64_t src = t + k - state_len;
    rows[k] = *reinterpret_cast<const uint4 *>(src < 0 ? state + (src + state_len) * C + c0 : x + src * C + c0);
  }
  uint4 taps[4]; // w[(c0 + j) * 4 + k], j = 0..7: 32 consecutive bf16 values
#pragma unroll
  for (int v = 0; v < 4; ++v)
    taps[v] = reinterpret_cast<const uint4 *>(w + static_cast<int64_t>(c0) * kernel)[v];
  const uint16_t *tap = reinterpret_cast<const uint16_t *>(taps);
  uint32_t out[4] = {0, 0, 0, 0};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float acc = 0.0f;
#pragma unroll
    for (int k = 0; k < kernel; ++k) {
      const uint16_t raw = reinterpret_cast<const uint16_t *>(&rows[k])[j];
      acc = __fadd_rn(acc, __fmul_rn(bf16_to_f32(raw), bf16_to_f32(tap[j * kernel + k])));
    }
    out[j >> 1] |= static_cast<uint32_t>(f32_to_bf16(__fmul_rn(acc, d_sigmoid(acc)))) << (16 * (j & 1));
  }
  *reinterpret_cast<uint4 *>(y + t * C + c0) = make_uint4(out[0], out[1], out[2], out[3]);
}

// New state = last kernel-1 rows of [state; x]; one thread per channel walks the rows in
// ascending order, which is the order the in-place update needs.
__global__ void conv_state_kernel(const uint16_t *__restrict__ x, uint16_t *__restrict__ state, int64_t S,
                                  int C, int kernel) {
  grid_dependency_sync();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C)
    return;
  const int state_len = kernel - 1;
  for (int s = 0; s < state_len; ++s) {
    const int64_t src = S - state_len + s;
    state[s * C + c] = src < 0 ? state[(src + state_len) * C + c] : x[src * C + c];
  }
}

cudaError_t launch_causal_conv1d(const uint16_t *x, const uint16_t *w, uint16_t *state, int64_t S, int C,
                                 int kernel, uint16_t *y, cudaStream_t stream) {
  if (S == 0)
    return cudaSuccess;
  const int64_t total = S * C;
  const auto aligned = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (kernel == 4 && C % 8 == 0 && S >= 16 && aligned(x) && aligned(w) && aligned(state) && aligned(y))
    launch_chained(causal_conv1d8_kernel, dim3(static_cast<unsigned>((total / 8 + 255) / 256)), dim3(256), 0, stream, x, w, state, S, C, y);
  else
    launch_chained(causal_conv1d_kernel, dim3(static_cast<unsigned>((total + 255) / 256)), dim3(256), 0, stream, x, w, state, S, C, kernel, y);
  launch_chained(conv_state_kernel, dim3((C + 255) / 256), dim3(256), 0, stream, x, state, S, C, kernel);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------
// gated_delta_net (LowerGatedDeltaNet.cpp:129-445).
//
// Step 1 (parallel over tokens): L2-normalised q and k per key head, beta and decay per
// value head.  Step 2 (sequential over tokens, parallel over value columns): one thread
// owns column v of a head's [dk, dv] state, keeps it in registers across the tokens of the
// call, and runs the two ascending-k chains of each token.
// ---------------------------------------------------------------------------------
// One warp per (token, key head) for the two norms (lane 0 adds the q squares in order,
// lane 1 the k squares), then one thread per (token, value head) for beta and decay.
__global__ void __launch_bounds__(128)
gdn_prepare_kernel(const uint16_t *__restrict__ conv, const uint16_t *__restrict__ a,
                   const uint16_t *__restrict__ b, const void *__restrict__ a_log, int a_log_dtype,
                   const void *__restrict__ dt_bias, int dt_dtype, int64_t S, int nk, int nv, int ab_stride, int dk, int dv,
                   int b_activated, float *__restrict__ qn, float *__restrict__ kn, float *__restrict__ beta,
                   float *__restrict__ decay) {
  extern __shared__ float prep_all[]; // per warp: q squares [dk], k squares [dk]
  grid_dependency_sync();
  const int lane = threadIdx.x & 31;
  const int warp_in_cta = threadIdx.x >> 5;
  const int64_t warp = blockIdx.x * static_cast<int64_t>(blockDim.x >> 5) + warp_in_cta;
  const int64_t channels = 2 * static_cast<int64_t>(nk) * dk + static_cast<int64_t>(nv) * dv;
  const int64_t norm_items = S * nk;
  if (warp < norm_items) {
    const int64_t t = warp / nk;
    const int kh = static_cast<int>(warp % nk);
    const uint16_t *qp = conv + t * channels + kh * dk;
    const uint16_t *kp = conv + t * channels + static_cast<int64_t>(nk) * dk + kh * dk;
    float *sq = prep_all + warp_in_cta * 2 * dk;
    for (int d = lane; d < dk; d += 32) {
      const float qv = bf16_to_f32(qp[d]), kv = bf16_to_f32(kp[d]);
      sq[d] = __fmul_rn(qv, qv);
      sq[dk + d] = __fmul_rn(kv, kv);
    }
    __syncwarp();
    float scale = 0.0f;
    if (lane < 2) {
      const float *mine = sq + lane * dk;
      float sum = 0.0f;
#pragma unroll 16
      for (int d = 0; d < dk; ++d)
        sum = __fadd_rn(sum, mine[d]);
      scale = d_rsqrt(__fadd_rn(sum, 1.0e-6f));
      if (lane == 0)
        scale = __fmul_rn(scale, static_cast<float>(1.0 / sqrt(static_cast<double>(dk))));
    }
    const float q_norm_scale = __shfl_sync(0xffffffffu, scale, 0);
    const float k_inv = __shfl_sync(0xffffffffu, scale, 1);
    float *qo = qn + (t * nk + kh) * dk;
    float *ko = kn + (t * nk + kh) * dk;
    for (int d = lane; d < dk; d += 32) {
      qo[d] = __fmul_rn(bf16_to_f32(qp[d]), q_norm_scale);
      ko[d] = __fmul_rn(bf16_to_f32(kp[d]), k_inv);
    }
    return;
  }
  const int64_t i = (warp - norm_items) * 32 + lane;
  if (i < S * nv) {
    const int h = static_cast<int>(i % nv);
    const int64_t ab = (i / nv) * ab_stride + h; // a and b may be rows of a wider matrix
    const float bv = bf16_to_f32(b[ab]);
    beta[i] = b_activated ? bv : d_sigmoid(bv);
    // dt_bias is widened from bf16, A_log is read as f32 (LowerGatedDeltaNet.cpp:233-246).
    const float dt = bf16_to_f32(f32_to_bf16(load_as_f32(dt_bias, dt_dtype, h)));
    const float a_plus_dt = __fadd_rn(bf16_to_f32(a[ab]), dt);
    const float softplus = d_log(__fadd_rn(1.0f, d_exp(a_plus_dt)));
    const float g = __fmul_rn(-d_exp(load_as_f32(a_log, a_log_dtype, h)), softplus);
    decay[i] = d_exp(g);
  }
}

// DK > 0: state column in registers (DK values).  DK == 0: any dk, state stays in memory.
template <int DK>
__global__ void __launch_bounds__(32)
gdn_recurrence_kernel(const uint16_t *__restrict__ conv, const float *__restrict__ qn,
                      const float *__restrict__ kn, const float *__restrict__ beta,
                      const float *__restrict__ decay, float *__restrict__ state, int64_t S, int nk,
                      int nv, int dk_rt, int dv, uint16_t *__restrict__ out) {
  grid_dependency_sync();
  const int dk = DK > 0 ? DK : dk_rt;
  const int h = blockIdx.x;
  const int v = blockIdx.y * 32 + threadIdx.x;
  const int kh = h / (nv / nk);
  const int64_t channels = 2 * static_cast<int64_t>(nk) * dk + static_cast<int64_t>(nv) * dv;
  const bool active = v < dv;
  float *col = state + static_cast<int64_t>(h) * dk * dv + (active ? v : 0);
  extern __shared__ __align__(16) float kq_sm[]; // kn[dk], qn[dk] of the current token
  float *k_sm = kq_sm, *q_sm = kq_sm + dk;

  float s[DK > 0 ? DK : 1];
  if (DK > 0) {
#pragma unroll
    for (int k = 0; k < DK; ++k)
      s[k] = active ? col[static_cast<int64_t>(k) * dv] : 0.0f;
  }
  // The inputs of token t+1 are fetched while token t is being computed.
  constexpr int kPre = DK > 0 ? DK / 32 : 1;
  float k_next[kPre], q_next[kPre];
  float dc_next = 0.0f, bt_next = 0.0f;
  uint16_t value_next = 0;
  auto fetch = [&](int64_t t) {
    if (DK > 0) {
#pragma unroll
      for (int u = 0; u < kPre; ++u) {
        k_next[u] = kn[(t * nk + kh) * dk + u * 32 + threadIdx.x];
        q_next[u] = qn[(t * nk + kh) * dk + u * 32 + threadIdx.x];
      }
    }
    dc_next = decay[t * nv + h];
    bt_next = beta[t * nv + h];
    value_next = active ? conv[t * channels + 2 * static_cast<int64_t>(nk) * dk + h * dv + v] : static_cast<uint16_t>(0);
  };
  fetch(0);
  for (int64_t t = 0; t < S; ++t) {
    __syncwarp();
    if (DK > 0) {
#pragma unroll
      for (int u = 0; u < kPre; ++u) {
        k_sm[u * 32 + threadIdx.x] = k_next[u];
        q_sm[u * 32 + threadIdx.x] = q_next[u];
      }
    } else {
      for (int d = threadIdx.x; d < dk; d += 32) {
        k_sm[d] = kn[(t * nk + kh) * dk + d];
        q_sm[d] = qn[(t * nk + kh) * dk + d];
      }
    }
    __syncwarp();
    const float dc = dc_next;
    const float bt = bt_next;
    const float value = bf16_to_f32(value_next);
    if (t + 1 < S)
      fetch(t + 1);
    float kv = 0.0f;
    if (DK > 0) {
      // s[k] is replaced by its decayed value here; the update below starts from it.
#pragma unroll
      for (int k4 = 0; k4 < DK; k4 += 4) {
        const float4 kk = *reinterpret_cast<const float4 *>(k_sm + k4);
        const float kv4[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          s[k4 + u] = __fmul_rn(s[k4 + u], dc);
          kv = __fadd_rn(kv, __fmul_rn(s[k4 + u], kv4[u]));
        }
      }
    } else if (active) {
      for (int k = 0; k < dk; ++k)
        kv = __fadd_rn(kv, __fmul_rn(__fmul_rn(col[static_cast<int64_t>(k) * dv], dc), k_sm[k]));
    }
    const float delta = __fmul_rn(__fsub_rn(value, kv), bt);
    float o = 0.0f;
    if (DK > 0) {
#pragma unroll
      for (int k4 = 0; k4 < DK; k4 += 4) {
        const float4 kk = *reinterpret_cast<const float4 *>(k_sm + k4);
        const float4 qq = *reinterpret_cast<const float4 *>(q_sm + k4);
        const float kv4[4] = {kk.x, kk.y, kk.z, kk.w};
        const float qv4[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          s[k4 + u] = __fadd_rn(s[k4 + u], __fmul_rn(kv4[u], delta));
          o = __fadd_rn(o, __fmul_rn(s[k4 + u], qv4[u]));
        }
      }
    } else if (active) {
      for (int k = 0; k < dk; ++k) {
        const float updated = __fadd_rn(__fmul_rn(col[static_cast<int64_t>(k) * dv], dc), __fmul_rn(k_sm[k], delta));
        col[static_cast<int64_t>(k) * dv] = updated;
        o = __fadd_rn(o, __fmul_rn(updated, q_sm[k]));
      }
    }
    if (active)
      out[t * nv * dv + h * dv + v] = f32_to_bf16(o);
  }
  if (DK > 0 && active) {
#pragma unroll
    for (int k = 0; k < DK; ++k)
      col[static_cast<int64_t>(k) * dv] = s[k];
  }
}

// The same recurrence for calls of more than one token, with two tokens in flight.  Token t+1's
// first chain, kv' = sum_k (s_k * dc') * k'_k, needs the state row k as token t leaves it, and
// token t's second pass finalises the rows in ascending k: so row k is decayed for token t+1 and
// folded into kv' right after it has been updated for token t.  Every value is produced by the
// same operations in the same order as in the kernel above; only the two dependent chains (o of
// token t, kv of token t+1) now run side by side instead of one after the other.
template <int DK>
__global__ void __launch_bounds__(32)
gdn_recurrence_pipelined_kernel(const uint16_t *__restrict__ conv, const float *__restrict__ qn,
                                const float *__restrict__ kn, const float *__restrict__ beta,
                                const float *__restrict__ decay, float *__restrict__ state, int64_t S, int nk,
                                int nv, int dv, uint16_t *__restrict__ out) {
  grid_dependency_sync();
  const int h = blockIdx.x;
  const int v = blockIdx.y * 32 + threadIdx.x;
  const int kh = h / (nv / nk);
  const int64_t channels = 2 * static_cast<int64_t>(nk) * DK + static_cast<int64_t>(nv) * dv;
  const bool active = v < dv;
  float *col = state + static_cast<int64_t>(h) * DK * dv + (active ? v : 0);
  __shared__ __align__(16) float kq_sm[2][2 * DK]; // per token parity: kn[DK], qn[DK]

  float s[DK];
#pragma unroll
  for (int k = 0; k < DK; ++k)
    s[k] = active ? col[static_cast<int64_t>(k) * dv] : 0.0f;

  constexpr int kPre = DK / 32;
  float k_next[kPre], q_next[kPre];
  float dc_next = 0.0f, bt_next = 0.0f;
  uint16_t value_next = 0;
  auto fetch = [&](int64_t t) { // inputs of token t into registers
#pragma unroll
    for (int u = 0; u < kPre; ++u) {
      k_next[u] = kn[(t * nk + kh) * DK + u * 32 + threadIdx.x];
      q_next[u] = qn[(t * nk + kh) * DK + u * 32 + threadIdx.x];
    }
    dc_next = decay[t * nv + h];
    bt_next = beta[t * nv + h];
    value_next = active ? conv[t * channels + 2 * static_cast<int64_t>(nk) * DK + h * dv + v] : static_cast<uint16_t>(0);
  };
  auto publish = [&](int parity) { // the fetched token's k and q into shared memory
#pragma unroll
    for (int u = 0; u < kPre; ++u) {
      kq_sm[parity][u * 32 + threadIdx.x] = k_next[u];
      kq_sm[parity][DK + u * 32 + threadIdx.x] = q_next[u];
    }
  };

  // token 0: decay and first chain on their own
  fetch(0);
  publish(0);
  float dc = dc_next, bt = bt_next, value = bf16_to_f32(value_next);
  if (S > 1)
    fetch(1);
  __syncwarp();
  float kv = 0.0f;
#pragma unroll
  for (int k4 = 0; k4 < DK; k4 += 4) {
    const float4 kk = *reinterpret_cast<const float4 *>(&kq_sm[0][k4]);
    const float kv4[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      s[k4 + u] = __fmul_rn(s[k4 + u], dc);
      kv = __fadd_rn(kv, __fmul_rn(s[k4 + u], kv4[u]));
    }
  }
  for (int64_t t = 0; t < S; ++t) {
    const int cur = static_cast<int>(t & 1);
    const float delta = __fmul_rn(__fsub_rn(value, kv), bt);
    float o = 0.0f;
    if (t + 1 < S) {
      // Token t+1 is in the registers: publish it to the other buffer (last read two passes ago)
      // and start fetching token t+2.
      publish(cur ^ 1);
      const float dc1 = dc_next;
      bt = bt_next;
      value = bf16_to_f32(value_next);
      if (t + 2 < S)
        fetch(t + 2);
      __syncwarp();
      float kv1 = 0.0f;
#pragma unroll
      for (int k4 = 0; k4 < DK; k4 += 4) {
        const float4 kk = *reinterpret_cast<const float4 *>(&kq_sm[cur][k4]);
        const float4 qq = *reinterpret_cast<const float4 *>(&kq_sm[cur][DK + k4]);
        const float4 kn1 = *reinterpret_cast<const float4 *>(&kq_sm[cur ^ 1][k4]);
        const float kv4[4] = {kk.x, kk.y, kk.z, kk.w};
        const float qv4[4] = {qq.x, qq.y, qq.z, qq.w};
        const float kw4[4] = {kn1.x, kn1.y, kn1.z, kn1.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          s[k4 + u] = __fadd_rn(s[k4 + u], __fmul_rn(kv4[u], delta)); // row k as token t leaves it
          o = __fadd_rn(o, __fmul_rn(s[k4 + u], qv4[u]));
          s[k4 + u] = __fmul_rn(s[k4 + u], dc1);                       // decayed for token t+1
          kv1 = __fadd_rn(kv1, __fmul_rn(s[k4 + u], kw4[u]));
        }
      }
      kv = kv1;
    } else {
#pragma unroll
      for (int k4 = 0; k4 < DK; k4 += 4) {
        const float4 kk = *reinterpret_cast<const float4 *>(&kq_sm[cur][k4]);
        const float4 qq = *reinterpret_cast<const float4 *>(&kq_sm[cur][DK + k4]);
        const float kv4[4] = {kk.x, kk.y, kk.z, kk.w};
        const float qv4[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          s[k4 + u] = __fadd_rn(s[k4 + u], __fmul_rn(kv4[u], delta));
          o = __fadd_rn(o, __fmul_rn(s[k4 + u], qv4[u]));
        }
      }
    }
    if (active)
      out[t * nv * dv + h * dv + v] = f32_to_bf16(o);
    __syncwarp();
  }
  if (active) {
#pragma unroll
    for (int k = 0; k < DK; ++k)
      col[static_cast<int64_t>(k) * dv] = s[k];
  }
}

// Fast form of the recurrence for calls of more than one token: the same two-tokens-in-flight loop,
// but a warp owns 8 value columns and each column's 128 state rows are shared by four lanes (32
// rows each), so the two dependent chains per token are 32 long instead of 128 and end in two
// shuffles; multiply and add are fused.  What bounds the exact kernel, and still bounds this one, is
// how fast ONE warp can walk its dependent instructions, so a head is spread over 16 independent
// warps instead of 4.  A token then takes a few hundred cycles, less than a trip to L2, so the
// inputs (k, q, decay, beta, the 8 values) arrive by cp.async in chunks of 8 tokens, three chunks in
// shared memory per warp: the one in use, the next (token t + 1's k is needed beside token t) and
// the one in flight.  The sums differ from the reference's order (row groups are added as a tree)
// and from its roundings (fused multiply-adds): results agree with the exact kernels to f32
// rounding noise, not bit for bit.  Measured with 4 columns and eight lanes per column instead:
// slower (twice the shared memory per column, so half the CTAs fit).
// grid (value head, dv / 32), 128 threads: four independent warps that share nothing.
constexpr int kSplitChunk = 8; // tokens per chunk
constexpr int kSplitWarps = 4;
constexpr int kSplitCols = 8;  // value columns per warp
constexpr int kSplitLanes = 32 / kSplitCols; // lanes per column

// A lane reads its 16-byte pieces of k and q at the same offset inside its own row group; the groups
// are kept 16 bytes out of step (rows + 4 floats apart) so that those reads fall into different banks.
template <int DK> struct SplitChunk {
  static constexpr int kRows = DK / kSplitLanes, kPitch = kRows + 4;
  float kq[kSplitChunk][2][kSplitLanes][kPitch]; // per token: kn and qn, by row group
  uint16_t value[kSplitChunk][kSplitCols];
  float dc[kSplitChunk], bt[kSplitChunk];
};

template <int DK>
__global__ void __launch_bounds__(32 * kSplitWarps)
gdn_recurrence_split_kernel(const uint16_t *__restrict__ conv, const float *__restrict__ qn,
                            const float *__restrict__ kn, const float *__restrict__ beta,
                            const float *__restrict__ decay, float *__restrict__ state, int S, int nk,
                            int nv, int dv, uint16_t *__restrict__ out) {
  constexpr int kRows = DK / kSplitLanes; // state rows per lane
  using Chunk = SplitChunk<DK>;
  extern __shared__ __align__(16) unsigned char split_sm[]; // Chunk [kSplitWarps][3]
  grid_dependency_sync();
  const int h = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, c = lane % kSplitCols, part = lane / kSplitCols;
  const int v0 = (blockIdx.y * kSplitWarps + warp) * kSplitCols, v = v0 + c;
  if (v0 >= dv) // the column groups need not fill the last CTA
    return;
  Chunk *chunks = reinterpret_cast<Chunk *>(split_sm) + warp * 3;
  const int kh = h / (nv / nk);
  const int64_t channels = 2 * static_cast<int64_t>(nk) * DK + static_cast<int64_t>(nv) * dv;
  float *col = state + static_cast<int64_t>(h) * DK * dv + static_cast<int64_t>(part) * kRows * dv + v;

  float s[kRows];
#pragma unroll
  for (int k = 0; k < kRows; ++k)
    s[k] = col[static_cast<int64_t>(k) * dv];

  auto copy = [](void *dst, const void *src, auto bytes) {
    if (decltype(bytes)::value == 16)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src)
                   : "memory");
    else
      asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src),
                   "n"(decltype(bytes)::value)
                   : "memory");
  };
  // Requests chunk `index` (tokens 8 index .. 8 index + 7, those below S) and closes the copy group.
  auto request = [&](int index) {
    Chunk &ch = chunks[index % 3];
    const int t0 = index * kSplitChunk;
    for (int i = lane; i < kSplitChunk * (2 * DK / 4); i += 32) { // 16-byte pieces of k and q
      const int token = i / (2 * DK / 4), piece = i % (2 * DK / 4);
      if (t0 + token < S) {
        const int which = piece / (DK / 4), row = (piece % (DK / 4)) * 4;
        const float *src = (which ? qn : kn) + (static_cast<int64_t>(t0 + token) * nk + kh) * DK + row;
        copy(&ch.kq[token][which][row / kRows][row % kRows], src, std::integral_constant<int, 16>());
      }
    }
    if (lane < kSplitChunk && t0 + lane < S) {
      copy(&ch.value[lane][0], conv + (t0 + lane) * channels + 2 * static_cast<int64_t>(nk) * DK + h * dv + v0,
           std::integral_constant<int, 2 * kSplitCols>());
      copy(&ch.dc[lane], decay + static_cast<int64_t>(t0 + lane) * nv + h, std::integral_constant<int, 4>());
      copy(&ch.bt[lane], beta + static_cast<int64_t>(t0 + lane) * nv + h, std::integral_constant<int, 4>());
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto over_parts = [](float x) { // the lanes of a column hold its row groups' partial sums
#pragma unroll
    for (int o = kSplitCols; o < 32; o <<= 1)
      x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
  };
  uint16_t *out_col = out + static_cast<int64_t>(h) * dv + v;
  const int64_t out_stride = static_cast<int64_t>(nv) * dv;

  request(0);
  request(1);
  float kv = 0.0f, bt = 0.0f, value = 0.0f;
  int slot = 0, cur_index = 0; // token t is slot `slot` of chunk `cur_index` (buffer cur_index % 3)
  const Chunk *cur = chunks;
  for (int t = 0; t < S; ++t) {
    if (slot == 0) { // chunk index + 2 goes into the buffer of the chunk that has just been left
      __syncwarp();
      request(cur_index + 2);
      asm volatile("cp.async.wait_group 1;" ::: "memory"); // all but the newest group: this chunk and the next
      __syncwarp();
    }
    if (t == 0) { // the first token's decay and first chain on their own
      const float dc = cur->dc[0];
      bt = cur->bt[0];
      value = bf16_to_f32(cur->value[0][c]);
#pragma unroll
      for (int k4 = 0; k4 < kRows; k4 += 4) {
        const float4 kk = *reinterpret_cast<const float4 *>(&cur->kq[0][0][part][k4]);
        const float kv4[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          s[k4 + u] *= dc;
          kv = __fmaf_rn(s[k4 + u], kv4[u], kv);
        }
      }
      kv = over_parts(kv);
    }
    const float delta = (value - kv) * bt;
    float o = 0.0f;
    // where token t + 1 lives
    const int nslot = slot + 1 == kSplitChunk ? 0 : slot + 1;
    const int nindex = nslot == 0 ? cur_index + 1 : cur_index;
    const Chunk *nxt = nslot == 0 ? chunks + nindex % 3 : cur;
    if (t + 1 < S) {
      const float dc1 = nxt->dc[nslot];
      bt = nxt->bt[nslot];
      value = bf16_to_f32(nxt->value[nslot][c]);
      float kv1[2] = {0.0f, 0.0f}, o2[2] = {0.0f, 0.0f}; // two interleaved partial sums per chain
#pragma unroll
      for (int k4 = 0; k4 < kRows; k4 += 4) {
        const float4 kk = *reinterpret_cast<const float4 *>(&cur->kq[slot][0][part][k4]);
        const float4 qq = *reinterpret_cast<const float4 *>(&cur->kq[slot][1][part][k4]);
        const float4 kn1 = *reinterpret_cast<const float4 *>(&nxt->kq[nslot][0][part][k4]);
        const float kv4[4] = {kk.x, kk.y, kk.z, kk.w};
        const float qv4[4] = {qq.x, qq.y, qq.z, qq.w};
        const float kw4[4] = {kn1.x, kn1.y, kn1.z, kn1.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          s[k4 + u] = __fmaf_rn(kv4[u], delta, s[k4 + u]); // row k as token t leaves it
          o2[u & 1] = __fmaf_rn(s[k4 + u], qv4[u], o2[u & 1]);
          s[k4 + u] *= dc1;                                // decayed for token t + 1
          kv1[u & 1] = __fmaf_rn(s[k4 + u], kw4[u], kv1[u & 1]);
        }
      }
      o = o2[0] + o2[1];
      kv = over_parts(kv1[0] + kv1[1]);
    } else {
#pragma unroll
      for (int k4 = 0; k4 < kRows; k4 += 4) {
        const float4 kk = *reinterpret_cast<const float4 *>(&cur->kq[slot][0][part][k4]);
        const float4 qq = *reinterpret_cast<const float4 *>(&cur->kq[slot][1][part][k4]);
        const float kv4[4] = {kk.x, kk.y, kk.z, kk.w};
        const float qv4[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          s[k4 + u] = __fmaf_rn(kv4[u], delta, s[k4 + u]);
          o = __fmaf_rn(s[k4 + u], qv4[u], o);
        }
      }
    }
    o = over_parts(o);
    if (part == 0)
      out_col[t * out_stride] = f32_to_bf16(o);
    slot = nslot, cur_index = nindex, cur = nxt;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int k = 0; k < kRows; ++k)
    col[static_cast<int64_t>(k) * dv] = s[k];
}

size_t gdn_scratch_floats(int64_t S, int nk, int nv, int dk) {
  return static_cast<size_t>(S) * (2 * static_cast<size_t>(nk) * dk + 2 * static_cast<size_t>(nv));
}

cudaError_t launch_gated_delta_net(const uint16_t *conv, const uint16_t *a, const uint16_t *b,
                                   const void *a_log, int a_log_dtype, const void *dt_bias, int dt_dtype,
                                   float *state, int64_t S, int nk, int nv, int dk, int dv,
                                   int b_activated, float *scratch, uint16_t *out, cudaStream_t stream, int ab_stride,
                                   int fast) {
  if (S == 0)
    return cudaSuccess;
  if (ab_stride <= 0)
    ab_stride = nv;
  if (nk <= 0 || nv <= 0 || nv % nk != 0)
    return cudaErrorInvalidValue;
  float *qn = scratch;
  float *kn = qn + S * nk * dk;
  float *beta = kn + S * nk * dk;
  float *decay = beta + S * nv;
  const int64_t warps = S * nk + (S * nv + 31) / 32;
  launch_chained(gdn_prepare_kernel, dim3(static_cast<unsigned>((warps + 3) / 4)), dim3(128), 4 * 2 * dk * sizeof(float), stream, 
      conv, a, b, a_log, a_log_dtype, dt_bias, dt_dtype, S, nk, nv, ab_stride, dk, dv, b_activated, qn, kn, beta, decay);
  dim3 grid(nv, (dv + 31) / 32);
  const size_t smem = 2 * static_cast<size_t>(dk) * sizeof(float);
  static const bool pipelined = [] {
    const char *flag = std::getenv("LLMCP_B200_GDN_PIPELINE");
    return !(flag && flag[0] == '0');
  }();
  if (dk == 128 && S > 1 && fast && dv % kSplitCols == 0 && S < (1 << 30)) {
    constexpr size_t split_bytes = kSplitWarps * 3 * sizeof(SplitChunk<128>);
    if (cudaError_t e = opt_in_shared_memory(reinterpret_cast<const void *>(gdn_recurrence_split_kernel<128>), split_bytes);
        e != cudaSuccess)
      return e;
    const int groups = dv / kSplitCols;
    launch_chained(gdn_recurrence_split_kernel<128>, dim3(nv, (groups + kSplitWarps - 1) / kSplitWarps), dim3(32 * kSplitWarps),
                   split_bytes, stream, conv, qn, kn, beta, decay, state, static_cast<int>(S), nk, nv, dv, out);
  }
  else if (dk == 128 && S > 1 && pipelined)
    launch_chained(gdn_recurrence_pipelined_kernel<128>, dim3(grid), dim3(32), 0, stream, conv, qn, kn, beta, decay, state, S, nk, nv, dv, out);
  else if (dk == 128)
    launch_chained(gdn_recurrence_kernel<128>, dim3(grid), dim3(32), smem, stream, conv, qn, kn, beta, decay, state, S, nk, nv, dk, dv, out);
  else
    launch_chained(gdn_recurrence_kernel<0>, dim3(grid), dim3(32), smem, stream, conv, qn, kn, beta, decay, state, S, nk, nv, dk, dv, out);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------
// One-token (decode) form of causal_conv1d + gated_delta_net + gated_rms_norm in two kernels.
// The arithmetic of every value is that of the general kernels above; only the grouping into
// launches differs, so that five dependent launches per layer become two.
// ---------------------------------------------------------------------------------
constexpr int kMaxConvKernel = 8;

// Convolution of one channel for the single new row, SiLU, bf16 rounding; the channel's state is
// shifted in place by the same thread (no other thread reads it).
__device__ __forceinline__ float conv_step(const uint16_t *__restrict__ x, const uint16_t *__restrict__ w,
                                           uint16_t *__restrict__ state, int C, int kernel, int c) {
  const int state_len = kernel - 1;
  uint16_t taps[kMaxConvKernel];
#pragma unroll
  for (int k = 0; k < kMaxConvKernel; ++k)
    if (k < kernel)
      taps[k] = k < state_len ? state[static_cast<int64_t>(k) * C + c] : x[c];
  float acc = 0.0f;
#pragma unroll
  for (int k = 0; k < kMaxConvKernel; ++k)
    if (k < kernel)
      acc = __fadd_rn(acc, __fmul_rn(bf16_to_f32(taps[k]), bf16_to_f32(w[c * kernel + k])));
#pragma unroll
  for (int k = 0; k + 1 < kMaxConvKernel; ++k)
    if (k < state_len)
      state[static_cast<int64_t>(k) * C + c] = taps[k + 1];
  return bf16_to_f32(f32_to_bf16(__fmul_rn(acc, d_sigmoid(acc))));
}

// CTA roles (dk threads each, one channel per thread): [0, nk) q heads, [nk, 2 nk) k heads
// (convolution, then the L2 norm with thread 0 adding the squares in order), then one CTA per dk
// value channels (convolution only), then one CTA that computes beta and decay, a value head per
// thread.
__global__ void __launch_bounds__(256)
gdn_decode_front_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ w, uint16_t *__restrict__ state,
                        int kernel, const uint16_t *__restrict__ a, const uint16_t *__restrict__ b,
                        const void *__restrict__ a_log, int a_log_dtype, const void *__restrict__ dt_bias,
                        int dt_dtype, int nk, int nv, int dk, int dv, int b_activated, float *__restrict__ qn,
                        float *__restrict__ kn, float *__restrict__ beta, float *__restrict__ decay,
                        uint16_t *__restrict__ conv_out, const GdnBatch batch) {
  extern __shared__ __align__(16) float front_sm[]; // dk squares
  __shared__ float scale_sm;
  grid_dependency_sync(true); // the step kernel behind is placed now and fetches its state meanwhile
  const int t = threadIdx.x;
  const int role = blockIdx.x;
  const int C = 2 * nk * dk + nv * dv;
  { // blockIdx.y: sequence of a batch of independent sequences (one token each)
    const int64_t seq = blockIdx.y;
    x += seq * C;
    conv_out += seq * C;
    state += seq * batch.conv_state;
    a += seq * batch.ab;
    b += seq * batch.ab;
    const int64_t scratch = seq * (2 * static_cast<int64_t>(nk) * dk + 2 * nv);
    qn += scratch, kn += scratch, beta += scratch, decay += scratch;
  }
  const int value_ctas = (nv * dv + dk - 1) / dk;
  if (role < 2 * nk) {
    const bool is_q = role < nk;
    const int head = is_q ? role : role - nk;
    const float v = conv_step(x, w, state, C, kernel, (is_q ? 0 : nk * dk) + head * dk + t);
    front_sm[t] = __fmul_rn(v, v);
    __syncthreads();
    if (t == 0) {
      float sum = 0.0f;
      for (int d = 0; d < dk; d += 16) { // dk % 16 == 0
        float4 sq[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          sq[u] = *reinterpret_cast<const float4 *>(front_sm + d + 4 * u);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          sum = __fadd_rn(sum, sq[u].x);
          sum = __fadd_rn(sum, sq[u].y);
          sum = __fadd_rn(sum, sq[u].z);
          sum = __fadd_rn(sum, sq[u].w);
        }
      }
      float scale = d_rsqrt(__fadd_rn(sum, 1.0e-6f));
      if (is_q)
        scale = __fmul_rn(scale, static_cast<float>(1.0 / sqrt(static_cast<double>(dk))));
      scale_sm = scale;
    }
    __syncthreads();
    (is_q ? qn : kn)[head * dk + t] = __fmul_rn(v, scale_sm);
  } else if (role < 2 * nk + value_ctas) {
    const int c = 2 * nk * dk + (role - 2 * nk) * dk + t;
    if (c < C)
      conv_out[c] = f32_to_bf16(conv_step(x, w, state, C, kernel, c));
  } else {
    for (int h = t; h < nv; h += blockDim.x) {
      const float bv = bf16_to_f32(b[h]);
      beta[h] = b_activated ? bv : d_sigmoid(bv);
      // dt_bias is widened from bf16, A_log is read as f32 (LowerGatedDeltaNet.cpp:233-246).
      const float dt = bf16_to_f32(f32_to_bf16(load_as_f32(dt_bias, dt_dtype, h)));
      const float a_plus_dt = __fadd_rn(bf16_to_f32(a[h]), dt);
      const float softplus = d_log(__fadd_rn(1.0f, d_exp(a_plus_dt)));
      const float g = __fmul_rn(-d_exp(load_as_f32(a_log, a_log_dtype, h)), softplus);
      decay[h] = d_exp(g);
    }
  }
}

// One CTA per value head, one thread per state column: the recurrence step of the token, then
// the head's gated RMSNorm (thread 0 adds the dv squares in order) and the int8 quantisation of
// the result for the output projection.  gate holds silu(z) when gate_activated.
template <int DK>
__global__ void __launch_bounds__(256)
gdn_decode_step_kernel(const uint16_t *__restrict__ conv, const float *__restrict__ qn, const float *__restrict__ kn,
                       const float *__restrict__ beta, const float *__restrict__ decay, float *__restrict__ state,
                       int nk, int nv, int dv, const uint16_t *__restrict__ gate, const void *__restrict__ norm_w,
                       int norm_w_dtype, float eps, int gate_activated, uint16_t *__restrict__ y,
                       int8_t *__restrict__ q_out, float *__restrict__ s_out, const GdnBatch batch) {
  extern __shared__ __align__(16) float step_sm[]; // kn[DK], qn[DK], squares[dv]
  __shared__ float rstd_sm;
  float *k_sm = step_sm, *q_sm = step_sm + DK, *sq_sm = step_sm + 2 * DK;
  const int h = blockIdx.x, v = threadIdx.x;
  const int kh = h / (nv / nk);
  const int64_t seq = blockIdx.y; // sequence of a batch (one token each)
  {
    conv += seq * (2 * static_cast<int64_t>(nk) * DK + static_cast<int64_t>(nv) * dv);
    const int64_t scratch = seq * (2 * static_cast<int64_t>(nk) * DK + 2 * nv);
    qn += scratch, kn += scratch, beta += scratch, decay += scratch;
    state += seq * batch.state;
    gate += seq * static_cast<int64_t>(nv) * dv;
  }
  float *col = state + static_cast<int64_t>(h) * DK * dv + v;
  // The recurrent state is this kernel's own (written by the same kernel one token earlier, which
  // finished long ago): it is requested before waiting for the kernel in front.
  float s[DK];
#pragma unroll
  for (int k = 0; k < DK; ++k)
    s[k] = col[static_cast<int64_t>(k) * dv];
  const float norm_weight = load_as_f32(norm_w, norm_w_dtype, v); // a weight: no need to wait for it either
  grid_dependency_sync(true);
  // The gate is needed only after both chains: requested now, it arrives while they run.
  const float gv = bf16_to_f32(gate[static_cast<int64_t>(h) * dv + v]);
  for (int d = v; d < DK; d += dv) {
    k_sm[d] = kn[kh * DK + d];
    q_sm[d] = qn[kh * DK + d];
  }
  const float dc = decay[h], bt = beta[h];
  const float value = bf16_to_f32(conv[2 * nk * DK + h * dv + v]);
  __syncthreads();
  float kv = 0.0f;
#pragma unroll
  for (int k4 = 0; k4 < DK; k4 += 4) {
    const float4 kk = *reinterpret_cast<const float4 *>(k_sm + k4);
    const float kv4[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      s[k4 + u] = __fmul_rn(s[k4 + u], dc);
      kv = __fadd_rn(kv, __fmul_rn(s[k4 + u], kv4[u]));
    }
  }
  const float delta = __fmul_rn(__fsub_rn(value, kv), bt);
  float o = 0.0f;
#pragma unroll
  for (int k4 = 0; k4 < DK; k4 += 4) {
    const float4 kk = *reinterpret_cast<const float4 *>(k_sm + k4);
    const float4 qq = *reinterpret_cast<const float4 *>(q_sm + k4);
    const float kv4[4] = {kk.x, kk.y, kk.z, kk.w};
    const float qv4[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      s[k4 + u] = __fadd_rn(s[k4 + u], __fmul_rn(kv4[u], delta));
      o = __fadd_rn(o, __fmul_rn(s[k4 + u], qv4[u]));
    }
  }
#pragma unroll
  for (int k = 0; k < DK; ++k)
    col[static_cast<int64_t>(k) * dv] = s[k];
  // gated RMSNorm over the head (LowerToLinalg.cpp:655-718, DecodeNormalization.cpp:118-131)
  const float xo = bf16_to_f32(f32_to_bf16(o));
  sq_sm[v] = __fmul_rn(xo, xo);
  __syncthreads();
  if (v == 0) {
    float sum = 0.0f;
#pragma unroll 16
    for (int d = 0; d < dv; ++d)
      sum = __fadd_rn(sum, sq_sm[d]);
    rstd_sm = d_rsqrt(__fadd_rn(__fdiv_rn(sum, static_cast<float>(dv)), eps));
  }
  __syncthreads();
  const int64_t element = (seq * nv + h) * dv + v;
  const float silu = gate_activated ? gv : __fmul_rn(gv, d_sigmoid(gv));
  float t = __fmul_rn(xo, silu);
  t = __fmul_rn(t, norm_weight);
  t = __fmul_rn(t, rstd_sm);
  const uint16_t r = f32_to_bf16(t);
  if (y)
    y[element] = r;
  if (q_out)
    warp_quant_block(bf16_to_f32(r), q_out, s_out, element, element / kBlock, v & 31);
}

// The same convolution in two halves: what does not depend on the kernel in front (the channel's
// state rows and taps' weights) is fetched first, the new row is applied after the wait.
struct ConvChannel {
  uint16_t taps[kMaxConvKernel];
  uint16_t weights[kMaxConvKernel];
};

__device__ __forceinline__ void conv_fetch(const uint16_t *__restrict__ w, const uint16_t *__restrict__ state, int C, int kernel,
                                           int c, ConvChannel &ch) {
#pragma unroll
  for (int k = 0; k < kMaxConvKernel; ++k)
    if (k < kernel) {
      ch.weights[k] = w[c * kernel + k];
      if (k < kernel - 1)
        ch.taps[k] = state[static_cast<int64_t>(k) * C + c];
    }
}

__device__ __forceinline__ float conv_apply(ConvChannel &ch, uint16_t x_new, uint16_t *__restrict__ state, int C, int kernel, int c) {
  const int state_len = kernel - 1;
#pragma unroll
  for (int k = 0; k < kMaxConvKernel; ++k)
    if (k == state_len)
      ch.taps[k] = x_new;
  float acc = 0.0f;
#pragma unroll
  for (int k = 0; k < kMaxConvKernel; ++k)
    if (k < kernel)
      acc = __fadd_rn(acc, __fmul_rn(bf16_to_f32(ch.taps[k]), bf16_to_f32(ch.weights[k])));
#pragma unroll
  for (int k = 0; k + 1 < kMaxConvKernel; ++k)
    if (k < state_len)
      state[static_cast<int64_t>(k) * C + c] = ch.taps[k + 1];
  return bf16_to_f32(f32_to_bf16(__fmul_rn(acc, d_sigmoid(acc))));
}

// Sum of `count` floats of shared memory as every thread of the CTA sees it afterwards:
// ordered (thread 0 adds them in index order, the reference's order) or, with tree_sum, a
// shuffle tree per warp and the warps' results in warp order.  count = blockDim.x = 128.
__device__ __forceinline__ float cta_sum_128(float *values, float *result, int tree_sum) {
  const int t = threadIdx.x;
  if (tree_sum) {
    float part = values[t];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, o));
    __syncthreads(); // every thread has read its value
    if ((t & 31) == 0)
      values[t >> 5] = part;
    __syncthreads();
    return __fadd_rn(__fadd_rn(values[0], values[1]), __fadd_rn(values[2], values[3]));
  }
  if (t == 0) {
    float sum = 0.0f;
    for (int d = 0; d < 128; d += 16) {
      float4 sq[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        sq[u] = *reinterpret_cast<const float4 *>(values + d + 4 * u);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        sum = __fadd_rn(sum, sq[u].x);
        sum = __fadd_rn(sum, sq[u].y);
        sum = __fadd_rn(sum, sq[u].z);
        sum = __fadd_rn(sum, sq[u].w);
      }
    }
    *result = sum;
  }
  __syncthreads();
  return *result;
}

// The whole one-token mixer in one launch: a thread-block cluster per key head, one CTA per value
// head of it, 128 threads (dk = dv = 128).  CTA 0 of the cluster convolves and normalises the key
// head's q channels, CTA 1 its k channels (a single CTA does both when a key head serves one value
// head), and each stores its 128 results into the shared memory of every CTA of the cluster; every
// CTA convolves its own value channels and computes its head's beta and decay, then runs the
// recurrence step, the gated RMSNorm and the quantisation as gdn_decode_step_kernel does.  The
// arithmetic of every value is that of the two-kernel form (bit-identical when tree_sum == 0).
template <int RATIO_MIN2>
__global__ void __launch_bounds__(128)
gdn_decode_fused_kernel(const uint16_t *__restrict__ x, const uint16_t *__restrict__ w, uint16_t *__restrict__ conv_state,
                        int kernel, const uint16_t *__restrict__ a, const uint16_t *__restrict__ b,
                        const void *__restrict__ a_log, int a_log_dtype, const void *__restrict__ dt_bias, int dt_dtype,
                        int nk, int nv, int b_activated, float *__restrict__ state, const uint16_t *__restrict__ gate,
                        const void *__restrict__ norm_w, int norm_w_dtype, float eps, int gate_activated, int tree_sum,
                        uint16_t *__restrict__ y, int8_t *__restrict__ q_out, float *__restrict__ s_out,
                        const GdnBatch batch) {
  constexpr int DK = 128, DV = 128;
  __shared__ __align__(16) float k_sm[DK];
  __shared__ __align__(16) float q_sm[DK];
  __shared__ __align__(16) float sq_sm[DV];
  __shared__ float sum_sm;
  const int h = blockIdx.x, t = threadIdx.x;
  const int ratio = nv / nk;
  const int kh = h / ratio, rank = h % ratio;
  const int C = 2 * nk * DK + nv * DV;
  const int64_t seq = blockIdx.y;
  x += seq * C;
  conv_state += seq * batch.conv_state;
  a += seq * batch.ab;
  b += seq * batch.ab;
  state += seq * batch.state;
  gate += seq * static_cast<int64_t>(nv) * DV;
  // Nothing below up to the wait depends on the kernel in front: the head's state column, the
  // channels' convolution state and weights, the norm weight, the per-head constants.
  float *col = state + static_cast<int64_t>(h) * DK * DV + t;
  float s[DK];
#pragma unroll
  for (int k = 0; k < DK; ++k)
    s[k] = col[static_cast<int64_t>(k) * DV];
  const float norm_weight = load_as_f32(norm_w, norm_w_dtype, t);
  // channels of this thread: one or two of the key head's (by cluster rank), one value channel
  const bool does_q = RATIO_MIN2 ? rank == 0 : true, does_k = RATIO_MIN2 ? rank == 1 : true;
  const int cq = kh * DK + t, ck = nk * DK + kh * DK + t, cv = 2 * nk * DK + h * DV + t;
  ConvChannel chq, chk, chv;
  if (does_q)
    conv_fetch(w, conv_state, C, kernel, cq, chq);
  if (does_k)
    conv_fetch(w, conv_state, C, kernel, ck, chk);
  conv_fetch(w, conv_state, C, kernel, cv, chv);
  const float dt = bf16_to_f32(f32_to_bf16(load_as_f32(dt_bias, dt_dtype, h)));
  const float minus_exp_a = -d_exp(load_as_f32(a_log, a_log_dtype, h));
  if (RATIO_MIN2) // every CTA of the cluster is running before anyone stores into its shared memory
    cluster_sync_all();
  grid_dependency_sync(true);
  const float gv = bf16_to_f32(gate[static_cast<int64_t>(h) * DV + t]);
  const uint16_t xq = does_q ? x[cq] : uint16_t(0), xk = does_k ? x[ck] : uint16_t(0), xv = x[cv];
  const float bv = bf16_to_f32(b[h]), av = bf16_to_f32(a[h]);
  if (does_q) {
    const float v = conv_apply(chq, xq, conv_state, C, kernel, cq);
    sq_sm[t] = __fmul_rn(v, v);
    __syncthreads();
    const float sum = cta_sum_128(sq_sm, &sum_sm, tree_sum);
    float scale = d_rsqrt(__fadd_rn(sum, 1.0e-6f));
    scale = __fmul_rn(scale, static_cast<float>(1.0 / sqrt(static_cast<double>(DK))));
    const float n = __fmul_rn(v, scale);
    if (RATIO_MIN2) {
      for (int r = 0; r < ratio; ++r)
        store_shared_cluster(q_sm + t, r, n);
    } else {
      q_sm[t] = n;
    }
  }
  if (does_k) {
    if (does_q)
      __syncthreads(); // sq_sm and sum_sm are reused
    const float v = conv_apply(chk, xk, conv_state, C, kernel, ck);
    sq_sm[t] = __fmul_rn(v, v);
    __syncthreads();
    const float sum = cta_sum_128(sq_sm, &sum_sm, tree_sum);
    const float n = __fmul_rn(v, d_rsqrt(__fadd_rn(sum, 1.0e-6f)));
    if (RATIO_MIN2) {
      for (int r = 0; r < ratio; ++r)
        store_shared_cluster(k_sm + t, r, n);
    } else {
      k_sm[t] = n;
    }
  }
  const float value = conv_apply(chv, xv, conv_state, C, kernel, cv);
  const float bt = b_activated ? bv : d_sigmoid(bv);
  // dt_bias is widened from bf16, A_log is read as f32 (LowerGatedDeltaNet.cpp:233-246).
  const float softplus = d_log(__fadd_rn(1.0f, d_exp(__fadd_rn(av, dt))));
  const float dc = d_exp(__fmul_rn(minus_exp_a, softplus));
  if (RATIO_MIN2)
    cluster_sync_all(); // q and k of the key head have arrived from the cluster's first two CTAs
  else
    __syncthreads();
  float kv = 0.0f;
#pragma unroll
  for (int k4 = 0; k4 < DK; k4 += 4) {
    const float4 kk = *reinterpret_cast<const float4 *>(k_sm + k4);
    const float kv4[4] = {kk.x, kk.y, kk.z, kk.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      s[k4 + u] = __fmul_rn(s[k4 + u], dc);
      kv = __fadd_rn(kv, __fmul_rn(s[k4 + u], kv4[u]));
    }
  }
  const float delta = __fmul_rn(__fsub_rn(value, kv), bt);
  float o = 0.0f;
#pragma unroll
  for (int k4 = 0; k4 < DK; k4 += 4) {
    const float4 kk = *reinterpret_cast<const float4 *>(k_sm + k4);
    const float4 qq = *reinterpret_cast<const float4 *>(q_sm + k4);
    const float kv4[4] = {kk.x, kk.y, kk.z, kk.w};
    const float qv4[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      s[k4 + u] = __fadd_rn(s[k4 + u], __fmul_rn(kv4[u], delta));
      o = __fadd_rn(o, __fmul_rn(s[k4 + u], qv4[u]));
    }
  }
#pragma unroll
  for (int k = 0; k < DK; ++k)
    col[static_cast<int64_t>(k) * DV] = s[k];
  // gated RMSNorm over the head (LowerToLinalg.cpp:655-718, DecodeNormalization.cpp:118-131)
  const float xo = bf16_to_f32(f32_to_bf16(o));
  __syncthreads(); // sq_sm may still be read by a slower warp of the q/k norm
  sq_sm[t] = __fmul_rn(xo, xo);
  __syncthreads();
  const float sum = cta_sum_128(sq_sm, &sum_sm, tree_sum);
  const float rstd = d_rsqrt(__fadd_rn(__fdiv_rn(sum, static_cast<float>(DV)), eps));
  const int64_t element = (seq * nv + h) * DV + t;
  const float silu = gate_activated ? gv : __fmul_rn(gv, d_sigmoid(gv));
  float r = __fmul_rn(xo, silu);
  r = __fmul_rn(r, norm_weight);
  r = __fmul_rn(r, rstd);
  const uint16_t bits = f32_to_bf16(r);
  if (y)
    y[element] = bits;
  if (q_out)
    warp_quant_block(bf16_to_f32(bits), q_out, s_out, element, element / kBlock, t & 31);
}

bool gdn_decode_single_kernel_supported(int kernel, int nk, int nv, int dk, int dv) {
  return kernel >= 1 && kernel <= kMaxConvKernel && dk == 128 && dv == 128 && nk > 0 && nv % nk == 0 && nv / nk <= 8;
}

bool gdn_decode_supported(int kernel, int nk, int nv, int dk, int dv) {
  return kernel >= 1 && kernel <= kMaxConvKernel && dk == 128 && dv % 32 == 0 && dv >= 32 && dv <= 256 && nk > 0 &&
         nv % nk == 0;
}

cudaError_t launch_gdn_decode(const uint16_t *qkv, const uint16_t *conv_w, uint16_t *conv_state, int kernel,
                              const uint16_t *a, const uint16_t *b, const void *a_log, int a_log_dtype,
                              const void *dt_bias, int dt_dtype, float *state, int nk, int nv, int dk, int dv,
                              int b_activated, const uint16_t *gate, const void *norm_w, int norm_w_dtype, float eps,
                              int gate_activated, float *scratch, uint16_t *conv_out, uint16_t *y, int8_t *q_out,
                              float *s_out, cudaStream_t stream, int sequences, const GdnBatch *strides, int single_kernel,
                              int tree_sum) {
  if (!gdn_decode_supported(kernel, nk, nv, dk, dv) || sequences < 1 || (sequences > 1 && !strides))
    return cudaErrorInvalidValue;
  const GdnBatch batch = strides ? *strides : GdnBatch{};
  if (single_kernel && gdn_decode_single_kernel_supported(kernel, nk, nv, dk, dv)) {
    const int ratio = nv / nk;
    if (ratio == 1)
      launch_chained(gdn_decode_fused_kernel<0>, dim3(nv, sequences), dim3(128), 0, stream, qkv, conv_w, conv_state, kernel, a, b,
                     a_log, a_log_dtype, dt_bias, dt_dtype, nk, nv, b_activated, state, gate, norm_w, norm_w_dtype, eps,
                     gate_activated, tree_sum, y, q_out, s_out, batch);
    else
      launch_chained_cluster(gdn_decode_fused_kernel<1>, dim3(nv, sequences), dim3(128), 0, stream, ratio, qkv, conv_w, conv_state,
                             kernel, a, b, a_log, a_log_dtype, dt_bias, dt_dtype, nk, nv, b_activated, state, gate, norm_w,
                             norm_w_dtype, eps, gate_activated, tree_sum, y, q_out, s_out, batch);
    return cudaGetLastError();
  }
  float *qn = scratch;
  float *kn = qn + nk * dk;
  float *beta = kn + nk * dk;
  float *decay = beta + nv;
  const int ctas = 2 * nk + (nv * dv + dk - 1) / dk + 1;
  launch_chained(gdn_decode_front_kernel, dim3(ctas, sequences), dim3(dk), dk * sizeof(float), stream, qkv, conv_w,
                 conv_state, kernel, a, b, a_log, a_log_dtype, dt_bias, dt_dtype, nk, nv, dk, dv, b_activated, qn, kn, beta,
                 decay, conv_out, batch);
  launch_chained(gdn_decode_step_kernel<128>, dim3(nv, sequences), dim3(dv), (2 * 128 + dv) * sizeof(float), stream, conv_out, qn,
                 kn, beta, decay, state, nk, nv, dv, gate, norm_w, norm_w_dtype, eps, gate_activated, y, q_out, s_out, batch);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------------
// attention (LowerAttention.cpp:160-601).
//   prepare : per (token, head) zero-centred RMSNorm over head_dim, rotate-half RoPE on
//             the first `rot` dims, bf16; q -> scratch, k and v -> KV cache.
//   scores  : s[t, h, j] = (sum_d q[d] * K[j, d]) * scale, ascending d, one thread per key.
//   combine : per (token, head) online softmax over key tiles of 64 in ascending key order,
//             one thread per head-dim lane; then divide, sigmoid gate, bf16.
// cache layout (one layer): [2, nkv, cap, hd] bf16.
// ---------------------------------------------------------------------------------
__global__ void attn_prepare_kernel(const uint16_t *__restrict__ qg, const uint16_t *__restrict__ k,
                                    const uint16_t *__restrict__ v, const uint16_t *__restrict__ q_norm,
                                    const uint16_t *__restrict__ k_norm, const float *__restrict__ cos,
                                    const float *__restrict__ sin, uint16_t *__restrict__ cache,
                                    const int64_t *__restrict__ position_ptr, int rows_from_position, int64_t S,
                                    int nh, int nkv, int hd, int rot, int64_t cap, uint16_t *__restrict__ qn, int tree_sum,
                                    int64_t cache_stride) {
  extern __shared__ float prep_sm[]; // per warp: hd values
  grid_dependency_sync();
  const int64_t position = *position_ptr;
  // cos/sin hold either the rows of this call (row t) or a table over all positions.
  const int64_t row_base = rows_from_position ? position : 0;
  const int lane = threadIdx.x & 31;
  const int warp_in_cta = threadIdx.x >> 5;
  const int64_t item = blockIdx.x * static_cast<int64_t>(blockDim.x >> 5) + warp_in_cta;
  const int per_token = nh + nkv;
  if (item >= S * per_token)
    return;
  const int64_t t = item / per_token;
  // cache_stride != 0: the rows are one token each of independent sequences at the same position,
  // row t with a cache of its own cache_stride elements further on; else tokens of one sequence.
  const int64_t tpos = cache_stride ? 0 : t;
  cache += t * cache_stride;
  const int which = static_cast<int>(item % per_token);
  const bool is_q = which < nh;
  const int head = is_q ? which : which - nh;
  const uint16_t *src = is_q ? qg + t * nh * 2 * hd + static_cast<int64_t>(head) * 2 * hd
                             : k + t * nkv * hd + static_cast<int64_t>(head) * hd;
  const uint16_t *weight = is_q ? q_norm : k_norm;
  uint16_t *dst = is_q ? qn + (t * nh + head) * hd
                       : cache + ((0 * static_cast<int64_t>(nkv) + head) * cap + position + tpos) * hd;
  float *tmp = prep_sm + warp_in_cta * hd;
  // Everything the later passes read from memory (norm weight, rotary rows, the value row to be
  // copied) is requested here, beside the input row, instead of after the serial sum.
  constexpr int kPerLane = 8; // head dimensions up to 256
  const bool prefetched = hd <= 32 * kPerLane;
  const uint16_t *vsrc = v + t * nkv * hd + static_cast<int64_t>(head) * hd;
  float w_reg[kPerLane], cos_reg[kPerLane], sin_reg[kPerLane];
  uint16_t v_reg[kPerLane];
  if (prefetched) {
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int d = lane + 32 * i;
      w_reg[i] = cos_reg[i] = sin_reg[i] = 0.0f;
      v_reg[i] = 0;
      if (d < hd) {
        w_reg[i] = bf16_to_f32(weight[d]);
        if (!is_q)
          v_reg[i] = vsrc[d];
        if (d < rot) {
          cos_reg[i] = cos[(row_base + tpos) * rot + d];
          sin_reg[i] = sin[(row_base + tpos) * rot + d];
        }
      }
    }
  }
  for (int d = lane; d < hd; d += 32) {
    const float x = bf16_to_f32(src[d]);
    tmp[d] = __fmul_rn(x, x);
  }
  __syncwarp();
  float inv = 0.0f;
  if (tree_sum) { // fast mode: lane partial sums, then a shuffle tree (another order than the reference's)
    float sum = 0.0f;
    for (int d = lane; d < hd; d += 32)
      sum = __fadd_rn(sum, tmp[d]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
    inv = d_rsqrt(__fadd_rn(__fmul_rn(sum, __fdiv_rn(1.0f, static_cast<float>(hd))), 1.0e-6f));
  } else if (lane == 0) {
    float sum = 0.0f;
    int d = 0;
    for (; d + 16 <= hd; d += 16) { // sixteen squares are fetched, then added in order
      float sq[16];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        sq[u] = tmp[d + u];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        sum = __fadd_rn(sum, sq[u]);
    }
    for (; d < hd; ++d)
      sum = __fadd_rn(sum, tmp[d]);
    inv = d_rsqrt(__fadd_rn(__fmul_rn(sum, __fdiv_rn(1.0f, static_cast<float>(hd))), 1.0e-6f));
  }
  if (!tree_sum)
    inv = __shfl_sync(0xffffffffu, inv, 0);
  __syncwarp();
  if (prefetched) {
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) {
        const float x = bf16_to_f32(src[d]);
        tmp[d] = __fmul_rn(__fmul_rn(x, inv), __fadd_rn(1.0f, w_reg[i]));
      }
    }
  } else {
    for (int d = lane; d < hd; d += 32) {
      const float x = bf16_to_f32(src[d]);
      const float centered = __fadd_rn(1.0f, bf16_to_f32(weight[d]));
      tmp[d] = __fmul_rn(__fmul_rn(x, inv), centered);
    }
  }
  __syncwarp();
  const int half = rot / 2;
  uint16_t *vdst = cache + ((1 * static_cast<int64_t>(nkv) + head) * cap + position + tpos) * hd;
  if (prefetched) {
#pragma unroll
    for (int i = 0; i < kPerLane; ++i) {
      const int d = lane + 32 * i;
      if (d < hd) {
        float r = tmp[d];
        if (d < rot) {
          const bool second = d >= half;
          const float rotated = __fmul_rn(second ? 1.0f : -1.0f, tmp[second ? d - half : d + half]);
          r = __fadd_rn(__fmul_rn(tmp[d], cos_reg[i]), __fmul_rn(rotated, sin_reg[i]));
        }
        dst[d] = f32_to_bf16(r);
        if (!is_q)
          vdst[d] = v_reg[i];
      }
    }
    return;
  }
  for (int d = lane; d < hd; d += 32) {
    float r = tmp[d];
    if (d < rot) {
      const bool second = d >= half;
      const float rotated = __fmul_rn(second ? 1.0f : -1.0f, tmp[second ? d - half : d + half]);
      r = __fadd_rn(__fmul_rn(tmp[d], cos[(row_base + tpos) * rot + d]), __fmul_rn(rotated, sin[(row_base + tpos) * rot + d]));
    }
    dst[d] = f32_to_bf16(r);
  }
  if (!is_q) {
    for (int d = lane; d < hd; d += 32)
      vdst[d] = vsrc[d];
  }
}

constexpr int kKeyTile = 64;     // LowerAttention.cpp:124
constexpr int kValueTile = 32;  // value rows per shared-memory stage (divides kKeyTile)
constexpr int kValueStages = 6; // stages in flight: 6 x 32 x 256 x 2 B = 96 KB at head_dim 256

// grid: (key tile, kv head, token); block: group * 64 threads (query head x key).
__global__ void attn_scores_kernel(const uint16_t *__restrict__ qn, const uint16_t *__restrict__ cache,
                                   const int64_t *__restrict__ position_ptr, int nh, int nkv, int hd, int64_t cap,
                                   int64_t score_stride, float *__restrict__ scores, int64_t cache_stride) {
  extern __shared__ __align__(16) unsigned char att_sm[];
  grid_dependency_sync();
  const int64_t position = *position_ptr;
  const int group = nh / nkv;
  const int64_t t = blockIdx.z;
  const int kvh = blockIdx.y;
  cache += t * cache_stride; // rows of independent sequences: a cache per row, every row at `position`
  const int64_t query_end = position + (cache_stride ? 0 : t) + 1;
  const int64_t start = static_cast<int64_t>(blockIdx.x) * kKeyTile;
  if (start >= query_end)
    return;
  const int keys = static_cast<int>(min(static_cast<int64_t>(kKeyTile), query_end - start));
  const int kstride = hd + 1; // floats per key row, odd to spread banks
  float *k_sm = reinterpret_cast<float *>(att_sm);           // [64][hd+1]
  float *q_sm = k_sm + kKeyTile * kstride;                   // [group][hd]
  const uint16_t *kc = cache + (static_cast<int64_t>(kvh) * cap + start) * hd;
  if ((hd & 7) == 0) {
    const int per_row = hd >> 3; // 16-byte pieces per key
    for (int i = threadIdx.x; i < keys * per_row; i += blockDim.x) {
      const int row = i / per_row, piece = i - row * per_row;
      const uint4 raw = reinterpret_cast<const uint4 *>(kc)[i];
      float *dst = k_sm + row * kstride + piece * 8;
      const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        dst[2 * u] = __uint_as_float(w[u] << 16);
        dst[2 * u + 1] = __uint_as_float(w[u] & 0xffff0000u);
      }
    }
  } else {
    for (int i = threadIdx.x; i < keys * hd; i += blockDim.x)
      k_sm[(i / hd) * kstride + (i % hd)] = bf16_to_f32(kc[i]);
  }
  for (int i = threadIdx.x; i < group * hd; i += blockDim.x)
    q_sm[i] = bf16_to_f32(qn[(t * nh + kvh * group) * hd + i]);
  __syncthreads();
  const int j = threadIdx.x % kKeyTile;
  const int g = threadIdx.x / kKeyTile;
  if (j >= keys || g >= group)
    return;
  const float *kr = k_sm + j * kstride;
  const float *qr = q_sm + g * hd;
  float dot = 0.0f;
#pragma unroll 16
  for (int d = 0; d < hd; ++d)
    dot = __fadd_rn(dot, __fmul_rn(qr[d], kr[d]));
  const float scale = __fdiv_rn(1.0f, __fsqrt_rn(static_cast<float>(hd)));
  scores[(t * nh + kvh * group + g) * score_stride + start + j] = __fmul_rn(dot, scale);
}

// The scores of one query token against 32 keys per CTA, for head dimensions that are a multiple
// of eight (the one-token step).  Compared with the kernel above: half the keys per CTA, so twice
// as many SMs fetch key rows; a thread's 16-byte pieces of the tile are all requested before the
// first is converted; rows are hd + 4 floats apart, so that keys and queries are read four
// dimensions at a time (a quarter warp's eight rows fall on distinct banks).  The dot product
// is the same ascending-d chain  dot = dot + q[d] * k[d].
// grid: (32-key tile, kv head, token); block: group * 32 threads (query head x key).
constexpr int kScoreKeys = 32;

__global__ void __launch_bounds__(256)
attn_scores_keys32_kernel(const uint16_t *__restrict__ qn, const uint16_t *__restrict__ cache,
                          const int64_t *__restrict__ position_ptr, int nh, int nkv, int hd, int64_t cap,
                          int64_t score_stride, float *__restrict__ scores, int64_t cache_stride) {
  extern __shared__ __align__(16) unsigned char att_sm[];
  grid_dependency_sync();
  const int64_t position = *position_ptr;
  const int group = nh / nkv;
  const int64_t t = blockIdx.z;
  const int kvh = blockIdx.y;
  cache += t * cache_stride; // rows of independent sequences: a cache per row, every row at `position`
  const int64_t query_end = position + (cache_stride ? 0 : t) + 1;
  const int64_t start = static_cast<int64_t>(blockIdx.x) * kScoreKeys;
  if (start >= query_end)
    return;
  const int keys = static_cast<int>(min(static_cast<int64_t>(kScoreKeys), query_end - start));
  const int kstride = hd + 4;
  float *k_sm = reinterpret_cast<float *>(att_sm); // [32][hd + 4]
  float *q_sm = k_sm + kScoreKeys * kstride;       // [group][hd]
  const uint4 *kc = reinterpret_cast<const uint4 *>(cache + (static_cast<int64_t>(kvh) * cap + start) * hd);
  const int per_row = hd >> 3; // 16-byte pieces per key
  const int pieces = keys * per_row;
  auto unpack = [](float *dst, const uint4 &raw) {
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float4 lo, hi;
    lo.x = __uint_as_float(w[0] << 16);
    lo.y = __uint_as_float(w[0] & 0xffff0000u);
    lo.z = __uint_as_float(w[1] << 16);
    lo.w = __uint_as_float(w[1] & 0xffff0000u);
    hi.x = __uint_as_float(w[2] << 16);
    hi.y = __uint_as_float(w[2] & 0xffff0000u);
    hi.z = __uint_as_float(w[3] << 16);
    hi.w = __uint_as_float(w[3] & 0xffff0000u);
    reinterpret_cast<float4 *>(dst)[0] = lo;
    reinterpret_cast<float4 *>(dst)[1] = hi;
  };
  for (int base = 0; base < pieces; base += 8 * blockDim.x) {
    uint4 raw[8];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const int i = base + n * blockDim.x + threadIdx.x;
      if (i < pieces)
        raw[n] = kc[i];
    }
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const int i = base + n * blockDim.x + threadIdx.x;
      if (i < pieces) {
        const int row = i / per_row, piece = i - row * per_row;
        unpack(k_sm + row * kstride + piece * 8, raw[n]);
      }
    }
  }
  const uint4 *qc = reinterpret_cast<const uint4 *>(qn + (t * nh + kvh * group) * hd);
  for (int i = threadIdx.x; i < group * per_row; i += blockDim.x)
    unpack(q_sm + i * 8, qc[i]);
  __syncthreads();
  const int j = threadIdx.x % kScoreKeys;
  const int g = threadIdx.x / kScoreKeys;
  if (j >= keys || g >= group)
    return;
  const float4 *kr = reinterpret_cast<const float4 *>(k_sm + j * kstride);
  const float4 *qr = reinterpret_cast<const float4 *>(q_sm + g * hd);
  float dot = 0.0f;
#pragma unroll 8
  for (int d4 = 0; d4 < (hd >> 2); ++d4) {
    const float4 kv = kr[d4], qv = qr[d4];
    dot = __fadd_rn(dot, __fmul_rn(qv.x, kv.x));
    dot = __fadd_rn(dot, __fmul_rn(qv.y, kv.y));
    dot = __fadd_rn(dot, __fmul_rn(qv.z, kv.z));
    dot = __fadd_rn(dot, __fmul_rn(qv.w, kv.w));
  }
  const float scale = __fdiv_rn(1.0f, __fsqrt_rn(static_cast<float>(hd)));
  scores[(t * nh + kvh * group + g) * score_stride + start + j] = __fmul_rn(dot, scale);
}

// The same scores for a block of kScoreTokens query tokens per CTA (prefill): the key tile is
// brought into shared memory once per block instead of once per token, and a thread advances the
// dot products of four tokens together, reading its key row four values at a time.  Every dot
// product is still the ascending-d chain  dot = dot + q[d] * k[d]  of the kernel above.
// grid: (key tile, kv head, token block); block: group * 64 threads (query head x key).
constexpr int kScoreTokens = 8;

__global__ void __launch_bounds__(256)
attn_scores_block_kernel(const uint16_t *__restrict__ qn, const uint16_t *__restrict__ cache,
                         const int64_t *__restrict__ position_ptr, int64_t S, int nh, int nkv, int hd, int64_t cap,
                         int64_t score_stride, float *__restrict__ scores) {
  extern __shared__ __align__(16) unsigned char att_sm[];
  grid_dependency_sync();
  const int64_t position = *position_ptr;
  const int group = nh / nkv;
  const int64_t t0 = static_cast<int64_t>(blockIdx.z) * kScoreTokens;
  const int tokens = static_cast<int>(min(static_cast<int64_t>(kScoreTokens), S - t0));
  const int kvh = blockIdx.y;
  const int64_t last_end = position + t0 + tokens; // keys the last token of the block sees
  const int64_t start = static_cast<int64_t>(blockIdx.x) * kKeyTile;
  if (start >= last_end)
    return;
  const int keys = static_cast<int>(min(static_cast<int64_t>(kKeyTile), last_end - start));
  const int kstride = hd + 4; // floats per key row: 16-byte aligned, four banks apart
  float *k_sm = reinterpret_cast<float *>(att_sm);  // [64][hd+4]
  float *q_sm = k_sm + kKeyTile * kstride;          // [tokens][group][hd]
  const uint16_t *kc = cache + (static_cast<int64_t>(kvh) * cap + start) * hd;
  const int per_row = hd >> 3; // 16-byte pieces per key (hd % 8 == 0)
  auto unpack = [](float *dst, const uint4 &raw) {
    float4 lo, hi;
    lo.x = __uint_as_float(raw.x << 16);
    lo.y = __uint_as_float(raw.x & 0xffff0000u);
    lo.z = __uint_as_float(raw.y << 16);
    lo.w = __uint_as_float(raw.y & 0xffff0000u);
    hi.x = __uint_as_float(raw.z << 16);
    hi.y = __uint_as_float(raw.z & 0xffff0000u);
    hi.z = __uint_as_float(raw.w << 16);
    hi.w = __uint_as_float(raw.w & 0xffff0000u);
    reinterpret_cast<float4 *>(dst)[0] = lo;
    reinterpret_cast<float4 *>(dst)[1] = hi;
  };
  // A thread's pieces are all requested before the first is converted: one round trip to
  // memory for the tile instead of one per piece.
  const int key_pieces = kKeyTile * per_row;
  for (int base = 0; base < key_pieces; base += 8 * blockDim.x) {
    uint4 raw[8];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const int i = base + n * blockDim.x + threadIdx.x;
      raw[n] = make_uint4(0u, 0u, 0u, 0u);
      if (i < key_pieces && i / per_row < keys)
        raw[n] = reinterpret_cast<const uint4 *>(kc)[i];
    }
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      const int i = base + n * blockDim.x + threadIdx.x;
      if (i < key_pieces) {
        const int row = i / per_row, piece = i - row * per_row;
        unpack(k_sm + row * kstride + piece * 8, raw[n]);
      }
    }
  }
  const int token_pieces = group * per_row; // 16-byte pieces of one token's query heads
  for (int i = threadIdx.x; i < kScoreTokens * token_pieces; i += blockDim.x) {
    const int tb = i / token_pieces, rest = i - tb * token_pieces;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (tb < tokens)
      raw = reinterpret_cast<const uint4 *>(qn + ((t0 + tb) * nh + kvh * group) * hd)[rest];
    unpack(q_sm + i * 8, raw);
  }
  __syncthreads();
  const int j = threadIdx.x % kKeyTile;
  const int g = threadIdx.x / kKeyTile;
  if (g >= group)
    return;
  const float4 *kr = reinterpret_cast<const float4 *>(k_sm + j * kstride);
  const float scale = __fdiv_rn(1.0f, __fsqrt_rn(static_cast<float>(hd)));
#pragma unroll
  for (int tb0 = 0; tb0 < kScoreTokens; tb0 += 4) {
    if (tb0 >= tokens)
      break;
    const float4 *q0 = reinterpret_cast<const float4 *>(q_sm + ((tb0 + 0) * group + g) * hd);
    const float4 *q1 = reinterpret_cast<const float4 *>(q_sm + ((tb0 + 1) * group + g) * hd);
    const float4 *q2 = reinterpret_cast<const float4 *>(q_sm + ((tb0 + 2) * group + g) * hd);
    const float4 *q3 = reinterpret_cast<const float4 *>(q_sm + ((tb0 + 3) * group + g) * hd);
    float dot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll 4
    for (int d4 = 0; d4 < (hd >> 2); ++d4) {
      const float4 kv = kr[d4];
      const float4 qv[4] = {q0[d4], q1[d4], q2[d4], q3[d4]};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        dot[u] = __fadd_rn(dot[u], __fmul_rn(qv[u].x, kv.x));
        dot[u] = __fadd_rn(dot[u], __fmul_rn(qv[u].y, kv.y));
        dot[u] = __fadd_rn(dot[u], __fmul_rn(qv[u].z, kv.z));
        dot[u] = __fadd_rn(dot[u], __fmul_rn(qv[u].w, kv.w));
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t t = t0 + tb0 + u;
      if (tb0 + u < tokens && start + j < position + t + 1)
        scores[(t * nh + kvh * group + g) * score_stride + start + j] = __fmul_rn(dot[u], scale);
    }
  }
}

// Bounded wait for a phase of a value-stage mbarrier; false when the limit ran out.
__device__ __forceinline__ bool value_wait(uint64_t *bar, uint32_t parity) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(bar));
  for (uint32_t spin = 0; spin < (1u << 22); ++spin) {
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

// grid: (head, token); block: hd rounded up to a warp multiple.
// Shared memory: the row's scores (turned into probabilities in place), then per key tile the
// running maximum and the correction factor.  The maxima, corrections and probabilities are
// formed tile by tile with the reference's operations but all up front; what is left for the
// ordered part is  acc = acc * c_tile;  acc += p_j * V[j][d]  in ascending key order.
__global__ void attn_combine_kernel(const float *__restrict__ scores, const uint16_t *__restrict__ cache,
                                    const uint16_t *__restrict__ qg, const int64_t *__restrict__ position_ptr,
                                    int nh, int nkv, int hd, int64_t cap, int64_t score_stride,
                                    uint16_t *__restrict__ out, int8_t *__restrict__ q_out,
                                    float *__restrict__ s_out, int64_t cache_stride) {
  extern __shared__ __align__(16) float comb_sm[];
  grid_dependency_sync(true);
  const int64_t position = *position_ptr;
  const int h = blockIdx.x;
  const int64_t t = blockIdx.y;
  const int kvh = h / (nh / nkv);
  const int d = threadIdx.x;
  const bool active = d < hd;
  cache += t * cache_stride; // rows of independent sequences: a cache per row, every row at `position`
  const int total = static_cast<int>(position + (cache_stride ? 0 : t) + 1);
  const int tiles = (total + kKeyTile - 1) / kKeyTile;
  float *p_sm = comb_sm;
  float *m_sm = comb_sm + (static_cast<int>(score_stride) + 3) / 4 * 4;
  float *c_sm = m_sm + (static_cast<int>(score_stride) + kKeyTile - 1) / kKeyTile;
  const float *srow = scores + (t * nh + h) * score_stride;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;

  // Value rows (32 keys x hd bf16, contiguous in the cache) stream through a ring of
  // shared-memory stages, one bulk copy per stage that signals the stage's mbarrier.  The first
  // stages are requested here, so that they travel while the probabilities are being formed.
  const bool bulk = (hd & 7) == 0;
  const uint16_t *vbase = cache + ((static_cast<int64_t>(nkv) + kvh) * cap) * hd;
  const int used_floats = static_cast<int>(c_sm - comb_sm) + (static_cast<int>(score_stride) + kKeyTile - 1) / kKeyTile;
  uint16_t *v_sm = reinterpret_cast<uint16_t *>(comb_sm + (used_floats + 3) / 4 * 4);
  const int stage_elems = kValueTile * hd;
  uint64_t *bars = reinterpret_cast<uint64_t *>(v_sm + kValueStages * stage_elems);
  const int value_tiles = (total + kValueTile - 1) / kValueTile;
  auto request = [&](int tile) {
    if (threadIdx.x == 0 && tile < value_tiles) {
      const uint32_t bytes = static_cast<uint32_t>(min(kValueTile, total - tile * kValueTile) * hd * 2);
      const uint32_t bar = static_cast<uint32_t>(__cvta_generic_to_shared(bars + tile % kValueStages));
      const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(v_sm + (tile % kValueStages) * stage_elems));
      // generic-proxy reads of the stage (before the barrier in front of this call) stay ahead of the copy
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                   "l"(vbase + static_cast<int64_t>(tile) * stage_elems), "r"(bytes), "r"(bar)
                   : "memory");
    }
  };
  if (bulk && threadIdx.x == 0) {
    for (int s = 0; s < kValueStages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(bars + s)))
                   : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int tile = 0; tile < kValueStages - 1; ++tile)
      request(tile);
  }

  for (int j = threadIdx.x; j < total; j += blockDim.x)
    p_sm[j] = srow[j];
  __syncthreads();
  for (int tile = warp; tile < tiles; tile += warps) {
    float m = -1.0e30f;
    for (int j = tile * kKeyTile + lane; j < min(total, (tile + 1) * kKeyTile); j += 32)
      m = fmaxf(m, p_sm[j]);
    for (int o = 16; o > 0; o >>= 1)
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0)
      m_sm[tile] = m;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float running = -1.0e30f;
    for (int tile = 0; tile < tiles; ++tile) {
      const float next = fmaxf(running, m_sm[tile]);
      c_sm[tile] = __fsub_rn(running, next); // exponent of the correction, exp taken below
      m_sm[tile] = next;
      running = next;
    }
  }
  __syncthreads();
  for (int tile = threadIdx.x; tile < tiles; tile += blockDim.x)
    c_sm[tile] = d_exp(c_sm[tile]);
  for (int j = threadIdx.x; j < total; j += blockDim.x)
    p_sm[j] = d_exp(__fsub_rn(p_sm[j], m_sm[j / kKeyTile]));
  __syncthreads();

  float acc = 0.0f, sum = 0.0f;
  if (bulk) {
    // Shared memory serves one wavefront per cycle, and with a thread per dimension every key
    // cost sixteen of them (eight warps, a probability and a 64-byte value piece each).  So the
    // first hd / 2 threads take two neighbouring dimensions each (one 32-bit load per key, a
    // full 128-byte wavefront per warp) and read the probabilities four at a time; the last
    // thread of the block keeps the denominator, which every thread used to repeat.  Per
    // dimension the operations and their order are unchanged.
    const int pair_threads = hd >> 1;
    const bool accumulates = static_cast<int>(threadIdx.x) < pair_threads;
    const bool sums = threadIdx.x == blockDim.x - 1; // blockDim.x >= hd, so never an accumulating thread
    float acc0 = 0.0f, acc1 = 0.0f;
    bool ok = true;
    int tile = 0;
    for (; tile < value_tiles; ++tile) {
      ok = value_wait(&bars[tile % kValueStages], (tile / kValueStages) & 1);
      // Stage `tile` has landed; after the barrier everyone has left stage `tile - 1`, which
      // the copy of tile + kValueStages - 1 may then overwrite.
      ok = __syncthreads_and(ok);
      if (!ok)
        break;
      request(tile + kValueStages - 1);
      const int first = tile * kValueTile;
      const bool corrected = (first & (kKeyTile - 1)) == 0;
      const float correction = corrected ? c_sm[first / kKeyTile] : 1.0f;
      const int count = min(kValueTile, total - first);
      if (accumulates) {
        const uint32_t *rows =
            reinterpret_cast<const uint32_t *>(v_sm + (tile % kValueStages) * stage_elems) + threadIdx.x;
        if (corrected) {
          acc0 = __fmul_rn(acc0, correction);
          acc1 = __fmul_rn(acc1, correction);
        }
        if (count == kValueTile) {
#pragma unroll
          for (int q = 0; q < kValueTile / 4; ++q) {
            const float4 p4 = *reinterpret_cast<const float4 *>(p_sm + first + 4 * q);
            const float pv[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const uint32_t pair = rows[(4 * q + u) * pair_threads];
              acc0 = __fadd_rn(acc0, __fmul_rn(pv[u], __uint_as_float(pair << 16)));
              acc1 = __fadd_rn(acc1, __fmul_rn(pv[u], __uint_as_float(pair & 0xffff0000u)));
            }
          }
        } else {
          for (int u = 0; u < count; ++u) {
            const float p = p_sm[first + u];
            const uint32_t pair = rows[u * pair_threads];
            acc0 = __fadd_rn(acc0, __fmul_rn(p, __uint_as_float(pair << 16)));
            acc1 = __fadd_rn(acc1, __fmul_rn(p, __uint_as_float(pair & 0xffff0000u)));
          }
        }
      } else if (sums) {
        if (corrected)
          sum = __fmul_rn(sum, correction);
        for (int u = 0; u < count; ++u)
          sum = __fadd_rn(sum, p_sm[first + u]);
      }
    }
    if (!ok) {
      // A copy did not arrive within the limit: give the copies still in flight one more
      // bounded chance to land before the CTA leaves, and report through the result.
      for (int pending = tile; pending < min(value_tiles, tile + kValueStages - 1); ++pending)
        value_wait(&bars[pending % kValueStages], (pending / kValueStages) & 1);
      acc0 = acc1 = sum = __int_as_float(0x7fc00000);
    }
    __syncthreads(); // probabilities and value stages are dead: their space carries the results across
    if (accumulates) {
      comb_sm[2 * threadIdx.x] = acc0;
      comb_sm[2 * threadIdx.x + 1] = acc1;
    }
    if (sums)
      comb_sm[hd] = sum;
    __syncthreads();
    acc = comb_sm[active ? d : 0];
    sum = comb_sm[hd];
  } else {
    const uint16_t *vc = vbase + (active ? d : 0);
    for (int j = 0; j < total; ++j) {
      if ((j & (kKeyTile - 1)) == 0) {
        const float correction = c_sm[j / kKeyTile];
        acc = __fmul_rn(acc, correction);
        sum = __fmul_rn(sum, correction);
      }
      const float p = p_sm[j];
      sum = __fadd_rn(sum, p);
      if (active)
        acc = __fadd_rn(acc, __fmul_rn(p, bf16_to_f32(vc[static_cast<int64_t>(j) * hd])));
    }
  }
  float result = 0.0f;
  const int64_t index = t * nh * hd + static_cast<int64_t>(h) * hd + d;
  if (active) {
    const float gate = bf16_to_f32(qg[t * nh * 2 * hd + static_cast<int64_t>(h) * 2 * hd + hd + d]);
    const float gated = __fmul_rn(__fdiv_rn(acc, sum), d_sigmoid(gate));
    const uint16_t bits = f32_to_bf16(gated);
    out[index] = bits;
    result = bf16_to_f32(bits);
  }
  if (q_out) { // the quantisation the following o_proj needs (Q8Decode.cpp:83-120); hd % 32 == 0
    float amax = fabsf(result);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = __fdiv_rn(amax, 127.0f);
    const float inv = amax == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
    if (active) {
      q_out[index] = static_cast<int8_t>(__float2int_rn(__fmul_rn(result, inv)));
      if (lane == 0)
        s_out[index >> 5] = scale;
    }
  }
}

// The same weighted sum for a block of kCombineTokens query tokens of one head per CTA (prefill):
// a value row is brought into shared memory once per block instead of once per token, and a
// thread accumulates two head dimensions for all tokens of the block.  hd / 2 threads accumulate;
// one more warp keeps the softmax denominators (lane tb walks token tb's probabilities in key
// order, which every dimension thread used to repeat).  Per (token, dimension) the operations and
// their order are those of the kernel above: correction at every 64-key tile, then
// acc = acc + p * v key by key.
constexpr int kCombineTokens = 8;
constexpr int kBlockStages = 4;

__global__ void __launch_bounds__(160)
attn_combine_block_kernel(const float *__restrict__ scores, const uint16_t *__restrict__ cache,
                          const uint16_t *__restrict__ qg, const int64_t *__restrict__ position_ptr, int64_t S, int nh,
                          int nkv, int hd, int64_t cap, int64_t score_stride, int p_stride, uint16_t *__restrict__ out,
                          int8_t *__restrict__ q_out, float *__restrict__ s_out) {
  extern __shared__ __align__(16) float comb_sm[];
  grid_dependency_sync(true);
  const int64_t position = *position_ptr;
  const int h = blockIdx.x;
  const int64_t t0 = static_cast<int64_t>(blockIdx.y) * kCombineTokens;
  const int tokens = static_cast<int>(min(static_cast<int64_t>(kCombineTokens), S - t0));
  const int kvh = h / (nh / nkv);
  const int total0 = static_cast<int>(position + t0 + 1);       // keys the first token sees
  const int total_last = total0 + tokens - 1;                   // keys the last token sees
  const int tiles_max = (total_last + kKeyTile - 1) / kKeyTile;
  const int tile_slots = (p_stride + kKeyTile - 1) / kKeyTile;
  float *p_sm = comb_sm;                                         // [tokens][p_stride]
  float *m_sm = p_sm + kCombineTokens * p_stride;                // [tokens][tile_slots]
  float *c_sm = m_sm + kCombineTokens * tile_slots;              // [tokens][tile_slots]
  float *sum_sm = c_sm + kCombineTokens * tile_slots;            // [tokens]
  uint16_t *v_sm = reinterpret_cast<uint16_t *>(sum_sm + kCombineTokens);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  const int pairs = hd >> 1;
  const int d = threadIdx.x;
  const bool consumer = d < pairs;        // dimensions 2 d and 2 d + 1
  const bool keeper = d >= pairs && lane < tokens; // the extra warp: lane tb keeps token tb's denominator

  // Value rows arrive by one bulk copy per 32-key stage (see the one-token kernel); the first
  // stages are requested before the probabilities are formed.  The first lane of the extra
  // warp issues the requests.
  const uint16_t *vbase = cache + ((static_cast<int64_t>(nkv) + kvh) * cap) * hd;
  const int stage_elems = kValueTile * hd;
  const int value_tiles = (total_last + kValueTile - 1) / kValueTile;
  uint64_t *bars = reinterpret_cast<uint64_t *>(v_sm + kBlockStages * stage_elems);
  auto request = [&](int tile) {
    if (d == pairs && tile < value_tiles) {
      const uint32_t bytes = static_cast<uint32_t>(min(kValueTile, total_last - tile * kValueTile) * hd * 2);
      const uint32_t bar = static_cast<uint32_t>(__cvta_generic_to_shared(bars + tile % kBlockStages));
      const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(v_sm + (tile % kBlockStages) * stage_elems));
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                   "l"(vbase + static_cast<int64_t>(tile) * stage_elems), "r"(bytes), "r"(bar)
                   : "memory");
    }
  };
  if (d == pairs) {
    for (int s = 0; s < kBlockStages; ++s)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(bars + s)))
                   : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    for (int tile = 0; tile < kBlockStages - 1; ++tile)
      request(tile);
  }

  // probabilities of every token of the block (as in the one-token kernel)
  for (int tb = 0; tb < tokens; ++tb) {
    const float *srow = scores + ((t0 + tb) * nh + h) * score_stride;
    for (int j = threadIdx.x; j < total0 + tb; j += blockDim.x)
      p_sm[tb * p_stride + j] = srow[j];
  }
  __syncthreads();
  for (int item = warp; item < tokens * tiles_max; item += warps) {
    const int tb = item / tiles_max, tile = item - tb * tiles_max;
    const int total = total0 + tb;
    float m = -1.0e30f;
    for (int j = tile * kKeyTile + lane; j < min(total, (tile + 1) * kKeyTile); j += 32)
      m = fmaxf(m, p_sm[tb * p_stride + j]);
    for (int o = 16; o > 0; o >>= 1)
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0)
      m_sm[tb * tile_slots + tile] = m;
  }
  __syncthreads();
  if (threadIdx.x < tokens) {
    const int tb = threadIdx.x;
    const int tiles = (total0 + tb + kKeyTile - 1) / kKeyTile;
    float running = -1.0e30f;
    for (int tile = 0; tile < tiles; ++tile) {
      const float next = fmaxf(running, m_sm[tb * tile_slots + tile]);
      c_sm[tb * tile_slots + tile] = __fsub_rn(running, next); // exponent of the correction, exp taken below
      m_sm[tb * tile_slots + tile] = next;
      running = next;
    }
  }
  __syncthreads();
  for (int tb = 0; tb < tokens; ++tb) {
    const int total = total0 + tb;
    const int tiles = (total + kKeyTile - 1) / kKeyTile;
    for (int tile = threadIdx.x; tile < tiles; tile += blockDim.x)
      c_sm[tb * tile_slots + tile] = d_exp(c_sm[tb * tile_slots + tile]);
    for (int j = threadIdx.x; j < total; j += blockDim.x)
      p_sm[tb * p_stride + j] = d_exp(__fsub_rn(p_sm[tb * p_stride + j], m_sm[tb * tile_slots + j / kKeyTile]));
  }
  __syncthreads();

  float acc0[kCombineTokens], acc1[kCombineTokens];
#pragma unroll
  for (int tb = 0; tb < kCombineTokens; ++tb)
    acc0[tb] = acc1[tb] = 0.0f;
  float sum = 0.0f; // keeper lanes only
  bool ok = true;
  int tile = 0;
  for (; tile < value_tiles; ++tile) {
    ok = value_wait(&bars[tile % kBlockStages], (tile / kBlockStages) & 1);
    // stage `tile` has landed; after the barrier stage `tile - 1` is free for the next copy
    ok = __syncthreads_and(ok);
    if (!ok)
      break;
    request(tile + kBlockStages - 1);
    const int first = tile * kValueTile;
    const int count = min(kValueTile, total_last - first);
    if (consumer) {
      const uint32_t *rows = reinterpret_cast<const uint32_t *>(v_sm + (tile % kBlockStages) * stage_elems) + d;
      if ((first & (kKeyTile - 1)) == 0) {
#pragma unroll
        for (int tb = 0; tb < kCombineTokens; ++tb) {
          if (tb < tokens && first < total0 + tb) {
            const float correction = c_sm[tb * tile_slots + first / kKeyTile];
            acc0[tb] = __fmul_rn(acc0[tb], correction);
            acc1[tb] = __fmul_rn(acc1[tb], correction);
          }
        }
      }
      if (first + kValueTile <= total0 && tokens == kCombineTokens) {
        // every key of the stage is visible to every token of the block
#pragma unroll 2
        for (int u4 = 0; u4 < kValueTile; u4 += 4) {
          float v0[4], v1[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const uint32_t v2 = rows[(u4 + u) * pairs];
            v0[u] = __uint_as_float(v2 << 16);
            v1[u] = __uint_as_float(v2 & 0xffff0000u);
          }
#pragma unroll
          for (int tb = 0; tb < kCombineTokens; ++tb) {
            const float4 p4 = *reinterpret_cast<const float4 *>(p_sm + tb * p_stride + first + u4);
            const float p[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              acc0[tb] = __fadd_rn(acc0[tb], __fmul_rn(p[u], v0[u]));
              acc1[tb] = __fadd_rn(acc1[tb], __fmul_rn(p[u], v1[u]));
            }
          }
        }
      } else {
        for (int u = 0; u < count; ++u) {
          const uint32_t v2 = rows[u * pairs];
          const float v0 = __uint_as_float(v2 << 16), v1 = __uint_as_float(v2 & 0xffff0000u);
#pragma unroll
          for (int tb = 0; tb < kCombineTokens; ++tb) {
            if (tb < tokens && first + u < total0 + tb) {
              const float p = p_sm[tb * p_stride + first + u];
              acc0[tb] = __fadd_rn(acc0[tb], __fmul_rn(p, v0));
              acc1[tb] = __fadd_rn(acc1[tb], __fmul_rn(p, v1));
            }
          }
        }
      }
    } else if (keeper) {
      const int tb = lane, total = total0 + tb;
      if ((first & (kKeyTile - 1)) == 0 && first < total)
        sum = __fmul_rn(sum, c_sm[tb * tile_slots + first / kKeyTile]);
      const int mine = min(count, total - first);
      for (int u = 0; u < mine; ++u)
        sum = __fadd_rn(sum, p_sm[tb * p_stride + first + u]);
    }
  }
  if (!ok) {
    // A copy did not arrive within the limit: one more bounded chance for the copies still in
    // flight to land before the CTA leaves; the result reports it as NaN.
    for (int pending = tile; pending < min(value_tiles, tile + kBlockStages - 1); ++pending)
      value_wait(&bars[pending % kBlockStages], (pending / kBlockStages) & 1);
    sum = __int_as_float(0x7fc00000);
  }
  if (keeper)
    sum_sm[lane] = sum;
  __syncthreads();
  // gate, bf16, and the quantisation the following o_proj needs (Q8Decode.cpp:83-120): a 32-wide
  // block is held by 16 neighbouring accumulating threads.
#pragma unroll
  for (int tb = 0; tb < kCombineTokens; ++tb) {
    if (tb >= tokens)
      break;
    const int64_t t = t0 + tb;
    const int64_t index = t * nh * hd + static_cast<int64_t>(h) * hd + 2 * d;
    float r0 = 0.0f, r1 = 0.0f;
    if (consumer) {
      const float denominator = sum_sm[tb];
      const uint32_t gate2 = *reinterpret_cast<const uint32_t *>(qg + t * nh * 2 * hd + static_cast<int64_t>(h) * 2 * hd + hd + 2 * d);
      const uint16_t b0 = f32_to_bf16(__fmul_rn(__fdiv_rn(acc0[tb], denominator), d_sigmoid(__uint_as_float(gate2 << 16))));
      const uint16_t b1 = f32_to_bf16(__fmul_rn(__fdiv_rn(acc1[tb], denominator), d_sigmoid(__uint_as_float(gate2 & 0xffff0000u))));
      *reinterpret_cast<uint32_t *>(out + index) = static_cast<uint32_t>(b0) | (static_cast<uint32_t>(b1) << 16);
      r0 = bf16_to_f32(b0);
      r1 = bf16_to_f32(b1);
    }
    if (q_out) { // hd % 32 == 0
      float amax = fmaxf(fabsf(r0), fabsf(r1));
#pragma unroll
      for (int o = 8; o > 0; o >>= 1)
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float scale = __fdiv_rn(amax, 127.0f);
      const float inv = amax == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
      if (consumer) {
        const uint32_t q0 = static_cast<uint32_t>(__float2int_rn(__fmul_rn(r0, inv))) & 0xffu;
        const uint32_t q1 = static_cast<uint32_t>(__float2int_rn(__fmul_rn(r1, inv))) & 0xffu;
        *reinterpret_cast<uint16_t *>(q_out + index) = static_cast<uint16_t>(q0 | (q1 << 8));
        if ((d & 15) == 0)
          s_out[index >> 5] = scale;
      }
    }
  }
}

static size_t combine_smem_bytes(int64_t score_stride, int hd) {
  const size_t tiles = static_cast<size_t>((score_stride + kKeyTile - 1) / kKeyTile);
  size_t bytes = ((static_cast<size_t>(score_stride) + 3) / 4 * 4 + 2 * tiles) * sizeof(float);
  bytes = (bytes + 15) / 16 * 16;
  if ((hd & 7) == 0)
    bytes += static_cast<size_t>(kValueStages) * kValueTile * hd * sizeof(uint16_t) + kValueStages * sizeof(uint64_t);
  return bytes;
}

size_t attn_scratch_bytes(int64_t S, int nh, int hd, int64_t max_position) {
  const size_t score_stride = static_cast<size_t>(max_position + S);
  return static_cast<size_t>(S) * nh * hd * sizeof(uint16_t) + 256 +
         static_cast<size_t>(S) * nh * score_stride * sizeof(float);
}

cudaError_t launch_attention_prepare(const uint16_t *qg, const uint16_t *k, const uint16_t *v, const uint16_t *q_norm,
                                     const uint16_t *k_norm, const float *cos, const float *sin, int rows_from_position,
                                     uint16_t *cache, const int64_t *position_dev, int64_t S, int nh, int nkv, int hd,
                                     int rot, int64_t cap, uint16_t *qn, cudaStream_t stream, int tree_sum, int64_t cache_stride) {
  const int64_t items = S * (nh + nkv);
  const int prepare_warps = items <= 64 ? 1 : 4; // decode: a CTA per head
  launch_chained(attn_prepare_kernel, dim3(static_cast<unsigned>((items + prepare_warps - 1) / prepare_warps)),
                 dim3(32 * prepare_warps), prepare_warps * hd * sizeof(float), stream, qg, k, v, q_norm, k_norm, cos, sin, cache,
                 position_dev, rows_from_position, S, nh, nkv, hd, rot, cap, qn, tree_sum, cache_stride);
  return cudaGetLastError();
}

cudaError_t launch_attention(const uint16_t *qg, const uint16_t *k, const uint16_t *v,
                             const uint16_t *q_norm, const uint16_t *k_norm, const float *cos,
                             const float *sin, int rows_from_position, uint16_t *cache,
                             const int64_t *position_dev, int64_t max_position, int64_t S, int nh, int nkv,
                             int hd, int rot, int64_t cap, void *scratch, uint16_t *out, int8_t *q_out, float *s_out,
                             cudaStream_t stream, int64_t cache_stride) {
  if (S == 0)
    return cudaSuccess;
  if (q_out && hd % kBlock != 0)
    return cudaErrorInvalidValue;
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0 || rot % 2 != 0 || rot > hd || max_position + (cache_stride ? 1 : S) > cap)
    return cudaErrorInvalidValue;
  const int group = nh / nkv;
  if (group * kKeyTile > 1024 || hd > 1024)
    return cudaErrorInvalidValue;
  uint16_t *qn = static_cast<uint16_t *>(scratch);
  const size_t qn_bytes = (static_cast<size_t>(S) * nh * hd * sizeof(uint16_t) + 255) / 256 * 256;
  float *scores = reinterpret_cast<float *>(static_cast<unsigned char *>(scratch) + qn_bytes);
  const int64_t score_stride = max_position + S;

  if (cudaError_t e = launch_attention_prepare(qg, k, v, q_norm, k_norm, cos, sin, rows_from_position, cache, position_dev, S,
                                               nh, nkv, hd, rot, cap, qn, stream, 0, cache_stride);
      e != cudaSuccess)
    return e;

  const size_t smem = (static_cast<size_t>(kKeyTile) * (hd + 1) + static_cast<size_t>(group) * hd) * sizeof(float);
  const size_t csmem = combine_smem_bytes(score_stride, hd);
  {
    cudaError_t e = opt_in_shared_memory(reinterpret_cast<const void *>(attn_scores_kernel), 200 * 1024);
    if (e == cudaSuccess)
      e = opt_in_shared_memory(reinterpret_cast<const void *>(attn_combine_kernel), 200 * 1024);
    if (e != cudaSuccess)
      return e;
  }
  if (smem > 200 * 1024 || csmem > 200 * 1024)
    return cudaErrorInvalidValue; // about 50,000 cached positions
  const size_t block_smem = (static_cast<size_t>(kKeyTile) * (hd + 4) + static_cast<size_t>(kScoreTokens) * group * hd) * sizeof(float);
  if (S >= 4 && cache_stride == 0 && (hd & 7) == 0 && group * kKeyTile <= 256 && block_smem <= 200 * 1024) {
    if (cudaError_t e = opt_in_shared_memory(reinterpret_cast<const void *>(attn_scores_block_kernel), 200 * 1024); e != cudaSuccess)
      return e;
    dim3 bgrid(static_cast<unsigned>((max_position + S + kKeyTile - 1) / kKeyTile), nkv,
               static_cast<unsigned>((S + kScoreTokens - 1) / kScoreTokens));
    launch_chained(attn_scores_block_kernel, dim3(bgrid), dim3(group * kKeyTile), block_smem, stream, qn, cache, position_dev, S,
                   nh, nkv, hd, cap, score_stride, scores);
  } else if ((hd & 7) == 0 && group * kScoreKeys <= 256 && (static_cast<size_t>(kScoreKeys) * (hd + 4) + static_cast<size_t>(group) * hd) * sizeof(float) <= 48 * 1024) {
    const size_t keys32_smem = (static_cast<size_t>(kScoreKeys) * (hd + 4) + static_cast<size_t>(group) * hd) * sizeof(float);
    dim3 sgrid(static_cast<unsigned>((max_position + S + kScoreKeys - 1) / kScoreKeys), nkv, static_cast<unsigned>(S));
    launch_chained(attn_scores_keys32_kernel, dim3(sgrid), dim3(group * kScoreKeys), keys32_smem, stream, qn, cache, position_dev, nh,
                   nkv, hd, cap, score_stride, scores, cache_stride);
  } else {
    dim3 sgrid(static_cast<unsigned>((max_position + S + kKeyTile - 1) / kKeyTile), nkv, static_cast<unsigned>(S));
    launch_chained(attn_scores_kernel, dim3(sgrid), dim3(group * kKeyTile), smem, stream, qn, cache, position_dev, nh, nkv, hd,
                   cap, score_stride, scores, cache_stride);
  }
  // Prefill: eight tokens of a head per CTA when their probabilities fit in shared memory.
  const int p_stride = static_cast<int>((score_stride + 3) / 4 * 4);
  const int tile_slots = (p_stride + kKeyTile - 1) / kKeyTile;
  const size_t block_csmem = (static_cast<size_t>(kCombineTokens) * (p_stride + 2 * tile_slots + 1)) * sizeof(float) + 16 +
                             static_cast<size_t>(kBlockStages) * kValueTile * hd * sizeof(uint16_t) +
                             kBlockStages * sizeof(uint64_t);
  if (S >= 4 && cache_stride == 0 && hd == 256 && block_csmem <= 200 * 1024) {
    if (cudaError_t e = opt_in_shared_memory(reinterpret_cast<const void *>(attn_combine_block_kernel), 200 * 1024); e != cudaSuccess)
      return e;
    dim3 bgrid(nh, static_cast<unsigned>((S + kCombineTokens - 1) / kCombineTokens));
    launch_chained(attn_combine_block_kernel, dim3(bgrid), dim3(hd / 2 + 32), block_csmem, stream, scores, cache, qg, position_dev,
                   S, nh, nkv, hd, cap, score_stride, p_stride, out, q_out, s_out);
  } else {
    dim3 cgrid(nh, static_cast<unsigned>(S));
    launch_chained(attn_combine_kernel, dim3(cgrid), dim3((hd + 31) / 32 * 32), csmem, stream, scores, cache, qg, position_dev, nh,
                   nkv, hd, cap, score_stride, out, q_out, s_out, cache_stride);
  }
  return cudaGetLastError();
}

} // namespace llmcp_b200
