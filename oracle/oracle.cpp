// CPU oracle for the llmcp Q8_0 operator set (TEST INFRASTRUCTURE ONLY).
//
// This file restates, in plain C++ loops, the arithmetic that the llmcp
// reference encodes in its MLIR emitters.  It exists to CHECK the CUDA path:
// only tests, the smoke check and the CPU-baseline leg of the benchmark may
// load it.  The CUDA library never links or calls anything in here.
//
// Parity status: the reference's kernels exist only as MLIR emitters that need
// an MLIR/LLVM 20 toolchain, so the reference itself cannot be executed next to
// this file.  The restatement is pinned instead by (1) the reference's own
// known-answer construction for the packed Q8 matmul (power-of-two block
// scales; tests/numeric/run_numeric.py:691-732), (2) its Python packers
// q8_0_blocks / q8_0_p4_bytes imported from the reference, and (3) the
// closed-form per-op formulas of tests/numeric/run_numeric.py:734-1110.
// Whole-model outputs on random-init weights have no reference pin.
//
// Conventions
//   * bf(x)  : f32 -> bf16 round-to-nearest-even -> f32 (arith.truncf).
//   * every f32 operation is a separate IEEE operation unless "fma" is
//     written; the file must be compiled with -ffp-contract=off.
//   * loops run in the order written; OpenMP is used only over loops the
//     reference marks parallel (independent output elements).
//   * exp/log: the reference calls libm expf/logf (math.exp / math.log1p ->
//     log(1+x) through convert-math-to-llvm).  libm results are not
//     bit-defined across platforms, so the oracle defines them as the f32
//     rounding of the double-precision function, which is the correctly
//     rounded f32 result in all but ~1e-8 of cases and can be reproduced on
//     the GPU bit for bit.
//   * rsqrt(x) = 1.0f / sqrtf(x)  (MLIR convert-math-to-llvm lowering).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#if defined(_OPENMP)
#include <omp.h>
#endif

namespace {

constexpr int64_t kBlock = 32;       // Q8PackedLayout.h:21
constexpr int64_t kLanes = 4;        // Q8PackedLayout.h:18
constexpr int64_t kRecordBytes = 136; // Q8PackedLayout.h:24-35 (8 + 128)

inline float bf16_to_f32(uint16_t v) {
  uint32_t bits = static_cast<uint32_t>(v) << 16;
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

inline uint16_t f32_to_bf16(float f) {
  uint32_t bits;
  std::memcpy(&bits, &f, 4);
  if ((bits & 0x7fffffffu) > 0x7f800000u)
    return static_cast<uint16_t>((bits >> 16) | 0x40); // quiet NaN
  uint32_t lsb = (bits >> 16) & 1u;
  bits += 0x7fffu + lsb;
  return static_cast<uint16_t>(bits >> 16);
}

inline float bf(float f) { return bf16_to_f32(f32_to_bf16(f)); }

inline float f16_to_f32(uint16_t v) {
  _Float16 h;
  std::memcpy(&h, &v, 2);
  return static_cast<float>(h);
}

inline uint16_t f32_to_f16(float f) {
  _Float16 h = static_cast<_Float16>(f); // round-to-nearest-even
  uint16_t v;
  std::memcpy(&v, &h, 2);
  return v;
}

inline float o_exp(float x) { return static_cast<float>(std::exp(static_cast<double>(x))); }
inline float o_log(float x) { return static_cast<float>(std::log(static_cast<double>(x))); }
inline float o_rsqrt(float x) { return 1.0f / std::sqrt(x); }
inline float o_sigmoid(float v) { return 1.0f / (1.0f + o_exp(-v)); }

// MatmulLoweringCommon.cpp:78-103
inline float apply_activation(float v, int activation) {
  switch (activation) {
  case 1: // silu: v * (1 / (1 + exp(-v)))
    return v * o_sigmoid(v);
  case 2: // sigmoid
    return o_sigmoid(v);
  case 3: // softplus: log(1 + exp(v))
    return o_log(1.0f + o_exp(v));
  default:
    return v;
  }
}

inline float load_act(const void *x, int is_bf16, int64_t index) {
  if (is_bf16)
    return bf16_to_f32(static_cast<const uint16_t *>(x)[index]);
  return static_cast<const float *>(x)[index];
}

// lib/Model/Quantization.cpp:92-116 (offline weight quantisation)
void quantize_row_q8_0(const float *values, int64_t cols, uint16_t *d,
                       int8_t *qs) {
  for (int64_t b = 0; b < cols / kBlock; ++b) {
    const float *v = values + b * kBlock;
    float amax = 0.0f;
    for (int64_t i = 0; i < kBlock; ++i)
      amax = std::max(amax, std::fabs(v[i]));
    if (amax == 0.0f) {
      d[b] = 0;
      std::memset(qs + b * kBlock, 0, kBlock);
      continue;
    }
    float scale = amax / 127.0f;
    d[b] = f32_to_f16(scale);
    for (int64_t i = 0; i < kBlock; ++i) {
      long q = std::lround(v[i] / scale);
      q = std::min(127L, std::max(-127L, q));
      qs[b * kBlock + i] = static_cast<int8_t>(q);
    }
  }
}

// Address of byte (row, col) inside a packed tensor.
// lib/Model/Quantization.cpp:184-211, LowerToLinalg.cpp:470-509
inline const uint8_t *record_of(const uint8_t *w, int64_t blocks, int64_t row,
                                int64_t block) {
  return w + ((row / kLanes) * blocks + block) * kRecordBytes;
}

inline int8_t packed_q(const uint8_t *w, int64_t blocks, int64_t row,
                       int64_t col) {
  const uint8_t *rec = record_of(w, blocks, row, col / kBlock);
  int64_t within = col % kBlock;
  return static_cast<int8_t>(
      rec[8 + (within / 4) * 16 + (row % kLanes) * 4 + (within % 4)]);
}

inline uint16_t packed_d(const uint8_t *w, int64_t blocks, int64_t row,
                         int64_t block) {
  const uint8_t *rec = record_of(w, blocks, row, block);
  int64_t lane = row % kLanes;
  return static_cast<uint16_t>(rec[lane * 2] | (rec[lane * 2 + 1] << 8));
}

// Q8Decode.cpp:83-120, Q8Matmul.cpp:93-141, Q8Scalar.cpp:84-124
void act_quant_row(const void *x, int is_bf16, int64_t base, int64_t K,
                   int8_t *q, float *s) {
  for (int64_t b = 0; b < K / kBlock; ++b) {
    float v[kBlock];
    float amax = 0.0f;
    for (int64_t i = 0; i < kBlock; ++i) {
      v[i] = load_act(x, is_bf16, base + b * kBlock + i);
      amax = std::fmax(amax, std::fabs(v[i]));
    }
    float scale = amax / 127.0f;
    s[b] = scale;
    float inv = amax == 0.0f ? 0.0f : 1.0f / scale;
    for (int64_t i = 0; i < kBlock; ++i) {
      float r = __builtin_roundevenf(v[i] * inv);
      q[b * kBlock + i] = static_cast<int8_t>(static_cast<int32_t>(r));
    }
  }
}

// A packed tensor expanded to row-major int8 plus f32 scales.  The integers
// and scale values are unchanged; only the arrangement differs, so that the
// inner product loops vectorise.
struct Unpacked {
  int64_t N = 0, K = 0;
  std::vector<int8_t> q;
  std::vector<float> d;
  const uint16_t *bf = nullptr; // a bf16 [N][K] matrix of an unquantised arena (mode 2): nothing to unpack
};

void unpack(const uint8_t *w, int64_t N, int64_t K, Unpacked &out) {
  out.N = N;
  out.K = K;
  const int64_t blocks = K / kBlock;
  out.q.resize(static_cast<size_t>(N * K));
  out.d.resize(static_cast<size_t>(N * blocks));
#pragma omp parallel for schedule(static)
  for (int64_t g = 0; g < N / kLanes; ++g) {
    for (int64_t b = 0; b < blocks; ++b) {
      const uint8_t *rec = w + (g * blocks + b) * kRecordBytes;
      for (int64_t lane = 0; lane < kLanes; ++lane) {
        int64_t row = g * kLanes + lane;
        uint16_t bits = static_cast<uint16_t>(rec[lane * 2] | (rec[lane * 2 + 1] << 8));
        out.d[row * blocks + b] = f16_to_f32(bits);
        int8_t *dst = out.q.data() + row * K + b * kBlock;
        for (int64_t c = 0; c < 8; ++c)
          std::memcpy(dst + c * 4, rec + 8 + c * 16 + lane * 4, 4);
      }
    }
  }
}

inline int32_t block_dot(const int8_t *a, const int8_t *w) {
  int32_t dot = 0;
  for (int64_t i = 0; i < kBlock; ++i)
    dot += static_cast<int32_t>(a[i]) * static_cast<int32_t>(w[i]);
  return dot;
}

// Q8Decode.cpp:131-225 / Q8Matmul.cpp:143-289 (mode 0, fused multiply-add)
// Q8Scalar.cpp:65-212 (mode 1, multiply then add)
// The bf16 linear of an unquantised arena, portable lowering
// (MatmulLoweringCommon.cpp:186-251): per 32-wide tile of K the f32 products are
// added in lane order starting from zero (an ordered vector reduction), and the
// tile's sum is added to the running f32 sum; activation, then the output type.
// pairs != 0: the order of the aarch64 lowering instead (MatmulLoweringCommon.cpp:253-322): four f32
// lanes, lane j of every 8-wide block receives the sum of the products 2j and 2j+1 (one rounding,
// as the two-way bf16 dot instruction forms it), and the lanes are added in order at the end.
void linear_bf16(const void *x, int x_bf16, int64_t M, int64_t K,
                 const uint16_t *w, int64_t N, void *y, int y_bf16,
                 int activation, int pairs = 0) {
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n) {
    const uint16_t *row = w + n * K;
    for (int64_t m = 0; m < M; ++m) {
      float acc = 0.0f;
      if (pairs) {
        float lanes[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int64_t k0 = 0; k0 < K; k0 += 8)
          for (int64_t j = 0; j < 4; ++j) {
            const double p0 = static_cast<double>(load_act(x, x_bf16, m * K + k0 + 2 * j)) * bf16_to_f32(row[k0 + 2 * j]);
            const double p1 = static_cast<double>(load_act(x, x_bf16, m * K + k0 + 2 * j + 1)) * bf16_to_f32(row[k0 + 2 * j + 1]);
            lanes[j] = lanes[j] + static_cast<float>(p0 + p1);
          }
        for (int64_t j = 0; j < 4; ++j)
          acc = acc + lanes[j];
      }
      for (int64_t k0 = 0; k0 < K && !pairs; k0 += kBlock) {
        float dot = 0.0f;
        for (int64_t i = 0; i < kBlock; ++i)
          dot = dot + load_act(x, x_bf16, m * K + k0 + i) * bf16_to_f32(row[k0 + i]);
        acc = acc + dot;
      }
      float v = apply_activation(acc, activation);
      if (y_bf16)
        static_cast<uint16_t *>(y)[m * N + n] = f32_to_bf16(v);
      else
        static_cast<float *>(y)[m * N + n] = v;
    }
  }
}

void linear_unpacked(const void *x, int x_bf16, int64_t M, int64_t K,
                     const Unpacked &w, void *y, int y_bf16, int activation,
                     int mode) {
  if (w.bf) {
    linear_bf16(x, x_bf16, M, K, w.bf, w.N, y, y_bf16, activation, mode == 3);
    return;
  }
  const int64_t N = w.N, blocks = K / kBlock;
  std::vector<int8_t> aq(static_cast<size_t>(M * K));
  std::vector<float> as(static_cast<size_t>(M * blocks));
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    act_quant_row(x, x_bf16, m * K, K, aq.data() + m * K, as.data() + m * blocks);
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n) {
    const int8_t *wq = w.q.data() + n * K;
    const float *wd = w.d.data() + n * blocks;
    for (int64_t m = 0; m < M; ++m) {
      const int8_t *a = aq.data() + m * K;
      const float *sa = as.data() + m * blocks;
      float acc = 0.0f;
      for (int64_t b = 0; b < blocks; ++b) {
        int32_t dot = block_dot(a + b * kBlock, wq + b * kBlock);
        float factor = sa[b] * wd[b];
        if (mode == 0)
          acc = std::fmaf(static_cast<float>(dot), factor, acc);
        else
          acc = acc + static_cast<float>(dot) * factor;
      }
      float v = apply_activation(acc, activation);
      if (y_bf16)
        static_cast<uint16_t *>(y)[m * N + n] = f32_to_bf16(v);
      else
        static_cast<float *>(y)[m * N + n] = v;
    }
  }
}

// LowerToLinalg.cpp:211-308, DecodeNormalization.cpp:70-145
void rms_norm_rows(const uint16_t *x, int64_t M, int64_t H, const void *w,
                   int w_bf16, float eps, int zero_centered, uint16_t *y) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    const uint16_t *row = x + m * H;
    float sum = 0.0f;
    for (int64_t d = 0; d < H; ++d) {
      float v = bf16_to_f32(row[d]);
      float sq = v * v;
      sum = sum + sq;
    }
    float mean = sum / static_cast<float>(H);
    float rstd = o_rsqrt(mean + eps);
    for (int64_t d = 0; d < H; ++d) {
      float v = bf16_to_f32(row[d]);
      float wt = load_act(w, w_bf16, d);
      if (zero_centered)
        wt = wt + 1.0f;
      float t = v * rstd;
      y[m * H + d] = f32_to_bf16(t * wt);
    }
  }
}

// LowerToLinalg.cpp:574-727, DecodeNormalization.cpp:96-131
void gated_rms_norm_rows(const uint16_t *x, const uint16_t *gate, const void *w,
                         int w_bf16, int64_t M, int64_t H, int64_t group,
                         float eps, int gate_activated, uint16_t *y) {
  const int64_t groups = H / group;
#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t g = 0; g < groups; ++g) {
      const int64_t base = m * H + g * group;
      float sum = 0.0f;
      for (int64_t d = 0; d < group; ++d) {
        float v = bf16_to_f32(x[base + d]);
        float sq = v * v;
        sum = sum + sq;
      }
      float mean = sum / static_cast<float>(group);
      float rstd = o_rsqrt(mean + eps);
      for (int64_t d = 0; d < group; ++d) {
        float v = bf16_to_f32(x[base + d]);
        float gv = bf16_to_f32(gate[base + d]);
        float silu = gate_activated ? gv : gv * o_sigmoid(gv);
        float wt = load_act(w, w_bf16, d);
        float t = v * silu;
        t = t * wt;
        t = t * rstd;
        y[base + d] = f32_to_bf16(t);
      }
    }
  }
}

// LowerCausalConv1d.cpp:74-182
void causal_conv1d_rows(const uint16_t *x, const uint16_t *w, uint16_t *state,
                        int64_t S, int64_t C, int64_t kernel, uint16_t *y) {
  const int64_t state_len = kernel - 1;
#pragma omp parallel for schedule(static)
  for (int64_t t = 0; t < S; ++t) {
    for (int64_t c = 0; c < C; ++c) {
      float acc = 0.0f;
      for (int64_t k = 0; k < kernel; ++k) {
        int64_t src = t + k - state_len;
        uint16_t raw = src < 0 ? state[(src + state_len) * C + c] : x[src * C + c];
        float prod = bf16_to_f32(raw) * bf16_to_f32(w[c * kernel + k]);
        acc = acc + prod;
      }
      float silu = acc * o_sigmoid(acc);
      y[t * C + c] = f32_to_bf16(silu);
    }
  }
  for (int64_t s = 0; s < state_len; ++s) {
    int64_t src = S - state_len + s;
    for (int64_t c = 0; c < C; ++c)
      state[s * C + c] = src < 0 ? state[(src + state_len) * C + c] : x[src * C + c];
  }
}

// LowerGatedDeltaNet.cpp:129-445
void gated_delta_net_rows(const uint16_t *conv, const uint16_t *a,
                          const uint16_t *b, const float *a_log,
                          const uint16_t *dt_bias, float *state, int64_t S,
                          int64_t nk, int64_t nv, int64_t dk, int64_t dv,
                          int b_activated, uint16_t *out) {
  const int64_t ratio = nv / nk;
  const int64_t q_dim = nk * dk;
  const int64_t channels = 2 * q_dim + nv * dv;
  const float q_scale = static_cast<float>(1.0 / std::sqrt(static_cast<double>(dk)));
  for (int64_t t = 0; t < S; ++t) {
    const uint16_t *row = conv + t * channels;
#pragma omp parallel for schedule(static)
    for (int64_t h = 0; h < nv; ++h) {
      const int64_t kh = h / ratio;
      const uint16_t *qp = row + kh * dk;
      const uint16_t *kp = row + q_dim + kh * dk;
      const uint16_t *vp = row + 2 * q_dim + h * dv;
      float q_sum = 0.0f, k_sum = 0.0f;
      for (int64_t i = 0; i < dk; ++i) {
        float v = bf16_to_f32(qp[i]);
        float sq = v * v;
        q_sum = q_sum + sq;
      }
      float q_norm_scale = o_rsqrt(q_sum + 1.0e-6f) * q_scale;
      for (int64_t i = 0; i < dk; ++i) {
        float v = bf16_to_f32(kp[i]);
        float sq = v * v;
        k_sum = k_sum + sq;
      }
      float k_inv = o_rsqrt(k_sum + 1.0e-6f);
      std::vector<float> qn(dk), kn(dk);
      for (int64_t i = 0; i < dk; ++i) {
        qn[i] = bf16_to_f32(qp[i]) * q_norm_scale;
        kn[i] = bf16_to_f32(kp[i]) * k_inv;
      }
      float b_value = bf16_to_f32(b[t * nv + h]);
      float beta = b_activated ? b_value : o_sigmoid(b_value);
      float a_plus_dt = bf16_to_f32(a[t * nv + h]) + bf16_to_f32(dt_bias[h]);
      float softplus = o_log(1.0f + o_exp(a_plus_dt));
      float g = (-o_exp(a_log[h])) * softplus;
      float decay = o_exp(g);
      float *s = state + h * dk * dv;
      for (int64_t v = 0; v < dv; ++v) {
        float kv = 0.0f;
        for (int64_t k = 0; k < dk; ++k) {
          float decayed = s[k * dv + v] * decay;
          float prod = decayed * kn[k];
          kv = kv + prod;
        }
        float delta = (bf16_to_f32(vp[v]) - kv) * beta;
        float o = 0.0f;
        for (int64_t k = 0; k < dk; ++k) {
          float decayed = s[k * dv + v] * decay;
          float update = kn[k] * delta;
          float updated = decayed + update;
          s[k * dv + v] = updated;
          float prod = updated * qn[k];
          o = o + prod;
        }
        out[t * nv * dv + h * dv + v] = f32_to_bf16(o);
      }
    }
  }
}

// LowerAttention.cpp:160-601.  `cache` is one layer: [2, nkv, cap, hd] bf16.
void attention_rows(const uint16_t *qg, const uint16_t *k, const uint16_t *v,
                    const uint16_t *q_norm, const uint16_t *k_norm,
                    const float *cos, const float *sin, uint16_t *cache,
                    int64_t position, int64_t S, int64_t nh, int64_t nkv,
                    int64_t hd, int64_t rot, int64_t cap, uint16_t *out) {
  const int64_t group = nh / nkv;
  const int64_t half = rot / 2;
  const float scale = 1.0f / std::sqrt(static_cast<float>(hd));
  const float inv_hd = 1.0f / static_cast<float>(hd);
  std::vector<uint16_t> qn(static_cast<size_t>(S * nh * hd));

  auto norm_rope = [&](const uint16_t *src, const uint16_t *weight, int64_t t,
                       uint16_t *dst) {
    float sum = 0.0f;
    for (int64_t d = 0; d < hd; ++d) {
      float x = bf16_to_f32(src[d]);
      float sq = x * x;
      sum = sum + sq;
    }
    float inv = o_rsqrt(sum * inv_hd + 1.0e-6f);
    std::vector<float> tmp(hd);
    for (int64_t d = 0; d < hd; ++d) {
      float x = bf16_to_f32(src[d]);
      float centered = 1.0f + bf16_to_f32(weight[d]);
      float n = x * inv;
      tmp[d] = n * centered;
    }
    for (int64_t d = 0; d < rot; ++d) {
      bool second = d >= half;
      int64_t partner = second ? d - half : d + half;
      float sign = second ? 1.0f : -1.0f;
      float rotated = sign * tmp[partner];
      float lhs = tmp[d] * cos[t * rot + d];
      float rhs = rotated * sin[t * rot + d];
      dst[d] = f32_to_bf16(lhs + rhs);
    }
    for (int64_t d = rot; d < hd; ++d)
      dst[d] = f32_to_bf16(tmp[d]);
  };

#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t t = 0; t < S; ++t)
    for (int64_t h = 0; h < nh; ++h)
      norm_rope(qg + t * nh * 2 * hd + h * 2 * hd, q_norm, t,
                qn.data() + (t * nh + h) * hd);

#pragma omp parallel for schedule(static) collapse(2)
  for (int64_t t = 0; t < S; ++t)
    for (int64_t kh = 0; kh < nkv; ++kh) {
      norm_rope(k + t * nkv * hd + kh * hd, k_norm, t,
                cache + ((0 * nkv + kh) * cap + position + t) * hd);
      std::memcpy(cache + ((1 * nkv + kh) * cap + position + t) * hd,
                  v + t * nkv * hd + kh * hd, static_cast<size_t>(hd) * 2);
    }

#pragma omp parallel for schedule(dynamic, 1) collapse(2)
  for (int64_t t = 0; t < S; ++t) {
    for (int64_t h = 0; h < nh; ++h) {
      const int64_t kh = h / group;
      const int64_t query_end = position + t + 1;
      const uint16_t *q = qn.data() + (t * nh + h) * hd;
      const uint16_t *kc = cache + (0 * nkv + kh) * cap * hd;
      const uint16_t *vc = cache + (1 * nkv + kh) * cap * hd;
      std::vector<float> acc(hd, 0.0f);
      float scores[64];
      float running_max = -1.0e30f;
      float running_sum = 0.0f;
      for (int64_t start = 0; start < query_end; start += 64) {
        int64_t end = std::min<int64_t>(start + 64, query_end);
        float tile_max = -1.0e30f;
        for (int64_t j = start; j < end; ++j) {
          float dot = 0.0f;
          for (int64_t d = 0; d < hd; ++d) {
            float prod = bf16_to_f32(q[d]) * bf16_to_f32(kc[j * hd + d]);
            dot = dot + prod;
          }
          float score = dot * scale;
          scores[j - start] = score;
          tile_max = std::fmax(tile_max, score);
        }
        float new_max = std::fmax(running_max, tile_max);
        float correction = o_exp(running_max - new_max);
        for (int64_t d = 0; d < hd; ++d)
          acc[d] = acc[d] * correction;
        float sum = running_sum * correction;
        for (int64_t j = start; j < end; ++j) {
          float p = o_exp(scores[j - start] - new_max);
          sum = sum + p;
          for (int64_t d = 0; d < hd; ++d) {
            float prod = p * bf16_to_f32(vc[j * hd + d]);
            acc[d] = acc[d] + prod;
          }
        }
        running_max = new_max;
        running_sum = sum;
      }
      const uint16_t *gate = qg + t * nh * 2 * hd + h * 2 * hd + hd;
      for (int64_t d = 0; d < hd; ++d) {
        float normalized = acc[d] / running_sum;
        float gated = normalized * o_sigmoid(bf16_to_f32(gate[d]));
        out[t * nh * hd + h * hd + d] = f32_to_bf16(gated);
      }
    }
  }
}

} // namespace

extern "C" {

// ---- scalar helpers exposed for tests ------------------------------------
uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
float orc_bf16_to_f32(uint16_t v) { return bf16_to_f32(v); }
uint16_t orc_f32_to_f16(float f) { return f32_to_f16(f); }
float orc_f16_to_f32(uint16_t v) { return f16_to_f32(v); }
float orc_exp(float x) { return o_exp(x); }

int orc_num_threads() {
#if defined(_OPENMP)
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// Number of OpenMP threads of the following calls, whatever OMP_NUM_THREADS said when the
// process started (launchers such as torchrun export OMP_NUM_THREADS=1).  Returns the new count.
int orc_set_num_threads(int threads) {
#if defined(_OPENMP)
  if (threads > 0) {
    omp_set_dynamic(0);
    omp_set_num_threads(threads);
  }
  return omp_get_max_threads();
#else
  (void)threads;
  return 1;
#endif
}

// ---- a1: weight quantisation and packing ----------------------------------
// lib/Model/Quantization.cpp:92-116.  d: [cols/32] f16 bits, qs: [cols].
void orc_quantize_row_q8_0(const float *values, int64_t cols, uint16_t *d,
                           int8_t *qs) {
  quantize_row_q8_0(values, cols, d, qs);
}

// lib/Model/Quantization.cpp:165-214.  src is [rows, cols] f32 or bf16;
// dst receives rows/4 * cols/32 records of 136 bytes.  Returns 0 on success.
int orc_pack_q8_0_p4(const void *src, int src_bf16, int64_t rows, int64_t cols,
                     uint8_t *dst) {
  if (rows <= 0 || cols <= 0 || rows % 8 != 0 || cols % kBlock != 0)
    return 1; // Q8PackedLayout.h:38-42
  const int64_t blocks = cols / kBlock;
#pragma omp parallel for schedule(static)
  for (int64_t g = 0; g < rows / kLanes; ++g) {
    std::vector<float> values(cols);
    std::vector<uint16_t> d(kLanes * blocks);
    std::vector<int8_t> qs(kLanes * cols);
    for (int64_t lane = 0; lane < kLanes; ++lane) {
      int64_t row = g * kLanes + lane;
      for (int64_t c = 0; c < cols; ++c)
        values[c] = load_act(src, src_bf16, row * cols + c);
      quantize_row_q8_0(values.data(), cols, d.data() + lane * blocks,
                        qs.data() + lane * cols);
    }
    for (int64_t b = 0; b < blocks; ++b) {
      uint8_t *rec = dst + (g * blocks + b) * kRecordBytes;
      for (int64_t lane = 0; lane < kLanes; ++lane)
        std::memcpy(rec + lane * 2, &d[lane * blocks + b], 2);
      for (int64_t c = 0; c < 8; ++c)
        for (int64_t lane = 0; lane < kLanes; ++lane)
          std::memcpy(rec + 8 + c * 16 + lane * 4,
                      qs.data() + lane * cols + b * kBlock + c * 4, 4);
    }
  }
  return 0;
}

// Reads back one element of a packed tensor: integer and f16 scale bits.
void orc_packed_element(const uint8_t *w, int64_t cols, int64_t row,
                        int64_t col, int8_t *q, uint16_t *d) {
  *q = packed_q(w, cols / kBlock, row, col);
  *d = packed_d(w, cols / kBlock, row, col / kBlock);
}

// ---- a2: activation quantisation -------------------------------------------
void orc_act_quant(const void *x, int x_bf16, int64_t M, int64_t K, int8_t *q,
                   float *s) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    act_quant_row(x, x_bf16, m * K, K, q + m * K, s + m * (K / kBlock));
}

// ---- a3/a4: int32 block dots and the Q8 linear -----------------------------
// dots: [M, N, K/32] int32.
void orc_block_dots(const int8_t *aq, int64_t M, int64_t K, const uint8_t *w,
                    int64_t N, int32_t *dots) {
  Unpacked u;
  unpack(w, N, K, u);
  const int64_t blocks = K / kBlock;
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < N; ++n)
    for (int64_t m = 0; m < M; ++m)
      for (int64_t b = 0; b < blocks; ++b)
        dots[(m * N + n) * blocks + b] =
            block_dot(aq + m * K + b * kBlock, u.q.data() + n * K + b * kBlock);
}

// activation: 0 none, 1 silu, 2 sigmoid, 3 softplus.
// mode: 0 = fma accumulate (SDOT paths), 1 = mul then add (scalar fallback).
void orc_linear_q8(const void *x, int x_bf16, int64_t M, int64_t K,
                   const uint8_t *w, int64_t N, void *y, int y_bf16,
                   int activation, int mode) {
  Unpacked u;
  unpack(w, N, K, u);
  linear_unpacked(x, x_bf16, M, K, u, y, y_bf16, activation, mode);
}

// Direct evaluation over the packed bytes, one scalar dot per element, exactly
// as Q8Scalar.cpp walks the records (no unpacking).  Used to validate unpack().
void orc_linear_q8_direct(const void *x, int x_bf16, int64_t M, int64_t K,
                          const uint8_t *w, int64_t N, void *y, int y_bf16,
                          int activation, int mode) {
  const int64_t blocks = K / kBlock;
  std::vector<int8_t> aq(static_cast<size_t>(M * K));
  std::vector<float> as(static_cast<size_t>(M * blocks));
  for (int64_t m = 0; m < M; ++m)
    act_quant_row(x, x_bf16, m * K, K, aq.data() + m * K, as.data() + m * blocks);
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    for (int64_t n = 0; n < N; ++n) {
      float acc = 0.0f;
      for (int64_t b = 0; b < blocks; ++b) {
        int32_t dot = 0;
        for (int64_t e = 0; e < kBlock; ++e)
          dot += static_cast<int32_t>(aq[m * K + b * kBlock + e]) *
                 static_cast<int32_t>(packed_q(w, blocks, n, b * kBlock + e));
        float factor = as[m * blocks + b] * f16_to_f32(packed_d(w, blocks, n, b));
        if (mode == 0)
          acc = std::fmaf(static_cast<float>(dot), factor, acc);
        else
          acc = acc + static_cast<float>(dot) * factor;
      }
      float v = apply_activation(acc, activation);
      if (y_bf16)
        static_cast<uint16_t *>(y)[m * N + n] = f32_to_bf16(v);
      else
        static_cast<float *>(y)[m * N + n] = v;
    }
  }
}

// bf16 weights [N][K] (an unquantised arena), portable lowering.
void orc_linear_bf16(const void *x, int x_bf16, int64_t M, int64_t K,
                     const uint16_t *w, int64_t N, void *y, int y_bf16,
                     int activation) {
  linear_bf16(x, x_bf16, M, K, w, N, y, y_bf16, activation);
}

// ---- a6: embedding gather ---------------------------------------------------
// LowerToLinalg.cpp:435-531
void orc_embedding_q8(const int64_t *tokens, int64_t S, const uint8_t *table,
                      int64_t hidden, uint16_t *out) {
  const int64_t blocks = hidden / kBlock;
#pragma omp parallel for schedule(static)
  for (int64_t r = 0; r < S; ++r) {
    const int64_t token = tokens[r];
    for (int64_t c = 0; c < hidden; ++c) {
      float scale = f16_to_f32(packed_d(table, blocks, token, c / kBlock));
      float value = static_cast<float>(packed_q(table, blocks, token, c)) * scale;
      out[r * hidden + c] = f32_to_bf16(value);
    }
  }
}

// ---- a7..a9: norms and pointwise -------------------------------------------
void orc_rms_norm(const uint16_t *x, int64_t M, int64_t H, const void *w,
                  int w_bf16, float eps, int zero_centered, uint16_t *y) {
  rms_norm_rows(x, M, H, w, w_bf16, eps, zero_centered, y);
}

// op: 0 add, 1 mul, 2 silu_mul(a = gate, b = up).  LowerToLinalg.cpp:312-427
void orc_pointwise(const uint16_t *a, const uint16_t *b, int64_t count, int op,
                   uint16_t *y) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < count; ++i) {
    float x = bf16_to_f32(a[i]), z = bf16_to_f32(b[i]);
    float r;
    if (op == 0)
      r = x + z;
    else if (op == 1)
      r = x * z;
    else {
      float silu = x * o_sigmoid(x);
      r = silu * z;
    }
    y[i] = f32_to_bf16(r);
  }
}

void orc_gated_rms_norm(const uint16_t *x, const uint16_t *gate, const void *w,
                        int w_bf16, int64_t M, int64_t H, int64_t group,
                        float eps, int gate_activated, uint16_t *y) {
  gated_rms_norm_rows(x, gate, w, w_bf16, M, H, group, eps, gate_activated, y);
}

// ---- a10..a12: conv, recurrence, attention ---------------------------------
void orc_causal_conv1d(const uint16_t *x, const uint16_t *w, uint16_t *state,
                       int64_t S, int64_t C, int64_t kernel, uint16_t *y) {
  causal_conv1d_rows(x, w, state, S, C, kernel, y);
}

void orc_gated_delta_net(const uint16_t *conv, const uint16_t *a,
                         const uint16_t *b, const float *a_log,
                         const uint16_t *dt_bias, float *state, int64_t S,
                         int64_t nk, int64_t nv, int64_t dk, int64_t dv,
                         int b_activated, uint16_t *out) {
  gated_delta_net_rows(conv, a, b, a_log, dt_bias, state, S, nk, nv, dk, dv,
                       b_activated, out);
}

void orc_attention(const uint16_t *qg, const uint16_t *k, const uint16_t *v,
                   const uint16_t *q_norm, const uint16_t *k_norm,
                   const float *cos, const float *sin, uint16_t *cache,
                   int64_t position, int64_t S, int64_t nh, int64_t nkv,
                   int64_t hd, int64_t rot, int64_t cap, uint16_t *out) {
  attention_rows(qg, k, v, q_norm, k_norm, cos, sin, cache, position, S, nh,
                 nkv, hd, rot, cap, out);
}

// ---- a13/a14: host helpers and the whole model -------------------------------
// lib/Runtime/AotRuntime.cpp:22-32
void orc_make_cos_sin(int64_t pos, int64_t rotary, float theta, float *cos,
                      float *sin) {
  for (int64_t d = 0; d < rotary / 2; ++d) {
    float inv_freq = 1.0f / std::pow(theta, static_cast<float>(2 * d) /
                                                static_cast<float>(rotary));
    float angle = static_cast<float>(pos) * inv_freq;
    cos[d] = cos[d + rotary / 2] = std::cos(angle);
    sin[d] = sin[d + rotary / 2] = std::sin(angle);
  }
}

// tools/llmcp-benchmark/llmcp-benchmark.cpp:51-54 (first maximum)
int64_t orc_argmax(const float *values, int64_t count) {
  return std::max_element(values, values + count) - values;
}

struct OrcModelConfig {
  int64_t hidden, intermediate, vocab, layers, full_interval;
  int64_t heads, kv_heads, head_dim, rotary;
  int64_t lin_k_heads, lin_v_heads, lin_k_dim, lin_v_dim, conv_kernel;
  float eps;
  int32_t mode; // accumulate mode of the linears
};

// Offsets (bytes from the arena base) of one layer's tensors, in a fixed
// order; unused entries are 0.  dtype flags say whether a small tensor is
// stored as bf16 (1) or f32 (0).
struct OrcLayer {
  uint64_t input_norm, post_norm;
  uint64_t qkv, z, a, b, conv, dt_bias, a_log, lin_norm, out_proj; // linear
  uint64_t q_proj, k_proj, v_proj, o_proj, q_norm, k_norm;         // full
  uint64_t gate, up, down;
  int32_t lin_norm_bf16, dt_bias_bf16, a_log_bf16, pad;
};

struct OrcModel {
  OrcModelConfig cfg;
  const uint8_t *arena;
  uint64_t embed, final_norm;
  std::vector<OrcLayer> layers;
  std::vector<Unpacked> cache; // unpacked weights, filled lazily
  Unpacked embed_unpacked;
  bool embed_ready = false;
};

void *orc_model_create(const OrcModelConfig *cfg, const uint8_t *arena,
                       uint64_t embed, uint64_t final_norm,
                       const OrcLayer *layers) {
  auto *m = new OrcModel();
  m->cfg = *cfg;
  m->arena = arena;
  m->embed = embed;
  m->final_norm = final_norm;
  m->layers.assign(layers, layers + cfg->layers);
  m->cache.resize(static_cast<size_t>(cfg->layers) * 16);
  return m;
}

void orc_model_destroy(void *handle) { delete static_cast<OrcModel *>(handle); }

} // extern "C"

namespace {

const Unpacked &weight(OrcModel &m, int64_t layer, int slot, uint64_t offset,
                       int64_t N, int64_t K) {
  Unpacked &u = m.cache[static_cast<size_t>(layer * 16 + slot)];
  if (u.N == 0) {
    if (m.cfg.mode >= 2) { // unquantised arena: bf16 [N][K] in place
      u.N = N;
      u.K = K;
      u.bf = reinterpret_cast<const uint16_t *>(m.arena + offset);
    } else {
      unpack(m.arena + offset, N, K, u);
    }
  }
  return u;
}

void pointwise(const uint16_t *a, const uint16_t *b, int64_t count, int op,
               uint16_t *y) {
  orc_pointwise(a, b, count, op, y);
}

// lib/Model/ModelBuilder.cpp:203-216 after FuseLinearActivations.cpp:27-43
void mlp(OrcModel &m, int64_t layer, const OrcLayer &L, const uint16_t *x,
         int64_t S, uint16_t *out) {
  const auto &c = m.cfg;
  std::vector<uint16_t> gate(S * c.intermediate), up(S * c.intermediate),
      act(S * c.intermediate);
  linear_unpacked(x, 1, S, c.hidden,
                  weight(m, layer, 0, L.gate, c.intermediate, c.hidden),
                  gate.data(), 1, /*silu*/ 1, c.mode);
  linear_unpacked(x, 1, S, c.hidden,
                  weight(m, layer, 1, L.up, c.intermediate, c.hidden), up.data(),
                  1, 0, c.mode);
  pointwise(gate.data(), up.data(), S * c.intermediate, 1, act.data());
  linear_unpacked(act.data(), 1, S, c.intermediate,
                  weight(m, layer, 2, L.down, c.hidden, c.intermediate), out, 1,
                  0, c.mode);
}

} // namespace

extern "C" {

// One call of the AOT entry (lib/Model/ModelBuilder.cpp:440-526): embedding,
// all layers, final norm, last row, lm_head.  kv: [full, 2, kv_heads, cap,
// head_dim] bf16; delta: [linear, v_heads, k_dim, v_dim] f32; conv: [linear,
// kernel-1, qkv_dim] bf16; cos/sin: [S, rotary]; logits: [vocab].
// If hidden_out is not null it receives the final-norm output [S, hidden].
void orc_model_forward(void *handle, const int64_t *tokens, int64_t S,
                       const float *cos, const float *sin, int64_t position,
                       uint16_t *kv, int64_t cap, float *delta, uint16_t *conv,
                       float *logits, uint16_t *hidden_out) {
  OrcModel &m = *static_cast<OrcModel *>(handle);
  const auto &c = m.cfg;
  const int64_t H = c.hidden;
  const int64_t qkv_dim = 2 * c.lin_k_heads * c.lin_k_dim + c.lin_v_heads * c.lin_v_dim;
  const int64_t value_dim = c.lin_v_heads * c.lin_v_dim;
  const int64_t q_out = c.heads * c.head_dim * 2;
  const int64_t kv_dim = c.kv_heads * c.head_dim;
  const int64_t attn_dim = c.heads * c.head_dim;

  std::vector<uint16_t> hidden(S * H), norm(S * H), residual(S * H),
      branch(S * H);
  if (c.mode >= 2) { // bf16 table: the rows themselves (LowerToLinalg.cpp:435-531)
    const uint16_t *table = reinterpret_cast<const uint16_t *>(m.arena + m.embed);
    for (int64_t r = 0; r < S; ++r)
      std::memcpy(hidden.data() + r * H, table + tokens[r] * H, static_cast<size_t>(H) * 2);
  } else {
    orc_embedding_q8(tokens, S, m.arena + m.embed, H, hidden.data());
  }

  int64_t linear_index = 0, full_index = 0;
  for (int64_t layer = 0; layer < c.layers; ++layer) {
    const OrcLayer &L = m.layers[layer];
    const bool is_full = (layer % c.full_interval) == c.full_interval - 1;
    rms_norm_rows(hidden.data(), S, H, m.arena + L.input_norm, 1, c.eps, 1,
                  norm.data());
    if (!is_full) {
      // ModelBuilder.cpp:218-276 with the three activation fusions applied.
      std::vector<uint16_t> qkv(S * qkv_dim), z(S * value_dim),
          a(S * c.lin_v_heads), b(S * c.lin_v_heads), convd(S * qkv_dim),
          gdn(S * value_dim), gated(S * value_dim);
      linear_unpacked(norm.data(), 1, S, H, weight(m, layer, 3, L.qkv, qkv_dim, H),
                      qkv.data(), 1, 0, c.mode);
      linear_unpacked(norm.data(), 1, S, H, weight(m, layer, 4, L.z, value_dim, H),
                      z.data(), 1, /*silu*/ 1, c.mode);
      linear_unpacked(norm.data(), 1, S, H,
                      weight(m, layer, 5, L.a, c.lin_v_heads, H), a.data(), 1, 0,
                      c.mode);
      linear_unpacked(norm.data(), 1, S, H,
                      weight(m, layer, 6, L.b, c.lin_v_heads, H), b.data(), 1,
                      /*sigmoid*/ 2, c.mode);
      causal_conv1d_rows(
          qkv.data(), reinterpret_cast<const uint16_t *>(m.arena + L.conv),
          conv + linear_index * (c.conv_kernel - 1) * qkv_dim, S, qkv_dim,
          c.conv_kernel, convd.data());
      // A_log and dt_bias follow the dtypes the lowering assumes (f32, bf16).
      std::vector<float> a_log(c.lin_v_heads);
      std::vector<uint16_t> dt(c.lin_v_heads);
      for (int64_t h = 0; h < c.lin_v_heads; ++h) {
        a_log[h] = load_act(m.arena + L.a_log, L.a_log_bf16, h);
        dt[h] = L.dt_bias_bf16
                    ? reinterpret_cast<const uint16_t *>(m.arena + L.dt_bias)[h]
                    : f32_to_bf16(reinterpret_cast<const float *>(m.arena + L.dt_bias)[h]);
      }
      gated_delta_net_rows(convd.data(), a.data(), b.data(), a_log.data(),
                           dt.data(),
                           delta + linear_index * c.lin_v_heads * c.lin_k_dim * c.lin_v_dim,
                           S, c.lin_k_heads, c.lin_v_heads, c.lin_k_dim,
                           c.lin_v_dim, /*b_activated*/ 1, gdn.data());
      gated_rms_norm_rows(gdn.data(), z.data(), m.arena + L.lin_norm,
                          L.lin_norm_bf16, S, value_dim, c.lin_v_dim, c.eps,
                          /*gate_activated*/ 1, gated.data());
      linear_unpacked(gated.data(), 1, S, value_dim,
                      weight(m, layer, 7, L.out_proj, H, value_dim),
                      branch.data(), 1, 0, c.mode);
      ++linear_index;
    } else {
      // ModelBuilder.cpp:278-319
      std::vector<uint16_t> qg(S * q_out), k(S * kv_dim), v(S * kv_dim),
          attn(S * attn_dim);
      linear_unpacked(norm.data(), 1, S, H, weight(m, layer, 8, L.q_proj, q_out, H),
                      qg.data(), 1, 0, c.mode);
      linear_unpacked(norm.data(), 1, S, H, weight(m, layer, 9, L.k_proj, kv_dim, H),
                      k.data(), 1, 0, c.mode);
      linear_unpacked(norm.data(), 1, S, H, weight(m, layer, 10, L.v_proj, kv_dim, H),
                      v.data(), 1, 0, c.mode);
      attention_rows(qg.data(), k.data(), v.data(),
                     reinterpret_cast<const uint16_t *>(m.arena + L.q_norm),
                     reinterpret_cast<const uint16_t *>(m.arena + L.k_norm), cos,
                     sin, kv + full_index * 2 * c.kv_heads * cap * c.head_dim,
                     position, S, c.heads, c.kv_heads, c.head_dim, c.rotary, cap,
                     attn.data());
      linear_unpacked(attn.data(), 1, S, attn_dim,
                      weight(m, layer, 11, L.o_proj, H, attn_dim), branch.data(),
                      1, 0, c.mode);
      ++full_index;
    }
    pointwise(hidden.data(), branch.data(), S * H, 0, residual.data());
    rms_norm_rows(residual.data(), S, H, m.arena + L.post_norm, 1, c.eps, 1,
                  norm.data());
    mlp(m, layer, L, norm.data(), S, branch.data());
    pointwise(residual.data(), branch.data(), S * H, 0, hidden.data());
  }

  rms_norm_rows(hidden.data(), S, H, m.arena + m.final_norm, 1, c.eps, 1,
                norm.data());
  if (hidden_out)
    std::memcpy(hidden_out, norm.data(), static_cast<size_t>(S * H) * 2);
  if (!m.embed_ready) {
    if (c.mode >= 2) {
      m.embed_unpacked.N = c.vocab;
      m.embed_unpacked.K = H;
      m.embed_unpacked.bf = reinterpret_cast<const uint16_t *>(m.arena + m.embed);
    } else {
      unpack(m.arena + m.embed, c.vocab, H, m.embed_unpacked);
    }
    m.embed_ready = true;
  }
  linear_unpacked(norm.data() + (S - 1) * H, 1, 1, H, m.embed_unpacked, logits,
                  0, 0, c.mode);
}

} // extern "C"
