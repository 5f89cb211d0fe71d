// Fast-mode attention for one query token (the decode step): llmcp.attention,
// LowerAttention.cpp:394-601, with the key range split over CTAs.
//
// The exact kernels (mixers.cu) keep the reference's order: scores, then one CTA per query head
// walks all keys in ascending order.  At batch 1 that leaves 16 CTAs streaming the value rows
// through 16 of 148 SMs.  Here a CTA owns (KV head, range of `chunk` keys) and serves the whole
// group of query heads that share the KV head: key rows and value rows are read from HBM once,
// straight into registers, each thread's loads all requested before the first is used.  Per
// 32-key tile: scores (eight threads per key, 1/8 of the head dimension each, three shuffles),
// a running (maximum, denominator) per head, and the probability-weighted value sum with eight
// dimensions per thread.  A second kernel merges the splits' (maximum, denominator, sum)
// triples, divides, applies the sigmoid gate, rounds to bf16 and quantises for o_proj.
//
// The result is the same function of the inputs as the reference's tile-ordered online softmax;
// only the order of the f32 additions differs (and exp is expf, not the rounded f64 function),
// so outputs agree with the exact kernels to f32 rounding, not bit for bit.

#include <algorithm>

#include "kernels.h"

namespace llmcp_b200 {

namespace {

constexpr int kSplitThreads = 256;
constexpr int kSplitTile = 32; // keys per inner tile

template <int HD, int GROUP> struct SplitLayout {
  static constexpr int PD = HD / 8;           // dimensions per thread in the score phase
  static constexpr int QS = PD + 4;           // padded: a quarter warp's eight parts hit distinct banks
  static constexpr int DG = HD / 8;           // groups of eight dimensions in the value phase
  static constexpr int KG = kSplitThreads / DG; // key groups
  static constexpr int KPG = kSplitTile / KG; // keys per group and tile
  static constexpr int kQ = GROUP * 8 * QS, kS = GROUP * kSplitTile, kC = 8, kR = KG * GROUP * HD;
  static constexpr size_t kBytes = static_cast<size_t>(kQ + kS + kC + kR) * sizeof(float);
  static_assert(HD % 64 == 0 && KPG >= 1, "head dimension 64, 128 or 256");
};

__device__ __forceinline__ void unpack8(const uint4 &raw, float *f) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int u = 0; u < 4; ++u) {
    f[2 * u] = __uint_as_float(w[u] << 16);
    f[2 * u + 1] = __uint_as_float(w[u] & 0xffff0000u);
  }
}

// grid: (split, kv head); block: 256 threads.
// part_acc: [nh][splits][HD] f32, part_ml: [nh][splits][2] f32 (running maximum, denominator).
template <int HD, int GROUP>
__global__ void __launch_bounds__(kSplitThreads)
attn_decode_split_kernel(const uint16_t *__restrict__ qn, const uint16_t *__restrict__ cache,
                         const int64_t *__restrict__ position_ptr, int nkv, int64_t cap, int chunk, int splits,
                         float *__restrict__ part_acc, float *__restrict__ part_ml, int64_t cache_stride) {
  using Lay = SplitLayout<HD, GROUP>;
  constexpr int PD = Lay::PD, QS = Lay::QS, DG = Lay::DG, KG = Lay::KG, KPG = Lay::KPG;
  extern __shared__ __align__(16) float split_sm[];
  float *q_sm = split_sm;        // [GROUP][8][QS]
  float *s_sm = q_sm + Lay::kQ;  // [GROUP][32]: scores, then probabilities
  float *c_sm = s_sm + Lay::kS;  // [GROUP]: correction of the running sums for this tile
  float *r_sm = c_sm + Lay::kC;  // [KG][GROUP][HD]
  grid_dependency_sync(true);
  const int total = static_cast<int>(*position_ptr) + 1;
  const int split = blockIdx.x, kvh = blockIdx.y;
  { // blockIdx.z: sequence of a batch (one query token each, a cache per sequence)
    const int64_t seq = blockIdx.z;
    const int64_t heads = static_cast<int64_t>(nkv) * GROUP;
    qn += seq * heads * HD;
    cache += seq * cache_stride;
    part_acc += seq * heads * splits * HD;
    part_ml += seq * heads * splits * 2;
  }
  const int begin = split * chunk;
  if (begin >= total)
    return; // the merge kernel reads the splits that hold keys only
  const int end = min(total, begin + chunk);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  for (int i = tid; i < GROUP * HD; i += kSplitThreads) {
    const int g = i / HD, d = i - g * HD;
    q_sm[(g * 8 + d / PD) * QS + d % PD] = bf16_to_f32(qn[static_cast<int64_t>(kvh * GROUP + g) * HD + d]);
  }
  const uint16_t *kbase = cache + static_cast<int64_t>(kvh) * cap * HD;
  const uint16_t *vbase = cache + (static_cast<int64_t>(nkv) + kvh) * cap * HD;
  const float scale = __fdiv_rn(1.0f, __fsqrt_rn(static_cast<float>(HD)));
  const int j = tid >> 3, part = tid & 7; // score phase: key of the tile, eighth of the head dimension
  const int dg = tid % DG, kg = tid / DG; // value phase: eight dimensions, group of KPG keys

  float acc[GROUP][8];
#pragma unroll
  for (int g = 0; g < GROUP; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e)
      acc[g][e] = 0.0f;
  float m_run = -1.0e30f, l_run = 0.0f; // of head `warp`, in the warps below GROUP

  for (int tile = begin; tile < end; tile += kSplitTile) {
    const int key = tile + j;
    uint4 kraw[PD / 8];
    if (key < end) {
#pragma unroll
      for (int u = 0; u < PD / 8; ++u)
        kraw[u] = reinterpret_cast<const uint4 *>(kbase + static_cast<int64_t>(key) * HD + part * PD)[u];
    }
    uint4 vraw[KPG];
#pragma unroll
    for (int u = 0; u < KPG; ++u) {
      const int vkey = tile + kg * KPG + u;
      vraw[u] = vkey < end ? *reinterpret_cast<const uint4 *>(vbase + static_cast<int64_t>(vkey) * HD + dg * 8)
                           : make_uint4(0u, 0u, 0u, 0u);
    }
    __syncthreads(); // the query is staged; the previous tile's probabilities have been used
    float dot[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; ++g)
      dot[g] = 0.0f;
    if (key < end) {
#pragma unroll
      for (int u = 0; u < PD / 8; ++u) {
        float kf[8];
        unpack8(kraw[u], kf);
#pragma unroll
        for (int g = 0; g < GROUP; ++g) {
          const float4 q0 = *reinterpret_cast<const float4 *>(q_sm + (g * 8 + part) * QS + 8 * u);
          const float4 q1 = *reinterpret_cast<const float4 *>(q_sm + (g * 8 + part) * QS + 8 * u + 4);
          dot[g] = __fmaf_rn(q0.x, kf[0], dot[g]);
          dot[g] = __fmaf_rn(q0.y, kf[1], dot[g]);
          dot[g] = __fmaf_rn(q0.z, kf[2], dot[g]);
          dot[g] = __fmaf_rn(q0.w, kf[3], dot[g]);
          dot[g] = __fmaf_rn(q1.x, kf[4], dot[g]);
          dot[g] = __fmaf_rn(q1.y, kf[5], dot[g]);
          dot[g] = __fmaf_rn(q1.z, kf[6], dot[g]);
          dot[g] = __fmaf_rn(q1.w, kf[7], dot[g]);
        }
      }
    }
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      dot[g] = __fadd_rn(dot[g], __shfl_xor_sync(0xffffffffu, dot[g], 1));
      dot[g] = __fadd_rn(dot[g], __shfl_xor_sync(0xffffffffu, dot[g], 2));
      dot[g] = __fadd_rn(dot[g], __shfl_xor_sync(0xffffffffu, dot[g], 4));
    }
    if (part == 0) {
#pragma unroll
      for (int g = 0; g < GROUP; ++g)
        s_sm[g * kSplitTile + j] = key < end ? __fmul_rn(dot[g], scale) : -1.0e30f;
    }
    __syncthreads();
    if (warp < GROUP) {
      const float sc = s_sm[warp * kSplitTile + lane];
      float m_tile = sc;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, o));
      const float m_new = fmaxf(m_run, m_tile);
      const float p = tile + lane < end ? expf(__fsub_rn(sc, m_new)) : 0.0f;
      float l_tile = p;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        l_tile = __fadd_rn(l_tile, __shfl_xor_sync(0xffffffffu, l_tile, o));
      const float corr = expf(__fsub_rn(m_run, m_new));
      s_sm[warp * kSplitTile + lane] = p;
      if (lane == 0)
        c_sm[warp] = corr;
      l_run = __fmaf_rn(l_run, corr, l_tile);
      m_run = m_new;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      const float corr = c_sm[g];
#pragma unroll
      for (int e = 0; e < 8; ++e)
        acc[g][e] = __fmul_rn(acc[g][e], corr);
    }
#pragma unroll
    for (int u = 0; u < KPG; ++u) {
      float vf[8];
      unpack8(vraw[u], vf);
#pragma unroll
      for (int g = 0; g < GROUP; ++g) {
        const float p = s_sm[g * kSplitTile + kg * KPG + u];
#pragma unroll
        for (int e = 0; e < 8; ++e)
          acc[g][e] = __fmaf_rn(p, vf[e], acc[g][e]);
      }
    }
  }
  // The key groups' sums meet in shared memory.
#pragma unroll
  for (int g = 0; g < GROUP; ++g) {
    float *dst = r_sm + (static_cast<size_t>(kg) * GROUP + g) * HD + dg * 8;
    *reinterpret_cast<float4 *>(dst) = make_float4(acc[g][0], acc[g][1], acc[g][2], acc[g][3]);
    *reinterpret_cast<float4 *>(dst + 4) = make_float4(acc[g][4], acc[g][5], acc[g][6], acc[g][7]);
  }
  __syncthreads();
  for (int i = tid; i < GROUP * HD; i += kSplitThreads) {
    const int g = i / HD, d = i - g * HD;
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < KG; ++k)
      sum = __fadd_rn(sum, r_sm[(static_cast<size_t>(k) * GROUP + g) * HD + d]);
    part_acc[(static_cast<size_t>(kvh * GROUP + g) * splits + split) * HD + d] = sum;
  }
  if (warp < GROUP && lane == 0) {
    float *ml = part_ml + (static_cast<size_t>(kvh * GROUP + warp) * splits + split) * 2;
    ml[0] = m_run;
    ml[1] = l_run;
  }
}

// grid: query head; block: kMergeGroups x HD threads.  Thread (g, d) folds splits g, g + 4, ... of head
// dimension d (every load of a round issued before the first use: the partial sums come from L2
// and a dependent chain over 30-70 splits would cost a round trip each); group 0 adds the four
// partial results in group order.
constexpr int kMergeGroups = 4;
constexpr int kMergeUnroll = 8;

template <int HD>
__global__ void __launch_bounds__(kMergeGroups *HD)
attn_decode_merge_kernel(const float *__restrict__ part_acc, const float *__restrict__ part_ml,
                         const uint16_t *__restrict__ qg, const int64_t *__restrict__ position_ptr, int chunk,
                         int splits, uint16_t *__restrict__ out, int8_t *__restrict__ q_out,
                         float *__restrict__ s_out) {
  __shared__ float group_l[kMergeGroups];
  __shared__ float group_o[kMergeGroups][HD];
  // blockIdx.y: sequence of a batch; its heads follow the previous sequence's in every buffer
  const int h = blockIdx.y * gridDim.x + blockIdx.x;
  const int d = threadIdx.x % HD, g = threadIdx.x / HD, lane = threadIdx.x & 31;
  grid_dependency_sync(true);
  const float gate = g == 0 ? bf16_to_f32(qg[static_cast<int64_t>(h) * 2 * HD + HD + d]) : 0.0f;
  const int total = static_cast<int>(*position_ptr) + 1;
  const int active = (total + chunk - 1) / chunk;
  const float *ml = part_ml + static_cast<size_t>(h) * splits * 2;
  const float *pa = part_acc + static_cast<size_t>(h) * splits * HD + d;
  // maximum over the splits: every warp folds all of them (lane-strided), so no second barrier
  float m = -1.0e30f;
  for (int s = lane; s < active; s += 32)
    m = fmaxf(m, ml[2 * s]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  float l = 0.0f, o = 0.0f;
  for (int s0 = g; s0 < active; s0 += kMergeGroups * kMergeUnroll) {
    float w[kMergeUnroll], a[kMergeUnroll], ls[kMergeUnroll];
#pragma unroll
    for (int u = 0; u < kMergeUnroll; ++u) {
      const int s = s0 + u * kMergeGroups;
      const bool on = s < active;
      a[u] = on ? pa[static_cast<size_t>(s) * HD] : 0.0f;
      w[u] = on ? ml[2 * s] : -1.0e30f;
      ls[u] = on ? ml[2 * s + 1] : 0.0f;
    }
#pragma unroll
    for (int u = 0; u < kMergeUnroll; ++u) {
      const float e = expf(__fsub_rn(w[u], m));
      l = __fmaf_rn(e, ls[u], l);
      o = __fmaf_rn(e, a[u], o);
    }
  }
  group_o[g][d] = o;
  if (d == 0)
    group_l[g] = l;
  __syncthreads();
  if (g != 0)
    return;
  l = group_l[0], o = group_o[0][d];
#pragma unroll
  for (int k = 1; k < kMergeGroups; ++k) {
    l = __fadd_rn(l, group_l[k]);
    o = __fadd_rn(o, group_o[k][d]);
  }
  const float sigmoid = __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-gate)));
  const uint16_t bits = f32_to_bf16(__fmul_rn(__fdiv_rn(o, l), sigmoid));
  const int64_t index = static_cast<int64_t>(h) * HD + d;
  out[index] = bits;
  if (q_out) // the quantisation o_proj needs (Q8Decode.cpp:83-120): a warp holds one 32-block
    warp_quant_block(bf16_to_f32(bits), q_out, s_out, index, index >> 5, lane);
}

// Keys per split: enough splits to give every SM a CTA or two, whole 32-key tiles.
int fast_chunk(int64_t max_total, int nkv) {
  const int64_t target_splits = std::max<int64_t>(1, 296 / std::max(1, nkv));
  const int64_t per = (max_total + target_splits - 1) / target_splits;
  return static_cast<int>(std::max<int64_t>(kSplitTile, (per + kSplitTile - 1) / kSplitTile * kSplitTile));
}

template <int HD, int GROUP>
cudaError_t launch_split(const uint16_t *qn, const uint16_t *cache, const int64_t *position_dev, int nkv, int64_t cap,
                         int chunk, int splits, float *part_acc, float *part_ml, cudaStream_t stream, int sequences,
                         int64_t cache_stride) {
  using Lay = SplitLayout<HD, GROUP>;
  if (cudaError_t e = opt_in_shared_memory(reinterpret_cast<const void *>(attn_decode_split_kernel<HD, GROUP>), Lay::kBytes);
      e != cudaSuccess)
    return e;
  launch_chained(attn_decode_split_kernel<HD, GROUP>, dim3(splits, nkv, sequences), dim3(kSplitThreads), Lay::kBytes, stream, qn,
                 cache, position_dev, nkv, cap, chunk, splits, part_acc, part_ml, cache_stride);
  return cudaGetLastError();
}

template <int HD>
cudaError_t launch_split_hd(int group, const uint16_t *qn, const uint16_t *cache, const int64_t *position_dev, int nkv,
                            int64_t cap, int chunk, int splits, float *part_acc, float *part_ml, cudaStream_t stream,
                            int sequences, int64_t cache_stride) {
  switch (group) {
  case 1:
    return launch_split<HD, 1>(qn, cache, position_dev, nkv, cap, chunk, splits, part_acc, part_ml, stream, sequences, cache_stride);
  case 2:
    return launch_split<HD, 2>(qn, cache, position_dev, nkv, cap, chunk, splits, part_acc, part_ml, stream, sequences, cache_stride);
  case 4:
    return launch_split<HD, 4>(qn, cache, position_dev, nkv, cap, chunk, splits, part_acc, part_ml, stream, sequences, cache_stride);
  default:
    return cudaErrorNotSupported;
  }
}

} // namespace

bool attention_decode_fast_supported(int nh, int nkv, int hd) {
  if (nh <= 0 || nkv <= 0 || nh % nkv != 0)
    return false;
  const int group = nh / nkv;
  return (hd == 128 || hd == 256) && (group == 1 || group == 2 || group == 4);
}

size_t attn_fast_scratch_bytes(int nh, int hd, int64_t max_position, int sequences) {
  const int64_t max_total = max_position + 1;
  // nkv is not known here: size for the smallest chunk the launcher can choose.
  const int64_t splits = (max_total + kSplitTile - 1) / kSplitTile;
  const size_t qn_bytes = (static_cast<size_t>(sequences) * nh * hd * sizeof(uint16_t) + 255) / 256 * 256;
  return qn_bytes + static_cast<size_t>(sequences) * nh * splits * (hd + 2) * sizeof(float) + 256;
}

cudaError_t launch_attention_decode_fast(const uint16_t *qg, const uint16_t *k, const uint16_t *v,
                                         const uint16_t *q_norm, const uint16_t *k_norm, const float *cos,
                                         const float *sin, int rows_from_position, uint16_t *cache,
                                         const int64_t *position_dev, int64_t max_position, int nh, int nkv, int hd,
                                         int rot, int64_t cap, void *scratch, uint16_t *out, int8_t *q_out,
                                         float *s_out, cudaStream_t stream, int sequences, int64_t cache_stride) {
  if (!attention_decode_fast_supported(nh, nkv, hd))
    return cudaErrorNotSupported;
  if (rot % 2 != 0 || rot > hd || max_position + 1 > cap || sequences < 1 || (sequences > 1 && cache_stride == 0))
    return cudaErrorInvalidValue;
  const int64_t max_total = max_position + 1;
  const int chunk = fast_chunk(max_total, nkv * sequences);
  const int splits = static_cast<int>((max_total + chunk - 1) / chunk);
  uint16_t *qn = static_cast<uint16_t *>(scratch);
  const size_t qn_bytes = (static_cast<size_t>(sequences) * nh * hd * sizeof(uint16_t) + 255) / 256 * 256;
  float *part_acc = reinterpret_cast<float *>(static_cast<unsigned char *>(scratch) + qn_bytes);
  float *part_ml = part_acc + static_cast<size_t>(sequences) * nh * splits * hd;
  if (cudaError_t e = launch_attention_prepare(qg, k, v, q_norm, k_norm, cos, sin, rows_from_position, cache, position_dev,
                                               sequences, nh, nkv, hd, rot, cap, qn, stream, 1, sequences > 1 ? cache_stride : 0);
      e != cudaSuccess)
    return e;
  const int group = nh / nkv;
  cudaError_t e = hd == 256 ? launch_split_hd<256>(group, qn, cache, position_dev, nkv, cap, chunk, splits, part_acc, part_ml, stream,
                                                   sequences, cache_stride)
                            : launch_split_hd<128>(group, qn, cache, position_dev, nkv, cap, chunk, splits, part_acc, part_ml, stream,
                                                   sequences, cache_stride);
  if (e != cudaSuccess)
    return e;
  if (hd == 256)
    launch_chained(attn_decode_merge_kernel<256>, dim3(nh, sequences), dim3(kMergeGroups * 256), 0, stream, part_acc, part_ml, qg, position_dev, chunk,
                   splits, out, q_out, s_out);
  else
    launch_chained(attn_decode_merge_kernel<128>, dim3(nh, sequences), dim3(kMergeGroups * 128), 0, stream, part_acc, part_ml, qg, position_dev, chunk,
                   splits, out, q_out, s_out);
  return cudaGetLastError();
}

} // namespace llmcp_b200
