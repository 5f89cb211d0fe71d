// Exact block-wide evaluation of the serial f32 sum  s = (((0 + p[0]) + p[1]) + ... + p[n-1]),
// p[i] >= 0, every addition rounded to nearest-even: the value a one-thread loop produces (the
// reference's rms_norm reduction, DecodeNormalization.cpp:96-105), in fewer dependent steps.
//
// While the running sum stays inside one binade [2^e, 2^(e+1)) it is an integer count S of
// u = 2^(e-23), and  RN(s + p) = u * RNE(S + p/u):  the term contributes floor(p/u), plus one if
// its remainder is above u/2, plus (on an exact tie) whatever makes the new count even, which
// depends on the parity of S alone.  A run of terms in one binade is therefore summarised by two
// integers, its total for an even and for an odd count on entry, and summaries compose
// associatively.
//
// Which binade the sum is in at each term is predicted from an approximate parallel prefix sum
// (any order; it differs from the serial sum by far less than the 2^-10 margin used).  Quads of
// terms that lie safely inside one binade are classified for it and summarised; consecutive
// quads of one binade are composed by a segmented warp scan into runs.  Quads near a power of
// two, and the first 64 terms (where the sum still doubles every few additions), stay serial.
// One thread then stitches the pieces in order: real additions for the serial quads, one integer
// addition per run.  Every prediction is verified on the way (the sum's exponent at the start of
// a run, no carry into the next binade at its end); if one fails, or the terms are not all
// finite, or the sum is zero or subnormal, the plain serial loop produces the result.  The
// result is therefore the serial sum bit for bit in every case; the prediction only decides how
// fast it is obtained.
#pragma once

#include "common.cuh"

namespace llmcp_b200 {

constexpr int kOrderedMaxWarps = 32;
constexpr int kOrderedMaxEntries = 96; // more runs than this: the plain chain is used

struct OrderedSumScratch {
  float warp_total[kOrderedMaxWarps];
  int run_count[kOrderedMaxWarps];
  uint4 entries[kOrderedMaxEntries]; // flat, in order.  x: binade (biased exponent) or -1 serial quad; y: even; z: odd; w: quad
  float result;
};

namespace ordered_sum {

constexpr uint32_t kLimit = 1u << 24;
constexpr uint32_t kSat = 1u << 26;
constexpr int kHeadQuads = 16; // the first 64 terms are added serially

struct Term {
  uint32_t count;
  int round; // 0 down/exact, 1 up, 2 tie
};

__device__ __forceinline__ Term classify(float p, int lsb) {
  const uint32_t b = __float_as_uint(p);
  const int exponent = static_cast<int>(b >> 23);
  const bool normal = exponent != 0;
  const uint32_t m = (b & 0x7fffffu) | (normal ? 0x800000u : 0u);
  const int p_lsb = normal ? exponent - 150 : -149;
  const int shift = lsb - p_lsb;
  // shift <= 0: the term is a multiple of the unit; 1..31: split it; >= 32: it vanishes
  const int right = min(max(shift, 0), 31), left = min(max(-shift, 0), 3);
  const uint32_t whole = shift > 0 ? (shift < 32 ? m >> right : 0u) : (left > 2 ? kSat : m << left);
  const uint32_t rest = (shift > 0 && shift < 32) ? (m & ((1u << right) - 1u)) : 0u;
  const uint32_t half = (shift > 0 && shift < 32) ? (1u << (right - 1)) : 1u;
  Term t;
  t.count = m == 0u ? 0u : whole;
  t.round = (m == 0u || rest < half) ? 0 : (rest > half ? 1 : 2);
  return t;
}
__device__ __forceinline__ uint32_t increment(Term t, uint32_t parity) {
  return t.count + (t.round == 1 ? 1u : (t.round == 2 ? ((parity + t.count) & 1u) : 0u));
}
__device__ __forceinline__ uint32_t saturate(uint32_t v) { return v < kSat ? v : kSat; }
__device__ __forceinline__ void compose(uint32_t a_even, uint32_t a_odd, uint32_t b_even, uint32_t b_odd,
                                        uint32_t &even, uint32_t &odd) {
  even = saturate(a_even + ((a_even & 1u) ? b_odd : b_even));
  odd = saturate(a_odd + (((1u + a_odd) & 1u) ? b_odd : b_even));
}
__device__ __forceinline__ float serial(const float *p_sm, int from, int to, float s) {
  int i = from;
  for (; i + 32 <= to; i += 32) {
    float4 t[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      t[u] = *reinterpret_cast<const float4 *>(p_sm + i + 4 * u);
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      s = __fadd_rn(s, t[u].x);
      s = __fadd_rn(s, t[u].y);
      s = __fadd_rn(s, t[u].z);
      s = __fadd_rn(s, t[u].w);
    }
  }
  for (; i < to; ++i)
    s = __fadd_rn(s, p_sm[i]);
  return s;
}

} // namespace ordered_sum

// Thread t holds terms [4t, 4t+4) in p (zeros beyond n); p_sm holds all n terms (16-byte aligned,
// visible to the block).  n % 4 == 0, blockDim.x * 4 >= n.  Every thread calls; all get the sum.
__device__ float block_ordered_sum(const float (&p)[4], const float *p_sm, int n, bool any_bad,
                                   OrderedSumScratch &sc) {
  using namespace ordered_sum;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int warps = (blockDim.x + 31) >> 5;
  const int quads = n >> 2;
  const bool active = tid < quads;
  // approximate prefix sums (any order): they only predict where the sum changes binade
  const float q = active ? (p[0] + p[1]) + (p[2] + p[3]) : 0.0f;
  float incl = q;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const float o = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d)
      incl += o;
  }
  if (lane == 31)
    sc.warp_total[warp] = incl;
  const bool serial_only = __syncthreads_or(any_bad ? 1 : 0) != 0;
  float base;
  {
    const float mine = lane < warps ? sc.warp_total[lane] : 0.0f; // warps <= 32
    float scan = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float o = __shfl_up_sync(0xffffffffu, scan, d);
      if (lane >= d)
        scan += o;
    }
    base = __shfl_sync(0xffffffffu, scan - mine, warp);
  }
  const float lo = base + (incl - q), hi = base + incl;
  // kind: -2 head or inactive (no entry), -1 serial quad, else the binade (biased exponent)
  int key = -2;
  uint32_t even = 0u, odd = 0u;
  if (active && tid >= kHeadQuads) {
    key = -1;
    const uint32_t e_lo = __float_as_uint(lo * 0.9990234375f) >> 23;  // 1 - 2^-10
    const uint32_t e_hi = __float_as_uint(hi * 1.0009765625f) >> 23;  // 1 + 2^-10
    if (lo > 0.0f && e_lo == e_hi && e_lo >= 1u && e_lo < 254u) {
      key = static_cast<int>(e_lo);
      const int lsb = key - 150;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const Term t = classify(p[u], lsb);
        even = saturate(even + increment(t, even & 1u));
        odd = saturate(odd + increment(t, (1u + odd) & 1u));
      }
    }
  }
  // runs inside the warp: consecutive clean quads of one binade; every serial quad is its own run
  const int prev_key = __shfl_up_sync(0xffffffffu, key, 1);
  const bool starts = key != -2 && (lane == 0 || key == -1 || prev_key != key);
  const uint32_t start_mask = __ballot_sync(0xffffffffu, starts);
  const int run = __popc(start_mask & (0xffffffffu >> (31 - lane))) - 1; // index of my run (if key != -2)
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const uint32_t o_even = __shfl_up_sync(0xffffffffu, even, d);
    const uint32_t o_odd = __shfl_up_sync(0xffffffffu, odd, d);
    const int o_run = __shfl_up_sync(0xffffffffu, run, d);
    const int o_key = __shfl_up_sync(0xffffffffu, key, d);
    if (lane >= d && key >= 0 && o_key == key && o_run == run)
      compose(o_even, o_odd, even, odd, even, odd);
  }
  const int next_run = __shfl_down_sync(0xffffffffu, run, 1);
  const int next_key = __shfl_down_sync(0xffffffffu, key, 1);
  const bool tail = key != -2 && (lane == 31 || next_key == -2 || next_run != run);
  if (lane == 0)
    sc.run_count[warp] = __popc(start_mask);
  __syncthreads();
  // every run's tail lane writes its entry at the run's place in the flat, ordered list
  int offset, total_runs;
  {
    int mine = lane < warps ? sc.run_count[lane] : 0; // warps <= 32
    int incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d)
        incl += o;
    }
    total_runs = __shfl_sync(0xffffffffu, incl, 31);
    offset = __shfl_sync(0xffffffffu, incl - mine, warp);
  }
  const bool listed = total_runs <= kOrderedMaxEntries;
  if (tail && listed)
    sc.entries[offset + run] = make_uint4(static_cast<uint32_t>(key), even, odd, static_cast<uint32_t>(tid));
  __syncthreads();
  if (tid == 0) {
    const int head = min(kHeadQuads * 4, n);
    float s = serial(p_sm, 0, head, 0.0f);
    bool ok = !serial_only && listed;
    if (ok) {
      // Eight entries at a time: their loads first, then a chain in registers.  A failed
      // prediction only clears `ok`; the chain runs on.
      for (int base_entry = 0; base_entry < total_runs; base_entry += 8) {
        uint4 e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
          e[i] = base_entry + i < total_runs ? sc.entries[base_entry + i] : make_uint4(0xfffffffeu, 0u, 0u, 0u);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (e[i].x == 0xffffffffu) { // serial quad
            const float4 terms = *reinterpret_cast<const float4 *>(p_sm + 4 * e[i].w);
            s = __fadd_rn(s, terms.x);
            s = __fadd_rn(s, terms.y);
            s = __fadd_rn(s, terms.z);
            s = __fadd_rn(s, terms.w);
          } else if (e[i].x != 0xfffffffeu) { // a run of clean quads in binade e.x
            const uint32_t bits = __float_as_uint(s);
            const uint32_t units = (bits & 0x7fffffu) | 0x800000u;
            const uint32_t next = units + ((units & 1u) ? e[i].z : e[i].y);
            ok = ok && (bits >> 23) == e[i].x && next < kLimit;
            s = __uint_as_float((bits & 0x7f800000u) | (next & 0x7fffffu));
          }
        }
      }
    }
    if (!ok)
      s = serial(p_sm, head, n, serial(p_sm, 0, head, 0.0f));
    sc.result = s;
  }
  __syncthreads();
  const float result = sc.result;
  __syncthreads();
  return result;
}

} // namespace llmcp_b200
