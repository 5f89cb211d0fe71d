// Exact block-wide evaluation of the serial f32 sum  s = (((0 + p[0]) + p[1]) + ... + p[n-1]),
// p[i] >= 0, every addition rounded to nearest-even: the value a one-thread loop produces (the
// reference's rms_norm reduction, DecodeNormalization.cpp:96-105), in fewer dependent steps.
//
// While the running sum stays inside one binade [2^e, 2^(e+1)) it is an integer count S of
// u = 2^(e-23), 2^23 <= S < 2^24, and  RN(s + p) = u * RNE(S + p/u).  What the addition adds to
// the count depends on S only through its parity (an exact tie goes to the even count).  So a
// stretch of terms in one binade is summarised by two integers, what it adds for an even and for
// an odd count on entry, and summaries compose associatively.
//
// The two integers of a quad of terms come from floating-point additions themselves: with the
// terms scaled by 1/u (exact, a power of two), the chain  2^23 + p0/u + p1/u + ...  in f32 makes
// the same rounding decisions as the real sum from an even count, and the chain from 2^23 + 1
// those from an odd count, as long as neither reaches 2^24.
//
// Which binade the sum is in at each term is predicted from an approximate parallel prefix sum
// (any order; it differs from the serial sum by far less than the 2^-10 margin used).  Quads of
// terms that lie safely inside one binade are summarised for it; consecutive quads of one binade
// are composed by a segmented warp scan into runs.  Quads near a power of two stay serial, and
// so does the head of the sum (at least 64 terms, where the sum still doubles every few
// additions; about a sixth of the terms when a spare warp can add them while the others scan).
// One thread then stitches the pieces in order: four real additions for a serial quad, one
// integer addition to the sum's bit pattern for a run.  Every prediction is verified on the way
// (the sum's exponent at the start of a run, no carry into the next binade at its end); if one
// fails, or the terms are not all finite and non-negative, or the sum is zero or tiny, the plain
// serial loop produces the result.
// The result is therefore the serial sum bit for bit in every case; the prediction only decides
// how fast it is obtained.
#pragma once

#include "common.cuh"

namespace llmcp_b200 {

constexpr int kOrderedMaxWarps = 32;
constexpr int kOrderedMaxEntries = 96; // more pieces than this: the plain chain is used
constexpr int kOrderedChunk = 8;       // padding behind the list: the stitch fetches up to seven entries ahead

// One piece of the sum per entry, in order.  A run of quads in one binade: x = 2^31 | binade
// (biased exponent), y = what it adds to an even count, z = what it adds to an odd count minus
// y (-1, 0 or 1), w = binade << 23.  A serial quad: its four terms as f32 bits (sign bit
// clear); four zeros serve as padding.
struct OrderedSumScratch {
  alignas(16) float warp_total[kOrderedMaxWarps];
  int run_count[kOrderedMaxWarps];
  uint4 entries[kOrderedMaxEntries + kOrderedChunk];
  float result;
};

namespace ordered_sum {

constexpr int kHeadQuads = 16;               // the first 64 terms are always added serially
constexpr int kHeadShare = 6;                // a spare warp adds about this fraction of the terms serially
constexpr uint32_t kSat = 1u << 26;          // a total this large fails the carry check anyway
constexpr uint32_t kRun = 0x80000000u;
constexpr uint32_t kEvenStart = 0x4b000000u; // 2^23 as f32 bits
constexpr uint32_t kOddStart = 0x4b000001u;  // 2^23 + 1

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

// One entry applied to the running sum, without branches: both forms are evaluated and one is
// kept.  `wrong` collects failed predictions: a run must find the sum in its binade and leave it
// there (e.w holds the binade in the exponent's place).
__device__ __forceinline__ float apply(float s, const uint4 e, uint32_t &wrong) {
  const uint32_t bits = __float_as_uint(s);
  const uint32_t next = (bits + e.y) + (bits & 1u) * e.z; // e.z: odd total minus even total
  const float added = __fadd_rn(__fadd_rn(__fadd_rn(__fadd_rn(s, __uint_as_float(e.x)), __uint_as_float(e.y)),
                                          __uint_as_float(e.z)), __uint_as_float(e.w));
  const bool run = static_cast<int32_t>(e.x) < 0;
  const uint32_t checked = static_cast<uint32_t>(static_cast<int32_t>(e.x) >> 31) & 0xff800000u;
  wrong |= ((bits ^ e.w) | (next ^ e.w)) & checked;
  return run ? __uint_as_float(next) : added;
}

} // namespace ordered_sum

// Thread t holds terms [4t, 4t+4) in p (zeros beyond n); p_sm holds all n terms (16-byte aligned,
// visible to the block).  n % 4 == 0, blockDim.x * 4 >= n, blockDim.x a multiple of 32.  Every
// thread calls; all get finish(sum), which one thread evaluates.  If the block's last warp holds
// no terms it stays out of the other warps' barriers (which then use barrier 1): one of its
// threads adds the head of the sum meanwhile, and stitches.  The caller synchronises the block
// before it reuses `sc`.
template <typename Finish>
__device__ float block_ordered_sum(const float (&p)[4], const float *p_sm, int n, bool any_bad,
                                   OrderedSumScratch &sc, Finish finish) {
  using namespace ordered_sum;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int quads = n >> 2;
  const bool spare = static_cast<int>(blockDim.x) - 32 >= quads;
  const int workers = static_cast<int>(blockDim.x) - (spare ? 32 : 0); // threads of the parallel part
  const int worker_warps = workers >> 5;
  const int stitcher = spare ? workers : 0;
  // a spare warp has the time of the parallel part for its serial head: a quarter of the terms
  const int head_quads = min(quads, spare ? max(kHeadQuads, (quads / kHeadShare) & ~31) : kHeadQuads);
  const int head = head_quads * 4;
  float head_sum = 0.0f;
  if (tid >= workers) {
    if (tid == stitcher)
      head_sum = serial(p_sm, 0, head, 0.0f);
  } else {
    const bool active = tid < quads;
    const bool bad = any_bad || ((__float_as_uint(p[0]) | __float_as_uint(p[1]) | __float_as_uint(p[2]) |
                                  __float_as_uint(p[3])) >> 31) != 0u;
    // approximate prefix sums (any order): they only predict where the sum changes binade
    const float q = active ? (p[0] + p[1]) + (p[2] + p[3]) : 0.0f;
    float incl = q;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const float o = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d)
        incl += o;
    }
    const bool warp_bad = __any_sync(0xffffffffu, bad);
    if (lane == 31)
      sc.warp_total[warp] = warp_bad ? __uint_as_float(0x7fc00000u) : incl; // not finite: the plain chain
    if (spare)
      asm volatile("bar.sync 1, %0;" ::"r"(workers) : "memory");
    else
      __syncthreads();
    // the sum of the totals of the warps in front (any order will do)
    float base = lane < warp ? sc.warp_total[lane] : 0.0f;
#pragma unroll
    for (int d = 16; d > 0; d >>= 1)
      base += __shfl_xor_sync(0xffffffffu, base, d);
    const float lo = base + (incl - q), hi = base + incl;
    // key: -2 head or inactive (no entry), -1 serial quad, else the binade (biased exponent)
    int key = -2;
    uint32_t even = 0u, odd = 0u;
    if (active && tid >= head_quads) {
      key = -1;
      const uint32_t e_lo = __float_as_uint(lo * 0.9990234375f) >> 23; // 1 - 2^-10
      const uint32_t e_hi = __float_as_uint(hi * 1.0009765625f) >> 23; // 1 + 2^-10
      if (lo > 0.0f && e_lo == e_hi && e_lo >= 24u && e_lo < 254u) {
        const float scale = __uint_as_float((277u - e_lo) << 23); // 1/u = 2^(150 - e)
        float from_even = __uint_as_float(kEvenStart), from_odd = __uint_as_float(kOddStart);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float scaled = __fmul_rn(p[u], scale);
          from_even = __fadd_rn(from_even, scaled);
          from_odd = __fadd_rn(from_odd, scaled);
        }
        if (from_even < 16777216.0f && from_odd < 16777216.0f) {
          key = static_cast<int>(e_lo);
          even = __float_as_uint(from_even) - kEvenStart;
          odd = __float_as_uint(from_odd) - kOddStart;
        }
      }
    }
    // runs inside the warp: consecutive clean quads of one binade; every serial quad is its own run
    const int prev_key = __shfl_up_sync(0xffffffffu, key, 1);
    const bool starts = key != -2 && (lane == 0 || key == -1 || prev_key != key);
    const uint32_t start_mask = __ballot_sync(0xffffffffu, starts);
    const uint32_t live_mask = __ballot_sync(0xffffffffu, key != -2);
    const uint32_t upto = start_mask & (0xffffffffu >> (31 - lane));
    const int run = __popc(upto) - 1;                           // index of my run (if key != -2)
    const int reach = key >= 0 ? lane - (31 - __clz(upto)) : 0; // lanes of my run in front of me
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const uint32_t o_even = __shfl_up_sync(0xffffffffu, even, d);
      const uint32_t o_odd = __shfl_up_sync(0xffffffffu, odd, d);
      if (d <= reach) { // the totals stay below 32 * 2^23
        const uint32_t new_even = o_even + ((o_even & 1u) ? odd : even);
        const uint32_t new_odd = o_odd + ((o_odd & 1u) ? even : odd);
        even = new_even;
        odd = new_odd;
      }
    }
    const bool tail = key != -2 && (lane == 31 || ((start_mask | ~live_mask) >> (lane + 1)) & 1u);
    if (lane == 0)
      sc.run_count[warp] = __popc(start_mask);
    if (spare)
      asm volatile("bar.sync 1, %0;" ::"r"(workers) : "memory");
    else
      __syncthreads();
    // every run's tail lane writes its entry at the run's place in the flat, ordered list
    const int count = lane < worker_warps ? sc.run_count[lane] : 0; // at most 32 warps
    const int total_runs = __reduce_add_sync(0xffffffffu, count);
    const int offset = __reduce_add_sync(0xffffffffu, lane < warp ? count : 0);
    if (total_runs <= kOrderedMaxEntries) {
      if (tail)
        sc.entries[offset + run] =
            key >= 0 ? make_uint4(kRun | static_cast<uint32_t>(key), min(even, kSat), min(odd, kSat) - min(even, kSat),
                                  static_cast<uint32_t>(key) << 23)
                     : make_uint4(__float_as_uint(p[0]), __float_as_uint(p[1]), __float_as_uint(p[2]),
                                  __float_as_uint(p[3]));
      if (tid < kOrderedChunk) // padding: the stitch fetches ahead and works in fours
        sc.entries[total_runs + tid] = make_uint4(0u, 0u, 0u, 0u); // four zero terms
    }
  }
  __syncthreads();
  if (warp == (stitcher >> 5)) {
    const int count = lane < worker_warps ? sc.run_count[lane] : 0;
    const int total_runs = __reduce_add_sync(0xffffffffu, count);
    const float total = lane < worker_warps ? sc.warp_total[lane] : 0.0f;
    const bool serial_only = __any_sync(0xffffffffu, !(fabsf(total) <= 3.402823466e38f));
    if (tid == stitcher) {
      if (!spare)
        head_sum = serial(p_sm, 0, head, 0.0f);
      float s = head_sum;
      bool ok = !serial_only && total_runs <= kOrderedMaxEntries;
      if (ok) {
        uint32_t wrong = 0u;
        // four entries in flight: each is fetched three entries before it is applied
        uint4 e0 = sc.entries[0], e1 = sc.entries[1], e2 = sc.entries[2], e3 = sc.entries[3];
        for (int first = 0; first < total_runs; first += 4) {
          s = apply(s, e0, wrong);
          e0 = sc.entries[first + 4];
          s = apply(s, e1, wrong);
          e1 = sc.entries[first + 5];
          s = apply(s, e2, wrong);
          e2 = sc.entries[first + 6];
          s = apply(s, e3, wrong);
          e3 = sc.entries[first + 7];
        }
        ok = wrong == 0u;
      }
      if (!ok)
        s = serial(p_sm, head, n, head_sum);
      sc.result = finish(s);
    }
    __syncwarp(); // the stitching thread's warp arrives at the barrier as a whole
  }
  __syncthreads();
  return sc.result;
}

} // namespace llmcp_b200
