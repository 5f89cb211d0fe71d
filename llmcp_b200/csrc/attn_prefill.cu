// Prefill attention (more than one query token) on the fifth-generation tensor cores: the fast form
// of LowerAttention.cpp:266-601 for head_dim 256.  The exact kernels of mixers.cu (one thread per
// (query head, key) dot chain, key-ordered weighted sum) stay the parity path; this one keeps their
// inputs and outputs -- normalised, rotated queries from attn_prepare_kernel, the KV cache as that
// kernel leaves it, (acc / sum) * sigmoid(gate) rounded to bf16 and quantised for o_proj -- and
// changes how the two contractions are evaluated:
//   scores  S = Q K^T     tcgen05.mma kind::f16 on bf16 operands, f32 accumulation in tensor memory;
//   weights P = exp(S * scale - m) rounded to bf16 (the exact kernels keep them in f32);
//   output  O = P V       tcgen05.mma again, V read from a transposed copy so that both operands of
//                         both contractions are K-major tiles with 128-byte swizzle.
// Two passes over the key tiles: the first finds every query row's maximum m and sum l (scores
// only), the second recomputes the scores, forms P against the final m and accumulates O in tensor
// memory without ever rescaling it.  The scores are cheap to compute twice (K tiles come from L2).
//
// One CTA per (128 query rows, query head), 192 threads:
//   warp 0      one lane issues the TMA loads: the Q tile once (4 boxes of 128 rows x 64 dims), per
//               key tile K (4 boxes of 64 keys x 64 dims) and, in pass two, V^T (256 dims x 64 keys);
//   warp 1      allocates tensor memory; one lane issues the MMAs (S of tile i + 1 before P V of tile
//               i, so that the softmax of a tile overlaps the next tile's scores);
//   warps 2-5   one thread per query row: tcgen05.ld of its 64 scores, mask, max / sum (pass one) or
//               P in shared memory in the operand layout (pass two), and the epilogue.
// Every mbarrier wait is bounded; a wait that runs out raises an abort flag that all roles observe,
// the loader waits (bounded) for its copies in flight, tensor memory is always released and the
// error word is set.

#include "kernels.h"
#include "tc_common.cuh"

namespace llmcp_b200 {

namespace {

using namespace tc;

constexpr int kHd = 256;            // head dimension
constexpr int kQTile = 128;         // query rows per CTA = tensor-memory lanes
constexpr int kKeyTile = 64;        // keys per tile = 128 bytes of bf16 weights per row of P
constexpr int kChunks = kHd / 64;   // 128-byte (64 bf16) slices of a head
constexpr int kQChunkBytes = kQTile * 128;    // 16 KB
constexpr int kKChunkBytes = kKeyTile * 128;  //  8 KB
constexpr int kQBytes = kChunks * kQChunkBytes;   // 64 KB
constexpr int kKBytes = kChunks * kKChunkBytes;   // 32 KB
constexpr int kVtBytes = kHd * 128;               // 32 KB: 256 dims x 64 keys
constexpr int kPBytes = kQTile * 128;             // 16 KB
constexpr int kStages = 2;
constexpr int kStageBytes = kKBytes + kVtBytes;   // 64 KB
constexpr int kSmemBytes = 1024 + kQBytes + kStages * kStageBytes + kPBytes + 256;
constexpr int kThreads = 192;
constexpr int kTmemColumns = 512;   // S: 2 x 64 columns at 0 and 64; O: 256 columns at 128
constexpr int kOColumn = 128;

// kind::f16 with bf16 operands, f32 accumulation, both operands K-major, M = 128.
template <int N> struct InstructionBf16 {
  static constexpr uint32_t value = (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(N >> 3) << 17) |
                                    (static_cast<uint32_t>(kQTile >> 4) << 24);
};

__device__ __forceinline__ void mma_bf16(uint32_t tmem, uint64_t a, uint64_t b, uint32_t instruction, uint32_t accumulate) {
  asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p; }"
               :
               : "r"(tmem), "l"(a), "l"(b), "r"(instruction), "r"(accumulate), "r"(0u)
               : "memory");
}

struct Barriers {
  uint64_t q_full;              // the Q tile has landed
  uint64_t full[kStages];       // a key tile's K (and V^T) have landed
  uint64_t empty[kStages];      // ... and are no longer needed by any MMA
  uint64_t s_full[2];           // scores of a tile are in tensor memory
  uint64_t s_empty[2];          // ... and have been read by the four softmax warps
  uint64_t p_full;              // P of a tile is in shared memory
  uint64_t p_empty;             // ... and the MMAs that read it have finished
  uint64_t o_full;              // every P V has been accumulated
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_vt, const uint16_t *__restrict__ qg,
                       const int64_t *__restrict__ position_ptr, int S, int nh, int nkv, int64_t cap,
                       uint16_t *__restrict__ out, int8_t *__restrict__ q_out, float *__restrict__ s_out,
                       int *__restrict__ error_out, uint32_t spin_limit) {
  extern __shared__ uint8_t raw_smem[];
  uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  uint8_t *q_sm = base;
  uint8_t *stage_sm = base + kQBytes;
  uint8_t *p_sm = stage_sm + kStages * kStageBytes;
  Barriers *bars = reinterpret_cast<Barriers *>(p_sm + kPBytes);
  volatile int *abort_flag = &bars->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y, q0 = blockIdx.x * kQTile;
  const int kvh = h / (nh / nkv);

  if (tid == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->s_full[i], 1);
      mbar_init(&bars->s_empty[i], 4);
    }
    mbar_init(&bars->p_full, 4);
    mbar_init(&bars->p_empty, 1);
    mbar_init(&bars->o_full, 1);
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"(kTmemColumns)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  grid_dependency_sync(); // queries, cache and the transposed values belong to the kernels in front

  const int64_t position = *position_ptr;
  const int rows = min(kQTile, S - q0);
  // keys 0 .. position + q0 + rows - 1 are visible to this tile's last row
  const int tiles = static_cast<int>((position + q0 + rows - 1) / kKeyTile) + 1;
  const int iterations = 2 * tiles;

  if (warp == 0) {
    // ---- loader -----------------------------------------------------------------------------
    if (lane == 0) {
      mbar_expect_tx(&bars->q_full, kQBytes);
      for (int c = 0; c < kChunks; ++c)
        tma_load_2d(q_sm + c * kQChunkBytes, &map_q, h * kHd + c * 64, q0, &bars->q_full);
      int issued = 0;
      for (int i = 0; i < iterations; ++i) {
        const int s = i % kStages;
        if (i >= kStages && !mbar_wait(&bars->empty[s], ((i / kStages) - 1) & 1, abort_flag, spin_limit))
          break;
        const bool second = i >= tiles;
        const int tile = second ? i - tiles : i;
        uint8_t *stage = stage_sm + s * kStageBytes;
        mbar_expect_tx(&bars->full[s], kKBytes + (second ? kVtBytes : 0));
        issued = i + 1;
        for (int c = 0; c < kChunks; ++c)
          tma_load_2d(stage + c * kKChunkBytes, &map_k, c * 64, static_cast<int>(kvh * cap) + tile * kKeyTile, &bars->full[s]);
        if (second)
          tma_load_2d(stage + kKBytes, &map_vt, tile * kKeyTile, kvh * kHd, &bars->full[s]);
      }
      if (*abort_flag) { // copies already requested still write into this CTA's shared memory
        mbar_wait_quiet(&bars->q_full, 0, spin_limit);
        for (int i = max(0, issued - kStages); i < issued; ++i)
          mbar_wait_quiet(&bars->full[i % kStages], (i / kStages) & 1, spin_limit);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue --------------------------------------------------------------------------
    if (lane == 0) {
      bool ok = mbar_wait(&bars->q_full, 0, abort_flag, spin_limit);
      auto issue_scores = [&](int i) {
        const int s = i % kStages, sb = i & 1;
        if (!mbar_wait(&bars->full[s], (i / kStages) & 1, abort_flag, spin_limit))
          return false;
        if (i >= 2 && !mbar_wait(&bars->s_empty[sb], ((i >> 1) - 1) & 1, abort_flag, spin_limit))
          return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(q_sm), k_addr = smem_u32(stage_sm + s * kStageBytes);
        for (int c = 0; c < kChunks; ++c)
          for (int ks = 0; ks < 4; ++ks)
            mma_bf16(tmem_base + sb * kKeyTile, operand_descriptor(q_addr + c * kQChunkBytes + ks * 32),
                     operand_descriptor(k_addr + c * kKChunkBytes + ks * 32), InstructionBf16<kKeyTile>::value, (c | ks) != 0);
        mma_commit(&bars->s_full[sb]);
        if (i < tiles)
          mma_commit(&bars->empty[s]); // pass one: the stage holds nothing else
        return true;
      };
      ok = ok && issue_scores(0);
      for (int i = 0; i < iterations && ok; ++i) {
        if (i + 1 < iterations)
          ok = issue_scores(i + 1);
        if (ok && i >= tiles) {
          const int j = i - tiles, s = i % kStages;
          ok = mbar_wait(&bars->p_full, j & 1, abort_flag, spin_limit);
          if (!ok)
            break;
          tc_fence_after();
          const uint32_t p_addr = smem_u32(p_sm), vt_addr = smem_u32(stage_sm + s * kStageBytes + kKBytes);
          for (int ks = 0; ks < 4; ++ks)
            mma_bf16(tmem_base + kOColumn, operand_descriptor(p_addr + ks * 32), operand_descriptor(vt_addr + ks * 32),
                     InstructionBf16<kHd>::value, (j | ks) != 0);
          mma_commit(&bars->empty[s]);
          mma_commit(&bars->p_empty);
        }
      }
      if (ok)
        mma_commit(&bars->o_full);
    }
  } else {
    // ---- softmax and epilogue: one thread per query row --------------------------------------
    const int quarter = warp & 3; // tensor-memory lanes 32 * quarter .. + 31 (fixed by the warp number)
    const int row = quarter * 32 + lane;
    const int t = q0 + row;
    const int64_t limit = position + t; // the last key this row sees
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    constexpr float kScale = 0.0625f;   // 1 / sqrt(256)
    constexpr float kMasked = -1.0e30f;
    float m = kMasked, l = 0.0f;
    bool ok = true;
    for (int i = 0; i < iterations && ok; ++i) {
      const int sb = i & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->s_full[sb], (i >> 1) & 1, abort_flag, spin_limit));
      if (!ok) // the warp leaves together: the tensor-memory loads are warp-wide
        break;
      tc_fence_after();
      uint32_t lo[32], hi[32];
      tmem_load32(lane_base + sb * kKeyTile, lo);
      tmem_load32(lane_base + sb * kKeyTile + 32, hi);
      tc_fence_before();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&bars->s_empty[sb]);
      const bool second = i >= tiles;
      const int64_t j0 = static_cast<int64_t>(second ? i - tiles : i) * kKeyTile;
      if (!second) {
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          if (j0 + u <= limit)
            m = fmaxf(m, __uint_as_float(lo[u]) * kScale);
          if (j0 + 32 + u <= limit)
            m = fmaxf(m, __uint_as_float(hi[u]) * kScale);
        }
        continue;
      }
      // pass two: weights against the row's final maximum, rounded to bf16; their sum is taken
      // over the rounded values, so that the row is normalised by exactly what multiplies V
      uint32_t packed[32];
#pragma unroll
      for (int u = 0; u < 32; u += 2) {
        const float p0 = j0 + u <= limit ? __expf(__uint_as_float(lo[u]) * kScale - m) : 0.0f;
        const float p1 = j0 + u + 1 <= limit ? __expf(__uint_as_float(lo[u + 1]) * kScale - m) : 0.0f;
        const float p2 = j0 + 32 + u <= limit ? __expf(__uint_as_float(hi[u]) * kScale - m) : 0.0f;
        const float p3 = j0 + 32 + u + 1 <= limit ? __expf(__uint_as_float(hi[u + 1]) * kScale - m) : 0.0f;
        const uint32_t w0 = f32x2_to_bf16x2_hw(p0, p1), w1 = f32x2_to_bf16x2_hw(p2, p3);
        packed[u >> 1] = w0;
        packed[16 + (u >> 1)] = w1;
        l += __uint_as_float(w0 << 16) + __uint_as_float(w0 & 0xffff0000u) + __uint_as_float(w1 << 16) +
             __uint_as_float(w1 & 0xffff0000u);
      }
      const int j = i - tiles;
      if (j >= 1) {
        ok = __all_sync(0xffffffffu, mbar_wait(&bars->p_empty, (j - 1) & 1, abort_flag, spin_limit));
        if (!ok)
          break;
      }
      // row `row` of the P tile: 128 bytes, its 16-byte chunk c at position c ^ (row % 8)
      uint8_t *p_row = p_sm + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4 *>(p_row + ((c ^ (row & 7)) << 4)) =
            make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // visible to the tensor core's reads
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&bars->p_full);
    }
    if (ok)
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full, 0, abort_flag, spin_limit));
    if (ok) {
      tc_fence_after();
      const float inv_l = 1.0f / l;
      const bool valid = t < S;
      const uint16_t *gate = qg + (static_cast<int64_t>(valid ? t : 0) * nh + h) * 2 * kHd + kHd;
      const int64_t index = (static_cast<int64_t>(valid ? t : 0) * nh + h) * kHd;
#pragma unroll 1
      for (int c = 0; c < kHd / 32; ++c) {
        uint32_t acc[32];
        __syncwarp(); // rows past the end skip the arithmetic below but take part in the warp-wide load
        tmem_load32(lane_base + kOColumn + c * 32, acc);
        if (!valid)
          continue;
        uint4 g4[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          g4[u] = reinterpret_cast<const uint4 *>(gate + c * 32)[u];
        const uint32_t *gw = reinterpret_cast<const uint32_t *>(g4);
        float r[32];
        uint32_t words[16];
        float amax = 0.0f;
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const float g0 = __uint_as_float(gw[u] << 16), g1 = __uint_as_float(gw[u] & 0xffff0000u);
          const float v0 = __uint_as_float(acc[2 * u]) * inv_l * (1.0f / (1.0f + __expf(-g0)));
          const float v1 = __uint_as_float(acc[2 * u + 1]) * inv_l * (1.0f / (1.0f + __expf(-g1)));
          words[u] = f32x2_to_bf16x2_hw(v0, v1);
          r[2 * u] = __uint_as_float(words[u] << 16);
          r[2 * u + 1] = __uint_as_float(words[u] & 0xffff0000u);
          amax = fmaxf(amax, fmaxf(fabsf(r[2 * u]), fabsf(r[2 * u + 1])));
        }
        uint4 *dst = reinterpret_cast<uint4 *>(out + index + c * 32);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          dst[u] = make_uint4(words[4 * u], words[4 * u + 1], words[4 * u + 2], words[4 * u + 3]);
        if (q_out) { // the quantisation the following o_proj needs (Q8Decode.cpp:83-120)
          const float scale = __fdiv_rn(amax, 127.0f);
          const float inv = amax == 0.0f ? 0.0f : __fdiv_rn(1.0f, scale);
          uint32_t q[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            uint32_t word = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b)
              word |= (static_cast<uint32_t>(__float2int_rn(__fmul_rn(r[4 * u + b], inv))) & 0xffu) << (8 * b);
            q[u] = word;
          }
          uint4 *qd = reinterpret_cast<uint4 *>(q_out + index + c * 32);
          qd[0] = make_uint4(q[0], q[1], q[2], q[3]);
          qd[1] = make_uint4(q[4], q[5], q[6], q[7]);
          s_out[(index >> 5) + c] = scale;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemColumns) : "memory");
  }
  if (tid == 0 && bars->abort_flag && error_out)
    atomicExch(error_out, 1);
}

// V rows [0, total) of one layer's cache, [nkv][cap][256], transposed into vt [nkv][256][ld] (keys
// contiguous), 64 x 64 tiles through shared memory.  grid (key tiles, 4, nkv), 256 threads.
__global__ void __launch_bounds__(256)
attn_transpose_v_kernel(const uint16_t *__restrict__ v_cache, const int64_t *__restrict__ position_ptr, int S, int64_t cap,
                        int64_t ld, uint16_t *__restrict__ vt) {
  __shared__ uint16_t tile[64][64 + 2];
  grid_dependency_sync();
  const int64_t total = *position_ptr + S;
  const int64_t key0 = static_cast<int64_t>(blockIdx.x) * 64;
  if (key0 >= total)
    return;
  const int d0 = blockIdx.y * 64, kvh = blockIdx.z;
  const uint16_t *src = v_cache + (static_cast<int64_t>(kvh) * cap + key0) * kHd + d0;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int key = i >> 6, d = i & 63;
    tile[key][d] = key0 + key < total ? src[static_cast<int64_t>(key) * kHd + d] : static_cast<uint16_t>(0);
  }
  __syncthreads();
  uint16_t *dst = vt + (static_cast<int64_t>(kvh) * kHd + d0) * ld + key0;
  for (int i = threadIdx.x; i < 64 * 64; i += 256) {
    const int d = i >> 6, key = i & 63;
    dst[static_cast<int64_t>(d) * ld + key] = tile[key][d];
  }
}

bool map_2d(CUtensorMap *map, const void *base, uint64_t cols, uint64_t rows, uint64_t row_bytes, uint32_t box_cols, uint32_t box_rows) {
  EncodeTiled encode = encode_tiled();
  if (!encode)
    return false;
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {row_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

} // namespace

bool attention_prefill_tc_supported(int nh, int nkv, int hd) { return hd == kHd && nkv > 0 && nh % nkv == 0; }

namespace {
int64_t key_pitch(int64_t cap) { return (cap + 63) / 64 * 64; }
size_t queries_bytes(int64_t S, int nh) { return (static_cast<size_t>(S) * nh * kHd * sizeof(uint16_t) + 1023) / 1024 * 1024; }
} // namespace

size_t attention_prefill_tc_scratch_bytes(int64_t S, int nh, int nkv, int64_t cap) {
  return queries_bytes(S, nh) + static_cast<size_t>(nkv) * kHd * static_cast<size_t>(key_pitch(cap)) * sizeof(uint16_t);
}

cudaError_t launch_attention_prefill_tc(const uint16_t *qg, const uint16_t *k, const uint16_t *v, const uint16_t *q_norm,
                                        const uint16_t *k_norm, const float *cos, const float *sin, int rows_from_position,
                                        uint16_t *cache, const int64_t *position_dev, int64_t max_position, int64_t S, int nh,
                                        int nkv, int hd, int rot, int64_t cap, void *scratch, uint16_t *out, int8_t *q_out,
                                        float *s_out, int *error_flag, cudaStream_t stream, uint32_t spin_limit) {
  if (S <= 0 || !attention_prefill_tc_supported(nh, nkv, hd) || S > (1 << 24) || rot % 2 != 0 || rot > hd || max_position + S > cap)
    return cudaErrorInvalidValue;
  if (spin_limit == 0)
    spin_limit = 1u << 26; // about a second
  uint16_t *qn = static_cast<uint16_t *>(scratch);
  uint16_t *vt = reinterpret_cast<uint16_t *>(static_cast<unsigned char *>(scratch) + queries_bytes(S, nh));
  // q/k norms, rotary embedding and the cache rows of the new tokens: the exact path's kernel, tree sums
  if (cudaError_t e = launch_attention_prepare(qg, k, v, q_norm, k_norm, cos, sin, rows_from_position, cache, position_dev, S, nh,
                                               nkv, hd, rot, cap, qn, stream, 1, 0);
      e != cudaSuccess)
    return e;
  const int64_t ld = key_pitch(cap);
  CUtensorMap map_q, map_k, map_vt;
  if (!map_2d(&map_q, qn, static_cast<uint64_t>(nh) * kHd, static_cast<uint64_t>(S), static_cast<uint64_t>(nh) * kHd * 2, 64, kQTile) ||
      !map_2d(&map_k, cache, kHd, static_cast<uint64_t>(nkv) * cap, kHd * 2, 64, kKeyTile) ||
      !map_2d(&map_vt, vt, static_cast<uint64_t>(ld), static_cast<uint64_t>(nkv) * kHd, static_cast<uint64_t>(ld) * 2, 64, kHd))
    return cudaErrorNotSupported;
  if (cudaError_t e = opt_in_shared_memory(reinterpret_cast<const void *>(attn_prefill_tc_kernel), kSmemBytes); e != cudaSuccess)
    return e;
  const uint16_t *v_cache = cache + static_cast<int64_t>(nkv) * cap * kHd;
  launch_chained(attn_transpose_v_kernel, dim3(static_cast<unsigned>(ld / 64), kHd / 64, nkv), dim3(256), 0, stream, v_cache,
                 position_dev, static_cast<int>(S), cap, ld, vt);
  launch_chained(attn_prefill_tc_kernel, dim3(static_cast<unsigned>((S + kQTile - 1) / kQTile), nh), dim3(kThreads), kSmemBytes, stream,
                 map_q, map_k, map_vt, qg, position_dev, static_cast<int>(S), nh, nkv, cap, out, q_out, s_out, error_flag, spin_limit);
  return cudaGetLastError();
}

} // namespace llmcp_b200
