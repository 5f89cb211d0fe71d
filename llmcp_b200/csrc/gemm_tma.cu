// Prefill GEMM (M > 1) on the fifth-generation tensor cores, operands fetched by TMA.
// Q8Matmul.cpp:143-289.
//
//   y[m, n] = act( chain_kb fma(float(dot_kb[m, n]), a_scale[m, kb] * w_scale[n, kb], acc) ),
//   dot_kb = sum of 32 int8 products.
//
// The per-block f32 chain is what bounds this GEMM: it runs on the CUDA cores, once per (row,
// column, 32-block), while the tensor core needs a fraction of that time for the block's dots.
// Two operand forms are implemented on one pipeline:
//   int8: the int8 planes the GEMV streams, tcgen05.mma kind::i8 (K = 32 = one quantisation block per
//         instruction), int32 dots, convert + multiply + fma per element in the epilogue;
//   f16 : the same integers held as f16 values (every integer up to 2048 is exact in f16), kind::f16
//         with f32 accumulation: a product is an integer below 2^14, a block's sum an integer below
//         2^19, both exact in f32, so the tensor core hands back float(dot) itself, bit for bit what
//         the conversion would give, and the epilogue is multiply + fma.  The price is operand planes
//         of twice the size in HBM and on the way from L2.
// Either form optionally with two-lane f32x2 multiplies and fmas (same roundings, half the
// instructions).  Measured on 1024 x 9216 x 2560: int8 199 us, int8 packed 177 us, f16 191 us,
// f16 packed 181 us (the cp.async-fed kernel of gemm_tc.cu: 222 us); what remains is the epilogue
// warps' instruction issue and the hand-off per block, not the tensor pipe (under 10 % busy).
//
// One CTA per 128 x 128 output tile, 576 threads:
//   warp  0     one lane issues the TMA loads (cp.async.bulk.tensor, 128-byte swizzle, no
//               multicast): per stage a box of 128 rows x 128 bytes of K of each operand (four
//               int8 or two f16 quantisation blocks) and those blocks' f32 scales of the tile's rows
//               and columns (scale planes are block-major, [K/32][rows], so a box is 128 consecutive
//               floats per block);
//   warp  1     one lane issues the MMAs into tensor-memory buffer kb % 4 (f16: two K = 16
//               instructions per block, the first overwrites, the second accumulates);
//   warps 2-17  epilogue: tcgen05.ld the buffer (thread = row, 32 columns), hand the buffer back,
//               then the arithmetic with the scales read from shared memory.
// Hand-offs are mbarriers; every wait is bounded (spin_limit polls) and a timed-out wait raises an
// abort flag that all roles observe, so a protocol error ends the kernel with an error code instead
// of hanging it; the loader then waits (bounded) for the copies it has in flight.  Tensor memory
// (512 columns) is allocated by warp 0 and always released.

#include <cuda.h>
#include <cuda_fp16.h>

#include <mutex>

#include "kernels.h"
#include "tc_common.cuh"

namespace llmcp_b200 {

namespace {

using namespace tc;

constexpr int kTileM = 128;
// Output tiles are 128 rows by TN columns, TN = 128 (four tensor-memory buffers) or 160 (three): the
// wider tile exists for matrices whose 128-wide tiles would leave a nearly empty last wave (N = 2560 at
// 1024 rows: 160 tiles on 148 SMs, against 128 tiles of 160 columns in one wave).
template <int TN> struct Tile {
  static_assert(TN == 128 || TN == 160, "tile widths with a tensor-memory plan");
  static constexpr int kBuffers = TN == 128 ? 4 : 3;  // TN columns of 32-bit accumulators each, 512 in all
  static constexpr int kStages = TN == 128 ? 6 : 5;
  static constexpr int kWarpColumns = TN / 4;         // columns per epilogue warp: 32, or 32 + 8
  static constexpr int kOperandBytesB = TN * 128;
};
constexpr int kMaxBuffers = 4, kMaxStages = 6;
constexpr int kEpilogueWarp0 = 2;
constexpr int kEpilogueWarps = 16;
constexpr int kThreads = 32 * (kEpilogueWarp0 + kEpilogueWarps);
constexpr int kOperandBytes = kTileM * 128;  // 16 KB per operand per stage: rows of 128 bytes of K
constexpr int kBarrierBytes = 256;

// F16: operands are f16 values (64 per 128-byte row = 2 quantisation blocks per stage);
// otherwise int8 (128 per row = 4 blocks per stage).
template <bool F16, int TN = 128> struct Form {
  static constexpr int kStageBlocks = F16 ? 2 : 4;
  static constexpr int kStageK = kStageBlocks * 32;                 // elements of K per stage
  static constexpr int kScaleBytesA = kStageBlocks * kTileM * 4;    // the rows' scales of a stage
  static constexpr int kScaleBytesB = kStageBlocks * TN * 4;        // the columns' scales
  static constexpr int kScaleBytes = (kScaleBytesA + kScaleBytesB + 1023) / 1024 * 1024;
  static constexpr int kStageBytes = kOperandBytes + Tile<TN>::kOperandBytesB + kScaleBytes; // multiples of 1024
  static constexpr size_t kSmemBytes = 1024 + Tile<TN>::kStages * kStageBytes + kBarrierBytes;
};

// kind::f16: f16 x f16 -> f32, both operands K-major, M = 128, N = TN, K = 16 per instruction.
// kind::i8: s8 x s8 -> s32, both operands K-major, M = 128, N = TN, K = 32 per instruction.
template <int TN> struct Instruction {
  static constexpr uint32_t kF16 = (1u << 4) | ((TN >> 3) << 17) | ((kTileM >> 4) << 24);
  static constexpr uint32_t kI8 = (2u << 4) | (1u << 7) | (1u << 10) | ((TN >> 3) << 17) | ((kTileM >> 4) << 24);
};

__device__ __forceinline__ void mma_f16(uint32_t tmem, uint64_t a, uint64_t b, uint32_t accumulate, uint32_t kInstructionF16) {
  asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p; }"
               :
               : "r"(tmem), "l"(a), "l"(b), "r"(kInstructionF16), "r"(accumulate), "r"(0u)
               : "memory");
}

__device__ __forceinline__ void mma_i8(uint32_t tmem, uint64_t a, uint64_t b, uint32_t kInstructionI8) {
  asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p; }"
               :
               : "r"(tmem), "l"(a), "l"(b), "r"(kInstructionI8), "r"(0u), "r"(0u)
               : "memory");
}

// Two f32 lanes per instruction (each lane rounds as the scalar instruction does).
__device__ __forceinline__ void mul2(float &d0, float &d1, float a0, float a1, float b0, float b1) {
  asm("{ .reg .b64 a, b, d; mov.b64 a, {%2, %3}; mov.b64 b, {%4, %5}; mul.rn.f32x2 d, a, b; mov.b64 {%0, %1}, d; }"
      : "=f"(d0), "=f"(d1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
__device__ __forceinline__ void fma2(float &c0, float &c1, float a0, float a1, float b0, float b1) {
  asm("{ .reg .b64 a, b, c; mov.b64 a, {%2, %3}; mov.b64 b, {%4, %5}; mov.b64 c, {%0, %1}; fma.rn.f32x2 c, a, b, c; mov.b64 {%0, %1}, c; }"
      : "+f"(c0), "+f"(c1)
      : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}

struct Barriers {
  uint64_t full[kMaxStages];     // stage landed in shared memory (one arrival + the copies' bytes)
  uint64_t empty[kMaxStages];    // stage no longer needed: MMA done (1) + every epilogue warp (scales read)
  uint64_t tfull[kMaxBuffers];   // a block's dot products are in the tensor-memory buffer
  uint64_t tempty[kMaxBuffers];  // the buffer has been read by all epilogue warps
  uint64_t done;                 // the last commit of the MMA lane has arrived (see the end of its loop)
  uint32_t tmem_base;
  int abort_flag;
};

// fault (test hook): 1 = the loader announces the first stage's bytes but never issues its copies,
// so the barrier of that stage cannot complete and every wait behind it has to run out.
// PACKED: the epilogue's multiplies and fmas as two-lane f32x2 instructions (same roundings).
template <bool F16, bool PACKED, bool DOTS, int TN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_q8_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_as, const __grid_constant__ CUtensorMap map_bs, int M, int K,
                    int N, void *__restrict__ y, int y_dtype, int activation, int32_t *__restrict__ dots_out,
                    int *__restrict__ error_out, uint32_t spin_limit, int fault) {
  using F = Form<F16, TN>;
  constexpr int kStageBlocks = F::kStageBlocks, kStageK = F::kStageK, kStageBytes = F::kStageBytes;
  constexpr int kTileN = TN, kTmemBuffers = Tile<TN>::kBuffers, kStages = Tile<TN>::kStages, kWarpColumns = Tile<TN>::kWarpColumns;
  constexpr int kOperandBytesB = Tile<TN>::kOperandBytesB;
  extern __shared__ uint8_t raw_smem[];
  uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  Barriers *bars = reinterpret_cast<Barriers *>(base + kStages * kStageBytes);
  volatile int *abort_flag = &bars->abort_flag;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nb = K / kBlock;
  const int iters = (nb + kStageBlocks - 1) / kStageBlocks;
  const int m0 = blockIdx.y * kTileM, n0 = blockIdx.x * kTileN;

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1 + kEpilogueWarps);
    }
    for (int i = 0; i < kTmemBuffers; ++i) {
      mbar_init(&bars->tfull[i], 1);
      mbar_init(&bars->tempty[i], kEpilogueWarps);
    }
    mbar_init(&bars->done, 1);
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"(512)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  grid_dependency_sync(); // barriers and tensor memory are set up; the operands belong to the kernel in front

  if (warp == 0) {
    // ---- loader ---------------------------------------------------------------------------
    if (lane == 0) {
      int issued = 0;
      for (int it = 0; it < iters; ++it) {
        const int s = it % kStages;
        if (it >= kStages && !mbar_wait(&bars->empty[s], ((it / kStages) - 1) & 1, abort_flag, spin_limit))
          break;
        uint8_t *stage = base + s * kStageBytes;
        mbar_expect_tx(&bars->full[s], kOperandBytes + kOperandBytesB + F::kScaleBytesA + F::kScaleBytesB);
        issued = it + 1;
        if (fault == 1 && it == 0)
          continue;
        const int k0 = it * kStageK, kb0 = it * kStageBlocks;
        tma_load_2d(stage, &map_a, k0, m0, &bars->full[s]);
        tma_load_2d(stage + kOperandBytes, &map_b, k0, n0, &bars->full[s]);
        tma_load_2d(stage + kOperandBytes + kOperandBytesB, &map_as, m0, kb0, &bars->full[s]);
        tma_load_2d(stage + kOperandBytes + kOperandBytesB + F::kScaleBytesA, &map_bs, n0, kb0, &bars->full[s]);
      }
      // Leaving after a failed wait: the copies already requested still write into this CTA's
      // shared memory, so each of them gets one more bounded wait before the CTA may exit.
      if (*abort_flag) {
        for (int it = max(0, issued - kStages); it < issued; ++it)
          if (!(fault == 1 && it == 0))
            mbar_wait_quiet(&bars->full[it % kStages], (it / kStages) & 1, spin_limit);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issue ------------------------------------------------------------------------
    if (lane == 0) {
      bool ok = true;
      for (int it = 0; it < iters && ok; ++it) {
        const int s = it % kStages;
        ok = mbar_wait(&bars->full[s], (it / kStages) & 1, abort_flag, spin_limit);
        if (!ok)
          break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(base + s * kStageBytes), b_addr = a_addr + kOperandBytes;
        const int blocks = min(kStageBlocks, nb - it * kStageBlocks);
        for (int j = 0; j < blocks; ++j) {
          const int kb = it * kStageBlocks + j;
          const int buf = kb % kTmemBuffers, use = kb / kTmemBuffers;
          if (use > 0) {
            ok = mbar_wait(&bars->tempty[buf], (use - 1) & 1, abort_flag, spin_limit);
            if (!ok)
              break;
            tc_fence_after();
          }
          const uint32_t d = tmem_base + buf * kTileN;
          if (F16) { // two K = 16 instructions per block: the first overwrites, the second accumulates
            mma_f16(d, operand_descriptor(a_addr + j * 64), operand_descriptor(b_addr + j * 64), 0u, Instruction<TN>::kF16);
            mma_f16(d, operand_descriptor(a_addr + j * 64 + 32), operand_descriptor(b_addr + j * 64 + 32), 1u, Instruction<TN>::kF16);
          } else {
            mma_i8(d, operand_descriptor(a_addr + j * 32), operand_descriptor(b_addr + j * 32), Instruction<TN>::kI8);
          }
          mma_commit(&bars->tfull[buf]);
        }
        mma_commit(&bars->empty[s]);
      }
      // A commit's arrival is asynchronous, and nothing else waits for the last ones on `empty`: the
      // CTA must not end (and hand its shared memory to the next CTA on this SM, possibly of another
      // kernel with its barriers elsewhere) while an arrival is still on its way.  Commits arrive in
      // order, so seeing this one means all have.
      mma_commit(&bars->done);
      mbar_wait_quiet(&bars->done, 0, spin_limit);
    }
  } else {
    // ---- epilogue ---------------------------------------------------------------------------
    const int quarter = warp & 3;                  // tensor-memory lanes 32*quarter .. +31 (fixed by the warp number)
    const int colq = (warp - kEpilogueWarp0) >> 2; // columns kWarpColumns * colq .. + kWarpColumns - 1
    const int row = quarter * 32 + lane;
    const int gm = m0 + row;
    float acc[kWarpColumns];
#pragma unroll
    for (int c = 0; c < kWarpColumns; ++c)
      acc[c] = 0.0f;
    bool ok = true;
    for (int kb = 0; kb < nb && ok; ++kb) {
      const int buf = kb % kTmemBuffers;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->tfull[buf], (kb / kTmemBuffers) & 1, abort_flag, spin_limit));
      if (!ok) // the whole warp leaves together: the tensor-memory loads below are warp-wide
        break;
      tc_fence_after();
      const int it = kb / kStageBlocks, s = it % kStages, j = kb % kStageBlocks;
      // The stage's scales arrived with the operands; observing the stage's own barrier (long
      // complete by now) is what makes the copied bytes visible to these loads.
      if (j == 0 && !__all_sync(0xffffffffu, mbar_wait(&bars->full[s], (it / kStages) & 1, abort_flag, spin_limit))) {
        ok = false;
        break;
      }
      const float *scales = reinterpret_cast<const float *>(base + s * kStageBytes + kOperandBytes + kOperandBytesB);
      const float a_scale = scales[j * kTileM + row];
      const float4 *w_scale = reinterpret_cast<const float4 *>(scales + kStageBlocks * kTileM + j * kTileN + colq * kWarpColumns);
      uint32_t raw[kWarpColumns];
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kTileN + colq * kWarpColumns;
      if (kWarpColumns == 32) {
        tmem_load32(taddr, *reinterpret_cast<uint32_t(*)[32]>(raw));
      } else { // 32 + 8 columns, one wait for both loads
        tmem_issue32(taddr, *reinterpret_cast<uint32_t(*)[32]>(raw));
        tmem_issue8(taddr + 32, *reinterpret_cast<uint32_t(*)[8]>(raw + 32));
        tmem_wait_loads();
      }
      // The buffer is handed back before any arithmetic, so that the MMA of a later block can
      // reuse it while this one is still being folded in.
      tc_fence_before();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&bars->tempty[buf]);
      float v[kWarpColumns];
#pragma unroll
      for (int u = 0; u < kWarpColumns; ++u)
        v[u] = F16 ? __uint_as_float(raw[u]) : __int2float_rn(static_cast<int>(raw[u]));
#pragma unroll
      for (int g = 0; g < kWarpColumns / 4; ++g) {
        const float4 w4 = w_scale[g];
        if (PACKED) {
          float f0, f1, f2, f3;
          mul2(f0, f1, a_scale, a_scale, w4.x, w4.y);
          mul2(f2, f3, a_scale, a_scale, w4.z, w4.w);
          fma2(acc[g * 4 + 0], acc[g * 4 + 1], v[g * 4 + 0], v[g * 4 + 1], f0, f1);
          fma2(acc[g * 4 + 2], acc[g * 4 + 3], v[g * 4 + 2], v[g * 4 + 3], f2, f3);
        } else {
          acc[g * 4 + 0] = __fmaf_rn(v[g * 4 + 0], __fmul_rn(a_scale, w4.x), acc[g * 4 + 0]);
          acc[g * 4 + 1] = __fmaf_rn(v[g * 4 + 1], __fmul_rn(a_scale, w4.y), acc[g * 4 + 1]);
          acc[g * 4 + 2] = __fmaf_rn(v[g * 4 + 2], __fmul_rn(a_scale, w4.z), acc[g * 4 + 2]);
          acc[g * 4 + 3] = __fmaf_rn(v[g * 4 + 3], __fmul_rn(a_scale, w4.w), acc[g * 4 + 3]);
        }
      }
      if (DOTS) {
        if (gm < M) {
#pragma unroll
          for (int u = 0; u < kWarpColumns; ++u) {
            const int gn = n0 + colq * kWarpColumns + u;
            if (gn < N)
              dots_out[(static_cast<size_t>(gm) * N + gn) * nb + kb] = F16 ? __float2int_rn(v[u]) : static_cast<int>(raw[u]);
          }
        }
      }
      if (j == kStageBlocks - 1 || kb == nb - 1) { // done with this stage's scales
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&bars->empty[s]);
      }
    }
    if (ok && gm < M) {
#pragma unroll
      for (int g = 0; g < kWarpColumns / 8; ++g) {
        const int gn = n0 + colq * kWarpColumns + g * 8;
        if (gn < N) { // N is a multiple of 8, so a group of eight is entirely inside or outside
          float o[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            o[u] = apply_activation(acc[g * 8 + u], activation);
          if (y_dtype == kBF16) {
            uint32_t packed[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
              packed[u] = static_cast<uint32_t>(f32_to_bf16(o[2 * u])) | (static_cast<uint32_t>(f32_to_bf16(o[2 * u + 1])) << 16);
            *reinterpret_cast<uint4 *>(static_cast<uint16_t *>(y) + static_cast<size_t>(gm) * N + gn) =
                make_uint4(packed[0], packed[1], packed[2], packed[3]);
          } else {
            float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(y) + static_cast<size_t>(gm) * N + gn);
            dst[0] = make_float4(o[0], o[1], o[2], o[3]);
            dst[1] = make_float4(o[4], o[5], o[6], o[7]);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
  }
  if (tid == 0 && bars->abort_flag && error_out)
    atomicExch(error_out, 1);
}

// int8 activations and their [M][K/32] scales -> f16 values [M][K] and block-major scales
// [K/32][ld] (ld = M rounded up to 4, the row pitch a tensor map needs).
__global__ void act_to_f16_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as, int64_t M, int K, int64_t ld,
                                  __half *__restrict__ ah, float *__restrict__ ast) {
  grid_dependency_sync();
  const int64_t words = M * (K / 4);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int nb = K / kBlock;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < words; i += stride) {
    const uint32_t v = reinterpret_cast<const uint32_t *>(aq)[i];
    const __half2 lo = __halves2half2(__int2half_rn(static_cast<int8_t>(v & 0xff)), __int2half_rn(static_cast<int8_t>((v >> 8) & 0xff)));
    const __half2 hi = __halves2half2(__int2half_rn(static_cast<int8_t>((v >> 16) & 0xff)), __int2half_rn(static_cast<int8_t>(v >> 24)));
    reinterpret_cast<uint2 *>(ah)[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
    if (i < M * nb) { // the first M * nb threads also move one scale each
      const int64_t m = i / nb, b = i % nb;
      ast[b * ld + m] = as[i];
    }
  }
}

// The weight planes of the same form, made once at load from the int8 / f16-scale planes.
__global__ void weights_to_f16_kernel(const int8_t *__restrict__ wq, const uint16_t *__restrict__ wd, int64_t N, int K,
                                      __half *__restrict__ wh, float *__restrict__ wst) {
  grid_dependency_sync();
  const int64_t words = N * (K / 4);
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  const int nb = K / kBlock;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < words; i += stride) {
    const uint32_t v = reinterpret_cast<const uint32_t *>(wq)[i];
    const __half2 lo = __halves2half2(__int2half_rn(static_cast<int8_t>(v & 0xff)), __int2half_rn(static_cast<int8_t>((v >> 8) & 0xff)));
    const __half2 hi = __halves2half2(__int2half_rn(static_cast<int8_t>((v >> 16) & 0xff)), __int2half_rn(static_cast<int8_t>(v >> 24)));
    reinterpret_cast<uint2 *>(wh)[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
    if (i < N * nb) {
      const int64_t n = i / nb, b = i % nb;
      wst[b * N + n] = f16_bits_to_f32(wd[i]);
    }
  }
}

// rows x K operand plane, K contiguous: boxes of 128 rows x 128 bytes of K (64 f16 or 128 int8),
// 128-byte swizzle; out-of-range parts read as zero.
bool operand_map(CUtensorMap *map, const void *plane, int64_t rows, int K, bool f16, int box_rows = kTileM) {
  EncodeTiled encode = encode_tiled();
  if (!encode)
    return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * (f16 ? 2 : 1)};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(f16 ? 64 : 128), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return encode(map, f16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(plane), dims,
                strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// nb x ld f32, block-major: boxes of a stage's blocks x 128 entries.
bool scale_map(CUtensorMap *map, const void *plane, int64_t entries, int64_t ld, int nb, int stage_blocks, int box_entries = kTileM) {
  EncodeTiled encode = encode_tiled();
  if (!encode)
    return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(entries), static_cast<cuuint64_t>(nb)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 4};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_entries), static_cast<cuuint32_t>(stage_blocks)};
  const cuuint32_t elem[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void *>(plane), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <bool F16, bool PACKED, int TN>
cudaError_t launch_tile(const void *a, const float *ast, int M, int K, const void *w, const float *wst, int N, void *y,
                        int y_dtype, int activation, int32_t *dots_out, int *error_flag, cudaStream_t stream, uint32_t spin_limit,
                        int fault) {
  using F = Form<F16, TN>;
  const int nb = K / kBlock;
  CUtensorMap map_a, map_b, map_as, map_bs;
  if (!operand_map(&map_a, a, M, K, F16) || !operand_map(&map_b, w, N, K, F16, TN) ||
      !scale_map(&map_as, ast, M, gemm_tc16_scale_pitch(M), nb, F::kStageBlocks) ||
      !scale_map(&map_bs, wst, N, N, nb, F::kStageBlocks, TN))
    return cudaErrorNotSupported;
  const void *kernel = dots_out ? reinterpret_cast<const void *>(gemm_q8_tma_kernel<F16, PACKED, true, TN>)
                                : reinterpret_cast<const void *>(gemm_q8_tma_kernel<F16, PACKED, false, TN>);
  if (cudaError_t e = opt_in_shared_memory(kernel, F::kSmemBytes); e != cudaSuccess)
    return e;
  dim3 grid((N + TN - 1) / TN, (M + kTileM - 1) / kTileM);
  if (dots_out)
    launch_chained(gemm_q8_tma_kernel<F16, PACKED, true, TN>, grid, dim3(kThreads), F::kSmemBytes, stream, map_a, map_b, map_as,
                   map_bs, M, K, N, y, y_dtype, activation, dots_out, error_flag, spin_limit, fault);
  else
    launch_chained(gemm_q8_tma_kernel<F16, PACKED, false, TN>, grid, dim3(kThreads), F::kSmemBytes, stream, map_a, map_b, map_as,
                   map_bs, M, K, N, y, y_dtype, activation, dots_out, error_flag, spin_limit, fault);
  return cudaGetLastError();
}

// Tile width for an M x N output: every wave of tiles costs about the same whatever it holds, a
// 160-wide tile a quarter more than a 128-wide one; LLMCP_B200_GEMM_TILE=128|160 overrides.
int choose_tile(int M, int N) {
  const char *flag = std::getenv("LLMCP_B200_GEMM_TILE");
  const int forced = flag ? std::atoi(flag) : 0;
  if (forced == 128 || forced == 160)
    return forced;
  int sm_count = 148;
  if (current_sm_count(&sm_count) != cudaSuccess || sm_count <= 0)
    sm_count = 148;
  const int64_t sms = sm_count;
  const int64_t rows = (M + kTileM - 1) / kTileM;
  const int64_t waves128 = (rows * ((N + 127) / 128) + sms - 1) / sms, waves160 = (rows * ((N + 159) / 160) + sms - 1) / sms;
  return waves160 * 5 < waves128 * 4 ? 160 : 128;
}

template <bool F16, bool PACKED>
cudaError_t launch_form(const void *a, const float *ast, int M, int K, const void *w, const float *wst, int N, void *y,
                        int y_dtype, int activation, int32_t *dots_out, int *error_flag, cudaStream_t stream, uint32_t spin_limit,
                        int fault) {
  if (choose_tile(M, N) == 160)
    return launch_tile<F16, PACKED, 160>(a, ast, M, K, w, wst, N, y, y_dtype, activation, dots_out, error_flag, stream, spin_limit, fault);
  return launch_tile<F16, PACKED, 128>(a, ast, M, K, w, wst, N, y, y_dtype, activation, dots_out, error_flag, stream, spin_limit, fault);
}

// [rows][K/32] scales -> block-major f32 [K/32][ld]; scales are f32 (activations) or f16 bits (weights).
__global__ void scales_block_major_kernel(const void *__restrict__ scales, int scales_are_f16, int64_t rows, int nb, int64_t ld,
                                          float *__restrict__ out) {
  grid_dependency_sync();
  const int64_t total = rows * nb;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / nb, b = i % nb;
    out[b * ld + r] = scales_are_f16 ? f16_bits_to_f32(static_cast<const uint16_t *>(scales)[i]) : static_cast<const float *>(scales)[i];
  }
}

} // namespace

int64_t gemm_tc16_scale_pitch(int64_t M) { return (M + 3) / 4 * 4; }

void launch_act_to_f16(const int8_t *aq, const float *as, int64_t M, int K, void *ah, float *ast, cudaStream_t stream) {
  const int64_t words = M * (K / 4);
  const int blocks = static_cast<int>(std::min<int64_t>((words + 255) / 256, 148 * 16));
  launch_chained(act_to_f16_kernel, dim3(blocks), dim3(256), 0, stream, aq, as, M, K, gemm_tc16_scale_pitch(M),
                 static_cast<__half *>(ah), ast);
}

void launch_weights_to_f16(const int8_t *wq, const uint16_t *wd, int64_t N, int K, void *wh, float *wst, cudaStream_t stream) {
  const int64_t words = N * (K / 4);
  const int blocks = static_cast<int>(std::min<int64_t>((words + 255) / 256, 148 * 16));
  launch_chained(weights_to_f16_kernel, dim3(blocks), dim3(256), 0, stream, wq, wd, N, K, static_cast<__half *>(wh), wst);
}

void launch_scales_block_major(const void *scales, int scales_are_f16, int64_t rows, int K, int64_t ld, float *out,
                               cudaStream_t stream) {
  const int nb = K / kBlock;
  const int blocks = static_cast<int>(std::min<int64_t>((rows * nb + 255) / 256, 148 * 8));
  launch_chained(scales_block_major_kernel, dim3(blocks), dim3(256), 0, stream, scales, scales_are_f16, rows, nb, ld, out);
}

cudaError_t launch_gemm_q8_tma(int form, const void *a, const float *ast, int M, int K, const void *w, const float *wst, int N,
                               void *y, int y_dtype, int activation, int32_t *dots_out, int *error_flag, cudaStream_t stream,
                               uint32_t spin_limit, int fault) {
  if (M <= 0 || N % 8 != 0 || K % kBlock != 0)
    return cudaErrorInvalidValue;
  if (spin_limit == 0)
    spin_limit = 1u << 26; // about a second
  switch (form) {
  case kGemmF16:
    return launch_form<true, false>(a, ast, M, K, w, wst, N, y, y_dtype, activation, dots_out, error_flag, stream, spin_limit, fault);
  case kGemmF16Packed:
    return launch_form<true, true>(a, ast, M, K, w, wst, N, y, y_dtype, activation, dots_out, error_flag, stream, spin_limit, fault);
  case kGemmI8:
    return launch_form<false, false>(a, ast, M, K, w, wst, N, y, y_dtype, activation, dots_out, error_flag, stream, spin_limit, fault);
  case kGemmI8Packed:
    return launch_form<false, true>(a, ast, M, K, w, wst, N, y, y_dtype, activation, dots_out, error_flag, stream, spin_limit, fault);
  default:
    return cudaErrorInvalidValue;
  }
}

} // namespace llmcp_b200
