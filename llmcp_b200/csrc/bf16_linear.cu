// linear / lm_head / embedding on bf16 weights: the path of an unquantised arena (`llmcp-pack --quant
// none`), MatmulLoweringCommon.cpp:186-251,509-527 and LowerToLinalg.cpp:435-531.
//
//   y[m, n] = act( sum_k f32(x[m, k]) * f32(w[n, k]) )   in f32, rounded to the output type.
//
// The reference's lowerings of this sum differ by target (BFDOT pairs on aarch64, 32-lane ordered
// tiles elsewhere) and its own tests hold it to a tolerance, so there is no operation order to
// reproduce bit for bit; the products of bf16 values are exact in f32 and only the order of the f32
// additions differs between implementations.
//   one row   : gemv_bf16_kernel, a warp per group of four weight rows, 16-byte streaming loads, the
//               input row as f32 in shared memory, lane partial sums and a shuffle tree;
//   many rows : gemm_bf16_tc_kernel, tcgen05.mma kind::f16 on bf16 operands, 128 x 128 tiles, K in
//               slices of 64 (128-byte swizzled rows) fetched by TMA into a six-stage ring, one f32
//               accumulator tile in tensor memory, epilogue by four warps.  Bounded waits as in the
//               other tensor-core kernels.

#include "kernels.h"
#include "tc_common.cuh"

namespace llmcp_b200 {

namespace {

using namespace tc;

constexpr int kGemvRows = 4;
constexpr int kGemvThreads = 256;

struct Words8 {
  uint32_t v[8];
};

// 32 bytes (16 bf16 weights), streamed: not kept in L1, first to leave L2.
__device__ __forceinline__ Words8 ld_stream_32(const void *p) {
  Words8 r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7])
               : "l"(p));
  return r;
}

__device__ __forceinline__ float dot16(const Words8 &w, const float *x) {
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    acc = __fmaf_rn(__uint_as_float(w.v[i] << 16), x[2 * i], acc);
    acc = __fmaf_rn(__uint_as_float(w.v[i] & 0xffff0000u), x[2 * i + 1], acc);
  }
  return acc;
}

// K % 16 == 0; lanes past the row's end skip.  N need not be a multiple of four.
__global__ void __launch_bounds__(kGemvThreads)
gemv_bf16_kernel(const uint16_t *__restrict__ x, int K, const uint16_t *__restrict__ w, int64_t N, void *__restrict__ y,
                 int y_dtype, int activation) {
  extern __shared__ __align__(16) float x_sm[]; // the input row as f32
  grid_dependency_sync();
  for (int k = threadIdx.x; k < K; k += kGemvThreads)
    x_sm[k] = bf16_to_f32(x[k]);
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int64_t warp = blockIdx.x * static_cast<int64_t>(kGemvThreads / 32) + (threadIdx.x >> 5);
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (kGemvThreads / 32);
  for (int64_t row0 = warp * kGemvRows; row0 < N; row0 += warps * kGemvRows) {
    float acc[kGemvRows];
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r)
      acc[r] = 0.0f;
    for (int k0 = lane * 16; k0 < K; k0 += 512) {
      Words8 wv[kGemvRows];
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r) // a row past the end re-reads the last one; its sum is dropped
        wv[r] = ld_stream_32(w + min(row0 + r, N - 1) * K + k0);
      float xv[16];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        *reinterpret_cast<float4 *>(xv + 4 * u) = *reinterpret_cast<const float4 *>(x_sm + k0 + 4 * u);
#pragma unroll
      for (int r = 0; r < kGemvRows; ++r)
        acc[r] += dot16(wv[r], xv);
    }
#pragma unroll
    for (int r = 0; r < kGemvRows; ++r) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], o);
      if (lane == 0 && row0 + r < N)
        store_from_f32(y, y_dtype, row0 + r, apply_activation(acc[r], activation));
    }
  }
}

// Rows `tokens[s]` of a bf16 table [vocab][H]; ids outside the table give a zero row and raise
// bit 2 of *status (as embedding_q8_kernel does).
__global__ void embedding_bf16_kernel(const int64_t *__restrict__ tokens, int64_t S, int H, int64_t vocab,
                                      const uint16_t *__restrict__ table, uint16_t *__restrict__ out, int *__restrict__ status) {
  grid_dependency_sync();
  const int64_t s = blockIdx.x;
  const int64_t token = tokens[s];
  const bool inside = token >= 0 && token < vocab;
  if (!inside && threadIdx.x == 0 && status)
    atomicOr(status, 4);
  for (int c = threadIdx.x; c < H; c += blockDim.x)
    out[s * H + c] = inside ? table[token * H + c] : static_cast<uint16_t>(0);
}

constexpr int kTile = 128;                 // rows and columns of an output tile
constexpr int kSliceBytes = kTile * 128;   // 16 KB: 128 rows x 64 bf16 of K
constexpr int kStages = 6;
constexpr int kStageBytes = 2 * kSliceBytes;
constexpr int kGemmThreads = 192;          // loader, MMA issue, four epilogue warps
constexpr int kGemmSmemBytes = 1024 + kStages * kStageBytes + 256;
// kind::f16, bf16 operands, f32 accumulation, both operands K-major, M = N = 128.
constexpr uint32_t kInstruction = (1u << 4) | (1u << 7) | (1u << 10) | ((kTile >> 3) << 17) | ((kTile >> 4) << 24);

struct GemmBarriers {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t done; // every MMA of the tile has finished
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void mma_bf16_tile(uint32_t tmem, uint64_t a, uint64_t b, uint32_t accumulate) {
  asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p; }"
               :
               : "r"(tmem), "l"(a), "l"(b), "r"(kInstruction), "r"(accumulate), "r"(0u)
               : "memory");
}

__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, int M, int K, int N,
                    void *__restrict__ y, int y_dtype, int activation, int *__restrict__ error_out, uint32_t spin_limit) {
  extern __shared__ uint8_t raw_smem[];
  uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
  GemmBarriers *bars = reinterpret_cast<GemmBarriers *>(base + kStages * kStageBytes);
  volatile int *abort_flag = &bars->abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
  const int slices = (K + 63) / 64; // a partial last slice reads zeros beyond K

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&bars->full[i], 1);
      mbar_init(&bars->empty[i], 1);
    }
    mbar_init(&bars->done, 1);
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)), "r"(kTile)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  grid_dependency_sync(); // the activations belong to the kernel in front

  if (warp == 0) {
    if (lane == 0) {
      int issued = 0;
      for (int it = 0; it < slices; ++it) {
        const int s = it % kStages;
        if (it >= kStages && !mbar_wait(&bars->empty[s], ((it / kStages) - 1) & 1, abort_flag, spin_limit))
          break;
        mbar_expect_tx(&bars->full[s], kStageBytes);
        issued = it + 1;
        tma_load_2d(base + s * kStageBytes, &map_x, it * 64, m0, &bars->full[s]);
        tma_load_2d(base + s * kStageBytes + kSliceBytes, &map_w, it * 64, n0, &bars->full[s]);
      }
      if (*abort_flag) // copies already requested still write into this CTA's shared memory
        for (int it = max(0, issued - kStages); it < issued; ++it)
          mbar_wait_quiet(&bars->full[it % kStages], (it / kStages) & 1, spin_limit);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      bool ok = true;
      for (int it = 0; it < slices && ok; ++it) {
        const int s = it % kStages;
        ok = mbar_wait(&bars->full[s], (it / kStages) & 1, abort_flag, spin_limit);
        if (!ok)
          break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(base + s * kStageBytes), b_addr = a_addr + kSliceBytes;
        for (int ks = 0; ks < 4; ++ks) // four K = 16 steps of 32 bytes inside the swizzled 128-byte rows
          mma_bf16_tile(tmem_base, operand_descriptor(a_addr + ks * 32), operand_descriptor(b_addr + ks * 32), (it | ks) != 0);
        mma_commit(&bars->empty[s]);
      }
      if (ok)
        mma_commit(&bars->done);
    }
  } else {
    const int quarter = warp & 3; // tensor-memory lanes 32 * quarter .. + 31 (fixed by the warp number)
    const int gm = m0 + quarter * 32 + lane;
    if (__all_sync(0xffffffffu, mbar_wait(&bars->done, 0, abort_flag, spin_limit))) {
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < kTile / 32; ++c) {
        uint32_t raw[32];
        __syncwarp();
        tmem_load32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + c * 32, raw);
        if (gm >= M)
          continue;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int gn = n0 + c * 32 + g * 8;
          if (gn >= N) // N is a multiple of 8: a group of eight is entirely inside or outside
            continue;
          float o[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            o[u] = apply_activation(__uint_as_float(raw[g * 8 + u]), activation);
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
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTile) : "memory");
  }
  if (tid == 0 && bars->abort_flag && error_out)
    atomicExch(error_out, 1);
}

bool bf16_map(CUtensorMap *map, const void *plane, int64_t rows, int K) {
  EncodeTiled encode = encode_tiled();
  if (!encode)
    return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
  const cuuint32_t box[2] = {64, kTile};
  const cuuint32_t elem[2] = {1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(plane), dims, strides, box, elem,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

} // namespace

cudaError_t launch_gemv_bf16(const uint16_t *x, int K, const uint16_t *w, int64_t N, void *y, int y_dtype, int activation,
                             cudaStream_t stream) {
  if (N <= 0 || K <= 0 || K % 16 != 0 || K > 12288)
    return cudaErrorInvalidValue;
  const int64_t groups = (N + kGemvRows - 1) / kGemvRows;
  const int ctas = static_cast<int>(std::min<int64_t>((groups + kGemvThreads / 32 - 1) / (kGemvThreads / 32), 148 * 8));
  launch_chained(gemv_bf16_kernel, dim3(ctas), dim3(kGemvThreads), static_cast<size_t>(K) * sizeof(float), stream, x, K, w, N, y,
                 y_dtype, activation);
  return cudaGetLastError();
}

cudaError_t launch_gemm_bf16_tc(const uint16_t *x, int M, int K, const uint16_t *w, int N, void *y, int y_dtype, int activation,
                                int *error_flag, cudaStream_t stream, uint32_t spin_limit) {
  if (M <= 0 || N <= 0 || N % 8 != 0 || K <= 0 || K % 8 != 0)
    return cudaErrorInvalidValue;
  if (spin_limit == 0)
    spin_limit = 1u << 26; // about a second
  CUtensorMap map_x, map_w;
  if (!bf16_map(&map_x, x, M, K) || !bf16_map(&map_w, w, N, K))
    return cudaErrorNotSupported;
  if (cudaError_t e = opt_in_shared_memory(reinterpret_cast<const void *>(gemm_bf16_tc_kernel), kGemmSmemBytes); e != cudaSuccess)
    return e;
  launch_chained(gemm_bf16_tc_kernel, dim3((N + kTile - 1) / kTile, (M + kTile - 1) / kTile), dim3(kGemmThreads), kGemmSmemBytes, stream,
                 map_x, map_w, M, K, N, y, y_dtype, activation, error_flag, spin_limit);
  return cudaGetLastError();
}

cudaError_t launch_embedding_bf16(const int64_t *tokens, int64_t S, int H, int64_t vocab, const uint16_t *table, uint16_t *out,
                                  int *status, cudaStream_t stream) {
  if (S <= 0)
    return cudaSuccess;
  launch_chained(embedding_bf16_kernel, dim3(static_cast<unsigned>(S)), dim3(256), 0, stream, tokens, S, H, vocab, table, out, status);
  return cudaGetLastError();
}

} // namespace llmcp_b200
