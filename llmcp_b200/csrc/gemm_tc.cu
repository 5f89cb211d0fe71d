// Prefill GEMM (M > 1) on the fifth-generation tensor cores.  Q8Matmul.cpp:143-289.
//
// y[m, n] = act( chain_kb fma(float(dot_kb[m, n]), a_scale[m, kb] * w_scale[n, kb], acc) ),
// dot_kb = sum of 32 int8 products.  One tcgen05.mma kind::i8 has K = 32, which is exactly one
// quantisation block, so every block's int32 dot products come out of the tensor core as their
// own 128 x 128 tile in tensor memory (accumulate flag off) and the f32 scale-and-accumulate
// chain runs on the CUDA cores in ascending block order: the result is bit-identical to the
// GEMV and to the CPU order of operations.
//
// One CTA per 128 x 128 output tile, 640 threads:
//   warps 0-2  loaders: cp.async 16-byte pieces of the int8 operands into a ring of
//              shared-memory stages (4 blocks = 128 bytes of K per row, 128-byte swizzle,
//              K-major, the layout the MMA's matrix descriptors name), plus the f32 scales;
//   warp  3    one lane issues the MMAs: block kb of a stage -> tensor-memory buffer kb % 4;
//   warps 4-19 epilogue: tcgen05.ld the buffer (thread = row, 32 columns each: four lane
//              quarters x four column quarters), hand the buffer back, then cvt / fmul / fma per
//              element.  Sixteen warps rather than eight: the loop is a chain of waits (barrier,
//              tensor-memory load) and more warps in different phases keep the issue slots busy.
// Hand-offs are mbarriers; every wait is bounded and a timed-out wait raises an abort flag
// that all roles observe, so a protocol error ends the kernel with an error code instead of
// hanging it.  Tensor memory (512 columns) is allocated by warp 0 and always released.

#include "kernels.h"

namespace llmcp_b200 {

namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 128;
constexpr int kStageBlocks = 4;               // quantisation blocks per shared-memory stage
constexpr int kStageK = kStageBlocks * 32;    // 128 bytes of K per row
constexpr int kStages = 4;
constexpr int kTmemBuffers = 4;               // 4 x 128 columns
constexpr int kLoaderThreads = 96;
constexpr int kMmaWarp = 3;
constexpr int kEpilogueWarp0 = 4;
constexpr int kEpilogueThreads = 512;
constexpr int kThreads = 640;
constexpr uint32_t kSpinLimit = 1u << 26;     // bounded waits (about a second)

constexpr int kOperandBytes = kTileM * kStageK;                 // 16 KB per operand per stage
constexpr int kScaleBytes = kTileM * kStageBlocks * 4;          // 2 KB per operand per stage
constexpr int kStageBytes = 2 * kOperandBytes + 2 * kScaleBytes; // 36 KB
constexpr int kBarrierBytes = 256;
constexpr size_t kSmemBytes = 1024 + kStages * kStageBytes + kBarrierBytes;

struct Shared {
  // offsets inside the dynamic shared memory, after alignment to 1024 bytes
  static __device__ __forceinline__ uint8_t *stage(uint8_t *base, int s) { return base + s * kStageBytes; }
  static __device__ __forceinline__ uint8_t *a_tile(uint8_t *base, int s) { return stage(base, s); }
  static __device__ __forceinline__ uint8_t *b_tile(uint8_t *base, int s) { return stage(base, s) + kOperandBytes; }
  static __device__ __forceinline__ float *a_scale(uint8_t *base, int s) {
    return reinterpret_cast<float *>(stage(base, s) + 2 * kOperandBytes);
  }
  static __device__ __forceinline__ float *b_scale(uint8_t *base, int s) {
    return reinterpret_cast<float *>(stage(base, s) + 2 * kOperandBytes + kScaleBytes);
  }
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("{ .reg .b64 t; mbarrier.arrive.shared::cta.b64 t, [%0]; }" ::"r"(smem_u32(bar)) : "memory");
}

// Waits for the phase with the given parity; gives up when `abort_flag` is raised or after
// kSpinLimit polls (and then raises it).  Returns false on failure.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
    uint32_t done;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(done)
                 : "r"(addr), "r"(parity)
                 : "memory");
    if (done)
      return true;
    if ((spin & 255) == 255 && *abort_flag)
      return false;
  }
  *abort_flag = 1;
  return false;
}

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t smem_address) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_address & 0x3ffffu) >> 4);  // start address
  d |= static_cast<uint64_t>(1) << 16;                         // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                 // stride byte offset: next 8-row group
  d |= static_cast<uint64_t>(1) << 46;                         // descriptor version for sm_100
  d |= static_cast<uint64_t>(2) << 61;                         // SWIZZLE_128B
  return d;
}

// kind::i8, signed x signed -> s32, both operands K-major, M = 128, N = 128.
constexpr uint32_t kInstruction = (2u << 4) | (1u << 7) | (1u << 10) | ((kTileN >> 3) << 17) | ((kTileM >> 4) << 24);

__device__ __forceinline__ void mma_i8(uint32_t tmem, uint64_t a, uint64_t b) {
  asm volatile("{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
               "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p; }"
               :
               : "r"(tmem), "l"(a), "l"(b), "r"(kInstruction), "r"(0u), "r"(0u)
               : "memory");
}

__device__ __forceinline__ void mma_commit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 32 consecutive columns of this thread's lane.
__device__ __forceinline__ void tmem_load32(uint32_t taddr, int32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void cp_async16(void *dst, const void *src, int bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(void *dst, const void *src, int bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes) : "memory");
}

} // namespace

namespace {

struct Barriers {
  uint64_t full[kStages];          // stage landed in shared memory (96 loader arrivals)
  uint64_t empty[kStages];         // stage no longer needed: MMA done (1) + every epilogue warp
  uint64_t tfull[kTmemBuffers];    // a block's dot products are in the tensor-memory buffer
  uint64_t tempty[kTmemBuffers];   // the buffer has been read by all epilogue warps
  uint64_t done;                   // the MMA lane's last commit has arrived
  uint32_t tmem_base;
  int abort_flag;
};

__global__ void __launch_bounds__(kThreads, 1)
gemm_q8_tc_kernel(const int8_t *__restrict__ aq, const float *__restrict__ as, int M, int K,
                  const int8_t *__restrict__ wq, const float *__restrict__ ws, int N, void *__restrict__ y,
                  int y_dtype, int activation, int32_t *__restrict__ dots_out, int *__restrict__ error_out) {
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
      mbar_init(&bars->full[i], kLoaderThreads);
      mbar_init(&bars->empty[i], 1 + kEpilogueThreads / 32);
    }
    for (int i = 0; i < kTmemBuffers; ++i) {
      mbar_init(&bars->tfull[i], 1);
      if (i == 0)
        mbar_init(&bars->done, 1);
      mbar_init(&bars->tempty[i], kEpilogueThreads / 32);
    }
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                 "r"(kTmemBuffers * kTileN)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  grid_dependency_sync(); // barriers and tensor memory are set up; the operands belong to the kernel in front

  if (tid < kLoaderThreads) {
    // ---- loaders ------------------------------------------------------------------------
    auto issue = [&](int it) {
      const int s = it % kStages;
      const int kb0 = it * kStageBlocks;
      uint8_t *a_dst = Shared::a_tile(base, s), *b_dst = Shared::b_tile(base, s);
      for (int p = tid; p < kTileM * 8; p += kLoaderThreads) {
        const int row = p >> 3, c = p & 7;
        const int kbyte = kb0 * 32 + c * 16;
        const int offset = row * 128 + ((c ^ (row & 7)) << 4);
        const bool a_ok = m0 + row < M && kbyte < K;
        cp_async16(a_dst + offset, a_ok ? aq + static_cast<size_t>(m0 + row) * K + kbyte : aq, a_ok ? 16 : 0);
        const bool b_ok = n0 + row < N && kbyte < K;
        cp_async16(b_dst + offset, b_ok ? wq + static_cast<size_t>(n0 + row) * K + kbyte : wq, b_ok ? 16 : 0);
      }
      float *a_sc = Shared::a_scale(base, s), *b_sc = Shared::b_scale(base, s);
      for (int p = tid; p < kTileM * kStageBlocks; p += kLoaderThreads) {
        const int j = p >> 7, row = p & 127; // [block][row]
        const bool a_ok = m0 + row < M && kb0 + j < nb;
        cp_async4(a_sc + p, a_ok ? as + static_cast<size_t>(m0 + row) * nb + kb0 + j : as, a_ok ? 4 : 0);
        const bool b_ok = n0 + row < N && kb0 + j < nb;
        cp_async4(b_sc + p, b_ok ? ws + static_cast<size_t>(n0 + row) * nb + kb0 + j : ws, b_ok ? 4 : 0);
      }
    };
    for (int it = 0; it < kStages - 1; ++it) {
      if (it < iters)
        issue(it);
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int it = 0; it < iters; ++it) {
      asm volatile("cp.async.wait_group %0;" ::"n"(kStages - 2) : "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(&bars->full[it % kStages]);
      const int next = it + kStages - 1;
      if (next < iters) {
        bool ok = true;
        if (next >= kStages)
          ok = mbar_wait(&bars->empty[next % kStages], ((next / kStages) - 1) & 1, abort_flag);
        if (!ok)
          break;
        issue(next);
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (warp == kMmaWarp) {
    // ---- MMA issue ------------------------------------------------------------------------
    if (lane == 0) {
      bool ok = true;
      for (int it = 0; it < iters && ok; ++it) {
        const int s = it % kStages;
        ok = mbar_wait(&bars->full[s], (it / kStages) & 1, abort_flag);
        if (!ok)
          break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(Shared::a_tile(base, s)), b_addr = smem_u32(Shared::b_tile(base, s));
        const int blocks = min(kStageBlocks, nb - it * kStageBlocks);
        for (int j = 0; j < blocks; ++j) {
          const int kb = it * kStageBlocks + j;
          const int buf = kb % kTmemBuffers, use = kb / kTmemBuffers;
          if (use > 0) {
            ok = mbar_wait(&bars->tempty[buf], (use - 1) & 1, abort_flag);
            if (!ok)
              break;
            tc_fence_after();
          }
          mma_i8(tmem_base + buf * kTileN, operand_descriptor(a_addr + j * 32), operand_descriptor(b_addr + j * 32));
          mma_commit(&bars->tfull[buf]);
        }
        mma_commit(&bars->empty[s]);
      }
      // Nothing else waits for the last arrivals on `empty`; commits arrive in order, so once this
      // one is in, none is still on its way into shared memory that the next CTA on this SM owns.
      mma_commit(&bars->done);
      mbar_wait(&bars->done, 0, abort_flag);
    }
  } else if (warp >= kEpilogueWarp0) {
    // ---- epilogue ---------------------------------------------------------------------------
    const int quarter = warp & 3;                   // tensor-memory lanes 32*quarter .. +31
    const int colq = (warp - kEpilogueWarp0) >> 2;  // columns 32*colq .. +31
    const int row = quarter * 32 + lane;
    const int gm = m0 + row;
    float acc[32];
#pragma unroll
    for (int c = 0; c < 32; ++c)
      acc[c] = 0.0f;
    bool ok = true;
    for (int kb = 0; kb < nb && ok; ++kb) {
      const int buf = kb % kTmemBuffers;
      ok = __all_sync(0xffffffffu, mbar_wait(&bars->tfull[buf], (kb / kTmemBuffers) & 1, abort_flag));
      if (!ok) // the whole warp leaves together: the tensor-memory loads below are warp-wide
        break;
      tc_fence_after();
      const int s = (kb / kStageBlocks) % kStages, j = kb % kStageBlocks;
      const float a_scale = Shared::a_scale(base, s)[j * kTileM + row];
      const float4 *w_scale = reinterpret_cast<const float4 *>(Shared::b_scale(base, s) + j * kTileN + colq * 32);
      // The buffer is handed back before any arithmetic, so that the MMA of a later block can
      // reuse it while this one is still being folded in.
      int32_t v[32];
      tmem_load32(tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buf * kTileN + colq * 32, v);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      tc_fence_before();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&bars->tempty[buf]);
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float4 w4 = w_scale[g];
        const float wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
        for (int u = 0; u < 4; ++u)
          acc[g * 4 + u] = __fmaf_rn(static_cast<float>(v[g * 4 + u]), __fmul_rn(a_scale, wv[u]), acc[g * 4 + u]);
      }
      if (dots_out && gm < M) {
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          const int gn = n0 + colq * 32 + u;
          if (gn < N)
            dots_out[(static_cast<size_t>(gm) * N + gn) * nb + kb] = v[u];
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
      for (int g = 0; g < 4; ++g) {
        const int gn = n0 + colq * 32 + g * 8;
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
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemBuffers * kTileN) : "memory");
  }
  if (tid == 0 && bars->abort_flag && error_out)
    atomicExch(error_out, 1);
}

} // namespace

size_t gemm_q8_tc_smem_bytes() { return kSmemBytes; }

cudaError_t launch_gemm_q8_tc(const int8_t *aq, const float *as, int M, int K, const int8_t *wq, const float *ws, int N,
                              void *y, int y_dtype, int activation, int32_t *dots_out, int *error_flag,
                              cudaStream_t stream) {
  if (M <= 0 || N % 8 != 0 || K % kBlock != 0)
    return cudaErrorInvalidValue;
  if (cudaError_t e = opt_in_shared_memory(reinterpret_cast<const void *>(gemm_q8_tc_kernel), kSmemBytes); e != cudaSuccess)
    return e;
  dim3 grid((N + kTileN - 1) / kTileN, (M + kTileM - 1) / kTileM);
  launch_chained(gemm_q8_tc_kernel, dim3(grid), dim3(kThreads), kSmemBytes, stream, aq, as, M, K, wq, ws, N, y, y_dtype, activation, dots_out,
                                                            error_flag);
  return cudaGetLastError();
}

} // namespace llmcp_b200
