// Launchers of the llmcp operator kernels.  All pointers are device pointers; every
// launcher enqueues on `stream` and returns without synchronising.
#pragma once

#include <algorithm>
#include <cstddef>
#include <cstdint>

#include "common.cuh"

namespace llmcp_b200 {

constexpr int kMaxGemvJobs = 4;
constexpr int kArgmaxParts = 512;

// One weight matrix of a decode GEMV launch; all jobs of a launch share the input row.
struct GemvJob {
  const int8_t *wq;   // [N][K] int8
  const uint16_t *wd; // [N][K/32] f16 bits
  void *y;            // [N] output
  int N;
  int activation;
  int y_dtype;
  int warp_begin;  // filled by the launcher
  int dots_offset; // filled by the launcher
};

// flags of a GEMV launch
constexpr int kGemvOverlapPrevious = 1; // programmatic dependent launch: start while the kernel in
                                        // front is still running, wait for it before reading x
constexpr int kGemvPrefetchL2 = 2;      // prefetch all weights of the launch into L2 up front
constexpr int kGemvNoCols = 8;          // do not use the block-column kernel for long rows
constexpr int kGemvFast = 16;           // fast mode: a row's block products are added by a parallel tree
                                        // instead of the reference's ascending fma chain (the int32 block
                                        // dots are unchanged; the f32 sum differs by rounding only)

// Memory that the GEMV launch behind this one will stream (its weight matrices and scales): this
// launch asks for it in L2 while it runs, so that HBM keeps streaming under the small kernels
// between two GEMVs and the next GEMV reads from L2.  Addresses 16-byte aligned, sizes multiples of 16.
constexpr int kMaxPrefetchRanges = 8;
struct PrefetchList {
  const void *ptr[kMaxPrefetchRanges];
  uint32_t bytes[kMaxPrefetchRanges];
  int count;
};

struct GemvJobs {
  GemvJob job[kMaxGemvJobs];
  int count;
  int flags;
  int *error_flag; // device int (optional): set to 1 if a bounded wait for a copy ran out
  PrefetchList next; // K in {2560, 4096, 9216} block-column kernels only
};

// d32 (optional): the same scales widened to f32, [N][K/32], for the tensor-core GEMM.
void launch_repack_p4(const uint8_t *src, int64_t N, int64_t K, int8_t *q, uint16_t *d, float *d32,
                      cudaStream_t stream);
void launch_act_quant(const void *x, int x_dtype, int64_t M, int64_t K, int8_t *q, float *s, cudaStream_t stream);
cudaError_t launch_gemv_q8(const int8_t *aq, const float *as, int K, const GemvJobs &jobs, int32_t *dots_out,
                           cudaStream_t stream, int rows_per_warp = 0);
// Specialised GEMV for K in {2560, 4096, 9216}; rows_per_group 0 = choose.
bool gemv_rows_supported(int K);
cudaError_t launch_gemv_q8_rows(const int8_t *aq, const float *as, int K, const GemvJobs &jobs, int32_t *dots_out,
                                cudaStream_t stream, int rows_per_group);
// One matrix with long rows (K = 4096, 9216): a thread per block column (gemv_cols.cu).
bool gemv_cols_supported(int K, const GemvJobs &jobs);
cudaError_t launch_gemv_q8_cols(const int8_t *aq, const float *as, int K, const GemvJobs &jobs, int32_t *dots_out,
                                cudaStream_t stream);
// gate and up projections of the MLP (K = 2560, N % 32 == 0 rows each), SiLU on the gate, their
// product rounded to bf16 (product, optional) and quantised to int8 blocks (q_out, s_out) in one
// launch; the values of launch_gemv_q8 x 2 + launch_pointwise(mul).  flags: kGemvOverlapPrevious, kGemvFast.
bool gemv_swiglu_supported(int K, int64_t N);
cudaError_t launch_gemv_q8_swiglu(const int8_t *aq, const float *as, int K, const int8_t *gate_q, const uint16_t *gate_d,
                                  const int8_t *up_q, const uint16_t *up_d, int64_t N, uint16_t *product, int8_t *q_out,
                                  float *s_out, int flags, cudaStream_t stream, const PrefetchList *next = nullptr);
cudaError_t launch_gemm_q8_dp4a(const int8_t *aq, const float *as, int M, int K, const int8_t *wq,
                                const uint16_t *wd, int N, void *y, int y_dtype, int activation,
                                int32_t *dots_out, cudaStream_t stream);
// Tensor-core GEMM (tcgen05, sm_100a).  ws: f32 weight scales [N][K/32].  error_flag (device int,
// optional) is set to 1 if a bounded wait inside the kernel ran out.
size_t gemm_q8_tc_smem_bytes();
cudaError_t launch_gemm_q8_tc(const int8_t *aq, const float *as, int M, int K, const int8_t *wq, const float *ws, int N,
                              void *y, int y_dtype, int activation, int32_t *dots_out, int *error_flag,
                              cudaStream_t stream);
// status (device int, optional): bit 1 is raised when a token id lies outside [0, vocab); such a
// row is written as zeros and the table is not read.
// Tensor-core GEMM with TMA-fed operands (gemm_tma.cu).  Operand planes are [rows][K] and scale
// planes block-major f32, [K/32][pitch] (pitch = gemm_tc16_scale_pitch(M) for activations, N for
// weights); `form` says what the operand planes hold and how the epilogue multiplies:
//   kGemmI8  / kGemmI8Packed : int8 values, tcgen05 kind::i8, int32 dots converted in the epilogue;
//   kGemmF16 / kGemmF16Packed: the same integers as f16 values, kind::f16, exact f32 dots;
//   *Packed: two-lane f32x2 multiplies and fmas.
// spin_limit 0 = default (about a second); fault: test hook, see the kernel.
enum GemmForm : int { kGemmI8 = 0, kGemmI8Packed = 1, kGemmF16 = 2, kGemmF16Packed = 3 };
int64_t gemm_tc16_scale_pitch(int64_t M);
void launch_act_to_f16(const int8_t *aq, const float *as, int64_t M, int K, void *ah, float *ast, cudaStream_t stream);
void launch_weights_to_f16(const int8_t *wq, const uint16_t *wd, int64_t N, int K, void *wh, float *wst, cudaStream_t stream);
void launch_scales_block_major(const void *scales, int scales_are_f16, int64_t rows, int K, int64_t ld, float *out,
                               cudaStream_t stream);
cudaError_t launch_gemm_q8_tma(int form, const void *a, const float *ast, int M, int K, const void *w, const float *wst, int N,
                               void *y, int y_dtype, int activation, int32_t *dots_out, int *error_flag, cudaStream_t stream,
                               uint32_t spin_limit = 0, int fault = 0);
// status (device int, optional): bit 1 is raised when a token id lies outside [0, vocab); such a
// row is written as zeros and the table is not read.
// Second form of the tensor-core GEMM (gemm_tma.cu): the int8 operands held as f16 values and the
// scales as block-major f32 planes, tcgen05 kind::f16 with exact f32 block dots, TMA loads.
//   ah  [M][K] f16, ast [K/32][pitch] f32 with pitch = gemm_tc16_scale_pitch(M)  (launch_act_to_f16)
//   wh  [N][K] f16, wst [K/32][N] f32                                          (launch_weights_to_f16)
// spin_limit 0 = default (about a second); fault: test hook, see the kernel.
int64_t gemm_tc16_scale_pitch(int64_t M);
void launch_act_to_f16(const int8_t *aq, const float *as, int64_t M, int K, void *ah, float *ast, cudaStream_t stream);
void launch_weights_to_f16(const int8_t *wq, const uint16_t *wd, int64_t N, int K, void *wh, float *wst, cudaStream_t stream);
cudaError_t launch_gemm_q8_tc16(const void *ah, const float *ast, int M, int K, const void *wh, const float *wst, int N, void *y,
                                int y_dtype, int activation, int32_t *dots_out, int *error_flag, cudaStream_t stream,
                                uint32_t spin_limit = 0, int fault = 0);
void launch_embedding_q8(const int64_t *tokens, int64_t S, int64_t hidden, int64_t vocab, const int8_t *wq,
                         const uint16_t *wd, uint16_t *out, int *status, cudaStream_t stream);
// scratch_v / scratch_i: kArgmaxParts entries each.  rows > 1: x is [rows, n], one first maximum per
// row into out_index[row] (out_value[row]); rows <= kArgmaxParts.
void launch_argmax(const float *x, int64_t n, float *scratch_v, int64_t *scratch_i, int64_t index_base,
                   int64_t *out_index, float *out_value, cudaStream_t stream, int rows = 1);

cudaError_t launch_rms_norm(const uint16_t *a, const uint16_t *b, int64_t M, int H, const void *w, int w_dtype,
                            float eps, int zero_centered, uint16_t *sum_out, uint16_t *y, int8_t *q, float *s,
                            cudaStream_t stream);
// Fast mode of rms_norm: the sum of squares is a tree reduction (warp shuffles), not the
// reference's serial order, so the result can differ from launch_rms_norm in the last bit of rstd.
// Rows with H % 8 == 0 and H <= 8192; cudaErrorNotSupported otherwise (nothing is launched).
cudaError_t launch_rms_norm_fast(const uint16_t *a, const uint16_t *b, int64_t M, int H, const void *w, int w_dtype,
                                 float eps, int zero_centered, uint16_t *sum_out, uint16_t *y, int8_t *q, float *s,
                                 cudaStream_t stream);
cudaError_t launch_gated_rms_norm(const uint16_t *x, const uint16_t *gate, const void *w, int w_dtype, int64_t M,
                                  int H, int group, float eps, int gate_activated, uint16_t *y, int8_t *q,
                                  float *s, cudaStream_t stream);
cudaError_t launch_pointwise(const uint16_t *a, const uint16_t *b, int64_t count, int op, uint16_t *y, int8_t *q,
                             float *s, cudaStream_t stream);

cudaError_t launch_causal_conv1d(const uint16_t *x, const uint16_t *w, uint16_t *state, int64_t S, int C,
                                 int kernel, uint16_t *y, cudaStream_t stream);
size_t gdn_scratch_floats(int64_t S, int nk, int nv, int dk);
cudaError_t launch_gated_delta_net(const uint16_t *conv, const uint16_t *a, const uint16_t *b, const void *a_log,
                                   int a_log_dtype, const void *dt_bias, int dt_dtype, float *state, int64_t S,
                                   int nk, int nv, int dk, int dv, int b_activated, float *scratch,
                                   uint16_t *out, cudaStream_t stream, int ab_stride = 0 /* row pitch of a and b; 0 = nv */,
                                   int fast = 0 /* S > 1, dk = 128: row quarters per lane, fused multiply-adds */);
// A batch of independent sequences, one token each, through the one-token kernels: element strides
// between consecutive sequences' buffers (inputs and outputs are rows of a [sequences, width] matrix).
struct GdnBatch {
  int64_t conv_state; // convolution state of a layer
  int64_t ab;         // a and b rows
  int64_t state;      // recurrent state of a layer
};
// One token of causal_conv1d + gated_delta_net + gated_rms_norm (+ quantisation) in two launches,
// or in one (single_kernel, where gdn_decode_single_kernel_supported: a thread-block cluster per
// key head exchanges the normalised q and k through distributed shared memory; conv_out is not
// written then); the same values as the three general launchers above produce.  tree_sum (single
// kernel only): the three 128-term sums as shuffle trees instead of in index order.
// scratch: gdn_scratch_floats(1, ..).
bool gdn_decode_supported(int kernel, int nk, int nv, int dk, int dv);
bool gdn_decode_single_kernel_supported(int kernel, int nk, int nv, int dk, int dv);
cudaError_t launch_gdn_decode(const uint16_t *qkv, const uint16_t *conv_w, uint16_t *conv_state, int kernel,
                              const uint16_t *a, const uint16_t *b, const void *a_log, int a_log_dtype,
                              const void *dt_bias, int dt_dtype, float *state, int nk, int nv, int dk, int dv,
                              int b_activated, const uint16_t *gate, const void *norm_w, int norm_w_dtype, float eps,
                              int gate_activated, float *scratch, uint16_t *conv_out, uint16_t *y, int8_t *q_out,
                              float *s_out, cudaStream_t stream, int sequences = 1, const GdnBatch *strides = nullptr,
                              int single_kernel = 0, int tree_sum = 0);
// The start position is read from device memory (position_dev) so that a captured launch can be
// replayed at another position; max_position bounds it (grid and scratch are sized for it).
// rows_from_position: cos/sin are tables indexed by absolute position instead of the call's rows.
// cache_stride != 0: the S rows are one token each of S independent sequences, all at the same
// position, row t using the cache cache_stride elements behind row t - 1's (batched decode).
// q_out / s_out (optional): int8 quantisation of the output for the linear that follows.
size_t attn_scratch_bytes(int64_t S, int nh, int hd, int64_t max_position);
cudaError_t launch_attention(const uint16_t *qg, const uint16_t *k, const uint16_t *v, const uint16_t *q_norm,
                             const uint16_t *k_norm, const float *cos, const float *sin, int rows_from_position,
                             uint16_t *cache, const int64_t *position_dev, int64_t max_position, int64_t S, int nh,
                             int nkv, int hd, int rot, int64_t cap, void *scratch, uint16_t *out, int8_t *q_out,
                             float *s_out, cudaStream_t stream, int64_t cache_stride = 0);

// The first of the three attention launches alone: q/k RMSNorm, partial RoPE, q -> qn scratch
// (bf16 [S, nh, hd]), k and v -> cache rows position .. position + S - 1.  tree_sum (fast mode):
// the sums of squares of the two norms are shuffle trees instead of the reference's serial sums.
cudaError_t launch_attention_prepare(const uint16_t *qg, const uint16_t *k, const uint16_t *v, const uint16_t *q_norm,
                                     const uint16_t *k_norm, const float *cos, const float *sin, int rows_from_position,
                                     uint16_t *cache, const int64_t *position_dev, int64_t S, int nh, int nkv, int hd,
                                     int rot, int64_t cap, uint16_t *qn, cudaStream_t stream, int tree_sum = 0,
                                     int64_t cache_stride = 0);
// Fast mode of the one-token attention: after the same prepare kernel, the key range is split
// over CTAs (each keeps a running maximum, denominator and weighted value sum for the query
// heads of one KV head) and a second kernel merges the splits, applies the sigmoid gate and
// quantises for o_proj.  The softmax is the same function as the reference's tile-ordered one
// but sums in another order, so results agree to f32 rounding, not bit for bit.
// bf16 weights [N][K] of an unquantised arena (MatmulLoweringCommon.cpp:186-251): y = act(x w^T) with
// f32 accumulation; one row through a streaming GEMV, more rows on the tensor cores (bf16 operands by
// TMA; error_flag as for the Q8 GEMM).  GEMV: K % 16 == 0; GEMM: K % 8 == 0 and N % 8 == 0.
cudaError_t launch_gemv_bf16(const uint16_t *x, int K, const uint16_t *w, int64_t N, void *y, int y_dtype, int activation,
                             cudaStream_t stream);
cudaError_t launch_gemm_bf16_tc(const uint16_t *x, int M, int K, const uint16_t *w, int N, void *y, int y_dtype, int activation,
                                int *error_flag, cudaStream_t stream, uint32_t spin_limit = 0);
cudaError_t launch_embedding_bf16(const int64_t *tokens, int64_t S, int H, int64_t vocab, const uint16_t *table, uint16_t *out,
                                  int *status, cudaStream_t stream);
// Fast mode of the prefill attention (S > 1, head_dim 256): the same prepare kernel, then both
// contractions on the tensor cores with the softmax weights rounded to bf16 (attn_prefill.cu).
// scratch: attention_prefill_tc_scratch_bytes.  error_flag (device int, optional) is set to 1 if a
// bounded wait inside the kernel ran out; three launches.
bool attention_prefill_tc_supported(int nh, int nkv, int hd);
size_t attention_prefill_tc_scratch_bytes(int64_t S, int nh, int nkv, int64_t cap);
cudaError_t launch_attention_prefill_tc(const uint16_t *qg, const uint16_t *k, const uint16_t *v, const uint16_t *q_norm,
                                        const uint16_t *k_norm, const float *cos, const float *sin, int rows_from_position,
                                        uint16_t *cache, const int64_t *position_dev, int64_t max_position, int64_t S, int nh,
                                        int nkv, int hd, int rot, int64_t cap, void *scratch, uint16_t *out, int8_t *q_out,
                                        float *s_out, int *error_flag, cudaStream_t stream, uint32_t spin_limit = 0);
bool attention_decode_fast_supported(int nh, int nkv, int hd);
size_t attn_fast_scratch_bytes(int nh, int hd, int64_t max_position, int sequences = 1);
cudaError_t launch_attention_decode_fast(const uint16_t *qg, const uint16_t *k, const uint16_t *v,
                                         const uint16_t *q_norm, const uint16_t *k_norm, const float *cos,
                                         const float *sin, int rows_from_position, uint16_t *cache,
                                         const int64_t *position_dev, int64_t max_position, int nh, int nkv, int hd,
                                         int rot, int64_t cap, void *scratch, uint16_t *out, int8_t *q_out,
                                         float *s_out, cudaStream_t stream, int sequences = 1, int64_t cache_stride = 0);

} // namespace llmcp_b200
