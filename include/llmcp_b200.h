/* C ABI of libllmcp_b200.so: a CUDA (sm_100a) implementation of llmcp's Q8_0 hot path.
 *
 * Three groups of entry points:
 *   1. the AOT ABI v2 symbols that llmcp's runtime resolves with dlsym, so the library can
 *      be passed to `llmcp-benchmark --aot` / `llmcp-run --aot` in place of a compiled model;
 *   2. one function per llmcp dialect operator (host pointers in, host pointers out) for
 *      operator-level parity checks, plus the same operators on device pointers;
 *   3. an engine handle for callers that want tokens, state and logits to stay on the GPU.
 *
 * All functions return 0 on success unless stated otherwise; on failure they return a
 * non-zero code and leave a message for llmcp_b200_last_error().  Nothing here falls back
 * to the CPU: without a CUDA device every compute entry fails.
 *
 * File paths in the comments are paths inside the llmcp project.
 */
#ifndef LLMCP_B200_H
#define LLMCP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- 1. AOT ABI v2 --------------------------------------------------------------- */

/* Replaces the generated `llmcp_model_abi_version` (lib/Model/ModelBuilder.cpp:528-536,
 * include/llmcp/Support/AotAbi.h:12); checked by lib/Runtime/AotRuntime.cpp:49-55. */
int32_t llmcp_model_abi_version(void);

/* Replace the generated `_mlir_ciface_llmcp_model_prefill` / `_decode`
 * (lib/Model/ModelBuilder.cpp:440-526; resolved at lib/Runtime/AotRuntime.cpp:56-64 and
 * called at :87-118).  Arguments, in order: tokens memref<?xindex>, cos memref<?x64xf32>,
 * sin memref<?x64xf32>, start position (index, by value), cache length (index, by value),
 * arena memref<?xi8>, kv memref<8x2x4x?x256xbf16>, delta memref<24x32x128x128xf32>,
 * conv memref<24x3x8192xbf16>, logits memref<1x248320xf32>; each memref is a pointer to
 * {T* base; T* data; int64 offset; int64 sizes[N]; int64 strides[N]}
 * (include/llmcp/Runtime/AotRuntime.h:52-58).  All buffers are host memory.  The logits row
 * is always fully written.  The generation state lives on the GPU: it is cleared when a call
 * starts at position 0 and the host kv/delta/conv buffers are neither read nor written
 * unless LLMCP_B200_SYNC_STATE=1 is set, in which case they are uploaded before and
 * downloaded after every call.  On a CUDA failure the row is filled with NaN and the message
 * is kept for llmcp_b200_last_error(). */
void _mlir_ciface_llmcp_model_prefill(void *tokens, void *cos, void *sin, void *start_pos, void *cache_length,
                                      void *arena, void *kv, void *delta, void *conv, void *logits);
void _mlir_ciface_llmcp_model_decode(void *tokens, void *cos, void *sin, void *start_pos, void *cache_length,
                                     void *arena, void *kv, void *delta, void *conv, void *logits);

/* Additive: copies the last error message (NUL terminated, truncated to `capacity`) and
 * returns its length; 0 means no error since the last llmcp_b200_clear_error(). */
size_t llmcp_b200_last_error(char *buffer, size_t capacity);
void llmcp_b200_clear_error(void);
/* Number of visible CUDA devices (0 without a driver or GPU). */
int llmcp_b200_device_count(void);
/* Device used by the AOT entries and by the host-pointer operators (default: current). */
int llmcp_b200_set_device(int device);
/* Releases every engine created by the AOT entries. */
void llmcp_b200_release_all(void);
/* Engines currently held by the AOT entry points: one per distinct (arena, kv, delta, conv) set of the
 * caller, at most LLMCP_B200_MAX_SESSIONS (default 4; the least recently used one is released beyond that). */
int llmcp_b200_session_count(void);
/* Kernel launches issued by this library since it was loaded. */
uint64_t llmcp_b200_launch_count(void);
/* Arithmetic mode (no counterpart in the reference, which has one order of operations).
 *   0 exact: every f32 result is bit-identical to the reference's order (default);
 *   1 fast : integer block dots, quantisation and bf16 rounding points unchanged; the reductions
 *            whose order only moves f32 rounding (rms_norm's sum of squares, a decode GEMV row's sum
 *            over its blocks, the one-token attention softmax over keys, the one-token
 *            gated-delta-net sums over the key dimension) run as parallel trees.  Bars: logits
 *            within 1e-2 of the exact mode, greedy tokens equal wherever the top-2 margin exceeds
 *            the logit difference.
 * The mode applies to engines created afterwards (the AOT entries create theirs at the first
 * call for a given arena and state) and to the host-pointer operators of group 2.
 * LLMCP_B200_MODE=fast|exact in the environment sets the initial value. */
int llmcp_b200_set_mode(int mode);
int llmcp_b200_get_mode(void);

/* ---- 2. operators ------------------------------------------------------------------ */
/* dtype: 0 = f32, 1 = bf16 (bit patterns in uint16).  activation: 0 none, 1 silu,
 * 2 sigmoid, 3 softplus (lib/Dialect/LLMCP/Transforms/MatmulLoweringCommon.cpp:78-103). */

/* Activation quantisation used by every Q8 linear (Q8Decode.cpp:83-120,
 * Q8Matmul.cpp:93-141): q [M,K] int8, scales [M,K/32] f32. */
int llmcp_op_act_quant(const void *x, int x_dtype, int64_t M, int64_t K, int8_t *q, float *scales);

/* llmcp.linear with weight_format = "q8_0_p4" (LLMCPOps.td:19-45, LLMCPOps.cpp:46-70;
 * kernels Q8Decode.cpp:131-225 for M = 1 and Q8Matmul.cpp:143-289 otherwise).
 * weight: N/4 * K/32 records of 136 bytes.  block_dots, if not NULL, receives the int32
 * dot product of every (row, column, 32-block): [M, N, K/32].  N % 8 == 0, K % 32 == 0. */
int llmcp_op_linear_q8(const void *x, int x_dtype, int64_t M, int64_t K, const uint8_t *weight, int64_t N,
                       void *y, int y_dtype, int activation, int32_t *block_dots);

/* llmcp.linear on the bf16 matrix of an unquantised arena (lib/Dialect/LLMCP/Transforms/
 * MatmulLoweringCommon.cpp:186-251,509-527): y = act(x w^T), x [M, K] and w [N, K] bf16, products and
 * sums in f32, y bf16 or f32.  One row runs a streaming GEMV, more rows the tensor cores; the order of
 * the f32 additions is this library's (the reference's differs by target), so results agree with the
 * reference to f32 rounding, as its own tests require (tests/numeric/run_numeric.py:676-688). */
int llmcp_op_linear_bf16(const uint16_t *x, int64_t M, int64_t K, const uint16_t *weight, int64_t N, void *y, int y_dtype,
                         int activation);

/* llmcp.lm_head (LLMCPOps.td:103-110, LowerToLinalg.cpp:729-765) followed by the host
 * argmax of tools/llmcp-benchmark/llmcp-benchmark.cpp:51-54 (first maximum).
 * hidden: [M, K] bf16; logits: [M, vocab] f32 (may be NULL); argmax: [M] (may be NULL). */
int llmcp_op_lm_head_q8(const uint16_t *hidden, int64_t M, int64_t K, const uint8_t *table, int64_t vocab,
                        float *logits, int64_t *argmax);

/* llmcp.embedding on a packed table (LLMCPOps.td:94-101, LowerToLinalg.cpp:435-531). */
int llmcp_op_embedding_q8(const int64_t *tokens, int64_t S, const uint8_t *table, int64_t vocab, int64_t hidden,
                          uint16_t *out);

/* llmcp.rms_norm (LLMCPOps.td:47-68, LowerToLinalg.cpp:211-308, DecodeNormalization.cpp:70-145). */
int llmcp_op_rms_norm(const uint16_t *x, int64_t M, int64_t H, const void *weight, int w_dtype, float eps,
                      int zero_centered, uint16_t *y);

/* llmcp.add (op 0), llmcp.mul (1), llmcp.silu_mul (2; a = gate, b = up)
 * (LLMCPOps.td:70-92, LowerToLinalg.cpp:312-427). */
int llmcp_op_pointwise(const uint16_t *a, const uint16_t *b, int64_t count, int op, uint16_t *y);

/* llmcp.gated_rms_norm (LLMCPOps.td:167-179, LowerToLinalg.cpp:574-727). */
int llmcp_op_gated_rms_norm(const uint16_t *x, const uint16_t *gate, const void *weight, int w_dtype, int64_t M,
                            int64_t H, int64_t group, float eps, int gate_activated, uint16_t *y);

/* llmcp.causal_conv1d with SiLU (LLMCPOps.td:112-123, LowerCausalConv1d.cpp:29-189).
 * x,y: [S, C] bf16; weight: [C, 1, kernel] bf16; state: [kernel-1, C] bf16, updated. */
int llmcp_op_causal_conv1d(const uint16_t *x, const uint16_t *weight, uint16_t *state, int64_t S, int64_t C,
                           int64_t kernel, uint16_t *y);

/* llmcp.gated_delta_net (LLMCPOps.td:125-143, LowerGatedDeltaNet.cpp:47-452).
 * conv: [S, 2*nk*dk + nv*dv] bf16; a,b: [S, nv] bf16; a_log: [nv] f32; dt_bias: [nv] bf16;
 * state: [nv, dk, dv] f32, updated; out: [S, nv*dv] bf16. */
int llmcp_op_gated_delta_net(const uint16_t *conv, const uint16_t *a, const uint16_t *b, const float *a_log,
                             const uint16_t *dt_bias, float *state, int64_t S, int64_t nk, int64_t nv, int64_t dk,
                             int64_t dv, int b_activated, uint16_t *out);

/* llmcp.attention (LLMCPOps.td:145-165, LowerAttention.cpp:54-607).  qg: [S, nh*2*hd];
 * k,v: [S, nkv*hd]; q_norm,k_norm: [hd] bf16; cos,sin: [S, rot] f32; cache: one layer
 * [2, nkv, cap, hd] bf16, updated at rows position .. position+S-1; out: [S, nh*hd]. */
int llmcp_op_attention(const uint16_t *qg, const uint16_t *k, const uint16_t *v, const uint16_t *q_norm,
                       const uint16_t *k_norm, const float *cos, const float *sin, uint16_t *cache, int64_t position,
                       int64_t S, int64_t nh, int64_t nkv, int64_t hd, int64_t rot, int64_t cap, uint16_t *out);

/* The same contraction on device pointers, enqueued on `stream` (a cudaStream_t) without
 * synchronising: for callers that keep weights and activations in HBM.
 *   llmcp_dev_repack_q8 : arena records -> q [N][K] int8 and d [N][K/32] f16 (device layout).
 *   llmcp_dev_act_quant : as llmcp_op_act_quant.
 *   llmcp_dev_gemv_q8   : M = 1 linear on already quantised input (Q8Decode.cpp:131-225).
 *                         rows_per_warp 0 = choose.  flags: 1 = launch as a programmatic
 *                         dependent of the kernel in front (weights are requested while that
 *                         kernel still runs; x is read only after it has finished), 2 = also
 *                         prefetch into L2 what the launch reads after its first round of
 *                         loads, 8 = use the row kernel where a block-column kernel would be
 *                         chosen, 16 = fast mode: a row's block products are added by a parallel
 *                         tree instead of the reference's ascending fma chain.
 *   llmcp_dev_gemm_q8   : M > 1 linear (Q8Matmul.cpp:143-289), integer dot products on dp4a.
 *   llmcp_dev_gemm_q8_tc: the same contraction on the tcgen05 tensor cores.  wd32 holds the
 *                         weight scales widened to f32, [N][K/32].  status (device int, may be
 *                         null) is set to 1 if a bounded wait inside the kernel ran out; the
 *                         caller reads it after synchronising.
 *   llmcp_dev_gemm_q8_tma: the M > 1 linear on the tensor cores with operands fetched by TMA
 *                         (cp.async.bulk.tensor, no multicast).  form: 0 int8 operand planes,
 *                         tcgen05 kind::i8, int32 dots converted in the epilogue; 2 the same integers
 *                         held as f16 values, kind::f16 (an f16 x f16 block dot of int8-valued operands
 *                         is an exact integer in f32, so the result is the same bit for bit and the
 *                         conversion disappears); 1 and 3: the same with two-lane f32x2 multiplies and
 *                         fmas.  a / w: [rows][K] int8 (forms 0, 1) or f16 (2, 3); a_scales / w_scales:
 *                         block-major f32 [K/32][pitch], pitch = llmcp_dev_gemm_q8_tma_scale_pitch(M)
 *                         (M rounded up to 4) for activations and N for weights.  status as above.
 *                         spin_limit: polls before a wait inside the kernel gives up (0 = default,
 *                         about a second).  fault: 0; 1 is a test hook that withholds the first
 *                         stage's copies so that the bounded waits run out (status becomes 1, y is
 *                         left unwritten, tensor memory is released).
 *   llmcp_dev_q8_gemm_planes: those planes from int8 values [rows][K] and their scales
 *                         [rows][K/32] (f32 for activations, f16 bits for weights when
 *                         scales_are_f16): scales_block_major always, values_f16 if not null.
 *   llmcp_dev_argmax    : first maximum of n f32 values; scratch: 512 floats + 512 int64. */
int llmcp_dev_repack_q8(const uint8_t *records, int64_t N, int64_t K, int8_t *q, uint16_t *d, void *stream);
int llmcp_dev_act_quant(const void *x, int x_dtype, int64_t M, int64_t K, int8_t *q, float *scales, void *stream);
int llmcp_dev_gemv_q8(const int8_t *aq, const float *as, int64_t K, const int8_t *wq, const uint16_t *wd, int64_t N,
                      void *y, int y_dtype, int activation, int rows_per_warp, int flags, void *stream);
/* The MLP's gate and up projections of one token with their product in one launch (K = 2560,
 * N % 32 == 0): product[i] = bf16(bf16(silu(gate_i . x)) * bf16(up_i . x)) (optional output) and its
 * int8 quantisation q_out [N], s_out [N/32] for the down projection -- the fused form of
 * lib/Dialect/LLMCP/Transforms/FuseLinearActivations.cpp:27-77 + the `mul` of LowerToLinalg.cpp:312-427
 * + Q8Decode.cpp:83-120.  flags: 1 and 16 as for llmcp_dev_gemv_q8.  q_out/s_out must not alias aq/as. */
int llmcp_dev_gemv_q8_swiglu(const int8_t *aq, const float *as, int64_t K, const int8_t *gate_q, const uint16_t *gate_d,
                             const int8_t *up_q, const uint16_t *up_d, int64_t N, uint16_t *product, int8_t *q_out,
                             float *s_out, int flags, void *stream);
int llmcp_dev_gemm_q8(const int8_t *aq, const float *as, int64_t M, int64_t K, const int8_t *wq, const uint16_t *wd,
                      int64_t N, void *y, int y_dtype, int activation, void *stream);
int llmcp_dev_gemm_q8_tc(const int8_t *aq, const float *as, int64_t M, int64_t K, const int8_t *wq, const float *wd32,
                         int64_t N, void *y, int y_dtype, int activation, int *status, void *stream);
int llmcp_dev_q8_gemm_planes(const int8_t *q, const void *scales, int scales_are_f16, int64_t rows, int64_t K, void *values_f16,
                             float *scales_block_major, void *stream);
int64_t llmcp_dev_gemm_q8_tma_scale_pitch(int64_t M);
int llmcp_dev_gemm_q8_tma(int form, const void *a, const float *a_scales, int64_t M, int64_t K, const void *w,
                          const float *w_scales, int64_t N, void *y, int y_dtype, int activation, int *status,
                          uint32_t spin_limit, int fault, void *stream);
int llmcp_dev_argmax(const float *x, int64_t n, float *scratch_values, int64_t *scratch_indices, int64_t *out_index,
                     void *stream);

/* No counterpart in the reference (its generated code allocates with malloc as it goes).
 * llmcp.gated_delta_net on device pointers for callers that may not allocate GPU memory:
 * a server that owns the whole GPU through its own pool, or a decode loop that cannot pay
 * for the synchronisation an allocation can cause.  Arguments as llmcp_op_gated_delta_net,
 * all of them device pointers; enqueued on `stream` (a cudaStream_t), not synchronised.
 * The working memory is a 256 KiB array built into the library (resident on every GPU that
 * loads it): calls with S * (2*nk*dk + 2*nv) > 65536 are refused with code 2 and a message.
 * All calls on a GPU share that array, so calls that overlap in time on one GPU race; its
 * old contents need no clearing.  The first call on each device resolves the array's device
 * address; make it before starting any stream capture.  Calls no cudaMalloc / cudaFree. */
int llmcp_dev_gated_delta_net_noalloc(const uint16_t *conv, const uint16_t *a, const uint16_t *b,
                                      const float *a_log, const uint16_t *dt_bias, float *state, int64_t S,
                                      int64_t nk, int64_t nv, int64_t dk, int64_t dv, int b_activated,
                                      uint16_t *out, void *stream);

/* ---- 3. engine --------------------------------------------------------------------- */

typedef struct llmcp_b200_dims {
  int64_t hidden, intermediate, vocab, layers, full_interval;
  int64_t heads, kv_heads, head_dim, rotary;
  int64_t lin_k_heads, lin_v_heads, lin_k_dim, lin_v_dim, conv_kernel;
  float eps, rope_theta;
} llmcp_b200_dims;

/* Qwen3.5-4B text dimensions (docs/model-spec.md:51-76, lib/Runtime/AotRuntime.cpp:41-43). */
void llmcp_b200_default_dims(llmcp_b200_dims *dims);

/* Container helpers (format of include/llmcp/Support/PackedWeights.h:21-58,
 * lib/Model/WeightLayout.cpp:96-268, lib/Model/WeightPacker.cpp:126-160).
 *   llmcp_b200_synthetic_bytes : size of a random-init container for `dims`.
 *   llmcp_b200_synthetic_fill  : writes it (arena, manifest, header last) from `seed`.
 *   llmcp_b200_pack_q8_0_p4    : lib/Model/Quantization.cpp:165-214 on an f32 matrix.
 *   llmcp_b200_validate        : the checks of lib/Runtime/WeightArena.cpp:39-123. */
uint64_t llmcp_b200_synthetic_bytes(const llmcp_b200_dims *dims);
int llmcp_b200_synthetic_fill(const llmcp_b200_dims *dims, uint64_t seed, uint8_t *file, uint64_t file_bytes);
int llmcp_b200_pack_q8_0_p4(const float *values, int64_t rows, int64_t cols, uint8_t *dst);
int llmcp_b200_validate(const uint8_t *file, uint64_t file_bytes);
/* Text <-> token ids, the two ends of llmcp-run (tools/llmcp-run/llmcp-run.cpp:626-690).  Host only.
 *   llmcp_b200_vocab_create   : from the text of a tokenizer.json (model.vocab + added_tokens, ByteLevel
 *                               decoder) or of a bare {"token": id} object; NULL + last_error on failure.
 *   llmcp_b200_vocab_decode   : the tokenizer's Decode(ids): GPT-2 byte alphabet back to bytes, then
 *                               lossy UTF-8 (ill-formed subsequences become U+FFFD); ids without a
 *                               token are skipped.  Text functions copy at most capacity - 1 bytes
 *                               and a terminating 0 into `out` and return the full length.
 *   llmcp_b200_vocab_encode   : the tokenizer's Encode(text) of tools/llmcp-run/llmcp-run.cpp:641 (tokenizers-cpp
 *                               over the Hugging Face byte-level BPE): added tokens are cut out whole, the
 *                               rest is split by the Qwen pre-tokenisation pattern, each piece is mapped to
 *                               the byte alphabet and merged by rank.  Writes at most `capacity` ids and
 *                               returns the full count; -1 + last_error when the tokenizer.json asks for a
 *                               pre-tokeniser, normaliser (other than NFC) or added-token option this code
 *                               does not restate, or the text is ill-formed UTF-8 (nothing is approximated).
 *   llmcp_b200_pretokenize    : the split step of that encoder alone: byte offsets at which the pieces of
 *                               `text` end (at most `capacity` written); returns the number of pieces.
 *   llmcp_b200_regex_split    : a Split pre-tokeniser on its own: `pattern` in the regular-expression subset the
 *                               library restates (csrc/text_regex.h), `behavior` one of removed, isolated,
 *                               merged_with_previous, merged_with_next, contiguous.  The pieces are written
 *                               one after the other into `out` (never more than `length` bytes) and their
 *                               byte lengths into `lengths`; returns their number, or -1 + last_error for
 *                               a pattern with a construct outside the subset.
 *   llmcp_b200_normalize_nfc  : Unicode Normalization Form C of a UTF-8 text, the normaliser the encoder
 *                               applies when the tokenizer.json names it.
 *   llmcp_b200_stream_*       : ByteLevelStreamingDecoder of tools/llmcp-run/StreamingDecoder.cpp:13-29:
 *                               append returns a complete chunk, or nothing while the decoded tail is
 *                               U+FFFD (bytes the next token may complete); finish emits the rest.
 *                               The vocabulary must outlive the stream.
 *   llmcp_b200_chat_prompt    : makeChatPrompt of tools/llmcp-run/llmcp-run.cpp:608-624. */
void *llmcp_b200_vocab_create(const char *json, uint64_t length);
void llmcp_b200_vocab_destroy(void *vocab);
int64_t llmcp_b200_vocab_size(const void *vocab);
int32_t llmcp_b200_vocab_token_to_id(const void *vocab, const char *token);
uint64_t llmcp_b200_vocab_decode(const void *vocab, const int32_t *ids, uint64_t count, char *out, uint64_t capacity);
int64_t llmcp_b200_vocab_encode(const void *vocab, const char *text, uint64_t length, int32_t *ids, uint64_t capacity);
int64_t llmcp_b200_pretokenize(const char *text, uint64_t length, int64_t *ends, uint64_t capacity);
uint64_t llmcp_b200_normalize_nfc(const char *text, uint64_t length, char *out, uint64_t capacity);
int64_t llmcp_b200_regex_split(const char *pattern, const char *text, uint64_t length, const char *behavior, int invert,
                               char *out, uint64_t out_capacity, int64_t *lengths, uint64_t capacity);
void *llmcp_b200_stream_create(const void *vocab);
void llmcp_b200_stream_destroy(void *stream);
uint64_t llmcp_b200_stream_append(void *stream, int32_t token, char *out, uint64_t capacity);
uint64_t llmcp_b200_stream_finish(void *stream, char *out, uint64_t capacity);
uint64_t llmcp_b200_chat_prompt(const char *user, const char *system, int thinking, char *out, uint64_t capacity);
/* Checkpoint → container, the job of llmcp's offline packer:
 *   llmcp_b200_parse_config     : model dimensions from the text of config.json, with the
 *                                 checks of lib/Model/ModelConfig.cpp:78-283.
 *   llmcp_b200_read_safetensors : header of one safetensors shard (lib/Model/Safetensors.cpp:
 *                                 61-172) as text, one line per tensor:
 *                                 name TAB dtype TAB absolute data offset TAB bytes TAB d0,d1,...
 *                                 Returns the text length, 0 on error.
 *   llmcp_b200_pack_checkpoint  : `llmcp-pack --model DIR --out FILE --quant none|q8_0
 *                                 [--dry-run] [--verbose]` (tools/llmcp-pack/llmcp-pack.cpp:44-89,
 *                                 lib/Model/WeightPacker.cpp:163-274); the three counters are what
 *                                 its summary line prints.  Host only: no GPU is touched. */
int llmcp_b200_parse_config(const char *json, uint64_t length, llmcp_b200_dims *dims);
/* A random-init checkpoint directory (config.json, one safetensors shard and its index) holding
 * the tensors llmcp_b200_synthetic_fill draws for (dims, seed): what llmcp-pack, the reference's
 * or this repository's, turns into that container.  Stands in for the real checkpoint
 * (docs/model-spec.md:51-76), which is not distributed with either project. */
int llmcp_b200_synthetic_checkpoint(const llmcp_b200_dims *dims, uint64_t seed, const char *model_dir);
uint64_t llmcp_b200_read_safetensors(const char *path, char *buffer, uint64_t capacity);
int llmcp_b200_pack_checkpoint(const char *model_dir, const char *output_path, const char *quant, int dry_run,
                               int verbose, uint64_t *tensors, uint64_t *source_bytes, uint64_t *arena_bytes);
/* Rotary cos/sin row of one position, f32 (lib/Runtime/AotRuntime.cpp:22-32). */
void llmcp_b200_make_cos_sin(int64_t position, int64_t rotary, float theta, float *cos_out, float *sin_out);
/* Copies the manifest JSON text of a container; returns its length. */
uint64_t llmcp_b200_manifest(const uint8_t *file, uint64_t file_bytes, char *buffer, uint64_t capacity);

/* Uploads a container (host memory: header, arena, manifest) to `device`, re-laying the
 * weights out for the GPU, and allocates state for `capacity` positions.  NULL on failure. */
void *llmcp_b200_engine_create(const uint8_t *file, uint64_t file_bytes, const llmcp_b200_dims *dims,
                               int64_t capacity, int device);
/* The same with an explicit arithmetic mode (see llmcp_b200_set_mode). */
void *llmcp_b200_engine_create_mode(const uint8_t *file, uint64_t file_bytes, const llmcp_b200_dims *dims,
                                    int64_t capacity, int device, int mode);
/* A batch of independent sequences (no counterpart in the reference, whose entry points take one
 * sequence: lib/Model/ModelBuilder.cpp:72-81, 440-526).  The engine keeps recurrent state,
 * convolution state and KV cache per sequence.  Sequences are prefilled one at a time:
 * llmcp_b200_engine_select_sequence, then llmcp_b200_engine_forward / _read_state as for one sequence.
 * Once all stand at the same position they are decoded together, one token each per step: the
 * projections become one contraction of `batch` rows on the tensor cores (the weights stream
 * from HBM once per step for all sequences), every other operator runs per sequence with the
 * arithmetic of the one-sequence path, so each sequence's logits equal its own one-sequence run's
 * (bit for bit in exact mode).
 *   llmcp_b200_engine_decode_batch  : tokens[batch] at `position` -> argmax[batch] and, if not
 *                                     null, logits[batch][vocab].
 *   llmcp_b200_engine_generate_batch: greedy decoding on the device: out_tokens[steps][batch]. */
void *llmcp_b200_engine_create_batch(const uint8_t *file, uint64_t file_bytes, const llmcp_b200_dims *dims, int64_t capacity,
                                     int device, int mode, int batch);
int llmcp_b200_engine_select_sequence(void *engine, int sequence);
int llmcp_b200_engine_decode_batch(void *engine, const int64_t *tokens, int64_t position, float *logits, int64_t *argmax);
int llmcp_b200_engine_generate_batch(void *engine, const int64_t *first_tokens, int64_t position, int64_t steps,
                                     int64_t *out_tokens, float *device_ms);

/* Tensor parallelism over the GPUs of one node (no counterpart in the reference, which is one
 * process on one device; what is split are the output rows of the linears that
 * lib/Model/ModelBuilder.cpp:218-319 builds, on the 8-row boundaries of
 * include/llmcp/Support/Q8PackedLayout.h:38-42).  One process per GPU.  Every linear is split by
 * output rows only, so each output element is computed by one rank with the unsplit arithmetic and
 * the results equal the single-GPU engine's bit for bit; recurrent and attention heads and their
 * state are split by head; the vocabulary projection by rows, with a (maximum, index) exchange
 * that keeps the first-maximum rule.  The exchange is this library's own kernel: every rank stores
 * its piece into buffers of its peers that are mapped through CUDA IPC and waits, bounded, for
 * their flags (no NCCL, no host round trip; part of the captured decode step).
 *   llmcp_b200_tp_slot_bytes : bytes per exchange slot for calls of up to max_tokens tokens.
 *   llmcp_b200_tp_create     : allocates this rank's exchange buffer on `device`; handle_out
 *                              receives 64 bytes to hand to the other ranks (any channel).
 *   llmcp_b200_tp_attach     : maps the peers' buffers; handles = size x 64 bytes in rank order.
 *   llmcp_b200_tp_all_gather : the exchange alone: this rank's [rows][row_bytes] piece -> slot
 *                              `slot` (0..2) of every rank, rows of size x row_bytes bytes; copied to
 *                              dst if not null.  Consecutive calls must name different slots.
 *                              status (device int, may be null): bit 2 is raised if a peer's flag did
 *                              not arrive within the wait limit.
 *   llmcp_b200_engine_create_tp: an engine that holds rank's share; every rank must then make the
 *                              same forward / generate calls.  llmcp_b200_engine_read_state returns
 *                              this rank's heads (llmcp_b200_engine_local_dims tells which). */
uint64_t llmcp_b200_tp_slot_bytes(const llmcp_b200_dims *dims, int64_t max_tokens);
void *llmcp_b200_tp_create(int rank, int size, uint64_t slot_bytes, int device, uint8_t *handle_out);
int llmcp_b200_tp_attach(void *tp, const uint8_t *handles);
void llmcp_b200_tp_destroy(void *tp);
int llmcp_b200_tp_all_gather(void *tp, const void *src, uint64_t row_bytes, uint64_t rows, int slot, void *dst, int *status,
                             void *stream);
void *llmcp_b200_engine_create_tp(const uint8_t *file, uint64_t file_bytes, const llmcp_b200_dims *dims, int64_t capacity,
                                  int device, int mode, void *tp, int64_t max_tokens);
int llmcp_b200_engine_local_dims(void *engine, llmcp_b200_dims *dims, int64_t *kv_head0);
void llmcp_b200_engine_destroy(void *engine);
int llmcp_b200_engine_reset(void *engine);
/* One forward over host tokens (the work of lib/Runtime/AotRuntime.cpp:68-120): logits
 * (vocab f32, may be NULL) and argmax (may be NULL) of the last position. */
int llmcp_b200_engine_forward(void *engine, const int64_t *tokens, int64_t S, int64_t position, float *logits,
                              int64_t *argmax);
/* The same forward with the logits of every position: `logits` holds S x vocab f32, row s for
 * token s.  This is the result of the tensor-returning `llmcp_model` function that the
 * reference builds beside the two AOT entries (lib/Model/ModelBuilder.cpp:406-438; its runtime
 * never resolves it): final norm over all rows, then an S x vocab x hidden Q8 contraction on
 * the tensor cores.  Generation state advances as in llmcp_b200_engine_forward. */
int llmcp_b200_engine_forward_all(void *engine, const int64_t *tokens, int64_t S, int64_t position, float *logits);
/* The decode loop of tools/llmcp-benchmark/llmcp-benchmark.cpp:94-101 kept on the device:
 * token, argmax and state never leave HBM.  out_tokens: `steps` ids; device_ms: CUDA-event
 * time of the loop (may be NULL). */
int llmcp_b200_engine_generate(void *engine, int64_t first_token, int64_t position, int64_t steps,
                               int64_t *out_tokens, float *device_ms);
/* State buffers in the layouts of lib/Runtime/AotRuntime.cpp:41-43 (any may be NULL). */
int llmcp_b200_engine_read_state(void *engine, uint16_t *kv, float *delta, uint16_t *conv);
/* Final-norm output of the last position (hidden bf16) of the most recent forward. */
int llmcp_b200_engine_read_hidden(void *engine, uint16_t *hidden);

#ifdef __cplusplus
}
#endif

#endif /* LLMCP_B200_H */
