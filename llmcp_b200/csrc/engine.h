// Model executor: owns the device copy of a packed arena (weights re-laid out for the GPU),
// the device-resident generation state, the activation workspace, and runs the graph of
// lib/Model/ModelBuilder.cpp:218-526 (after FuseLinearActivations.cpp:27-77) with the kernels
// of this library.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "format.h"

namespace llmcp_b200 {

class TpComm;

struct Q8Weight {
  int8_t *q = nullptr;   // [N][K]
  uint16_t *d = nullptr; // [N][K/32] f16 bits
  float *d32 = nullptr;  // [N][K/32] the same scales as f32 (tensor-core GEMM, int8 form)
  void *h = nullptr;     // [N][K] the integers as f16 values (tensor-core GEMM, f16 form)
  float *d32t = nullptr; // [K/32][N] the scales as f32, block-major (tensor-core GEMM, f16 form)
  const uint16_t *bf = nullptr; // [N][K] bf16: the matrix of an unquantised arena (q, d unused then)
  int N = 0, K = 0;
};

struct SmallTensor {
  void *data = nullptr;
  int dtype = 0; // DType
};

struct LayerWeights {
  bool full = false;
  SmallTensor input_norm, post_norm;
  Q8Weight qkv, z, a, b, out_proj;
  SmallTensor conv, dt_bias, a_log, lin_norm;
  Q8Weight q_proj, k_proj, v_proj, o_proj;
  SmallTensor q_norm, k_norm;
  Q8Weight gate, up, down;
};

// Prefill GEMM forms by name ("dp4a", "i8-cpasync", "i8", "i8x2", "f16", "f16x2"; see kernels.h GemmForm).
constexpr int kDefaultGemmKind = 2 + 1; // TMA-fed int8 planes (nothing beside the GEMV's planes), packed arithmetic
int gemm_kind_from_name(const char *name);

// Arithmetic mode of an engine.
//   kModeExact: every f32 result is bit-identical to the reference's order of operations.
//   kModeFast : the integer block dots, the quantisation and the rounding points are unchanged, but
//               reductions whose order only affects f32 rounding (rms_norm's sum of squares, a GEMV
//               row's sum over blocks, the attention softmax over keys of the one-token step) are
//               evaluated as parallel trees.  Logits agree with the exact mode within 1e-2.
enum Mode : int { kModeExact = 0, kModeFast = 1 };
// Mode of engines created without an explicit one: LLMCP_B200_MODE=fast|exact in the environment,
// else what set_default_mode() last stored, else exact.
int default_mode();
void set_default_mode(int mode);

class Engine {
public:
  // `base` points at the first byte of a mapped container (header, arena, manifest).
  // mode: kModeExact, kModeFast, or -1 for default_mode().
  // Throws std::runtime_error with a readable message on any failure.
  // tp: exchange context of a tensor-parallel group (null or size 1: the whole model on this GPU).
  // A rank of size G holds 1/G of every projection's output rows, 1/G of the recurrent and
  // attention heads (KV heads are duplicated when G exceeds their number) and 1/G of the
  // vocabulary projection; every rank must make the same calls.  max_tokens bounds the rows of one
  // call under tensor parallelism (the exchange slots are sized for it).
  // batch: number of independent sequences the engine keeps state for (1: the reference's case).
  // Sequences are prefilled one at a time (forward_host after select_sequence) and can then be
  // decoded together, one token each per step, at a common position (decode_batch / generate_batch):
  // the projections then run as one contraction of `batch` rows on the tensor cores, recurrent state,
  // convolution state and KV cache stay per sequence.
  Engine(const uint8_t *base, uint64_t file_bytes, const ModelDims &dims, int64_t capacity, int device, int mode = -1,
         TpComm *tp = nullptr, int64_t max_tokens = 1024, int batch = 1);
  // Bytes per exchange slot an engine with these dimensions needs for calls of up to max_tokens rows.
  static size_t tp_slot_bytes(const ModelDims &dims, int64_t max_tokens);
  // Why these dimensions cannot be split over `size` ranks, or "" if they can.
  static std::string tp_unsupported(const ModelDims &dims, int size);
  ~Engine();
  Engine(const Engine &) = delete;
  Engine &operator=(const Engine &) = delete;

  const ModelDims &dims() const { return dims_; }
  // Dimensions of this rank's share: head counts divided by the group size (state buffers and
  // upload_state / download_state use these); hidden, intermediate and vocab stay global.
  const ModelDims &local_dims() const { return local_; }
  int64_t kv_head0() const { return kv_head0_; } // first KV head of this rank
  int tp_rank() const { return tp_rank_; }
  int tp_size() const { return tp_size_; }
  int64_t capacity() const { return capacity_; }
  int device() const { return device_; }
  int mode() const { return mode_; }
  cudaStream_t stream() const { return stream_; }

  int batch() const { return batch_; }
  // The sequence whose state forward_host / forward_all_host / generate / upload_state /
  // download_state address (0 after construction).
  void select_sequence(int sequence);
  // One token of every sequence, all at `position`: tokens_host[batch] in; the argmax of every
  // sequence's logits to argmax_host[batch] and, if not null, the logits rows to
  // logits_host[batch][vocab].
  void decode_batch(const int64_t *tokens_host, int64_t position, float *logits_host, int64_t *argmax_host);
  // Greedy decoding of all sequences on the device for `steps` steps from `position`:
  // out_tokens_host[steps][batch]; device_ms, if not null, the CUDA-event time of the loop.
  void generate_batch(const int64_t *first_tokens_host, int64_t position, int64_t steps, int64_t *out_tokens_host,
                      float *device_ms);
  void reset_state();
  // Host <-> device copies of the three state buffers in the reference's layouts:
  // kv [full, 2, kv_heads, capacity, head_dim] bf16, delta [linear, v_heads, k_dim, v_dim] f32,
  // conv [linear, kernel-1, qkv_dim] bf16.
  void upload_state(const uint16_t *kv, const float *delta, const uint16_t *conv);
  void download_state(uint16_t *kv, float *delta, uint16_t *conv);

  // One AOT entry call with host buffers: S tokens starting at `position`; writes the last
  // position's logits (vocab f32) to `logits_host` if not null and returns its argmax.
  // cos/sin may be null, in which case the rows are computed from the position.
  int64_t forward_host(const int64_t *tokens, int64_t S, int64_t position, const float *cos, const float *sin,
                       float *logits_host);

  // The same forward, but the logits of every position are written: logits_host holds
  // S x vocab floats (the result of the reference's tensor-returning `llmcp_model`,
  // lib/Model/ModelBuilder.cpp:406-438).  State advances exactly as in forward_host.
  void forward_all_host(const int64_t *tokens, int64_t S, int64_t position, float *logits_host);

  // Greedy generation that never leaves the device: feeds `first_token` at `position`, then
  // each step's argmax to the next, for `steps` steps.  out_tokens_host (steps entries) gets
  // the argmax of every step; device_ms, if not null, the CUDA-event time of the loop.
  void generate(int64_t first_token, int64_t position, int64_t steps, int64_t *out_tokens_host, float *device_ms);

  // Device pointers for inspection by tests.
  const float *logits_device() const { return logits_; }
  const uint16_t *final_hidden_device() const { return final_hidden_; }

  uint64_t launches() const { return launches_; }

private:
  void release() noexcept; // frees everything the engine holds; safe on a half-built engine
  void validate_tokens(const int64_t *tokens, int64_t S) const;
  void check_status(); // throws if the device status word copied to token_pinned_ is non-zero
  void rms_norm(const uint16_t *a, const uint16_t *b, int64_t S, const SmallTensor &w, uint16_t *sum_out, uint16_t *y);
  void load_weights(const uint8_t *base, const Manifest &manifest);
  void ensure_workspace(int64_t S, int64_t position);
  // Enqueues one forward over S tokens whose ids are at tokens_dev.  The start position is read
  // from position_dev_ by the kernels; max_position bounds it (grid and scratch sizing).  cos/sin
  // are the rows of this call, or tables over all positions when rows_from_position is set.
  // rows_are_sequences: the S rows are one token each of the engine's `batch` sequences (S == batch).
  void run(const int64_t *tokens_dev, int64_t S, int64_t max_position, const float *cos_dev, const float *sin_dev,
           int rows_from_position, bool rows_are_sequences = false);
  void set_position(int64_t position);
  // The single-token forward over the staging buffers (tokens_, cos_, sin_, position_dev_),
  // captured once as a CUDA graph and replayed for every decode step.
  void decode_step();
  void linear(const Q8Weight &w, int64_t S, void *y, int y_dtype, int activation);
  void check(cudaError_t e, const char *what);

  // Tensor parallelism: all-gathers of quantised rows (int8 + scales) and of bf16 rows.
  void gather_quant(int64_t S, int64_t k_local, const int8_t **q, const float **s, const int8_t *src_q = nullptr,
                    const float *src_s = nullptr);
  const uint16_t *gather_rows(const uint16_t *src, int64_t S, int64_t n_local);

  ModelDims dims_;
  ModelDims local_;
  TpComm *tp_ = nullptr;
  int tp_rank_ = 0, tp_size_ = 1;
  int64_t max_tokens_ = 1024;
  int64_t kv_head0_ = 0;   // first KV head of this rank
  int64_t hidden_rows_ = 0, inter_rows_ = 0, vocab_rows_ = 0, vocab_row0_ = 0; // this rank's output rows
  int batch_ = 1, sequence_ = 0;
  size_t kv_seq_ = 0, delta_seq_ = 0, conv_seq_ = 0; // elements of one sequence's state buffers
  float *batch_logits_ = nullptr;   // [batch][vocab] logits of a batched step
  int64_t *batch_tokens_ = nullptr; // [batch] argmax of a batched step (device)
  int exchange_ = 0;       // exchanges issued so far by the running forward (slot rule of TpComm)
  bool gather_logits_ = false; // tensor parallel: the next forward also assembles the full logits row
  Q8Weight lm_head_;       // the rows of the tied table this rank multiplies (a view into embed_)
  uint8_t *argmax_pair_ = nullptr; // {f32 maximum, pad, i64 index} of this rank's logits
  int64_t capacity_ = 0;
  int device_ = 0;
  int mode_ = kModeExact;
  cudaStream_t stream_ = nullptr;
  // Independent GEMMs of a prefill (the projections that share an input) can run side by side: a
  // fork event on stream_, one side stream and one join event per extra matrix
  // (LLMCP_B200_CONCURRENT_GEMMS=0|1).  On for a batch of sequences; off for a single sequence: it
  // takes 3 ms off a 1024-token prefill, but in fast mode every decode step that follows in the same
  // process then measured 75 us longer, also when the streams are destroyed right after the
  // prefill; the cause was not found.
  static constexpr int kSideStreams = 3;
  cudaStream_t side_streams_[kSideStreams] = {};
  cudaEvent_t fork_event_ = nullptr, join_events_[kSideStreams] = {};
  bool concurrent_gemms_ = false;
  void make_side_streams();
  void drop_side_streams() noexcept;
  uint64_t launches_ = 0;

  std::vector<void *> allocations_;
  std::vector<LayerWeights> layers_;
  Q8Weight embed_;
  SmallTensor final_norm_;

  // state
  uint16_t *kv_ = nullptr;
  float *delta_ = nullptr;
  uint16_t *conv_ = nullptr;
  float *cos_table_ = nullptr, *sin_table_ = nullptr; // [capacity, rotary]

  // workspace (sized for ws_tokens_ rows)
  int64_t ws_tokens_ = 0;
  size_t attn_scratch_bytes_ = 0;
  int64_t *tokens_ = nullptr;
  float *cos_ = nullptr, *sin_ = nullptr;
  uint16_t *hidden_[2] = {nullptr, nullptr};
  uint16_t *branch_ = nullptr, *mlp_out_ = nullptr;
  int8_t *aq_ = nullptr;
  float *as_ = nullptr;
  uint16_t *qkv_ = nullptr, *z_ = nullptr, *a_ = nullptr, *b_ = nullptr, *convd_ = nullptr, *gdn_ = nullptr;
  uint16_t *qg_ = nullptr, *k_ = nullptr, *v_ = nullptr, *attn_ = nullptr;
  uint16_t *gate_ = nullptr, *up_ = nullptr;
  float *gdn_scratch_ = nullptr;
  void *attn_scratch_ = nullptr;
  std::vector<void *> ws_allocations_;

  // outputs
  uint16_t *final_hidden_ = nullptr; // [hidden] last row after the final norm
  float *logits_ = nullptr;          // [vocab]
  float *all_logits_ = nullptr;      // [S, vocab] while forward_all_host runs, else null
  float *argmax_v_ = nullptr;
  int64_t *argmax_i_ = nullptr;
  int64_t *next_token_ = nullptr; // device scalar
  int64_t *generated_ = nullptr;  // device [capacity]
  float *logits_pinned_ = nullptr;
  int64_t *token_pinned_ = nullptr;
  int64_t *position_dev_ = nullptr; // device scalar: start position of the running call
  // Inputs of the one-token step behind position_dev_ in one device block: token, cos row, sin row.
  int64_t *dec_tokens_ = nullptr;
  float *dec_cos_ = nullptr, *dec_sin_ = nullptr;
  size_t step_block_bytes_ = 0;
  int64_t *step_dev_ = nullptr;     // device scalar: index into generated_
  int64_t *position_pinned_ = nullptr; // pinned packet with the layout of the block at position_dev_
  cudaGraphExec_t decode_graph_ = nullptr;
  uint64_t decode_graph_launches_ = 0;
  bool use_graph_ = true;
  bool use_tensor_cores_ = true;
  int gemm_kind_ = kDefaultGemmKind; // prefill GEMM form, see gemm_kind_from_name()
  void *ah_ = nullptr;    // [rows][max K] activations as f16 values (GEMM kind 2)
  float *ast_ = nullptr;  // [max K / 32][pitch] their scales, block-major
  int *gemm_error_ = nullptr; // device flag raised by a timed-out wait in the GEMM
  int gemv_flags_ = 3; // kGemvOverlapPrevious | kGemvPrefetchL2
  bool bf16_weights_ = false;   // unquantised arena: bf16 matrices, bf16 activations between operators
  uint16_t *xb_ = nullptr;      // bf16 input rows of the next linear (bf16 arenas)
  bool tc_prefill_attention_ = true; // fast mode, more than one token: attention contractions on the tensor cores
  bool fuse_swiglu_ = true;   // one-token MLP: gate, up, product and quantisation in one launch
  bool prefetch_next_ = true; // one token: a GEMV asks for the next GEMV's weights in L2 while it runs
  // one-token gated-delta-net layers: 0 five launches, 1 two, 2 one (a cluster per key head; measured
  // slower than two: the recurrent state can then be fetched only after the projections have finished)
  int fuse_decode_mixer_ = 1;
};

} // namespace llmcp_b200
