// Exchange step of the tensor-parallel engine: one process per GPU, every rank holds a buffer that
// its peers map through CUDA IPC, and an all-gather is one kernel per rank that stores the rank's
// piece straight into every peer's buffer over NVLink, publishes a flag and waits (bounded) for
// the peers' flags.  No NCCL, no host round trip: the kernel is enqueued on the engine's stream
// and is part of the captured decode step.
//
// The reference is single-process (there is nothing to cite for the exchange itself); what is
// exchanged are the outputs of the row-sharded linears of lib/Model/ModelBuilder.cpp:218-319.
#pragma once

#include <cstddef>
#include <cstdint>

#include <cuda_runtime.h>

namespace llmcp_b200 {

constexpr int kTpMaxRanks = 8;
constexpr int kTpSlots = 3;          // gathered results land in one of these slots (chosen by the caller)
constexpr int kTpMaxSegments = 3;    // pieces of one exchange (e.g. int8 values and their scales)
constexpr size_t kTpHandleBytes = 64; // sizeof(cudaIpcMemHandle_t)

// One matrix of an exchange: this rank contributes `rows` rows of `row_bytes` bytes (its columns of
// every row); the gathered matrix has rows of size * row_bytes bytes with the ranks' columns in
// rank order, starting `offset` bytes into the slot.
struct TpSegment {
  const void *src;   // this rank's piece [rows][row_bytes] (device memory of this rank)
  size_t row_bytes;  // a multiple of 16
  size_t rows;
  size_t offset;     // a multiple of 16
};

class TpComm {
public:
  // Allocates this rank's buffer (slots * slot_bytes of data plus the flag words) on the current
  // device and fills `handle` (kTpHandleBytes) for the peers.  Throws std::runtime_error on failure.
  TpComm(int rank, int size, size_t slot_bytes, void *handle);
  ~TpComm();
  TpComm(const TpComm &) = delete;
  TpComm &operator=(const TpComm &) = delete;

  // Maps the peers' buffers: handles holds `size` handles of kTpHandleBytes, in rank order.
  void attach(const void *handles);

  int rank() const { return rank_; }
  int size() const { return size_; }
  size_t slot_bytes() const { return slot_bytes_; }
  // Start of slot `slot` of this rank's buffer.
  uint8_t *slot(int slot) const { return local_ + static_cast<size_t>(slot) * slot_bytes_; }

  // Enqueues one all-gather of up to kTpMaxSegments segments into slot `slot`: afterwards that slot
  // of every rank holds every segment's gathered matrix.  status (device int, optional): bit 2 (value 4) is raised
  // if a peer's flag did not arrive within the wait limit.  Every rank must issue the same
  // sequence of calls.  Slot rule: a peer may already be writing exchange e + 1 while this rank
  // still reads the result of exchange e, so consecutive exchanges must name different slots, and
  // a result has to be consumed (by kernels enqueued) before the exchange after the next one.
  // A call captured into a CUDA graph may be replayed: the exchange number lives in device
  // memory and advances with every execution.
  cudaError_t all_gather(const TpSegment *segments, int count, int slot, int *status, cudaStream_t stream);

private:
  int rank_, size_;
  size_t slot_bytes_;
  uint8_t *local_ = nullptr;
  uint8_t *peer_[kTpMaxRanks] = {};
  unsigned int *flags_ = nullptr; // [kTpSlots][kTpMaxRanks] inside local_
  unsigned int *count_dev_ = nullptr; // exchanges completed so far (device word)
  bool attached_ = false;
};

} // namespace llmcp_b200
