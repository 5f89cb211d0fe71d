#include "tp_comm.h"

#include <cstring>
#include <stdexcept>
#include <string>

#include "common.cuh"

namespace llmcp_b200 {

namespace {

constexpr unsigned int kTpSpinLimit = 1u << 24; // polls of a peer's flag before giving up (about a second)

struct GatherArgs {
  TpSegment segment[kTpMaxSegments];
  int count;
  uint8_t *peer[kTpMaxRanks]; // every rank's buffer as mapped here (peer[rank] is the local one)
  int rank, size, slot;
  size_t slot_bytes;
  unsigned int *flags;        // local [kTpSlots][kTpMaxRanks]
  size_t flags_offset;        // of the flag words inside a buffer
  unsigned int *count_dev;    // local: exchanges completed
  int *status;
};

// One CTA.  Phase 1: this rank's pieces go to the same place of every rank's slot (peer stores, 16
// bytes per thread and step).  Phase 2: after a system-wide fence, the exchange number is stored
// into this rank's flag word in every peer's buffer.  Phase 3: wait until every peer's flag word in
// the local buffer has reached the exchange number; the pieces that belong to it were stored, and
// fenced, before it.
__global__ void __launch_bounds__(1024)
tp_all_gather_kernel(const GatherArgs a) {
  // The pieces are written by the kernel in front.  The kernel behind (usually a projection that
  // reads the gathered rows) is released at once: it is placed and requests its weights while the
  // exchange is under way, and reads the rows only after this kernel has finished.
  grid_dependency_sync(true);
  const unsigned int number = *a.count_dev + 1;
  const int t = threadIdx.x;
  for (int g = 0; g < a.count; ++g) {
    const TpSegment seg = a.segment[g];
    const size_t per_row = seg.row_bytes / 16, vectors = per_row * seg.rows;
    const uint4 *src = static_cast<const uint4 *>(seg.src);
    for (size_t i = t; i < vectors * a.size; i += blockDim.x) {
      const int peer = static_cast<int>(i / vectors);
      const size_t v = i - peer * vectors, row = v / per_row, col = v - row * per_row;
      uint4 *dst = reinterpret_cast<uint4 *>(a.peer[peer] + static_cast<size_t>(a.slot) * a.slot_bytes + seg.offset +
                                             (row * a.size + a.rank) * seg.row_bytes);
      dst[col] = src[v];
    }
  }
  __threadfence_system();
  __syncthreads();
  if (t < a.size) {
    volatile unsigned int *flag =
        reinterpret_cast<volatile unsigned int *>(a.peer[t] + a.flags_offset) + a.slot * kTpMaxRanks + a.rank;
    *flag = number;
  }
  bool ok = true;
  if (t < a.size) {
    volatile unsigned int *flag = a.flags + a.slot * kTpMaxRanks + t;
    unsigned int spin = 0;
    while (static_cast<int>(*flag - number) < 0) {
      if (++spin > kTpSpinLimit) {
        ok = false;
        break;
      }
    }
    __threadfence_system(); // the pieces stored before the flag are visible to the kernels behind
  }
  if (!ok && a.status)
    atomicOr(a.status, 4);
  __syncthreads();
  if (t == 0)
    *a.count_dev = number;
}

void check(cudaError_t e, const char *what) {
  if (e != cudaSuccess)
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

} // namespace

TpComm::TpComm(int rank, int size, size_t slot_bytes, void *handle) : rank_(rank), size_(size) {
  if (size < 1 || size > kTpMaxRanks || rank < 0 || rank >= size)
    throw std::runtime_error("tensor parallel: rank / size out of range (at most 8 ranks)");
  slot_bytes_ = (slot_bytes + 255) / 256 * 256;
  const size_t data = slot_bytes_ * kTpSlots;
  const size_t total = data + 256 /* flags */ + 256 /* counter */;
  check(cudaMalloc(&local_, total), "cudaMalloc(exchange buffer)");
  check(cudaMemset(local_, 0, total), "cudaMemset(exchange buffer)");
  flags_ = reinterpret_cast<unsigned int *>(local_ + data);
  count_dev_ = reinterpret_cast<unsigned int *>(local_ + data + 256);
  peer_[rank] = local_;
  static_assert(sizeof(cudaIpcMemHandle_t) == kTpHandleBytes, "IPC handle size");
  if (handle) {
    cudaIpcMemHandle_t h;
    check(cudaIpcGetMemHandle(&h, local_), "cudaIpcGetMemHandle");
    std::memcpy(handle, &h, sizeof(h));
  }
  if (size == 1)
    attached_ = true;
}

TpComm::~TpComm() {
  for (int r = 0; r < size_; ++r)
    if (r != rank_ && peer_[r])
      cudaIpcCloseMemHandle(peer_[r]);
  if (local_)
    cudaFree(local_);
}

void TpComm::attach(const void *handles) {
  if (attached_)
    return;
  for (int r = 0; r < size_; ++r) {
    if (r == rank_)
      continue;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, static_cast<const uint8_t *>(handles) + static_cast<size_t>(r) * kTpHandleBytes, sizeof(h));
    void *p = nullptr;
    check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    peer_[r] = static_cast<uint8_t *>(p);
  }
  attached_ = true;
}

cudaError_t TpComm::all_gather(const TpSegment *segments, int count, int slot, int *status, cudaStream_t stream) {
  if (!attached_ || count < 1 || count > kTpMaxSegments || slot < 0 || slot >= kTpSlots)
    return cudaErrorInvalidValue;
  GatherArgs a{};
  a.count = count;
  size_t largest = 0;
  for (int g = 0; g < count; ++g) {
    a.segment[g] = segments[g];
    const size_t bytes = segments[g].row_bytes * segments[g].rows;
    if (segments[g].row_bytes % 16 || segments[g].offset % 16 || segments[g].offset + bytes * size_ > slot_bytes_)
      return cudaErrorInvalidValue;
    largest = std::max(largest, bytes * size_);
  }
  for (int r = 0; r < size_; ++r)
    a.peer[r] = peer_[r];
  a.rank = rank_;
  a.size = size_;
  a.slot = slot;
  a.slot_bytes = slot_bytes_;
  a.flags = flags_;
  a.flags_offset = slot_bytes_ * kTpSlots;
  a.count_dev = count_dev_;
  a.status = status;
  const int threads = static_cast<int>(std::min<size_t>(1024, std::max<size_t>(64, (largest / 16 + 31) / 32 * 32)));
  launch_chained(tp_all_gather_kernel, dim3(1), dim3(threads), 0, stream, a);
  return cudaGetLastError();
}

} // namespace llmcp_b200
