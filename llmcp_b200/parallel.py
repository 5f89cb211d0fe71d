"""Multi-GPU pieces of the path: one process per GPU over ``torch.distributed``.

The reference is single-process; what shards naturally here is (a) independent sequences
(replicas, no collective on the data path) and (b) the 248320-row tied lm_head, whose rows
split across ranks with one tiny exchange step: a (max, index) reduction that reproduces the
host argmax of tools/llmcp-benchmark/llmcp-benchmark.cpp:51-54 (the first maximum wins).

``reduce_argmax``, ``gather_rows`` and ``vocab_shard`` are backend-agnostic (gloo on CPU in the
tests, NCCL on GPUs); ``ShardedLmHead`` runs the shard's GEMV and argmax with the CUDA library.

(c) Any Q8 ``linear`` splits the same way by output rows (``ColumnParallelLinear``): a shard is a
contiguous byte range of the packed weight, every output element is computed by one rank with
the unsharded arithmetic, and one all-gather assembles the row, so the result is bit-identical
to the single-GPU product.  A split along K would change the order of the f32 additions and is
not offered.

(d) ``TensorParallel`` is the whole model split that way inside the engine (C++ / CUDA): this
module only hands the ranks each other's buffer handles; the exchanges themselves are kernels of
the library that store into the peers' memory, with no call into ``torch.distributed``.
"""
import ctypes as C

import numpy as np


def vocab_shard(vocab, world, rank):
    """Rows [begin, end) of rank ``rank``: equal shards whose size is a multiple of 8 (the packed
    layout groups rows in eights, include/llmcp/Support/Q8PackedLayout.h:38-42)."""
    if vocab % (8 * world) != 0:
        raise ValueError(f"vocabulary {vocab} does not split into {world} shards of whole 8-row groups")
    rows = vocab // world
    return rank * rows, (rank + 1) * rows


def shard_packed_rows(packed, vocab, hidden, begin, end):
    """Byte range of rows [begin, end) inside a packed q8_0_p4 table (group-major layout)."""
    if begin % 4 or end % 4:
        raise ValueError("shard boundaries must be multiples of 4 rows")
    record_bytes = (hidden // 32) * 136
    return packed[(begin // 4) * record_bytes:(end // 4) * record_bytes]


def reduce_argmax(local_value, local_index, group=None, device="cpu"):
    """All ranks contribute their shard's (maximum, global index); every rank gets the global
    first maximum: the largest value, and among equal values the lowest index."""
    import torch
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(local_value), int(local_index)
    world = dist.get_world_size(group)
    # value and index travel as two exact 64-bit words
    mine = torch.tensor([np.float64(local_value).view(np.int64), int(local_index)], dtype=torch.int64, device=device)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine, group=group)
    best_value, best_index = None, None
    for item in gathered:
        bits, index = (int(v) for v in item.cpu().tolist())
        value = float(np.int64(bits).view(np.float64))
        if best_value is None or value > best_value or (value == best_value and index < best_index):
            best_value, best_index = value, index
    return best_value, best_index


def max_over_ranks(value, device="cpu", group=None):
    import torch
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return float(value)
    t = torch.tensor([float(value)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())


class ShardedLmHead:
    """Rows [begin, end) of the tied lm_head on this rank's GPU (LowerToLinalg.cpp:729-765).

    ``packed`` is the full packed table (host numpy uint8) or this rank's slice of it.  ``step``
    quantises the final hidden row, runs the shard's decode GEMV and argmax on the device and
    returns the global (value, token) after the cross-rank reduction.
    """

    def __init__(self, packed_shard, rows, hidden, row_begin, device_index):
        import torch
        import llmcp_b200 as L
        self.torch, self.L, self.lib = torch, L, L.lib()
        self.rows, self.hidden, self.row_begin = rows, hidden, row_begin
        self.device = torch.device("cuda", device_index)
        nb = hidden // 32
        with torch.cuda.device(self.device):
            records = torch.from_numpy(np.ascontiguousarray(packed_shard)).to(self.device)
            self.wq = torch.empty((rows, hidden), dtype=torch.int8, device=self.device)
            self.wd = torch.empty((rows, nb), dtype=torch.float16, device=self.device)
            self.aq = torch.empty(hidden, dtype=torch.int8, device=self.device)
            self.scales = torch.empty(nb, dtype=torch.float32, device=self.device)
            self.logits = torch.empty(rows, dtype=torch.float32, device=self.device)
            self.part_v = torch.empty(512, dtype=torch.float32, device=self.device)
            self.part_i = torch.empty(512, dtype=torch.int64, device=self.device)
            self.best = torch.empty(1, dtype=torch.int64, device=self.device)
            stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            self._check(self.lib.llmcp_dev_repack_q8(self._p(records), C.c_int64(rows), C.c_int64(hidden),
                                                     self._p(self.wq), self._p(self.wd), stream))
            torch.cuda.synchronize()

    @staticmethod
    def _p(t):
        return C.c_void_p(t.data_ptr())

    def _check(self, code):
        if code != 0:
            raise self.L.LlmcpError(self.L.last_error())

    def step(self, hidden_bf16_bits, group=None):
        torch = self.torch
        with torch.cuda.device(self.device):
            h = torch.from_numpy(np.ascontiguousarray(hidden_bf16_bits, dtype=np.uint16).view(np.int16)).to(self.device)
            stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            self._check(self.lib.llmcp_dev_act_quant(self._p(h), 1, C.c_int64(1), C.c_int64(self.hidden),
                                                     self._p(self.aq), self._p(self.scales), stream))
            self._check(self.lib.llmcp_dev_gemv_q8(self._p(self.aq), self._p(self.scales), C.c_int64(self.hidden),
                                                   self._p(self.wq), self._p(self.wd), C.c_int64(self.rows),
                                                   self._p(self.logits), 0, 0, 0, 0, stream))
            self._check(self.lib.llmcp_dev_argmax(self._p(self.logits), C.c_int64(self.rows), self._p(self.part_v),
                                                  self._p(self.part_i), self._p(self.best), stream))
            torch.cuda.synchronize()
            index = int(self.best.item())
            value = float(self.logits[index].item())
        return reduce_argmax(value, self.row_begin + index, group=group, device=self.device)


def gather_rows(local, group=None):
    """All-gather of equally sized 1-D shards (a torch tensor per rank, CPU with gloo or CUDA with
    NCCL) into the full row, in rank order."""
    import torch
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local
    world = dist.get_world_size(group)
    # Moved as bytes: nothing is computed on the way, and NCCL has no 16-bit integer type for
    # the bf16 bit patterns.
    raw = local.contiguous().view(torch.uint8)
    out = torch.empty(world * raw.numel(), dtype=torch.uint8, device=local.device)
    dist.all_gather_into_tensor(out, raw, group=group)
    return out.view(local.dtype)


class ColumnParallelLinear:
    """Rows [begin, end) of a Q8 ``linear`` on this rank's GPU (one-token form, Q8Decode.cpp:131-225).

    ``packed_shard`` is this rank's slice of the packed weight (``shard_packed_rows``).  ``local``
    quantises the input row and runs the shard's GEMV with the fused epilogue; ``forward`` adds the
    all-gather.  Outputs are bf16 bit patterns (int16 tensors) or float32.
    """

    def __init__(self, packed_shard, rows, K, device_index, y_bf16=True, activation="none"):
        import torch
        import llmcp_b200 as L
        self.torch, self.L, self.lib = torch, L, L.lib()
        self.rows, self.K, self.y_bf16 = rows, K, y_bf16
        self.activation = L.ACTIVATIONS[activation]
        self.device = torch.device("cuda", device_index)
        nb = K // 32
        with torch.cuda.device(self.device):
            records = torch.from_numpy(np.ascontiguousarray(packed_shard)).to(self.device)
            self.wq = torch.empty((rows, K), dtype=torch.int8, device=self.device)
            self.wd = torch.empty((rows, nb), dtype=torch.float16, device=self.device)
            self.aq = torch.empty(K, dtype=torch.int8, device=self.device)
            self.scales = torch.empty(nb, dtype=torch.float32, device=self.device)
            self.y = torch.empty(rows, dtype=torch.int16 if y_bf16 else torch.float32, device=self.device)
            stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            self._check(self.lib.llmcp_dev_repack_q8(self._p(records), C.c_int64(rows), C.c_int64(K),
                                                     self._p(self.wq), self._p(self.wd), stream))
            torch.cuda.synchronize()

    @staticmethod
    def _p(t):
        return C.c_void_p(t.data_ptr())

    def _check(self, code):
        if code != 0:
            raise self.L.LlmcpError(self.L.last_error())

    def local(self, x_bf16_bits):
        torch = self.torch
        with torch.cuda.device(self.device):
            x = torch.from_numpy(np.ascontiguousarray(x_bf16_bits, dtype=np.uint16).view(np.int16)).to(self.device)
            stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            self._check(self.lib.llmcp_dev_act_quant(self._p(x), 1, C.c_int64(1), C.c_int64(self.K), self._p(self.aq),
                                                     self._p(self.scales), stream))
            self._check(self.lib.llmcp_dev_gemv_q8(self._p(self.aq), self._p(self.scales), C.c_int64(self.K),
                                                   self._p(self.wq), self._p(self.wd), C.c_int64(self.rows),
                                                   self._p(self.y), int(self.y_bf16), self.activation, 0, 0, stream))
            torch.cuda.synchronize()
        return self.y

    def forward(self, x_bf16_bits, group=None):
        return gather_rows(self.local(x_bf16_bits), group=group)


class TensorParallel:
    """A tensor-parallel group of engines, one process per GPU (llmcp_b200_tp_* in
    include/llmcp_b200.h).  Creating it allocates this rank's exchange buffer and swaps the
    CUDA IPC handles of all ranks through ``torch.distributed`` (the only use of it: any other
    channel that moves 64 bytes per rank would do).  Pass it to ``llmcp_b200.Engine(..., tp=group)``.
    """

    def __init__(self, dims, rank, world, device, max_tokens=1024, group=None):
        import torch.distributed as dist
        import llmcp_b200 as L
        lib = L.lib()
        self.rank, self.world, self.max_tokens = rank, world, max_tokens
        slot_bytes = int(lib.llmcp_b200_tp_slot_bytes(C.byref(dims), C.c_int64(max_tokens)))
        mine = (C.c_uint8 * 64)()
        handle = lib.llmcp_b200_tp_create(int(rank), int(world), C.c_uint64(slot_bytes), int(device), mine)
        if not handle:
            raise L.LlmcpError(L.last_error())
        self.handle = C.c_void_p(handle)
        if world > 1:
            handles = [None] * world
            dist.all_gather_object(handles, bytes(mine), group=group)
            blob = b"".join(handles)
            if lib.llmcp_b200_tp_attach(self.handle, blob) != 0:
                raise L.LlmcpError(L.last_error())

    def all_gather(self, src, slot, stream=0):
        """The exchange alone (for tests): ``src`` is a torch CUDA tensor [rows, cols] of this rank;
        returns [rows, world * cols]."""
        import torch
        import llmcp_b200 as L
        rows, cols = src.shape
        row_bytes = cols * src.element_size()
        out = torch.empty((rows, self.world * cols), dtype=src.dtype, device=src.device)
        status = torch.zeros(1, dtype=torch.int32, device=src.device)
        rc = L.lib().llmcp_b200_tp_all_gather(self.handle, C.c_void_p(src.data_ptr()), C.c_uint64(row_bytes), C.c_uint64(rows),
                                              int(slot), C.c_void_p(out.data_ptr()), C.c_void_p(status.data_ptr()),
                                              C.c_void_p(stream or torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise L.LlmcpError(L.last_error())
        torch.cuda.synchronize()
        if int(status.item()) != 0:
            raise L.LlmcpError("all-gather: a peer's flag did not arrive within the wait limit")
        return out

    def close(self):
        import llmcp_b200 as L
        if self.handle:
            L.lib().llmcp_b200_tp_destroy(self.handle)
            self.handle = None
