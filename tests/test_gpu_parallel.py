"""Row-sharded Q8 linears on two GPUs (NCCL).  The vocabulary-sharded lm_head: every rank runs the
decode GEMV and argmax of its rows with the CUDA library, one (max, index) exchange gives the
token the unsharded host argmax of tools/llmcp-benchmark/llmcp-benchmark.cpp:51-54 picks.  A
column-parallel layer projection: the all-gathered row equals the unsharded operator's output."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import llmcp_b200 as L
    from llmcp_b200 import parallel
    torch.cuda.set_device(rank)
    L.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        rng = np.random.default_rng(11)
        vocab, hidden = 4096, 2560
        w = (rng.standard_normal((vocab, hidden)) * 0.02).astype(np.float32)
        w[3000] = w[700]  # equal logits on two ranks: the lower index has to win
        packed = oracle.pack_q8_0_p4(w)
        h = oracle.f32_to_bf16(rng.standard_normal((1, hidden)).astype(np.float32))
        h[0] = oracle.f32_to_bf16(oracle.bf16_to_f32(h[0]) + 4.0 * np.sign(w[700]))
        begin, end = parallel.vocab_shard(vocab, world, rank)
        shard = parallel.shard_packed_rows(packed, vocab, hidden, begin, end)
        head = parallel.ShardedLmHead(shard, end - begin, hidden, begin, rank)
        value, token = head.step(h[0])
        full = oracle.linear_q8(h, packed, vocab, y_bf16=False)[0]
        local = head.logits.cpu().numpy()
        # a column-parallel layer projection with its fused epilogue: the gathered row equals the
        # unsharded operator's output bit for bit
        n_rows = 9216
        wl = (rng.standard_normal((n_rows, hidden)) * 0.02).astype(np.float32)
        packed_l = oracle.pack_q8_0_p4(wl)
        lb, le = parallel.vocab_shard(n_rows, world, rank)
        layer = parallel.ColumnParallelLinear(parallel.shard_packed_rows(packed_l, n_rows, hidden, lb, le), le - lb,
                                              hidden, rank, y_bf16=True, activation="silu")
        row = layer.forward(h[0]).cpu().numpy().view(np.uint16)
        want_row = oracle.linear_q8(h, packed_l, n_rows, y_bf16=True, activation="silu")[0]
        results[rank] = (value, token, float(full.max()), oracle.argmax(full),
                         np.array_equal(local, full[begin:end]) and np.array_equal(row, want_row))
    finally:
        dist.destroy_process_group()


def test_column_parallel_shards_on_one_gpu():
    """Both shards of a column-parallel linear computed on one device and concatenated: the
    sharding arithmetic without a second GPU (K = 9216 and 2560, bf16 and f32 outputs)."""
    from llmcp_b200 import parallel
    rng = np.random.default_rng(3)
    for n_rows, K, y_bf16, activation in ((2560, 9216, True, "none"), (4096, 2560, False, "sigmoid")):
        w = (rng.standard_normal((n_rows, K)) * 0.02).astype(np.float32)
        packed = oracle.pack_q8_0_p4(w)
        x = oracle.f32_to_bf16(rng.standard_normal((1, K)).astype(np.float32))
        parts = []
        for rank in range(2):
            begin, end = parallel.vocab_shard(n_rows, 2, rank)
            layer = parallel.ColumnParallelLinear(parallel.shard_packed_rows(packed, n_rows, K, begin, end), end - begin, K,
                                                  0, y_bf16=y_bf16, activation=activation)
            parts.append(layer.forward(x[0]).cpu().numpy())
        got = np.concatenate(parts)
        want = oracle.linear_q8(x, packed, n_rows, y_bf16=y_bf16, activation=activation)[0]
        assert np.array_equal(got.view(np.uint16) if y_bf16 else got, want)


def test_sharded_lm_head_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert len(results) == world
        for rank in range(world):
            value, token, want_value, want_token, shard_equal = results[rank]
            assert shard_equal, "a rank's logits must equal its rows of the unsharded product"
            assert token == want_token == 700 and value == want_value
