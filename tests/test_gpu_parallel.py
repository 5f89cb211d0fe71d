"""Vocabulary-sharded lm_head on two GPUs (NCCL): every rank runs the decode GEMV and argmax of
its rows with the CUDA library, one (max, index) exchange gives the token the unsharded host
argmax of tools/llmcp-benchmark/llmcp-benchmark.cpp:51-54 picks."""
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
        results[rank] = (value, token, float(full.max()), oracle.argmax(full), np.array_equal(local, full[begin:end]))
    finally:
        dist.destroy_process_group()


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
