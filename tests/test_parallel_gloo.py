"""The multi-rank host logic on CPU ranks (gloo, world size 2): vocabulary sharding of the
packed table and the (max, index) reduction that stands for the host argmax."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from llmcp_b200 import parallel


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.default_rng(5)
        vocab, hidden = 64, 96
        w = (rng.standard_normal((vocab, hidden)) * 0.02).astype(np.float32)
        w[40] = w[9]  # equal logits on two ranks: the lower index has to win
        packed = oracle.pack_q8_0_p4(w)
        h = oracle.f32_to_bf16(rng.standard_normal((1, hidden)).astype(np.float32))
        h[0] = oracle.f32_to_bf16(oracle.bf16_to_f32(h[0]) + 4.0 * np.sign(w[9]))  # make row 9 / 40 the maximum
        begin, end = parallel.vocab_shard(vocab, world, rank)
        shard = parallel.shard_packed_rows(packed, vocab, hidden, begin, end)
        local = oracle.linear_q8(h, shard, end - begin, y_bf16=False)[0]
        index = oracle.argmax(local)
        value, token = parallel.reduce_argmax(local[index], begin + index)
        full = oracle.linear_q8(h, packed, vocab, y_bf16=False)[0]
        slowest = parallel.max_over_ranks(float(rank + 1))
        # a column-parallel linear: every rank's rows, gathered in rank order, are the unsharded row
        row = parallel.gather_rows(torch.from_numpy(local.copy())).numpy()
        bits = torch.from_numpy(oracle.f32_to_bf16(local).view(np.int16).copy())  # bf16 bit patterns travel as int16
        row16 = parallel.gather_rows(bits).numpy().view(np.uint16)
        gathered = np.array_equal(row, full) and np.array_equal(row16, oracle.f32_to_bf16(full))
        results[rank] = (value, token, float(full.max()), oracle.argmax(full),
                         np.array_equal(local, full[begin:end]) and gathered, slowest)
    finally:
        dist.destroy_process_group()


def test_vocab_sharded_argmax_two_ranks():
    world = 2
    with mp.Manager() as manager:
        results = manager.dict()
        mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        assert len(results) == world
        for rank in range(world):
            value, token, want_value, want_token, shard_equal, slowest = results[rank]
            assert shard_equal, "a shard of the packed table must give the same logits as the whole table"
            assert token == want_token == 9 and value == want_value
            assert slowest == 2.0


def test_vocab_shard_boundaries():
    for world in (1, 2, 4, 8):
        bounds = [parallel.vocab_shard(248320, world, r) for r in range(world)]
        assert bounds[0][0] == 0 and bounds[-1][1] == 248320
        assert all(b % 8 == 0 and e % 8 == 0 for b, e in bounds)
        assert all(bounds[i][1] == bounds[i + 1][0] for i in range(world - 1))
    with pytest.raises(ValueError):
        parallel.vocab_shard(248320, 3, 0)
    assert parallel.reduce_argmax(1.5, 7) == (1.5, 7)  # no process group: identity
    one = torch.arange(4.0)
    assert parallel.gather_rows(one) is one
