"""Whole-model oracle self-consistency on the CPU (tiny dimensions)."""
import numpy as np

import llmcp_b200 as L
import oracle

from test_gpu_model import TINY, oracle_dims


def make(seed=5, **changes):
    d = L.default_dims().copy(**{**TINY, **changes})
    data = L.synthetic_container(d, seed)
    arena = L.Arena().from_buffer(data)
    return d, data, oracle.Model(data, arena.manifest, oracle_dims(d))


def test_prefill_equals_token_by_token_decode():
    """Every operator computes a row the same way in prefill and decode mode, so one call over S
    tokens and S single-token calls must agree bit for bit, state included."""
    d, data, model = make()
    prompt = [7, 200, 31, 31, 0, 255, 9]
    whole = model.new_state(16)
    logits = model.forward(whole, prompt, 0)
    stepped = model.new_state(16)
    for i, token in enumerate(prompt):
        last = model.forward(stepped, [token], i)
    assert np.isfinite(logits).all() and logits.std() > 0
    assert np.array_equal(logits.view(np.uint32), last.view(np.uint32))
    for key in ("kv", "delta", "conv"):
        assert np.array_equal(whole[key].view(np.uint8), stepped[key].view(np.uint8)), key
    chunked = model.new_state(16)
    model.forward(chunked, prompt[:4], 0)
    again = model.forward(chunked, prompt[4:], 4)
    assert np.array_equal(again.view(np.uint32), logits.view(np.uint32))


def test_accumulate_modes_differ_only_slightly():
    d, data, model = make()
    arena = L.Arena().from_buffer(data)
    other = oracle.Model(data, arena.manifest, oracle_dims(d), mode="muladd")
    a = model.forward(model.new_state(8), [1, 2, 3], 0)
    b = other.forward(other.new_state(8), [1, 2, 3], 0)
    assert np.abs(a - b).max() < 1e-2


def test_state_is_used():
    d, data, model = make()
    state = model.new_state(8)
    first = model.forward(state, [5], 0)
    second = model.forward(state, [5], 1)
    assert not np.array_equal(first, second)
    assert state["delta"].any() and state["conv"].any() and state["kv"][:, :, :, :2].any()
    assert not state["kv"][:, :, :, 2:].any()
