"""A batch of independent sequences on a B200: prefilled one by one, decoded together.  Each
sequence is checked against its own one-sequence run of the CPU oracle: logits bit for bit in
exact mode (the batched step changes which kernel does the contraction, not the arithmetic of any
output element), greedy tokens, and the per-sequence state.  Two prompt sets, as the batched
benchmark configuration needs: identical prompts (every row the same: hides nothing but also
proves nothing about state separation) and a different random prompt per sequence."""
import numpy as np
import pytest

import llmcp_b200 as L
import oracle

pytestmark = pytest.mark.gpu

TINY = dict(hidden=64, intermediate=96, vocab=256, layers=4, full_interval=4, heads=4, kv_heads=2,
            head_dim=32, rotary=8, lin_k_heads=2, lin_v_heads=8, lin_k_dim=16, lin_v_dim=32, conv_kernel=4)
SMALL = dict(hidden=256, intermediate=512, vocab=2048, layers=8, full_interval=4, heads=4, kv_heads=2,
             head_dim=256, rotary=64, lin_k_heads=2, lin_v_heads=8, lin_k_dim=128, lin_v_dim=128, conv_kernel=4)


def oracle_dims(d):
    return dict(full_interval=d.full_interval, heads=d.heads, kv_heads=d.kv_heads, head_dim=d.head_dim,
                rotary=d.rotary, lin_k_heads=d.lin_k_heads, lin_v_heads=d.lin_v_heads, lin_k_dim=d.lin_k_dim,
                lin_v_dim=d.lin_v_dim, conv_kernel=d.conv_kernel)


def run_batch(dims, batch, prompt_len, steps, mode, same_prompts, seed=5, full_size=False):
    d = L.default_dims() if full_size else L.default_dims().copy(**dims)
    data = L.synthetic_container(d, 20261125)
    rng = np.random.default_rng(seed)
    if same_prompts:
        prompts = [[9419 % d.vocab] * prompt_len] * batch
    else:
        prompts = [rng.integers(0, d.vocab, prompt_len).tolist() for _ in range(batch)]
    capacity = prompt_len + steps + 6
    engine = L.Engine(data, d, capacity=capacity, mode=mode, batch=batch)
    model = oracle.Model(data, L.Arena().from_buffer(data).manifest, oracle_dims(d))
    states = [model.new_state(capacity) for _ in range(batch)]
    firsts, want_first, worst = [], [], 0.0
    for b in range(batch):
        engine.select_sequence(b)
        logits, token = engine.forward(prompts[b], 0)
        want = model.forward(states[b], prompts[b], 0)
        worst = max(worst, float(np.abs(logits - want).max()))
        firsts.append(token)
        want_first.append(oracle.argmax(want))
    tokens, want_tokens = list(want_first), list(want_first)
    pos = prompt_len
    for _ in range(steps):  # step by step, logits of every sequence against its own oracle run (teacher forced)
        logits, argmax = engine.decode_batch(want_tokens, pos)
        nxt = []
        for b in range(batch):
            want = model.forward(states[b], [want_tokens[b]], pos)
            worst = max(worst, float(np.abs(logits[b] - want).max()))
            nxt.append(oracle.argmax(want))
            if mode == "exact":
                assert np.array_equal(logits[b].view(np.uint32), want.view(np.uint32)), (b, pos)
                assert int(argmax[b]) == nxt[b]
        want_tokens = nxt
        pos += 1
    # the device-resident batched loop against the oracle's chains
    generated, ms = engine.generate_batch(want_tokens, pos, 3)
    chains = []
    for b in range(batch):
        chain, token = [], want_tokens[b]
        for i in range(3):
            token = oracle.argmax(model.forward(states[b], [token], pos + i))
            chain.append(token)
        chains.append(chain)
    state_ok = True
    if mode == "exact":
        for b in (0, batch - 1):
            engine.select_sequence(b)
            got = engine.read_state()
            used = pos + 3
            state_ok &= bool(np.array_equal(got["delta"].view(np.uint32), states[b]["delta"].view(np.uint32)))
            state_ok &= bool(np.array_equal(got["conv"], states[b]["conv"]))
            state_ok &= bool(np.array_equal(got["kv"][:, :, :, :used], states[b]["kv"][:, :, :, :used]))
    engine.close()
    model.close()
    return dict(firsts=firsts, want_first=want_first, worst=worst, generated=generated.T.tolist(), chains=chains,
                state_ok=state_ok, ms=ms)


@pytest.mark.parametrize("name,dims,batch", [("tiny", TINY, 3), ("small", SMALL, 5), ("small", SMALL, 64)])
@pytest.mark.parametrize("same_prompts", [True, False])
def test_batch_matches_each_sequences_own_oracle_run(name, dims, batch, same_prompts):
    r = run_batch(dims, batch, prompt_len=6, steps=3 if batch > 8 else 5, mode="exact", same_prompts=same_prompts)
    assert r["firsts"] == r["want_first"]
    assert r["worst"] == 0.0
    assert r["generated"] == r["chains"]
    assert r["state_ok"]
    if not same_prompts:
        assert len({tuple(c) for c in r["chains"]}) > 1  # the sequences really differ


def test_batch_fast_mode_stays_close():
    r = run_batch(SMALL, 6, prompt_len=6, steps=4, mode="fast", same_prompts=False)
    assert r["firsts"] == r["want_first"] or r["worst"] > 0
    assert r["worst"] <= 0.2, r["worst"]  # rounding-order differences only


def test_batch_engine_rejects_misuse():
    d = L.default_dims().copy(**TINY)
    data = L.synthetic_container(d, 1)
    single = L.Engine(data, d, capacity=8)
    with pytest.raises(L.LlmcpError):
        L.lib().llmcp_b200_clear_error()
        L._check(L.lib().llmcp_b200_engine_select_sequence(single.handle, 1))
    single.close()
    engine = L.Engine(data, d, capacity=8, batch=2)
    with pytest.raises(L.LlmcpError, match="outside the vocabulary"):
        engine.decode_batch([1, d.vocab], 0)
    with pytest.raises(L.LlmcpError):
        engine.decode_batch([1, 2], 8)  # past the cache
    engine.close()


@pytest.mark.slow
def test_batch_64_full_size_model():
    """Qwen3.5-4B dimensions, 64 sequences with different 4-token prompts, two batched steps."""
    r = run_batch(None, 64, prompt_len=4, steps=2, mode="exact", same_prompts=False, full_size=True)
    assert r["firsts"] == r["want_first"] and r["worst"] == 0.0 and r["generated"] == r["chains"] and r["state_ok"]
