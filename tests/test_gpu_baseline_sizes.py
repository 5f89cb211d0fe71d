"""Parity at the sizes the benchmark configurations name (exact mode, through the C ABI).

The operator tests elsewhere cover the shapes' edges on small cases; these run each hot-path
operator once at full size against the CPU oracle, with the bit-exact bar: int32 block dots,
f32 / bf16 outputs, cache and state bytes.  Inputs are seeded synthetic tensors with the shapes
and distributions of the configurations (seed 20261125 + configuration index).  They take tens of
seconds of oracle time each and are marked slow; `-m gpu` still selects them.
"""
import numpy as np
import pytest

import llmcp_b200 as L
import oracle

pytestmark = [pytest.mark.gpu, pytest.mark.slow]
f = oracle.bf16_to_f32
SEED = 20261125


def bf16(a):
    return oracle.f32_to_bf16(np.asarray(a, dtype=np.float32))


def normal(rng, *shape, scale=1.0):
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)).astype(np.float32)


def test_config1_linear_1024x9216x2560_with_block_dots():
    """Prefill GEMM on the tensor cores at the gate/up projection's shape: every int32 block dot
    [1024, 9216, 80] and every f32 output bit for bit; then the same weights at M = 1."""
    rng = np.random.default_rng(SEED + 1)
    M, N, K = 1024, 9216, 2560
    packed = oracle.pack_q8_0_p4(normal(rng, N, K, scale=0.02))
    x = normal(rng, M, K)
    y, dots = L.ops.linear_q8(x, packed, N, x_bf16=False, y_bf16=False, want_dots=True)
    q, _ = oracle.act_quant(x, False)
    want_dots = oracle.block_dots(q, packed, N)
    assert dots.shape == want_dots.shape == (M, N, K // 32)
    assert np.array_equal(dots, want_dots)
    del dots, want_dots
    want = oracle.linear_q8(x, packed, N, x_bf16=False, y_bf16=False)
    assert np.array_equal(y.view(np.uint32), want.view(np.uint32)), np.abs(y - want).max()
    y1, dots1 = L.ops.linear_q8(x[:1], packed, N, x_bf16=False, y_bf16=False, want_dots=True)
    assert np.array_equal(y1.view(np.uint32), want[:1].view(np.uint32))
    assert np.array_equal(dots1, oracle.block_dots(q[:1], packed, N))


def test_config2_lm_head_all_248320_rows():
    """The tied vocabulary projection at full size: logits bit for bit, argmax = first maximum."""
    rng = np.random.default_rng(SEED + 2)
    vocab, K = 248320, 2560
    table = normal(rng, vocab, K, scale=0.02)
    table[200000] = table[31]  # equal logits far apart: the lower index must win if they are the maximum
    packed = oracle.pack_q8_0_p4(table)
    del table
    h = oracle.rms_norm(bf16(normal(rng, 1, K)), np.zeros(K, np.uint16))
    logits, argmax = L.ops.lm_head_q8(h, packed, vocab)
    want = oracle.linear_q8(h, packed, vocab, y_bf16=False)
    assert np.array_equal(logits.view(np.uint32), want.view(np.uint32))
    assert logits[0, 31] == logits[0, 200000]
    assert int(argmax[0]) == oracle.argmax(want[0])
    print(f"lm_head top-2 margin {oracle.top2_margin(want[0]):.4e}")


@pytest.mark.parametrize("nk,nv", [(16, 16), (16, 32)])
def test_config3_gated_delta_net_1024_then_128_steps(nk, nv):
    """T = 1024 prefill, then 128 single-token calls carrying the state; outputs and the final
    f32 state bit for bit."""
    rng = np.random.default_rng(SEED + 3 + nv)
    dk = dv = 128
    T, steps = 1024, 128
    channels = 2 * nk * dk + nv * dv
    conv = bf16(normal(rng, T + steps, channels))
    a = bf16(normal(rng, T + steps, nv))
    b = bf16(normal(rng, T + steps, nv))
    a_log = np.zeros(nv, np.float32)
    dt = np.zeros(nv, np.uint16)
    zero = np.zeros((nv, dk, dv), np.float32)
    out, state = L.ops.gated_delta_net(conv[:T], a[:T], b[:T], a_log, dt, zero, nk, nv, dk, dv)
    want, want_state = oracle.gated_delta_net(conv[:T], a[:T], b[:T], a_log, dt, zero, nk, nv, dk, dv)
    assert np.array_equal(out, want)
    assert np.array_equal(state.view(np.uint32), want_state.view(np.uint32))
    for t in range(T, T + steps):
        out, state = L.ops.gated_delta_net(conv[t:t + 1], a[t:t + 1], b[t:t + 1], a_log, dt, state, nk, nv, dk, dv)
        want, want_state = oracle.gated_delta_net(conv[t:t + 1], a[t:t + 1], b[t:t + 1], a_log, dt, want_state, nk, nv, dk, dv)
        assert np.array_equal(out, want), t
    assert np.array_equal(state.view(np.uint32), want_state.view(np.uint32))
    assert np.isfinite(state).all()


def test_config4_attention_prefill_1024_and_decode_at_1024_and_8192():
    rng = np.random.default_rng(SEED + 4)
    nh, nkv, hd, rot = 16, 4, 256, 64
    norm = np.zeros(hd, np.uint16)  # stored 0 = unit gain (zero-centred)

    def rows(pos, S):
        cs = [L.make_cos_sin(pos + t, rot, 1e7) for t in range(S)]
        return np.stack([c[0] for c in cs]), np.stack([c[1] for c in cs])

    # prefill of 1024 tokens at position 0, then one token at position 1024 on the cache it left
    T, cap = 1024, 1025
    qg, k, v = bf16(normal(rng, T, nh * 2 * hd)), bf16(normal(rng, T, nkv * hd)), bf16(normal(rng, T, nkv * hd))
    cos, sin = rows(0, T)
    cache = np.zeros((2, nkv, cap, hd), np.uint16)
    out, cache_gpu = L.ops.attention(qg, k, v, norm, norm, cos, sin, cache, 0, nh, nkv, hd, rot)
    want, cache_cpu = oracle.attention(qg, k, v, norm, norm, cos, sin, cache, 0, nh, nkv, hd, rot)
    assert np.array_equal(cache_gpu, cache_cpu)
    assert np.array_equal(out, want), np.abs(f(out) - f(want)).max()
    qg1, k1, v1 = bf16(normal(rng, 1, nh * 2 * hd)), bf16(normal(rng, 1, nkv * hd)), bf16(normal(rng, 1, nkv * hd))
    cos, sin = rows(T, 1)
    out, cache_gpu = L.ops.attention(qg1, k1, v1, norm, norm, cos, sin, cache_gpu, T, nh, nkv, hd, rot)
    want, cache_cpu = oracle.attention(qg1, k1, v1, norm, norm, cos, sin, cache_cpu, T, nh, nkv, hd, rot)
    assert np.array_equal(cache_gpu, cache_cpu) and np.array_equal(out, want)
    # one token against 8192 cached keys (32 MiB of KV per layer)
    pos, cap = 8192, 8193
    cache = bf16(normal(rng, 2, nkv, cap, hd))
    cos, sin = rows(pos, 1)
    out, cache_gpu = L.ops.attention(qg1, k1, v1, norm, norm, cos, sin, cache, pos, nh, nkv, hd, rot)
    want, cache_cpu = oracle.attention(qg1, k1, v1, norm, norm, cos, sin, cache, pos, nh, nkv, hd, rot)
    assert np.array_equal(cache_gpu, cache_cpu) and np.array_equal(out, want)


def test_config5_whole_model_1024_prefill_128_greedy_steps():
    """Qwen3.5-4B dimensions, random-init: 1024 x token 9419 through the prefill entry, then 128
    greedy steps through the decode entry, against the oracle on the same arena: logits bit for
    bit at every step, tokens equal; the oracle's top-1/top-2 margins are printed (they say how
    much logit error a token comparison on these weights could absorb)."""
    d = L.default_dims()
    data = L.synthetic_container(d, SEED)
    arena = L.Arena().from_buffer(data)
    runtime = L.AotRuntime(d)
    capacity = 1024 + 128 + 1
    assert runtime.init(max_sequence=capacity)
    model = oracle.Model(data, arena.manifest, dict(
        full_interval=d.full_interval, heads=d.heads, kv_heads=d.kv_heads, head_dim=d.head_dim, rotary=d.rotary,
        lin_k_heads=d.lin_k_heads, lin_v_heads=d.lin_v_heads, lin_k_dim=d.lin_k_dim, lin_v_dim=d.lin_v_dim,
        conv_kernel=d.conv_kernel))
    state = model.new_state(capacity)
    tokens, pos, margins = [9419] * 1024, 0, []
    for step in range(129):
        logits = runtime.forward(arena, tokens, pos, pos + len(tokens))
        assert logits is not None and not L.last_error()
        want = model.forward(state, tokens, pos)
        assert np.array_equal(logits.view(np.uint32), want.view(np.uint32)), (step, float(np.abs(logits - want).max()))
        margins.append(oracle.top2_margin(want))
        pos += len(tokens)
        tokens = [int(np.argmax(logits))]
        assert tokens[0] == oracle.argmax(want)
    print(f"top-2 margin over 129 positions: min {min(margins):.4e}, median {float(np.median(margins)):.4e}")
    L.lib().llmcp_b200_release_all()
    model.close()
