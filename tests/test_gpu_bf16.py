"""Unquantised (bf16) arenas on a B200: `llmcp-pack --quant none` containers through the engine and
the AOT entries, and the bf16 linear on its own.

The reference lowers the bf16 sum differently per target (MatmulLoweringCommon.cpp:186-251 portable,
253-330 BFDOT) and holds it to a tolerance in its own tests (tests/numeric/run_numeric.py:676-688:
relative 2e-2, absolute 1e-2), so the bar here is a tolerance as well: against a plain f32 matrix
product, and against the oracle's restatement of the portable lowering."""
import numpy as np
import pytest

import llmcp_b200 as L
import oracle

pytestmark = pytest.mark.gpu
f = oracle.bf16_to_f32

SMALL = dict(hidden=256, intermediate=512, vocab=2048, layers=8, full_interval=4, heads=4, kv_heads=2,
             head_dim=256, rotary=64, lin_k_heads=2, lin_v_heads=8, lin_k_dim=128, lin_v_dim=128, conv_kernel=4)


def bf16(a):
    return oracle.f32_to_bf16(np.asarray(a, dtype=np.float32))


@pytest.mark.parametrize("M,N,K", [(1, 2560, 4096), (1, 9216, 2560), (1, 50, 2560), (5, 136, 288), (128, 128, 64), (130, 264, 2560),
                                   (1024, 2560, 9216)])
def test_linear_bf16_against_f32_product(M, N, K):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(M + N + K)
    x, w = bf16(rng.standard_normal((M, K))), bf16(rng.standard_normal((N, K)) * 0.05)
    want = (torch.from_numpy(f(x)).double() @ torch.from_numpy(f(w)).double().T).numpy()  # products exact, sum in f64
    got = L.ops.linear_bf16(x, w, y_bf16=False)
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= 2e-5 * scale, (np.abs(got - want).max(), scale)
    if M * N * K <= 130 * 264 * 2560:  # the oracle's ordered tile sums, where it finishes quickly
        ref = oracle.linear_bf16(x, w, y_bf16=False)
        assert np.abs(got - ref).max() <= 2e-5 * scale
    for activation in ("none", "silu", "sigmoid"):
        got_b = f(L.ops.linear_bf16(x, w, activation=activation))
        act = {"none": lambda v: v, "silu": lambda v: v / (1 + np.exp(-v)), "sigmoid": lambda v: 1 / (1 + np.exp(-v))}[activation]
        np.testing.assert_allclose(got_b, act(want), rtol=2e-2, atol=1e-2)  # the reference's own bar
        assert np.abs(got_b - act(want)).max() <= 2.0 ** -7 * max(1.0, np.abs(act(want)).max())  # one bf16 rounding


def oracle_dims(d):
    return dict(full_interval=d.full_interval, heads=d.heads, kv_heads=d.kv_heads, head_dim=d.head_dim,
                rotary=d.rotary, lin_k_heads=d.lin_k_heads, lin_v_heads=d.lin_v_heads, lin_k_dim=d.lin_k_dim,
                lin_v_dim=d.lin_v_dim, conv_kernel=d.conv_kernel)


@pytest.mark.parametrize("mode", ["exact", "fast"])
def test_bf16_arena_through_engine_and_aot_entries(tmp_path, mode):
    """A checkpoint packed with --quant none: prefill and greedy steps against the oracle's bf16 model.
    The order of the f32 additions inside a linear is not fixed by the reference (its portable and its
    aarch64 lowerings differ), and a sum that lands on the other side of a bf16 rounding moves the
    whole model's logits a little; the bar is the spread between the oracle's restatements of
    those two lowerings on the same positions (factor 2: both are maxima over 2048 x 7 samples)."""
    d = L.default_dims().copy(**SMALL)
    L.synthetic_checkpoint(d, 3, tmp_path)
    L.pack_checkpoint(tmp_path, tmp_path / "weights.bin", quant="none")
    data = np.fromfile(tmp_path / "weights.bin", dtype=np.uint8)
    arena = L.Arena().from_buffer(data)
    assert arena.quantization == "none"
    model = oracle.Model(data, arena.manifest, oracle_dims(d), mode="bf16")
    other = oracle.Model(data, arena.manifest, oracle_dims(d), mode="bf16-pairs")
    state, other_state = model.new_state(24), other.new_state(24)

    def cos_sin(pos, n):
        rows = [L.make_cos_sin(pos + t, d.rotary, d.rope_theta) for t in range(n)]
        return dict(cos=np.stack([r[0] for r in rows]), sin=np.stack([r[1] for r in rows]))

    prompt = [17, 5, 900, 2047, 0, 33, 33, 1, 2]
    engine = L.Engine(data, d, capacity=24, mode=mode)
    logits, token = engine.forward(prompt, 0)
    want = model.forward(state, prompt, 0, **cos_sin(0, len(prompt)))
    worst = float(np.abs(logits - want).max())
    spread = float(np.abs(other.forward(other_state, prompt, 0, **cos_sin(0, len(prompt))) - want).max())
    tokens = [oracle.argmax(want)]
    for step in range(6):
        pos = len(prompt) + step
        logits, _ = engine.forward([tokens[-1]], pos)
        want = model.forward(state, [tokens[-1]], pos, **cos_sin(pos, 1))
        worst = max(worst, float(np.abs(logits - want).max()))
        spread = max(spread, float(np.abs(other.forward(other_state, [tokens[-1]], pos, **cos_sin(pos, 1)) - want).max()))
        margin = oracle.top2_margin(want)
        if margin > 2 * worst:
            assert int(np.argmax(logits)) == oracle.argmax(want), (step, margin, worst)
        tokens.append(oracle.argmax(want))
    assert np.isfinite(logits).all()
    assert worst <= 2.0 * spread + 1e-3, (worst, spread)
    engine.close()
    model.close()
    other.close()
    # the drop-in entry points take the same container
    L.lib().llmcp_b200_clear_error()  # a message left by an earlier, deliberately failing call
    runtime = L.AotRuntime(d)
    assert runtime.init(max_sequence=24)
    got = runtime.forward(arena, prompt, 0, len(prompt))
    assert got is not None and not L.last_error()
    L.lib().llmcp_b200_release_all()
