"""Whole-model parity on a B200 through the drop-in AOT ABI and the engine interface.

The reference has no whole-model pin for random-init weights (its golden tokens need the
real checkpoint), so parity here is against the CPU oracle on the identical packed arena:
logits bit-identical (bar from the task: max_abs <= 1e-2), greedy tokens identical, and the
generation state (KV cache, recurrent state, conv state) bit-identical.
"""
import numpy as np
import pytest

import llmcp_b200 as L
import oracle

pytestmark = pytest.mark.gpu

TINY = dict(hidden=64, intermediate=96, vocab=256, layers=4, full_interval=4, heads=4, kv_heads=2,
            head_dim=32, rotary=8, lin_k_heads=2, lin_v_heads=8, lin_k_dim=16, lin_v_dim=32, conv_kernel=4)
# Model-shaped heads (128-wide recurrent state in registers, 256-wide attention heads), few layers.
SMALL = dict(hidden=256, intermediate=512, vocab=2048, layers=8, full_interval=4, heads=4, kv_heads=2,
             head_dim=256, rotary=64, lin_k_heads=2, lin_v_heads=8, lin_k_dim=128, lin_v_dim=128, conv_kernel=4)


def oracle_dims(d):
    return dict(full_interval=d.full_interval, heads=d.heads, kv_heads=d.kv_heads, head_dim=d.head_dim,
                rotary=d.rotary, lin_k_heads=d.lin_k_heads, lin_v_heads=d.lin_v_heads, lin_k_dim=d.lin_k_dim,
                lin_v_dim=d.lin_v_dim, conv_kernel=d.conv_kernel)


def run_both(dims, seed, prompt, steps, capacity, data=None):
    L.lib().llmcp_b200_clear_error()  # a message left by an earlier, deliberately failing call
    if data is None:
        data = L.synthetic_container(dims, seed)
    arena = L.Arena().from_buffer(data)
    runtime = L.AotRuntime(dims)
    assert runtime.init(max_sequence=capacity)
    model = oracle.Model(data, arena.manifest, oracle_dims(dims))
    state = model.new_state(capacity)

    def cos_sin(pos, n):
        rows = [L.make_cos_sin(pos + t, dims.rotary, dims.rope_theta) for t in range(n)]
        return np.stack([r[0] for r in rows]), np.stack([r[1] for r in rows])

    got_tokens, want_tokens, worst = [], [], 0.0
    tokens, pos = list(prompt), 0
    for step in range(steps + 1):
        logits = runtime.forward(arena, tokens, pos, pos + len(tokens))
        assert logits is not None and not L.last_error()
        cos, sin = cos_sin(pos, len(tokens))
        want = model.forward(state, tokens if step == 0 else [want_tokens[-1]], pos, cos=cos, sin=sin)
        worst = max(worst, float(np.abs(logits - want).max()))
        assert np.isfinite(logits).all()
        assert np.array_equal(logits.view(np.uint32), want.view(np.uint32)), (step, worst)
        got_tokens.append(int(np.argmax(logits)))
        want_tokens.append(oracle.argmax(want))
        pos += len(tokens)
        tokens = [got_tokens[-1]]
    assert got_tokens == want_tokens
    L.lib().llmcp_b200_release_all()
    return data, arena, model, state, want_tokens


@pytest.mark.parametrize("name,dims", [("tiny", TINY), ("small", SMALL)])
def test_aot_abi_matches_oracle(name, dims):
    d = L.default_dims().copy(**dims)
    prompt = [9419 % d.vocab] * 5 + [3, 1, 4]
    run_both(d, 20261125, prompt, steps=6, capacity=24)


def test_engine_matches_aot_and_oracle_state():
    d = L.default_dims().copy(**SMALL)
    prompt = [17, 5, 900, 2047, 0, 33, 33]
    data, arena, model, state, want_tokens = run_both(d, 7, prompt, steps=4, capacity=16)
    engine = L.Engine(data, d, capacity=16)
    logits, token = engine.forward(prompt, 0)
    assert token == want_tokens[0] == int(np.argmax(logits))
    # the same steps, but never leaving the device
    generated, ms = engine.generate(token, len(prompt), 4)
    assert generated.tolist() == want_tokens[1:5] and ms > 0
    dev = engine.read_state()
    assert np.array_equal(dev["delta"].view(np.uint32), state["delta"].view(np.uint32))
    assert np.array_equal(dev["conv"], state["conv"])
    used = len(prompt) + 4
    assert np.array_equal(dev["kv"][:, :, :, :used], state["kv"][:, :, :, :used])
    # a prompt split into two prefill chunks gives the same result as one (state carried on device)
    engine.reset()
    engine.forward(prompt[:3], 0, want_logits=False)
    logits2, token2 = engine.forward(prompt[3:], 3)
    assert token2 == token and np.array_equal(logits2.view(np.uint32), logits.view(np.uint32))
    engine.close()


@pytest.mark.parametrize("heads", [(2, 8), (4, 8), (8, 8)])
def test_one_launch_recurrent_layer_matches_oracle(monkeypatch, heads):
    """LLMCP_B200_FUSE_MIXER=2: convolution, q/k norms, recurrence step, gated norm and quantisation
    of a one-token gated-delta-net layer in one launch (a thread-block cluster per key head: 4, 2
    and 1 value heads per key head).  Same tokens and state as the oracle."""
    nk, nv = heads
    d = L.default_dims().copy(**dict(SMALL, lin_k_heads=nk, lin_v_heads=nv))
    prompt = [17, 5, 900, 2047, 0, 33, 33]
    data = L.synthetic_container(d, 5)
    arena = L.Arena().from_buffer(data)
    model = oracle.Model(data, arena.manifest, oracle_dims(d))
    state = model.new_state(16)

    def cos_sin(pos, n):
        rows = [L.make_cos_sin(pos + t, d.rotary, d.rope_theta) for t in range(n)]
        return dict(cos=np.stack([r[0] for r in rows]), sin=np.stack([r[1] for r in rows]))

    want = [oracle.argmax(model.forward(state, prompt, 0, **cos_sin(0, len(prompt))))]
    for step in range(5):
        want.append(oracle.argmax(model.forward(state, [want[-1]], len(prompt) + step, **cos_sin(len(prompt) + step, 1))))
    monkeypatch.setenv("LLMCP_B200_FUSE_MIXER", "2")
    engine = L.Engine(data, d, capacity=16)
    _, token = engine.forward(prompt, 0)
    generated, _ = engine.generate(token, len(prompt), 5)
    assert [token] + generated.tolist() == want
    dev = engine.read_state()
    assert np.array_equal(dev["delta"].view(np.uint32), state["delta"].view(np.uint32))
    assert np.array_equal(dev["conv"], state["conv"])
    engine.close()


def test_packed_checkpoint_matches_oracle(tmp_path):
    """A checkpoint packed by this repository's llmcp-pack, with random norm gains, A_log and
    dt_bias (the synthetic model has them at their neutral values), through the AOT entries."""
    import test_checkpoint as ck
    ck.write_checkpoint(tmp_path, seed=11)
    L.pack_checkpoint(tmp_path, tmp_path / "weights.bin", quant="q8_0")
    data = np.fromfile(tmp_path / "weights.bin", dtype=np.uint8)
    d = L.parse_config((tmp_path / "config.json").read_text())
    assert all(getattr(d, k) == v for k, v in ck.TINY.items())
    run_both(d, 0, [5, 200, 31, 7, 7, 9], steps=5, capacity=16, data=data)


def test_all_position_logits_match_oracle():
    """llmcp_b200_engine_forward_all: row s equals the oracle's logits for the prefix of s + 1
    tokens, bit for bit (the S x vocab contraction runs on the tensor cores, the oracle's last
    row is a GEMV); a one-token call continues the sequence through the GEMV path."""
    d = L.default_dims().copy(**SMALL)
    data = L.synthetic_container(d, 5)
    arena = L.Arena().from_buffer(data)
    model = oracle.Model(data, arena.manifest, oracle_dims(d))
    prompt = [17, 5, 900, 2047, 0, 33, 33, 1200, 64]
    engine = L.Engine(data, d, capacity=16)
    rows = engine.forward_all(prompt, 0)
    assert rows.shape == (len(prompt), d.vocab) and np.isfinite(rows).all()
    for s in range(len(prompt)):
        want = model.forward(model.new_state(16), prompt[:s + 1], 0)
        assert np.array_equal(rows[s].view(np.uint32), want.view(np.uint32)), s
    state = model.new_state(16)
    model.forward(state, prompt, 0)
    want = model.forward(state, [77], len(prompt))
    step = engine.forward_all([77], len(prompt))
    assert np.array_equal(step[0].view(np.uint32), want.view(np.uint32))
    engine.close()


def test_one_token_prompt_uses_decode_entry():
    d = L.default_dims().copy(**TINY)
    run_both(d, 3, [7], steps=3, capacity=8)  # AotRuntime.cpp:116: sequence == 1 -> decode entry


def test_capacity_is_enforced():
    d = L.default_dims().copy(**TINY)
    data = L.synthetic_container(d, 1)
    engine = L.Engine(data, d, capacity=4)
    with pytest.raises(L.LlmcpError):
        engine.forward([1, 2, 3, 4, 5], 0)
    runtime = L.AotRuntime(d)
    runtime.init(max_sequence=4)
    assert runtime.forward(L.Arena().from_buffer(data), [1, 2, 3], 2, 5) is None  # AotRuntime.cpp:72-74
    engine.close()


@pytest.mark.slow
def test_full_size_model_short_run():
    """Qwen3.5-4B dimensions, random-init: 16-token prefill and 4 greedy steps against the oracle."""
    d = L.default_dims()
    prompt = [9419] * 16
    run_both(d, 20261125, prompt, steps=4, capacity=32)


def test_bad_token_ids_are_refused_before_any_launch():
    """A token id outside [0, vocab) (a -1 pad, an id of another vocabulary) is an error, not an
    out-of-bounds read of the embedding table: nothing is copied or launched."""
    d = L.default_dims().copy(**TINY)
    data = L.synthetic_container(d, 1)
    engine = L.Engine(data, d, capacity=8)
    for bad in ([-1], [3, d.vocab], [2 ** 40]):
        before = L.launch_count()
        with pytest.raises(L.LlmcpError, match="outside the vocabulary"):
            engine.forward(bad, 0)
        with pytest.raises(L.LlmcpError, match="outside the vocabulary"):
            engine.forward_all(bad, 0)
        assert L.launch_count() == before
    with pytest.raises(L.LlmcpError, match="outside the vocabulary"):
        engine.generate(-5, 0, 2)
    logits, token = engine.forward([1, 2, 3], 0)  # the engine is still usable
    assert np.isfinite(logits).all() and 0 <= token < d.vocab
    engine.close()
    # the AOT entry reports through NaN logits and the error message (the ABI returns void)
    runtime = L.AotRuntime(d)
    assert runtime.init(max_sequence=8)
    L.lib().llmcp_b200_clear_error()
    row = runtime.forward(L.Arena().from_buffer(data), [d.vocab + 7], 0, 1)
    assert np.isnan(row).all() and "outside the vocabulary" in L.last_error()
    L.lib().llmcp_b200_clear_error()
    L.lib().llmcp_b200_release_all()


def test_engines_on_two_devices_in_one_process():
    """Kernel attributes (the dynamic shared-memory opt-in) are per device: a second engine on
    another GPU of the same process must run its prefill (tensor-core GEMM, attention) too."""
    if L.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    d = L.default_dims().copy(**SMALL)
    data = L.synthetic_container(d, 9)
    prompt = [5, 6, 7, 8, 9, 10, 11, 12]
    results = []
    for device in (0, 1):
        engine = L.Engine(data, d, capacity=16, device=device)
        logits, token = engine.forward(prompt, 0)
        generated, _ = engine.generate(token, len(prompt), 3)
        results.append((logits, token, generated.tolist()))
        engine.close()
    L.set_device(0)
    assert np.array_equal(results[0][0].view(np.uint32), results[1][0].view(np.uint32))
    assert results[0][1:] == results[1][1:]


@pytest.mark.slow
def test_llmcp_benchmark_binary_against_oracle(tmp_path):
    """The C++ driver (same options and output lines as the reference's llmcp-benchmark) on the
    full-size synthetic container through libllmcp_b200.so: seven `key: value` lines, and with
    --verbose the generated ids, which must be the oracle's greedy tokens."""
    import pathlib
    import subprocess
    tool = L._PACKAGE / "bin" / "llmcp-benchmark"
    assert tool.exists(), "run python -m llmcp_b200.build"
    weights = pathlib.Path("/dev/shm") / "llmcp_b200_synth_20261125.bin"
    run = subprocess.run([str(tool), "--weights", str(weights), "--aot", str(L.LIBRARY_PATH), "--prefill-tokens", "32",
                          "--decode-tokens", "6", "--token", "9419", "--verbose", "--synthetic", "20261125"],
                         capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, run.stderr
    lines = dict(line.split(": ", 1) if ": " in line else (line.split(":")[0], line.split(":", 1)[1])
                 for line in run.stdout.strip().splitlines())
    for key in ("prefill_tokens", "decode_tokens", "prefill_seconds", "decode_seconds", "total_seconds",
                "prefill_tokens_per_second", "decode_tokens_per_second"):
        assert key in lines, run.stdout
    assert int(lines["prefill_tokens"]) == 32 and int(lines["decode_tokens"]) == 6
    assert float(lines["decode_tokens_per_second"]) > 0
    generated = [int(v) for v in lines["generated_tokens"].split()]
    d = L.default_dims()
    data = np.fromfile(weights, dtype=np.uint8)
    arena = L.Arena().from_buffer(data)
    model = oracle.Model(data, arena.manifest, oracle_dims(d))
    state = model.new_state(48)
    logits = model.forward(state, [9419] * 32, 0)
    want, pos = [], 32
    for _ in range(len(generated)):
        want.append(oracle.argmax(logits))
        logits = model.forward(state, [want[-1]], pos)
        pos += 1
    assert generated == want
    model.close()


@pytest.mark.slow
def test_llmcp_run_binary_against_oracle(tmp_path):
    """The C++ generation driver (the AOT half of the reference's llmcp-run) on the full-size synthetic
    container through libllmcp_b200.so: `output: <streamed text>`, then `tokens: ...`, which must be the
    oracle's greedy tokens; generation stops in front of the end-of-turn token; without new tokens the
    `aot logits: N next T` line."""
    import json
    import pathlib
    import subprocess
    tool = L._PACKAGE / "bin" / "llmcp-run"
    assert tool.exists(), "run python -m llmcp_b200.build"
    d = L.default_dims()
    # a ByteLevel vocabulary of the model's size: the 256 bytes, then "<n>" for every other id
    alphabet, nxt = [], 256
    for byte in range(256):
        direct = 33 <= byte <= 126 or 161 <= byte <= 172 or byte >= 174
        alphabet.append(chr(byte if direct else nxt))
        nxt += 0 if direct else 1
    vocab = {alphabet[b]: b for b in range(256)}
    vocab.update({f"<{i}>": i for i in range(256, d.vocab)})
    blob = json.dumps({"model": {"type": "BPE", "vocab": vocab, "merges": []}, "added_tokens": [], "decoder": {"type": "ByteLevel"}})
    (tmp_path / "tokenizer.json").write_text(blob)
    weights = pathlib.Path("/dev/shm") / "llmcp_b200_synth_20261125.bin"
    prompt = [9419] * 8
    base = [str(tool), "--weights", str(weights), "--aot", str(L.LIBRARY_PATH), "--synthetic", "20261125",
            "--token-ids", ",".join(map(str, prompt)), "--tokenizer", str(tmp_path / "tokenizer.json")]
    run = subprocess.run(base + ["--max-new-tokens", "6"], capture_output=True, text=True, timeout=900)
    assert run.returncode == 0, run.stderr
    out_line, tokens_line = run.stdout.strip().split("\n")
    generated = [int(v) for v in tokens_line.removeprefix("tokens:").split()]
    data = np.fromfile(weights, dtype=np.uint8)
    arena = L.Arena().from_buffer(data)
    model = oracle.Model(data, arena.manifest, oracle_dims(d))
    state = model.new_state(40)
    logits = model.forward(state, prompt, 0)
    want = []
    for step in range(6):
        want.append(oracle.argmax(logits))
        logits = model.forward(state, [want[-1]], len(prompt) + step)
    model.close()
    assert generated == want
    v = L.Vocab(blob)
    assert out_line == "output: " + v.decode(generated)
    v.close()
    # the third token as end-of-turn token: two tokens come out
    if want[2] not in want[:2]:
        run = subprocess.run(base + ["--max-new-tokens", "6", "--eos-token", str(want[2])], capture_output=True, text=True, timeout=900)
        assert run.returncode == 0, run.stderr
        assert [int(x) for x in run.stdout.strip().split("\n")[-1].removeprefix("tokens:").split()] == want[:2]
    run = subprocess.run(base, capture_output=True, text=True, timeout=900)
    assert run.returncode == 0 and run.stdout.strip() == f"aot logits: {d.vocab} next {want[0]}", run.stdout


def test_llmcp_run_text_prompt(tmp_path):
    """`llmcp-run --text ... --chat`: the driver encodes the chat-wrapped prompt itself and generates
    the same tokens as a run that is handed the ids (ids from the package-checked encoder)."""
    import json
    import pathlib
    import subprocess
    tool = L._PACKAGE / "bin" / "llmcp-run"
    golden = json.loads((pathlib.Path(__file__).parent / "golden" / "bpe_encoder.json").read_text())
    (tmp_path / "tokenizer.json").write_text(golden["tokenizer"])
    v = L.Vocab(golden["tokenizer"])
    ids = v.encode(L.chat_prompt("Hello world, it's 12 o'clock", thinking=False))
    assert len(ids) > 8 and ids[0] == v.token_to_id("<|im_start|>")
    weights = pathlib.Path("/dev/shm") / "llmcp_b200_synth_20261125.bin"
    base = [str(tool), "--weights", str(weights), "--aot", str(L.LIBRARY_PATH), "--synthetic", "20261125",
            "--tokenizer", str(tmp_path / "tokenizer.json"), "--max-new-tokens", "4", "--eos-token", "-1"]
    by_text = subprocess.run(base + ["--text", "Hello world, it's 12 o'clock", "--chat", "--no-thinking"], capture_output=True, text=True, timeout=900)
    by_ids = subprocess.run(base + ["--token-ids", ",".join(map(str, ids))], capture_output=True, text=True, timeout=900)
    assert by_text.returncode == 0 and by_ids.returncode == 0, by_text.stderr + by_ids.stderr
    assert by_text.stdout == by_ids.stdout and by_text.stdout.strip().split("\n")[-1].startswith("tokens:")
    assert len(by_text.stdout.strip().split("\n")[-1].split()) == 5
    v.close()


def test_aot_sessions_are_bounded(monkeypatch):
    """A caller that reallocates its state buffers (as the reference's AotRuntime::init does) gets a new
    engine each time; beyond LLMCP_B200_MAX_SESSIONS the least recently used one is released, and a
    released session's caller simply gets a fresh engine on its next call (state starts at position 0)."""
    monkeypatch.setenv("LLMCP_B200_MAX_SESSIONS", "2")
    lib = L.lib()
    lib.llmcp_b200_release_all()
    d = L.default_dims().copy(**TINY)
    data = L.synthetic_container(d, 9)
    arena = L.Arena().from_buffer(data)
    prompt = [1, 2, 3, 4]
    runtimes, first = [], None
    for _ in range(3):
        runtime = L.AotRuntime(d)
        assert runtime.init(max_sequence=16)
        logits = runtime.forward(arena, prompt, 0, len(prompt))
        assert logits is not None and not L.last_error()
        first = logits if first is None else first
        assert np.array_equal(logits.view(np.uint32), first.view(np.uint32))
        runtimes.append(runtime)
        assert lib.llmcp_b200_session_count() <= 2
    assert lib.llmcp_b200_session_count() == 2
    # the first runtime's session was released: a call at position 0 builds it again
    again = runtimes[0].forward(arena, prompt, 0, len(prompt))
    assert np.array_equal(again.view(np.uint32), first.view(np.uint32)) and lib.llmcp_b200_session_count() == 2
    lib.llmcp_b200_release_all()
    assert lib.llmcp_b200_session_count() == 0
