"""The CPU oracle against the vectors taken from the reference's numeric tests.

Each case mirrors one case of the reference's tests/numeric/run_numeric.py and uses
the tolerance that file uses; the Q8 known-answer cases are additionally required to
be exact, which the construction (power-of-two block scales) allows.
"""
import numpy as np
import pytest

import oracle
from conftest import assert_close

f = oracle.bf16_to_f32


def check_packer(w_bits, python_packed, exact):
    """The restated C++ packer against the reference's Python packer (q8_0_p4_bytes).

    The two round differently on purpose in the reference itself: the C++ packer uses
    lround(x / scale) in f32 (lib/Model/Quantization.cpp:107-111), the Python one
    round(x * (1 / scale)) in double.  They agree on every scale and, where no value sits
    within rounding noise of a half-way point, on every integer; elsewhere they may differ
    by one count.
    """
    mine = oracle.pack_q8_0_p4(w_bits, src_bf16=True)
    assert mine.shape == python_packed.shape
    records = mine.reshape(-1, 136)
    theirs = python_packed.reshape(-1, 136)
    assert np.array_equal(records[:, :8], theirs[:, :8]), "f16 scales differ"
    delta = records[:, 8:].view(np.int8).astype(np.int32) - theirs[:, 8:].view(np.int8)
    assert np.abs(delta).max() <= 1
    if exact:
        assert not delta.any()
    else:
        assert np.count_nonzero(delta) <= 0.01 * delta.size


@pytest.mark.parametrize("case", ["linear_q8_p4_decode", "linear_q8_p4_prefill",
                                  "linear_q8_p4_prefill_boundaries",
                                  "linear_q8_p4_decode_boundaries"])
@pytest.mark.parametrize("mode", ["fma", "muladd"])
def test_linear_q8(golden, case, mode):
    c = golden(case)
    n = c["w"].shape[0]
    check_packer(c["w"], c["packed"], exact=case.endswith("boundaries"))
    y = oracle.linear_q8(c["x"], c["packed"], n, mode=mode)
    assert_close(f(y), c["ref"], c["tol"], case)
    if case.endswith("boundaries"):
        assert np.array_equal(f(y), c["ref"].astype(np.float32))
    direct = oracle.linear_q8(c["x"], c["packed"], n, mode=mode, direct=True)
    assert np.array_equal(direct, y)


@pytest.mark.parametrize("case", ["lm_head_q8_p4", "lm_head_q8_p4_decode"])
def test_lm_head_q8(golden, case):
    c = golden(case)
    y = oracle.linear_q8(c["x"], c["packed"], c["w"].shape[0], y_bf16=False)
    assert_close(y, c["ref"], c["tol"], case)


def test_embedding_q8(golden):
    c = golden("embedding_q8_p4")
    check_packer(c["table"], c["packed"], exact=True)
    y = oracle.embedding_q8(c["tokens"], c["packed"], c["table"].shape[1])
    assert_close(f(y), c["ref"], c["tol"], "embedding")
    assert np.array_equal(f(y), c["ref"])


def test_rms_norm(golden):
    c = golden("rms_zero_centered")
    assert_close(f(oracle.rms_norm(c["x"], c["w"], zero_centered=True)), c["ref"], c["tol"])
    c = golden("rms_plain")
    assert_close(f(oracle.rms_norm(c["x"], c["w"], zero_centered=False)), c["ref"], c["tol"])


def test_pointwise(golden):
    c = golden("add")
    assert np.array_equal(f(oracle.pointwise(c["a"], c["b"], "add")), c["ref"])
    c = golden("silu_mul")
    assert_close(f(oracle.pointwise(c["gate"], c["up"], "silu_mul")), c["ref"], c["tol"])
    c = golden("mul_silu_mul")
    product = oracle.pointwise(c["gate"], c["up"], "mul")
    assert_close(f(oracle.pointwise(c["gate"], product, "silu_mul")), c["ref"], c["tol"])


def test_gated_rms_norm(golden):
    c = golden("gated_rms_norm")
    y = oracle.gated_rms_norm(c["x"], c["gate"], c["w"], int(c["group"]))
    assert_close(f(y), c["ref"], c["tol"])
    c = golden("gated_rms_norm_activated")
    y = oracle.gated_rms_norm(c["x"], c["gate"], c["w"], int(c["group"]), gate_activated=True)
    assert_close(f(y), c["ref"], c["tol"])


@pytest.mark.parametrize("case", ["causal_conv1d", "causal_conv1d_decode"])
def test_causal_conv1d(golden, case):
    c = golden(case)
    y, state = oracle.causal_conv1d(c["x"], c["w"].reshape(c["w"].shape[0], -1), c["state"],
                                    int(c["kernel"]))
    assert_close(f(y), c["ref"], c["tol"], case)
    assert np.array_equal(state, c["ref_state"])


def test_gated_delta_net(golden):
    cases = [n for n in golden.names() if n.startswith("gated_delta_net")]
    assert len(cases) == 7
    for case in cases:
        c = golden(case)
        seq, nk, nv, dk, dv = (int(v) for v in c["dims"])
        out, state = oracle.gated_delta_net(c["conv"], c["a"], c["b"], c["a_log"], c["dt_bias"],
                                            c["state"], nk, nv, dk, dv)
        assert_close(f(out), c["ref"], c["tol"], case)
        assert_close(state, c["ref_state"], c["tol"], case + " state")


@pytest.mark.parametrize("case", ["attention", "attention_decode"])
def test_attention(golden, case):
    c = golden(case)
    seq, nh, nkv, hd, rot, cap, pos = (int(v) for v in c["dims"])
    out, cache = oracle.attention(c["qg"], c["k"], c["v"], c["q_norm"], c["k_norm"], c["cos"],
                                  c["sin"], c["cache"], pos, nh, nkv, hd, rot)
    assert_close(f(out), c["ref"], c["tol"], case)
    assert_close(f(cache), f(c["ref_cache"]), c["tol"], case + " cache")


def test_quantization_byte_pins(golden):
    """tests/unittests/QuantizationTest.cpp:57-89 and llmcp-matmul-benchmark.cpp:271-293,331-335."""
    d, qs = oracle.quantize_row_q8_0(np.ones(64, dtype=np.float32))
    assert d.view(np.uint8).reshape(-1, 2).tolist() == [[0x08, 0x20]] * 2
    assert (qs == 127).all()
    values = np.ones(64, dtype=np.float32)
    values[32:] = 0
    d, qs = oracle.quantize_row_q8_0(values)
    assert d[1] == 0 and (qs[32:] == 0).all()
    # all-127 weights with scale 0x2008 times an all-ones input: every output equals K.
    K, N = 64, 8
    packed = oracle.pack_q8_0_p4(np.ones((N, K), dtype=np.float32))
    y = oracle.linear_q8(np.ones((1, K), dtype=np.float32), packed, N, x_bf16=False, y_bf16=False)
    assert np.allclose(y, K, rtol=2e-3)


def test_packed_shape_rule():
    """Q8PackedLayout.h:38-42: rows % 8 == 0 and cols % 32 == 0."""
    with pytest.raises(ValueError):
        oracle.pack_q8_0_p4(np.zeros((4, 32), dtype=np.float32))
    with pytest.raises(ValueError):
        oracle.pack_q8_0_p4(np.zeros((8, 48), dtype=np.float32))


def test_act_quant_properties():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 96)).astype(np.float32)
    x[1, 32:64] = 0
    q, s = oracle.act_quant(x, x_bf16=False)
    assert (s[1, 1] == 0) and (q[1, 32:64] == 0).all()
    amax = np.abs(x.reshape(3, 3, 32)).max(-1)
    assert np.array_equal(s, (amax / np.float32(127)).astype(np.float32))
    assert np.abs(q).max() <= 127 and (np.abs(q.reshape(3, 3, 32)).max(-1)[amax > 0] == 127).all()


def test_block_dots_match_numpy():
    rng = np.random.default_rng(2)
    w = (rng.standard_normal((16, 64)) * 0.02).astype(np.float32)
    x = rng.standard_normal((2, 64)).astype(np.float32)
    packed = oracle.pack_q8_0_p4(w)
    q, _ = oracle.act_quant(x, x_bf16=False)
    dots = oracle.block_dots(q, packed, 16)
    wq = np.stack([oracle.quantize_row_q8_0(row)[1] for row in w]).astype(np.int32)
    want = np.einsum("mbk,nbk->mnb", q.astype(np.int32).reshape(2, 2, 32), wq.reshape(16, 2, 32))
    assert np.array_equal(dots, want)
