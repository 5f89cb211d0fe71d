"""Operator parity on a B200: every llmcp operator through the C ABI against the CPU oracle
and against the vectors taken from the reference's numeric tests.

Bars: int8 quantisation, int32 block dots, indices and state bytes are bit-exact; f32/bf16
results are required to be bit-identical to the oracle as well (the kernels keep the
reference's operation order, and exp/log are defined as the f32 rounding of the f64
function on both sides), which is stricter than the reference's own tolerances; the golden
cases are checked with the tolerance the reference's harness uses.
"""
import numpy as np
import pytest

import llmcp_b200 as L
import oracle
from conftest import assert_close

pytestmark = pytest.mark.gpu
f = oracle.bf16_to_f32


def bf16(a):
    return oracle.f32_to_bf16(np.asarray(a, dtype=np.float32))


def rand_bf16(rng, *shape, scale=1.0):
    return bf16(rng.standard_normal(shape) * scale)


@pytest.mark.parametrize("M,K", [(1, 32), (1, 2560), (3, 96), (19, 288), (64, 9216)])
@pytest.mark.parametrize("x_bf16", [True, False])
def test_act_quant(M, K, x_bf16):
    rng = np.random.default_rng(M * 100 + K)
    x = rng.standard_normal((M, K)).astype(np.float32) * rng.choice([1e-3, 1.0, 30.0], size=(M, 1)).astype(np.float32)
    x[0, :32] = 0  # a zero block: scale 0, integers 0 (Q8Decode.cpp:108-114)
    if x_bf16:
        x = bf16(x)
    q, s = L.ops.act_quant(x, x_bf16)
    oq, os_ = oracle.act_quant(x, x_bf16)
    assert np.array_equal(q, oq) and np.array_equal(s.view(np.uint32), os_.view(np.uint32))
    assert s[0, 0] == 0 and not q[0, :32].any()


@pytest.mark.parametrize("case", ["linear_q8_p4_decode", "linear_q8_p4_prefill", "linear_q8_p4_prefill_boundaries",
                                  "linear_q8_p4_decode_boundaries"])
def test_linear_q8_golden(golden, case):
    c = golden(case)
    N = c["w"].shape[0]
    y, dots = L.ops.linear_q8(c["x"], c["packed"], N, want_dots=True)
    assert_close(f(y), c["ref"], c["tol"], case)
    if case.endswith("boundaries"):
        assert np.array_equal(f(y), c["ref"])
    q, _ = oracle.act_quant(c["x"])
    assert np.array_equal(dots, oracle.block_dots(q, c["packed"], N))
    assert np.array_equal(y, oracle.linear_q8(c["x"], c["packed"], N))


@pytest.mark.parametrize("case", ["lm_head_q8_p4", "lm_head_q8_p4_decode"])
def test_lm_head_golden(golden, case):
    c = golden(case)
    logits, argmax = L.ops.lm_head_q8(c["x"], c["packed"], c["w"].shape[0])
    assert_close(logits, c["ref"], c["tol"], case)
    want = oracle.linear_q8(c["x"], c["packed"], c["w"].shape[0], y_bf16=False)
    assert np.array_equal(logits.view(np.uint32), want.view(np.uint32))
    assert argmax.tolist() == [oracle.argmax(row) for row in want]


# (M, N, K): decode and prefill shapes of the model plus ragged tile edges.
LINEAR_SHAPES = [(1, 9216, 2560), (1, 2560, 9216), (1, 2560, 4096), (1, 32, 2560), (1, 8, 32), (1, 136, 288),
                 (2, 8, 32), (19, 136, 288), (64, 64, 64), (65, 72, 96), (128, 1024, 2560), (1024, 256, 2560)]


@pytest.mark.parametrize("M,N,K", LINEAR_SHAPES)
def test_linear_q8_bit_exact(M, N, K):
    rng = np.random.default_rng(N + K + M)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    packed = oracle.pack_q8_0_p4(w)
    x = rand_bf16(rng, M, K)
    x[0, :32] = 0
    for activation, y_bf16 in (("none", True), ("none", False), ("silu", True), ("sigmoid", True), ("softplus", False)):
        y, dots = L.ops.linear_q8(x, packed, N, y_bf16=y_bf16, activation=activation, want_dots=True)
        want = oracle.linear_q8(x, packed, N, y_bf16=y_bf16, activation=activation)
        assert np.array_equal(y.view(np.uint16 if y_bf16 else np.uint32), want.view(np.uint16 if y_bf16 else np.uint32)), \
            (activation, y_bf16, np.abs(y.astype(np.float64) - want).max())
        if activation == "none" and y_bf16:
            q, _ = oracle.act_quant(x)
            assert np.array_equal(dots, oracle.block_dots(q, packed, N))


def test_linear_q8_f32_input_and_rows_per_warp():
    rng = np.random.default_rng(9)
    N, K = 512, 2560
    packed = oracle.pack_q8_0_p4((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    x = rng.standard_normal((1, K)).astype(np.float32)
    y = L.ops.linear_q8(x, packed, N, x_bf16=False, y_bf16=False)
    assert np.array_equal(y.view(np.uint32), oracle.linear_q8(x, packed, N, x_bf16=False, y_bf16=False).view(np.uint32))


def test_linear_q8_rejects_bad_shapes():
    with pytest.raises(L.LlmcpError):
        L.ops.linear_q8(np.zeros((1, 32), np.uint16), np.zeros(4 * 34, np.uint8), 4)  # N % 8 (Q8PackedLayout.h:38-42)
    with pytest.raises(L.LlmcpError):
        L.ops.linear_q8(np.zeros((1, 32), np.uint16), np.zeros(10, np.uint8), 8)      # size rule (LLMCPOps.cpp:46-70)
    y = L.ops.linear_q8(np.zeros((0, 32), np.uint16), np.zeros(8 * 34, np.uint8), 8)
    assert y.shape == (0, 8)


def test_lm_head_large_vocab_argmax_first_maximum():
    rng = np.random.default_rng(4)
    vocab, K = 31040, 2560  # one shard of the 248320-row table at TP = 8
    w = (rng.standard_normal((vocab, K)) * 0.02).astype(np.float32)
    w[20000] = w[777]  # duplicate rows: equal logits, the lower index must win
    packed = oracle.pack_q8_0_p4(w)
    h = oracle.rms_norm(rand_bf16(rng, 2, K), np.zeros(K, np.uint16))
    logits, argmax = L.ops.lm_head_q8(h, packed, vocab)
    want = oracle.linear_q8(h, packed, vocab, y_bf16=False)
    assert np.array_equal(logits.view(np.uint32), want.view(np.uint32))
    assert argmax.tolist() == [oracle.argmax(row) for row in want]
    boosted = w.copy()
    boosted[777] *= 0
    boosted[20000] *= 0
    boosted[[777, 20000]] += (f(h[0]) / np.abs(f(h[0])).max() * 0.05).astype(np.float32)
    packed = oracle.pack_q8_0_p4(boosted)
    logits, argmax = L.ops.lm_head_q8(h[:1], packed, vocab)
    assert logits[0, 777] == logits[0, 20000] == logits.max() and argmax[0] == 777


def test_embedding(golden):
    c = golden("embedding_q8_p4")
    out = L.ops.embedding_q8(c["tokens"], c["packed"], *c["table"].shape)
    assert np.array_equal(f(out), c["ref"])
    rng = np.random.default_rng(5)
    packed = oracle.pack_q8_0_p4((rng.standard_normal((512, 2560)) * 0.02).astype(np.float32))
    tokens = np.array([0, 511, 3, 3, 258], dtype=np.int64)
    assert np.array_equal(L.ops.embedding_q8(tokens, packed, 512, 2560), oracle.embedding_q8(tokens, packed, 2560))
    with pytest.raises(L.LlmcpError):
        L.ops.embedding_q8(np.array([512]), packed, 512, 2560)


def test_rms_norm(golden):
    for case, zc in (("rms_zero_centered", True), ("rms_plain", False)):
        c = golden(case)
        assert_close(f(L.ops.rms_norm(c["x"], c["w"], zero_centered=zc)), c["ref"], c["tol"], case)
    rng = np.random.default_rng(6)
    for M, H in ((1, 2560), (5, 2560), (1024, 2560), (3, 72), (2, 7)):
        x = rand_bf16(rng, M, H, scale=3.0)
        w = rand_bf16(rng, H, scale=0.1)
        for zc in (True, False):
            assert np.array_equal(L.ops.rms_norm(x, w, zero_centered=zc), oracle.rms_norm(x, w, zero_centered=zc))
        wf = rng.standard_normal(H).astype(np.float32)
        assert np.array_equal(L.ops.rms_norm(x, wf, w_bf16=False), oracle.rms_norm(x, wf, w_bf16=False))


def adversarial_rows(rng, M, H):
    """Rows that stress the order of the sum of squares: wide dynamic range, outliers, growing
    and repeating magnitudes, many exact rounding ties, zeros in front, all zeros, infinities."""
    rows = []
    position = np.arange(H, dtype=np.float64)
    for r in range(M):
        kind = r % 12
        scale = 2.0 ** rng.integers(-30, 30)
        if kind == 0:
            x = rng.standard_normal(H)
        elif kind == 1:
            x = rng.standard_normal(H) * scale
        elif kind == 2:
            x = np.where(rng.random(H) < 0.02, rng.standard_normal(H) * 100.0, rng.standard_normal(H) * 0.1)
        elif kind == 3:
            x = 1.01 ** position * 1e-6
        elif kind == 4:
            x = rng.integers(0, 8, H) * 0.25
        elif kind == 5:
            x = np.where(position % 97 == 0, 0.0, rng.random(H))
        elif kind == 6:
            x = 2.0 ** (position % 40 - 20)
        elif kind == 7:
            x = np.where(position < 5, 0.0, rng.standard_normal(H) * scale)
        elif kind == 8:
            x = 1.0 + rng.integers(0, 3, H) * 0.5
        elif kind == 9:
            x = np.zeros(H)
        elif kind == 10:
            x = rng.standard_normal(H) * 2.0 ** rng.integers(-8, 8, H)
        else:
            x = rng.standard_normal(H)
            x[rng.integers(0, H)] = np.inf if r % 24 == 11 else 1e30
        rows.append(x)
    return bf16(np.stack(rows))


@pytest.mark.parametrize("H", [2560, 4096, 1024, 96, 8192])
def test_rms_norm_sum_order(H):
    """The sum of squares is the reference's serial sum whatever the data, both from the
    one-thread chain and from the block-wide evaluation."""
    rng = np.random.default_rng(H)
    x = adversarial_rows(rng, 600, H)
    w = rand_bf16(rng, H, scale=0.1)
    with np.errstate(all="ignore"):
        want = oracle.rms_norm(x, w)
        got = L.ops.rms_norm(x, w)  # many rows: one thread per row adds the squares
        # few rows per call: the whole block evaluates the same serial sum
        few = np.concatenate([L.ops.rms_norm(x[i:i + 48], w) for i in range(0, len(x), 48)])
    assert np.array_equal(few, got), np.argwhere((few != got).any(axis=1)).ravel()[:10]
    # NaN results (rows holding an infinity) are compared as NaN: the payload is the processor's.
    is_nan = lambda v: (v & 0x7fff) > 0x7f80
    same = (got == want) | (is_nan(got) & is_nan(want))
    assert same.all(), np.argwhere(~same.all(axis=1)).ravel()[:10]


def test_pointwise(golden):
    c = golden("add")
    assert np.array_equal(f(L.ops.pointwise(c["a"], c["b"], "add")), c["ref"])
    c = golden("silu_mul")
    assert_close(f(L.ops.pointwise(c["gate"], c["up"], "silu_mul")), c["ref"], c["tol"])
    c = golden("mul_silu_mul")
    product = L.ops.pointwise(c["gate"], c["up"], "mul")
    assert_close(f(L.ops.pointwise(c["gate"], product, "silu_mul")), c["ref"], c["tol"])
    rng = np.random.default_rng(7)
    a, b = rand_bf16(rng, 1024, 96, scale=4.0), rand_bf16(rng, 1024, 96, scale=4.0)
    for op in ("add", "mul", "silu_mul"):
        assert np.array_equal(L.ops.pointwise(a, b, op), oracle.pointwise(a, b, op)), op


def test_gated_rms_norm(golden):
    c = golden("gated_rms_norm")
    assert_close(f(L.ops.gated_rms_norm(c["x"], c["gate"], c["w"], int(c["group"]))), c["ref"], c["tol"])
    c = golden("gated_rms_norm_activated")
    assert_close(f(L.ops.gated_rms_norm(c["x"], c["gate"], c["w"], int(c["group"]), gate_activated=True)), c["ref"], c["tol"])
    rng = np.random.default_rng(8)
    for M, H, group in ((1, 4096, 128), (33, 4096, 128), (2, 24, 12), (3, 64, 64)):
        x, g = rand_bf16(rng, M, H, scale=2.0), rand_bf16(rng, M, H, scale=2.0)
        w = rng.standard_normal(group).astype(np.float32)
        for activated in (False, True):
            got = L.ops.gated_rms_norm(x, g, w, group, gate_activated=activated)
            assert np.array_equal(got, oracle.gated_rms_norm(x, g, w, group, gate_activated=activated))
        wb = rand_bf16(rng, group)
        assert np.array_equal(L.ops.gated_rms_norm(x, g, wb, group, w_bf16=True),
                              oracle.gated_rms_norm(x, g, wb, group, w_bf16=True))


def test_causal_conv1d(golden):
    for case in ("causal_conv1d", "causal_conv1d_decode"):
        c = golden(case)
        w = c["w"].reshape(c["w"].shape[0], -1)
        y, state = L.ops.causal_conv1d(c["x"], w, c["state"], int(c["kernel"]))
        assert_close(f(y), c["ref"], c["tol"], case)
        assert np.array_equal(state, c["ref_state"])
    rng = np.random.default_rng(10)
    for S, C, kernel in ((1, 8192, 4), (2, 8192, 4), (3, 64, 4), (1024, 8192, 4), (5, 40, 2), (1, 16, 6)):
        x, w = rand_bf16(rng, S, C), rand_bf16(rng, C, kernel, scale=0.5)
        state = rand_bf16(rng, kernel - 1, C)
        y, new_state = L.ops.causal_conv1d(x, w, state, kernel)
        oy, ostate = oracle.causal_conv1d(x, w, state, kernel)
        assert np.array_equal(y, oy) and np.array_equal(new_state, ostate), (S, C, kernel)


def test_gated_delta_net(golden):
    for case in [n for n in golden.names() if n.startswith("gated_delta_net")]:
        c = golden(case)
        seq, nk, nv, dk, dv = (int(v) for v in c["dims"])
        out, state = L.ops.gated_delta_net(c["conv"], c["a"], c["b"], c["a_log"], c["dt_bias"], c["state"], nk, nv, dk, dv)
        assert_close(f(out), c["ref"], c["tol"], case)
        assert_close(state, c["ref_state"], c["tol"], case + " state")
        oo, os_ = oracle.gated_delta_net(c["conv"], c["a"], c["b"], c["a_log"], c["dt_bias"], c["state"], nk, nv, dk, dv)
        assert np.array_equal(out, oo) and np.array_equal(state.view(np.uint32), os_.view(np.uint32)), case
    rng = np.random.default_rng(11)
    # BASELINE config 3 uses 16/16 heads, the model 16/32; both, prefill and single steps.
    for S, nk, nv, dk, dv in ((1, 16, 32, 128, 128), (7, 16, 16, 128, 128), (64, 16, 32, 128, 128), (3, 2, 4, 128, 64)):
        channels = 2 * nk * dk + nv * dv
        conv, a = rand_bf16(rng, S, channels), rand_bf16(rng, S, nv)
        a_log = (rng.standard_normal(nv) * 0.2).astype(np.float32)
        dt = rand_bf16(rng, nv, scale=0.2)
        state = (rng.standard_normal((nv, dk, dv)) * 0.1).astype(np.float32)
        for activated in (False, True):
            b = rand_bf16(rng, S, nv) if not activated else bf16(1 / (1 + np.exp(-rng.standard_normal((S, nv)))))
            out, new_state = L.ops.gated_delta_net(conv, a, b, a_log, dt, state, nk, nv, dk, dv, b_activated=activated)
            oo, os_ = oracle.gated_delta_net(conv, a, b, a_log, dt, state, nk, nv, dk, dv, b_activated=activated)
            assert np.array_equal(out, oo), (S, nk, nv, activated)
            assert np.array_equal(new_state.view(np.uint32), os_.view(np.uint32))


def test_attention(golden):
    for case in ("attention", "attention_decode"):
        c = golden(case)
        seq, nh, nkv, hd, rot, cap, pos = (int(v) for v in c["dims"])
        out, cache = L.ops.attention(c["qg"], c["k"], c["v"], c["q_norm"], c["k_norm"], c["cos"], c["sin"], c["cache"],
                                     pos, nh, nkv, hd, rot)
        assert_close(f(out), c["ref"], c["tol"], case)
        assert_close(f(cache), f(c["ref_cache"]), c["tol"], case + " cache")
    rng = np.random.default_rng(12)
    nh, nkv, hd, rot = 16, 4, 256, 64
    q_norm, k_norm = rand_bf16(rng, hd, scale=0.1), rand_bf16(rng, hd, scale=0.1)
    # prefill at 0; a chunk appended after it; single-token steps at 63/64/65 (tile edges) and 1024.
    for S, pos, cap in ((70, 0, 80), (5, 64, 80), (1, 63, 80), (1, 64, 80), (1, 65, 80), (1, 1024, 1032), (130, 0, 130),
                        (300, 0, 300)):  # 300 keys: the value ring of the prefill kernel wraps twice
        qg, k, v = rand_bf16(rng, S, nh * 2 * hd), rand_bf16(rng, S, nkv * hd), rand_bf16(rng, S, nkv * hd)
        cos = np.stack([L.make_cos_sin(pos + t)[0] for t in range(S)])
        sin = np.stack([L.make_cos_sin(pos + t)[1] for t in range(S)])
        cache = rand_bf16(rng, 2, nkv, cap, hd)
        out, new_cache = L.ops.attention(qg, k, v, q_norm, k_norm, cos, sin, cache, pos, nh, nkv, hd, rot)
        oo, oc = oracle.attention(qg, k, v, q_norm, k_norm, cos, sin, cache, pos, nh, nkv, hd, rot)
        assert np.array_equal(new_cache, oc), (S, pos)
        assert np.array_equal(out, oo), (S, pos, np.abs(f(out) - f(oo)).max())
    with pytest.raises(L.LlmcpError):
        L.ops.attention(qg, k, v, q_norm, k_norm, cos, sin, cache, cap, nh, nkv, hd, rot)  # past the cache


@pytest.mark.parametrize("N,K", [(2560, 4096), (2560, 9216), (9216, 2560), (1024, 2560), (248, 4096)])
def test_gemv_kernel_variants(N, K):
    """The block-column and row decode GEMV kernels and the oracle agree bit for bit."""
    import ctypes as C
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(N + K)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    packed = oracle.pack_q8_0_p4(w)
    x = rand_bf16(rng, 1, K)
    want = oracle.linear_q8(x, packed, N, y_bf16=False)[0]
    lib = L.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: C.c_void_p(t.data_ptr())
    records = torch.from_numpy(packed).cuda()
    wq = torch.empty((N, K), dtype=torch.int8, device="cuda")
    wd = torch.empty((N, K // 32), dtype=torch.float16, device="cuda")
    assert lib.llmcp_dev_repack_q8(ptr(records), C.c_int64(N), C.c_int64(K), ptr(wq), ptr(wd), stream) == 0
    xd = torch.from_numpy(x.view(np.int16)).cuda()
    aq = torch.empty(K, dtype=torch.int8, device="cuda")
    scales = torch.empty(K // 32, dtype=torch.float32, device="cuda")
    assert lib.llmcp_dev_act_quant(ptr(xd), 1, C.c_int64(1), C.c_int64(K), ptr(aq), ptr(scales), stream) == 0
    for flags in (0, 1, 3, 8, 9):  # default kernels, dependent launch, L2 prefetch, row kernel
        y = torch.full((N,), float("nan"), dtype=torch.float32, device="cuda")
        rc = lib.llmcp_dev_gemv_q8(ptr(aq), ptr(scales), C.c_int64(K), ptr(wq), ptr(wd), C.c_int64(N), ptr(y), 0, 0, 0,
                                   flags, stream)
        assert rc == 0, L.last_error()
        torch.cuda.synchronize()
        got = y.cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"flags {flags}"


@pytest.mark.parametrize("N", [9216, 1152, 64])
def test_gemv_swiglu_one_launch(N):
    """gate and up projections, SiLU, product and the product's int8 quantisation in one launch:
    bit for bit what the oracle's linear(silu) x linear -> mul -> act_quant chain gives (exact form),
    and within the fast form's bar (a bf16 step of the product on near-ties)."""
    import ctypes as C
    torch = pytest.importorskip("torch")
    K = 2560
    rng = np.random.default_rng(N)
    packed = [oracle.pack_q8_0_p4((rng.standard_normal((N, K)) * 0.02).astype(np.float32)) for _ in range(2)]
    x = rand_bf16(rng, 1, K)
    gate = oracle.linear_q8(x, packed[0], N, activation="silu")
    up = oracle.linear_q8(x, packed[1], N)
    want = oracle.pointwise(gate, up, "mul")
    want_q, want_s = oracle.act_quant(want)
    lib = L.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: C.c_void_p(t.data_ptr())
    planes = []
    for records in packed:
        wq = torch.empty((N, K), dtype=torch.int8, device="cuda")
        wd = torch.empty((N, K // 32), dtype=torch.float16, device="cuda")
        assert lib.llmcp_dev_repack_q8(ptr(torch.from_numpy(records).cuda()), C.c_int64(N), C.c_int64(K), ptr(wq), ptr(wd), stream) == 0
        planes += [wq, wd]
    xd = torch.from_numpy(x.view(np.int16)).cuda()
    aq = torch.empty(K, dtype=torch.int8, device="cuda")
    scales = torch.empty(K // 32, dtype=torch.float32, device="cuda")
    assert lib.llmcp_dev_act_quant(ptr(xd), 1, C.c_int64(1), C.c_int64(K), ptr(aq), ptr(scales), stream) == 0
    for flags in (0, 1, 16, 17):
        product = torch.zeros(N, dtype=torch.int16, device="cuda")
        q = torch.zeros(N, dtype=torch.int8, device="cuda")
        s = torch.zeros(N // 32, dtype=torch.float32, device="cuda")
        rc = lib.llmcp_dev_gemv_q8_swiglu(ptr(aq), ptr(scales), C.c_int64(K), ptr(planes[0]), ptr(planes[1]), ptr(planes[2]),
                                          ptr(planes[3]), C.c_int64(N), ptr(product), ptr(q), ptr(s), flags, stream)
        assert rc == 0, L.last_error()
        torch.cuda.synchronize()
        got = product.cpu().numpy().view(np.uint16)[None]
        if flags & 16:
            steps = np.abs(got.astype(np.int32) - want.astype(np.int32))
            assert steps.max() <= 2 and (steps != 0).mean() < 0.05, (flags, steps.max(), (steps != 0).mean())
            again_q, again_s = oracle.act_quant(got)  # the quantisation itself is exact on the kernel's own product
            assert np.array_equal(q.cpu().numpy()[None], again_q) and np.array_equal(s.cpu().numpy()[None], again_s)
        else:
            assert np.array_equal(got, want), flags
            assert np.array_equal(q.cpu().numpy()[None], want_q), flags
            assert np.array_equal(s.cpu().numpy()[None].view(np.uint32), want_s.view(np.uint32)), flags
    # refusals: the product may not overwrite the input, other K
    assert lib.llmcp_dev_gemv_q8_swiglu(ptr(aq), ptr(scales), C.c_int64(K), ptr(planes[0]), ptr(planes[1]), ptr(planes[2]),
                                        ptr(planes[3]), C.c_int64(N), None, ptr(aq), ptr(s), 0, stream) != 0
    assert lib.llmcp_dev_gemv_q8_swiglu(ptr(aq), ptr(scales), C.c_int64(4096), ptr(planes[0]), ptr(planes[1]), ptr(planes[2]),
                                        ptr(planes[3]), C.c_int64(N), None, ptr(q), ptr(s), 0, stream) != 0


def _tma_gemm_setup(torch, M, N, K, seed):
    """Operand and scale planes of the TMA-fed tensor-core GEMM on the device, and the oracle's result."""
    import ctypes as C
    rng = np.random.default_rng(seed)
    packed = oracle.pack_q8_0_p4((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    x = rand_bf16(rng, M, K)
    want = oracle.linear_q8(x, packed, N, y_bf16=False)
    lib = L.lib()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ptr = lambda t: C.c_void_p(t.data_ptr())
    records = torch.from_numpy(packed).cuda()
    wq = torch.empty((N, K), dtype=torch.int8, device="cuda")
    wd = torch.empty((N, K // 32), dtype=torch.float16, device="cuda")
    assert lib.llmcp_dev_repack_q8(ptr(records), C.c_int64(N), C.c_int64(K), ptr(wq), ptr(wd), stream) == 0
    xd = torch.from_numpy(x.view(np.int16)).cuda()
    aq = torch.empty((M, K), dtype=torch.int8, device="cuda")
    scales = torch.empty((M, K // 32), dtype=torch.float32, device="cuda")
    assert lib.llmcp_dev_act_quant(ptr(xd), 1, C.c_int64(M), C.c_int64(K), ptr(aq), ptr(scales), stream) == 0
    lib.llmcp_dev_gemm_q8_tma_scale_pitch.restype = C.c_int64
    pitch = int(lib.llmcp_dev_gemm_q8_tma_scale_pitch(C.c_int64(M)))
    ah = torch.empty((M, K), dtype=torch.float16, device="cuda")
    ast = torch.zeros((K // 32, pitch), dtype=torch.float32, device="cuda")
    wh = torch.empty((N, K), dtype=torch.float16, device="cuda")
    wst = torch.empty((K // 32, N), dtype=torch.float32, device="cuda")
    assert lib.llmcp_dev_q8_gemm_planes(ptr(aq), ptr(scales), 0, C.c_int64(M), C.c_int64(K), ptr(ah), ptr(ast), stream) == 0
    assert lib.llmcp_dev_q8_gemm_planes(ptr(wq), ptr(wd), 1, C.c_int64(N), C.c_int64(K), ptr(wh), ptr(wst), stream) == 0
    torch.cuda.synchronize()
    # the planes hold the same integers and the same scale values
    assert torch.equal(ah.to(torch.int8), aq) and torch.equal(wh.to(torch.int8), wq)
    assert torch.equal(ast[:, :M].t().contiguous(), scales) and torch.equal(wst.t().contiguous(), wd.float())
    # the scale planes alone (the int8 forms need nothing else)
    ast2, wst2 = torch.zeros_like(ast), torch.zeros_like(wst)
    assert lib.llmcp_dev_q8_gemm_planes(None, ptr(scales), 0, C.c_int64(M), C.c_int64(K), None, ptr(ast2), stream) == 0
    assert lib.llmcp_dev_q8_gemm_planes(None, ptr(wd), 1, C.c_int64(N), C.c_int64(K), None, ptr(wst2), stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(ast2, ast) and torch.equal(wst2, wst)
    return lib, stream, ptr, {"aq": aq, "wq": wq, "ah": ah, "wh": wh, "ast": ast, "wst": wst}, want


def _tma_gemm(lib, stream, ptr, planes, form, M, N, K, y, status, spin_limit=0, fault=0):
    import ctypes as C
    a, w = (planes["ah"], planes["wh"]) if form >= 2 else (planes["aq"], planes["wq"])
    rc = lib.llmcp_dev_gemm_q8_tma(form, ptr(a), ptr(planes["ast"]), C.c_int64(M), C.c_int64(K), ptr(w), ptr(planes["wst"]),
                                   C.c_int64(N), ptr(y), 0, 0, ptr(status), C.c_uint32(spin_limit), fault, stream)
    assert rc == 0, L.last_error()


@pytest.mark.parametrize("M,N,K", [(128, 256, 2560), (300, 136, 288), (2, 8, 32), (1024, 1024, 4096)])
def test_gemm_tma_device_entry(M, N, K):
    """llmcp_dev_gemm_q8_tma on device planes, all four forms: bit-identical to the oracle."""
    torch = pytest.importorskip("torch")
    lib, stream, ptr, planes, want = _tma_gemm_setup(torch, M, N, K, M + N + K)
    for form in range(4):
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        y = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
        _tma_gemm(lib, stream, ptr, planes, form, M, N, K, y, status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32)), form


@pytest.mark.parametrize("form", [1, 3])
def test_gemm_tma_bounded_wait_runs_out_and_recovers(form):
    """The test hook withholds the first stage's copies: every wait behind it must give up after its
    bounded number of polls, the kernel must report through the status word, write nothing, free
    its tensor memory and leave the context usable: the next launch is correct."""
    torch = pytest.importorskip("torch")
    M, N, K = 256, 384, 2560
    lib, stream, ptr, planes, want = _tma_gemm_setup(torch, M, N, K, 99)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = torch.full((M, N), 7.0, dtype=torch.float32, device="cuda")
    _tma_gemm(lib, stream, ptr, planes, form, M, N, K, y, status, spin_limit=1 << 12, fault=1)
    torch.cuda.synchronize()  # returns: nothing hangs
    assert int(status.item()) == 1
    assert bool((y == 7.0).all()), "a tile that gave up writes no output"
    status.zero_()
    for _ in range(3):  # tensor memory was released: full-occupancy launches still fit
        _tma_gemm(lib, stream, ptr, planes, form, M, N, K, y, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_linear_q8_every_gemm_form(monkeypatch):
    """Every prefill GEMM form stays selectable and exact, int32 block dots included."""
    rng = np.random.default_rng(21)
    M, N, K = 130, 264, 2560
    packed = oracle.pack_q8_0_p4((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    x = rand_bf16(rng, M, K)
    want = oracle.linear_q8(x, packed, N, y_bf16=False)
    q, _ = oracle.act_quant(x)
    want_dots = oracle.block_dots(q, packed, N)
    for form in ("i8-cpasync", "dp4a", "i8", "i8x2", "f16", "f16x2"):
        monkeypatch.setenv("LLMCP_B200_GEMM", form)
        y, dots = L.ops.linear_q8(x, packed, N, y_bf16=False, want_dots=True)
        assert np.array_equal(y.view(np.uint32), want.view(np.uint32)), form
        assert np.array_equal(dots, want_dots), form


def test_linear_q8_both_tile_widths(monkeypatch):
    """The TMA-fed GEMM with 128- and with 160-column tiles (the second exists for matrices whose
    128-wide tiles would leave a nearly empty last wave): every form exact, block dots included, a
    partial last tile in both directions, bf16 output with an activation; and the automatic choice on
    a 1024 x 2560 output (160 tiles of 128 columns against 128 tiles of 160 in one wave)."""
    rng = np.random.default_rng(33)
    M, N, K = 130, 264, 2560
    packed = oracle.pack_q8_0_p4((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    x = rand_bf16(rng, M, K)
    want = oracle.linear_q8(x, packed, N, y_bf16=False)
    want_silu = oracle.linear_q8(x, packed, N, activation="silu")
    q, _ = oracle.act_quant(x)
    want_dots = oracle.block_dots(q, packed, N)
    for tile in ("128", "160"):
        monkeypatch.setenv("LLMCP_B200_GEMM_TILE", tile)
        for form in ("i8", "i8x2", "f16", "f16x2"):
            monkeypatch.setenv("LLMCP_B200_GEMM", form)
            y, dots = L.ops.linear_q8(x, packed, N, y_bf16=False, want_dots=True)
            assert np.array_equal(y.view(np.uint32), want.view(np.uint32)), (tile, form)
            assert np.array_equal(dots, want_dots), (tile, form)
            assert np.array_equal(L.ops.linear_q8(x, packed, N, activation="silu"), want_silu), (tile, form)
    monkeypatch.delenv("LLMCP_B200_GEMM_TILE")
    monkeypatch.delenv("LLMCP_B200_GEMM")
    M, N, K = 1024, 2560, 256
    packed = oracle.pack_q8_0_p4((rng.standard_normal((N, K)) * 0.02).astype(np.float32))
    x = rand_bf16(rng, M, K)
    y, dots = L.ops.linear_q8(x, packed, N, y_bf16=False, want_dots=True)
    assert np.array_equal(y.view(np.uint32), oracle.linear_q8(x, packed, N, y_bf16=False).view(np.uint32))
    assert np.array_equal(dots, oracle.block_dots(oracle.act_quant(x)[0], packed, N))

