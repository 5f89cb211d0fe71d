#!/usr/bin/env python3
"""Generates tests/golden/llmcp_numeric.npz from the reference's numeric test file.

Run inside a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

The reference's tests/numeric/run_numeric.py is imported for its Q8_0 helpers
(q8_0_blocks, q8_0_dequant, q8_0_p4_bytes; run_numeric.py:105-148).  The inputs
are drawn with the same seed and in the same order as its main()
(run_numeric.py:676-1110), and the expected values are the closed-form PyTorch
formulas that main() compares the compiled kernels against, restated here
because they are inline in main() and cannot be imported.  Every case stores its
inputs, the expected outputs and the (rel, abs) tolerance the reference uses.

The fixture travels with the repository; the reference checkout does not.
"""
import importlib.util
import pathlib
import sys

import numpy as np
import torch

bf16 = torch.bfloat16


def bits(t):
    """bf16 tensor -> uint16 numpy array of its bit patterns."""
    return t.to(bf16).contiguous().view(torch.int16).numpy().astype(np.uint16)


def f32(t):
    return t.float().contiguous().numpy()


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <checkout of the llmcp project>")
    ref_root = pathlib.Path(sys.argv[1])
    spec = importlib.util.spec_from_file_location(
        "run_numeric", ref_root / "tests/numeric/run_numeric.py")
    rn = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(rn)

    out = {}

    def put(case, tol, **arrays):
        for key, value in arrays.items():
            out[f"{case}/{key}"] = np.asarray(value)
        out[f"{case}/tol"] = np.asarray(tol, dtype=np.float64)

    def packed(w):
        return np.asarray(rn.q8_0_p4_bytes(w.tolist()), dtype=np.int64).astype(np.uint8)

    def dequant(t):
        return torch.tensor(rn.q8_0_dequant(t.tolist()), dtype=torch.float32).reshape(t.shape)

    torch.manual_seed(0)

    # run_numeric.py:676-689 (bf16 linears: consumed to keep the RNG stream aligned)
    torch.randn(2, 4); torch.randn(3, 4)
    torch.randn(2, 64); torch.randn(64, 64)

    rng = torch.Generator().manual_seed(0)
    m, n, k = 19, 136, 288
    blocks = k // 32

    def exact_q8_operand(rows):
        values = torch.randint(-63, 64, (rows, blocks, 32), generator=rng)
        values[:, :, 0] = 127
        exponents = torch.randint(-6, -4, (rows, blocks, 1), generator=rng)
        return torch.ldexp(values.float(), exponents).reshape(rows, k).to(bf16)

    # run_numeric.py:702-718
    x = torch.randn(1, 64).to(bf16)
    w = torch.randn(64, 64).to(bf16)
    wq = dequant(w)
    ref = (dequant(x) @ wq.T).to(bf16).float()
    put("linear_q8_p4_decode", (1e-2, 2e-3), x=bits(x), w=bits(w), packed=packed(w), ref=f32(ref))
    x = torch.randn(8, 64).to(bf16)
    ref = (dequant(x) @ wq.T).to(bf16).float()
    put("linear_q8_p4_prefill", (2e-2, 5e-3), x=bits(x), w=bits(w), packed=packed(w), ref=f32(ref))
    # run_numeric.py:719-732 (exact known-answer construction)
    x = exact_q8_operand(m)
    w = exact_q8_operand(n)
    x[0, -32:] = 0
    ref = (x.float() @ w.float().T).to(bf16).float()
    put("linear_q8_p4_prefill_boundaries", (1e-5, 1e-6), x=bits(x), w=bits(w), packed=packed(w), ref=f32(ref))
    x = exact_q8_operand(1)
    w = exact_q8_operand(n)
    x[0, -32:] = 0
    ref = (x.float() @ w.float().T).to(bf16).float()
    put("linear_q8_p4_decode_boundaries", (1e-5, 1e-6), x=bits(x), w=bits(w), packed=packed(w), ref=f32(ref))

    # run_numeric.py:734-749 rms_norm
    x = torch.randn(2, 8).to(bf16)
    w = torch.randn(8).to(bf16)
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)
    put("rms_zero_centered", (2e-2, 1e-2), x=bits(x), w=bits(w),
        ref=f32((xf * rstd * (1.0 + w.float())).to(bf16)))
    put("rms_plain", (2e-2, 1e-2), x=bits(x), w=bits(w),
        ref=f32((xf * rstd * w.float()).to(bf16)))

    # run_numeric.py:751-759 add
    a = torch.randn(2, 4).to(bf16)
    b = torch.randn(2, 4).to(bf16)
    put("add", (2e-2, 1e-2), a=bits(a), b=bits(b), ref=f32((a.float() + b.float()).to(bf16)))

    # run_numeric.py:761-782 silu_mul and mul -> silu_mul
    gate = torch.randn(2, 4).to(bf16)
    up = torch.randn(2, 4).to(bf16)
    put("silu_mul", (2e-2, 1e-2), gate=bits(gate), up=bits(up),
        ref=f32((gate.float() * torch.sigmoid(gate.float()) * up.float()).to(bf16)))
    product = (gate.float() * up.float()).to(bf16).float()
    put("mul_silu_mul", (2e-2, 1e-2), gate=bits(gate), up=bits(up),
        ref=f32((gate.float() * torch.sigmoid(gate.float()) * product).to(bf16)))

    # run_numeric.py:784-799 embedding
    torch.randn(4, 3)
    table_q8 = torch.randn(8, 32).to(bf16)
    tokens = [2, 0]
    ref = dequant(table_q8)[tokens].to(bf16).float()
    put("embedding_q8_p4", (2e-2, 1e-2), table=bits(table_q8), packed=packed(table_q8),
        tokens=np.asarray(tokens, dtype=np.int64), ref=f32(ref))

    # run_numeric.py:801-826 gated_rms_norm
    m2, groups, group = 2, 2, 4
    x = torch.randn(m2, groups * group).to(bf16)
    gate = torch.randn(m2, groups * group).to(bf16)
    weight = torch.randn(group).float()
    xf = x.float().view(m2, groups, group)
    gf = gate.float().view(m2, groups, group)
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6)
    ref = (xf * rstd * weight * torch.nn.functional.silu(gf)).view(m2, -1).to(bf16)
    put("gated_rms_norm", (2e-2, 1e-2), x=bits(x), gate=bits(gate), w=f32(weight),
        group=group, ref=f32(ref))
    ref = (xf * rstd * weight * gf).view(m2, -1).to(bf16)
    put("gated_rms_norm_activated", (2e-2, 1e-2), x=bits(x), gate=bits(gate), w=f32(weight),
        group=group, ref=f32(ref))

    # run_numeric.py:828-862 lm_head
    torch.randn(2, 3); torch.randn(4, 3)
    hidden = torch.randn(2, 64).to(bf16)
    table = torch.randn(64, 64).to(bf16)
    tq = dequant(table)
    put("lm_head_q8_p4", (2e-2, 5e-3), x=bits(hidden), w=bits(table), packed=packed(table),
        ref=f32(dequant(hidden) @ tq.T))
    hidden = torch.randn(1, 64).to(bf16)
    put("lm_head_q8_p4_decode", (1e-2, 2e-3), x=bits(hidden), w=bits(table), packed=packed(table),
        ref=f32(dequant(hidden) @ tq.T))
    torch.randn(2, 64); torch.randn(64, 64)
    for sequence in (1, 7):
        torch.randn(sequence, 64)

    # run_numeric.py:864-907 causal_conv1d (the Python formula rounds the sum to
    # bf16 before SiLU; the lowering does not, hence the loose tolerance)
    channels, kernel = 4, 3
    state_len = kernel - 1
    weight = None
    for case, seq in (("causal_conv1d", 3), ("causal_conv1d_decode", 1)):
        x = torch.randn(seq, channels).to(bf16)
        if weight is None:
            weight = torch.randn(channels, 1, kernel).to(bf16)
        state = torch.randn(1, state_len, channels).to(bf16)
        padded = torch.cat([state[0], x], dim=0)
        y = torch.empty(seq, channels, dtype=bf16)
        for t in range(seq):
            for c in range(channels):
                acc = 0.0
                for kk in range(kernel):
                    acc += float(padded[t + kk, c].float()) * float(weight[c, 0, kk].float())
                y[t, c] = torch.tensor(acc).to(bf16)
        y = (y.float() * torch.sigmoid(y.float())).to(bf16)
        put(case, (2e-2, 1e-2), x=bits(x), w=bits(weight), state=bits(state[0]),
            kernel=kernel, ref=f32(y), ref_state=bits(padded[-state_len:]))

    # run_numeric.py:909-1029 gated_delta_net
    def gdn_case(case, seq, num_k, num_v, head_k, head_v, tol, a_log=None, dt_bias=None):
        channels = 2 * num_k * head_k + num_v * head_v
        conv = torch.randn(seq, channels).to(bf16)
        a = torch.randn(seq, num_v).to(bf16)
        b = torch.randn(seq, num_v).to(bf16)
        if a_log is None:
            a_log = torch.randn(num_v).float()
            dt_bias = torch.randn(num_v).to(bf16)
        state = torch.randn(1, num_v, head_k, head_v).float()
        q = conv[:, :num_k * head_k].float().view(seq, num_k, head_k)
        kk = conv[:, num_k * head_k:2 * num_k * head_k].float().view(seq, num_k, head_k)
        v = conv[:, 2 * num_k * head_k:].float().view(seq, num_v, head_v)
        ref_state = state.clone()
        ref_out = torch.empty(seq, num_v * head_v, dtype=bf16)
        for t in range(seq):
            for h in range(num_v):
                kh = h // (num_v // num_k)
                qh = q[t, kh]
                key = kk[t, kh]
                qh = qh * torch.rsqrt((qh * qh).sum() + 1e-6)
                key = key * torch.rsqrt((key * key).sum() + 1e-6)
                qh = qh / (head_k ** 0.5)
                beta = torch.sigmoid(b[t, h].float())
                g = -torch.exp(a_log[h]) * torch.nn.functional.softplus(
                    a[t, h].float() + dt_bias[h].float())
                ref_state[0, h] = ref_state[0, h] * torch.exp(g)
                predicted = (ref_state[0, h] * key.unsqueeze(-1)).sum(dim=0)
                delta = (v[t, h] - predicted) * beta
                ref_state[0, h] = ref_state[0, h] + key.unsqueeze(-1) * delta
                o = (ref_state[0, h] * qh.unsqueeze(-1)).sum(dim=0)
                ref_out[t, h * head_v:(h + 1) * head_v] = o.to(bf16)
        put(case, tol, conv=bits(conv), a=bits(a), b=bits(b), a_log=f32(a_log),
            dt_bias=bits(dt_bias), state=f32(state[0]),
            dims=np.asarray([seq, num_k, num_v, head_k, head_v], dtype=np.int64),
            ref=f32(ref_out), ref_state=f32(ref_state[0]))
        return a_log, dt_bias

    a_log, dt_bias = gdn_case("gated_delta_net", 2, 2, 4, 2, 2, (2e-2, 1e-2))
    gdn_case("gated_delta_net_decode", 1, 2, 4, 2, 2, (2e-2, 1e-2), a_log, dt_bias)
    for seq, head_k, head_v in ((1, 5, 8), (3, 5, 8), (3, 5, 16), (1, 5, 7), (1, 9, 4)):
        gdn_case(f"gated_delta_net_{seq}_{head_k}_{head_v}", seq, 2, 4, head_k, head_v,
                 (2e-2, 1e-3))

    # run_numeric.py:1031-1110 attention
    num_heads, num_kv_heads, head_dim, rotary = 2, 1, 4, 2
    cap = 2
    q_norm = k_norm = None

    def attention_case(case, seq, position):
        nonlocal q_norm, k_norm
        qg = torch.randn(seq, num_heads * 2 * head_dim).to(bf16)
        kx = torch.randn(seq, num_kv_heads * head_dim).to(bf16)
        vx = torch.randn(seq, num_kv_heads * head_dim).to(bf16)
        if q_norm is None:
            q_norm = torch.randn(head_dim).to(bf16)
            k_norm = torch.randn(head_dim).to(bf16)
        cos = torch.randn(seq, rotary).float()
        sin = torch.randn(seq, rotary).float()
        cache = torch.randn(1, 2, num_kv_heads, cap, head_dim).to(bf16)
        q_ = qg.view(-1, num_heads, 2, head_dim)[:, :, 0, :].float()
        gate_ = qg.view(-1, num_heads, 2, head_dim)[:, :, 1, :].float()
        kf_ = kx.view(-1, num_kv_heads, head_dim).float()
        vf_ = vx.view(-1, num_kv_heads, head_dim).float()

        def norm_rope(xx, weight):
            inv = torch.rsqrt(xx.pow(2).mean(-1, keepdim=True) + 1e-6)
            y = xx * inv * (1.0 + weight.float())
            o = y.clone()
            for d in range(rotary):
                partner = d - rotary // 2 if d >= rotary // 2 else d + rotary // 2
                sign = 1.0 if d >= rotary // 2 else -1.0
                o[..., d] = y[..., d] * cos[:, d].view(-1, 1) + sign * y[..., partner] * sin[:, d].view(-1, 1)
            return o.to(bf16)

        qn_ = norm_rope(q_, q_norm)
        kn_ = norm_rope(kf_, k_norm)
        ref_cache = cache.clone()
        nq = qn_.shape[0]
        ref_cache[0, 0, :, position:position + nq, :] = kn_.transpose(0, 1)
        ref_cache[0, 1, :, position:position + nq, :] = vf_.transpose(0, 1)
        scale = 1.0 / (head_dim ** 0.5)
        ref_out = torch.empty(nq, num_heads * head_dim, dtype=bf16)
        group = num_heads // num_kv_heads
        for t in range(nq):
            gp = position + t
            for h in range(num_heads):
                kh = h // group
                scores = (qn_[t, h].float() @ ref_cache[0, 0, kh, :gp + 1].float().T) * scale
                probs = torch.softmax(scores, dim=-1)
                ctx = probs @ ref_cache[0, 1, kh, :gp + 1].float()
                ref_out[t, h * head_dim:(h + 1) * head_dim] = (ctx * torch.sigmoid(gate_[t, h])).to(bf16)
        put(case, (2e-2, 1e-2), qg=bits(qg), k=bits(kx), v=bits(vx), q_norm=bits(q_norm),
            k_norm=bits(k_norm), cos=f32(cos), sin=f32(sin), cache=bits(cache[0]),
            dims=np.asarray([seq, num_heads, num_kv_heads, head_dim, rotary, cap, position],
                            dtype=np.int64),
            ref=f32(ref_out), ref_cache=bits(ref_cache[0]))

    attention_case("attention", 2, 0)
    attention_case("attention_decode", 1, 1)

    # Byte-level pins of tests/unittests/QuantizationTest.cpp:57-89: bf16 1.0 x 64
    # -> scale bytes 08 20 and all q = 127; a zero block -> d = 0, q = 0.
    put("quant_pins", (0.0, 0.0), ones_scale_bytes=np.asarray([0x08, 0x20], dtype=np.uint8))

    target = pathlib.Path(__file__).with_name("llmcp_numeric.npz")
    np.savez_compressed(target, **out)
    print(f"wrote {target} with {len(out)} arrays")


if __name__ == "__main__":
    main()
