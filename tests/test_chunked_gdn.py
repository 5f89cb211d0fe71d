"""The chunk-parallel form of the gated delta rule against the token-by-token form (numpy models in
oracle/chunked_gdn.py; no GPU).  In float64 the two agree to rounding; with the matrix products'
factors rounded to tf32 or bf16 (what a tensor-core kernel would feed) the distance to the exact
recurrence is what such a kernel's tolerance has to allow for, so it is measured and bounded here."""
import numpy as np
import pytest

from oracle import chunked_gdn


def head_inputs(rng, T, dk=128, dv=128):
    q = rng.standard_normal((T, dk))
    k = rng.standard_normal((T, dk))
    q = q / np.sqrt((q * q).sum(1, keepdims=True) + 1e-6) / np.sqrt(dk)  # the operator's q and k norms
    k = k / np.sqrt((k * k).sum(1, keepdims=True) + 1e-6)
    v = rng.standard_normal((T, dv))
    beta = 1 / (1 + np.exp(-rng.standard_normal(T)))
    a_plus_dt = rng.standard_normal(T) + 0.2 * rng.standard_normal()
    decay = np.exp(-np.exp(0.2 * rng.standard_normal()) * np.log1p(np.exp(a_plus_dt)))
    state = 0.1 * rng.standard_normal((dk, dv))
    return q, k, v, beta, decay, state


@pytest.mark.parametrize("T,chunk", [(1, 64), (63, 64), (64, 64), (200, 64), (256, 16), (130, 128)])
def test_chunked_equals_sequential_in_float64(T, chunk):
    rng = np.random.default_rng(T + chunk)
    x = head_inputs(rng, T)
    want_out, want_state = chunked_gdn.sequential(*x)
    got_out, got_state = chunked_gdn.chunked(*x, chunk=chunk)
    assert np.abs(got_out - want_out).max() <= 1e-12 * max(1.0, np.abs(want_out).max())
    assert np.abs(got_state - want_state).max() <= 1e-12 * max(1.0, np.abs(want_state).max())


@pytest.mark.parametrize("operand,bar", [("tf32", 2e-3), ("bf16", 1.5e-2)])
def test_rounded_operands_stay_within_a_kernel_tolerance(operand, bar):
    """1024 tokens, chunks of 64: worst output error relative to the largest output, and the same for
    the final state, with rounded factors and float32 sums."""
    rng = np.random.default_rng(7)
    x = head_inputs(rng, 1024)
    want_out, want_state = chunked_gdn.sequential(*x)
    got_out, got_state = chunked_gdn.chunked(*x, chunk=64, operand=operand)
    out_error = np.abs(got_out - want_out).max() / np.abs(want_out).max()
    state_error = np.abs(got_state - want_state).max() / np.abs(want_state).max()
    print(f"{operand}: output {out_error:.2e}, state {state_error:.2e}")
    assert out_error <= bar and state_error <= bar


def test_strong_decay_does_not_overflow():
    rng = np.random.default_rng(3)
    q, k, v, beta, decay, state = head_inputs(rng, 192)
    decay = np.full_like(decay, 1e-3)  # gamma underflows inside a chunk; the ratios are formed in log space
    want_out, want_state = chunked_gdn.sequential(q, k, v, beta, decay, state)
    for operand in (None, "tf32"):
        got_out, got_state = chunked_gdn.chunked(q, k, v, beta, decay, state, chunk=64, operand=operand)
        assert np.isfinite(got_out).all() and np.isfinite(got_state).all()
        assert np.abs(got_out - want_out).max() <= 2e-3 * np.abs(want_out).max()
