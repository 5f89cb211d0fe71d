"""The gated delta rule in chunks (test infrastructure only): a numpy model of the chunk-parallel
form of the recurrence of lib/Dialect/LLMCP/Transforms/LowerGatedDeltaNet.cpp:129-445, for one head,
next to the token-by-token form it must agree with.

Per token t, with the state S (dk x dv), the normalised key k and query q, the value v, the decay g
(a scalar in (0, 1]) and the write strength beta, the reference does

    S <- g S;   delta = beta (v - S^T k);   S <- S + k delta^T;   o = S^T q.

Over a chunk of C tokens that starts from S0, with gamma_i = g_1 ... g_i:

    A_ij  = beta_i (gamma_i / gamma_j) (k_i . k_j)            for j < i, else 0
    Delta = (I + A)^-1 diag(beta) (V - diag(gamma) K S0)      (a unit lower-triangular solve)
    O     = diag(gamma) Q S0 + tril(Q K^T * Gamma) Delta      (Gamma_ij = gamma_i / gamma_j, j <= i)
    S_C   = gamma_C S0 + (K * (gamma_C / gamma))^T Delta

so a chunk is six small matrix products and one triangular solve, and only the chunks of a head
are sequential.  `operand` rounds the factors of those products the way a tensor-core kernel would
(None: float64 throughout; "bf16" or "tf32": rounded factors, float32 sums), which is what the
tolerance of such a kernel has to be judged on.
"""
import numpy as np


def _round(x, operand):
    if operand is None:
        return x
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    drop = 16 if operand == "bf16" else 13  # bf16 keeps 8 bits of significand, tf32 11
    bits = (bits + (1 << (drop - 1)) - 1 + ((bits >> drop) & 1)) >> drop << drop
    return bits.astype(np.uint32).view(np.float32)


def sequential(q, k, v, beta, decay, state):
    """Token by token in float64: outputs (T x dv) and the final state."""
    s = np.array(state, dtype=np.float64)
    out = np.empty((q.shape[0], s.shape[1]))
    for t in range(q.shape[0]):
        s *= decay[t]
        delta = beta[t] * (v[t] - s.T @ k[t])
        s += np.outer(k[t], delta)
        out[t] = s.T @ q[t]
    return out, s


def chunked(q, k, v, beta, decay, state, chunk=64, operand=None):
    """The same in chunks; the last chunk may be short."""
    dtype = np.float64 if operand is None else np.float32
    s = np.array(state, dtype=dtype)
    out = np.empty((q.shape[0], s.shape[1]), dtype=dtype)
    mm = lambda a, b: (_round(a, operand) @ _round(b, operand)).astype(dtype)
    for start in range(0, q.shape[0], chunk):
        stop = min(start + chunk, q.shape[0])
        Q, K, V = (x[start:stop].astype(dtype) for x in (q, k, v))
        b = beta[start:stop].astype(dtype)
        log_gamma = np.cumsum(np.log(decay[start:stop].astype(np.float64)))
        gamma = np.exp(log_gamma).astype(dtype)
        ratio = np.exp(np.minimum(log_gamma[:, None] - log_gamma[None, :], 0.0)).astype(dtype)  # gamma_i / gamma_j, used for j <= i
        n = stop - start
        lower = np.tril(np.ones((n, n), dtype=bool), -1)
        A = np.where(lower, b[:, None] * ratio * mm(K, K.T), 0).astype(dtype)
        rhs = b[:, None] * (V - gamma[:, None] * mm(K, s))
        delta = np.empty_like(rhs)
        for i in range(n):  # forward substitution, rows in float32 / float64 (a kernel does it blockwise)
            delta[i] = rhs[i] - A[i, :i] @ delta[:i]
        scores = np.where(lower | np.eye(n, dtype=bool), ratio * mm(Q, K.T), 0).astype(dtype)
        out[start:stop] = gamma[:, None] * mm(Q, s) + mm(scores, delta)
        to_end = np.exp(log_gamma[-1] - log_gamma).astype(dtype)  # gamma_C / gamma_j
        s = gamma[-1] * s + mm((K * to_end[:, None]).T, delta)
    return out, s
