"""ctypes binding of the CPU oracle (test infrastructure only).

The oracle restates the reference's arithmetic on the host; it is the checker
for the CUDA path.  Only the test-suite, the smoke check and the CPU-baseline
leg of the benchmark import this module.  Nothing in ``llmcp_b200`` does.
"""
import ctypes as C
import os
import pathlib
import subprocess

import numpy as np

_HERE = pathlib.Path(__file__).resolve().parent
_LIB = None

ACT = {"none": 0, "silu": 1, "sigmoid": 2, "softplus": 3}
# bf16 / bf16-pairs: an unquantised arena (bf16 matrices), portable lowering / the aarch64 lowering's order
MODE = {"fma": 0, "muladd": 1, "bf16": 2, "bf16-pairs": 3}


def build(force=False):
    """Compiles liboracle.so next to this file (needs g++)."""
    target = _HERE / "liboracle.so"
    source = _HERE / "oracle.cpp"
    if force or not target.exists() or target.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-B", "liboracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return target


def lib():
    global _LIB
    if _LIB is None:
        target = _HERE / "liboracle.so"
        if not target.exists():
            build()
        _LIB = C.CDLL(str(target))
        _LIB.orc_bf16_to_f32.restype = C.c_float
        _LIB.orc_bf16_to_f32.argtypes = [C.c_uint16]
        _LIB.orc_f32_to_bf16.restype = C.c_uint16
        _LIB.orc_f32_to_bf16.argtypes = [C.c_float]
        _LIB.orc_f32_to_f16.restype = C.c_uint16
        _LIB.orc_f32_to_f16.argtypes = [C.c_float]
        _LIB.orc_f16_to_f32.restype = C.c_float
        _LIB.orc_f16_to_f32.argtypes = [C.c_uint16]
        _LIB.orc_exp.restype = C.c_float
        _LIB.orc_exp.argtypes = [C.c_float]
        _LIB.orc_argmax.restype = C.c_int64
        _LIB.orc_model_create.restype = C.c_void_p
    return _LIB


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _i(v):
    return C.c_int64(int(v))


def bf16_to_f32(a):
    """uint16 bit patterns -> float32 values."""
    a = np.ascontiguousarray(a, dtype=np.uint16)
    return (a.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16(a):
    """float32 -> uint16 bit patterns, round to nearest even."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = a.view(np.uint32)
    rounded = b + 0x7FFF + ((b >> 16) & 1)
    return (rounded >> 16).astype(np.uint16)


def num_threads():
    return int(lib().orc_num_threads())


def set_num_threads(threads=None):
    """Use ``threads`` OpenMP threads (default: every core this process may run on) for the calls
    that follow, overriding an OMP_NUM_THREADS inherited from a launcher.  Returns the count."""
    if threads is None:
        threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    return int(lib().orc_set_num_threads(int(threads)))


def pack_q8_0_p4(w, src_bf16=False):
    """[rows, cols] f32 (or bf16 bits) -> packed q8_0_p4 bytes."""
    w = np.ascontiguousarray(w, dtype=np.uint16 if src_bf16 else np.float32)
    rows, cols = w.shape
    out = np.empty(rows * (cols // 32) * 34, dtype=np.uint8)
    rc = lib().orc_pack_q8_0_p4(_p(w), int(src_bf16), _i(rows), _i(cols), _p(out))
    if rc != 0:
        raise ValueError("packed Q8_0 needs rows % 8 == 0 and cols % 32 == 0")
    return out


def quantize_row_q8_0(values):
    values = np.ascontiguousarray(values, dtype=np.float32)
    cols = values.shape[0]
    d = np.empty(cols // 32, dtype=np.uint16)
    qs = np.empty(cols, dtype=np.int8)
    lib().orc_quantize_row_q8_0(_p(values), _i(cols), _p(d), _p(qs))
    return d, qs


def act_quant(x, x_bf16=True):
    x = np.ascontiguousarray(x, dtype=np.uint16 if x_bf16 else np.float32)
    M, K = x.shape
    q = np.empty((M, K), dtype=np.int8)
    s = np.empty((M, K // 32), dtype=np.float32)
    lib().orc_act_quant(_p(x), int(x_bf16), _i(M), _i(K), _p(q), _p(s))
    return q, s


def block_dots(aq, packed, N):
    aq = np.ascontiguousarray(aq, dtype=np.int8)
    M, K = aq.shape
    dots = np.empty((M, N, K // 32), dtype=np.int32)
    lib().orc_block_dots(_p(aq), _i(M), _i(K), _p(packed), _i(N), _p(dots))
    return dots


def linear_q8(x, packed, N, x_bf16=True, y_bf16=True, activation="none", mode="fma",
              direct=False):
    x = np.ascontiguousarray(x, dtype=np.uint16 if x_bf16 else np.float32)
    M, K = x.shape
    y = np.empty((M, N), dtype=np.uint16 if y_bf16 else np.float32)
    fn = lib().orc_linear_q8_direct if direct else lib().orc_linear_q8
    fn(_p(x), int(x_bf16), _i(M), _i(K), _p(packed), _i(N), _p(y), int(y_bf16),
       ACT[activation], MODE[mode])
    return y


def linear_bf16(x, w, x_bf16=True, y_bf16=True, activation="none"):
    """bf16 weights [N][K] (an unquantised arena): MatmulLoweringCommon.cpp:186-251, the portable lowering."""
    x = np.ascontiguousarray(x, dtype=np.uint16 if x_bf16 else np.float32)
    w = np.ascontiguousarray(w, dtype=np.uint16)
    M, K = x.shape
    N = w.shape[0]
    y = np.empty((M, N), dtype=np.uint16 if y_bf16 else np.float32)
    lib().orc_linear_bf16(_p(x), int(x_bf16), _i(M), _i(K), _p(w), _i(N), _p(y), int(y_bf16), ACT[activation])
    return y


def embedding_q8(tokens, packed, hidden):
    tokens = np.ascontiguousarray(tokens, dtype=np.int64)
    out = np.empty((tokens.shape[0], hidden), dtype=np.uint16)
    lib().orc_embedding_q8(_p(tokens), _i(tokens.shape[0]), _p(packed), _i(hidden), _p(out))
    return out


def rms_norm(x, w, eps=1e-6, zero_centered=True, w_bf16=True):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    w = np.ascontiguousarray(w, dtype=np.uint16 if w_bf16 else np.float32)
    M, H = x.shape
    y = np.empty_like(x)
    lib().orc_rms_norm(_p(x), _i(M), _i(H), _p(w), int(w_bf16), C.c_float(eps),
                       int(zero_centered), _p(y))
    return y


def pointwise(a, b, op):
    a = np.ascontiguousarray(a, dtype=np.uint16)
    b = np.ascontiguousarray(b, dtype=np.uint16)
    y = np.empty_like(a)
    lib().orc_pointwise(_p(a), _p(b), _i(a.size), {"add": 0, "mul": 1, "silu_mul": 2}[op], _p(y))
    return y


def gated_rms_norm(x, gate, w, group, eps=1e-6, gate_activated=False, w_bf16=False):
    x = np.ascontiguousarray(x, dtype=np.uint16)
    gate = np.ascontiguousarray(gate, dtype=np.uint16)
    w = np.ascontiguousarray(w, dtype=np.uint16 if w_bf16 else np.float32)
    M, H = x.shape
    y = np.empty_like(x)
    lib().orc_gated_rms_norm(_p(x), _p(gate), _p(w), int(w_bf16), _i(M), _i(H), _i(group),
                             C.c_float(eps), int(gate_activated), _p(y))
    return y


def causal_conv1d(x, w, state, kernel):
    """Returns (y, new_state); state is [kernel-1, C] bf16 bits (copied)."""
    x = np.ascontiguousarray(x, dtype=np.uint16)
    w = np.ascontiguousarray(w, dtype=np.uint16)
    state = np.array(state, dtype=np.uint16, copy=True)
    S, Cc = x.shape
    y = np.empty_like(x)
    lib().orc_causal_conv1d(_p(x), _p(w), _p(state), _i(S), _i(Cc), _i(kernel), _p(y))
    return y, state


def gated_delta_net(conv, a, b, a_log, dt_bias, state, nk, nv, dk, dv, b_activated=False):
    """Returns (out, new_state); state is [nv, dk, dv] f32 (copied)."""
    conv = np.ascontiguousarray(conv, dtype=np.uint16)
    a = np.ascontiguousarray(a, dtype=np.uint16)
    b = np.ascontiguousarray(b, dtype=np.uint16)
    a_log = np.ascontiguousarray(a_log, dtype=np.float32)
    dt_bias = np.ascontiguousarray(dt_bias, dtype=np.uint16)
    state = np.array(state, dtype=np.float32, copy=True)
    S = conv.shape[0]
    out = np.empty((S, nv * dv), dtype=np.uint16)
    lib().orc_gated_delta_net(_p(conv), _p(a), _p(b), _p(a_log), _p(dt_bias), _p(state), _i(S),
                              _i(nk), _i(nv), _i(dk), _i(dv), int(b_activated), _p(out))
    return out, state


def attention(qg, k, v, q_norm, k_norm, cos, sin, cache, position, nh, nkv, hd, rot):
    """cache: [2, nkv, cap, hd] bf16 bits (copied).  Returns (out, new_cache)."""
    qg = np.ascontiguousarray(qg, dtype=np.uint16)
    k = np.ascontiguousarray(k, dtype=np.uint16)
    v = np.ascontiguousarray(v, dtype=np.uint16)
    q_norm = np.ascontiguousarray(q_norm, dtype=np.uint16)
    k_norm = np.ascontiguousarray(k_norm, dtype=np.uint16)
    cos = np.ascontiguousarray(cos, dtype=np.float32)
    sin = np.ascontiguousarray(sin, dtype=np.float32)
    cache = np.array(cache, dtype=np.uint16, copy=True)
    S = qg.shape[0]
    cap = cache.shape[2]
    out = np.empty((S, nh * hd), dtype=np.uint16)
    lib().orc_attention(_p(qg), _p(k), _p(v), _p(q_norm), _p(k_norm), _p(cos), _p(sin),
                        _p(cache), _i(position), _i(S), _i(nh), _i(nkv), _i(hd), _i(rot),
                        _i(cap), _p(out))
    return out, cache


def make_cos_sin(positions, rotary=64, theta=1.0e7):
    positions = list(positions)
    cos = np.empty((len(positions), rotary), dtype=np.float32)
    sin = np.empty((len(positions), rotary), dtype=np.float32)
    for i, pos in enumerate(positions):
        lib().orc_make_cos_sin(_i(pos), _i(rotary), C.c_float(theta), _p(cos[i]), _p(sin[i]))
    return cos, sin


def argmax(values):
    values = np.ascontiguousarray(values, dtype=np.float32)
    return int(lib().orc_argmax(_p(values), _i(values.size)))


def top2_margin(logits):
    """Difference between the largest and the second largest logit of a row: a greedy token is
    only pinned by a comparison whose logit error stays below half of this."""
    row = np.asarray(logits, dtype=np.float32).ravel()
    top = np.partition(row, row.size - 2)[-2:]
    return float(top[1] - top[0])


class ModelConfig(C.Structure):
    _fields_ = [(n, C.c_int64) for n in (
        "hidden", "intermediate", "vocab", "layers", "full_interval", "heads", "kv_heads",
        "head_dim", "rotary", "lin_k_heads", "lin_v_heads", "lin_k_dim", "lin_v_dim",
        "conv_kernel")] + [("eps", C.c_float), ("mode", C.c_int32)]


class Layer(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in (
        "input_norm", "post_norm", "qkv", "z", "a", "b", "conv", "dt_bias", "a_log", "lin_norm",
        "out_proj", "q_proj", "k_proj", "v_proj", "o_proj", "q_norm", "k_norm", "gate", "up",
        "down")] + [(n, C.c_int32) for n in ("lin_norm_bf16", "dt_bias_bf16", "a_log_bf16", "pad")]


_LAYER_NAMES = {
    "input_norm": "input_layernorm.weight", "post_norm": "post_attention_layernorm.weight",
    "qkv": "linear_attn.in_proj_qkv.weight", "z": "linear_attn.in_proj_z.weight",
    "a": "linear_attn.in_proj_a.weight", "b": "linear_attn.in_proj_b.weight",
    "conv": "linear_attn.conv1d.weight", "dt_bias": "linear_attn.dt_bias",
    "a_log": "linear_attn.A_log", "lin_norm": "linear_attn.norm.weight",
    "out_proj": "linear_attn.out_proj.weight", "q_proj": "self_attn.q_proj.weight",
    "k_proj": "self_attn.k_proj.weight", "v_proj": "self_attn.v_proj.weight",
    "o_proj": "self_attn.o_proj.weight", "q_norm": "self_attn.q_norm.weight",
    "k_norm": "self_attn.k_norm.weight", "gate": "mlp.gate_proj.weight",
    "up": "mlp.up_proj.weight", "down": "mlp.down_proj.weight",
}


class Model:
    """Whole-model oracle over a packed arena held in a numpy uint8 array.

    ``manifest`` is the parsed JSON manifest of the arena (a dict); ``dims`` gives the
    head counts that tensor shapes alone do not determine.
    """

    def __init__(self, arena, manifest, dims, mode="fma", eps=1e-6):
        self.arena = arena
        tensors = {t["name"]: t for t in manifest["tensors"]}
        prefix = "model.language_model."
        embed = tensors[prefix + "embed_tokens.weight"]
        layers = 1 + max(int(n.split(".")[3]) for n in tensors if n.startswith(prefix + "layers."))
        cfg = ModelConfig()
        cfg.vocab, cfg.hidden = embed["shape"]
        cfg.layers = layers
        cfg.intermediate = tensors[prefix + "layers.0.mlp.gate_proj.weight"]["shape"][0]
        for key, value in dims.items():
            setattr(cfg, key, value)
        cfg.eps = eps
        cfg.mode = MODE[mode]
        self.cfg = cfg
        arr = (Layer * layers)()
        for i in range(layers):
            for field, suffix in _LAYER_NAMES.items():
                t = tensors.get(f"{prefix}layers.{i}.{suffix}")
                if t is None:
                    continue
                setattr(arr[i], field, t["offset"])
                if field in ("lin_norm", "dt_bias", "a_log"):
                    setattr(arr[i], field + "_bf16", int(t["dtype"] == "BF16"))
        self._layers = arr
        self.handle = C.c_void_p(lib().orc_model_create(
            C.byref(cfg), _p(arena), C.c_uint64(embed["offset"]),
            C.c_uint64(tensors[prefix + "norm.weight"]["offset"]), arr))
        n_full = layers // cfg.full_interval
        n_lin = layers - n_full
        self.n_full, self.n_lin = n_full, n_lin
        self.qkv_dim = 2 * cfg.lin_k_heads * cfg.lin_k_dim + cfg.lin_v_heads * cfg.lin_v_dim

    def new_state(self, capacity):
        c = self.cfg
        return {
            "cap": capacity,
            "kv": np.zeros((self.n_full, 2, c.kv_heads, capacity, c.head_dim), dtype=np.uint16),
            "delta": np.zeros((self.n_lin, c.lin_v_heads, c.lin_k_dim, c.lin_v_dim), dtype=np.float32),
            "conv": np.zeros((self.n_lin, c.conv_kernel - 1, self.qkv_dim), dtype=np.uint16),
        }

    def forward(self, state, tokens, position, theta=1.0e7, want_hidden=False, cos=None, sin=None):
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        S = tokens.shape[0]
        if cos is None:
            cos, sin = make_cos_sin(range(position, position + S), self.cfg.rotary, theta)
        cos = np.ascontiguousarray(cos, dtype=np.float32)
        sin = np.ascontiguousarray(sin, dtype=np.float32)
        logits = np.empty(self.cfg.vocab, dtype=np.float32)
        hidden = np.empty((S, self.cfg.hidden), dtype=np.uint16) if want_hidden else None
        lib().orc_model_forward(self.handle, _p(tokens), _i(S), _p(cos), _p(sin), _i(position),
                                _p(state["kv"]), _i(state["cap"]), _p(state["delta"]),
                                _p(state["conv"]), _p(logits),
                                _p(hidden) if want_hidden else None)
        return (logits, hidden) if want_hidden else logits

    def close(self):
        if self.handle:
            lib().orc_model_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
