"""Python binding of libllmcp_b200.so and a host-side mirror of llmcp's runtime classes.

``ops``       one function per llmcp dialect operator on numpy arrays (host in, host out);
``Arena``     the packed weight container (lib/Runtime/WeightArena.cpp);
``AotRuntime``  the loader that calls the AOT ABI v2 entry points with MLIR memref
              descriptors exactly as lib/Runtime/AotRuntime.cpp:68-120 does;
``Engine``    the additive device-resident interface.

Everything computes on the GPU through the shared library.  There is no CPU fallback: if the
library has not been built, or no CUDA device is present, calls raise.
"""
import ctypes as C
import json
import mmap
import os
import pathlib

import numpy as np

_PACKAGE = pathlib.Path(__file__).resolve().parent
LIBRARY_PATH = _PACKAGE / "libllmcp_b200.so"

DTYPE_F32, DTYPE_BF16 = 0, 1
ACTIVATIONS = {"none": 0, "silu": 1, "sigmoid": 2, "softplus": 3}

_lib = None


class LlmcpError(RuntimeError):
    pass


class Dims(C.Structure):
    """llmcp_b200_dims (include/llmcp_b200.h)."""
    _fields_ = [(n, C.c_int64) for n in (
        "hidden", "intermediate", "vocab", "layers", "full_interval", "heads", "kv_heads", "head_dim",
        "rotary", "lin_k_heads", "lin_v_heads", "lin_k_dim", "lin_v_dim", "conv_kernel")] + [
        ("eps", C.c_float), ("rope_theta", C.c_float)]

    def copy(self, **changes):
        out = Dims.from_buffer_copy(self)
        for key, value in changes.items():
            setattr(out, key, value)
        return out

    @property
    def qkv_dim(self):
        return 2 * self.lin_k_heads * self.lin_k_dim + self.lin_v_heads * self.lin_v_dim

    @property
    def full_layers(self):
        return self.layers // self.full_interval

    @property
    def linear_layers(self):
        return self.layers - self.full_layers


def lib():
    """Loads the shared library (built by ``python -m llmcp_b200.build``)."""
    global _lib
    if _lib is None:
        if not LIBRARY_PATH.exists():
            raise LlmcpError(f"{LIBRARY_PATH} is missing: run `python -m llmcp_b200.build` (needs nvcc)")
        handle = C.CDLL(str(LIBRARY_PATH))
        handle.llmcp_model_abi_version.restype = C.c_int32
        handle.llmcp_b200_last_error.restype = C.c_size_t
        handle.llmcp_b200_launch_count.restype = C.c_uint64
        handle.llmcp_b200_synthetic_bytes.restype = C.c_uint64
        handle.llmcp_b200_manifest.restype = C.c_uint64
        handle.llmcp_b200_read_safetensors.restype = C.c_uint64
        handle.llmcp_b200_engine_create.restype = C.c_void_p
        handle.llmcp_b200_engine_create_mode.restype = C.c_void_p
        handle.llmcp_b200_engine_create_tp.restype = C.c_void_p
        handle.llmcp_b200_engine_create_batch.restype = C.c_void_p
        handle.llmcp_b200_tp_create.restype = C.c_void_p
        handle.llmcp_b200_tp_slot_bytes.restype = C.c_uint64
        handle.llmcp_b200_vocab_create.restype = C.c_void_p
        handle.llmcp_b200_vocab_size.restype = C.c_int64
        handle.llmcp_b200_vocab_token_to_id.restype = C.c_int32
        handle.llmcp_b200_vocab_encode.restype = C.c_int64
        handle.llmcp_b200_pretokenize.restype = C.c_int64
        handle.llmcp_b200_regex_split.restype = C.c_int64
        handle.llmcp_b200_stream_create.restype = C.c_void_p
        for name in ("vocab_decode", "stream_append", "stream_finish", "chat_prompt", "normalize_nfc"):
            getattr(handle, "llmcp_b200_" + name).restype = C.c_uint64
        handle._mlir_ciface_llmcp_model_prefill.restype = None
        handle._mlir_ciface_llmcp_model_decode.restype = None
        _lib = handle
    return _lib


def last_error():
    buf = C.create_string_buffer(4096)
    lib().llmcp_b200_last_error(buf, C.c_size_t(len(buf)))
    return buf.value.decode(errors="replace")


def _check(code):
    if code != 0:
        raise LlmcpError(last_error() or f"llmcp_b200 call failed with code {code}")


def device_count():
    return int(lib().llmcp_b200_device_count())


def set_device(index):
    _check(lib().llmcp_b200_set_device(int(index)))


def launch_count():
    return int(lib().llmcp_b200_launch_count())


MODES = {"exact": 0, "fast": 1}


def set_mode(mode):
    """Arithmetic mode of engines created afterwards and of the host-pointer operators:
    ``"exact"`` (bit-identical to the reference's order of operations) or ``"fast"``
    (parallel-tree reductions; see llmcp_b200_set_mode in include/llmcp_b200.h)."""
    _check(lib().llmcp_b200_set_mode(MODES[mode] if isinstance(mode, str) else int(mode)))


def get_mode():
    return {v: k for k, v in MODES.items()}[int(lib().llmcp_b200_get_mode())]


def default_dims():
    d = Dims()
    lib().llmcp_b200_default_dims(C.byref(d))
    return d


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _i(v):
    return C.c_int64(int(v))


def _np_dtype(code):
    return np.uint16 if code == DTYPE_BF16 else np.float32


class ops:
    """The llmcp dialect operators (include/llmcp/Dialect/LLMCP/IR/LLMCPOps.td:19-179)."""

    @staticmethod
    def act_quant(x, x_bf16=True):
        x = np.ascontiguousarray(x, dtype=np.uint16 if x_bf16 else np.float32)
        M, K = x.shape
        q = np.empty((M, K), dtype=np.int8)
        s = np.empty((M, K // 32), dtype=np.float32)
        _check(lib().llmcp_op_act_quant(_p(x), int(x_bf16), _i(M), _i(K), _p(q), _p(s)))
        return q, s

    @staticmethod
    def linear_q8(x, packed, N, x_bf16=True, y_bf16=True, activation="none", want_dots=False):
        x = np.ascontiguousarray(x, dtype=np.uint16 if x_bf16 else np.float32)
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        M, K = x.shape
        if packed.size != N * (K // 32) * 34:
            raise LlmcpError("packed weight size does not match N * (K + K / 32 * 2)")  # LLMCPOps.cpp:46-70
        y = np.empty((M, N), dtype=np.uint16 if y_bf16 else np.float32)
        dots = np.empty((M, N, K // 32), dtype=np.int32) if want_dots else None
        _check(lib().llmcp_op_linear_q8(_p(x), int(x_bf16), _i(M), _i(K), _p(packed), _i(N), _p(y), int(y_bf16),
                                        ACTIVATIONS[activation], _p(dots)))
        return (y, dots) if want_dots else y

    @staticmethod
    def linear_bf16(x, w, y_bf16=True, activation="none"):
        """llmcp.linear on the bf16 matrix ``w`` [N, K] of an unquantised arena; ``x`` [M, K] bf16."""
        x = np.ascontiguousarray(x, dtype=np.uint16)
        w = np.ascontiguousarray(w, dtype=np.uint16)
        M, K = x.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise LlmcpError("the weight's second dimension must equal the input's")
        y = np.empty((M, N), dtype=np.uint16 if y_bf16 else np.float32)
        _check(lib().llmcp_op_linear_bf16(_p(x), _i(M), _i(K), _p(w), _i(N), _p(y), int(y_bf16), ACTIVATIONS[activation]))
        return y

    @staticmethod
    def lm_head_q8(hidden, packed, vocab):
        hidden = np.ascontiguousarray(hidden, dtype=np.uint16)
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        M, K = hidden.shape
        logits = np.empty((M, vocab), dtype=np.float32)
        argmax = np.empty(M, dtype=np.int64)
        _check(lib().llmcp_op_lm_head_q8(_p(hidden), _i(M), _i(K), _p(packed), _i(vocab), _p(logits), _p(argmax)))
        return logits, argmax

    @staticmethod
    def embedding_q8(tokens, packed, vocab, hidden):
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        packed = np.ascontiguousarray(packed, dtype=np.uint8)
        out = np.empty((tokens.shape[0], hidden), dtype=np.uint16)
        _check(lib().llmcp_op_embedding_q8(_p(tokens), _i(tokens.shape[0]), _p(packed), _i(vocab), _i(hidden), _p(out)))
        return out

    @staticmethod
    def rms_norm(x, w, eps=1e-6, zero_centered=True, w_bf16=True):
        x = np.ascontiguousarray(x, dtype=np.uint16)
        w = np.ascontiguousarray(w, dtype=np.uint16 if w_bf16 else np.float32)
        M, H = x.shape
        y = np.empty_like(x)
        _check(lib().llmcp_op_rms_norm(_p(x), _i(M), _i(H), _p(w), int(w_bf16), C.c_float(eps), int(zero_centered), _p(y)))
        return y

    @staticmethod
    def pointwise(a, b, op):
        a = np.ascontiguousarray(a, dtype=np.uint16)
        b = np.ascontiguousarray(b, dtype=np.uint16)
        y = np.empty_like(a)
        _check(lib().llmcp_op_pointwise(_p(a), _p(b), _i(a.size), {"add": 0, "mul": 1, "silu_mul": 2}[op], _p(y)))
        return y

    @staticmethod
    def gated_rms_norm(x, gate, w, group, eps=1e-6, gate_activated=False, w_bf16=False):
        x = np.ascontiguousarray(x, dtype=np.uint16)
        gate = np.ascontiguousarray(gate, dtype=np.uint16)
        w = np.ascontiguousarray(w, dtype=np.uint16 if w_bf16 else np.float32)
        M, H = x.shape
        y = np.empty_like(x)
        _check(lib().llmcp_op_gated_rms_norm(_p(x), _p(gate), _p(w), int(w_bf16), _i(M), _i(H), _i(group),
                                             C.c_float(eps), int(gate_activated), _p(y)))
        return y

    @staticmethod
    def causal_conv1d(x, w, state, kernel):
        x = np.ascontiguousarray(x, dtype=np.uint16)
        w = np.ascontiguousarray(w, dtype=np.uint16)
        state = np.array(state, dtype=np.uint16, copy=True)
        S, channels = x.shape
        y = np.empty_like(x)
        _check(lib().llmcp_op_causal_conv1d(_p(x), _p(w), _p(state), _i(S), _i(channels), _i(kernel), _p(y)))
        return y, state

    @staticmethod
    def gated_delta_net(conv, a, b, a_log, dt_bias, state, nk, nv, dk, dv, b_activated=False):
        conv = np.ascontiguousarray(conv, dtype=np.uint16)
        a = np.ascontiguousarray(a, dtype=np.uint16)
        b = np.ascontiguousarray(b, dtype=np.uint16)
        a_log = np.ascontiguousarray(a_log, dtype=np.float32)
        dt_bias = np.ascontiguousarray(dt_bias, dtype=np.uint16)
        state = np.array(state, dtype=np.float32, copy=True)
        S = conv.shape[0]
        out = np.empty((S, nv * dv), dtype=np.uint16)
        _check(lib().llmcp_op_gated_delta_net(_p(conv), _p(a), _p(b), _p(a_log), _p(dt_bias), _p(state), _i(S), _i(nk),
                                              _i(nv), _i(dk), _i(dv), int(b_activated), _p(out)))
        return out, state

    @staticmethod
    def attention(qg, k, v, q_norm, k_norm, cos, sin, cache, position, nh, nkv, hd, rot):
        qg = np.ascontiguousarray(qg, dtype=np.uint16)
        k = np.ascontiguousarray(k, dtype=np.uint16)
        v = np.ascontiguousarray(v, dtype=np.uint16)
        q_norm = np.ascontiguousarray(q_norm, dtype=np.uint16)
        k_norm = np.ascontiguousarray(k_norm, dtype=np.uint16)
        cos = np.ascontiguousarray(cos, dtype=np.float32)
        sin = np.ascontiguousarray(sin, dtype=np.float32)
        cache = np.array(cache, dtype=np.uint16, copy=True)
        S, cap = qg.shape[0], cache.shape[2]
        out = np.empty((S, nh * hd), dtype=np.uint16)
        _check(lib().llmcp_op_attention(_p(qg), _p(k), _p(v), _p(q_norm), _p(k_norm), _p(cos), _p(sin), _p(cache),
                                        _i(position), _i(S), _i(nh), _i(nkv), _i(hd), _i(rot), _i(cap), _p(out)))
        return out, cache


def pack_q8_0_p4(values):
    """lib/Model/Quantization.cpp:165-214 on an f32 matrix -> packed bytes."""
    values = np.ascontiguousarray(values, dtype=np.float32)
    rows, cols = values.shape
    out = np.empty(rows * (cols // 32) * 34 if cols % 32 == 0 else 0, dtype=np.uint8)
    _check(lib().llmcp_b200_pack_q8_0_p4(_p(values), _i(rows), _i(cols), _p(out)))
    return out


def synthetic_container(dims, seed):
    """A random-init, q8_0-packed container for ``dims`` as a numpy uint8 array."""
    size = int(lib().llmcp_b200_synthetic_bytes(C.byref(dims)))
    if size == 0:
        raise LlmcpError(last_error())
    data = np.empty(size, dtype=np.uint8)
    _check(lib().llmcp_b200_synthetic_fill(C.byref(dims), C.c_uint64(seed), _p(data), C.c_uint64(size)))
    return data


def parse_config(text):
    """Model dimensions from the text of a checkpoint's config.json (lib/Model/ModelConfig.cpp:78-283)."""
    raw = text.encode() if isinstance(text, str) else bytes(text)
    d = Dims()
    _check(lib().llmcp_b200_parse_config(raw, C.c_uint64(len(raw)), C.byref(d)))
    return d


def read_safetensors(path):
    """Header of one safetensors shard: ``{name: (dtype, absolute data offset, bytes, shape)}``
    (lib/Model/Safetensors.cpp:137-172).  No tensor data is read."""
    raw = os.fsencode(str(path))
    lib().llmcp_b200_clear_error()  # a length of 0 is an error only if one was recorded by this call
    size = int(lib().llmcp_b200_read_safetensors(raw, None, C.c_uint64(0)))
    if size == 0 and last_error():
        raise LlmcpError(last_error())
    buf = C.create_string_buffer(size + 1)
    lib().llmcp_b200_read_safetensors(raw, buf, C.c_uint64(size + 1))
    out = {}
    for line in buf.value.decode().splitlines():
        name, dtype, offset, nbytes, shape = line.split("\t")
        out[name] = (dtype, int(offset), int(nbytes), tuple(int(v) for v in shape.split(",") if v))
    return out


def synthetic_checkpoint(dims, seed, model_dir):
    """Writes a random-init checkpoint directory (config.json + safetensors) with the tensors of
    ``synthetic_container(dims, seed)`` before quantisation."""
    _check(lib().llmcp_b200_synthetic_checkpoint(C.byref(dims), C.c_uint64(seed), os.fsencode(str(model_dir))))


def pack_checkpoint(model_dir, output_path=None, quant="none", dry_run=False, verbose=False):
    """``llmcp-pack``: packs ``model_dir`` (config.json + safetensors) into the container file
    ``output_path`` (tools/llmcp-pack/llmcp-pack.cpp:44-89).  Returns
    ``(tensors, source_bytes, arena_bytes)``, the figures of the tool's summary line."""
    counters = [C.c_uint64(0) for _ in range(3)]
    _check(lib().llmcp_b200_pack_checkpoint(
        os.fsencode(str(model_dir)), os.fsencode(str(output_path)) if output_path else None, quant.encode(),
        int(bool(dry_run)), int(bool(verbose)), *[C.byref(c) for c in counters]))
    return tuple(int(c.value) for c in counters)


def _text_call(fn, *args):
    """Calls a C function that fills (out, capacity) and returns the full length; returns bytes."""
    size = int(fn(*args, None, C.c_uint64(0)))
    buf = C.create_string_buffer(size + 1)
    fn(*args, buf, C.c_uint64(size + 1))
    return buf.raw[:size]


class Vocab:
    """Text <-> token ids of a ByteLevel tokenizer: what llmcp-run gets from ``tokenizers::Tokenizer``
    (``Encode``, ``Decode``, ``TokenToId``; tools/llmcp-run/llmcp-run.cpp:635-690).  ``json`` is the text of a
    tokenizer.json or of a bare ``{"token": id}`` object."""

    def __init__(self, json):
        raw = json.encode() if isinstance(json, str) else bytes(json)
        self._handle = lib().llmcp_b200_vocab_create(raw, C.c_uint64(len(raw)))
        if not self._handle:
            raise LlmcpError(last_error())

    def __len__(self):
        return int(lib().llmcp_b200_vocab_size(C.c_void_p(self._handle)))

    def token_to_id(self, token):
        return int(lib().llmcp_b200_vocab_token_to_id(C.c_void_p(self._handle), token.encode()))

    def decode(self, ids):
        arr = (C.c_int32 * len(ids))(*ids)
        return _text_call(lib().llmcp_b200_vocab_decode, C.c_void_p(self._handle), arr, C.c_uint64(len(ids))).decode()

    def encode(self, text):
        """``Encode(text)`` of the same tokenizer (llmcp-run.cpp:641): byte-level BPE after the Qwen
        pre-tokenisation split; raises when the tokenizer.json describes anything else."""
        raw = text.encode() if isinstance(text, str) else bytes(text)
        capacity = len(raw) + 16  # a piece never yields more ids than it has bytes
        ids = (C.c_int32 * capacity)()
        n = int(lib().llmcp_b200_vocab_encode(C.c_void_p(self._handle), raw, C.c_uint64(len(raw)), ids, C.c_uint64(capacity)))
        if n < 0:
            raise LlmcpError(last_error())
        return list(ids[:n])

    def close(self):
        if self._handle:
            lib().llmcp_b200_vocab_destroy(C.c_void_p(self._handle))
            self._handle = None


def pretokenize(text):
    """The pieces the Qwen pre-tokenisation pattern cuts ``text`` into (the Split step in front of
    the byte-level BPE), as a list of strings."""
    raw = text.encode()
    ends = (C.c_int64 * (len(raw) + 1))()
    n = int(lib().llmcp_b200_pretokenize(raw, C.c_uint64(len(raw)), ends, C.c_uint64(len(raw) + 1)))
    cuts = [0] + list(ends[:n])
    return [raw[a:b].decode() for a, b in zip(cuts, cuts[1:])]


def regex_split(pattern, text, behavior="isolated", invert=False):
    """The pieces a ``Split`` pre-tokeniser with this pattern cuts ``text`` into (the library's own
    regular-expression matcher; raises for a pattern with a construct it does not restate)."""
    raw = text.encode()
    out = C.create_string_buffer(len(raw) + 1)
    lengths = (C.c_int64 * (len(raw) + 1))()
    n = int(lib().llmcp_b200_regex_split(pattern.encode(), raw, C.c_uint64(len(raw)), behavior.encode(), int(bool(invert)), out,
                                         C.c_uint64(len(raw) + 1), lengths, C.c_uint64(len(raw) + 1)))
    if n < 0:
        raise LlmcpError(last_error())
    pieces, at, data = [], 0, out.raw
    for size in lengths[:n]:
        pieces.append(data[at:at + size].decode())
        at += size
    return pieces


def normalize_nfc(text):
    """Unicode Normalization Form C, as the encoder applies it under an NFC tokenizer."""
    raw = text.encode()
    out = C.create_string_buffer(3 * len(raw) + 16)  # NFC never grows a UTF-8 text threefold
    n = int(lib().llmcp_b200_normalize_nfc(raw, C.c_uint64(len(raw)), out, C.c_uint64(len(out))))
    return out.raw[:n].decode()


class StreamingDecoder:
    """``ByteLevelStreamingDecoder`` of tools/llmcp-run/StreamingDecoder.h: ``append`` returns a
    complete chunk or "" while a character's bytes are incomplete; ``finish`` emits the rest."""

    def __init__(self, vocab):
        self._vocab = vocab  # must outlive the stream
        self._handle = lib().llmcp_b200_stream_create(C.c_void_p(vocab._handle))

    def _once(self, fn, *args):
        # these calls consume the pending ids, so they are made once, with a buffer no chunk outgrows
        buf = C.create_string_buffer(1 << 16)
        size = int(fn(C.c_void_p(self._handle), *args, buf, C.c_uint64(len(buf))))
        if size >= len(buf):
            raise LlmcpError("a streamed chunk longer than 64 KiB was cut")
        return buf.raw[:size].decode()

    def append(self, token):
        return self._once(lib().llmcp_b200_stream_append, C.c_int32(token))

    def finish(self):
        return self._once(lib().llmcp_b200_stream_finish)

    def close(self):
        if self._handle:
            lib().llmcp_b200_stream_destroy(C.c_void_p(self._handle))
            self._handle = None


def chat_prompt(user, system="", thinking=True):
    """``makeChatPrompt`` of tools/llmcp-run/llmcp-run.cpp:608-624."""
    return _text_call(lib().llmcp_b200_chat_prompt, user.encode(), system.encode(), int(bool(thinking))).decode()


class Arena:
    """The packed weight container: header, arena, JSON manifest (lib/Runtime/WeightArena.cpp:27-129).

    ``load`` maps a file, ``from_buffer`` adopts a numpy uint8 array.  A failed load leaves
    the previously loaded contents in place.
    """

    def __init__(self):
        self.data = None
        self.size = 0
        self.quantization = "none"
        self.manifest = None
        self.weights = {}
        self._map = None

    def _adopt(self, data, keep):
        _check(lib().llmcp_b200_validate(_p(data), C.c_uint64(data.size)))
        length = int(lib().llmcp_b200_manifest(_p(data), C.c_uint64(data.size), None, C.c_uint64(0)))
        arena_bytes = int.from_bytes(data[16:24].tobytes(), "little")
        manifest = json.loads(data[arena_bytes:arena_bytes + length].tobytes().decode())
        self.data, self.size, self._map = data, arena_bytes, keep
        self.manifest = manifest
        self.quantization = manifest["quantization"]
        self.weights = {t["name"]: t for t in manifest["tensors"]}

    def load(self, path):
        with open(path, "rb") as f:
            mapped = mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ)
        data = np.frombuffer(mapped, dtype=np.uint8)
        if data.size < 64:
            raise LlmcpError("packed weights file is too small")
        self._adopt(data, mapped)
        return self

    def from_buffer(self, data):
        self._adopt(np.ascontiguousarray(data, dtype=np.uint8), None)
        return self

    def get(self, name):
        return self.weights[name]


def _memref(rank):
    class MemRef(C.Structure):
        _fields_ = [("base", C.c_void_p), ("data", C.c_void_p), ("offset", C.c_int64),
                    ("sizes", C.c_int64 * rank), ("strides", C.c_int64 * rank)]
    return MemRef


_MemRef1, _MemRef2, _MemRef3, _MemRef4, _MemRef5 = (_memref(r) for r in (1, 2, 3, 4, 5))


def _descriptor(cls, array, sizes=None):
    sizes = list(array.shape if sizes is None else sizes)
    strides = [1] * len(sizes)
    for i in range(len(sizes) - 2, -1, -1):
        strides[i] = strides[i + 1] * sizes[i + 1]
    d = cls()
    d.base = d.data = array.ctypes.data
    d.offset = 0
    for i, (size, stride) in enumerate(zip(sizes, strides)):
        d.sizes[i] = size
        d.strides[i] = stride
    return d


def make_cos_sin(position, rotary=64, theta=1.0e7):
    """lib/Runtime/AotRuntime.cpp:22-32 (computed by the library's C++ host code, in f32)."""
    cos = np.empty(rotary, dtype=np.float32)
    sin = np.empty(rotary, dtype=np.float32)
    lib().llmcp_b200_make_cos_sin(_i(position), _i(rotary), C.c_float(theta), _p(cos), _p(sin))
    return cos, sin


class AotRuntime:
    """Mirror of mlir::llmcp::runtime::AotRuntime (lib/Runtime/AotRuntime.cpp:39-120).

    ``init`` loads a shared library that exports the AOT ABI v2 symbols and allocates the
    host state buffers; ``forward`` marshals memref descriptors and calls the prefill entry
    for more than one token, else the decode entry.  ``dims`` defaults to the constants the
    reference hard-codes for Qwen3.5-4B.
    """

    def __init__(self, dims=None):
        self.dims = dims or default_dims()
        self.handle = None
        self.capacity = 0

    def init(self, path=None, max_sequence=0, cos_sin=None):
        d = self.dims
        self.capacity = int(max_sequence)
        self.kv = np.zeros((d.full_layers, 2, d.kv_heads, self.capacity, d.head_dim), dtype=np.uint16)
        self.delta = np.zeros((d.linear_layers, d.lin_v_heads, d.lin_k_dim, d.lin_v_dim), dtype=np.float32)
        self.conv = np.zeros((d.linear_layers, d.conv_kernel - 1, d.qkv_dim), dtype=np.uint16)
        self._cos_sin = cos_sin or (lambda pos: make_cos_sin(pos, d.rotary, d.rope_theta))
        for cached in ("_fixed", "_one", "_out"):  # descriptors of the buffers just replaced
            self.__dict__.pop(cached, None)
        try:
            self.handle = C.CDLL(str(path or LIBRARY_PATH))
            version = self.handle.llmcp_model_abi_version
            version.restype = C.c_int32
            if version() != 2:
                return False
            self._prefill = self.handle._mlir_ciface_llmcp_model_prefill
            self._decode = self.handle._mlir_ciface_llmcp_model_decode
        except (OSError, AttributeError):
            return False
        for fn in (self._prefill, self._decode):
            fn.restype = None
            fn.argtypes = [C.c_void_p] * 10
        return True

    def forward(self, arena, tokens, start_pos, cache_length, logits=None):
        """One call of the prefill (more than one token) or decode entry.  Returns the logits
        row, or None when the sequence does not fit (AotRuntime.cpp:72-74).

        ``logits`` may be a caller-owned float32 array of ``vocab`` elements that is written
        and returned, the way the reference's drivers pass one vector to every call
        (llmcp-benchmark.cpp:84-101); without it a fresh array is returned.  The descriptors of
        the buffers that do not change between calls (arena, kv, delta, conv) and the
        one-token input buffers are built once and kept.
        """
        d = self.dims
        sequence = len(tokens)
        if sequence == 0 or start_pos < 0 or start_pos > self.capacity or sequence > self.capacity - start_pos:
            return None
        if logits is None:
            logits = np.empty(d.vocab, dtype=np.float32)  # the entry writes every element
        elif logits.dtype != np.float32 or logits.size != d.vocab or not logits.flags.c_contiguous:
            raise LlmcpError("logits must be a contiguous float32 array of vocab elements")
        fixed = self.__dict__.get("_fixed")
        if fixed is None or fixed[0] is not arena.data:
            fixed = (arena.data, _descriptor(_MemRef1, arena.data, sizes=[arena.size]), _descriptor(_MemRef5, self.kv),
                     _descriptor(_MemRef4, self.delta), _descriptor(_MemRef3, self.conv))
            self._fixed = fixed
        _, ra, rk, rd, rv = fixed
        if sequence == 1:
            one = self.__dict__.get("_one")
            if one is None:
                token_data = np.empty(1, dtype=np.int64)
                cos = np.empty((1, d.rotary), dtype=np.float32)
                sin = np.empty((1, d.rotary), dtype=np.float32)
                one = self._one = (token_data, cos, sin, _descriptor(_MemRef1, token_data),
                                   _descriptor(_MemRef2, cos), _descriptor(_MemRef2, sin))
            token_data, cos, sin, rt, rc, rs = one
            token_data[0] = tokens[0]
            cos[0], sin[0] = self._cos_sin(start_pos)
        else:
            token_data = np.ascontiguousarray(tokens, dtype=np.int64)
            cos = np.empty((sequence, d.rotary), dtype=np.float32)
            sin = np.empty((sequence, d.rotary), dtype=np.float32)
            for t in range(sequence):
                cos[t], sin[t] = self._cos_sin(start_pos + t)
            rt = _descriptor(_MemRef1, token_data)
            rc = _descriptor(_MemRef2, cos)
            rs = _descriptor(_MemRef2, sin)
        out = self.__dict__.get("_out")
        if out is None or out[0] is not logits:
            out = self._out = (logits, _descriptor(_MemRef2, logits, sizes=[1, d.vocab]))
        fn = self._prefill if sequence > 1 else self._decode
        fn(C.addressof(rt), C.addressof(rc), C.addressof(rs), C.c_void_p(start_pos), C.c_void_p(cache_length),
           C.addressof(ra), C.addressof(rk), C.addressof(rd), C.addressof(rv), C.addressof(out[1]))
        return logits


class Engine:
    """Device-resident executor (llmcp_b200_engine_* in include/llmcp_b200.h)."""

    def __init__(self, container, dims=None, capacity=1160, device=0, mode=None, tp=None, max_tokens=1024, batch=1):
        """``tp``: a ``parallel.TensorParallel`` group; the engine then holds this rank's share of
        the model and every rank has to make the same calls (see llmcp_b200_engine_create_tp).
        ``batch``: number of independent sequences with state of their own (``select_sequence``,
        ``decode_batch``, ``generate_batch``)."""
        self.dims = dims or default_dims()
        self.container = np.ascontiguousarray(container, dtype=np.uint8)
        self.capacity = capacity
        self.tp = tp
        self.batch = int(batch)
        if self.batch > 1:
            mode_code = get_mode() if mode is None else mode
            self.handle = lib().llmcp_b200_engine_create_batch(
                _p(self.container), C.c_uint64(self.container.size), C.byref(self.dims), _i(capacity), int(device),
                MODES[mode_code] if isinstance(mode_code, str) else int(mode_code), self.batch)
        elif tp is not None:
            mode_code = get_mode() if mode is None else mode
            self.handle = lib().llmcp_b200_engine_create_tp(
                _p(self.container), C.c_uint64(self.container.size), C.byref(self.dims), _i(capacity), int(device),
                MODES[mode_code] if isinstance(mode_code, str) else int(mode_code), tp.handle, _i(max_tokens))
        elif mode is None:
            self.handle = lib().llmcp_b200_engine_create(_p(self.container), C.c_uint64(self.container.size),
                                                         C.byref(self.dims), _i(capacity), int(device))
        else:
            self.handle = lib().llmcp_b200_engine_create_mode(
                _p(self.container), C.c_uint64(self.container.size), C.byref(self.dims), _i(capacity), int(device),
                MODES[mode] if isinstance(mode, str) else int(mode))
        if not self.handle:
            raise LlmcpError(last_error())
        self.handle = C.c_void_p(self.handle)

    def reset(self):
        _check(lib().llmcp_b200_engine_reset(self.handle))

    def forward(self, tokens, position, want_logits=True):
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        logits = np.empty(self.dims.vocab, dtype=np.float32) if want_logits else None
        argmax = C.c_int64(-1)
        _check(lib().llmcp_b200_engine_forward(self.handle, _p(tokens), _i(tokens.shape[0]), _i(position),
                                               _p(logits), C.byref(argmax)))
        return logits, int(argmax.value)

    def forward_all(self, tokens, position):
        """Logits of every position, ``[len(tokens), vocab]`` float32 (llmcp_b200_engine_forward_all)."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        logits = np.empty((tokens.shape[0], self.dims.vocab), dtype=np.float32)
        _check(lib().llmcp_b200_engine_forward_all(self.handle, _p(tokens), _i(tokens.shape[0]), _i(position),
                                                   _p(logits)))
        return logits

    def select_sequence(self, sequence):
        """The sequence of the batch that forward / generate / read_state address from now on."""
        _check(lib().llmcp_b200_engine_select_sequence(self.handle, int(sequence)))

    def decode_batch(self, tokens, position, want_logits=True):
        """One token of every sequence at a common position: (logits [batch, vocab] or None, argmax [batch])."""
        tokens = np.ascontiguousarray(tokens, dtype=np.int64)
        assert tokens.shape == (self.batch,)
        logits = np.empty((self.batch, self.dims.vocab), dtype=np.float32) if want_logits else None
        argmax = np.empty(self.batch, dtype=np.int64)
        _check(lib().llmcp_b200_engine_decode_batch(self.handle, _p(tokens), _i(position), _p(logits), _p(argmax)))
        return logits, argmax

    def generate_batch(self, first_tokens, position, steps):
        """Greedy decoding of all sequences on the device: (tokens [steps, batch], milliseconds)."""
        first_tokens = np.ascontiguousarray(first_tokens, dtype=np.int64)
        assert first_tokens.shape == (self.batch,)
        out = np.empty((steps, self.batch), dtype=np.int64)
        ms = C.c_float(0)
        _check(lib().llmcp_b200_engine_generate_batch(self.handle, _p(first_tokens), _i(position), _i(steps), _p(out),
                                                      C.byref(ms)))
        return out, float(ms.value)

    def generate(self, first_token, position, steps):
        out = np.empty(steps, dtype=np.int64)
        ms = C.c_float(0)
        _check(lib().llmcp_b200_engine_generate(self.handle, _i(first_token), _i(position), _i(steps), _p(out),
                                                C.byref(ms)))
        return out, float(ms.value)

    def local_dims(self):
        """(dims of this rank's share, its first KV head): head counts divided by the group size."""
        d = Dims()
        first = C.c_int64(0)
        _check(lib().llmcp_b200_engine_local_dims(self.handle, C.byref(d), C.byref(first)))
        return d, int(first.value)

    def read_state(self):
        """The state buffers in the reference's layouts; under tensor parallelism this rank's heads."""
        d = self.local_dims()[0] if self.tp is not None else self.dims
        kv = np.empty((d.full_layers, 2, d.kv_heads, self.capacity, d.head_dim), dtype=np.uint16)
        delta = np.empty((d.linear_layers, d.lin_v_heads, d.lin_k_dim, d.lin_v_dim), dtype=np.float32)
        conv = np.empty((d.linear_layers, d.conv_kernel - 1, d.qkv_dim), dtype=np.uint16)
        _check(lib().llmcp_b200_engine_read_state(self.handle, _p(kv), _p(delta), _p(conv)))
        return {"kv": kv, "delta": delta, "conv": conv}

    def read_hidden(self):
        out = np.empty(self.dims.hidden, dtype=np.uint16)
        _check(lib().llmcp_b200_engine_read_hidden(self.handle, _p(out)))
        return out

    def close(self):
        if self.handle:
            lib().llmcp_b200_engine_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
