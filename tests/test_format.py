"""Host-side formats: container header and manifest checks, layout, Q8_0 packing, the
synthetic checkpoint, and the exported C ABI.  No GPU is needed."""
import ctypes as C
import json
import re

import numpy as np
import pytest

import llmcp_b200 as L
import oracle

TINY = dict(hidden=64, intermediate=96, vocab=256, layers=4, full_interval=4, heads=4, kv_heads=2,
            head_dim=32, rotary=8, lin_k_heads=2, lin_v_heads=8, lin_k_dim=16, lin_v_dim=32, conv_kernel=4)


def tiny_dims(**changes):
    return L.default_dims().copy(**{**TINY, **changes})


def test_every_declared_symbol_is_exported():
    header = (L._PACKAGE.parent / "include" / "llmcp_b200.h").read_text()
    names = set(re.findall(r"\b(_mlir_ciface_\w+|llmcp_\w+)\s*\(", header))
    assert len(names) >= 30
    lib = L.lib()
    for name in sorted(names):
        assert hasattr(lib, name), f"{name} is declared in include/llmcp_b200.h but not exported"
    assert lib.llmcp_model_abi_version() == 2  # include/llmcp/Support/AotAbi.h:12


def test_compute_entries_fail_loudly_without_a_gpu():
    if L.device_count() > 0:
        pytest.skip("a CUDA device is present")
    x = np.zeros((1, 32), dtype=np.uint16)
    with pytest.raises(L.LlmcpError, match="no CUDA device"):
        L.ops.act_quant(x)
    with pytest.raises(L.LlmcpError, match="no CUDA device"):
        L.Engine(L.synthetic_container(tiny_dims(), 1), tiny_dims(), capacity=8)


def test_default_dims_are_the_reference_constants():
    d = L.default_dims()  # lib/Runtime/AotRuntime.cpp:41-43,81,85
    assert (d.full_layers, d.kv_heads, d.head_dim) == (8, 4, 256)
    assert (d.linear_layers, d.lin_v_heads, d.lin_k_dim, d.lin_v_dim) == (24, 32, 128, 128)
    assert (d.conv_kernel - 1, d.qkv_dim, d.rotary, d.vocab) == (3, 8192, 64, 248320)
    assert abs(d.rope_theta - 1e7) < 1 and abs(d.eps - 1e-6) < 1e-12


def test_f16_and_bf16_conversions_match_the_oracle():
    lib = L.lib()
    rng = np.random.default_rng(0)
    values = np.concatenate([
        rng.standard_normal(2000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 2000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e6, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                  6.1e-5, 6.0e-8, 1.0 / 127, 0.02 / 127], dtype=np.float32)])
    pack = np.zeros(8 * 32, dtype=np.float32)
    for v in values:
        # the product's converter is reached through the packer: scale = amax / 127
        pack[:] = 0
        pack[0] = v * np.float32(127)
        if not np.isfinite(pack[0]):
            continue
        mine = L.pack_q8_0_p4(pack.reshape(8, 32))
        want = oracle.lib().orc_f32_to_f16(C.c_float(np.float32(np.abs(pack[0])) / np.float32(127)))
        assert int(mine[0]) | (int(mine[1]) << 8) == want, v


def test_pack_matches_oracle_and_golden(golden):
    rng = np.random.default_rng(3)
    for rows, cols in ((8, 32), (16, 96), (136, 288)):
        w = (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32)
        w[0, :32] = 0
        assert np.array_equal(L.pack_q8_0_p4(w), oracle.pack_q8_0_p4(w))
    for case in ("linear_q8_p4_prefill_boundaries", "linear_q8_p4_decode_boundaries"):
        c = golden(case)
        assert np.array_equal(L.pack_q8_0_p4(oracle.bf16_to_f32(c["w"])), c["packed"])
    with pytest.raises(L.LlmcpError):
        L.pack_q8_0_p4(np.zeros((4, 32), dtype=np.float32))  # Q8PackedLayout.h:38-42
    with pytest.raises(L.LlmcpError):
        L.pack_q8_0_p4(np.zeros((8, 48), dtype=np.float32))


def test_quantization_byte_pins():
    """tests/unittests/QuantizationTest.cpp:57-89."""
    ones = L.pack_q8_0_p4(np.ones((8, 64), dtype=np.float32)).reshape(-1, 136)
    assert (ones[:, :8].reshape(-1, 2) == [0x08, 0x20]).all()
    assert (ones[:, 8:].view(np.int8) == 127).all()
    half = np.ones((8, 64), dtype=np.float32)
    half[:, 32:] = 0
    rec = L.pack_q8_0_p4(half).reshape(-1, 136)
    assert (rec[1::2, :8] == 0).all() and (rec[1::2, 8:] == 0).all()


def test_layout_matches_the_reference_rules():
    """lib/Model/WeightLayout.cpp:96-268 and tests/unittests/WeightLayoutTest.cpp."""
    d = L.default_dims()
    size = int(L.lib().llmcp_b200_synthetic_bytes(C.byref(d)))
    # Q8 arena of the real model: 4,469,519,936 bytes, 426 tensors (docs/int8-quantization.md:720-724)
    manifest_len = size - 4469519936
    assert 0 < manifest_len < 200000
    data = L.synthetic_container(tiny_dims(layers=8), 7)
    arena = L.Arena().from_buffer(data)
    m = arena.manifest
    assert m["header_bytes"] == 64 and m["alignment"] == 64 and m["quantization"] == "q8_0"
    assert m["block_size"] == 32 and m["quant_layout"] == "q8_0_p4" and m["num_groups"] == 2
    tensors = m["tensors"]
    assert tensors[0]["name"] == "model.language_model.embed_tokens.weight" and tensors[0]["offset"] == 64
    assert tensors[-1]["name"] == "model.language_model.norm.weight"
    for t in tensors:
        assert t["offset"] % 64 == 0
        two_d = len(t["shape"]) == 2
        assert (t["dtype"] == "Q8_0") == (two_d and t["shape"][0] % 8 == 0 and t["shape"][1] % 32 == 0)
    group0 = [t for t in tensors if ".layers.0." in t["name"]][0]["offset"]
    group1 = [t for t in tensors if ".layers.4." in t["name"]][0]["offset"]
    assert group1 - group0 == m["group_stride"]
    order = [t["name"].split("layers.0.")[1] for t in tensors if ".layers.0." in t["name"]]
    assert order == ["input_layernorm.weight", "post_attention_layernorm.weight", "linear_attn.in_proj_qkv.weight",
                     "linear_attn.in_proj_z.weight", "linear_attn.in_proj_a.weight", "linear_attn.in_proj_b.weight",
                     "linear_attn.conv1d.weight", "linear_attn.dt_bias", "linear_attn.A_log",
                     "linear_attn.norm.weight", "linear_attn.out_proj.weight", "mlp.gate_proj.weight",
                     "mlp.up_proj.weight", "mlp.down_proj.weight"]
    full = [t["name"].split("layers.3.")[1] for t in tensors if ".layers.3." in t["name"]]
    assert full[2:8] == ["self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                         "self_attn.o_proj.weight", "self_attn.q_norm.weight", "self_attn.k_norm.weight"]


def test_real_model_tensor_count():
    d = L.default_dims()
    layout_size = int(L.lib().llmcp_b200_synthetic_bytes(C.byref(d)))
    assert layout_size > 4469519936
    # 1 + 24 * 14 + 8 * 11 + 1 tensors
    assert 1 + 24 * 14 + 8 * 11 + 1 == 426


def test_synthetic_container_contents():
    dims = tiny_dims()
    data = L.synthetic_container(dims, 11)
    again = L.synthetic_container(dims, 11)
    other = L.synthetic_container(dims, 12)
    assert np.array_equal(data, again) and not np.array_equal(data, other)
    arena = L.Arena().from_buffer(data)
    t = arena.get("model.language_model.layers.0.mlp.gate_proj.weight")
    rows, cols = t["shape"]
    rec = data[t["offset"]:t["offset"] + t["size"]].reshape(-1, 136)
    scales = oracle.lib().orc_f16_to_f32
    d0 = scales(C.c_uint16(int(rec[0, 0]) | int(rec[0, 1]) << 8))
    assert 0.02 * 1.0 / 127 < d0 < 0.02 * 6.0 / 127  # amax of 32 draws of 0.02 N(0,1)
    q = rec[:, 8:].view(np.int8)
    assert np.abs(q).max() == 127 and abs(float(q.mean())) < 2.0
    norm = arena.get("model.language_model.layers.0.linear_attn.norm.weight")
    assert norm["dtype"] == "F32"
    assert (data[norm["offset"]:norm["offset"] + norm["size"]].view(np.float32) == 1.0).all()
    gain = arena.get("model.language_model.layers.0.input_layernorm.weight")
    assert gain["dtype"] == "BF16" and not data[gain["offset"]:gain["offset"] + gain["size"]].any()
    conv = arena.get("model.language_model.layers.0.linear_attn.conv1d.weight")
    cw = oracle.bf16_to_f32(data[conv["offset"]:conv["offset"] + conv["size"]].view(np.uint16))
    assert 0.3 < cw.std() < 0.7


def corrupt(data, mutate):
    broken = data.copy()
    mutate(broken)
    return broken


def test_container_corruption_matrix():
    """tests/unittests/PackedWeightsTest.cpp:97-134: every damaged container is rejected."""
    data = L.synthetic_container(tiny_dims(), 5)
    arena_bytes = int.from_bytes(data[16:24].tobytes(), "little")
    manifest = json.loads(data[arena_bytes:].tobytes())
    L.Arena().from_buffer(data)

    def with_manifest(change):
        m = json.loads(json.dumps(manifest))
        change(m)
        text = (json.dumps(m) + "\n").encode()
        out = np.concatenate([data[:arena_bytes], np.frombuffer(text, dtype=np.uint8)])
        out[32:40] = np.frombuffer(len(text).to_bytes(8, "little"), dtype=np.uint8)
        return out

    def set_(path, value):
        def change(m):
            node = m
            for key in path[:-1]:
                node = node[key]
            node[path[-1]] = value
        return change

    def drop(key):
        return lambda m: m.pop(key)

    bad = [
        corrupt(data, lambda b: b.__setitem__(0, ord("X"))),                       # magic
        corrupt(data, lambda b: b.__setitem__(8, 2)),                              # version
        corrupt(data, lambda b: b.__setitem__(12, 32)),                            # header size
        corrupt(data, lambda b: b.__setitem__(slice(16, 24), 0)),                  # arena bytes < header
        corrupt(data, lambda b: b.__setitem__(24, (int(b[24]) + 64) % 256)),       # manifest offset != arena bytes
        corrupt(data, lambda b: b.__setitem__(slice(32, 40), 0)),                  # empty manifest
        data[:-1],                                                                 # truncated manifest
        data[:40],                                                                 # too small
        with_manifest(set_(["total_bytes"], arena_bytes + 64)),
        with_manifest(set_(["header_bytes"], 128)),
        with_manifest(set_(["quantization"], "q4_0")),
        with_manifest(set_(["block_size"], 64)),
        with_manifest(set_(["quant_layout"], "q8_0")),
        with_manifest(set_(["tensors"], [])),
        with_manifest(set_(["tensors", 0, "offset"], 32)),
        with_manifest(set_(["tensors", 0, "offset"], 96 + 1)),
        with_manifest(set_(["tensors", 0, "size"], manifest["tensors"][0]["size"] + 34)),
        with_manifest(set_(["tensors", 1, "dtype"], "F16")),
        with_manifest(set_(["tensors", 1, "offset"], arena_bytes)),
        with_manifest(set_(["tensors", 1, "name"], manifest["tensors"][0]["name"])),
        with_manifest(set_(["tensors", 0, "shape"], [256, 48])),
        with_manifest(drop("tensors")),
    ]
    for index, broken in enumerate(bad):
        with pytest.raises(L.LlmcpError):
            L.Arena().from_buffer(broken)
        assert L.last_error(), index


def test_failed_reload_keeps_the_arena(tmp_path):
    """tests/unittests/PackedWeightsTest.cpp:72-95."""
    data = L.synthetic_container(tiny_dims(), 5)
    good = tmp_path / "weights.bin"
    good.write_bytes(data.tobytes())
    bad = tmp_path / "broken.bin"
    bad.write_bytes(b"LLMCPWGX" + data.tobytes()[8:])
    arena = L.Arena().load(good)
    names = set(arena.weights)
    with pytest.raises(L.LlmcpError):
        arena.load(bad)
    assert set(arena.weights) == names and arena.size == int.from_bytes(data[16:24].tobytes(), "little")


def test_cos_sin_matches_the_oracle():
    for pos in (0, 1, 1023, 8192):
        mine = L.make_cos_sin(pos)
        want = oracle.make_cos_sin([pos])
        assert np.array_equal(mine[0], want[0][0]) and np.array_equal(mine[1], want[1][0])
