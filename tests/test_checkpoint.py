"""The offline packer: config.json, safetensors headers, the arena layout of a checkpoint and
`llmcp-pack`.  The cases follow the reference's unit tests (tests/unittests/ModelConfigTest.cpp,
SafetensorsTest.cpp, WeightLayoutTest.cpp, PackedWeightsTest.cpp:136-236): a tiny checkpoint is
written to disk, packed, loaded back, and every tensor compared with its source (byte copy) or
with the oracle's Q8_0 packer (quantised tensors).  No GPU is needed."""
import json
import struct
import subprocess

import numpy as np
import pytest

import llmcp_b200 as L
import oracle

TINY = dict(hidden=64, intermediate=96, vocab=256, layers=4, full_interval=4, heads=4, kv_heads=2,
            head_dim=32, rotary=8, lin_k_heads=2, lin_v_heads=8, lin_k_dim=16, lin_v_dim=32, conv_kernel=4)


def tiny_config(**text_changes):
    text = {
        "attention_bias": False, "attn_output_gate": True, "head_dim": TINY["head_dim"], "hidden_act": "silu",
        "hidden_size": TINY["hidden"], "intermediate_size": TINY["intermediate"],
        "layer_types": ["linear_attention"] * 3 + ["full_attention"],
        "linear_conv_kernel_dim": 4, "linear_key_head_dim": TINY["lin_k_dim"],
        "linear_num_key_heads": TINY["lin_k_heads"], "linear_num_value_heads": TINY["lin_v_heads"],
        "linear_value_head_dim": TINY["lin_v_dim"], "max_position_embeddings": 4096,
        "num_attention_heads": TINY["heads"], "num_hidden_layers": TINY["layers"],
        "num_key_value_heads": TINY["kv_heads"], "rms_norm_eps": 1e-06,
        "rope_parameters": {"mrope_interleaved": True, "mrope_section": [2, 1, 1], "partial_rotary_factor": 0.25,
                            "rope_theta": 10000000, "rope_type": "default"},
        "tie_word_embeddings": True, "vocab_size": TINY["vocab"]}
    text.update(text_changes)
    return {"architectures": ["Qwen3_5ForConditionalGeneration"], "tie_word_embeddings": True, "text_config": text}


def expected_tensors():
    """(name, shape, dtype) in arena order for TINY (lib/Model/WeightLayout.cpp:134-266)."""
    h, inter = TINY["hidden"], TINY["intermediate"]
    qkv = 2 * TINY["lin_k_heads"] * TINY["lin_k_dim"] + TINY["lin_v_heads"] * TINY["lin_v_dim"]
    value = TINY["lin_v_heads"] * TINY["lin_v_dim"]
    out = [("model.language_model.embed_tokens.weight", (TINY["vocab"], h), "BF16")]
    for layer in range(TINY["layers"]):
        p = f"model.language_model.layers.{layer}."
        out += [(p + "input_layernorm.weight", (h,), "BF16"), (p + "post_attention_layernorm.weight", (h,), "BF16")]
        if layer % 4 != 3:
            out += [(p + "linear_attn.in_proj_qkv.weight", (qkv, h), "BF16"),
                    (p + "linear_attn.in_proj_z.weight", (value, h), "BF16"),
                    (p + "linear_attn.in_proj_a.weight", (TINY["lin_v_heads"], h), "BF16"),
                    (p + "linear_attn.in_proj_b.weight", (TINY["lin_v_heads"], h), "BF16"),
                    (p + "linear_attn.conv1d.weight", (qkv, 1, 4), "BF16"),
                    (p + "linear_attn.dt_bias", (TINY["lin_v_heads"],), "BF16"),
                    (p + "linear_attn.A_log", (TINY["lin_v_heads"],), "F32"),
                    (p + "linear_attn.norm.weight", (TINY["lin_v_dim"],), "F32"),
                    (p + "linear_attn.out_proj.weight", (h, value), "BF16")]
        else:
            q_out = TINY["heads"] * TINY["head_dim"] * 2
            kv = TINY["kv_heads"] * TINY["head_dim"]
            out += [(p + "self_attn.q_proj.weight", (q_out, h), "BF16"), (p + "self_attn.k_proj.weight", (kv, h), "BF16"),
                    (p + "self_attn.v_proj.weight", (kv, h), "BF16"),
                    (p + "self_attn.o_proj.weight", (h, TINY["heads"] * TINY["head_dim"]), "BF16"),
                    (p + "self_attn.q_norm.weight", (TINY["head_dim"],), "BF16"),
                    (p + "self_attn.k_norm.weight", (TINY["head_dim"],), "BF16")]
        out += [(p + "mlp.gate_proj.weight", (inter, h), "BF16"), (p + "mlp.up_proj.weight", (inter, h), "BF16"),
                (p + "mlp.down_proj.weight", (h, inter), "BF16")]
    out.append(("model.language_model.norm.weight", (h,), "BF16"))
    return out


def write_shard(path, tensors):
    """tensors: list of (name, dtype, shape, bytes).  Writes one safetensors file."""
    header, blob = {"__metadata__": {"format": "pt"}}, b""
    for name, dtype, shape, data in tensors:
        header[name] = {"dtype": dtype, "shape": list(shape), "data_offsets": [len(blob), len(blob) + len(data)]}
        blob += data
    text = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(text)) + text + blob)
    return 8 + len(text)


def write_checkpoint(directory, seed=7, shards=2, index=True, skip=None, reshape=None, config=None):
    """A random tiny checkpoint; returns {name: (dtype, shape, raw bytes)}."""
    rng = np.random.default_rng(seed)
    sources, per_shard = {}, [[] for _ in range(shards)]
    for i, (name, shape, dtype) in enumerate(expected_tensors()):
        if name == skip:
            continue
        if reshape and name == reshape[0]:
            shape = reshape[1]
        values = (rng.standard_normal(shape) * (0.02 if len(shape) == 2 else 1.0)).astype(np.float32)
        data = values.tobytes() if dtype == "F32" else oracle.f32_to_bf16(values).tobytes()
        sources[name] = (dtype, tuple(shape), data)
        per_shard[i % shards].append((name, dtype, shape, data))
    weight_map = {}
    for s, tensors in enumerate(per_shard):
        file = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        write_shard(directory / file, tensors)
        weight_map.update({t[0]: file for t in tensors})
    if index:
        (directory / "model.safetensors.index.json").write_text(
            json.dumps({"metadata": {"total_size": 0}, "weight_map": weight_map}))
    (directory / "config.json").write_text(json.dumps(config or tiny_config()))
    return sources


# ---- config.json -----------------------------------------------------------------------------

def test_config_gives_the_model_dimensions():
    d = L.parse_config(json.dumps(tiny_config()))
    for key, value in TINY.items():
        assert getattr(d, key) == value, key
    assert abs(d.eps - 1e-6) < 1e-12 and abs(d.rope_theta - 1e7) < 1
    # head_dim defaults to hidden / heads; the layer pattern to every fourth layer full
    text = tiny_config()["text_config"]
    del text["head_dim"], text["layer_types"]
    d = L.parse_config(json.dumps({"text_config": text}))
    assert d.head_dim == TINY["hidden"] // TINY["heads"] and d.full_interval == 4


@pytest.mark.parametrize("change, message", [
    ({"hidden_act": "gelu"}, "unsupported hidden_act 'gelu'"),
    ({"num_key_value_heads": 3}, "num_attention_heads must be divisible by num_key_value_heads"),
    ({"linear_num_key_heads": 3}, "linear_num_value_heads must be divisible by linear_num_key_heads"),
    ({"num_hidden_layers": 6, "layer_types": ["linear_attention"] * 6}, "unsupported layer pattern"),
    ({"layer_types": ["linear_attention"] * 3}, "layer_types has 3 entries, expected 4"),
    ({"layer_types": ["linear_attention"] * 3 + ["sliding"]}, "unknown layer type 'sliding'"),
    ({"rms_norm_eps": 0.0}, "rms_norm_eps must be positive"),
    ({"vocab_size": "many"}, "missing or invalid integer field 'vocab_size'"),
])
def test_config_errors(change, message):
    with pytest.raises(L.LlmcpError, match=message):
        L.parse_config(json.dumps(tiny_config(**change)))


def test_config_needs_text_config_and_a_tied_head():
    with pytest.raises(L.LlmcpError, match="'text_config' object"):
        L.parse_config("{}")
    config = tiny_config()
    config["tie_word_embeddings"] = False
    with pytest.raises(L.LlmcpError, match="untied lm_head"):
        L.parse_config(json.dumps(config))


# ---- safetensors headers ---------------------------------------------------------------------

def test_safetensors_header_offsets(tmp_path):  # SafetensorsTest.cpp:34-55
    start = write_shard(tmp_path / "a.safetensors", [("a", "BF16", (2, 3), bytes(12)), ("b", "F32", (1,), bytes(4))])
    tensors = L.read_safetensors(tmp_path / "a.safetensors")
    assert tensors == {"a": ("BF16", start, 12, (2, 3)), "b": ("F32", start + 12, 4, (1,))}


def raw_shard(path, header, data_bytes):
    text = json.dumps(header).encode()
    path.write_bytes(struct.pack("<Q", len(text)) + text + bytes(data_bytes))


@pytest.mark.parametrize("header, data_bytes, message", [
    ({"a": {"dtype": "BF16", "shape": [2, 3], "data_offsets": [0, 10]}}, 12, "data size does not match dtype and shape"),
    ({"a": {"dtype": "Q4", "shape": [2], "data_offsets": [0, 2]}}, 2, "unsupported safetensors dtype 'Q4'"),
    ({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}, 4, "extends past end of file"),
    ({"a": {"dtype": "F32", "shape": [2]}}, 8, "missing data_offsets"),
    ({"a": {"dtype": "F32", "shape": [-2], "data_offsets": [0, 8]}}, 8, "invalid shape"),
    ({"a": {"shape": [2], "data_offsets": [0, 8]}}, 8, "missing dtype"),
])
def test_safetensors_header_errors(tmp_path, header, data_bytes, message):  # SafetensorsTest.cpp:57-77
    raw_shard(tmp_path / "bad.safetensors", header, data_bytes)
    with pytest.raises(L.LlmcpError, match=message):
        L.read_safetensors(tmp_path / "bad.safetensors")


def test_safetensors_file_errors(tmp_path):
    (tmp_path / "short.safetensors").write_bytes(b"abc")
    with pytest.raises(L.LlmcpError, match="too small"):
        L.read_safetensors(tmp_path / "short.safetensors")
    (tmp_path / "huge.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(L.LlmcpError, match="invalid safetensors header size"):
        L.read_safetensors(tmp_path / "huge.safetensors")
    with pytest.raises(L.LlmcpError, match="cannot open"):
        L.read_safetensors(tmp_path / "absent.safetensors")


# ---- packing ---------------------------------------------------------------------------------

@pytest.mark.parametrize("quant", ["none", "q8_0"])
def test_pack_and_load_tiny_checkpoint(tmp_path, quant):  # PackedWeightsTest.cpp:136-236
    sources = write_checkpoint(tmp_path)
    out = tmp_path / f"{quant}.bin"
    tensors, source_bytes, arena_bytes = L.pack_checkpoint(tmp_path, out, quant=quant)
    assert tensors == len(sources) == 55  # the count WeightLayoutTest.cpp:135 expects for four layers
    assert source_bytes == sum(len(s[2]) for s in sources.values())
    assert not (tmp_path / f"{quant}.bin.json").exists()  # no sidecar: the manifest is embedded

    arena = L.Arena()
    arena.load(out)
    assert arena.size == arena_bytes and arena.size % 64 == 0
    assert arena.quantization == quant
    manifest = json.loads(bytes(arena.data[arena.size:]).decode())
    assert manifest["model"] == str(tmp_path) and manifest["num_groups"] == 1 and manifest["alignment"] == 64
    assert ("quant_layout" in manifest) == (quant == "q8_0")
    assert [t["name"] for t in manifest["tensors"]] == [t[0] for t in expected_tensors()]
    quantised = 0
    for entry in manifest["tensors"]:
        dtype, shape, data = sources[entry["name"]]
        got = bytes(arena.data[entry["offset"]:entry["offset"] + entry["size"]])
        assert entry["offset"] % 64 == 0 and entry["source_size"] == len(data) and tuple(entry["shape"]) == shape
        packable = len(shape) == 2 and shape[0] % 8 == 0 and shape[1] % 32 == 0
        if quant == "q8_0" and packable:
            quantised += 1
            assert entry["dtype"] == "Q8_0" and entry["size"] == shape[0] * (shape[1] // 32) * 34
            bits = np.frombuffer(data, dtype=np.uint16).reshape(shape)
            assert got == oracle.pack_q8_0_p4(bits, src_bf16=True).tobytes(), entry["name"]
        else:
            assert entry["dtype"] == dtype and got == data, entry["name"]
    assert quantised == (0 if quant == "none" else 32)  # embedding + 3 x 5 + 4 + 4 x 3 matrices


def test_packed_layout_equals_the_synthetic_layout(tmp_path):
    """The layout planned from checkpoint headers and the one the synthetic generator uses
    are the same function of the dimensions."""
    write_checkpoint(tmp_path)
    L.pack_checkpoint(tmp_path, tmp_path / "w.bin", quant="q8_0")
    arena = L.Arena()
    arena.load(tmp_path / "w.bin")
    packed = json.loads(bytes(arena.data[arena.size:]).decode())
    container = L.synthetic_container(L.default_dims().copy(**TINY), 1)
    reference = L.Arena()
    reference.from_buffer(container)
    synthetic = json.loads(bytes(reference.data[reference.size:]).decode())
    assert packed["total_bytes"] == synthetic["total_bytes"] and packed["group_stride"] == synthetic["group_stride"]
    key = lambda t: (t["name"], t["offset"], t["size"], t["dtype"], t["shape"], t["source_size"])
    assert [key(t) for t in packed["tensors"]] == [key(t) for t in synthetic["tensors"]]


def test_single_shard_without_index_and_f32_source(tmp_path):
    rng = np.random.default_rng(3)
    tensors, sources = [], {}
    for name, shape, dtype in expected_tensors():
        if name.endswith("mlp.down_proj.weight"):
            dtype = "F32"  # an f32 matrix is quantised from its f32 values
        values = (rng.standard_normal(shape) * 0.02).astype(np.float32)
        data = values.tobytes() if dtype == "F32" else oracle.f32_to_bf16(values).tobytes()
        tensors.append((name, dtype, shape, data))
        sources[name] = (dtype, values)
    write_shard(tmp_path / "model.safetensors", tensors)
    (tmp_path / "config.json").write_text(json.dumps(tiny_config()))
    L.pack_checkpoint(tmp_path, tmp_path / "w.bin", quant="q8_0")
    arena = L.Arena()
    arena.load(tmp_path / "w.bin")
    name = "model.language_model.layers.1.mlp.down_proj.weight"
    weight = arena.get(name)
    assert weight["dtype"] == "Q8_0" and weight["source_size"] == 64 * 96 * 4
    got = bytes(arena.data[weight["offset"]:weight["offset"] + weight["size"]])
    assert got == oracle.pack_q8_0_p4(sources[name][1]).tobytes()


def test_dry_run_writes_nothing(tmp_path):
    write_checkpoint(tmp_path)
    tensors, _, arena_bytes = L.pack_checkpoint(tmp_path, None, quant="q8_0", dry_run=True)
    assert tensors == 55 and arena_bytes > 64
    assert not list(tmp_path.glob("*.bin"))
    with pytest.raises(L.LlmcpError, match="output path is required"):
        L.pack_checkpoint(tmp_path, None, quant="q8_0")


def test_pack_rejects_a_bad_checkpoint(tmp_path):  # WeightLayoutTest.cpp:148-170
    name = "model.language_model.layers.2.linear_attn.in_proj_z.weight"
    (tmp_path / "missing").mkdir()
    write_checkpoint(tmp_path / "missing", skip=name)
    with pytest.raises(L.LlmcpError, match=f"missing tensor '{name}'"):
        L.pack_checkpoint(tmp_path / "missing", tmp_path / "w.bin", quant="q8_0")
    (tmp_path / "shape").mkdir()
    write_checkpoint(tmp_path / "shape", reshape=(name, (256, 32)))
    with pytest.raises(L.LlmcpError, match=f"tensor '{name}' dimension 1 is 32, expected 64"):
        L.pack_checkpoint(tmp_path / "shape", tmp_path / "w.bin", quant="q8_0")
    (tmp_path / "rank").mkdir()
    write_checkpoint(tmp_path / "rank", reshape=(name, (256 * 64,)))
    with pytest.raises(L.LlmcpError, match="has rank 1, expected 2"):
        L.pack_checkpoint(tmp_path / "rank", tmp_path / "w.bin", quant="q8_0")
    (tmp_path / "empty").mkdir()
    (tmp_path / "empty" / "config.json").write_text(json.dumps(tiny_config()))
    with pytest.raises(L.LlmcpError, match="no safetensors shards found"):
        L.pack_checkpoint(tmp_path / "empty", tmp_path / "w.bin", quant="q8_0")
    with pytest.raises(L.LlmcpError, match="unknown quantization mode 'q4_0'"):
        L.pack_checkpoint(tmp_path / "missing", tmp_path / "w.bin", quant="q4_0")
    assert not (tmp_path / "w.bin").exists()


def test_llmcp_pack_tool(tmp_path):  # tools/llmcp-pack/llmcp-pack.cpp:44-89
    tool = L._PACKAGE / "bin" / "llmcp-pack"
    if not tool.exists():
        pytest.skip("llmcp-pack has not been built")
    write_checkpoint(tmp_path, shards=1)
    out = tmp_path / "weights.bin"
    run = subprocess.run([str(tool), "--model", str(tmp_path), f"--out={out}", "--quant", "q8_0", "--verbose"],
                         capture_output=True, text=True)
    assert run.returncode == 0, run.stderr
    lines = run.stdout.strip().splitlines()
    assert len(lines) == 56 and lines[0].split()[0] == "64"  # the embedding table sits right behind the header
    assert lines[-1].startswith("packed 55 tensors, ") and lines[-1].endswith(f"quant q8_0 -> {out}")
    arena = L.Arena()
    arena.load(out)
    assert arena.quantization == "q8_0"
    run = subprocess.run([str(tool), "--model", str(tmp_path), "--dry-run"], capture_output=True, text=True)
    assert run.returncode == 0 and run.stdout.startswith("validated 55 tensors, ")
    run = subprocess.run([str(tool), "--model", str(tmp_path)], capture_output=True, text=True)
    assert run.returncode == 1 and "--out is required unless --dry-run is set" in run.stderr


def test_packed_synthetic_checkpoint_is_the_synthetic_container(tmp_path):
    """The random-init checkpoint written as safetensors, packed by llmcp-pack, is byte for byte
    the container the synthetic generator writes directly: both routes to a weights file agree."""
    dims = L.default_dims().copy(**TINY)
    L.synthetic_checkpoint(dims, 9, tmp_path)
    parsed = L.parse_config((tmp_path / "config.json").read_text())
    assert all(getattr(parsed, k) == v for k, v in TINY.items())
    assert abs(parsed.eps - dims.eps) < 1e-12 and parsed.rope_theta == dims.rope_theta
    headers = L.read_safetensors(tmp_path / "model.safetensors")
    assert len(headers) == 55 and headers["model.language_model.layers.0.linear_attn.A_log"][0] == "F32"
    out = tmp_path / "weights.bin"
    L.pack_checkpoint(tmp_path, out, quant="q8_0")
    packed = np.fromfile(out, dtype=np.uint8)
    direct = L.synthetic_container(dims, 9)
    arena_bytes = int.from_bytes(direct[16:24].tobytes(), "little")
    assert int.from_bytes(packed[16:24].tobytes(), "little") == arena_bytes
    assert np.array_equal(packed[64:arena_bytes], direct[64:arena_bytes])
    a, b = json.loads(packed[arena_bytes:].tobytes()), json.loads(direct[arena_bytes:].tobytes())
    assert a.pop("model") == str(tmp_path) and b.pop("model") == "synthetic"
    assert a == b
    # a different seed gives different weights
    other = L.synthetic_container(dims, 10)
    assert not np.array_equal(other[64:arena_bytes], direct[64:arena_bytes])
