"""Token ids -> text of the llmcp-run driver: ByteLevel decoding, the streaming decoder and the chat
template.  The cases are those of the reference's tests/unittests/StreamingDecoderTest.cpp (same
vocabulary construction, same id sequences and expectations); the HuggingFace `tokenizers` package,
which the reference's tokenizer dependency wraps, is the independent check where it is installed.
Host-only: no GPU."""
import json
import subprocess

import numpy as np
import pytest

import llmcp_b200 as L


def byte_alphabet():
    """GPT-2 byte alphabet (StreamingDecoderTest.cpp:20-37)."""
    out, nxt = [], 256
    for byte in range(256):
        direct = 33 <= byte <= 126 or 161 <= byte <= 172 or byte >= 174
        out.append(chr(byte if direct else nxt))
        nxt += 0 if direct else 1
    return out


def make_vocab():
    """StreamingDecoderTest.cpp:39-53: the 256 bytes, three tokens that mix complete text with a
    partial next character, and a bracketed token."""
    a = byte_alphabet()
    vocab = {a[b]: b for b in range(256)}
    vocab["A" + a[0xE4]] = 256
    vocab[a[0xB8] + a[0xAD] + "B" + a[0xF0]] = 257
    vocab[a[0x9F] + a[0x98] + a[0x80]] = 258
    vocab["<|test|>"] = 259
    return vocab


@pytest.fixture(scope="module")
def vocab():
    v = L.Vocab(json.dumps(make_vocab(), ensure_ascii=True))  # \\uXXXX escapes exercise the reader
    yield v
    v.close()


def hf_tokenizer():
    tokenizers = pytest.importorskip("tokenizers")
    tok = tokenizers.Tokenizer(tokenizers.models.BPE(vocab=make_vocab(), merges=[]))
    tok.pre_tokenizer = tokenizers.pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)
    tok.decoder = tokenizers.decoders.ByteLevel()
    return tok


def stream(vocab, ids):
    decoder = L.StreamingDecoder(vocab)
    text = ""
    for i in ids:
        text += decoder.append(i)  # .decode() inside raises on a chunk that is not UTF-8
    text += decoder.finish()
    assert decoder.finish() == ""
    decoder.close()
    return text


def test_emits_ascii_immediately_and_buffers_split_characters(vocab):
    d = L.StreamingDecoder(vocab)
    assert d.append(ord("A")) == "A"
    assert d.append(0xE4) == "" and d.append(0xB8) == ""
    assert d.append(0xAD) == "中"
    assert d.append(0xF0) == "" and d.append(0x9F) == "" and d.append(0x98) == ""
    assert d.append(0x80) == "😀"
    assert d.append(ord("B")) == "B"
    assert d.finish() == ""
    d.close()


def test_matches_full_decode_at_every_token_limit(vocab):
    for text in ["中文你好，世界！", "🙂🚀🧑‍💻", "é\n A 中 😀 B", "literal � replacement", "ASCII\n\t text"]:
        ids = list(text.encode())  # with no merges every byte is its own token
        assert vocab.decode(ids) == text
        for count in range(len(ids) + 1):
            prefix = ids[:count]
            assert stream(vocab, prefix) == vocab.decode(prefix)
            assert vocab.decode(prefix) == bytes(prefix).decode("utf-8", errors="replace")


def test_mixed_tokens_and_bracketed_text(vocab):
    ids = [256, 257, 258, 259]
    assert stream(vocab, ids) == "A中B😀<|test|>" == vocab.decode(ids)
    assert vocab.token_to_id("<|test|>") == 259 and vocab.token_to_id("<|absent|>") == -1
    assert len(vocab) == 260
    assert vocab.decode([5, 100000, -3, 65]) == "\x05A"  # ids without a token are skipped


def test_preserves_invalid_bytes_and_final_partial_characters(vocab):
    """StreamingDecoderTest.cpp:104-115: 128 random 32-byte sequences (std::mt19937(0) % 256)."""
    raw = np.random.RandomState(0)._bit_generator.random_raw(128 * 32)
    assert int(raw[0]) == 2357136044  # first output of mt19937 seeded with 0
    trials = (raw % 256).astype(int).reshape(128, 32)
    tok = None
    try:
        tok = hf_tokenizer()
    except pytest.skip.Exception:
        pass
    for ids in trials.tolist():
        full = vocab.decode(ids)
        assert stream(vocab, ids) == full
        assert full == bytes(ids).decode("utf-8", errors="replace")
        if tok is not None:
            assert full == tok.decode(ids, skip_special_tokens=False)


def test_against_the_tokenizers_package():
    """Decode of the package the reference's dependency wraps, on mixed tokens, on every prefix."""
    tok = hf_tokenizer()
    v = L.Vocab(json.dumps(make_vocab(), ensure_ascii=False))
    rng = np.random.default_rng(3)
    for _ in range(200):
        ids = rng.integers(0, 260, size=int(rng.integers(1, 24))).tolist()
        assert v.decode(ids) == tok.decode(ids, skip_special_tokens=False), ids
    v.close()


def test_tokenizer_json_with_added_tokens(tmp_path):
    """A tokenizer.json: model.vocab, added_tokens (the end-of-turn token the driver stops at), ByteLevel decoder."""
    a = byte_alphabet()
    blob = {"model": {"type": "BPE", "vocab": {a[b]: b for b in range(256)}, "merges": []},
            "added_tokens": [{"id": 256, "content": "<|im_start|>", "special": True},
                             {"id": 257, "content": "<|im_end|>", "special": True}],
            "decoder": {"type": "ByteLevel"}}
    v = L.Vocab(json.dumps(blob))
    assert v.token_to_id("<|im_end|>") == 257 and len(v) == 258
    assert v.decode([256] + list("hé".encode()) + [257]) == "<|im_start|>hé<|im_end|>"
    v.close()
    blob["decoder"] = {"type": "WordPiece"}
    with pytest.raises(L.LlmcpError, match="ByteLevel"):
        L.Vocab(json.dumps(blob))
    with pytest.raises(L.LlmcpError):
        L.Vocab("[1, 2]")


def test_chat_prompt():
    """llmcp-run.cpp:608-624."""
    assert L.chat_prompt("Hi") == "<|im_start|>user\nHi<|im_end|>\n<|im_start|>assistant\n<think>\n"
    assert L.chat_prompt("Hi", thinking=False).endswith("<|im_start|>assistant\n<think>\n\n</think>\n\n")
    assert L.chat_prompt("Hi", system="Be brief").startswith("<|im_start|>system\nBe brief<|im_end|>\n<|im_start|>user\nHi")


def test_llmcp_run_prompt_only_paths():
    tool = L._PACKAGE / "bin" / "llmcp-run"
    assert tool.exists(), "run python -m llmcp_b200.build"
    run = subprocess.run([str(tool), "--text", "Hello", "--chat", "--no-thinking", "--print-prompt"], capture_output=True, text=True)
    assert run.returncode == 0 and run.stdout == L.chat_prompt("Hello", thinking=False)
    run = subprocess.run([str(tool), "--text", "Hello", "--aot", "x.so"], capture_output=True, text=True)
    assert run.returncode == 1 and "--token-ids" in run.stderr
    run = subprocess.run([str(tool), "--tokens", "5"], capture_output=True, text=True)
    assert run.returncode == 1 and "--aot" in run.stderr
