"""Text <-> token ids of the llmcp-run driver: ByteLevel decoding, the streaming decoder, the chat
template, and the byte-level BPE encoder behind --text.  The cases are those of the reference's tests/unittests/StreamingDecoderTest.cpp (same
vocabulary construction, same id sequences and expectations); the HuggingFace `tokenizers` package,
which the reference's tokenizer dependency wraps, is the independent check where it is installed.
The encoder is held to that package's own answers: a committed fixture (tests/golden/bpe_encoder.json,
written by tests/golden/make_bpe_golden.py) and, where the package is installed, live comparisons.
Host-only: no GPU."""
import json
import pathlib
import random
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
    assert run.returncode == 1 and "--tokenizer" in run.stderr
    run = subprocess.run([str(tool), "--tokens", "5"], capture_output=True, text=True)
    assert run.returncode == 1 and "--aot" in run.stderr


# ---- text -> ids ---------------------------------------------------------------------------------
GOLDEN = pathlib.Path(__file__).parent / "golden" / "bpe_encoder.json"
QWEN_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*"
                r"|\s*[\r\n]+|\s+(?!\S)|\s+")


@pytest.fixture(scope="module")
def golden():
    return json.loads(GOLDEN.read_text())


def test_pretokenize_against_the_committed_pieces(golden):
    for case in golden["cases"]:
        assert L.pretokenize(case["text"]) == case["pieces"], case["text"]
    assert L.pretokenize("") == []


def test_encode_against_the_committed_ids(golden):
    v = L.Vocab(golden["tokenizer"])
    for case in golden["cases"]:
        ids = v.encode(case["text"])
        assert ids == case["ids"], case["text"]
        if "\u0301" not in case["text"]:  # decode(encode(text)) is the text (the byte alphabet loses nothing)
            assert v.decode(ids) == case["text"]
    assert v.encode("") == []
    # the chat template's markers come out as single ids, the text between them as pieces
    prompt = L.chat_prompt("What's 2+2?", thinking=False)
    ids = v.encode(prompt)
    assert ids[0] == v.token_to_id("<|im_start|>") and ids.count(v.token_to_id("<|im_end|>")) == 1
    assert v.token_to_id("<think>") in ids and v.decode(ids) == prompt
    v.close()


def test_pretokenize_every_code_point_against_the_package():
    """Each code point, in the positions where its class matters (inside a word, after a space, after
    an apostrophe, doubled), against the regular-expression engine of the `tokenizers` package."""
    tokenizers = pytest.importorskip("tokenizers")
    split = tokenizers.pre_tokenizers.Split(tokenizers.Regex(QWEN_PATTERN), behavior="isolated", invert=False)
    points = [cp for cp in range(0x110000) if not 0xD800 <= cp <= 0xDFFF]
    for start in range(0, len(points), 4096):
        text = "".join("x" + chr(cp) + "y" + chr(cp) + chr(cp) + " " + chr(cp) + "'" + chr(cp) + "\n" for cp in points[start:start + 4096])
        assert L.pretokenize(text) == [p for p, _ in split.pre_tokenize_str(text)], hex(points[start])


def test_encode_random_texts_against_the_package(golden):
    tokenizers = pytest.importorskip("tokenizers")
    tok = tokenizers.Tokenizer.from_str(golden["tokenizer"])
    v = L.Vocab(golden["tokenizer"])
    rng = random.Random(11)
    alphabet = list("abcXYZ'sStTrReEvVmMlLdD  \t\n\r.,!?-_()123") + ["\r\n", "\u017f", "\u212a", "é", "你", "好", "😀", "\u00a0", "\u3000", "\u200b",
                                                                  "\x85", "\x1c", "<|im_start|>", "<think>", "<|im_end|>", "<", "|", ">"]
    for _ in range(3000):
        text = "".join(rng.choice(alphabet) for _ in range(rng.randint(1, 40)))
        assert v.encode(text) == tok.encode(text, add_special_tokens=False).ids, repr(text)
    v.close()


def test_ignore_merges_and_string_merges(golden):
    """`ignore_merges` (a piece that is a token is taken whole) and merges written as "left right"
    strings (tokenizer.json files written before the pair form)."""
    tokenizers = pytest.importorskip("tokenizers")
    blob = json.loads(golden["tokenizer"])
    blob["model"]["merges"] = [m if isinstance(m, str) else " ".join(m) for m in blob["model"]["merges"]]
    blob["model"]["ignore_merges"] = True
    a = byte_alphabet()
    whole = a[ord(" ")] + "zzqq"  # a token no merge sequence reaches
    blob["model"]["vocab"][whole] = max(blob["model"]["vocab"].values()) + 10
    text = json.dumps(blob)
    tok, v = tokenizers.Tokenizer.from_str(text), L.Vocab(text)
    for sample in [" zzqq", "a zzqq zzqq!", "zzqq", "Hello world, it's a fine day."]:
        assert v.encode(sample) == tok.encode(sample, add_special_tokens=False).ids
    assert v.encode(" zzqq") == [blob["model"]["vocab"][whole]]
    v.close()


def test_encoder_refuses_what_it_does_not_restate(golden):
    blob = json.loads(golden["tokenizer"])
    # another pattern: decoding still works, encoding says why not
    other = json.loads(golden["tokenizer"])
    other["pre_tokenizer"]["pretokenizers"][0]["pattern"]["Regex"] = r"(?<=\s)\w+|\s+"  # look-behind
    v = L.Vocab(json.dumps(other))
    assert v.decode([v.token_to_id("<|im_end|>")]) == "<|im_end|>"
    with pytest.raises(L.LlmcpError, match="look-behind"):
        v.encode("hello")
    v.close()
    # a pre-tokeniser step that is not restated, and a step behind ByteLevel
    other = json.loads(golden["tokenizer"])
    other["pre_tokenizer"]["pretokenizers"].insert(0, {"type": "Digits", "individual_digits": True})
    v = L.Vocab(json.dumps(other))
    with pytest.raises(L.LlmcpError, match="Digits"):
        v.encode("hello")
    v.close()
    other = json.loads(golden["tokenizer"])
    other["pre_tokenizer"]["pretokenizers"].reverse()
    v = L.Vocab(json.dumps(other))
    with pytest.raises(L.LlmcpError, match="behind ByteLevel"):
        v.encode("hello")
    v.close()
    # a bare vocabulary has no merges
    v = L.Vocab(json.dumps(make_vocab()))
    with pytest.raises(L.LlmcpError, match="merges"):
        v.encode("hello")
    v.close()
    # an added token with whitespace stripping
    other = json.loads(golden["tokenizer"])
    other["added_tokens"][0]["lstrip"] = True
    v = L.Vocab(json.dumps(other))
    with pytest.raises(L.LlmcpError, match="lstrip"):
        v.encode("hello")
    v.close()
    # a normaliser other than NFC
    other = json.loads(golden["tokenizer"])
    other["normalizer"] = {"type": "Lowercase"}
    v = L.Vocab(json.dumps(other))
    with pytest.raises(L.LlmcpError, match="normalizer"):
        v.encode("hello")
    v.close()
    # model options that change the result
    for key, value, word in (("dropout", 0.1, "dropout"), ("byte_fallback", True, "byte_fallback"), ("end_of_word_suffix", "</w>", "suffix")):
        other = json.loads(golden["tokenizer"])
        other["model"][key] = value
        v = L.Vocab(json.dumps(other))
        with pytest.raises(L.LlmcpError, match=word):
            v.encode("hello")
        v.close()
    other = json.loads(golden["tokenizer"])
    del other["model"]["vocab"][byte_alphabet()[0x41]]  # "A"
    v = L.Vocab(json.dumps(other))
    with pytest.raises(L.LlmcpError, match="merge names|byte alphabet"):
        v.encode("hello")
    v.close()
    # ill-formed UTF-8
    v = L.Vocab(json.dumps(blob))
    with pytest.raises(L.LlmcpError, match="ill-formed"):
        v.encode(b"ab\xffcd")
    v.close()


def nfc_tokenizer(golden):
    blob = json.loads(golden["tokenizer"])
    assert blob["normalizer"] is None
    blob["normalizer"] = {"type": "NFC"}
    return json.dumps(blob)


def test_nfc_against_the_committed_forms(golden):
    """Under an NFC normaliser (the shipped Qwen tokenizer.json has one) the text between added tokens is
    normalised before it is split: marks put into canonical order, pairs composed, Hangul by arithmetic."""
    v = L.Vocab(nfc_tokenizer(golden))
    for case in golden["nfc_cases"]:
        if "<|" not in case["text"]:
            assert L.normalize_nfc(case["text"]) == case["nfc"], case["text"].encode("unicode_escape")
        assert v.encode(case["text"]) == case["ids"], case["text"].encode("unicode_escape")
    assert L.normalize_nfc("") == "" and L.normalize_nfc("plain ascii") == "plain ascii"
    # a Sequence that holds only NFC is NFC
    blob = json.loads(nfc_tokenizer(golden))
    blob["normalizer"] = {"type": "Sequence", "normalizers": [{"type": "NFC"}]}
    w = L.Vocab(json.dumps(blob))
    assert w.encode("cafe\u0301 \u1112\u1161") == v.encode("cafe\u0301 \u1112\u1161")
    w.close()
    # an added token is cut out of the raw text: the mark behind <|im_end|> does not reach into it
    ids = v.encode("<|im_end|>\u0301")
    assert ids[0] == v.token_to_id("<|im_end|>") and len(ids) > 1
    v.close()
    # an added token that is matched after normalisation is not restated
    blob = json.loads(nfc_tokenizer(golden))
    blob["added_tokens"][-1]["normalized"] = True
    v = L.Vocab(json.dumps(blob))
    with pytest.raises(L.LlmcpError, match="normalized"):
        v.encode("hello")
    v.close()


def test_nfc_every_code_point_against_the_package(golden):
    """Each code point alone, after a base, in front of two marks and behind a mark of the highest class,
    against the package's normaliser (its tables are older than Unicode 15: what it does not know
    stays as it is, here too); then random mixtures of marks, jamo and decomposable characters, and the
    NFC tokenizer's ids on them."""
    tokenizers = pytest.importorskip("tokenizers")
    import unicodedata
    nfc = tokenizers.normalizers.NFC().normalize_str
    points = [cp for cp in range(0x110000) if not 0xD800 <= cp <= 0xDFFF]
    for start in range(0, len(points), 4096):
        text = "".join(chr(c) + "|a" + chr(c) + "|" + chr(c) + "\u0323\u0301|a\u0345" + chr(c) + "|" for c in points[start:start + 4096])
        assert L.normalize_nfc(text) == nfc(text), hex(points[start])
    rng = random.Random(5)
    special = [c for c in points if unicodedata.combining(chr(c))] + list(range(0x1100, 0x1200)) + list(range(0xAC00, 0xAC40))
    special += [c for c in points if unicodedata.decomposition(chr(c)) and not unicodedata.decomposition(chr(c)).startswith("<")]
    text = nfc_tokenizer(golden)
    tok, v = tokenizers.Tokenizer.from_str(text), L.Vocab(text)
    for _ in range(20000):
        sample = "".join(chr(rng.choice(special if rng.random() < 0.8 else points)) for _ in range(rng.randint(1, 10)))
        assert L.normalize_nfc(sample) == nfc(sample), sample.encode("unicode_escape")
    for _ in range(2000):
        sample = "".join(rng.choice(["a", "e", " ", "\n", "<|im_end|>", "'s"]) if rng.random() < 0.5 else chr(rng.choice(special)) for _ in range(rng.randint(1, 16)))
        assert v.encode(sample) == tok.encode(sample, add_special_tokens=False).ids, sample.encode("unicode_escape")
    v.close()


def test_llmcp_run_tokenize_only(tmp_path, golden):
    """llmcp-run.cpp:646-653: --tokenize-only prints the ids of --text and --expect-token checks the first."""
    tool = L._PACKAGE / "bin" / "llmcp-run"
    path = tmp_path / "tokenizer.json"
    path.write_text(golden["tokenizer"])
    v = L.Vocab(golden["tokenizer"])
    want = v.encode(L.chat_prompt("Hello world", system="Be brief", thinking=False))
    base = [str(tool), "--tokenizer", str(path), "--text", "Hello world", "--chat", "--system", "Be brief", "--no-thinking", "--tokenize-only"]
    run = subprocess.run(base, capture_output=True, text=True)
    assert run.returncode == 0 and run.stdout.strip() == ",".join(map(str, want)), run.stderr
    assert subprocess.run(base + ["--expect-token", str(want[0])], capture_output=True).returncode == 0
    assert subprocess.run(base + ["--expect-token", str(want[0] + 1)], capture_output=True).returncode == 1
    run = subprocess.run([str(tool), "--tokenize-only", "--tokens", "77"], capture_output=True, text=True)
    assert run.returncode == 0 and run.stdout.strip() == "77"
    v.close()


# ---- the regular-expression matcher behind Split and ByteLevel -----------------------------------
# Patterns in the styles byte-level tokenizers use: contractions, optional leading character, digit
# groups, possessive and lazy quantifiers, case classes with marks, look-ahead, scripts, explicit ranges.
SPLIT_PATTERNS = [
    QWEN_PATTERN,
    r"'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+",
    r"'(?i:[sdmt]|ll|ve|re)|[^\r\n\p{L}\p{N}]?+\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]++[\r\n]*|\s*[\r\n]|\s+(?!\S)|\s+",
    r"[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]*[\p{Ll}\p{Lm}\p{Lo}\p{M}]+(?i:'s|'t|'re|'ve|'m|'ll|'d)?"
    r"|[^\r\n\p{L}\p{N}]?[\p{Lu}\p{Lt}\p{Lm}\p{Lo}\p{M}]+[\p{Ll}\p{Lm}\p{Lo}\p{M}]*(?i:'s|'t|'re|'ve|'m|'ll|'d)?"
    r"|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n/]*|\s*[\r\n]+|\s+(?!\S)|\s+",
    r"\p{N}{1,3}", r"[\u4e00-\u9fa5\u3040-\u309f\u30a0-\u30ff]+", r"\s?\p{L}+|\s?\p{P}+|\d", r"\w+|[^\w\s]+", r" ",
    r"a|b*?c|[^abc]{2,}?d", r"(?:ab)+|(?>a+)b|x(?=y)|\bfoo\b", r"(?i)hello|WORLD", r"x(?i)a|B", r"[\x41-\x5a]+|\x{1F600}",
    r"\p{Han}+|\p{Hiragana}+|\p{Katakana}+", r"[\p{L}\p{M}]+|[\p{P}\p{S}]|\p{Zs}+|\P{L}", r"\S+\s*",
    r"^\w+|\w+$|\n^", r"\A\s+|\s+\z|a{2}?b",
]
FUZZ_ALPHABET = list("abcXYZ'sStTrReEvVmMlLdD  \t\n\r.,!?-_()/12345foo") + [
    "\r\n", "\u017f", "\u212a", "é", "É", "ß", "你", "好", "ひ", "カ", "😀", "\u00a0", "\u3000", "\u0301", "\u200b", "\x85", "\u01c5",
    "\u02b0", "\u2177", "«", "$", "+", "²", "½", "٣", "hello", "WORLD", "World", "xa", "xB"]


def fuzz_texts(count, seed):
    rng = random.Random(seed)
    fixed = ["", " ", "Hello world, it's 12345 o'clock!!\n\n  x", "fooBarBaz foo's FOO'S 1234567 a\r\n\r\n b"]
    return fixed + ["".join(rng.choice(FUZZ_ALPHABET) for _ in range(rng.randint(1, 30))) for _ in range(count)]


def test_regex_split_against_the_package():
    tokenizers = pytest.importorskip("tokenizers")
    texts = fuzz_texts(250, 2)
    for pattern in SPLIT_PATTERNS:
        for behavior in ("isolated", "removed", "merged_with_previous", "merged_with_next", "contiguous"):
            for invert in (False, True):
                split = tokenizers.pre_tokenizers.Split(tokenizers.Regex(pattern), behavior=behavior, invert=invert)
                for text in texts if (behavior, invert) == ("isolated", False) else texts[:60]:
                    want = [piece for piece, _ in split.pre_tokenize_str(text)]
                    assert L.regex_split(pattern, text, behavior, invert) == want, (pattern, behavior, invert, text)


def test_random_patterns_against_the_package():
    """Patterns thrown together from the constructs the matcher takes: where both it and the package
    accept one, the pieces are the same (a pattern the matcher refuses is not an error here)."""
    tokenizers = pytest.importorskip("tokenizers")
    rng = random.Random(21)
    atoms = ["a", "b", "c", " ", r"\s", r"\S", r"\d", r"\w", r"\p{L}", r"\p{N}", r"\P{L}", "[ab]", r"[^a\s]", "[a-c]", ".", r"\r", r"\n", "(?:", "(", ")",
             "|", "?", "*", "+", "{1,2}", "{2}", "?+", "*?", "+?", "(?i:", "(?=", "(?!", "(?>", "^", "$", r"\b", "'", "x", "é", "你", "{2}?", "{1,}?",
             r"\A", r"\z", r"\B", "(?i)", "A", "S", r"[^\r\n\p{L}]", r"[\w-]", "[]a]", r"[a\]]", r"\.", r"\x41", "\u212a", "\u017f", "-", "{", "}", ",", "1"]
    texts = ["", "a", "ab cab  abc\n", "aab b\r\nc", "x'a é你 1a2", "   ", "abcabcabc", "AbS\u017f\u212a-a]1{2}, A.a", "\n\na\n"]
    compared = 0
    for _ in range(6000):
        pattern = "".join(rng.choice(atoms) for _ in range(rng.randint(1, 8)))
        try:
            ours = [L.regex_split(pattern, text) for text in texts]
        except L.LlmcpError:
            continue
        try:
            split = tokenizers.pre_tokenizers.Split(tokenizers.Regex(pattern), behavior="isolated")
            theirs = [[piece for piece, _ in split.pre_tokenize_str(text)] for text in texts]
        except Exception:
            continue
        assert ours == theirs, pattern
        compared += 1
    assert compared > 1500


def test_regex_classes_on_every_code_point():
    """Each class on the string of all code points: what a Split with behaviour "removed" leaves."""
    tokenizers = pytest.importorskip("tokenizers")
    text = "".join(chr(cp) for cp in range(0x110000) if not 0xD800 <= cp <= 0xDFFF)
    for cls in (r"\w", r"[\w]", r"\W", r"[^\w]", r"\s", r"\S", r"\d", r"\D", r".", r"\p{L}", r"\P{L}", r"\p{Lu}", r"\p{Ll}", r"\p{Lt}", r"\p{Lm}",
                r"\p{Lo}", r"\p{M}", r"\p{Mn}", r"\p{N}", r"\p{Nd}", r"\p{P}", r"\p{S}", r"\p{Z}", r"\p{Zs}", r"\p{C}", r"\p{Cn}", r"\p{Cf}",
                r"\p{Han}", r"\p{Hangul}", r"\p{Latin}", r"\p{Cyrillic}", r"[^\s\p{L}\p{N}]", r"\p{Letter}", r"\p{^L}"):
        pattern = "(?:%s)+" % cls
        split = tokenizers.pre_tokenizers.Split(tokenizers.Regex(pattern), behavior="removed", invert=False)
        assert L.regex_split(pattern, text, "removed") == [piece for piece, _ in split.pre_tokenize_str(text)], cls


def test_regex_refuses_what_it_does_not_restate():
    for pattern, word in ((r"(?<=a)b", "look-behind"), (r"(a)\1", "back-references"), (r"[a&&[b]]", "intersections"), (r"[a[:alpha:]]", "nested"), (r"\p{Greekish}", "unknown property"),
                          (r"(?i)é", "non-ASCII"), (r"(a*)*", "can be empty"), (r"(?m)a", "flag"), (r"a{2,1}", "quantifier"), (r"(a", "missing"),
                          (r"a)", "unmatched"), (r"\h", "escape")):
        with pytest.raises(L.LlmcpError, match=word):
            L.regex_split(pattern, "abc")
    with pytest.raises(L.LlmcpError, match="empty string"):
        L.regex_split(r"a?", "bbb")
    with pytest.raises(L.LlmcpError, match="behaviour"):
        L.regex_split(r"a", "bbb", behavior="sideways")


def trained(tokenizers, pre_tokenizer, normalizer=None):
    tok = tokenizers.Tokenizer(tokenizers.models.BPE())
    tok.pre_tokenizer = pre_tokenizer
    if normalizer is not None:
        tok.normalizer = normalizer
    tok.decoder = tokenizers.decoders.ByteLevel()
    corpus = ["Hello world, it's a fine day. I'll say they've done 12345 things!\n\n  indented\tcode();\r\n",
              "Größe naïve café — «quotes» … 你好世界 こんにちは カタカナ мир", "def f(x):\n    return x**2 + 1  # comment 2024-01-31\n",
              "   spaces   everywhere   \n \n\t\n", "emoji 😀😃 and ½ ² ٣ numbers"] * 20
    trainer = tokenizers.trainers.BpeTrainer(vocab_size=480, special_tokens=["<|endoftext|>", "<|im_end|>"],
                                             initial_alphabet=tokenizers.pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tok.train_from_iterator(corpus, trainer)
    return tok


def test_encode_with_other_pre_tokenizers():
    """Tokenizers set up the way other byte-level BPE models ship them: ByteLevel with its own pattern
    (with and without the prefix space), several Split steps in a row, a literal-string Split."""
    tokenizers = pytest.importorskip("tokenizers")
    P, R = tokenizers.pre_tokenizers, tokenizers.Regex
    setups = [
        P.ByteLevel(add_prefix_space=False, use_regex=True),
        P.ByteLevel(add_prefix_space=True, use_regex=True),
        P.Sequence([P.Split(R(SPLIT_PATTERNS[2]), behavior="isolated"), P.ByteLevel(add_prefix_space=False, use_regex=False)]),
        P.Sequence([P.Split(R(r"\p{N}{1,3}"), behavior="isolated"), P.Split(R(SPLIT_PATTERNS[5]), behavior="isolated"),
                    P.Split(R(SPLIT_PATTERNS[3]), behavior="isolated"), P.ByteLevel(add_prefix_space=False, use_regex=False)]),
        P.Sequence([P.Split(" ", behavior="merged_with_next"), P.Split(R(r"\d"), behavior="isolated"),
                    P.ByteLevel(add_prefix_space=False, use_regex=False)]),
        P.Sequence([P.Split(R(r"\s+"), behavior="removed"), P.ByteLevel(add_prefix_space=False, use_regex=True)]),
    ]
    texts = fuzz_texts(400, 4) + ["<|im_end|>x<|im_end|> y", "a<|endoftext|>"]
    for number, setup in enumerate(setups):
        tok = trained(tokenizers, setup, tokenizers.normalizers.NFC() if number == 3 else None)
        v = L.Vocab(tok.to_str())
        for text in texts:
            assert v.encode(text) == tok.encode(text, add_special_tokens=False).ids, (number, text)
        v.close()
