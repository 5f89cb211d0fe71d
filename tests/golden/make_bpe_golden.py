"""Writes tests/golden/bpe_encoder.json: a small byte-level BPE tokenizer with the Qwen pre-tokenisation
pattern, trained here by the Hugging Face `tokenizers` package (the library the reference's tokenizer
dependency wraps; tools/llmcp-run/llmcp-run.cpp:635-641 calls its Encode), and that package's own
answers on a list of texts: the pieces of the split step, the ids of the whole encoder, the NFC form,
and the ids of the same tokenizer with an NFC normaliser in front (as the shipped Qwen tokenizer has).

    python tests/golden/make_bpe_golden.py
"""
import json
import pathlib
import random

from tokenizers import AddedToken, Regex, Tokenizer, decoders, models, normalizers, pre_tokenizers, trainers

PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*"
           r"|\s*[\r\n]+|\s+(?!\S)|\s+")

CORPUS = [
    "Hello world, it's a fine day. I'll say they've done 12345 things!\n\n  indented\tcode();\r\n",
    "Größe naïve café Ünïcödé — «quotes» … 你好世界 こんにちは мир привет",
    "def f(x):\n    return x**2 + 1  # comment\n",
    "   spaces   everywhere   \n \n\t\n",
    "emoji 😀😃 and ½ ² ٣ numbers ௧",
    "<|im_start|>user\nWhat's 2+2?<|im_end|>\n<|im_start|>assistant\n<think>\n\n</think>\n\n4",
]

ALPHABET = list("abcXYZ'sStTrReEvVmMlLdD  \t\n\r.,!?-_()123٣½²") + [
    "\r\n", "ſ", "K", "é", "ß", "你", "好", "😀", " ", " ", "　", "́", "​", "\x85", "\x1c",
    "ǅ", "ª", "ⅷ", "Ᲊ", "\U000105c0", "<|im_start|>", "<think>", "</think>", "<|im_end|>", "<|endoftext|>", "<", "|"]


def build():
    tok = Tokenizer(models.BPE())
    tok.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(PATTERN), behavior="isolated", invert=False),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)])
    tok.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=512, special_tokens=["<|endoftext|>", "<|im_start|>", "<|im_end|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet(), show_progress=False)
    tok.train_from_iterator(CORPUS * 20, trainer)
    tok.add_tokens([AddedToken("<think>", special=False, normalized=False),
                    AddedToken("</think>", special=False, normalized=False)])
    return tok


def texts():
    rng = random.Random(7)
    fixed = CORPUS + ["", " ", "  ", "\n", " \n ", "a  b", "a   ", "a \n  b", "'S 'T 'RE 'lL 'ſ x'ſ 'K", "don't DON'T",
                      "1234 x1y2", " !!\n\nx", "<|im_start|><|im_end|><think>", "<|im_start", "tab\t\tend\t"]
    return fixed + ["".join(rng.choice(ALPHABET) for _ in range(rng.randint(1, 24))) for _ in range(400)]


def nfc_texts():
    """Marks in and out of canonical order, pairs that compose and pairs that do not, singletons,
    conjoining Hangul, marks the package's (older) tables take for starters, then random mixtures."""
    rng = random.Random(9)
    pool = [chr(c) for c in list(range(0x300, 0x370)) + list(range(0x1100, 0x1113)) + list(range(0x1161, 0x1176))
            + list(range(0x11A8, 0x11C3)) + [0x212B, 0x2126, 0x1E9B, 0xFB1D, 0x9CB, 0x9C7, 0x9BE, 0x1DF6, 0x898, 0x10D24, 0xAC00, 0xAC01]]
    pool += list("aeiouAEOcnN ") + ["é", "ü", "ǖ", "ệ", "ṩ"]
    fixed = ["cafe\u0301", "e\u0323\u0302", "e\u0302\u0323", "\u212b", "\u1112\u1161\u11ab", "\u1e9b\u0323", "a\u0345\u0301",
             "q\u0307\u0323", "\u0344", "\u0958", "\u09c7\u09be", "a\u1df6\u0323", "<|im_start|>e\u0301<|im_end|>\u0301"]
    return fixed + ["".join(rng.choice(pool) for _ in range(rng.randint(2, 12))) for _ in range(300)]


def main():
    tok = build()
    split = pre_tokenizers.Split(Regex(PATTERN), behavior="isolated", invert=False)
    cases = [{"text": t, "pieces": [p for p, _ in split.pre_tokenize_str(t)],
              "ids": tok.encode(t, add_special_tokens=False).ids} for t in texts()]
    nfc = normalizers.NFC()
    tok.normalizer = nfc
    nfc_cases = [{"text": t, "nfc": nfc.normalize_str(t), "ids": tok.encode(t, add_special_tokens=False).ids} for t in nfc_texts()]
    tok.normalizer = None
    target = pathlib.Path(__file__).with_name("bpe_encoder.json")
    target.write_text(json.dumps({"tokenizer": tok.to_str(), "cases": cases, "nfc_cases": nfc_cases}, ensure_ascii=True))
    print(target, target.stat().st_size, "bytes", len(cases), "cases", len(nfc_cases), "NFC cases")


if __name__ == "__main__":
    main()
