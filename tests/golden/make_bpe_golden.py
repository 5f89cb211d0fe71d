"""Writes tests/golden/bpe_encoder.json: a small byte-level BPE tokenizer with the Qwen pre-tokenisation
pattern, trained here by the Hugging Face `tokenizers` package (the library the reference's tokenizer
dependency wraps; tools/llmcp-run/llmcp-run.cpp:635-641 calls its Encode), and that package's own
answers on a list of texts: the pieces of the split step and the ids of the whole encoder.

    python tests/golden/make_bpe_golden.py
"""
import json
import pathlib
import random

from tokenizers import AddedToken, Regex, Tokenizer, decoders, models, pre_tokenizers, trainers

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


def main():
    tok = build()
    split = pre_tokenizers.Split(Regex(PATTERN), behavior="isolated", invert=False)
    cases = [{"text": t, "pieces": [p for p, _ in split.pre_tokenize_str(t)],
              "ids": tok.encode(t, add_special_tokens=False).ids} for t in texts()]
    target = pathlib.Path(__file__).with_name("bpe_encoder.json")
    target.write_text(json.dumps({"tokenizer": tok.to_str(), "cases": cases}, ensure_ascii=True))
    print(target, target.stat().st_size, "bytes", len(cases), "cases")


if __name__ == "__main__":
    main()
