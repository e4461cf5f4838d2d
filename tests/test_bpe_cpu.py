"""The byte-level BPE encoder and decoder (Tokenizer.encode_bpe / decode_bpe, the CLI's --bpe) against the
HF `tokenizers` library on a tokenizer.json of the Qwen2 layout: added ChatML tokens, the NFC normaliser, the
Qwen2 pre-tokenizer pattern as a Split step, ByteLevel without its own regex, BPE merges learned here on a small
corpus.
The reference has no such encoder (inference/src/io/tokenizer.cpp:86-135 drops spaces and newlines); its authors
run HF for correct ids (tools/tokenize_correctly.py:11-36), which is what this test compares with, id for id."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tensor-ffn_b200"))

tokenizers = pytest.importorskip("tokenizers")

QWEN2_PATTERN = (r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*"
                 r"|\s*[\r\n]+|\s+(?!\S)|\s+")
SPECIALS = ["<|endoftext|>", "<|im_start|>", "<|im_end|>"]

CORPUS = [
    "def fibonacci(n):\n    if n < 2:\n        return n\n    return fibonacci(n - 1) + fibonacci(n - 2)\n",
    "The quick brown fox jumps over the lazy dog. It's 12345 o'clock, isn't it? We'll see, they've said.",
    "for (int i = 0; i < n; ++i) { sum += a[i] * b[i]; }  // dot product\r\n",
    "Größe, naïve café, façade — «quoted» … and 日本語のテキスト, 中文字符, русский текст, ελληνικά.",
    "tabs\tand\ttabs,   runs   of   spaces,\n\n\nblank lines and trailing space   \n",
    "emoji 🙂🚀 and numbers 3.14159 2024-11-25 0xDEADBEEF 1e-9 ١٢٣ ⅓",
    "I'M SHOUTING, YOU'RE NOT. HE'D'VE. 'Twas 'tis.",
    "system\nYou are a helpful coding assistant.", "user\n", "assistant\n",
] * 4


@pytest.fixture(scope="module")
def tok_dir(tmp_path_factory):
    from tokenizers import Regex, Tokenizer, decoders, models, normalizers, pre_tokenizers, trainers
    t = Tokenizer(models.BPE())
    t.normalizer = normalizers.NFC()
    t.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(QWEN2_PATTERN), behavior="isolated", invert=False),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False),
    ])
    t.decoder = decoders.ByteLevel()
    trainer = trainers.BpeTrainer(vocab_size=700, special_tokens=SPECIALS, show_progress=False,
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    t.train_from_iterator(CORPUS, trainer)
    d = str(tmp_path_factory.mktemp("bpe_tok"))
    t.save(os.path.join(d, "tokenizer.json"))
    return d, t


CASES = [
    "Hello, world!",
    "def add(a, b):\n    return a + b\n",
    "  leading spaces and trailing  ",
    "a\n\n\nb \n c\t\td",
    "It's they'll WE'VE I'm he'd don't 'sup",
    "x=12345+678;y=9",
    "naïve café — 日本語 русский 🙂🚀 …",
    "\r\n\r\n  \r\n",
    "   ",
    " ",
    "a",
    "!!!???...\n\n",
    "tab\there  \n  there",
    "١٢٣ ⅓ ²",
    "<|im_start|>system\nYou are a helpful coding assistant.<|im_end|>\n<|im_start|>user\nhi there<|im_end|>\n"
    "<|im_start|>assistant\n",
    "text<|endoftext|>more text <|im_end|",
    "fibonacci(n - 1) + fibonacci(n - 2)",
    " non-breaking em space　ideographic",
    # not in NFC: combining sequences, marks out of canonical order, Hangul jamo, singletons
    "cafe\u0301 A\u030a a\u0323\u0307 a\u0307\u0323 \u1100\u1161\u11a8 \u1112\u1161 \u212b \u2126 \u0958 q\u0307\u0323",
    "\u0301leading mark, \u0041\u0300\u0301\u0302 stacked, \uac00\u11a8 syllable + final",
]


def test_bpe_encode_matches_hf(tok_dir):
    import tffn
    d, hf = tok_dir
    ours = tffn.Tokenizer(d)
    for text in CASES:
        want = hf.encode(text, add_special_tokens=False).ids
        got = ours.encode_bpe(text)
        assert got == want, (text, got, want)
    assert ours.encode_bpe("") == []


def test_bpe_decode_round_trip(tok_dir):
    import unicodedata

    import tffn
    d, hf = tok_dir
    ours = tffn.Tokenizer(d)
    for text in CASES:
        ids = ours.encode_bpe(text)
        want = unicodedata.normalize("NFC", text)  # what the normaliser makes of the input
        assert ours.decode_bpe(ids) == want
        # token by token, as the command line prints them: the bytes concatenate to the same text
        raw = b"".join(_decode_bytes(ours, [i]) for i in ids)
        assert raw.decode("utf-8") == want


def test_nfc_matches_unicodedata_on_seeded_strings(tok_dir):
    """the normaliser alone (through encode + decode, which are otherwise lossless): random strings over starters,
    combining marks of several classes, precomposed letters, Hangul jamo and syllables, compatibility singletons"""
    import random
    import unicodedata

    import tffn
    d, _ = tok_dir
    ours = tffn.Tokenizer(d)
    rng = random.Random(11)
    pool = ([chr(c) for c in range(0x300, 0x330)] + [chr(c) for c in (0x5B0, 0x5B4, 0x5BC, 0x64B, 0x651, 0x93C, 0x94D, 0xF71, 0xF72, 0xF74)]
            + list("aeiouAEOUcnsyzdD ") + list("áàâäåçéèêëñöüÅΩǺẛ̣") + [chr(c) for c in (0x1100, 0x1102, 0x1161, 0x1163, 0x11A8, 0x11AF, 0xAC00, 0xAC01, 0xD55C)]
            + [chr(c) for c in (0x212B, 0x2126, 0x0340, 0x0341, 0x0343, 0x0344, 0x0958, 0x0F43, 0xFB1D, 0x1E9B, 0x1D15E)])
    for _ in range(500):
        text = "".join(rng.choice(pool) for _ in range(rng.randint(1, 12)))
        assert ours.decode_bpe(ours.encode_bpe(text)) == unicodedata.normalize("NFC", text), [hex(ord(c)) for c in text]


def _decode_bytes(tok, ids):
    import ctypes

    import numpy as np
    import tffn
    a = np.ascontiguousarray(ids, dtype=np.uint32)
    n = tffn._L.tffn_tokenizer_decode_bpe(tok._h, a.ctypes.data, a.size, None, 0)
    buf = ctypes.create_string_buffer(n + 1)
    tffn._L.tffn_tokenizer_decode_bpe(tok._h, a.ctypes.data, a.size, buf, n + 1)
    return buf.raw[:n]


def test_bpe_seeded_random_text_matches_hf(tok_dir):
    """random strings over an alphabet that mixes letters, digits, marks, spaces, newlines, quotes"""
    import random

    import tffn
    d, hf = tok_dir
    ours = tffn.Tokenizer(d)
    rng = random.Random(7)
    alphabet = list("abcXYZ019 .,'\n\r\t-_(){}é日я🙂") + ["'s", "'LL", "  ", "\n\n", "<|im_end|>"]
    for _ in range(300):
        text = "".join(rng.choice(alphabet) for _ in range(rng.randint(1, 40)))
        assert ours.encode_bpe(text) == hf.encode(text, add_special_tokens=False).ids, repr(text)


def test_reference_encoder_unchanged(tok_dir):
    """the default encoder keeps the reference's behaviour (spaces and newlines vanish): --bpe is opt-in"""
    import tffn
    d, _ = tok_dir
    ours = tffn.Tokenizer(d)
    assert ours.encode("a b") == ours.encode("ab")
    assert ours.encode_bpe("a b") != ours.encode_bpe("ab")
