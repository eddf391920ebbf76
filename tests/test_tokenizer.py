"""The native byte-pair tokenizer (nfai_tokenizer_*, host only) against the literal restatement of the reference's
Tokenizer.cs in oracle/tokenizer_oracle.py. Token ids are integers: every comparison is exact."""
import os
import time

import numpy as np
import pytest

from nfai_b200 import NfaiError
from nfai_b200.tokenizer import Tokenizer
from oracle.tokenizer_oracle import OracleTokenizer

from . import tok_util

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def pair():
    md = tok_util.metadata()
    native = Tokenizer(md)
    ref = OracleTokenizer(md["tokenizer.ggml.tokens"], md["tokenizer.ggml.merges"], 0, 1)
    yield native, ref, md
    native.close()


EDGE_CASES = [
    "", " ", "  ", "\n", "\n\n", " \n ", "a", " a", "  a", "   a b", "a  ", "a \n", "a\n\nb", "tab\tseparated\twords",
    "line one\r\nline two\r\n", "it's we're THEY'VE i'M you'LL he'D don't", "12345678 90 1", "x=1;y=22;z=333;w=4444",
    "!!! ??? ... --- \n\n", " ,a", ",a", "\ta", "\t\ta", "1a2b3c", "naïve café", "привет мир", "日本語 テスト",
    "emoji \U0001F600 end", "a b", "a b", "mixed  \t \n  \t x", "'", "''s", "'s's", "a'LLb",
    "trailing spaces   ", "   leading", "The quick brown fox jumps over a lazy dog.", "tokenizer merges streaming kernels",
]


def _outcome(fn):
    """The ids, or "error" when the call fails the way the reference does (an exception)."""
    try:
        return fn()
    except (NfaiError, KeyError):
        return "error"


@pytest.mark.parametrize("text", EDGE_CASES)
def test_chat_template_matches_reference(pair, text):
    native, ref, _ = pair
    for bos in (True, False):
        assert _outcome(lambda: native.tokenize(text, add_bos=bos)) == _outcome(lambda: ref.tokenize(text, add_bos=bos))


def test_text_before_the_first_special_token_is_dropped(pair):
    native, ref, _ = pair
    a = native.encode("dropped words<|eot_id|>kept words")
    assert a == ref.encode("dropped words<|eot_id|>kept words") == native.encode("<|eot_id|>kept words")
    assert native.encode("no special token at all") == ref.encode("no special token at all") == []


def test_random_strings_match_reference(pair):
    native, ref, _ = pair
    rng = np.random.default_rng(11)
    alphabet = list("abcdefghijklmnopqrstuvwxyzTHEQUICK0123456789 \n\t.,;:'!?-()éïüßпривет日本語") + ["  ", "\n\n", "\r\n", "'s", "'re", "\U0001F600"]
    encoded = 0
    for _ in range(300):
        n = int(rng.integers(1, 60))
        s = "".join(alphabet[int(i)] for i in rng.integers(0, len(alphabet), n))
        got = _outcome(lambda: native.encode("<|eot_id|>" + s))
        assert got == _outcome(lambda: ref.encode("<|eot_id|>" + s)), repr(s)
        encoded += got != "error"
    assert encoded >= 290  # the alphabet is inside the vocabulary: these are real encodings, not matching failures


def test_whitespace_and_punctuation_runs_match_reference(pair):
    """The pattern's alternatives differ only in how they carve up runs of spaces, line breaks and punctuation."""
    native, ref, _ = pair
    rng = np.random.default_rng(12)
    alphabet = [" ", " ", "\n", "\r", "\t", "a", "B", "7", ".", "'", "-", "s", "l"]
    for _ in range(400):
        n = int(rng.integers(1, 24))
        s = "".join(alphabet[int(i)] for i in rng.integers(0, len(alphabet), n))
        assert native.encode("<|eot_id|>" + s) == ref.encode("<|eot_id|>" + s), repr(s)


def test_detokenize_round_trip(pair):
    native, ref, _ = pair
    text = "The quick brown fox\njumps over 12345 lazy dogs, doesn't it?  Yes."
    ids = native.encode("<|eot_id|>" + text)
    assert native.detokenize(ids) == ref.detokenize(ids) == "<|eot_id|>" + text
    with pytest.raises(NfaiError):
        native.detokenize([10 ** 6])


def test_errors_match_reference(pair):
    native, ref, _ = pair
    with pytest.raises(NfaiError):
        native.tokenize("<|no_such_token|>")          # the prompt smuggles in an unknown special token
    with pytest.raises(KeyError):
        ref.tokenize("<|no_such_token|>")
    with pytest.raises(NfaiError):
        native.tokenize("ЖЖЖ 中")    # characters without a vocabulary entry
    with pytest.raises(KeyError):
        ref.tokenize("ЖЖЖ 中")


def test_duplicate_entries_resolve_like_the_reference():
    tokens = [b"<|eot_id|>", b"a", b"b", b"ab", b"c", b"ab", b"abc", b"bc"]   # "ab" twice: the last id wins
    merges = ["a b", "b c", "a b", "ab c"]                                      # "a b" twice: the first rank wins
    md = {"tokenizer.ggml.tokens": tokens, "tokenizer.ggml.merges": merges,
          "tokenizer.ggml.bos_token_id": 0, "tokenizer.ggml.eos_token_id": 0}
    native, ref = Tokenizer(md), OracleTokenizer(tokens, merges, 0, 0)
    for s in ("ab", "abc", "bc", "abcabc", "cab", "aabbc"):
        got = native.encode("<|eot_id|>" + s)
        assert got == ref.encode("<|eot_id|>" + s)
    assert native.encode("<|eot_id|>ab") == [0, 5]
    assert native.encode("<|eot_id|>abc") == [0, 6]      # "a b" (rank 0) before "b c" (rank 1), then "ab c"
    native.close()


def test_golden_token_ids(pair):
    native, ref, _ = pair
    g = np.load(os.path.join(GOLDEN, "tokenizer.npz"), allow_pickle=False)
    texts = [t for t in bytes(g["texts"]).decode("utf-8").split("\x00")]
    offs = g["offsets"]
    for i, t in enumerate(texts):
        want = list(g["ids"][offs[i]:offs[i + 1]])
        assert ref.tokenize(t) == want
        assert native.tokenize(t) == want


def test_hash_map_is_faster_than_the_list_scan(pair):
    native, ref, _ = pair
    text = " ".join(tok_util._WORDS * 3)
    t0 = time.perf_counter()
    a = native.tokenize(text)
    t1 = time.perf_counter()
    b = ref.tokenize(text)
    t2 = time.perf_counter()
    assert a == b
    assert (t1 - t0) < (t2 - t1)


def test_compiled_reference_scan_equals_the_python_restatement(pair):
    """orc_bpe_merge_scan (the reference's merge search in C++, used for timing) against the Python loop."""
    _, ref, md = pair
    fast = OracleTokenizer(md["tokenizer.ggml.tokens"], md["tokenizer.ggml.merges"], 0, 1, compiled=True)
    for text in EDGE_CASES + [" ".join(tok_util._WORDS)]:
        assert _outcome(lambda: fast.tokenize(text)) == _outcome(lambda: ref.tokenize(text))


def test_pretokenisation_matches_the_pattern_on_unicode_text(pair):
    """The hand-written matcher against the pattern itself (third-party `regex` on UTF-16 code units) on random text
    drawn from letters, numbers, marks, punctuation, symbols, separators and controls of many scripts."""
    import unicodedata

    from oracle.tokenizer_oracle import META, utf16_units
    native, _, _ = pair
    rng = np.random.default_rng(21)
    pools = {}
    for cp in list(range(0x20, 0x3000)) + list(range(0x3040, 0x3100)) + list(range(0x4E00, 0x4E80)) + list(range(0xAC00, 0xAC40)) + \
            list(range(0xFF00, 0xFFEF)) + [0x09, 0x0A, 0x0B, 0x0C, 0x0D, 0x85, 0x1F600, 0x1F680, 0x10400, 0x1D7D8]:
        if 0xD800 <= cp <= 0xDFFF:
            continue
        pools.setdefault(unicodedata.category(chr(cp))[0], []).append(chr(cp))
    common = list(" \n\r\t'abcXYZ019.,!-")
    checked = 0
    for trial in range(600):
        n = int(rng.integers(1, 40))
        chars = []
        for _ in range(n):
            if rng.random() < 0.5:
                chars.append(common[int(rng.integers(0, len(common)))])
            else:
                cat = list(pools)[int(rng.integers(0, len(pools)))]
                chars.append(pools[cat][int(rng.integers(0, len(pools[cat])))])
        text = "".join(chars)
        want = [m.end() for m in META.finditer(utf16_units(text))]
        assert native.pretokenize_ends(text) == want, repr(text)
        checked += len(want)
    assert checked > 5000
