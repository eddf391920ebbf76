"""A small synthetic byte-pair vocabulary for the tokenizer tests: trained here on a made-up corpus, so that every
merge result is a vocabulary entry (as in a real GGUF) without shipping anybody's vocabulary."""
from collections import Counter
from typing import Dict, List, Tuple

from oracle.tokenizer_oracle import META, OracleTokenizer, utf16_units

SPECIALS = ["<|begin_of_text|>", "<|end_of_text|>", "<|start_header_id|>", "<|end_header_id|>", "<|eot_id|>"]

_WORDS = ("the quick brown fox jumps over a lazy dog while seven wizards quietly box with jade vexing daft zebras "
          "token tokens tokenizer tokenize merge merges merging merged rank ranks ranking stream streams streaming "
          "kernel kernels shared memory register registers tensor tensors layer layers attention head heads cache "
          "position positions decode decoding prefill prompt prompts model models weight weights number numbers").split()
_EXTRA = ["naïve café déjà vu über straße", "привет мир это тест слова", "日本語 テスト 文字 漢字", "x = 12345 + 67 * 890;",
          "it's we're they've I'm you'll he'd DON'T", "a,b;c.d!e?f -- (g) [h] {i} <j>", "tab\there\tand\r\nwindows\r\nlines",
          "emoji \U0001F600 and \U0001F680 rockets", "A1B22C333D4444E55555", "  double  spaces   and    more\n\n\nnewlines \n x"]


def corpus() -> str:
    lines = []
    for i in range(60):
        lines.append(" ".join(_WORDS[(i * 7 + j * 3) % len(_WORDS)] for j in range(9)).capitalize() + ".")
    return "\n".join(lines + _EXTRA * 3)


def train_bpe(n_merges: int = 400) -> Tuple[List[bytes], List[str]]:
    text = utf16_units(corpus())
    words: Counter = Counter()
    alphabet = set()
    for m in META.finditer(text):
        units = tuple(OracleTokenizer.initial_units(m.group(0)))
        words[units] += 1
        alphabet.update(units)
    # every printable ASCII character, space and newline can always be encoded
    for cp in list(range(0x21, 0x7F)) + [0x20, 0x0A, 0x09, 0x0D]:
        alphabet.update(OracleTokenizer.initial_units(chr(cp)))
    merges: List[str] = []
    vocab_words: Dict[Tuple[bytes, ...], int] = dict(words)
    for _ in range(n_merges):
        pairs: Counter = Counter()
        for w, c in vocab_words.items():
            for a, b in zip(w, w[1:]):
                pairs[(a, b)] += c
        if not pairs:
            break
        (a, b), cnt = min(pairs.items(), key=lambda kv: (-kv[1], kv[0]))
        if cnt < 2:
            break
        try:
            merges.append(a.decode("utf-8") + " " + b.decode("utf-8"))
        except UnicodeDecodeError:
            break
        new_words: Dict[Tuple[bytes, ...], int] = {}
        for w, c in vocab_words.items():
            out, i = [], 0
            while i < len(w):
                if i + 1 < len(w) and w[i] == a and w[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(w[i])
                    i += 1
            new_words[tuple(out)] = new_words.get(tuple(out), 0) + c
        vocab_words = new_words
    tokens = [s.encode("utf-8") for s in SPECIALS] + sorted(alphabet)
    seen = set(tokens)
    for m in merges:
        a, b = m.split(" ", 1)
        t = (a + b).encode("utf-8")
        if t not in seen:
            tokens.append(t)
            seen.add(t)
    return tokens, merges


def metadata(n_merges: int = 400) -> Dict[str, object]:
    tokens, merges = train_bpe(n_merges)
    return {"tokenizer.ggml.tokens": tokens, "tokenizer.ggml.merges": merges,
            "tokenizer.ggml.bos_token_id": 0, "tokenizer.ggml.eos_token_id": 1}
