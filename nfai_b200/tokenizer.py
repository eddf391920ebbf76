"""Host-side mirror of the reference's Tokenizer (NFAI.Models.Llama3/Tokenizer.cs) over the native byte-pair
tokenizer of libnfai_cuda (nfai_tokenizer_*): same constructor input (the GGUF metadata), same methods."""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Sequence

from . import _lib
from ._lib import NfaiError


def _as_bytes(x) -> bytes:
    return x.encode("utf-8") if isinstance(x, str) else bytes(x)


class Tokenizer:
    def __init__(self, metadata: Dict[str, object]):
        """metadata: `tokenizer.ggml.tokens` (str or bytes entries), `tokenizer.ggml.merges` ("left right" strings),
        `tokenizer.ggml.bos_token_id`, `tokenizer.ggml.eos_token_id` (Tokenizer.cs:16-58)."""
        self._lib = _lib.load()
        tokens = [_as_bytes(t) for t in metadata["tokenizer.ggml.tokens"]]
        merges = [_as_bytes(m) for m in metadata["tokenizer.ggml.merges"]]
        self.BosTokenId = int(metadata["tokenizer.ggml.bos_token_id"])
        self.EosTokenId = int(metadata["tokenizer.ggml.eos_token_id"])
        self._keep = (tokens, merges)
        tok_ptrs = (C.c_char_p * len(tokens))(*tokens)
        tok_lens = (C.c_uint32 * len(tokens))(*[len(t) for t in tokens])
        mer_ptrs = (C.c_char_p * len(merges))(*merges)
        mer_lens = (C.c_uint32 * len(merges))(*[len(m) for m in merges])
        handle = C.c_void_p()
        rc = self._lib.nfai_tokenizer_create(C.cast(tok_ptrs, C.c_void_p), C.cast(tok_lens, C.c_void_p), len(tokens),
                                             C.cast(mer_ptrs, C.c_void_p), C.cast(mer_lens, C.c_void_p), len(merges),
                                             self.BosTokenId, self.EosTokenId, C.byref(handle))
        if rc != 0:
            raise NfaiError(rc, "nfai_tokenizer_create: malformed vocabulary or merges")
        self.handle = handle

    def close(self):
        if getattr(self, "handle", None):
            self._lib.nfai_tokenizer_destroy(self.handle)
            self.handle = None

    Dispose = close

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != 0:
            raise NfaiError(rc, self._lib.nfai_tokenizer_last_error(self.handle).decode("utf-8", "replace"))

    def _ids(self, call) -> List[int]:
        cap = 256
        while True:
            buf = (C.c_uint32 * cap)()
            n = C.c_size_t()
            rc = call(buf, cap, C.byref(n))
            if rc != 0 and n.value > cap:
                cap = n.value
                continue
            self._check(rc)
            return list(buf[:n.value])

    def encode(self, text: str) -> List[int]:
        """Text that already holds its special tokens (Tokenizer.cs:93-180)."""
        b = text.encode("utf-8")
        return self._ids(lambda buf, cap, n: self._lib.nfai_tokenizer_encode(self.handle, b, len(b), C.cast(buf, C.c_void_p), cap, n))

    def pretokenize_ends(self, text: str) -> List[int]:
        """End offsets (UTF-16 code units) of the pieces the pre-tokenisation pattern cuts `text` into (test tap)."""
        b = text.encode("utf-8")
        return self._ids(lambda buf, cap, n: self._lib.nfai_tokenizer_pretokenize(self.handle, b, len(b), C.cast(buf, C.c_void_p), cap, n))

    def tokenize(self, prompt: str, add_bos: bool = True) -> List[int]:
        """Tokenizer.Tokenize: the chat template around the user prompt (Tokenizer.cs:68-182)."""
        b = prompt.encode("utf-8")
        return self._ids(lambda buf, cap, n: self._lib.nfai_tokenizer_encode_chat(self.handle, b, len(b), 1 if add_bos else 0,
                                                                                  C.cast(buf, C.c_void_p), cap, n))

    Tokenize = tokenize

    def detokenize(self, ids: Sequence[int]) -> str:
        """Tokenizer.Detokenize (Tokenizer.cs:432-462)."""
        arr = (C.c_uint32 * len(ids))(*[int(i) for i in ids])
        cap = 64 + 16 * len(ids)
        while True:
            buf = C.create_string_buffer(cap)
            n = C.c_size_t()
            rc = self._lib.nfai_tokenizer_decode(self.handle, C.cast(arr, C.c_void_p), len(ids), C.cast(buf, C.c_void_p), cap, C.byref(n))
            if rc != 0 and n.value > cap:
                cap = n.value
                continue
            self._check(rc)
            return buf.raw[:n.value].decode("utf-8", errors="replace")

    Detokenize = detokenize
