"""CPU restatement of the reference tokenizer (NFAI.Models.Llama3/Tokenizer.cs) -- TEST INFRASTRUCTURE ONLY.

It follows the reference literally, including what makes it slow: the merge search compares every adjacent pair of a
word with every entry of the merges list (Tokenizer.cs:130-166). Only the tests may import this module.
PARITY UNPINNED: the reference holds no tokenizer test vectors and cannot run here (no .NET); the pattern is evaluated
with the third-party `regex` module on UTF-16 code units, which is what System.Text.RegularExpressions sees.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import regex

# Tokenizer.cs:109-111
META = regex.compile(
    r"(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+")
# Tokenizer.cs:93-95
SPECIAL = regex.compile(r"<\|[^|>]+?\|>", regex.IGNORECASE)


def utf16_units(text: str) -> str:
    """The string as .NET sees it: one element per UTF-16 code unit (astral characters become two lone surrogates)."""
    out = []
    for ch in text:
        cp = ord(ch)
        if cp >= 0x10000:
            cp -= 0x10000
            out.append(chr(0xD800 + (cp >> 10)))
            out.append(chr(0xDC00 + (cp & 0x3FF)))
        else:
            out.append(ch)
    return "".join(out)


def unit_bytes(ch: str) -> bytes:
    """Encoding.UTF8.GetBytes(ch.ToString()): a lone surrogate becomes U+FFFD."""
    cp = ord(ch)
    if 0xD800 <= cp <= 0xDFFF:
        return b"\xef\xbf\xbd"
    return ch.encode("utf-8")


class OracleTokenizer:
    def __init__(self, tokens: Sequence[bytes], merges: Sequence[str], bos_id: int, eos_id: int, compiled: bool = False):
        """compiled=True runs the same merge loop in C++ (orc_bpe_merge_scan of the oracle library): the reference's
        algorithm at compiled speed, for timing; the Python loop below stays the readable statement of it."""
        self.compiled = compiled
        # Tokenizer.cs:50-57: a repeated byte string keeps the last id
        self.bytes_to_id: Dict[bytes, int] = {}
        self.id_to_bytes: Dict[int, bytes] = {}
        for i, t in enumerate(tokens):
            self.bytes_to_id[bytes(t)] = i
            self.id_to_bytes[i] = bytes(t)
        # Tokenizer.cs:32-40: split at the first space
        self.merges: List[Tuple[bytes, bytes]] = []
        for m in merges:
            sp = m.index(" ")
            self.merges.append((m[:sp].encode("utf-8"), m[sp + 1:].encode("utf-8")))
        self.bos_id, self.eos_id = bos_id, eos_id
        if compiled:
            import ctypes as C

            import numpy as np

            from . import oracle as _o
            self._C, self._np = C, np
            self._lib = _o.lib()
            self._lib.orc_bpe_merge_scan.restype = C.c_uint32
            self._lib.orc_bpe_merge_scan.argtypes = [C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p]
            flat = bytearray()
            offs = [0]
            for a, b in self.merges:
                flat += a
                offs.append(len(flat))
                flat += b
                offs.append(len(flat))
            self._merge_bytes = np.frombuffer(bytes(flat) or b"\0", np.uint8).copy()
            self._merge_off = np.array(offs, np.uint64)

    def _merge_compiled(self, parts: List[bytes]) -> List[bytes]:
        np, C = self._np, self._C
        flat = b"".join(parts)
        offs = np.zeros(len(parts) + 1, np.uint32)
        offs[1:] = np.cumsum([len(p) for p in parts])
        data = np.frombuffer(flat or b"\0", np.uint8).copy()
        out = np.zeros(len(parts) + 1, np.uint32)
        n = self._lib.orc_bpe_merge_scan(data.ctypes.data_as(C.c_void_p), offs.ctypes.data_as(C.c_void_p), len(parts),
                                         self._merge_bytes.ctypes.data_as(C.c_void_p), self._merge_off.ctypes.data_as(C.c_void_p),
                                         len(self.merges), out.ctypes.data_as(C.c_void_p))
        return [flat[int(out[i]):int(out[i + 1])] for i in range(n)]

    # Tokenizer.cs:242-267
    @staticmethod
    def initial_units(s: str) -> List[bytes]:
        out = []
        for ch in s:
            if ch in (" ", "\n"):
                b = bytearray(ch.encode("utf-8"))
                b[-1] = (b[-1] + (0x8A - 0x0A)) & 0xFF
                out.append(bytes([0xC4]) + bytes(b))
            else:
                out.append(unit_bytes(ch))
        return out

    # Tokenizer.cs:115-180
    def encode(self, template: str) -> List[int]:
        template = utf16_units(template)
        specials = list(SPECIAL.finditer(template))
        ids: List[int] = []
        for i, m in enumerate(specials):
            nxt = specials[i + 1].start() if i + 1 < len(specials) else len(template)
            special = m.group(0).encode("utf-8")
            if special not in self.bytes_to_id:
                raise KeyError(m.group(0))
            ids.append(self.bytes_to_id[special])
            text = template[m.end():nxt]
            for w in META.finditer(text):
                parts = self.initial_units(w.group(0))
                if self.compiled:
                    parts = self._merge_compiled(parts)
                while not self.compiled:
                    best_merge, best_first = -1, -1
                    for j in range(len(parts) - 1):
                        left, right = parts[j], parts[j + 1]
                        for k, (a, b) in enumerate(self.merges):
                            if left == a and right == b:
                                if best_merge == -1 or k < best_merge:
                                    best_merge, best_first = k, j
                                break
                    if best_merge == -1:
                        break
                    parts[best_first] = parts[best_first] + parts[best_first + 1]
                    del parts[best_first + 1]
                for p in parts:
                    if p not in self.bytes_to_id:
                        raise KeyError(p)
                    ids.append(self.bytes_to_id[p])
        return ids

    # Tokenizer.cs:68-91
    def tokenize(self, prompt: str, add_bos: bool = True) -> List[int]:
        system_prompt = "You are a helpful assistant."
        if add_bos:
            template = ("<|begin_of_text|><|start_header_id|>system<|end_header_id|>\n\n" + system_prompt +
                        "<|eot_id|><|start_header_id|>user<|end_header_id|>\n\n" + prompt +
                        "<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n")
        else:
            template = ("\n\n<|start_header_id|>user<|end_header_id|>\n\n" + prompt +
                        "<|eot_id|><|start_header_id|>assistant<|end_header_id|>\n\n")
        return self.encode(template.replace("\r", ""))

    # Tokenizer.cs:432-462
    def detokenize(self, ids: Sequence[int]) -> str:
        data = b"".join(self.id_to_bytes[i] for i in ids)
        return data.decode("utf-8", errors="replace").replace("Ġ", " ").replace("Ċ", "\n")
