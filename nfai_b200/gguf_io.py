"""GGUF reading (the subset the reference's parser accepts) and writing of synthetic models.

`Parser` mirrors NFAI.GGUF/Parser.cs: header and magic (:130-143), the 13 metadata value types including nested
arrays (:145-236), tensor infos with GGUF ne-order shapes (:244-307), data alignment (:32-33,125-128), then the
factory loop (:36-44). Tensor data stays in the file and is streamed on demand, as ComputeCollection does.
Only F32 and F16 tensors can be uploaded to the CUDA backend.
"""
from __future__ import annotations

import struct
from typing import BinaryIO, Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np

GGUF_MAGIC = 0x46554747  # "GGUF" little endian
GGML_F32, GGML_F16 = 0, 1
_TYPE_SIZE = {GGML_F32: 4, GGML_F16: 2}

# metadata value types
_U8, _I8, _U16, _I16, _U32, _I32, _F32, _BOOL, _STR, _ARR, _U64, _I64, _F64 = range(13)
_SCALAR = {_U8: "<B", _I8: "<b", _U16: "<H", _I16: "<h", _U32: "<I", _I32: "<i", _F32: "<f", _BOOL: "<?",
           _U64: "<Q", _I64: "<q", _F64: "<d"}


class ComputeCollection:
    """A lazy tensor: (file, offset, length, shape in ne order, element size).
    Mirrors NFAI.Core/ComputeCollection.cs:6-61 and AbstractComputeCollection.cs:36-79."""

    CHUNK_BYTES = 10 * 1024 * 1024  # AbstractComputeCollection.cs:39

    def __init__(self, name: str, shape: Sequence[int], type_size: int, *, path: Optional[str] = None,
                 offset: int = 0, array: Optional[np.ndarray] = None):
        self.Name = name
        self.Shape = tuple(int(s) for s in shape)
        self.TypeSize = int(type_size)
        self.Length = int(np.prod(self.Shape)) if self.Shape else 0
        self._path, self._offset, self._array = path, offset, array

    def get_data_raw(self, widen_half: bool = False) -> Iterator[bytes]:
        """File-order chunks of at most 10 MiB of source bytes. With widen_half=True halves are expanded to
        float32 first, which is what the reference's GetDataRaw yields (AbstractComputeCollection.cs:62-77)."""
        total = self.Length * self.TypeSize
        if self._array is not None:
            flat = np.ascontiguousarray(self._array).reshape(-1).view(np.uint8)
            reader = lambda o, n: flat[o:o + n].tobytes()  # noqa: E731
            fh = None
        else:
            fh = open(self._path, "rb")
            def reader(o, n, fh=fh):
                fh.seek(self._offset + o)
                return fh.read(n)
        try:
            cur = 0
            while cur < total:
                n = min(self.CHUNK_BYTES, total - cur)
                buf = reader(cur, n)
                if len(buf) != n:
                    raise IOError(f"tensor {self.Name}: short read")
                cur += n
                if widen_half and self.TypeSize == 2:
                    yield np.frombuffer(buf, dtype=np.float16).astype(np.float32).tobytes()
                else:
                    yield buf
        finally:
            if fh is not None:
                fh.close()

    def to_numpy(self) -> np.ndarray:
        dt = np.float16 if self.TypeSize == 2 else np.float32
        data = b"".join(self.get_data_raw())
        return np.frombuffer(data, dtype=dt).reshape(tuple(reversed(self.Shape)))


def _read(fh: BinaryIO, fmt: str):
    size = struct.calcsize(fmt)
    b = fh.read(size)
    if len(b) != size:
        raise IOError("unexpected end of GGUF file")
    return struct.unpack(fmt, b)[0]


def _read_str(fh: BinaryIO) -> str:
    n = _read(fh, "<Q")
    return fh.read(n).decode("utf-8", errors="replace")


def _read_value(fh: BinaryIO, vtype: int):
    if vtype in _SCALAR:
        return _read(fh, _SCALAR[vtype])
    if vtype == _STR:
        return _read_str(fh)
    if vtype == _ARR:
        etype = _read(fh, "<I")
        n = _read(fh, "<Q")
        return [_read_value(fh, etype) for _ in range(n)]
    raise ValueError(f"unknown GGUF metadata type {vtype}")


def read_gguf(path: str) -> Tuple[Dict[str, object], List[ComputeCollection]]:
    with open(path, "rb") as fh:
        if _read(fh, "<I") != GGUF_MAGIC:
            raise ValueError("not a GGUF file")
        version = _read(fh, "<I")
        if version < 2:
            raise ValueError(f"GGUF version {version} not supported")
        n_tensors = _read(fh, "<Q")
        n_kv = _read(fh, "<Q")
        meta: Dict[str, object] = {}
        for _ in range(n_kv):
            key = _read_str(fh)
            vtype = _read(fh, "<I")
            meta[key] = _read_value(fh, vtype)
        infos = []
        for _ in range(n_tensors):
            name = _read_str(fh)
            ndim = _read(fh, "<I")
            shape = [_read(fh, "<Q") for _ in range(ndim)]
            ggml_type = _read(fh, "<I")
            offset = _read(fh, "<Q")
            infos.append((name, shape, ggml_type, offset))
        alignment = int(meta.get("general.alignment", 32))
        pos = fh.tell()
        data_start = (pos + alignment - 1) // alignment * alignment
    tensors = []
    for name, shape, ggml_type, offset in infos:
        if ggml_type not in _TYPE_SIZE:
            raise ValueError(f"tensor {name}: ggml type {ggml_type} is not F32/F16")
        tensors.append(ComputeCollection(name, shape, _TYPE_SIZE[ggml_type], path=path, offset=data_start + offset))
    return meta, tensors


def write_synthetic_gguf(cfg, path: str, seed: int = 0) -> None:
    """Write the seeded synthetic model `cfg` as a GGUF file with the Python `gguf` writer."""
    import gguf

    from . import synth
    w = gguf.GGUFWriter(path, "llama")
    for key, val in synth.metadata(cfg).items():
        if key == "general.architecture":
            continue  # written by the GGUFWriter constructor
        if isinstance(val, str):
            w.add_string(key, val)
        elif isinstance(val, float):
            w.add_float32(key, val)
        else:
            w.add_uint32(key, int(val))
    for name, _ne, _dt, arr in synth.iter_tensors(cfg, seed):
        w.add_tensor(name, arr)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


class Parser:
    """Mirror of NFAI.GGUF/Parser.cs:17-45: Parser(factories).parse(options) -> IInferenceProvider."""

    def __init__(self, factories):
        self.factories = list(factories)
        self.Tokenizer = None  # Parser.cs:13: set by parse() when the file carries a vocabulary

    def parse(self, options):
        meta, tensors = read_gguf(options.GGUFPath)
        if "tokenizer.ggml.tokens" in meta and "tokenizer.ggml.bos_token_id" in meta:
            from .tokenizer import Tokenizer
            md = dict(meta)
            md.setdefault("tokenizer.ggml.merges", [])
            md.setdefault("tokenizer.ggml.eos_token_id", md["tokenizer.ggml.bos_token_id"])
            self.Tokenizer = Tokenizer(md)
        for f in self.factories:
            model = f.try_create(meta, tensors, options)
            if model is not None:
                return model
        raise RuntimeError("no model factory accepted this GGUF file")
