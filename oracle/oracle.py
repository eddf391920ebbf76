"""ctypes wrapper over the CPU oracle (libnfai_oracle.so) -- TEST INFRASTRUCTURE ONLY.

The oracle is the checker for the CUDA library. Only the tests, the smoke check and the CPU-baseline /
reference legs of the benchmark may import this module; the product package never does.
PARITY UNPINNED: the reference holds no golden vectors for this path and cannot run here; see the header of
nfai_oracle.cpp.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libnfai_oracle.so")


class OrcHParams(C.Structure):
    _fields_ = [
        ("H", C.c_uint32), ("L", C.c_uint32), ("qH", C.c_uint32), ("kvH", C.c_uint32), ("d", C.c_uint32),
        ("ropeDim", C.c_uint32), ("F", C.c_uint32), ("V", C.c_uint32), ("ctx", C.c_uint32),
        ("eps", C.c_float), ("rope_theta", C.c_float), ("mode", C.c_int32),
    ]


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside it (g++ only; seconds)."""
    src = os.path.join(_HERE, "nfai_oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libnfai_oracle.so"], check=True, capture_output=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    build()
    try:
        L = C.CDLL(_SO)
    except OSError:
        build(force=True)
        L = C.CDLL(_SO)
    fp = C.POINTER(C.c_float)
    L.orc_create.restype = C.c_void_p
    L.orc_create.argtypes = [C.POINTER(OrcHParams)]
    L.orc_destroy.argtypes = [C.c_void_p]
    L.orc_last_error.restype = C.c_char_p
    L.orc_last_error.argtypes = [C.c_void_p]
    L.orc_set_tensor.argtypes = [C.c_void_p, C.c_char_p, C.c_int, C.c_void_p, C.c_uint64]
    L.orc_set_threads.argtypes = [C.c_int]
    L.orc_max_threads.restype = C.c_int
    L.orc_reset.argtypes = [C.c_void_p]
    L.orc_position.restype = C.c_uint32
    L.orc_position.argtypes = [C.c_void_p]
    L.orc_set_position.argtypes = [C.c_void_p, C.c_uint32]
    L.orc_set_mode.argtypes = [C.c_void_p, C.c_int]
    L.orc_argmax.restype = C.c_uint32
    L.orc_argmax.argtypes = [fp, C.c_uint64]
    L.orc_decode.argtypes = [C.c_void_p, C.c_uint32, fp]
    L.orc_read_kv.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, fp, fp]
    L.orc_write_kv.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, fp, fp]
    L.orc_read_hidden.argtypes = [C.c_void_p, C.c_uint32, fp]
    L.orc_read_attn.argtypes = [C.c_void_p, C.c_uint32, fp, fp]
    L.orc_op_half_to_float.argtypes = [C.c_void_p, fp, C.c_uint64]
    L.orc_op_rmsnorm.argtypes = [fp, fp, C.c_uint32, C.c_float, fp, C.c_int]
    L.orc_op_matvec.argtypes = [fp, C.c_void_p, C.c_int, C.c_uint64, C.c_uint64, fp, C.c_int]
    L.orc_op_rope.argtypes = [fp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_uint32]
    L.orc_op_rope_table.argtypes = [C.c_uint32, C.c_float, fp]
    L.orc_op_attention.argtypes = [fp, fp, fp, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, fp,
                                   C.c_int]
    L.orc_op_silu_mul.argtypes = [fp, fp, C.c_uint32, fp]
    L.orc_sample_top_p.restype = C.c_uint32
    L.orc_sample_top_p.argtypes = [fp, C.c_uint64, C.c_float, C.c_float, C.c_int, C.c_float]
    _lib = L
    return L


def _fp(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.POINTER(C.c_float))


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


class OracleModel:
    """The whole forward path on the CPU: feed token ids, read logits (and taps)."""

    def __init__(self, cfg, ctx: int, mode: int = 0):
        self.cfg = cfg
        self.ctx = ctx
        hp = OrcHParams(cfg.H, cfg.L, cfg.qH, cfg.kvH, cfg.d, cfg.ropeDim, cfg.F, cfg.V, ctx, cfg.eps,
                        cfg.rope_theta, mode)
        self._h = lib().orc_create(C.byref(hp))
        if not self._h:
            raise ValueError("orc_create rejected the hyper-parameters")

    def close(self):
        if self._h:
            lib().orc_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc: int):
        if rc != 0:
            raise RuntimeError(f"oracle error {rc}: {lib().orc_last_error(self._h).decode()}")

    def set_tensor(self, name: str, arr: np.ndarray):
        arr = np.ascontiguousarray(arr)
        if arr.dtype == np.float32:
            dt = 0
        elif arr.dtype == np.float16:
            dt = 1
        else:
            raise TypeError(arr.dtype)
        self._check(lib().orc_set_tensor(self._h, name.encode(), dt, arr.ctypes.data_as(C.c_void_p), arr.size))

    def load_synthetic(self, seed: int = 0):
        from nfai_b200 import synth
        for name, _ne, _dt, arr in synth.iter_tensors(self.cfg, seed):
            self.set_tensor(name, arr)
        return self

    def set_mode(self, mode: int):
        lib().orc_set_mode(self._h, mode)

    def reset(self):
        lib().orc_reset(self._h)

    @property
    def position(self) -> int:
        return lib().orc_position(self._h)

    def set_position(self, pos: int):
        lib().orc_set_position(self._h, pos)

    def decode(self, token: int, want_logits: bool = True) -> Optional[np.ndarray]:
        if want_logits:
            out = np.empty(self.cfg.V, dtype=np.float32)
            self._check(lib().orc_decode(self._h, int(token), _fp(out)))
            return out
        self._check(lib().orc_decode(self._h, int(token), None))
        return None

    def prefill(self, tokens) -> np.ndarray:
        """Token by token, as the reference ingests a prompt (NFAI.Models.Llama3/LlamaModel.cs:103-126);
        returns the last token's logits."""
        toks = list(tokens)
        for t in toks[:-1]:
            self.decode(int(t), want_logits=False)
        return self.decode(int(toks[-1]))

    def read_kv(self, layer: int, pos: int):
        kvDim = self.cfg.kvDim
        k = np.empty(kvDim, np.float32)
        v = np.empty(kvDim, np.float32)
        self._check(lib().orc_read_kv(self._h, layer, pos, _fp(k), _fp(v)))
        return k, v

    def write_kv(self, layer: int, pos: int, k: np.ndarray, v: np.ndarray):
        self._check(lib().orc_write_kv(self._h, layer, pos, _fp(_f32(k)), _fp(_f32(v))))

    def read_hidden(self, layer: int) -> np.ndarray:
        out = np.empty(self.cfg.H, np.float32)
        self._check(lib().orc_read_hidden(self._h, layer, _fp(out)))
        return out

    def read_attn(self, layer: int):
        q = np.empty(self.cfg.qDim, np.float32)
        o = np.empty(self.cfg.qDim, np.float32)
        self._check(lib().orc_read_attn(self._h, layer, _fp(q), _fp(o)))
        return q, o


def argmax(v: np.ndarray) -> int:
    v = _f32(v)
    return int(lib().orc_argmax(_fp(v), v.size))


def set_threads(n: int):
    lib().orc_set_threads(n)


def max_threads() -> int:
    return lib().orc_max_threads()


# ---- stand-alone operators ---------------------------------------------------------------------------------

def half_to_float(a: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float16)
    out = np.empty(a.shape, np.float32)
    lib().orc_op_half_to_float(a.ctypes.data_as(C.c_void_p), _fp(out), a.size)
    return out


def rmsnorm(x, g, eps: float, mode: int = 0) -> np.ndarray:
    x, g = _f32(x), _f32(g)
    y = np.empty_like(x)
    lib().orc_op_rmsnorm(_fp(x), _fp(g), x.size, eps, _fp(y), mode)
    return y


def matvec(x, W: np.ndarray, mode: int = 0) -> np.ndarray:
    """y = W x with W[N][K] row-major in float32 or float16."""
    x = _f32(x)
    W = np.ascontiguousarray(W)
    N, K = W.shape
    assert x.size == K
    dt = 0 if W.dtype == np.float32 else 1
    assert W.dtype in (np.float32, np.float16)
    y = np.empty(N, np.float32)
    lib().orc_op_matvec(_fp(x), W.ctypes.data_as(C.c_void_p), dt, K, N, _fp(y), mode)
    return y


def rope(v, heads: int, d: int, rope_dim: int, theta_base: float, pos: int) -> np.ndarray:
    out = _f32(v).copy()
    lib().orc_op_rope(_fp(out), heads, d, rope_dim, theta_base, pos)
    return out


def rope_table(rope_dim: int, theta_base: float) -> np.ndarray:
    out = np.empty(rope_dim // 2, np.float32)
    lib().orc_op_rope_table(rope_dim, theta_base, _fp(out))
    return out


def attention(q, kc, vc, seq: int, qH: int, kvH: int, d: int, eps: float, mode: int = 0) -> np.ndarray:
    """q[qH*d]; kc, vc [>=seq][kvH*d] position-major float32."""
    q, kc, vc = _f32(q), _f32(kc), _f32(vc)
    out = np.empty(qH * d, np.float32)
    lib().orc_op_attention(_fp(q), _fp(kc), _fp(vc), seq, qH, kvH, d, eps, _fp(out), mode)
    return out


def silu_mul(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    h = np.empty_like(gate)
    lib().orc_op_silu_mul(_fp(gate), _fp(up), gate.size, _fp(h))
    return h


def sample_top_p(logits, temperature: float = 0.5, top_p: float = 0.95, top_k: int = 40, u: float = 0.5) -> int:
    """NFAI.Models.Llama3/SamplingUtils.cs:5-33 with the uniform random number `u` supplied by the caller."""
    logits = _f32(logits)
    return int(lib().orc_sample_top_p(_fp(logits), logits.size, temperature, top_p, top_k, u))
