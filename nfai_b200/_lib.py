"""ctypes binding of libnfai_cuda.so (the C ABI declared in include/nfai_cuda.h).

There is no CPU fallback: if the library is missing or does not load, importing the symbols raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libnfai_cuda.so")

OK = 0
ERR_ARG, ERR_STATE, ERR_OOM, ERR_CUDA, ERR_NCCL, ERR_CONTEXT_FULL, ERR_TIMEOUT = 1, 2, 3, 4, 5, 6, 7
F32, F16 = 0, 1

ERROR_NAMES = {
    ERR_ARG: "NFAI_ERR_ARG", ERR_STATE: "NFAI_ERR_STATE", ERR_OOM: "NFAI_ERR_OOM", ERR_CUDA: "NFAI_ERR_CUDA",
    ERR_NCCL: "NFAI_ERR_NCCL", ERR_CONTEXT_FULL: "NFAI_ERR_CONTEXT_FULL", ERR_TIMEOUT: "NFAI_ERR_TIMEOUT",
}


class HParams(C.Structure):
    _fields_ = [
        ("H", C.c_uint32), ("L", C.c_uint32), ("qH", C.c_uint32), ("kvH", C.c_uint32), ("d", C.c_uint32),
        ("ropeDim", C.c_uint32), ("F", C.c_uint32), ("V", C.c_uint32), ("ctx", C.c_uint32),
        ("eps", C.c_float), ("rope_theta", C.c_float),
        ("weight_dtype", C.c_int32), ("kv_dtype", C.c_int32), ("tied", C.c_int32),
    ]


class NfaiError(RuntimeError):
    """A failed library call; `.code` is the NFAI_ERR_* status (the C# shim throws InvalidOperationException)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{ERROR_NAMES.get(code, code)}: {message}")
        self.code = code


# name -> (restype, argtypes); every symbol include/nfai_cuda.h declares
_vp, _u32, _i, _f, _sz = C.c_void_p, C.c_uint32, C.c_int, C.c_float, C.c_size_t
_pp = C.POINTER(C.c_void_p)
SIGNATURES = {
    "nfai_version": (C.c_char_p, []),
    "nfai_last_error": (C.c_char_p, [_vp]),
    "nfai_ctx_create": (_i, [_i, _pp]),
    "nfai_tp_unique_id": (_i, [_vp, _sz]),
    "nfai_ctx_create_tp": (_i, [_i, _i, _i, _vp, _sz, _pp]),
    "nfai_tp_export_peer": (_i, [_vp, _vp, _sz]),
    "nfai_tp_import_peers": (_i, [_vp, _vp, _i]),
    "nfai_ctx_destroy": (_i, [_vp]),
    "nfai_ctx_set_wait_ns": (_i, [_vp, C.c_uint64]),
    "nfai_op_xchg_area_bytes": (_sz, []),
    "nfai_op_gemv_xchg": (_i, [_vp, _vp, _i, _u32, _u32, _vp, _vp, _f, _vp, _pp, _i, _i, _u32, _vp, _vp, _u32, C.c_uint64]),
    "nfai_op_lm_head_xchg": (_i, [_vp, _vp, _i, _vp, _vp, _f, _u32, _u32, _u32, _vp, _pp, _i, _i, _u32, _i, _i, _vp,
                                  C.c_uint64]),
    "nfai_model_create": (_i, [_vp, C.POINTER(HParams), _pp]),
    "nfai_model_tensor_begin": (_i, [_vp, C.c_char_p, _i, C.POINTER(C.c_uint64), _i]),
    "nfai_model_tensor_chunk": (_i, [_vp, _vp, _sz]),
    "nfai_model_tensor_end": (_i, [_vp]),
    "nfai_model_finalize": (_i, [_vp]),
    "nfai_model_load_gguf": (_i, [_vp, C.c_char_p, _u32, _i, _pp]),
    "nfai_gguf_probe": (_i, [C.c_char_p, _u32, C.POINTER(HParams), C.c_char_p, _sz]),
    "nfai_model_get_hparams": (_i, [_vp, C.POINTER(HParams)]),
    "nfai_model_destroy": (_i, [_vp]),
    "nfai_prefill": (_i, [_vp, C.POINTER(_u32), _i, C.POINTER(_f), C.POINTER(_u32)]),
    "nfai_decode": (_i, [_vp, _u32, C.POINTER(_f), C.POINTER(_u32)]),
    "nfai_decode_greedy": (_i, [_vp, _u32, _i, C.POINTER(_u32), C.POINTER(_f)]),
    "nfai_decode_sampled": (_i, [_vp, _u32, _i, _f, _f, _i, _vp, _vp, C.POINTER(_f)]),
    "nfai_sample_top_p": (_i, [_vp, _f, _f, _i, _f, C.POINTER(_u32)]),
    "nfai_op_sample_top_p": (_i, [_vp, _vp, _u32, _f, _f, _i, _f, _vp]),
    "nfai_kv_snapshot_create": (_i, [_vp, _pp]),
    "nfai_kv_snapshot_restore": (_i, [_vp, _vp]),
    "nfai_kv_snapshot_destroy": (None, [_vp]),
    "nfai_kv_snapshot_position": (_u32, [_vp]),
    "nfai_tokenizer_create": (_i, [_vp, _vp, _u32, _vp, _vp, _u32, _u32, _u32, _pp]),
    "nfai_tokenizer_destroy": (None, [_vp]),
    "nfai_tokenizer_last_error": (C.c_char_p, [_vp]),
    "nfai_tokenizer_encode": (_i, [_vp, C.c_char_p, _sz, _vp, _sz, C.POINTER(_sz)]),
    "nfai_tokenizer_encode_chat": (_i, [_vp, C.c_char_p, _sz, _i, _vp, _sz, C.POINTER(_sz)]),
    "nfai_tokenizer_pretokenize": (_i, [_vp, C.c_char_p, _sz, _vp, _sz, C.POINTER(_sz)]),
    "nfai_tokenizer_decode": (_i, [_vp, _vp, _sz, _vp, _sz, C.POINTER(_sz)]),
    "nfai_position": (_i, [_vp, C.POINTER(_u32)]),
    "nfai_reset": (_i, [_vp]),
    "nfai_read_kv": (_i, [_vp, _u32, _u32, C.POINTER(_f), C.POINTER(_f)]),
    "nfai_write_kv": (_i, [_vp, _u32, _u32, C.POINTER(_f), C.POINTER(_f)]),
    "nfai_write_kv_range": (_i, [_vp, _u32, _u32, _u32, C.POINTER(_f), C.POINTER(_f)]),
    "nfai_set_position": (_i, [_vp, _u32]),
    "nfai_read_hidden": (_i, [_vp, _u32, C.POINTER(_f)]),
    "nfai_profile_kernel": (_i, [_vp, _i, _i, C.POINTER(_f), C.POINTER(C.c_uint64)]),
    "nfai_model_tune": (_i, [_vp, _i, _i, _i, _i, _i]),
    "nfai_model_set_prefetch": (_i, [_vp, C.c_uint64, C.c_uint64, _i]),
    "nfai_step_launches": (_i, [_vp, C.POINTER(_i)]),
    "nfai_op_embed": (_i, [_vp, _vp, _i, _u32, _u32, _u32, _vp]),
    "nfai_op_gemv": (_i, [_vp, _vp, _i, _u32, _u32, _vp, _vp, _f, _vp, _vp]),
    "nfai_op_qkv_rope": (_i, [_vp, _vp, _i, _vp, _vp, _f, _u32, _u32, _u32, _u32, _u32, _vp, _u32, _vp, _vp, _vp, _i]),
    "nfai_op_ffn_gate_up": (_i, [_vp, _vp, _i, _vp, _vp, _f, _u32, _u32, _vp]),
    "nfai_op_attn_decode": (_i, [_vp, _vp, _vp, _vp, _i, _u32, _u32, _u32, _u32, _vp, _vp, _sz]),
    "nfai_op_attn_scratch_bytes": (_sz, [_u32, _u32, _u32, _u32]),
    "nfai_op_attn_decode_static": (_i, [_vp, _vp, _vp, _vp, _i, _u32, _u32, _u32, _u32, _vp]),
    "nfai_op_gemm_f16": (_i, [_vp, _vp, _vp, _u32, _u32, _u32, _vp]),
    "nfai_op_lm_head": (_i, [_vp, _vp, _i, _vp, _vp, _f, _u32, _u32, _vp, _vp]),
}

_lib = None


def load() -> C.CDLL:
    """Load the library and bind every declared symbol; raises if anything is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m nfai_b200.build` (needs nvcc); there is no fallback path")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc: int, ctx_handle=None):
    if rc != OK:
        msg = load().nfai_last_error(ctx_handle)
        raise NfaiError(rc, msg.decode() if msg else "")
