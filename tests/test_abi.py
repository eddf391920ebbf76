"""The C-ABI library loads without a GPU and exports every symbol include/nfai_cuda.h declares."""
import ctypes as C
import os
import re

import pytest

from nfai_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "nfai_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nfai_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared_symbols()
    for must in ("nfai_ctx_create", "nfai_model_create", "nfai_model_tensor_begin", "nfai_model_tensor_chunk",
                 "nfai_model_tensor_end", "nfai_model_finalize", "nfai_prefill", "nfai_decode", "nfai_decode_greedy",
                 "nfai_last_error", "nfai_model_destroy", "nfai_ctx_destroy"):
        assert must in names


def test_library_exports_every_declared_symbol():
    lib = C.CDLL(_lib.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_binding_covers_every_declared_symbol():
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    _lib.load()


def test_calls_without_a_gpu_fail_with_a_status_not_a_crash():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = _lib.load()
    h = C.c_void_p()
    rc = lib.nfai_ctx_create(0, C.byref(h))
    assert rc != _lib.OK and not h.value
    assert lib.nfai_last_error(None)
    assert lib.nfai_version().startswith(b"nfai_cuda")
    # null handles are argument errors, never a crash
    assert lib.nfai_decode(None, 0, None, None) == _lib.ERR_ARG
    assert lib.nfai_model_finalize(None) == _lib.ERR_ARG
    assert lib.nfai_ctx_destroy(None) == _lib.OK
    assert lib.nfai_op_attn_scratch_bytes(32, 8, 64, 4096) > 0
    assert lib.nfai_op_attn_scratch_bytes(0, 8, 64, 4096) == 0
