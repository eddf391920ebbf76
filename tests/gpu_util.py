"""Helpers for the GPU parity tests: device buffers come from torch, every compute call goes through the C ABI."""
import ctypes as C

import numpy as np
import torch

from nfai_b200 import _lib


def dev(a: np.ndarray) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    torch.cuda.synchronize()
    return t


def ptr(t) -> C.c_void_p:
    return C.c_void_p(t.data_ptr()) if t is not None else None


def host(t: torch.Tensor) -> np.ndarray:
    torch.cuda.synchronize()
    return t.cpu().numpy()


def call(ctx, fn_name, *args):
    lib = _lib.load()
    torch.cuda.synchronize()
    rc = getattr(lib, fn_name)(ctx.handle, *args)
    _lib.check(rc, ctx.handle)


def dtype_code(np_dtype) -> int:
    return _lib.F16 if np.dtype(np_dtype) == np.float16 else _lib.F32


def rel_err(got, want) -> float:
    return float(np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64)).max()
                 / max(np.abs(want).max(), 1e-30))
