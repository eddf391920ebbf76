"""nfai_op_attn_decode_static: attention for callers that cannot allocate device memory.

Some hosts of this library run attention at a point where they may not call cudaMalloc (a fixed device-memory
budget already spent, or a per-token loop that cannot afford the device-wide synchronisation an allocation implies).
For them the library carries a 256 KiB scratch array of its own. This test calls that entry point through the C ABI
twice in a row, with different sequence lengths so that the second call finds the first call's leftovers in the
shared array, and checks each result against nfai_op_attn_decode (caller-owned scratch) on the same inputs.
The file name makes pytest collect it last.
"""
import ctypes as C

import numpy as np
import pytest

from nfai_b200 import _lib

from .gpu_util import call, dev, host, ptr, rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TOL = 1e-4  # the tolerance of the kernel-level parity tests


def run_both(cuda_ctx, qH, kvH, d, seq, kvdtype, seed):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal(qH * d).astype(np.float32)
    kc = rng.standard_normal((seq, kvH * d)).astype(kvdtype)
    vc = rng.standard_normal((seq, kvH * d)).astype(kvdtype)
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    code = _lib.F16 if kvdtype == np.float16 else _lib.F32
    lib = _lib.load()
    nbytes = lib.nfai_op_attn_scratch_bytes(qH, kvH, d, seq)
    scratch = torch.zeros(nbytes // 4 + 1, dtype=torch.float32, device="cuda")
    want = torch.empty(qH * d, dtype=torch.float32, device="cuda")
    call(cuda_ctx, "nfai_op_attn_decode", ptr(dq), ptr(dk), ptr(dv), code, seq, qH, kvH, d, ptr(want), ptr(scratch),
         C.c_size_t(nbytes))
    got = torch.full((qH * d,), float("nan"), dtype=torch.float32, device="cuda")
    call(cuda_ctx, "nfai_op_attn_decode_static", ptr(dq), ptr(dk), ptr(dv), code, seq, qH, kvH, d, ptr(got))
    return host(got), host(want), (q, kc, vc)


def test_static_scratch_matches_caller_scratch_twice_in_a_row(cuda_ctx, oracle):
    # first call: long enough to split the range over several CTAs (partials + tickets in the static array)
    got, want, _ = run_both(cuda_ctx, 32, 8, 64, 5000, np.float16, 1)
    assert np.isfinite(got).all() and rel_err(got, want) < TOL
    # second call straight after: other geometry, other split count, leftovers of the first call in the array
    got, want, (q, kc, vc) = run_both(cuda_ctx, 24, 8, 128, 1700, np.float32, 2)
    assert np.isfinite(got).all() and rel_err(got, want) < TOL
    # the same result against the CPU restatement of the reference's three attention shaders
    ref = oracle.attention(q, kc.astype(np.float32), vc.astype(np.float32), 1700, 24, 8, 128, 1e-5)
    assert rel_err(got, ref) < TOL
    # and a short one that does not split at all
    got, want, _ = run_both(cuda_ctx, 8, 2, 32, 40, np.float32, 3)
    assert rel_err(got, want) < TOL


def test_static_scratch_rejects_what_it_cannot_hold(cuda_ctx):
    qH, kvH, d, seq = 32, 8, 128, 20000  # 32 heads x 18 splits x 130 floats = 300 KB: beyond the built-in 256 KiB
    lib = _lib.load()
    assert lib.nfai_op_attn_scratch_bytes(qH, kvH, d, seq) > (256 << 10)
    buf = torch.zeros(16, dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.NfaiError) as e:
        call(cuda_ctx, "nfai_op_attn_decode_static", ptr(buf), ptr(buf), ptr(buf), _lib.F32, seq, qH, kvH, d, ptr(buf))
    assert e.value.code == _lib.ERR_ARG and "256 KiB" in str(e.value)


def test_static_scratch_limit_is_where_the_header_says(cuda_ctx):
    """32 query heads of dimension 128: 7 680 positions still fit the built-in array, 7 681 do not."""
    lib = _lib.load()
    assert lib.nfai_op_attn_scratch_bytes(32, 8, 128, 7680) <= (256 << 10) < lib.nfai_op_attn_scratch_bytes(32, 8, 128, 7681)
    got, want, _ = run_both(cuda_ctx, 32, 8, 128, 7680, np.float16, 4)
    assert np.isfinite(got).all() and rel_err(got, want) < TOL
    buf = torch.zeros(16, dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.NfaiError) as e:
        call(cuda_ctx, "nfai_op_attn_decode_static", ptr(buf), ptr(buf), ptr(buf), _lib.F16, 7681, 32, 8, 128, ptr(buf))
    assert e.value.code == _lib.ERR_ARG
