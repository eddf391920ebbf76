"""The tensor-parallel exchange on ONE GPU: the kernels that push partial rows into every rank's exchange area and
the kernels that pull the sum are run rank after rank over areas that all sit in this GPU's memory, and compared with
the CPU oracle's unsharded arithmetic. A pull whose peer never publishes must end with NFAI_ERR_TIMEOUT, and the
context must work afterwards. Nothing here waits on another launch: every flag is either already set or never set.
"""
import ctypes as C

import numpy as np
import pytest

from nfai_b200 import _lib

from .gpu_util import call, dev, dtype_code, host, ptr, rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TOL = 1e-4


def make_areas(world):
    lib = _lib.load()
    nbytes = lib.nfai_op_xchg_area_bytes()
    bufs = [torch.zeros(nbytes // 4 + 64, dtype=torch.float32, device="cuda") for _ in range(world)]
    arr = (C.c_void_p * world)()
    for r, b in enumerate(bufs):
        base = (b.data_ptr() + 255) // 256 * 256
        arr[r] = base
    return bufs, arr


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_row_parallel_push_then_pull_matches_the_unsharded_oracle(cuda_ctx, oracle, world, dtype):
    """down projection split by input columns over `world` ranks, sum + residual pulled by a normalising GEMV."""
    rng = np.random.default_rng(world * 11 + (dtype == np.float16))
    H, F, N2 = 256, 512 * world, 96
    Wd = (rng.standard_normal((H, F)) * 0.05).astype(dtype)          # row-parallel matrix, unsharded
    h = rng.standard_normal(F).astype(np.float32)
    resid = rng.standard_normal(H).astype(np.float32)
    W2 = (rng.standard_normal((N2, H)) * 0.05).astype(dtype)         # the consumer (stands for QKV / gate-up)
    gain = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    eps = 1e-5
    bufs, areas = make_areas(world)
    Fl = F // world
    for epoch in (1, 2, 3):  # three exchanges in a row over the same areas: both parities and a reuse
        hh = h * epoch
        for r in range(world):
            dW = dev(np.ascontiguousarray(Wd[:, r * Fl:(r + 1) * Fl]))
            dx = dev(hh[r * Fl:(r + 1) * Fl])
            call(cuda_ctx, "nfai_op_gemv_xchg", ptr(dW), dtype_code(dtype), H, Fl, ptr(dx), None, C.c_float(0), None,
                 areas, world, r, 0, None, None, epoch, 0)
        # oracle: per-rank partials in float32, summed in rank order, then the residual
        total = np.zeros(H, np.float32)
        for r in range(world):
            total = total + oracle.matvec(hh[r * Fl:(r + 1) * Fl], Wd[:, r * Fl:(r + 1) * Fl].astype(np.float32))
        x_want = resid + total
        y_want = oracle.matvec(oracle.rmsnorm(x_want, gain, eps), W2.astype(np.float32))
        stores = []
        for r in range(world):
            dres, dW2, dg = dev(resid), dev(W2), dev(gain)
            store = torch.zeros(H, dtype=torch.float32, device="cuda")
            y = torch.zeros(N2, dtype=torch.float32, device="cuda")
            call(cuda_ctx, "nfai_op_gemv_xchg", ptr(dW2), dtype_code(dtype), N2, H, None, ptr(dg), C.c_float(eps), ptr(y),
                 areas, world, r, epoch, ptr(dres), ptr(store), 0, 0)
            stores.append(host(store))
            assert rel_err(host(y), y_want) < TOL
            assert rel_err(stores[-1], x_want) < 1e-5
        for r in range(1, world):
            assert np.array_equal(stores[r], stores[0])  # every rank holds the bit-identical residual stream


def test_vocabulary_sharded_argmax_pairs(cuda_ctx, oracle):
    rng = np.random.default_rng(3)
    world, H, V = 4, 128, 1024
    W = (rng.standard_normal((V, H)) * 0.05).astype(np.float32)
    W[900] = W[37]  # equal maxima candidates in different shards: the lower global index must win
    x = rng.standard_normal(H).astype(np.float32)
    gain = np.ones(H, np.float32)
    logits = oracle.matvec(oracle.rmsnorm(x, gain, 1e-5), W)
    best = int(np.argmax(logits))
    if best in (37, 900):
        best = 37
    bufs, areas = make_areas(world)
    Vl = V // world
    dx, dg = dev(x), dev(gain)
    for r in range(world):
        dW = dev(np.ascontiguousarray(W[r * Vl:(r + 1) * Vl]))
        lg = torch.zeros(Vl, dtype=torch.float32, device="cuda")
        call(cuda_ctx, "nfai_op_lm_head_xchg", ptr(dW), _lib.F32, ptr(dx), ptr(dg), C.c_float(1e-5), H, Vl, r * Vl,
             ptr(lg), areas, world, r, 1, 1, 0, None, 0)
        assert rel_err(host(lg), logits[r * Vl:(r + 1) * Vl]) < TOL
    for r in range(world):
        am = torch.zeros(1, dtype=torch.int32, device="cuda")
        call(cuda_ctx, "nfai_op_lm_head_xchg", None, _lib.F32, None, None, C.c_float(0), 0, 0, 0, None, areas, world, r,
             1, 0, 1, ptr(am), 0)
        assert int(host(am)[0]) == oracle.argmax(logits) == best


def test_a_pull_without_its_peer_times_out_and_the_context_survives(cuda_ctx, oracle):
    """Rank 1 of 2 never publishes exchange 1: rank 0's pull gives up after 2 ms with NFAI_ERR_TIMEOUT (the kernel
    returns by itself), leaves the residual store untouched, and the next calls on the context succeed."""
    rng = np.random.default_rng(9)
    H, N = 256, 64
    W = (rng.standard_normal((N, H)) * 0.05).astype(np.float32)
    resid = rng.standard_normal(H).astype(np.float32)
    bufs, areas = make_areas(2)
    dW, dres = dev(W), dev(resid)
    part = rng.standard_normal(H).astype(np.float32)
    Wid = np.eye(H, dtype=np.float32)
    dI, dp = dev(Wid), dev(part)
    # rank 0 pushes its part (identity matrix: the pushed rows are `part`); rank 1 stays silent
    call(cuda_ctx, "nfai_op_gemv_xchg", ptr(dI), _lib.F32, H, H, ptr(dp), None, C.c_float(0), None, areas, 2, 0, 0, None,
         None, 1, 0)
    store = torch.full((H,), 7.0, dtype=torch.float32, device="cuda")
    y = torch.zeros(N, dtype=torch.float32, device="cuda")
    with pytest.raises(_lib.NfaiError) as e:
        call(cuda_ctx, "nfai_op_gemv_xchg", ptr(dW), _lib.F32, N, H, None, None, C.c_float(0), ptr(y), areas, 2, 0, 1,
             ptr(dres), ptr(store), 0, 2_000_000)
    assert e.value.code == _lib.ERR_TIMEOUT
    assert np.all(host(store) == 7.0)
    # the same for the pair exchange
    am = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.NfaiError) as e:
        call(cuda_ctx, "nfai_op_lm_head_xchg", None, _lib.F32, None, None, C.c_float(0), 0, 0, 0, None, areas, 2, 0, 1, 0, 1,
             ptr(am), 2_000_000)
    assert e.value.code == _lib.ERR_TIMEOUT
    # now rank 1 delivers: the very same pull succeeds, and so does an ordinary kernel on the context
    call(cuda_ctx, "nfai_op_gemv_xchg", ptr(dI), _lib.F32, H, H, ptr(dp), None, C.c_float(0), None, areas, 2, 1, 0, None,
         None, 1, 0)
    call(cuda_ctx, "nfai_op_gemv_xchg", ptr(dW), _lib.F32, N, H, None, None, C.c_float(0), ptr(y), areas, 2, 0, 1,
         ptr(dres), ptr(store), 0, 2_000_000)
    x_want = resid + (part + part)
    assert rel_err(host(store), x_want) < 1e-6
    assert rel_err(host(y), oracle.matvec(x_want, W)) < TOL
    y2 = torch.zeros(N, dtype=torch.float32, device="cuda")
    dx = dev(x_want)
    call(cuda_ctx, "nfai_op_gemv", ptr(dW), _lib.F32, N, H, ptr(dx), None, C.c_float(0), None, ptr(y2))
    assert rel_err(host(y2), oracle.matvec(x_want, W)) < TOL


def test_a_model_step_reports_a_timeout_as_a_status(cuda_ctx):
    """nfai_ctx_set_wait_ns is accepted, rejects zero, and a one-GPU model keeps working with a tiny budget (it has no
    waits on peers to run out)."""
    lib = _lib.load()
    assert lib.nfai_ctx_set_wait_ns(cuda_ctx.handle, 0) == _lib.ERR_ARG
    assert lib.nfai_ctx_set_wait_ns(cuda_ctx.handle, 1000) == _lib.OK
    assert lib.nfai_ctx_set_wait_ns(cuda_ctx.handle, 1_000_000_000) == _lib.OK
