"""Kernel-level parity: every CUDA kernel of the path against the matching oracle function, through the C ABI.

Tolerances: float32 weights rel 1e-4 of the largest output (the north star's logits bound; observed ~1e-6),
float16 weights the same bound because the halves are widened exactly and accumulated in float32; embedding
rows and arg-max indices bit-exact.
"""
import ctypes as C

import numpy as np
import pytest

from nfai_b200 import _lib

from .gpu_util import call, dev, dtype_code, host, ptr, rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

TOL = 1e-4


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_embed_is_bit_exact(cuda_ctx, oracle, dtype):
    rng = np.random.default_rng(0)
    V, H = 97, 200
    E = rng.standard_normal((V, H)).astype(dtype)
    dE = dev(E)
    out = torch.empty(H, dtype=torch.float32, device="cuda")
    for tok in (0, 5, V - 1):
        call(cuda_ctx, "nfai_op_embed", ptr(dE), dtype_code(dtype), H, V, tok, ptr(out))
        assert np.array_equal(host(out).view(np.uint32), E[tok].astype(np.float32).view(np.uint32))
    with pytest.raises(_lib.NfaiError) as e:
        call(cuda_ctx, "nfai_op_embed", ptr(dE), dtype_code(dtype), H, V, V, ptr(out))
    assert e.value.code == _lib.ERR_ARG


@pytest.mark.parametrize("N,K", [(1, 8), (7, 40), (64, 256), (100, 264), (33, 37), (5, 3), (2048, 2048), (300, 8192)])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("norm,resid", [(False, False), (True, False), (False, True), (True, True)])
def test_gemv(cuda_ctx, oracle, N, K, dtype, norm, resid):
    rng = np.random.default_rng(N * 7919 + K)
    W = (rng.standard_normal((N, K)) * 0.05).astype(dtype)
    x = rng.standard_normal(K).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    r = rng.standard_normal(N).astype(np.float32)
    eps = 1e-5
    xin = oracle.rmsnorm(x, g, eps) if norm else x
    want = oracle.matvec(xin, W) + (r if resid else 0)
    dW, dx, dg, dr = dev(W), dev(x), dev(g), dev(r)
    y = torch.empty(N, dtype=torch.float32, device="cuda")
    call(cuda_ctx, "nfai_op_gemv", ptr(dW), dtype_code(dtype), N, K, ptr(dx), ptr(dg) if norm else None,
         C.c_float(eps), ptr(dr) if resid else None, ptr(y))
    assert rel_err(host(y), want) < TOL


@pytest.mark.parametrize("shape", ["1,2,2,0", "1,8,2,0", "2,2,1,0", "2,8,4,0", "4,2,2,0", "4,4,2,0",
                                   "2,1,2,1", "2,2,2,1", "2,2,1,1", "2,3,1,1", "2,4,1,1", "2,3,1,1,0,5"])
@pytest.mark.parametrize("N,K,dtype", [(203, 1544, np.float16), (64, 256, np.float32), (1000, 2048, np.float16),
                                       (37, 8192, np.float16), (5000, 520, np.float32)])
def test_gemv_launch_shapes(cuda_ctx, oracle, monkeypatch, shape, N, K, dtype):
    """Every tunable launch shape (rows per warp, depth, CTAs per SM, mode 0 = registers / 1 = shared-memory rings fed by
    bulk copies with `depth` stages per warp, K split, stages asked into L2 ahead) computes the same thing, through
    every epilogue. K = 2 048 with float16 weights takes the ring kernel's x-in-registers form, the other shapes its
    shared-memory form (ragged chunks, float32 weights)."""
    monkeypatch.setenv("NFAI_TUNE_OP", shape)
    rng = np.random.default_rng(N + K)
    W = (rng.standard_normal((N, K)) * 0.05).astype(dtype)
    x = rng.standard_normal(K).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    r = rng.standard_normal(N).astype(np.float32)
    dW, dx, dg, dr = dev(W), dev(x), dev(g), dev(r)
    y = torch.empty(N, dtype=torch.float32, device="cuda")
    call(cuda_ctx, "nfai_op_gemv", ptr(dW), dtype_code(dtype), N, K, ptr(dx), ptr(dg), C.c_float(1e-5), ptr(dr), ptr(y))
    a = oracle.rmsnorm(x, g, 1e-5)
    assert rel_err(host(y), oracle.matvec(a, W) + r) < TOL
    # logits + arg-max through the same shape
    logits = torch.empty(N, dtype=torch.float32, device="cuda")
    am = torch.zeros(1, dtype=torch.int32, device="cuda")
    call(cuda_ctx, "nfai_op_lm_head", ptr(dW), dtype_code(dtype), ptr(dx), ptr(dg), C.c_float(1e-5), K, N, ptr(logits), ptr(am))
    got = host(logits)
    assert rel_err(got, oracle.matvec(a, W)) < TOL
    assert int(host(am)[0]) == oracle.argmax(got)
    if N % 2 == 0:  # gate/up pairs
        h = torch.empty(N // 2, dtype=torch.float32, device="cuda")
        call(cuda_ctx, "nfai_op_ffn_gate_up", ptr(dW), dtype_code(dtype), ptr(dx), ptr(dg), C.c_float(1e-5), K, N // 2, ptr(h))
        yy = oracle.matvec(a, W)
        assert rel_err(host(h), oracle.silu_mul(yy[0::2], yy[1::2])) < TOL


def rope_cs_table(oracle, ctx, rope_dim, theta):
    f = oracle.rope_table(rope_dim, theta)
    tab = np.empty((ctx, rope_dim // 2, 2), np.float32)
    for p in range(ctx):
        th = (f * np.float32(p)).astype(np.float32)
        tab[p, :, 0] = np.cos(th.astype(np.float64))
        tab[p, :, 1] = np.sin(th.astype(np.float64))
    return tab


@pytest.mark.parametrize("H,qH,kvH,d,rope_dim", [(256, 8, 2, 32, 32), (256, 4, 2, 64, 64), (384, 6, 2, 128, 128),
                                                 (256, 4, 2, 64, 32), (100, 2, 1, 32, 32)])
@pytest.mark.parametrize("wdtype,kvdtype", [(np.float32, np.float32), (np.float16, np.float16), (np.float16, np.float32)])
def test_qkv_rope(cuda_ctx, oracle, H, qH, kvH, d, rope_dim, wdtype, kvdtype):
    rng = np.random.default_rng(H + d)
    qDim, kvDim = qH * d, kvH * d
    W = (rng.standard_normal((qDim + 2 * kvDim, H)) * 0.05).astype(wdtype)
    x = rng.standard_normal(H).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    eps, theta, pos, ctx = 1e-5, 500000.0, 5, 8
    a = oracle.rmsnorm(x, g, eps)
    y = oracle.matvec(a, W)
    q_want = oracle.rope(y[:qDim], qH, d, rope_dim, theta, pos)
    k_want = oracle.rope(y[qDim:qDim + kvDim], kvH, d, rope_dim, theta, pos)
    v_want = y[qDim + kvDim:]
    tab = rope_cs_table(oracle, ctx, rope_dim, theta)
    dW, dx, dg, dtab = dev(W), dev(x), dev(g), dev(tab)
    tdt = torch.float16 if kvdtype == np.float16 else torch.float32
    kc = torch.zeros(ctx * kvDim, dtype=tdt, device="cuda")
    vc = torch.zeros(ctx * kvDim, dtype=tdt, device="cuda")
    q = torch.empty(qDim, dtype=torch.float32, device="cuda")
    call(cuda_ctx, "nfai_op_qkv_rope", ptr(dW), dtype_code(wdtype), ptr(dx), ptr(dg), C.c_float(eps), H, qH, kvH, d,
         rope_dim, ptr(dtab), pos, ptr(q), ptr(kc), ptr(vc), dtype_code(kvdtype))
    assert rel_err(host(q), q_want) < TOL
    kch, vch = host(kc).astype(np.float32).reshape(ctx, kvDim), host(vc).astype(np.float32).reshape(ctx, kvDim)
    kv_tol = TOL if kvdtype == np.float32 else 1e-3  # one float16 rounding of the stored row
    assert rel_err(kch[pos], k_want) < kv_tol
    assert rel_err(vch[pos], v_want) < kv_tol
    other = [p for p in range(ctx) if p != pos]
    assert not kch[other].any() and not vch[other].any()  # only row `pos` is written


@pytest.mark.parametrize("H,F", [(256, 768), (100, 50), (2048, 512)])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_ffn_gate_up(cuda_ctx, oracle, H, F, dtype):
    rng = np.random.default_rng(F)
    Wg = (rng.standard_normal((F, H)) * 0.05).astype(dtype)
    Wu = (rng.standard_normal((F, H)) * 0.05).astype(dtype)
    x = rng.standard_normal(H).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    eps = 1e-5
    a = oracle.rmsnorm(x, g, eps)
    want = oracle.silu_mul(oracle.matvec(a, Wg), oracle.matvec(a, Wu))
    Wgu = np.empty((2 * F, H), dtype)
    Wgu[0::2], Wgu[1::2] = Wg, Wu
    dW, dx, dg = dev(Wgu), dev(x), dev(g)
    h = torch.empty(F, dtype=torch.float32, device="cuda")
    call(cuda_ctx, "nfai_op_ffn_gate_up", ptr(dW), dtype_code(dtype), ptr(dx), ptr(dg), C.c_float(eps), H, F, ptr(h))
    assert rel_err(host(h), want) < TOL


@pytest.mark.parametrize("qH,kvH,d", [(8, 2, 32), (4, 2, 64), (32, 8, 64), (24, 8, 128), (8, 1, 64), (5, 5, 32)])
@pytest.mark.parametrize("seq", [1, 2, 31, 32, 33, 100, 700, 5000, 32768])
@pytest.mark.parametrize("kvdtype", [np.float32, np.float16])
def test_attention_decode(cuda_ctx, oracle, qH, kvH, d, seq, kvdtype):
    if seq == 5000 and (qH, kvH, d) not in ((32, 8, 64), (8, 1, 64), (24, 8, 128)):
        pytest.skip("long sequences on three geometries only")
    if seq == 32768 and (qH, kvH, d) != (32, 8, 64):
        pytest.skip("the longest sequence on the long-context configuration's geometry only")
    rng = np.random.default_rng(seq * 31 + d)
    kvDim = kvH * d
    q = rng.standard_normal(qH * d).astype(np.float32)
    kc = rng.standard_normal((seq, kvDim)).astype(kvdtype)
    vc = rng.standard_normal((seq, kvDim)).astype(kvdtype)
    want = oracle.attention(q, kc.astype(np.float32), vc.astype(np.float32), seq, qH, kvH, d, 1e-5)
    lib = _lib.load()
    nbytes = lib.nfai_op_attn_scratch_bytes(qH, kvH, d, seq)
    scratch = torch.zeros(nbytes // 4 + 1, dtype=torch.float32, device="cuda")
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    out = torch.empty(qH * d, dtype=torch.float32, device="cuda")
    for _ in range(2):  # twice: the split tickets must be back at zero after a launch
        out.zero_()
        call(cuda_ctx, "nfai_op_attn_decode", ptr(dq), ptr(dk), ptr(dv), dtype_code(kvdtype), seq, qH, kvH, d, ptr(out),
             ptr(scratch), C.c_size_t(nbytes))
        assert rel_err(host(out), want) < TOL
    with pytest.raises(_lib.NfaiError):
        call(cuda_ctx, "nfai_op_attn_decode", ptr(dq), ptr(dk), ptr(dv), dtype_code(kvdtype), seq, qH, kvH, d, ptr(out),
             ptr(scratch), C.c_size_t(max(0, nbytes - 256)))


def test_attention_peaked_scores(cuda_ctx, oracle):
    """Large score spread: the online softmax must agree with the clamped three-pass softmax."""
    rng = np.random.default_rng(5)
    qH, kvH, d, seq = 4, 2, 64, 300
    q = (rng.standard_normal(qH * d) * 6).astype(np.float32)
    kc = (rng.standard_normal((seq, kvH * d)) * 3).astype(np.float32)
    vc = rng.standard_normal((seq, kvH * d)).astype(np.float32)
    want = oracle.attention(q, kc, vc, seq, qH, kvH, d, 1e-5)
    lib = _lib.load()
    nbytes = lib.nfai_op_attn_scratch_bytes(qH, kvH, d, seq)
    scratch = torch.zeros(nbytes // 4 + 1, dtype=torch.float32, device="cuda")
    out = torch.empty(qH * d, dtype=torch.float32, device="cuda")
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    call(cuda_ctx, "nfai_op_attn_decode", ptr(dq), ptr(dk), ptr(dv), _lib.F32, seq, qH, kvH, d, ptr(out), ptr(scratch),
         C.c_size_t(nbytes))
    assert rel_err(host(out), want) < TOL


@pytest.mark.parametrize("V,H", [(4096, 256), (1000, 100), (128256, 256), (7, 16)])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_lm_head_and_argmax(cuda_ctx, oracle, V, H, dtype):
    rng = np.random.default_rng(V)
    W = (rng.standard_normal((V, H)) * 0.05).astype(dtype)
    x = rng.standard_normal(H).astype(np.float32)
    g = (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    eps = 1e-5
    want = oracle.matvec(oracle.rmsnorm(x, g, eps), W)
    dW, dx, dg = dev(W), dev(x), dev(g)
    logits = torch.empty(V, dtype=torch.float32, device="cuda")
    am = torch.zeros(1, dtype=torch.int32, device="cuda")
    call(cuda_ctx, "nfai_op_lm_head", ptr(dW), dtype_code(dtype), ptr(dx), ptr(dg), C.c_float(eps), H, V, ptr(logits), ptr(am))
    got = host(logits)
    assert rel_err(got, want) < TOL
    # the index is exact on the logits the device produced: lowest index of their maximum
    assert int(host(am)[0]) == oracle.argmax(got)


def test_argmax_ties_pick_the_lowest_index(cuda_ctx, oracle):
    V, H = 5000, 64
    W = np.zeros((V, H), np.float32)
    x = np.ones(H, np.float32)
    for row in (4321, 77, 3000):  # equal maxima
        W[row, 0] = 2.0
    dW, dx = dev(W), dev(x)
    logits = torch.empty(V, dtype=torch.float32, device="cuda")
    am = torch.zeros(1, dtype=torch.int32, device="cuda")
    call(cuda_ctx, "nfai_op_lm_head", ptr(dW), _lib.F32, ptr(dx), None, C.c_float(0), H, V, ptr(logits), ptr(am))
    assert int(host(am)[0]) == 77 == oracle.argmax(host(logits))
    W[:] = 0  # all equal -> index 0
    dW = dev(W)
    call(cuda_ctx, "nfai_op_lm_head", ptr(dW), _lib.F32, ptr(dx), None, C.c_float(0), H, V, ptr(logits), ptr(am))
    assert int(host(am)[0]) == 0


@pytest.mark.parametrize("qH,kvH,d", [(8, 1, 64), (4, 1, 128), (3, 1, 128)])
@pytest.mark.parametrize("kernel", ["tensor-core", "tile-staged"])
def test_attention_more_splits_than_one_merge_pass(cuda_ctx, oracle, monkeypatch, qH, kvH, d, kernel):
    """One KV head (a rank of an 8-way tensor-parallel group) and 70 000 positions: the sequence is cut into more than
    a hundred splits, so the last CTA merges the partials in several passes with a carried row."""
    monkeypatch.setenv("NFAI_ATTN_MMA", "1" if kernel == "tensor-core" else "0")
    monkeypatch.setenv("NFAI_ATTN_RING", "1")
    seq = 70000
    rng = np.random.default_rng(seq + d + qH)
    q = rng.standard_normal(qH * d).astype(np.float32)
    kc = rng.standard_normal((seq, kvH * d)).astype(np.float16)
    vc = rng.standard_normal((seq, kvH * d)).astype(np.float16)
    want = oracle.attention(q, kc.astype(np.float32), vc.astype(np.float32), seq, qH, kvH, d, 1e-5)
    lib = _lib.load()
    nbytes = lib.nfai_op_attn_scratch_bytes(qH, kvH, d, seq)
    scratch = torch.zeros(nbytes // 4 + 1, dtype=torch.float32, device="cuda")
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    out = torch.empty(qH * d, dtype=torch.float32, device="cuda")
    for _ in range(2):
        out.zero_()
        call(cuda_ctx, "nfai_op_attn_decode", ptr(dq), ptr(dk), ptr(dv), _lib.F16, seq, qH, kvH, d, ptr(out), ptr(scratch),
             C.c_size_t(nbytes))
        assert rel_err(host(out), want) < TOL


@pytest.mark.parametrize("qH,kvH,d", [(32, 8, 64), (24, 8, 128), (4, 2, 64), (8, 1, 64), (6, 2, 128)])
@pytest.mark.parametrize("seq", [1, 2, 15, 16, 17, 100, 255, 256, 257, 700, 5000, 20000, 32768])
@pytest.mark.parametrize("kernel", ["tensor-core", "tile-staged"])
def test_attention_long_context_kernels_every_length(cuda_ctx, oracle, monkeypatch, qH, kvH, d, seq, kernel):
    """The two long-context kernels (query heads as the rows of an MMA tile; K and V through shared-memory rings on the
    CUDA cores) forced on for every length of a float16 cache."""
    monkeypatch.setenv("NFAI_ATTN_MMA", "1" if kernel == "tensor-core" else "0")
    if seq == 20000 and (qH, kvH, d) not in ((32, 8, 64), (24, 8, 128)):
        pytest.skip("the longest sequences on few geometries only")
    if seq == 32768 and (qH, kvH, d) != (32, 8, 64):
        pytest.skip("the longest sequences on few geometries only")
    monkeypatch.setenv("NFAI_ATTN_RING", "1")
    rng = np.random.default_rng(seq * 17 + d + qH)
    kvDim = kvH * d
    q = rng.standard_normal(qH * d).astype(np.float32)
    kc = rng.standard_normal((seq, kvDim)).astype(np.float16)
    vc = rng.standard_normal((seq, kvDim)).astype(np.float16)
    want = oracle.attention(q, kc.astype(np.float32), vc.astype(np.float32), seq, qH, kvH, d, 1e-5)
    lib = _lib.load()
    nbytes = lib.nfai_op_attn_scratch_bytes(qH, kvH, d, seq)
    scratch = torch.zeros(nbytes // 4 + 1, dtype=torch.float32, device="cuda")
    dq, dk, dv = dev(q), dev(kc), dev(vc)
    out = torch.empty(qH * d, dtype=torch.float32, device="cuda")
    for _ in range(2):
        out.zero_()
        call(cuda_ctx, "nfai_op_attn_decode", ptr(dq), ptr(dk), ptr(dv), _lib.F16, seq, qH, kvH, d, ptr(out), ptr(scratch),
             C.c_size_t(nbytes))
        assert rel_err(host(out), want) < TOL
    # the register-streaming kernel gives the same answer on the same inputs
    monkeypatch.setenv("NFAI_ATTN_RING", "0")
    out2 = torch.empty(qH * d, dtype=torch.float32, device="cuda")
    call(cuda_ctx, "nfai_op_attn_decode", ptr(dq), ptr(dk), ptr(dv), _lib.F16, seq, qH, kvH, d, ptr(out2), ptr(scratch),
         C.c_size_t(nbytes))
    assert rel_err(host(out2), host(out)) < TOL
