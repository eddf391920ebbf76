"""CPU tests of the oracle: against an independent float64 numpy restatement, against hand-computable cases and
against the committed golden fixtures (the reference holds no vectors for this path: parity is unpinned)."""
import os

import numpy as np
import pytest

from nfai_b200 import synth

from . import np_ref

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_half_widening_is_exact(oracle):
    allbits = np.arange(65536, dtype=np.uint16).view(np.float16)
    got = oracle.half_to_float(allbits)
    want = allbits.astype(np.float32)
    finite = np.isfinite(want)
    assert np.array_equal(got[finite].view(np.uint32), want[finite].view(np.uint32))
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[np.isinf(want)], want[np.isinf(want)])


def test_matvec_sequential_order(oracle):
    # 1e8 + 1 - 1e8 in float32 depends on the order: the oracle must go k ascending like the shader loop
    W = np.array([[1e8, 1.0, -1e8, 1.0]], np.float32)
    x = np.ones(4, np.float32)
    assert oracle.matvec(x, W)[0] == np.float32(1.0)  # ((1e8+1)-1e8)+1 = 0+1
    assert oracle.matvec(x, W, mode=1)[0] == np.float32(2.0)  # double accumulation keeps both ones


@pytest.mark.parametrize("N,K", [(1, 1), (3, 5), (8, 64), (17, 129), (64, 256)])
@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_matvec_vs_numpy(oracle, N, K, dtype):
    rng = np.random.default_rng(N * 1000 + K)
    W = rng.standard_normal((N, K)).astype(dtype)
    x = rng.standard_normal(K).astype(np.float32)
    want = W.astype(np.float64) @ x.astype(np.float64)
    got = oracle.matvec(x, W)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5 * np.sqrt(K))


def test_rmsnorm(oracle):
    rng = np.random.default_rng(1)
    x = rng.standard_normal(300).astype(np.float32)
    g = rng.standard_normal(300).astype(np.float32)
    want = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean() + 1e-5) * g
    assert np.allclose(oracle.rmsnorm(x, g, 1e-5), want, rtol=1e-6, atol=1e-6)


def test_rope_table_and_rotation(oracle):
    f = oracle.rope_table(64, 500000.0)
    want = (1.0 / np.power(np.float32(500000.0), (np.arange(32, dtype=np.float32) / np.float32(32)))).astype(np.float32)
    assert np.allclose(f, want, rtol=1e-6)
    assert f[0] == 1.0
    v = np.arange(2 * 64, dtype=np.float32)
    assert np.array_equal(oracle.rope(v, 2, 64, 64, 500000.0, 0), v)  # position 0 is the identity
    out = oracle.rope(v, 2, 64, 64, 500000.0, 7)
    a, b = v[0::2].astype(np.float64), v[1::2].astype(np.float64)
    th = np.tile(f.astype(np.float64) * 7, 2)
    assert np.allclose(out[0::2], np.cos(th) * a - np.sin(th) * b, rtol=1e-5, atol=1e-4)
    assert np.allclose(out[1::2], np.sin(th) * a + np.cos(th) * b, rtol=1e-5, atol=1e-4)
    # partial rotary dimension: elements beyond ropeDim are copied
    out2 = oracle.rope(v, 2, 64, 32, 500000.0, 7)
    assert np.array_equal(out2[32:64], v[32:64]) and np.array_equal(out2[96:128], v[96:128])


@pytest.mark.parametrize("qH,kvH,d,seq", [(8, 2, 32, 1), (8, 2, 32, 37), (4, 2, 64, 70), (6, 2, 128, 19)])
def test_attention_vs_numpy(oracle, qH, kvH, d, seq):
    rng = np.random.default_rng(seq)
    q = rng.standard_normal(qH * d).astype(np.float32)
    kc = rng.standard_normal((seq + 3, kvH * d)).astype(np.float32)
    vc = rng.standard_normal((seq + 3, kvH * d)).astype(np.float32)
    got = oracle.attention(q, kc, vc, seq, qH, kvH, d, 1e-5)
    want = np.zeros(qH * d)
    for h in range(qH):
        g = h // (qH // kvH)
        s = kc[:seq, g * d:(g + 1) * d].astype(np.float64) @ q[h * d:(h + 1) * d] / np.sqrt(d)
        w = np.exp(s - s.max())
        w /= w.sum()
        want[h * d:(h + 1) * d] = w @ vc[:seq, g * d:(g + 1) * d]
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)


def test_silu_mul(oracle):
    g = np.linspace(-20, 20, 101).astype(np.float32)
    u = np.linspace(3, -3, 101).astype(np.float32)
    want = u * (g / (1 + np.exp(-g.astype(np.float64))))
    assert np.allclose(oracle.silu_mul(g, u), want, rtol=1e-6, atol=1e-7)


def test_argmax_lowest_index(oracle):
    v = np.array([1, 5, 3, 5, 5], np.float32)
    assert oracle.argmax(v) == 1
    assert oracle.argmax(np.zeros(7, np.float32)) == 0


@pytest.mark.parametrize("key", ["c0", "c0p", "s3"])
def test_model_vs_float64_numpy(oracle, key):
    cfg = synth.get_config(key, gain_std=0.1)
    W = {n: a for n, _, _, a in synth.iter_tensors(cfg, 0)}
    toks = synth.prompt_ids(cfg, 10, 0)
    ref = np_ref.forward(cfg, W, toks)
    m = oracle.OracleModel(cfg, ctx=16).load_synthetic(0)
    got = np.array([m.decode(int(t)) for t in toks])
    assert np.abs(got - ref).max() / np.abs(ref).max() < 1e-5
    m2 = oracle.OracleModel(cfg, ctx=16, mode=1).load_synthetic(0)
    got2 = np.array([m2.decode(int(t)) for t in toks])
    assert np.abs(got2 - ref).max() / np.abs(ref).max() < 2e-6
    assert [oracle.argmax(g) for g in got] == list(ref.argmax(1))


def test_context_overflow_is_an_error(oracle):
    cfg = synth.get_config("c0")
    m = oracle.OracleModel(cfg, ctx=2).load_synthetic(0)
    m.decode(1, want_logits=False)
    m.decode(2, want_logits=False)
    with pytest.raises(RuntimeError):
        m.decode(3)


@pytest.mark.parametrize("key", ["c0", "c0p", "c0_gain", "s3_f16_untied", "s2_f16_d128"])
def test_oracle_reproduces_golden(oracle, key):
    from tests.golden.make_golden import CASES
    cfg_key, over, n_prompt, n_greedy, keep = CASES[key]
    g = np.load(os.path.join(GOLDEN, f"{key}.npz"))
    cfg = synth.get_config(cfg_key, **over)
    assert np.array_equal(g["prompt"], synth.prompt_ids(cfg, n_prompt, 0))
    m = oracle.OracleModel(cfg, ctx=n_prompt + n_greedy).load_synthetic(0)
    kept = []
    am = []
    for i, t in enumerate(g["prompt"]):
        lg = m.decode(int(t))
        am.append(oracle.argmax(lg))
        if i in keep:
            kept.append(lg)
    assert np.array_equal(np.array(am, np.uint32), g["prompt_argmax"])
    # same machine class and libm give the same bits; allow a few ulps for a different libm
    assert np.allclose(np.stack(kept), g["logits"], rtol=0, atol=2e-6)
    tk = am[-1]
    greedy = [tk]
    while len(greedy) < n_greedy:
        tk = oracle.argmax(m.decode(tk))
        greedy.append(tk)
    assert np.array_equal(np.array(greedy, np.uint32), g["greedy"])


# ---- sampling (NFAI.Models.Llama3/SamplingUtils.cs:5-33) ----------------------------------------------------

def _np_top_p(logits, T, top_p, top_k, u):
    """Independent restatement in numpy (float64 where LINQ's Sum is double)."""
    s = (logits.astype(np.float32) / np.float32(T)).astype(np.float32)
    e = np.exp((s - s.max()).astype(np.float32)).astype(np.float32)
    p = (e / np.float32(e.astype(np.float64).sum())).astype(np.float32)
    order = np.argsort(-p, kind="stable")[:top_k]
    keep, cum = [], np.float32(0)
    for i in order:
        cum = np.float32(cum + p[i])
        keep.append(i)
        if cum >= np.float32(top_p):
            break
    tot = np.float32(p[keep].astype(np.float64).sum())
    run = np.float32(0)
    for i in keep:
        run = np.float32(run + np.float32(p[i] / tot))
        if np.float32(u) < run:
            return int(i)
    return int(keep[-1])


def test_sample_top_p_matches_numpy(oracle):
    rng = np.random.default_rng(5)
    for V in (7, 300, 4096):
        logits = (rng.standard_normal(V) * 3).astype(np.float32)
        for u in (0.0, 0.03, 0.4, 0.77, 0.999):
            for (T, p, k) in ((0.5, 0.95, 40), (1.0, 0.5, 5), (2.0, 1.5, 64)):
                assert oracle.sample_top_p(logits, T, p, min(k, 64), u) == _np_top_p(logits, T, p, k, u)


def test_sample_top_p_edges(oracle):
    # a peaked distribution always yields its peak; u = 0 yields the arg-max; ties keep index order
    logits = np.full(100, -30.0, np.float32)
    logits[42] = 10.0
    for u in (0.0, 0.5, 0.999):
        assert oracle.sample_top_p(logits, u=u) == 42
    flat = np.zeros(10, np.float32)
    assert oracle.sample_top_p(flat, 1.0, 1.0, 10, 0.0) == 0
    assert oracle.sample_top_p(flat, 1.0, 1.0, 10, 0.95) == 9
    assert oracle.sample_top_p(flat, 1.0, 1.0, 3, 0.99) == 2     # top_k cuts the flat tail in index order
    assert oracle.sample_top_p(flat, 1.0, 0.25, 10, 0.99) == 2   # 0.1+0.1+0.1 >= 0.25 stops after three


def test_sampling_golden(oracle):
    from tests.golden.make_golden import sample_logits
    cases = np.load(os.path.join(GOLDEN, "sample_top_p.npz"))["cases"]
    assert len(cases) > 60
    cache = {}
    for V, T, p, k, u, tok in cases:
        V = int(V)
        logits = cache.setdefault(V, sample_logits(V))
        assert oracle.sample_top_p(logits, float(T), float(p), int(k), float(np.float32(u))) == int(tok)
