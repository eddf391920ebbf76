"""Whole-path parity through the reference-facing interface (LlamaModel over the C ABI) against the CPU oracle.

Tolerances (from the path's specification): float32 model logits max|a-b|/max|b| <= 1e-4; float16 models
max|a-b| <= 2e-2; greedy token sequences identical on the tiny float32 configuration; embedding rows and arg-max
indices bit-exact.
"""
import os

import numpy as np
import pytest

from nfai_b200 import LlamaModelFactory, ModelOptions, NfaiError, Parser, _lib, create_synthetic_model, gguf_io, synth

from .gpu_util import rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
REL_F32 = 1e-4
ABS_F16 = 2e-2


@pytest.fixture(scope="module")
def factory():
    f = LlamaModelFactory(0)
    yield f
    f.Dispose()


def make(cfg, ctx, factory, **kw):
    return create_synthetic_model(cfg, ctx, factory=factory, **kw)


def check_logits(cfg, got, want):
    if cfg.dtype == "f32":
        assert rel_err(got, want) <= REL_F32
    else:
        assert float(np.abs(got - want).max()) <= ABS_F16


@pytest.mark.parametrize("key,over", [("c0", {}), ("c0p", {}), ("c0", {"gain_std": 0.1}), ("s3", {"gain_std": 0.1}),
                                      ("s2", {}), ("s1", {})])
def test_teacher_forced_logits_and_taps(factory, oracle, key, over):
    cfg = synth.get_config(key, **over)
    n = 24 if key != "s1" else 8
    toks = synth.prompt_ids(cfg, n, 0)
    ref = oracle.OracleModel(cfg, ctx=n).load_synthetic(0)
    m = make(cfg, n, factory, kv_dtype="f32")
    for i, t in enumerate(toks):
        want = ref.decode(int(t))
        got, am = m.decode(int(t))
        check_logits(cfg, got, want)
        assert am == oracle.argmax(got)  # bit-exact index on the device's own logits
        assert m.position == i + 1
        if i in (0, n - 1):
            for l in range(cfg.L):
                assert rel_err(m.read_hidden(l), ref.read_hidden(l)) <= 1e-4
                k, v = m.read_kv(l, i)
                kr, vr = ref.read_kv(l, i)
                assert rel_err(k, kr) <= 1e-4 and rel_err(v, vr) <= 1e-4
    m.Dispose()


def test_config0_prefill_and_64_greedy_tokens_match(factory, oracle):
    g = np.load(os.path.join(GOLDEN, "c0.npz"))
    cfg = synth.get_config("c0")
    m = make(cfg, 128, factory)
    logits, am = m.prefill(g["prompt"])
    assert rel_err(logits, g["logits"][-1]) <= REL_F32
    assert am == int(g["prompt_argmax"][-1]) == int(g["greedy"][0])
    toks, ms = m.decode_greedy(am, 63)
    assert list(toks) == list(g["greedy"][1:])
    assert ms > 0
    # the same through the host-driven loop (RunAsync with token ids)
    m.reset()
    assert m.run_tokens(g["prompt"], 64) == list(g["greedy"])
    m.Dispose()


@pytest.mark.parametrize("key", ["c0p", "c0_gain", "s3_f16_untied", "s2_f16_d128"])
def test_golden_fixtures(factory, key):
    from tests.golden.make_golden import CASES
    cfg_key, over, n_prompt, n_greedy, keep = CASES[key]
    g = np.load(os.path.join(GOLDEN, f"{key}.npz"))
    cfg = synth.get_config(cfg_key, **over)
    m = make(cfg, n_prompt + n_greedy, factory, kv_dtype="f32")
    j = 0
    for i, t in enumerate(g["prompt"]):
        got, am = m.decode(int(t))
        if i in keep:
            check_logits(cfg, got, g["logits"][j])
            j += 1
    toks, _ = m.decode_greedy(am, n_greedy - 1)
    if cfg.dtype == "f32":
        assert am == int(g["greedy"][0]) and list(toks) == list(g["greedy"][1:])
    m.Dispose()


@pytest.mark.parametrize("key,n", [("c0p", 40), ("s3", 40), ("s3", 300), ("s1", 130), ("s2", 70), ("s2", 300)])
def test_prefill_equals_token_by_token(factory, key, n):
    """Float32 models ingest the prompt token by token (identical results); float16 models use the batched
    tensor-core path, whose float16 activations must keep logits and cache rows inside the float16 tolerance."""
    cfg = synth.get_config(key, gain_std=0.1)
    toks = synth.prompt_ids(cfg, n, 1)
    a = make(cfg, n + 24, factory)
    b = make(cfg, n + 24, factory)
    la, ama = a.prefill(toks)
    for t in toks:
        lb, amb = b.decode(int(t))
    f32 = cfg.dtype == "f32"
    assert float(np.abs(la - lb).max()) <= (1e-5 if f32 else ABS_F16)
    if f32:
        assert ama == amb
    assert a.position == b.position == n
    for l in range(cfg.L):
        for p in (0, 17, n - 1):
            ka, va = a.read_kv(l, p)
            kb, vb = b.read_kv(l, p)
            tol = 1e-5 if f32 else 1e-2
            assert rel_err(ka, kb) <= tol and rel_err(va, vb) <= tol
        assert rel_err(a.read_hidden(l), b.read_hidden(l)) <= (1e-5 if f32 else 1e-2)
    # decoding continues from the batched prompt inside the tolerance
    for t in (3, 5, 7):
        la, _ = a.decode(t)
        lb, _ = b.decode(t)
        assert float(np.abs(la - lb).max()) <= (1e-5 if f32 else ABS_F16)
    # prompt in two pieces continues at the next position
    a.reset()
    a.prefill(toks[:13], want_logits=False)
    lc, amc = a.prefill(toks[13:])
    lb2 = None
    b.reset()
    for t in toks:
        lb2, _ = b.decode(int(t))
    assert float(np.abs(lc - lb2).max()) <= (1e-5 if f32 else ABS_F16)
    a.Dispose()
    b.Dispose()


@pytest.mark.parametrize("key", ["s3", "s2"])
def test_batched_prefill_against_oracle(factory, oracle, key):
    cfg = synth.get_config(key, gain_std=0.1)
    n = 280  # more than one chunk of 256 tokens
    toks = synth.prompt_ids(cfg, n, 2)
    ref = oracle.OracleModel(cfg, ctx=n + 8).load_synthetic(0)
    want = ref.prefill(toks)
    m = make(cfg, n + 8, factory, kv_dtype="f32")
    got, am = m.prefill(toks)
    assert float(np.abs(got - want).max()) <= ABS_F16
    assert am == oracle.argmax(got)
    tk = am
    for _ in range(4):
        want = ref.decode(tk)
        got, tk2 = m.decode(tk)
        assert float(np.abs(got - want).max()) <= ABS_F16
        tk = oracle.argmax(want)
    m.Dispose()


def test_fp16_kv_cache_stays_inside_the_fp16_bound(factory, oracle):
    cfg = synth.get_config("s1")
    toks = synth.prompt_ids(cfg, 12, 0)
    ref = oracle.OracleModel(cfg, ctx=12).load_synthetic(0)
    m = make(cfg, 12, factory, kv_dtype="f16")
    for t in toks:
        want = ref.decode(int(t))
        got, _ = m.decode(int(t))
        assert float(np.abs(got - want).max()) <= ABS_F16
    m.Dispose()


def test_widened_upload_equals_raw_half_upload(factory):
    """Chunks widened to float32 (what the reference's GetDataRaw yields) narrow back exactly on the device."""
    cfg = synth.get_config("s3")
    toks = synth.prompt_ids(cfg, 6, 0)
    a = make(cfg, 8, factory)
    b = make(cfg, 8, factory, widen_half=True)
    la, _ = a.prefill(toks)
    lb, _ = b.prefill(toks)
    assert np.array_equal(la.view(np.uint32), lb.view(np.uint32))
    a.Dispose()
    b.Dispose()


def test_gguf_file_through_parser(factory, oracle, tmp_path):
    cfg = synth.get_config("c0p", gain_std=0.1)
    path = os.path.join(tmp_path, "m.gguf")
    gguf_io.write_synthetic_gguf(cfg, path, seed=2)
    model = Parser([factory]).parse(ModelOptions(GGUFPath=path, KVCacheSize=16))
    assert model.ModelName == cfg.name
    ref = oracle.OracleModel(cfg, ctx=16).load_synthetic(2)
    toks = synth.prompt_ids(cfg, 8, 2)
    for t in toks:
        want = ref.decode(int(t))
        got, _ = model.decode(int(t))
        assert rel_err(got, want) <= REL_F32
    model.Dispose()


@pytest.mark.parametrize("key", ["c0p", "s3"])
def test_native_gguf_loader(factory, tmp_path, key):
    """The native loader (mmap + raw pass-through) builds the same model as the tensor-by-tensor upload."""
    from nfai_b200 import LlamaModel
    cfg = synth.get_config(key, gain_std=0.1)
    path = os.path.join(tmp_path, "m.gguf")
    gguf_io.write_synthetic_gguf(cfg, path, seed=4)
    a = LlamaModel.from_gguf_native(factory.ctx, path, 32)
    b = create_synthetic_model(cfg, 32, seed=4, factory=factory)
    assert (a.V, a.H, a.L) == (cfg.V, cfg.H, cfg.L) and a.weight_dtype == cfg.dtype
    assert a.hp.qH == cfg.qH and a.hp.kvH == cfg.kvH and a.hp.F == cfg.F and a.hp.tied == (1 if cfg.tied else 0)
    toks = synth.prompt_ids(cfg, 6, 4)
    for t in toks:
        la, ama = a.decode(int(t))
        lb, amb = b.decode(int(t))
        assert np.array_equal(la.view(np.uint32), lb.view(np.uint32)) and ama == amb
    a.Dispose()
    b.Dispose()
    with pytest.raises(NfaiError) as e:
        LlamaModel.from_gguf_native(factory.ctx, os.path.join(tmp_path, "missing.gguf"), 8)
    assert e.value.code == _lib.ERR_ARG
    bad = os.path.join(tmp_path, "bad.gguf")
    with open(bad, "wb") as fh:
        fh.write(b"NOPE" + bytes(64))
    with pytest.raises(NfaiError) as e:
        LlamaModel.from_gguf_native(factory.ctx, bad, 8)
    assert e.value.code == _lib.ERR_ARG
    trunc = os.path.join(tmp_path, "trunc.gguf")
    with open(path, "rb") as src, open(trunc, "wb") as dst:
        dst.write(src.read(os.path.getsize(path) // 2))
    with pytest.raises(NfaiError) as e:
        LlamaModel.from_gguf_native(factory.ctx, trunc, 8)
    assert e.value.code == _lib.ERR_ARG


def test_errors_are_statuses(factory):
    cfg = synth.get_config("c0")
    m = make(cfg, 4, factory)
    with pytest.raises(NfaiError) as e:
        m.decode(cfg.V)
    assert e.value.code == _lib.ERR_ARG
    m.prefill([1, 2, 3], want_logits=False)
    with pytest.raises(NfaiError) as e:
        m.prefill([1, 2], want_logits=False)
    assert e.value.code == _lib.ERR_CONTEXT_FULL
    m.decode(4, want_logits=False)
    with pytest.raises(NfaiError) as e:
        m.decode(5)
    assert e.value.code == _lib.ERR_CONTEXT_FULL
    assert m.position == 4
    with pytest.raises(NfaiError) as e:
        m.decode_greedy(1, 1)
    assert e.value.code == _lib.ERR_CONTEXT_FULL
    m.reset()
    assert m.position == 0
    m.decode(1)
    m.Dispose()


def test_upload_state_machine(factory):
    import ctypes as C
    lib = _lib.load()
    cfg = synth.get_config("c0")
    hp = _lib.HParams(cfg.H, cfg.L, cfg.qH, cfg.kvH, cfg.d, cfg.ropeDim, cfg.F, cfg.V, 8, cfg.eps, cfg.rope_theta,
                      _lib.F32, _lib.F32, 1)
    h = C.c_void_p()
    _lib.check(lib.nfai_model_create(factory.ctx.handle, C.byref(hp), C.byref(h)), factory.ctx.handle)
    shape = (C.c_uint64 * 2)(cfg.H, cfg.qDim)
    assert lib.nfai_model_tensor_chunk(h, b"\0" * 16, 16) == _lib.ERR_STATE
    assert lib.nfai_model_tensor_begin(h, b"blk.0.nonsense.weight", _lib.F32, shape, 2) == _lib.ERR_ARG
    assert lib.nfai_model_tensor_begin(h, b"blk.9.attn_q.weight", _lib.F32, shape, 2) == _lib.ERR_ARG
    bad = (C.c_uint64 * 2)(cfg.H + 1, cfg.qDim)
    assert lib.nfai_model_tensor_begin(h, b"blk.0.attn_q.weight", _lib.F32, bad, 2) == _lib.ERR_ARG
    assert lib.nfai_model_tensor_begin(h, b"blk.0.attn_q.weight", 7, shape, 2) == _lib.ERR_ARG
    assert lib.nfai_model_tensor_begin(h, b"blk.0.attn_q.weight", _lib.F32, shape, 2) == _lib.OK
    assert lib.nfai_model_tensor_begin(h, b"blk.0.attn_k.weight", _lib.F32, shape, 2) == _lib.ERR_STATE
    assert lib.nfai_model_tensor_chunk(h, b"\0" * 6, 6) == _lib.ERR_ARG       # not a whole number of elements
    assert lib.nfai_model_tensor_chunk(h, b"\0" * 64, 64) == _lib.OK
    assert lib.nfai_model_tensor_end(h) == _lib.ERR_ARG                        # too few bytes
    assert lib.nfai_model_finalize(h) == _lib.ERR_STATE                        # tensors missing
    assert lib.nfai_decode(h, 0, None, None) == _lib.ERR_STATE                 # not finalized
    assert lib.nfai_last_error(factory.ctx.handle)
    assert lib.nfai_model_destroy(h) == _lib.OK


def test_full_size_1b_properties(factory, oracle):
    """The benchmark configuration at full size: determinism, prompt-vs-stepwise equality, a few oracle logits."""
    cfg = synth.get_config("c1")
    m = make(cfg, 160, factory)
    toks = synth.prompt_ids(cfg, 128, 0)
    logits, am = m.prefill(toks)
    first, _ = m.decode_greedy(am, 16)
    m.reset()
    logits2, am2 = m.prefill(toks)
    second, _ = m.decode_greedy(am2, 16)
    assert np.array_equal(logits.view(np.uint32), logits2.view(np.uint32)) and am == am2
    assert list(first) == list(second)
    assert am == oracle.argmax(logits)
    # oracle on the first 3 positions (about 2.5 GB of weights per CPU token)
    ref = oracle.OracleModel(cfg, ctx=4).load_synthetic(0)
    m.reset()
    for t in toks[:3]:
        want = ref.decode(int(t))
        got, _ = m.decode(int(t))
        assert float(np.abs(got - want).max()) <= ABS_F16
    ms, nbytes = m.profile_kernel("ffn_gate_up", 8)
    assert ms > 0 and nbytes == 2 * cfg.F * cfg.H * 2 + cfg.H * 4
    assert m.step_launches() == 3 + 5 * cfg.L
    m.Dispose()


@pytest.mark.parametrize("key", ["c2", "c3"])
def test_full_size_3b_and_8b_against_the_oracle(factory, oracle, key):
    """The 3B-architecture model (head_dim 128, 28 layers) and the 8B-architecture model (untied LM head, 32 layers)
    at full size: three teacher-forced positions against the CPU oracle, float16 bound."""
    cfg = synth.get_config(key)
    m = make(cfg, 8, factory, kv_dtype="f16")
    ref = oracle.OracleModel(cfg, ctx=8).load_synthetic(0)
    toks = synth.prompt_ids(cfg, 3, 0)
    worst = 0.0
    for t in toks:
        want = ref.decode(int(t))
        got, am = m.decode(int(t))
        worst = max(worst, float(np.abs(got - want).max()))
        assert am == oracle.argmax(got)
    assert worst <= ABS_F16, worst
    # the batched prompt path over the same three tokens ends at the same logits
    m.reset()
    got, _ = m.prefill(toks)
    assert float(np.abs(got - want).max()) <= ABS_F16
    assert m.step_launches() == 3 + 5 * cfg.L
    ref.close()
    m.Dispose()


def test_full_size_long_context_decode_against_the_oracle(factory, oracle):
    """The long-context configuration at full size: the 1B-architecture model with a float16 cache seeded to 32 768
    positions (random rows, the same on both sides; ingesting a 32 768-token prompt on the CPU would take an hour),
    then two decode steps at positions 32 768 and 32 769 against the oracle."""
    cfg = synth.get_config("c1")
    n = 32768
    m = make(cfg, n + 8, factory, kv_dtype="f16")
    ref = oracle.OracleModel(cfg, ctx=n + 8).load_synthetic(0)
    rng = np.random.default_rng(4)
    for l in range(cfg.L):
        k = (rng.standard_normal((n, cfg.kvDim), dtype=np.float32) * 0.5).astype(np.float16).astype(np.float32)
        v = (rng.standard_normal((n, cfg.kvDim), dtype=np.float32) * 0.5).astype(np.float16).astype(np.float32)
        m.write_kv_range(l, 0, k, v)
        for p in range(n):
            ref.write_kv(l, p, k[p], v[p])
    m.set_position(n)
    ref.set_position(n)
    for t in synth.prompt_ids(cfg, 2, 3):
        want = ref.decode(int(t))
        got, am = m.decode(int(t))
        assert np.isfinite(got).all()
        assert float(np.abs(got - want).max()) <= ABS_F16
        assert am == oracle.argmax(got)
    ref.close()
    m.Dispose()


@pytest.mark.parametrize("key", ["s3", "s2"])
def test_long_cache_attention_ignores_stale_rows(factory, oracle, monkeypatch, key):
    """A cache longer than 4096 positions selects the tile-staged attention kernel; rows past the sequence hold
    NaN here and must not leak into the result."""
    cfg = synth.get_config(key)
    n = 20
    toks = synth.prompt_ids(cfg, n, 0)
    ref = oracle.OracleModel(cfg, ctx=n).load_synthetic(0)
    m = make(cfg, 4200, factory, kv_dtype="f16")
    nan = np.full(cfg.kvDim, np.nan, np.float32)
    for l in range(cfg.L):
        for pos in list(range(0, 40)) + [4199]:
            m.write_kv(l, pos, nan, nan)
    for t in toks:
        want = ref.decode(int(t))
        got, am = m.decode(int(t))
        assert np.isfinite(got).all()
        assert float(np.abs(got - want).max()) <= ABS_F16
    m.Dispose()


def test_prompt_in_several_passes_equals_one_pass(monkeypatch):
    """A prompt longer than the pass length is ingested in several passes; later passes attend to the cache rows of
    the earlier ones."""
    cfg = synth.get_config("s3", gain_std=0.1)
    toks = synth.prompt_ids(cfg, 150, 4)
    out = {}
    for chunk in ("64", "2048"):
        monkeypatch.setenv("NFAI_PREFILL_CHUNK", chunk)
        f = LlamaModelFactory(0)
        m = create_synthetic_model(cfg, 160, factory=f)
        logits, am = m.prefill(toks)
        out[chunk] = (logits, am, m.read_kv(1, 149), m.read_hidden(1))
        m.Dispose()
        f.Dispose()
    assert float(np.abs(out["64"][0] - out["2048"][0]).max()) <= 2e-3
    assert rel_err(out["64"][2][0], out["2048"][2][0]) <= 2e-3 and rel_err(out["64"][2][1], out["2048"][2][1]) <= 2e-3
    assert rel_err(out["64"][3], out["2048"][3]) <= 2e-3


@pytest.mark.parametrize("key,kv", [("c0", "f32"), ("s3", "f16")])
def test_snapshot_restore_rewinds_exactly(factory, key, kv):
    """A later turn that starts from a restored snapshot sees bit-identical logits; the shared prefix is ingested once."""
    cfg = synth.get_config(key)
    toks = synth.prompt_ids(cfg, 14, 3)
    m = make(cfg, 64, factory, kv_dtype=kv)
    m.prefill(toks, want_logits=False)
    snap = m.snapshot()
    assert snap.position == m.position == 14
    first = [m.decode(t)[0].copy() for t in (3, 5, 7)]
    drawn = m.sample_top_p(u=0.25)
    m.decode(9)                       # wander off: different tokens, more positions
    m.prefill(synth.prompt_ids(cfg, 9, 5), want_logits=False)
    snap.restore()
    assert m.position == 14
    again = [m.decode(t)[0].copy() for t in (3, 5, 7)]
    for a, b in zip(first, again):
        assert np.array_equal(a, b)
    assert m.sample_top_p(u=0.25) == drawn
    # rewinding also works after a reset, and the logits of the snapshot's own step come back
    m.reset()
    snap.restore()
    assert m.sample_top_p(u=0.0) == m.sample_top_p(u=0.0)
    assert [m.decode(t)[1] for t in (3, 5, 7)] == [oracle_argmax(x) for x in first]
    # a snapshot belongs to its model
    other = make(cfg, 64, factory, kv_dtype=kv)
    with pytest.raises(NfaiError):
        snap.restore(other)
    snap.close()
    other.Dispose()
    m.Dispose()


def oracle_argmax(v):
    from oracle import oracle as O
    return O.argmax(v)
