"""The fused decode step (one persistent kernel per token) against the per-kernel path and the oracle."""
import numpy as np
import pytest

from nfai_b200 import LlamaModelFactory, create_synthetic_model, synth

from .gpu_util import rel_err

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.fixture(scope="module")
def factory():
    f = LlamaModelFactory(0)
    yield f
    f.Dispose()


@pytest.mark.parametrize("mode", [1, 2], ids=["register-prefetch", "rings"])
@pytest.mark.parametrize("key,over,kv", [("c0", {}, "f32"), ("c0p", {"gain_std": 0.1}, "f32"), ("s3", {"gain_std": 0.1}, "f16"),
                                         ("s2", {}, "f32"), ("s1", {}, "f16")])
def test_fused_step_matches_per_kernel_path_and_oracle(factory, oracle, key, over, kv, mode):
    cfg = synth.get_config(key, **over)
    n = 20 if key != "s1" else 8
    toks = synth.prompt_ids(cfg, n, 0)
    ref = oracle.OracleModel(cfg, ctx=64).load_synthetic(0)
    a = create_synthetic_model(cfg, 64, factory=factory, kv_dtype=kv)
    b = create_synthetic_model(cfg, 64, factory=factory, kv_dtype=kv)
    b.set_fused_step(mode)
    assert b.step_launches() == 1 and a.step_launches() == 3 + 5 * cfg.L
    for i, t in enumerate(toks):
        want = ref.decode(int(t))
        la, ama = a.decode(int(t))
        lb, amb = b.decode(int(t))
        tol = 1e-4 if (cfg.dtype == "f32" and kv == "f32") else 2e-3
        assert rel_err(lb, want) <= tol
        assert rel_err(lb, la) <= 1e-4  # same arithmetic, different summation order in attention
        assert amb == oracle.argmax(lb)
        assert b.position == i + 1
    # greedy on the device and a head-less prompt through the fused kernel
    ga, _ = a.decode_greedy(ama, 12)
    gb, _ = b.decode_greedy(amb, 12)
    if ama == amb:
        assert list(ga) == list(gb)
    b.reset()
    a.reset()
    la, ama = a.prefill(toks)
    lb, amb = b.prefill(toks)
    assert rel_err(lb, la) <= 1e-4 and ama == amb
    for l in range(cfg.L):
        ka, va = a.read_kv(l, n - 1)
        kb, vb = b.read_kv(l, n - 1)
        kv_tol = 1e-5 if kv == "f32" else 2e-3  # a float16 cache row may round the other way by one ulp
        assert rel_err(kb, ka) <= kv_tol and rel_err(vb, va) <= kv_tol
        assert rel_err(b.read_hidden(l), a.read_hidden(l)) <= 1e-4
    b.set_fused_step(False)
    assert b.step_launches() == 3 + 5 * cfg.L
    a.Dispose()
    b.Dispose()


@pytest.mark.parametrize("mode", [1, 2], ids=["register-prefetch", "rings"])
def test_fused_step_long_context_splits(factory, oracle, mode):
    """Attention inside the fused step with several splits: seed the cache, then compare one step."""
    cfg = synth.get_config("s3", gain_std=0.1)
    ctx = 1500
    rng = np.random.default_rng(0)
    a = create_synthetic_model(cfg, ctx, factory=factory, kv_dtype="f32")
    b = create_synthetic_model(cfg, ctx, factory=factory, kv_dtype="f32")
    b.set_fused_step(mode)
    npos = 1200
    for l in range(cfg.L):
        for p in range(npos):
            k = rng.standard_normal(cfg.kvDim).astype(np.float32)
            v = rng.standard_normal(cfg.kvDim).astype(np.float32)
            a.write_kv(l, p, k, v)
            b.write_kv(l, p, k, v)
    a.set_position(npos)
    b.set_position(npos)
    for t in (5, 9, 11):
        la, _ = a.decode(t)
        lb, _ = b.decode(t)
        assert rel_err(lb, la) <= 1e-4
    a.Dispose()
    b.Dispose()
