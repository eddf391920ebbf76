"""On-device temperature / top-k / top-p sampling against the CPU oracle's SamplingUtils.TopP port
(NFAI.Models.Llama3/SamplingUtils.cs:5-33). Token ids are integers: the comparison is exact. The device and the
host exponentials may differ in the last bit, so a case is kept only when every decision the algorithm takes
(the top_p cut, the draw) has a margin far above that."""
import ctypes as C

import numpy as np
import pytest
import torch

from .gpu_util import call, dev, host, ptr
from nfai_b200 import api, synth

pytestmark = pytest.mark.gpu


def _margin(logits, T, top_p, top_k, u):
    """Smallest distance between a compared quantity and its threshold, in float64."""
    s = logits.astype(np.float64) / T
    p = np.exp(s - s.max())
    p /= p.sum()
    order = np.argsort(-p, kind="stable")[:top_k]
    cum = np.cumsum(p[order])
    m = np.abs(cum - top_p).min()
    n = int(np.argmax(cum >= top_p)) + 1 if (cum >= top_p).any() else len(order)
    run = np.cumsum(p[order[:n]] / p[order[:n]].sum())
    m = min(m, np.abs(run - u).min())
    # equal probabilities are ordered by index on both sides; nearly equal ones could swap
    d = np.diff(-p[order])
    near = d[(d > 0)]
    if near.size:
        m = min(m, (near / p[order][:-1][d > 0]).min())
    return m


def _sample(ctx, logits, T, p, k, u):
    d = dev(logits.astype(np.float32))
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    call(ctx, "nfai_op_sample_top_p", ptr(d), logits.size, C.c_float(T), C.c_float(p), k, C.c_float(u), ptr(tok))
    return int(host(tok)[0])


@pytest.mark.parametrize("V", [7, 300, 4096, 32000, 128256, 300000])
def test_sample_matches_oracle(cuda_ctx, oracle, V):
    rng = np.random.default_rng(V)
    checked = 0
    for trial in range(6):
        logits = (rng.standard_normal(V) * (1.0 + trial)).astype(np.float32)
        for (T, p, k) in ((0.5, 0.95, 40), (1.0, 0.5, 5), (2.0, 1.5, 64), (0.7, 0.9, 1)):
            for u in rng.random(5, dtype=np.float32).tolist() + [0.0]:
                if _margin(logits, T, p, k, u) < 1e-4:
                    continue
                assert _sample(cuda_ctx, logits, T, p, k, u) == oracle.sample_top_p(logits, T, p, k, u), (trial, T, p, k, u)
                checked += 1
    assert checked > 60


def test_sample_edges(cuda_ctx, oracle):
    logits = np.full(5000, -30.0, np.float32)
    logits[4242] = 10.0
    for u in (0.0, 0.5, 0.999):
        assert _sample(cuda_ctx, logits, 0.5, 0.95, 40, u) == 4242
    flat = np.zeros(20000, np.float32)  # every probability equal: order is by index, across slices too
    assert _sample(cuda_ctx, flat, 1.0, 1.0, 10, 0.0) == 0
    assert _sample(cuda_ctx, flat, 1.0, 1.0, 10, 0.95) == oracle.sample_top_p(flat, 1.0, 1.0, 10, 0.95) == 9
    assert _sample(cuda_ctx, flat, 1.0, 1.0, 3, 0.99) == 2
    ties = np.zeros(50000, np.float32)
    for i in (49999, 3, 25000, 25001):
        ties[i] = 8.0
    for u, want in ((0.1, 3), (0.3, 25000), (0.6, 25001), (0.9, 49999)):
        assert _sample(cuda_ctx, ties, 1.0, 0.999, 40, u) == oracle.sample_top_p(ties, 1.0, 0.999, 40, u) == want


def test_sample_rejects_bad_arguments(cuda_ctx):
    d = dev(np.zeros(100, np.float32))
    tok = torch.zeros(1, dtype=torch.int32, device="cuda")
    for (T, p, k, u) in ((0.0, 0.9, 40, 0.5), (0.5, 0.0, 40, 0.5), (0.5, 0.9, 0, 0.5), (0.5, 0.9, 65, 0.5), (0.5, 0.9, 40, 1.0)):
        with pytest.raises(Exception):
            call(cuda_ctx, "nfai_op_sample_top_p", ptr(d), 100, C.c_float(T), C.c_float(p), k, C.c_float(u), ptr(tok))


def test_model_sampling_follows_the_step_logits(oracle):
    cfg = synth.get_config("c0")
    factory = api.LlamaModelFactory(0)
    m = api.create_synthetic_model(cfg, 32, factory=factory)
    logits, am = m.prefill(synth.prompt_ids(cfg, 5, 0))
    rng = np.random.default_rng(3)
    n = 0
    for u in rng.random(12, dtype=np.float32).tolist():
        if _margin(logits, 0.5, 0.95, 40, u) < 1e-4:
            continue
        assert m.sample_top_p(u=u) == oracle.sample_top_p(logits, u=u)
        n += 1
    assert n >= 8
    # the sampled token is a legal next input, and u = 0 draws the arg-max of the new logits
    tok = m.sample_top_p(u=0.3)
    logits2, am2 = m.decode(tok)
    assert m.sample_top_p(u=0.0) == am2 == oracle.argmax(logits2)
    m.Dispose()
    factory.Dispose()


def test_model_sampling_needs_logits(oracle):
    cfg = synth.get_config("c0")
    factory = api.LlamaModelFactory(0)
    m = api.create_synthetic_model(cfg, 8, factory=factory)
    with pytest.raises(api.NfaiError):
        m.sample_top_p()
    m.Dispose()
    factory.Dispose()


def test_sampling_golden(cuda_ctx):
    """The committed draws of the oracle (tests/golden/sample_top_p.npz) reproduced on the device."""
    import os
    from tests.golden.make_golden import sample_logits
    cases = np.load(os.path.join(os.path.dirname(__file__), "golden", "sample_top_p.npz"))["cases"]
    cache = {}
    for V, T, p, k, u, tok in cases:
        V = int(V)
        logits = cache.setdefault(V, sample_logits(V))
        assert _sample(cuda_ctx, logits, float(T), float(p), int(k), float(np.float32(u))) == int(tok)


def test_sampled_loop_on_the_device_equals_the_per_token_calls(oracle):
    """nfai_decode_sampled: step + draw fed back on the device, against decode() + sample_top_p() per token."""
    cfg = synth.get_config("c0")
    factory = api.LlamaModelFactory(0)
    a = api.create_synthetic_model(cfg, 64, factory=factory)
    b = api.create_synthetic_model(cfg, 64, factory=factory)
    prompt = synth.prompt_ids(cfg, 6, 2)
    _, am = a.prefill(prompt)
    b.prefill(prompt, want_logits=False)
    us = np.random.default_rng(8).random(24, dtype=np.float32)
    want, tok = [], am
    for u in us:
        logits, _ = a.decode(tok)
        tok = a.sample_top_p(u=float(u))
        if _margin(logits, 0.5, 0.95, 40, float(u)) >= 1e-4:
            assert tok == oracle.sample_top_p(logits, u=float(u))
        want.append(tok)
    got, ms = b.decode_sampled(am, us)
    assert list(got) == want and ms > 0
    assert a.position == b.position == 6 + 24
    # the loop leaves the model ready for the next call: same continuation on both
    la, _ = a.decode(want[-1])
    lb, _ = b.decode(want[-1])
    assert np.array_equal(la, lb)
    with pytest.raises(api.NfaiError):
        b.decode_sampled(am, [1.5])
    a.Dispose()
    b.Dispose()
    factory.Dispose()
