"""Generate the golden fixtures in this directory from the CPU oracle.

    python tests/golden/make_golden.py

The reference has no golden vectors for this path and cannot run here, so these fixtures pin the ORACLE
(float32, sequential order) on seeded synthetic models: they catch any later drift of the oracle, of the model
generator and of the CUDA path. Each .npz holds, for one configuration: the prompt, the teacher-forced logits
at a few prompt positions, the arg-max of every prompt position and the greedy continuation.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from nfai_b200 import synth  # noqa: E402
from oracle import oracle as O  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))

# key -> (config key, overrides, prompt length, greedy steps, positions whose logits are stored)
CASES = {
    "c0": ("c0", {}, 64, 64, [0, 1, 31, 63]),
    "c0p": ("c0p", {}, 64, 64, [0, 63]),
    "c0_gain": ("c0", {"gain_std": 0.1}, 16, 16, [0, 15]),
    "s3_f16_untied": ("s3", {"gain_std": 0.1}, 24, 16, [0, 23]),
    "s2_f16_d128": ("s2", {}, 16, 8, [15]),
}


def make(key: str):
    cfg_key, over, n_prompt, n_greedy, keep = CASES[key]
    cfg = synth.get_config(cfg_key, **over)
    m = O.OracleModel(cfg, ctx=n_prompt + n_greedy).load_synthetic(0)
    prompt = synth.prompt_ids(cfg, n_prompt, 0)
    kept, argmaxes = [], []
    logits = None
    for i, t in enumerate(prompt):
        logits = m.decode(int(t))
        argmaxes.append(O.argmax(logits))
        if i in keep:
            kept.append(logits.copy())
    greedy = []
    tk = argmaxes[-1]
    greedy.append(tk)
    greedy_logits_last = None
    while len(greedy) < n_greedy:
        greedy_logits_last = m.decode(tk)
        tk = O.argmax(greedy_logits_last)
        greedy.append(tk)
    np.savez_compressed(
        os.path.join(HERE, f"{key}.npz"),
        prompt=prompt.astype(np.uint32),
        keep=np.array(keep, np.int32),
        logits=np.stack(kept).astype(np.float32),
        prompt_argmax=np.array(argmaxes, np.uint32),
        greedy=np.array(greedy, np.uint32),
        greedy_logits_last=greedy_logits_last.astype(np.float32),
    )
    print(key, "greedy head:", greedy[:8])


# Sampling (SamplingUtils.TopP): seeded logits vectors and, for a grid of (temperature, top_p, top_k, u), the token
# the oracle draws. Only well-conditioned draws are kept (every comparison the algorithm makes has a margin far above
# the last-bit differences between exponential implementations), so that the device may be held to them exactly.
SAMPLE_V = (300, 4096, 128256)
SAMPLE_PARAMS = ((0.5, 0.95, 40), (1.0, 0.5, 5), (2.0, 1.5, 64), (0.7, 0.9, 1))


def sample_margin(logits, T, top_p, top_k, u):
    s = logits.astype(np.float64) / T
    p = np.exp(s - s.max())
    p /= p.sum()
    order = np.argsort(-p, kind="stable")[:top_k]
    cum = np.cumsum(p[order])
    m = np.abs(cum - top_p).min()
    n = int(np.argmax(cum >= top_p)) + 1 if (cum >= top_p).any() else len(order)
    run = np.cumsum(p[order[:n]] / p[order[:n]].sum())
    m = min(m, np.abs(run - u).min())
    d = np.diff(-p[order])
    if (d > 0).any():
        m = min(m, (d[d > 0] / p[order][:-1][d > 0]).min())
    return m


def sample_logits(V: int) -> np.ndarray:
    return (np.random.default_rng(1000 + V).standard_normal(V) * 2.5).astype(np.float32)


def make_sampling():
    rows = []
    for V in SAMPLE_V:
        logits = sample_logits(V)
        us = np.random.default_rng(V).random(8, dtype=np.float32).tolist() + [0.0]
        for (T, p, k) in SAMPLE_PARAMS:
            for u in us:
                if sample_margin(logits, T, p, k, u) < 1e-4:
                    continue
                rows.append((V, T, p, k, u, O.sample_top_p(logits, T, p, k, u)))
    np.savez_compressed(os.path.join(HERE, "sample_top_p.npz"), cases=np.array(rows, np.float64))
    print("sampling cases:", len(rows))


# Tokenizer: the oracle's ids for the chat-templated form of a few texts over the synthetic vocabulary of
# tests/tok_util.py.
TOKENIZER_TEXTS = ["The quick brown fox jumps over a lazy dog.", "it's 12345 tokens,  isn't it?\n\nYes: naïve café!",
                   "tab\tand\r\nwindows lines", "привет мир 日本語 \U0001F600"]


def make_tokenizer():
    from oracle.tokenizer_oracle import OracleTokenizer
    from tests import tok_util
    md = tok_util.metadata()
    ref = OracleTokenizer(md["tokenizer.ggml.tokens"], md["tokenizer.ggml.merges"], 0, 1)
    ids, offs = [], [0]
    for t in TOKENIZER_TEXTS:
        ids += ref.tokenize(t)
        offs.append(len(ids))
    np.savez_compressed(os.path.join(HERE, "tokenizer.npz"), texts=np.frombuffer("\x00".join(TOKENIZER_TEXTS).encode("utf-8"), np.uint8),
                        ids=np.array(ids, np.uint32), offsets=np.array(offs, np.int64))
    print("tokenizer cases:", len(TOKENIZER_TEXTS), "ids:", len(ids))


if __name__ == "__main__":
    for k in CASES:
        make(k)
    make_sampling()
    make_tokenizer()
