"""Generate tests/golden/bench_c1_parity.npz: what bench.py checks its benchmark model against at every GPU count.

    python tests/golden/make_bench_parity.py            # CPU oracle part (a minute or two of host time)
    python tests/golden/make_bench_parity.py --gpu      # adds the one-GPU part (needs a B200); keeps the oracle part

The benchmark workload is the Llama-3.2-1B-architecture float16 model (seed 0) with its 128-token prompt. Stored:
the logits after the prompt at 2 048 fixed vocabulary indices and the arg-max, from the CPU oracle (token by token,
float32 arithmetic in the reference's order) and from this library on one GPU (float16 cache, batched prompt
path), plus the greedy continuation of both. A tensor-parallel run all-gathers its logits and compares: within
2e-2 of the oracle (the float16 bound of the path's specification) and within 2e-3 of the one-GPU run.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from nfai_b200 import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "bench_c1_parity.npz")
PROMPT_LEN, N_GREEDY, N_IDX = 128, 16, 2048


def indices(V):
    return np.sort(np.random.default_rng(99).choice(V, N_IDX, replace=False)).astype(np.int64)


def oracle_part():
    from oracle import oracle as O
    cfg = synth.get_config("c1")
    m = O.OracleModel(cfg, ctx=PROMPT_LEN + N_GREEDY + 2).load_synthetic(0)
    prompt = synth.prompt_ids(cfg, PROMPT_LEN, 0)
    logits = m.prefill(prompt)
    tk = O.argmax(logits)
    greedy = [tk]
    gaps = []
    for _ in range(N_GREEDY - 1):
        lg = m.decode(tk)
        top2 = np.partition(lg, -2)[-2:]
        gaps.append(float(top2[1] - top2[0]))
        tk = O.argmax(lg)
        greedy.append(tk)
    return {"idx": indices(cfg.V), "oracle_logits": logits[indices(cfg.V)].astype(np.float32),
            "oracle_argmax": np.uint32(greedy[0]), "oracle_greedy": np.array(greedy, np.uint32),
            "oracle_top2_gap": np.array(gaps, np.float32), "prompt": prompt}


def gpu_part():
    from nfai_b200 import create_synthetic_model
    cfg = synth.get_config("c1")
    m = create_synthetic_model(cfg, PROMPT_LEN + N_GREEDY + 8, kv_dtype="f16")
    prompt = synth.prompt_ids(cfg, PROMPT_LEN, 0)
    logits, am = m.prefill(prompt)
    toks, _ = m.decode_greedy(am, N_GREEDY - 1)
    m.Dispose()
    return {"gpu1_logits": logits[indices(cfg.V)].astype(np.float32), "gpu1_argmax": np.uint32(am),
            "gpu1_greedy": np.array([am] + [int(t) for t in toks], np.uint32)}


if __name__ == "__main__":
    old = dict(np.load(PATH)) if os.path.exists(PATH) else {}
    old.update(gpu_part() if "--gpu" in sys.argv else oracle_part())
    np.savez_compressed(PATH, **old)
    print({k: (v.shape if hasattr(v, "shape") else v) for k, v in old.items()})
