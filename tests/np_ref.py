"""An independent float64 numpy statement of the Llama-3 forward path, used only to cross-check the C++ oracle."""
import numpy as np


def forward(cfg, W, tokens):
    """Teacher-forced logits [len(tokens)][V] in float64."""
    d, qH, kvH = cfg.d, cfg.qH, cfg.kvH
    f = 1.0 / (cfg.rope_theta ** (np.arange(d // 2) / (d / 2)))
    kc = [[] for _ in range(cfg.L)]
    vc = [[] for _ in range(cfg.L)]
    outs = []

    def norm(x, g):
        return x / np.sqrt((x * x).mean() + cfg.eps) * g

    def rope(v, heads, p):
        v = v.reshape(heads, d // 2, 2).copy()
        th = f * p
        c, s = np.cos(th), np.sin(th)
        a, b = v[..., 0].copy(), v[..., 1].copy()
        v[..., 0] = c * a - s * b
        v[..., 1] = s * a + c * b
        return v.reshape(-1)

    for p, t in enumerate(tokens):
        x = W["token_embd.weight"][int(t)].astype(np.float64)
        for l in range(cfg.L):
            g = lambda n: W[f"blk.{l}.{n}.weight"].astype(np.float64)  # noqa: E731
            a = norm(x, g("attn_norm"))
            q = rope(g("attn_q") @ a, qH, p)
            k = rope(g("attn_k") @ a, kvH, p)
            v = g("attn_v") @ a
            kc[l].append(k)
            vc[l].append(v)
            K = np.stack(kc[l]).reshape(p + 1, kvH, d)
            V = np.stack(vc[l]).reshape(p + 1, kvH, d)
            o = np.zeros(qH * d)
            for h in range(qH):
                gg = h // (qH // kvH)
                s = K[:, gg, :] @ q[h * d:(h + 1) * d] / np.sqrt(d)
                w = np.exp(s - s.max())
                w /= w.sum()
                o[h * d:(h + 1) * d] = w @ V[:, gg, :]
            x = x + g("attn_output") @ o
            b = norm(x, g("ffn_norm"))
            gate = g("ffn_gate") @ b
            up = g("ffn_up") @ b
            x = x + g("ffn_down") @ (up * gate / (1 + np.exp(-gate)))
        y = norm(x, W["output_norm.weight"].astype(np.float64))
        head = W.get("output.weight", W["token_embd.weight"]).astype(np.float64)
        outs.append(head @ y)
    return np.array(outs)
