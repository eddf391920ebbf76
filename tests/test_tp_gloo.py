"""World-size-2 CPU test (gloo) of the tensor-parallel host logic: the partition of one block into rank shards plus
an all-reduce reproduces the unsharded oracle, and the unique-id rendezvous gives every rank the same bytes."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from nfai_b200 import synth, tp
    from oracle import oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        uid = tp.share_unique_id(dist, rank, lambda: bytes(range(128)))
        cfg = synth.get_config("s3", gain_std=0.1)
        W = {n: a for n, _, _, a in synth.iter_tensors(cfg, 0)}
        sh = tp.shard_ranges(cfg, world, rank)

        def cut(name):
            (r0, r1), (c0, c1) = sh[name]
            return np.ascontiguousarray(W["blk.0." + name][r0:r1, c0:c1])

        # reference: the oracle's block-0 output for one token at position 3 after three cached tokens
        ref = O.OracleModel(cfg, ctx=8).load_synthetic(0)
        toks = synth.prompt_ids(cfg, 4, 0)
        for t in toks:
            ref.decode(int(t), want_logits=False)
        want = ref.read_hidden(0)
        # sharded: this rank's heads attend over the oracle's cache (its own KV heads), then O; then the FFN shard
        x = W["token_embd.weight"][int(toks[-1])].astype(np.float32)
        pos = 3
        a = O.rmsnorm(x, W["blk.0.attn_norm.weight"], cfg.eps)
        qh, kvh = cfg.qH // world, cfg.kvH // world
        q = O.rope(O.matvec(a, cut("attn_q.weight")), qh, cfg.d, cfg.ropeDim, cfg.rope_theta, pos)
        kc = np.zeros((pos + 1, kvh * cfg.d), np.float32)
        vc = np.zeros((pos + 1, kvh * cfg.d), np.float32)
        for p in range(pos + 1):
            k, v = ref.read_kv(0, p)
            kc[p] = k[rank * kvh * cfg.d:(rank + 1) * kvh * cfg.d]
            vc[p] = v[rank * kvh * cfg.d:(rank + 1) * kvh * cfg.d]
        # the rank's own K/V row of the new token equals the oracle's rows of its heads
        k_new = O.rope(O.matvec(a, cut("attn_k.weight")), kvh, cfg.d, cfg.ropeDim, cfg.rope_theta, pos)
        assert np.allclose(k_new, kc[pos], atol=1e-6)
        o = O.attention(q, kc, vc, pos + 1, qh, kvh, cfg.d, cfg.eps)
        part = torch.from_numpy(O.matvec(o, cut("attn_output.weight")))
        dist.all_reduce(part)
        x1 = x + part.numpy()
        b = O.rmsnorm(x1, W["blk.0.ffn_norm.weight"], cfg.eps)
        h = O.silu_mul(O.matvec(b, cut("ffn_gate.weight")), O.matvec(b, cut("ffn_up.weight")))
        part = torch.from_numpy(O.matvec(h, cut("ffn_down.weight")))
        dist.all_reduce(part)
        x2 = x1 + part.numpy()
        err = float(np.abs(x2 - want).max() / np.abs(want).max())
        return (rank, uid, err)
    finally:
        dist.destroy_process_group()


def test_two_rank_partition_and_rendezvous():
    from .mp_util import run_ranks
    res = run_ranks(_worker, 2, timeout=120)
    assert {r[0] for r in res} == {0, 1}
    assert res[0][1] == res[1][1] == bytes(range(128))
    for _, _, err in res:
        assert err < 1e-5


def test_shard_ranges_cover_every_matrix_once():
    from nfai_b200 import synth, tp
    for key, world in (("c1", 8), ("c2", 4), ("c3", 8), ("c0", 2)):
        cfg = synth.get_config(key)
        for name, (N, K) in {"attn_q.weight": (cfg.qDim, cfg.H), "attn_output.weight": (cfg.H, cfg.qDim),
                             "ffn_gate.weight": (cfg.F, cfg.H), "ffn_down.weight": (cfg.H, cfg.F),
                             "lm_head": (cfg.V, cfg.H)}.items():
            cover = np.zeros((N if N < 4096 else 4096, 1), np.int32)  # rows are enough to see the tiling
            cols = np.zeros(K, np.int32)
            for r in range(world):
                (r0, r1), (c0, c1) = tp.shard_ranges(cfg, world, r)[name]
                if (c0, c1) == (0, K):
                    cover[min(r0, len(cover)):min(r1, len(cover))] += 1
                else:
                    cols[c0:c1] += 1
                    assert (r0, r1) == (0, N)
            assert cover.max() <= 1 and cols.max() <= 1
            assert cover.all() or cols.all()
    with pytest.raises(ValueError):
        tp.shard_ranges(synth.get_config("c0"), 4, 0)  # kvH = 2 does not divide by 4


def _shared_source_worker(rank: int, world: int, port: int):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from nfai_b200 import synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = synth.get_config("s3", gain_std=0.1)
        src = synth.SharedTensorSource(cfg, 0, dist, torch.device("cpu"))
        same = True
        for name, ne, dt in src.specs:
            a = src.get(name)
            b = synth.gen_tensor(cfg, name, ne, dt, 0)
            same = same and a.dtype == b.dtype and a.shape == b.shape and bool(np.array_equal(a, b))
        src.close()
        return same
    finally:
        dist.destroy_process_group()


def test_ranks_share_the_generation_of_the_synthetic_model():
    """Every tensor is generated by one rank and broadcast: all ranks end up with exactly the tensors a single process
    generates (the benchmark uses this so that N ranks do not generate the model N times)."""
    from .mp_util import run_ranks
    assert run_ranks(_shared_source_worker, 2, timeout=120, port_base=29300) == [True, True]
