"""Tensor-parallel plumbing on the host: which part of each tensor a rank keeps, and the rendezvous that shares the
NCCL unique id. The library does the sharding itself at upload (csrc/api.cu: resolve_target); `shard_ranges` states
the same partition in Python so that it can be checked without a GPU and used by hosts that pre-slice their files.

Partition (the reference is single-device; this follows the classic column-then-row split of each block):
  attn_q / attn_k / attn_v : output rows of the rank's KV-head group (and of the query heads that share it)
  attn_output              : input columns of those query heads          -> partial sums, all-reduced
  ffn_gate / ffn_up        : output rows [r F/n, (r+1) F/n)
  ffn_down                 : input columns [r F/n, (r+1) F/n)            -> partial sums, all-reduced
  LM head                  : vocabulary rows [r V/n, (r+1) V/n)           -> (max, index) pairs gathered
  token_embd, norm gains   : replicated
"""
from __future__ import annotations

from typing import Callable, Dict, Optional, Tuple

Range = Tuple[int, int]


def check_divisible(cfg, world: int) -> None:
    if world not in (1, 2, 4, 8):
        raise ValueError("tensor-parallel width must be 1, 2, 4 or 8")
    if cfg.kvH % world or cfg.F % world or cfg.V % world:
        raise ValueError("kvH, F and V must divide by the tensor-parallel width")


def shard_ranges(cfg, world: int, rank: int) -> Dict[str, Tuple[Range, Range]]:
    """suffix of the tensor name -> ((row_lo, row_hi), (col_lo, col_hi)) of the [N][K] matrix this rank keeps."""
    check_divisible(cfg, world)
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    qd, kvd, f, v = cfg.qDim // world, cfg.kvDim // world, cfg.F // world, cfg.V // world
    H = cfg.H
    return {
        "attn_q.weight": ((rank * qd, (rank + 1) * qd), (0, H)),
        "attn_k.weight": ((rank * kvd, (rank + 1) * kvd), (0, H)),
        "attn_v.weight": ((rank * kvd, (rank + 1) * kvd), (0, H)),
        "attn_output.weight": ((0, H), (rank * qd, (rank + 1) * qd)),
        "ffn_gate.weight": ((rank * f, (rank + 1) * f), (0, H)),
        "ffn_up.weight": ((rank * f, (rank + 1) * f), (0, H)),
        "ffn_down.weight": ((0, H), (rank * f, (rank + 1) * f)),
        "lm_head": ((rank * v, (rank + 1) * v), (0, H)),
    }


def share_unique_id(dist, rank: int, make_uid: Callable[[], bytes], device: Optional[str] = None) -> bytes:
    """Rank 0 makes the 128-byte NCCL unique id, every rank returns the same bytes (broadcast over `dist`)."""
    import torch
    buf = torch.zeros(128, dtype=torch.uint8, device=device or "cpu")
    if rank == 0:
        uid = make_uid()
        if len(uid) != 128:
            raise ValueError("unique id must be 128 bytes")
        buf.copy_(torch.frombuffer(bytearray(uid), dtype=torch.uint8))
    dist.broadcast(buf, 0)
    return bytes(buf.cpu().numpy().tobytes())


def connect_peers(dist, ctx, device: Optional[str] = None) -> None:
    """Gather every rank's 128-byte exchange-area descriptor and import the whole set on this rank, so that the
    all-reduces of the decode step run as the library's own peer-memory kernel instead of NCCL calls."""
    import torch
    mine = torch.frombuffer(bytearray(ctx.export_peer()), dtype=torch.uint8).to(device or "cpu")
    world = dist.get_world_size()
    parts = [torch.zeros(128, dtype=torch.uint8, device=device or "cpu") for _ in range(world)]
    dist.all_gather(parts, mine)
    ctx.import_peers(b"".join(bytes(p.cpu().numpy().tobytes()) for p in parts))
