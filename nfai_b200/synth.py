"""Seeded synthetic Llama-3-architecture models (stand-ins for real checkpoints, which need a network).

Weights are N(0, 0.02^2) in the configuration's storage type, RMSNorm gains are 1.0 (float32), prompts are
uniform random token ids. Every tensor has its own RNG stream derived from (seed, tensor name), so a tensor
can be generated on its own, in any order, in a file or in memory, with identical bits.

Tensor names and shapes follow what the reference looks up:
  token_embd.weight, output_norm.weight (NFAI.Models.Llama3/LlamaModel.cs:43,58) and
  blk.{i}.{attn_norm,attn_q,attn_k,attn_v,attn_output,ffn_norm,ffn_down,ffn_gate,ffn_up}.weight
  (NFAI.Vulkan.Shaders/TransformerBlock.cs:41-99).
Shapes are given in GGUF "ne" order (innermost first), the order NFAI.GGUF/Parser.cs:252-258 reads; the
numpy arrays are the reverse, i.e. W[N][K] row-major, so that W[n*K + k] is the element the reference's
matrix multiply reads (NFAI.Vulkan.Shaders/MatrixMultiplyShader.cs:260).
"""
from __future__ import annotations

import zlib
from dataclasses import dataclass, replace
from typing import Dict, Iterator, List, Tuple

import numpy as np


@dataclass(frozen=True)
class ModelConfig:
    name: str
    H: int
    L: int
    qH: int
    kvH: int
    d: int
    F: int
    V: int
    dtype: str = "f32"          # storage type of the matrices: "f32" or "f16"
    tied: bool = True
    rope_theta: float = 500000.0
    eps: float = 1e-5
    gain_std: float = 0.0        # 0 -> RMSNorm gains exactly 1.0 (the benchmark configurations)
    weight_std: float = 0.02

    @property
    def qDim(self) -> int:
        return self.qH * self.d

    @property
    def kvDim(self) -> int:
        return self.kvH * self.d

    @property
    def ropeDim(self) -> int:
        return self.d

    def matrix_params(self) -> int:
        per_layer = self.H * self.qDim + 2 * self.H * self.kvDim + self.qDim * self.H + 3 * self.H * self.F
        head = self.V * self.H
        return self.L * per_layer + head * (1 if self.tied else 2)

    def streamed_matrix_params(self) -> int:
        """Matrix elements one decode step reads: every layer matrix once plus one LM-head matrix."""
        per_layer = self.H * self.qDim + 2 * self.H * self.kvDim + self.qDim * self.H + 3 * self.H * self.F
        return self.L * per_layer + self.V * self.H


# The benchmark configurations, in the order the baseline lists them.
CONFIGS: Dict[str, ModelConfig] = {
    # tiny FP32 model; head_dim 32
    "c0": ModelConfig("c0-tiny-f32", H=256, L=2, qH=8, kvH=2, d=32, F=768, V=4096, dtype="f32"),
    # same size, head_dim 64: the one small shape inside the reference's self-consistent envelope
    "c0p": ModelConfig("c0p-tiny-f32-d64", H=256, L=2, qH=4, kvH=2, d=64, F=768, V=4096, dtype="f32"),
    "c1": ModelConfig("llama-3.2-1b-arch-f16", H=2048, L=16, qH=32, kvH=8, d=64, F=8192, V=128256, dtype="f16"),
    "c2": ModelConfig("llama-3.2-3b-arch-f16", H=3072, L=28, qH=24, kvH=8, d=128, F=8192, V=128256, dtype="f16"),
    "c3": ModelConfig("llama-3.1-8b-arch-f16", H=4096, L=32, qH=32, kvH=8, d=128, F=14336, V=128256, dtype="f16",
                      tied=False),
    # scaled-down FP16 models with the 1B/3B head geometry, for parity tests the CPU finishes in seconds
    "s1": ModelConfig("scaled-1b-f16", H=2048, L=2, qH=32, kvH=8, d=64, F=8192, V=8192, dtype="f16"),
    "s2": ModelConfig("scaled-3b-f16", H=768, L=2, qH=6, kvH=2, d=128, F=2048, V=4096, dtype="f16"),
    "s3": ModelConfig("scaled-8b-f16-untied", H=512, L=2, qH=8, kvH=2, d=64, F=1536, V=2048, dtype="f16",
                      tied=False),
}
CONFIGS["c4"] = replace(CONFIGS["c1"], name="llama-3.2-1b-arch-f16-longctx")


def get_config(key: str, **overrides) -> ModelConfig:
    cfg = CONFIGS[key]
    return replace(cfg, **overrides) if overrides else cfg


def tensor_specs(cfg: ModelConfig) -> List[Tuple[str, Tuple[int, ...], str]]:
    """(name, GGUF ne-order shape, dtype) for every tensor of the model, in file order."""
    w = cfg.dtype
    specs: List[Tuple[str, Tuple[int, ...], str]] = [("token_embd.weight", (cfg.H, cfg.V), w)]
    for i in range(cfg.L):
        p = f"blk.{i}."
        specs += [
            (p + "attn_norm.weight", (cfg.H,), "f32"),
            (p + "attn_q.weight", (cfg.H, cfg.qDim), w),
            (p + "attn_k.weight", (cfg.H, cfg.kvDim), w),
            (p + "attn_v.weight", (cfg.H, cfg.kvDim), w),
            (p + "attn_output.weight", (cfg.qDim, cfg.H), w),
            (p + "ffn_norm.weight", (cfg.H,), "f32"),
            (p + "ffn_gate.weight", (cfg.H, cfg.F), w),
            (p + "ffn_up.weight", (cfg.H, cfg.F), w),
            (p + "ffn_down.weight", (cfg.F, cfg.H), w),
        ]
    specs.append(("output_norm.weight", (cfg.H,), "f32"))
    if not cfg.tied:
        specs.append(("output.weight", (cfg.H, cfg.V), w))
    return specs


def _rng(seed: int, name: str) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(np.random.SeedSequence([int(seed), zlib.crc32(name.encode())])))


def gen_tensor(cfg: ModelConfig, name: str, shape_ne: Tuple[int, ...], dtype: str, seed: int = 0) -> np.ndarray:
    """The tensor's values as a C-contiguous numpy array of shape reversed(shape_ne)."""
    shape = tuple(reversed(shape_ne))
    rng = _rng(seed, name)
    if name.endswith("_norm.weight"):
        if cfg.gain_std == 0.0:
            return np.ones(shape, dtype=np.float32)
        return (1.0 + cfg.gain_std * rng.standard_normal(shape, dtype=np.float32)).astype(np.float32)
    a = rng.standard_normal(shape, dtype=np.float32)
    a *= np.float32(cfg.weight_std)
    return a.astype(np.float16) if dtype == "f16" else a


class TensorSource:
    """Generates the tensors of one synthetic model a few ahead of the consumer, on worker threads.

    Every tensor has its own random stream (seed, name), so the values do not depend on who generates them or in which
    order; numpy fills large arrays without the interpreter lock, so the workers run in parallel. At most
    `workers` tensors are held at a time."""

    def __init__(self, cfg: ModelConfig, seed: int = 0, workers: int = 0):
        import concurrent.futures as cf
        import os
        self.cfg, self.seed = cfg, seed
        self.specs = list(tensor_specs(cfg))
        self.index = {name: i for i, (name, _ne, _dt) in enumerate(self.specs)}
        # one process per GPU shares the host cores: divide them among the ranks
        ranks = max(1, int(os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")) or 1))
        self.workers = workers or max(1, min(8, ((os.cpu_count() or 2) - 1) // ranks))
        self.pool = cf.ThreadPoolExecutor(max_workers=self.workers)
        self.futures = {}

    def _submit(self, i: int):
        if 0 <= i < len(self.specs) and i not in self.futures:
            name, ne, dt = self.specs[i]
            self.futures[i] = self.pool.submit(gen_tensor, self.cfg, name, ne, dt, self.seed)

    def get(self, name: str) -> np.ndarray:
        i = self.index[name]
        self._submit(i)
        for j in range(i + 1, i + 1 + self.workers):
            self._submit(j)
        return self.futures.pop(i).result()

    def close(self):
        self.pool.shutdown(wait=False, cancel_futures=True)
        self.futures.clear()


class SharedTensorSource(TensorSource):
    """The same tensors for several ranks of one job without every rank generating all of them: tensor i is generated
    by rank i mod world and broadcast over the job's process group (device to device), so the host cores generate the
    model once instead of once per rank. Every rank must ask for the tensors in the same order."""

    def __init__(self, cfg: ModelConfig, seed: int, dist, device):
        import os
        self.dist, self.device = dist, device
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        cpus = (os.cpu_count() or 2) - 1
        super().__init__(cfg, seed, workers=max(1, min(8, cpus // max(1, int(os.environ.get("LOCAL_WORLD_SIZE", self.world))))))

    def _submit(self, i: int):
        if i % self.world == self.rank:
            super()._submit(i)

    def get(self, name: str) -> np.ndarray:
        import torch
        i = self.index[name]
        _n, ne, dt = self.specs[i]
        owner = i % self.world
        np_dtype = np.float16 if (dt == "f16" and not name.endswith("_norm.weight")) else np.float32
        shape = tuple(reversed(ne))
        if owner == self.rank:
            for j in range(i, i + self.world * (self.workers + 1), self.world):
                self._submit(j)
            arr = np.ascontiguousarray(self.futures.pop(i).result())
            assert arr.dtype == np_dtype and arr.shape == shape, (name, arr.dtype, arr.shape)
            t = torch.from_numpy(arr.reshape(-1).view(np.uint8)).to(self.device)
        else:
            t = torch.empty(int(np.prod(shape)) * np.dtype(np_dtype).itemsize, dtype=torch.uint8, device=self.device)
        self.dist.broadcast(t, src=owner)
        if owner != self.rank:
            arr = t.cpu().numpy().view(np_dtype).reshape(shape)
        return arr


def iter_tensors(cfg: ModelConfig, seed: int = 0) -> Iterator[Tuple[str, Tuple[int, ...], str, np.ndarray]]:
    src = TensorSource(cfg, seed)
    try:
        for name, shape_ne, dtype in src.specs:
            yield name, shape_ne, dtype, src.get(name)
    finally:
        src.close()


def prompt_ids(cfg: ModelConfig, n: int, seed: int = 0) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64(int(seed) + 1))
    return rng.integers(0, cfg.V, size=n, dtype=np.int64).astype(np.uint32)


def metadata(cfg: ModelConfig) -> Dict[str, object]:
    """The metadata keys the reference reads (NFAI.Models.Llama3/LlamaModel.cs:23-39,
    NFAI.Models.Llama3/LlamaModelFactory.cs:36)."""
    return {
        "general.architecture": "llama",
        "general.name": cfg.name,
        "general.alignment": 32,
        "llama.block_count": cfg.L,
        "llama.embedding_length": cfg.H,
        "llama.feed_forward_length": cfg.F,
        "llama.attention.head_count": cfg.qH,
        "llama.attention.head_count_kv": cfg.kvH,
        "llama.attention.key_length": cfg.d,
        "llama.attention.value_length": cfg.d,
        "llama.attention.layer_norm_rms_epsilon": cfg.eps,
        "llama.rope.freq_base": cfg.rope_theta,
        "llama.rope.dimension_count": cfg.ropeDim,
        "llama.vocab_size": cfg.V,
        "tokenizer.ggml.bos_token_id": 0,
        "tokenizer.ggml.eos_token_id": 1,
    }


def decode_bytes(cfg: ModelConfig, pos: int, kv_bytes: int) -> int:
    """Algorithmic bytes one decode step at 0-based position `pos` must move: every matrix once in its
    storage type, the norm gains, one embedding row, K and V of positions 0..pos read and one K,V row written.
    Activations, partial results and logits are not counted."""
    wbytes = 2 if cfg.dtype == "f16" else 4
    gains = (2 * cfg.L + 1) * cfg.H * 4
    kv_read = 2 * cfg.L * cfg.kvDim * kv_bytes * (pos + 1)
    kv_write = 2 * cfg.L * cfg.kvDim * kv_bytes
    return cfg.streamed_matrix_params() * wbytes + gains + cfg.H * wbytes + kv_read + kv_write
