"""Host-side mirror of the reference's model interface over the C ABI (what NFAI.Cuda does in C#).

The reference's toolchain (.NET) is not available where this package is developed, so the same call sequence a
C# NFAI.Cuda project makes through P/Invoke is driven from here through ctypes, with the reference's names:
ModelOptions, LlamaModelFactory.TryCreate, LlamaModel (NFAI.Models/ModelOptions.cs, NFAI.Models.Llama3/
LlamaModelFactory.cs, LlamaModel.cs). Token ids go in and come out (the tokenizer is untouched CPU string code).
Every compute step runs in libnfai_cuda.so; nothing here falls back to the CPU.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np

from . import _lib
from ._lib import F16, F32, HParams, NfaiError, check
from .gguf_io import ComputeCollection


@dataclass
class ModelOptions:
    """NFAI.Models/ModelOptions.cs:3-8 plus optional fields with defaults so existing configurations still bind."""
    GGUFPath: str = ""
    KVCacheSize: int = 512
    KVCacheDType: str = "auto"   # "f32" (the reference's cache type), "f16", or "auto" = the weights' type
    Device: int = 0
    WeightDType: str = "auto"    # "auto" = as stored in the file


class CudaContext:
    """One CUDA device: stream, pinned staging, timing events (replaces Vk + Device + VulkanBufferManager)."""

    def __init__(self, device: int = 0, rank: int = 0, world: int = 1, nccl_uid: Optional[bytes] = None):
        lib = _lib.load()
        h = C.c_void_p()
        if world > 1:
            buf = C.create_string_buffer(nccl_uid, len(nccl_uid))
            check(lib.nfai_ctx_create_tp(device, rank, world, buf, len(nccl_uid), C.byref(h)))
        else:
            check(lib.nfai_ctx_create(device, C.byref(h)))
        self.handle = h
        self.device, self.rank, self.world = device, rank, world

    @staticmethod
    def tp_unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        check(_lib.load().nfai_tp_unique_id(buf, 128))
        return buf.raw

    def export_peer(self) -> bytes:
        buf = C.create_string_buffer(128)
        check(_lib.load().nfai_tp_export_peer(self.handle, buf, 128), self.handle)
        return buf.raw

    def import_peers(self, descs: bytes):
        n = len(descs) // 128
        buf = C.create_string_buffer(descs, len(descs))
        check(_lib.load().nfai_tp_import_peers(self.handle, buf, n), self.handle)

    def close(self):
        if self.handle:
            _lib.load().nfai_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _dtype_code(name: str) -> int:
    return {"f32": F32, "f16": F16}[name]


class LlamaModel:
    """IInferenceProvider for general.architecture == "llama" (NFAI.Models.Llama3/LlamaModel.cs:10-175).

    The constructor reads the same metadata keys as the reference (:23-39), finds the same tensors (:43,58 and
    NFAI.Vulkan.Shaders/TransformerBlock.cs:41-99) and streams them to the device.
    """

    def __init__(self, ctx: CudaContext, metadata: Dict[str, object], tensors: Sequence[ComputeCollection],
                 context_size: int = 1024, kv_dtype: str = "auto", weight_dtype: str = "auto",
                 widen_half: bool = False):
        self.ctx = ctx
        self._lib = _lib.load()
        md = metadata
        self.bos_token = int(md["tokenizer.ggml.bos_token_id"])
        self.eos_token = int(md["tokenizer.ggml.eos_token_id"])
        rope_theta = float(md["llama.rope.freq_base"])
        rope_dim = int(md["llama.rope.dimension_count"])
        eps = float(next((v for k, v in md.items() if "epsilon" in k), 0.0))
        qH = int(md["llama.attention.head_count"])
        kvH = int(md["llama.attention.head_count_kv"])
        d = int(md["llama.attention.key_length"])
        L = int(md["llama.block_count"])
        self.ModelName = str(md.get("general.name", "unknown"))
        by_name = {t.Name: t for t in tensors}
        embd = next(t for t in tensors if "token" in t.Name)          # LlamaModel.cs:43
        H, V = embd.Shape[0], embd.Shape[1]
        gate0 = next(t for t in tensors if "blk.0.ffn_gate" in t.Name)
        F = gate0.Shape[1]
        tied = "output.weight" not in by_name
        stored = "f16" if embd.TypeSize == 2 else "f32"
        wdt = stored if weight_dtype == "auto" else weight_dtype
        kvdt = wdt if kv_dtype == "auto" else kv_dtype
        self.hp = HParams(H, L, qH, kvH, d, rope_dim, F, V, int(context_size), eps, rope_theta, _dtype_code(wdt),
                          _dtype_code(kvdt), 1 if tied else 0)
        self.V, self.H, self.L = V, H, L
        self.kv_dtype, self.weight_dtype = kvdt, wdt
        h = C.c_void_p()
        check(self._lib.nfai_model_create(ctx.handle, C.byref(self.hp), C.byref(h)), ctx.handle)
        self.handle = h
        try:
            names = ["token_embd.weight", "output_norm.weight"] + ([] if tied else ["output.weight"])
            for i in range(L):
                names += [f"blk.{i}.{n}.weight" for n in ("attn_norm", "attn_q", "attn_k", "attn_v", "attn_output",
                                                          "ffn_norm", "ffn_gate", "ffn_up", "ffn_down")]
            for name in names:
                # the reference matches by substring (x.Name.Contains(...)); exact names are the same tensors
                t = by_name.get(name) or next(x for x in tensors if name.rsplit(".weight", 1)[0] in x.Name)
                self.upload(t, widen_half=widen_half)
            check(self._lib.nfai_model_finalize(self.handle), ctx.handle)
        except Exception:
            self.Dispose()
            raise

    @classmethod
    def from_gguf_native(cls, ctx: CudaContext, path: str, context_size: int = 1024, kv_dtype: str = "auto") -> "LlamaModel":
        """Load a GGUF file with the library's native loader (mmap, raw float16 pass-through)."""
        self = cls.__new__(cls)
        self.ctx = ctx
        self._lib = _lib.load()
        h = C.c_void_p()
        kv = -1 if kv_dtype == "auto" else _dtype_code(kv_dtype)
        check(self._lib.nfai_model_load_gguf(ctx.handle, path.encode(), int(context_size), kv, C.byref(h)), ctx.handle)
        self.handle = h
        self.hp = HParams()
        check(self._lib.nfai_model_get_hparams(h, C.byref(self.hp)), ctx.handle)
        self.V, self.H, self.L = self.hp.V, self.hp.H, self.hp.L
        self.kv_dtype = "f16" if self.hp.kv_dtype == F16 else "f32"
        self.weight_dtype = "f16" if self.hp.weight_dtype == F16 else "f32"
        self.ModelName = os.path.basename(path)
        self.bos_token, self.eos_token = 0, 1
        return self

    # -- upload -------------------------------------------------------------------------------------------------
    def upload(self, t: ComputeCollection, widen_half: bool = False):
        shape = (C.c_uint64 * len(t.Shape))(*t.Shape)
        src = F32 if (t.TypeSize == 4 or widen_half) else F16
        check(self._lib.nfai_model_tensor_begin(self.handle, t.Name.encode(), src, shape, len(t.Shape)), self.ctx.handle)
        for chunk in t.get_data_raw(widen_half=widen_half):
            check(self._lib.nfai_model_tensor_chunk(self.handle, chunk, len(chunk)), self.ctx.handle)
        check(self._lib.nfai_model_tensor_end(self.handle), self.ctx.handle)

    # -- the hot path -------------------------------------------------------------------------------------------
    def _fp(self, a: Optional[np.ndarray]):
        return a.ctypes.data_as(C.POINTER(C.c_float)) if a is not None else None

    def prefill(self, tokens: Iterable[int], want_logits: bool = True) -> Tuple[Optional[np.ndarray], int]:
        toks = np.ascontiguousarray(np.fromiter((int(t) for t in tokens), dtype=np.uint32))
        logits = np.empty(self.V, np.float32) if want_logits else None
        am = C.c_uint32()
        check(self._lib.nfai_prefill(self.handle, toks.ctypes.data_as(C.POINTER(C.c_uint32)), toks.size,
                                     self._fp(logits), C.byref(am)), self.ctx.handle)
        return logits, am.value

    def decode(self, token: int, want_logits: bool = True) -> Tuple[Optional[np.ndarray], int]:
        logits = np.empty(self.V, np.float32) if want_logits else None
        am = C.c_uint32()
        check(self._lib.nfai_decode(self.handle, int(token), self._fp(logits), C.byref(am)), self.ctx.handle)
        return logits, am.value

    def decode_greedy(self, first_token: int, n_steps: int) -> Tuple[np.ndarray, float]:
        out = np.empty(n_steps, np.uint32)
        ms = C.c_float()
        check(self._lib.nfai_decode_greedy(self.handle, int(first_token), n_steps,
                                           out.ctypes.data_as(C.POINTER(C.c_uint32)), C.byref(ms)), self.ctx.handle)
        return out, ms.value

    def decode_sampled(self, first_token: int, us: Sequence[float], temperature: float = 0.5, top_p: float = 0.95,
                       top_k: int = 40) -> Tuple[np.ndarray, float]:
        """len(us) steps with SamplingUtils.TopP after each, fed back on the device; returns (tokens, milliseconds)."""
        u = np.ascontiguousarray(us, np.float32)
        out = np.empty(len(u), np.uint32)
        ms = C.c_float()
        check(self._lib.nfai_decode_sampled(self.handle, int(first_token), len(u), temperature, top_p, top_k,
                                            u.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), C.byref(ms)),
              self.ctx.handle)
        return out, ms.value

    def snapshot(self) -> "KvSnapshot":
        """Copy of the cache rows, logits and position at this point (device memory); restore() rewinds to it."""
        h = C.c_void_p()
        check(self._lib.nfai_kv_snapshot_create(self.handle, C.byref(h)), self.ctx.handle)
        return KvSnapshot(self, h)

    def sample_top_p(self, temperature: float = 0.5, top_p: float = 0.95, top_k: int = 40, u: float = 0.5) -> int:
        """SamplingUtils.TopP on the device over the last step's logits; `u` is the uniform draw."""
        tok = C.c_uint32()
        check(self._lib.nfai_sample_top_p(self.handle, temperature, top_p, top_k, u, C.byref(tok)), self.ctx.handle)
        return tok.value

    def run_tokens(self, prompt: Iterable[int], max_new: int, stop_at_eos: bool = False) -> List[int]:
        """LlamaModel.RunAsync with token ids in place of text and arg-max in place of TopP
        (LlamaModel.cs:99-174): ingest the prompt, then feed each prediction back."""
        _, tk = self.prefill(prompt, want_logits=False)
        out = [tk]
        while len(out) < max_new and not (stop_at_eos and tk == self.eos_token):
            _, tk = self.decode(tk, want_logits=False)
            out.append(tk)
        return out

    @property
    def position(self) -> int:
        p = C.c_uint32()
        check(self._lib.nfai_position(self.handle, C.byref(p)), self.ctx.handle)
        return p.value

    def reset(self):
        check(self._lib.nfai_reset(self.handle), self.ctx.handle)

    def set_position(self, pos: int):
        check(self._lib.nfai_set_position(self.handle, int(pos)), self.ctx.handle)

    # -- taps ---------------------------------------------------------------------------------------------------
    def _kv_len(self) -> int:
        return self.hp.kvH * self.hp.d // self.ctx.world

    def read_kv(self, layer: int, pos: int) -> Tuple[np.ndarray, np.ndarray]:
        k = np.empty(self._kv_len(), np.float32)
        v = np.empty(self._kv_len(), np.float32)
        check(self._lib.nfai_read_kv(self.handle, layer, pos, self._fp(k), self._fp(v)), self.ctx.handle)
        return k, v

    def write_kv(self, layer: int, pos: int, k: np.ndarray, v: np.ndarray):
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        check(self._lib.nfai_write_kv(self.handle, layer, pos, self._fp(k), self._fp(v)), self.ctx.handle)

    def write_kv_range(self, layer: int, pos0: int, k: np.ndarray, v: np.ndarray):
        """k, v: [n][kv width] rows for positions pos0 .. pos0+n-1 of one layer."""
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        assert k.shape == v.shape and k.ndim == 2 and k.shape[1] == self._kv_len()
        check(self._lib.nfai_write_kv_range(self.handle, layer, pos0, k.shape[0], self._fp(k), self._fp(v)),
              self.ctx.handle)

    def read_hidden(self, layer: int) -> np.ndarray:
        out = np.empty(self.H, np.float32)
        check(self._lib.nfai_read_hidden(self.handle, layer, self._fp(out)), self.ctx.handle)
        return out

    # -- measurement --------------------------------------------------------------------------------------------
    KERNELS = {"ffn_gate_up": 0, "ffn_down": 1, "qkv_rope": 2, "attn_out": 3, "lm_head": 4, "attention": 5}

    def profile_kernel(self, which: str, iters: int) -> Tuple[float, int]:
        ms = C.c_float()
        nbytes = C.c_uint64()
        check(self._lib.nfai_profile_kernel(self.handle, self.KERNELS[which], iters, C.byref(ms), C.byref(nbytes)),
              self.ctx.handle)
        return ms.value, nbytes.value

    def tune(self, which: str, mode: int, rows_per_warp: int, depth: int, ctas_per_sm: int):
        check(self._lib.nfai_model_tune(self.handle, self.KERNELS[which], mode, rows_per_warp, depth, ctas_per_sm),
              self.ctx.handle)

    def set_prefetch(self, lookahead_bytes: int, extra_bytes: int = 0, mode: int = 1):
        check(self._lib.nfai_model_set_prefetch(self.handle, int(lookahead_bytes), int(extra_bytes), mode),
              self.ctx.handle)

    def step_launches(self) -> int:
        n = C.c_int()
        check(self._lib.nfai_step_launches(self.handle, C.byref(n)), self.ctx.handle)
        return n.value

    def Dispose(self):
        if getattr(self, "handle", None):
            self._lib.nfai_model_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.Dispose()
        except Exception:
            pass


class KvSnapshot:
    """Handle of nfai_kv_snapshot_*: belongs to one model, close() it before the model."""

    def __init__(self, model: "LlamaModel", handle):
        self.model, self.handle = model, handle

    @property
    def position(self) -> int:
        return int(self.model._lib.nfai_kv_snapshot_position(self.handle))

    def restore(self, model: Optional["LlamaModel"] = None):
        m = model or self.model
        check(m._lib.nfai_kv_snapshot_restore(m.handle, self.handle), m.ctx.handle)

    def close(self):
        if self.handle:
            self.model._lib.nfai_kv_snapshot_destroy(self.handle)
            self.handle = None


class LlamaModelFactory:
    """NFAI.Models.Llama3/LlamaModelFactory.cs:7-45: the parameterless constructor opens the device, TryCreate
    accepts general.architecture == "llama"."""

    def __init__(self, device: int = 0, rank: int = 0, world: int = 1, nccl_uid: Optional[bytes] = None):
        self.ctx = CudaContext(device, rank, world, nccl_uid)

    def try_create(self, metadata: Dict[str, object], tensors: Sequence[ComputeCollection],
                   options: ModelOptions) -> Optional[LlamaModel]:
        if str(metadata.get("general.architecture", "")) != "llama":
            return None
        return LlamaModel(self.ctx, metadata, tensors, options.KVCacheSize, kv_dtype=options.KVCacheDType,
                          weight_dtype=options.WeightDType)

    TryCreate = try_create

    def Dispose(self):
        self.ctx.close()


def synthetic_tensors(cfg, seed: int = 0, dist=None, device=None) -> List[ComputeCollection]:
    """The seeded synthetic model as lazy in-memory ComputeCollections (no file). With `dist` (an initialised
    torch.distributed module) and `device` the ranks of the job share the work of generating it."""
    from . import synth
    src = synth.SharedTensorSource(cfg, seed, dist, device) if dist is not None else synth.TensorSource(cfg, seed)
    return [_LazySynth(src, name, ne, dt) for name, ne, dt in src.specs]


class _LazySynth(ComputeCollection):
    """Generates its values when streamed, so a large model never sits in host memory twice."""

    def __init__(self, source, name, ne, dt):
        super().__init__(name, ne, 2 if dt == "f16" else 4)
        self._source = source  # shared by the tensors of one model: generates a few tensors ahead on worker threads

    def get_data_raw(self, widen_half: bool = False):
        self._array = self._source.get(self.Name)
        try:
            yield from super().get_data_raw(widen_half=widen_half)
        finally:
            self._array = None


def create_synthetic_model(cfg, ctx_size: int, *, seed: int = 0, device: int = 0, kv_dtype: str = "auto",
                           factory: Optional[LlamaModelFactory] = None, widen_half: bool = False) -> LlamaModel:
    from . import synth
    factory = factory or LlamaModelFactory(device)
    model = LlamaModel(factory.ctx, synth.metadata(cfg), synthetic_tensors(cfg, seed), ctx_size, kv_dtype=kv_dtype,
                       widen_half=widen_half)
    model._factory = factory  # keep the context alive as long as the model
    return model
