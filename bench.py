"""Benchmark of the Llama-3 batch-1 decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c1]

A step is one decoded token (one replay of the captured decode step). At N = 1 the workload is the
Llama-3.2-1B-architecture FP16 model, 128-token random prompt, then K greedy decode steps; for N > 1 the same
model runs tensor-parallel over the N GPUs (strong scaling), one rank per GPU under torchrun.
Prints ONE JSON line on rank 0.

  value      tokens/s with everything resident in HBM: K greedy steps fed back on the device, timed with CUDA events
             on the library's stream, max over ranks.
  e2e        tokens/s through the reference-facing call (nfai_decode): host token in, arg-max out, copies and
             synchronisation inside the timed region.
  roofline   the dominant kernel (FFN gate/up GEMV): algorithmic bytes per launch / mean launch time, against the
             measured HBM copy bandwidth.
  cpu_baseline  the CPU oracle (a port of the reference's arithmetic; the reference itself needs .NET + Vulkan and
             cannot run here) timed on the host cores on a few tokens of the same workload.

--impl reference times that CPU port with all host threads on the same workload (rank 0 only).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel (FFN gate/up GEMV of configs[1]
# on one GPU), from an ncu capture of this kernel; it goes stale when the kernel's memory behaviour changes, so the
# capture it came from is named beside it.
NCU_TRAFFIC = {("c1", 1): {"bytes": 67165440 + 710400,
                           "capture": "ncu --set full --clock-control none -k regex:gemv_kernel -s 170 -c 4 of "
                                      "bench.py --steps 2 --warmup 3 --prompt-len 2 --min-timed-s 0: the gate/up launch "
                                      "(67.165 MB read + 0.710 MB written against 67.117 MB algorithmic)"}}
PROMPT_LEN = 128
MIN_TIMED_S = 1.0  # the K-step loop is repeated until this much device time has been measured; the median is reported


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


def measured_tflops():
    """(sustained, burst) dense bf16 TFLOP/s of this pool's B200s; the fallback is an earlier measurement."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as fh:
            d = json.load(fh)
            return float(d["bf16_tflops_sustained"]), float(d["bf16_tflops"]), "measured"
    except Exception:
        return 1400.0, 1590.0, "fallback"


def parity_against_fixture(logits, greedy_tokens):
    """The benchmark model against the committed fixture of the same model: logits after the prompt at 2 048 fixed
    indices (CPU oracle and one-GPU run) and the first greedy tokens."""
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "bench_c1_parity.npz")
    if not os.path.exists(path):
        return {"unavailable": "fixture missing"}
    g = np.load(path)
    sub = np.asarray(logits, np.float32)[g["idx"]]
    out = {"max_abs_vs_oracle": float(np.abs(sub - g["oracle_logits"]).max()), "tolerance_abs": 2e-2,
           "argmax_equals_oracle": bool(int(np.argmax(logits)) == int(g["oracle_argmax"]))}
    n = min(len(greedy_tokens), len(g["oracle_greedy"]) - 1)
    out["greedy_tokens_equal_oracle"] = int(sum(int(a) == int(b) for a, b in zip(greedy_tokens[:n], g["oracle_greedy"][1:1 + n])))
    out["greedy_tokens_compared"] = n
    if "gpu1_logits" in g.files:
        out["max_abs_vs_tp1_golden"] = float(np.abs(sub - g["gpu1_logits"]).max())
        out["tokens_equal"] = bool(all(int(a) == int(b) for a, b in zip(greedy_tokens[:n], g["gpu1_greedy"][1:1 + n])))
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 9:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline(cfg, threads: int, tokens: int, seed: int = 0):
    """Time `tokens` decode steps of the CPU oracle at positions PROMPT_LEN.. (cache rows below are zero-filled;
    the arithmetic and the bytes moved are those of the real workload)."""
    from oracle import oracle as O
    m = O.OracleModel(cfg, ctx=PROMPT_LEN + tokens + 2).load_synthetic(seed)
    O.set_threads(threads)
    m.set_position(PROMPT_LEN)
    m.decode(1)  # warm-up token (page in the weights)
    t0 = time.perf_counter()
    tk = 1
    for _ in range(tokens):
        tk = O.argmax(m.decode(tk))
    dt = time.perf_counter() - t0
    m.close()
    return tokens / dt, dt / tokens


def workload_name(cfg_key: str, cfg, steps: int) -> str:
    label = f"configs[{cfg_key[1:]}]" if cfg_key[0] == "c" else cfg_key
    return (f"{label}: {cfg.name} batch 1, {PROMPT_LEN}-token uniform-random prompt, "
            f"{steps} greedy decode steps")


def run_reference(args, cfg):
    """The reference's arithmetic on the host cores (CPU port; the reference's own Vulkan path is unavailable)."""
    from oracle import oracle as O
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    O.set_threads(threads)
    m = O.OracleModel(cfg, ctx=PROMPT_LEN + args.warmup + args.steps + 2).load_synthetic(args.seed)
    m.set_position(PROMPT_LEN)
    tk = 1
    t_w = time.perf_counter()
    for _ in range(max(1, args.warmup)):
        tk = O.argmax(m.decode(tk))
    per_tok = (time.perf_counter() - t_w) / max(1, args.warmup)
    budget_s = 150.0
    steps = max(1, min(args.steps, int(budget_s / max(per_tok, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(steps):
        tk = O.argmax(m.decode(tk))
    dt = time.perf_counter() - t0
    val = steps / dt
    sample = f"{steps} decode steps at positions {PROMPT_LEN + max(1, args.warmup)}.. of the same model (KV rows below are zero-filled)"
    line = {
        "impl": "reference", "metric": "decode tok/s (batch 1)", "value": val, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(args.config, cfg, args.steps), "weights": cfg.dtype,
                   "note": "CPU port of the reference's shader arithmetic; the reference's Vulkan path (GPU or lavapipe) is unavailable on this box"},
        "cpu_baseline": {"value": val, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, cfg):
    import torch

    from nfai_b200 import LlamaModel, LlamaModelFactory, synth, synthetic_tensors

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    dist = None
    uid = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        from nfai_b200 import CudaContext, tp
        uid = tp.share_unique_id(dist, rank, CudaContext.tp_unique_id, device="cuda")

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    K, W = args.steps, max(args.warmup, 3)
    ctx_size = PROMPT_LEN + max(W + K, 16) + 8  # room for the parity check's 15 greedy steps whatever K is
    factory = LlamaModelFactory(local_rank, rank, world, uid)
    exchange = "none"
    if world > 1:
        exchange = "nccl"
        if not args.nccl_allreduce:
            from nfai_b200 import tp as _tp
            _tp.connect_peers(dist, factory.ctx, device="cuda")
            exchange = "peer-memory push all-reduce (own kernel over NVLink)"
    t_load = time.perf_counter()
    # the ranks of a tensor-parallel job share the generation of the synthetic weights (each tensor is made by one
    # rank and broadcast), so that the host cores do it once
    shared = dict(dist=dist, device=torch.device("cuda", local_rank)) if dist is not None else {}
    model = LlamaModel(factory.ctx, synth.metadata(cfg), synthetic_tensors(cfg, args.seed, **shared), ctx_size,
                       kv_dtype=args.kv_dtype)
    load_s = time.perf_counter() - t_load
    prompt = synth.prompt_ids(cfg, PROMPT_LEN, args.seed)
    model.prefill(prompt, want_logits=False)  # first call: one-time set-up (function attributes, tensor maps)
    model.reset()
    barrier()
    t_pf = time.perf_counter()
    _, am = model.prefill(prompt, want_logits=False)
    barrier()
    prefill_s = time.perf_counter() - t_pf

    # ---- parity of the model being timed (every GPU count): logits after the prompt (all-gathered under tensor
    # parallelism) and the first greedy tokens against the committed fixture of the same seeded model
    parity = None
    if args.config == "c1" and PROMPT_LEN == 128 and args.seed == 0:
        model.reset()
        lg, am_p = model.prefill(prompt, want_logits=True)
        g_toks, _ = model.decode_greedy(am_p, 15)
        if rank == 0:
            parity = parity_against_fixture(lg, [int(t) for t in g_toks])
        model.set_position(PROMPT_LEN)

    # ---- value: device-resident greedy decode, CUDA events on the library's stream. The K-step loop is repeated
    # from the same position until at least MIN_TIMED_S of device time has been measured; the median counts.
    import statistics as st
    toks_w, _ = model.decode_greedy(am, W)
    first_tok = int(toks_w[-1])
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    reps_ms, toks = [], None
    while True:
        model.set_position(PROMPT_LEN + W)
        barrier()
        toks_r, ms_r = model.decode_greedy(first_tok, K)
        barrier()
        t = torch.tensor([ms_r], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        reps_ms.append(float(t.item()))
        toks = toks_r if toks is None else toks
        if sum(reps_ms) >= MIN_TIMED_S * 1e3 or len(reps_ms) >= 400:
            break
    ms = st.median(reps_ms)

    # ---- e2e: the reference-facing call per token, host token in / arg-max out, repeated the same way
    e2e_reps, e2e_toks = [], None
    while True:
        model.set_position(PROMPT_LEN)
        tk = am
        for _ in range(W):
            _, tk = model.decode(tk, want_logits=False)
        barrier()
        t0 = time.perf_counter()
        seq = []
        for _ in range(K):
            _, tk = model.decode(tk, want_logits=False)
            seq.append(tk)
        barrier()
        t = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device="cuda")
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_reps.append(float(t.item()))
        e2e_toks = seq if e2e_toks is None else e2e_toks
        if sum(e2e_reps) >= MIN_TIMED_S or len(e2e_reps) >= 400:
            break
    e2e_s = st.median(e2e_reps)
    clocks = sampler.stop() if rank == 0 else None
    same_tokens = [int(t) for t in toks] == [int(t) for t in e2e_toks]

    # ---- roofline of the dominant kernel, timed alone with events on the same stream
    peak, peak_kind = measured_peak()
    kern = {}
    for name in ("ffn_gate_up", "ffn_down", "qkv_rope", "attn_out", "lm_head", "attention"):
        kms, kbytes = model.profile_kernel(name, 64 if name != "lm_head" else 16)
        kern[name] = {"us": kms * 1e3, "bytes": kbytes, "gbs": kbytes / (kms * 1e-3) / 1e9}
    # ---- sampled decoding with the draw on the device (temperature 0.5, top-p 0.95, top-k 40 as in the reference)
    sampled = None
    if world == 1:
        import numpy as np
        model.set_position(PROMPT_LEN)
        us = np.random.default_rng(args.seed + 7).random(K, dtype=np.float32)
        model.decode_sampled(am, us[:min(W, K)])
        model.set_position(PROMPT_LEN)
        _, sms = model.decode_sampled(am, us)
        sampled = {"value": K / (sms * 1e-3), "unit": "tok/s", "steps": K,
                   "what": "decode step + top-p draw fed back on the device (nfai_decode_sampled)"}
    # ---- the prompt path at a length where it is tensor-core bound: a 2 048-token pass of the same architecture
    pf2048 = None
    if world == 1 and cfg.dtype == "f16" and args.config == "c1" and not args.no_prefill_2048:
        model.Dispose()
        model = LlamaModel(factory.ctx, synth.metadata(cfg), synthetic_tensors(cfg, args.seed), 2048 + 8,
                           kv_dtype=args.kv_dtype)
        long_prompt = synth.prompt_ids(cfg, 2048, args.seed + 5)
        model.prefill(long_prompt, want_logits=False)
        times = []
        for _ in range(5):
            model.reset()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            model.prefill(long_prompt, want_logits=False)
            torch.cuda.synchronize()
            times.append(time.perf_counter() - t0)
        tsec = st.median(times)
        flops = (2.0 * (cfg.streamed_matrix_params() - cfg.V * cfg.H) * 2048 + 2.0 * 2048 * 2048 * cfg.qDim * cfg.L
                 + 2.0 * cfg.V * cfg.H)
        sus, burst, kind = measured_tflops()
        pf2048 = {"tokens": 2048, "ms": tsec * 1e3, "tok_s": 2048 / tsec, "tflops": flops / tsec / 1e12,
                  "frac_of_sustained_bf16": flops / tsec / 1e12 / sus, "frac_of_burst_bf16": flops / tsec / 1e12 / burst,
                  "peak_kind": kind, "timing": "host clock around nfai_prefill with a synchronise on both sides, median of 5",
                  "flops": "2 x layer matrix params x T + causal attention 2 T^2 qDim L + one LM-head row"}
    launches = model.step_launches()
    kv_bytes = 2 if model.kv_dtype == "f16" else 4
    first_pos = PROMPT_LEN + W
    step_bytes = sum(synth.decode_bytes(cfg, p, kv_bytes) for p in range(first_pos, first_pos + K)) / K / world
    model.Dispose()
    factory.Dispose()
    if rank != 0:
        if dist is not None:
            dist.barrier()
            dist.destroy_process_group()
        return

    dom = kern["ffn_gate_up"]
    value = K / (ms * 1e-3)
    line = {
        "metric": "decode tok/s (batch 1)", "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "timed": {"reps": len(reps_ms), "device_s": sum(reps_ms) * 1e-3, "statistic": "median over reps of K steps",
                  "min_ms_per_step": min(reps_ms) / K, "max_ms_per_step": max(reps_ms) / K, "e2e_reps": len(e2e_reps)},
        "tp_parity" if world > 1 else "parity": parity,
        "dtype": "f32 accumulate over " + cfg.dtype + " weights", "data": "synthetic",
        "config": {"workload": workload_name(args.config, cfg, K), "weights": cfg.dtype, "kv_cache": model.kv_dtype,
                   "parallelism": f"tp{world}", "exchange": exchange, "l2": "inputs larger than L2: every step streams all weights "
                   f"({cfg.streamed_matrix_params() * 2 / 1e9:.2f} GB at TP1) against a 126 MB L2",
                   "seed": args.seed},
        "e2e": {"value": K / e2e_s, "unit": "tok/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 32,
                "same_tokens_as_device_loop": same_tokens},
        "gpu_launches": K * launches,
        "roofline": {"bound": "hbm", "kernel": "gemv_kernel (FFN gate/up + RMSNorm + SiLU*up)", "achieved": dom["gbs"],
                     "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": dom["gbs"] / peak, "traffic": (NCU_TRAFFIC.get((args.config, world)) or {}).get("bytes"),
                     "traffic_capture": (NCU_TRAFFIC.get((args.config, world)) or {}).get("capture"),
                     "launch_us": dom["us"], "bytes_per_launch": dom["bytes"]},
        "step_roofline": {"bytes_per_token_per_gpu": step_bytes, "achieved_gbs": step_bytes / (ms / K * 1e-3) / 1e9,
                          "frac_of_8tbs": step_bytes / (ms / K * 1e-3) / 8e12,
                          "frac_of_measured": step_bytes / (ms / K * 1e-3) / 1e9 / peak},
        "sampled": sampled,
        "kernels": kern,
        "clocks": clocks,
        "load_s": load_s, "prefill_tok_s": PROMPT_LEN / prefill_s,
        "prefill": {"tokens": PROMPT_LEN, "ms": prefill_s * 1e3, "tok_s": PROMPT_LEN / prefill_s,
                    "path": ("batched tensor-core GEMM" + (", NCCL all-reduce of [tokens][H] after O and down" if world > 1 else ""))
                            if cfg.dtype == "f16" else "token by token",
                    "tflops": (2.0 * (cfg.streamed_matrix_params() - cfg.V * cfg.H) * PROMPT_LEN
                               + 2.0 * PROMPT_LEN * PROMPT_LEN * cfg.qDim * cfg.L) / prefill_s / 1e12},
    }
    line["kernels"]["lm_head"]["note"] = ("timed alone the loop re-reads one matrix: the part of it that stays in the "
                                          "126 MB L2 lifts this figure a few percent above the HBM copy peak")
    if pf2048 is not None:
        line["prefill_2048"] = pf2048
    if world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        n_tok = 8
        v, s_per = cpu_baseline(cfg, threads, n_tok, args.seed)
        v1, _ = cpu_baseline(cfg, 1, 2, args.seed)
        line["cpu_baseline"] = {"value": v, "unit": "tok/s", "cores": threads, "kind": "port",
                                "sample": f"{n_tok} decode steps at positions {PROMPT_LEN + 1}.. of the same model "
                                          "(KV rows below are zero-filled), all host threads",
                                "one_thread": {"value": v1, "unit": "tok/s", "cores": 1, "sample": "2 decode steps"}}
        line["vs_cpu_port"] = {"device_loop": value / v, "e2e": (K / e2e_s) / v,
                               "note": "GPU over the CPU port of the reference's arithmetic on this box's host cores; "
                                       "vs_baseline stays null: the reference publishes no number for this metric"}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c1", choices=["c0", "c1", "c2", "c3", "c4", "s1"])
    ap.add_argument("--kv-dtype", default="f16", choices=["f16", "f32", "auto"])
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-prefill-2048", action="store_true", help="skip the 2 048-token prompt measurement")
    ap.add_argument("--min-timed-s", type=float, default=1.0,
                    help="repeat the K-step loop until this much device time is measured (0: one repetition, for profilers)")
    ap.add_argument("--nccl-allreduce", action="store_true", help="N > 1: use NCCL all-reduces instead of the peer-memory kernel")
    ap.add_argument("--prompt-len", type=int, default=0,
                    help="0 = the configuration's own prompt length (c1 128, c2 2048, c3 1024, c4 32768)")
    args = ap.parse_args()
    global PROMPT_LEN, MIN_TIMED_S
    MIN_TIMED_S = args.min_timed_s
    PROMPT_LEN = args.prompt_len or {"c2": 2048, "c3": 1024, "c4": 32768}.get(args.config, 128)
    from nfai_b200 import synth
    cfg = synth.get_config(args.config)
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
