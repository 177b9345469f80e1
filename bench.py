#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Llama-3.2-1B (the third configuration of
BASELINE.json), a batch of 8 and a context of 8192 tokens.  A "step" is one decode step of
the whole batch.  One JSON line is printed:

  value      decoded tokens per second, timed on the device with CUDA events around K steps
             (each step: metadata to the device, the captured model graph, the sampling kernel)
  e2e        the same through the Python entry point (Engine.step): token ids come from host
             memory and sampled ids go back to it every step
  prefill    one 2,048-token prompt in one step; frac = flops / time / bf16 peak
  roofline   bytes a decode step must read (every weight once, the cache of the live requests)
             / its time, against the measured copy bandwidth
  points     decode tokens per second at batch 1 and 64

Every timed step reads well over 126 MB (weights alone are 2.5 GB), so no input stays in L2
between iterations.  tamnd/fastmlx publishes no number to compare with, and cannot run here
(`--impl reference` says why).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_1B = {
    "model_type": "llama", "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 16, "hidden_size": 2048, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "intermediate_size": 8192, "vocab_size": 128256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 131072,
}
LLAMA_3B = dict(LLAMA_1B, num_hidden_layers=28, hidden_size=3072, num_attention_heads=24, head_dim=128)
LLAMA_8B = dict(LLAMA_1B, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, head_dim=128,
                intermediate_size=14336, tie_word_embeddings=False,
                rope_scaling=dict(LLAMA_1B["rope_scaling"], factor=8.0))
SHAPES = {"1b": ("llama-3.2-1b-shape", LLAMA_1B), "3b": ("llama-3.2-3b-shape", LLAMA_3B),
          "8b": ("llama-3.1-8b-shape", LLAMA_8B)}
FULL_LAYERS = 16
CONTEXT = 8192
BATCH = 8
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        flat = {}

        def walk(x):
            if isinstance(x, dict):
                for k, v in x.items():
                    if isinstance(v, (int, float)):
                        flat.setdefault(k, float(v))
                    else:
                        walk(v)
        walk(d)
        out = {"hbm_gbs": flat.get("hbm_gbs"), "bf16_tflops": flat.get("bf16_tflops_sustained") or flat.get("bf16_tflops"),
               "source": "measured"}
        if out["hbm_gbs"] and out["bf16_tflops"]:
            return out
    except (OSError, ValueError):
        pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML from a thread, five times a second,
    while a region is timed (reading only; nothing is set).  Each query stalls kernel launches
    for a moment (spawning nvidia-smi, or polling every 20 ms, slowed the timed steps by a
    third), so the default run times enough steps for the region to last about a second."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, period: float = 0.2):
        self.period, self.samples, self.max_mhz = period, [], None
        self._stop, self._thread, self._h = None, None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(int(os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0] or 0)
                                                         if os.environ.get("CUDA_VISIBLE_DEVICES", "0").split(",")[0].isdigit() else 0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._h = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
                try:
                    why = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    why = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                self.samples.append((mhz, why))
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self._h is None:
            return
        import threading
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def stop(self):
        if self._thread is None:
            return
        self._stop.set()
        self._thread.join()
        self._thread = None

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        mhz = sorted(m for m, _ in self.samples)
        reasons = [n for n, bit in self.REASONS.items() if any(w & bit for _, w in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(self.samples)}


def model_numbers(engine, cfg: dict) -> dict:
    """Bytes and flops of the model as built (whatever number of layers it has)."""
    model = engine.model
    weight_bytes = model.weight_bytes()
    L, d, I = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_token_matmul = L * 2 * (d * (nh + 2 * nkv) * hd + nh * hd * d + 3 * d * I)
    return {"weight_bytes": weight_bytes, "kv_bytes_per_token": engine.manager.bytes_per_token(),
            "matmul_flops_per_token": per_token_matmul, "head_flops_per_row": 2 * d * cfg["vocab_size"],
            "attn_flops_causal": lambda T: L * 2 * 2 * nh * hd * T * (T + 1) // 2}


def rand_prompt(n: int, vocab: int, seed: int) -> list[int]:
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def fill(engine, batch: int, prompt_len: int, vocab: int, seed: int) -> list[str]:
    """Submit `batch` requests and step until every prompt is in the cache and each request
    has drawn its first token."""
    from fastmlx_b200 import SamplingParams
    sp = SamplingParams(max_tokens=1 << 20, temperature=0.0, ignore_eos=True)
    ids = [engine.submit(rand_prompt(prompt_len, vocab, seed + i), sp) for i in range(batch)]
    while any(r.num_computed < len(r.prompt_token_ids) or not r.output_token_ids for r in engine._requests.values()):
        engine.step()
    return ids


def drain(engine, ids) -> None:
    engine.flush()
    for rid in ids:
        engine.abort(rid)
    while engine.has_unfinished():
        engine.step()


def device_decode(engine, steps: int, warmup: int, sampler: ClockSampler | None = None, runs: int = 1) -> tuple[float, int]:
    """K decode steps of the live requests timed with CUDA events: the step function (metadata
    to the device, the model graph) and the sampling kernel, nothing read back in between.
    Tokens fed are fixed ids: the work of a step does not depend on them.  The region of K
    steps is timed `runs` times and the fastest is kept (another tenant's burst on the host
    has doubled single readings on this pool).  -> (ms per step, launches of this package's
    kernels in one region)."""
    import torch
    from fastmlx_b200.engine.batch import StepEntry
    engine.flush()
    reqs = list(engine.scheduler.running)
    fn = engine.step_fn

    def one():
        entries = [StepEntry(r.cache, [17], [0]) for r in reqs]
        logits = fn.run(entries, check=False)
        return engine.rt.k.sample(logits)

    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    k = engine.rt.k
    best, launches = None, 0
    if sampler:
        sampler.start()
    for _ in range(runs):
        l0, g0 = k.launch_count(), fn.graph_kernel_launches
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(steps):
            one()
        t1.record()
        torch.cuda.synchronize()
        launches = (k.launch_count() - l0) + (fn.graph_kernel_launches - g0)
        ms = t0.elapsed_time(t1) / steps
        best = ms if best is None else min(best, ms)
    if sampler:
        sampler.stop()
    fn.check_status()
    # the scheduler's view of these requests: their caches grew by every token fed
    fed = warmup + steps * runs
    for r in reqs:
        r.output_token_ids.extend([17] * fed)
        r.num_computed += fed
    return best, launches


def e2e_decode(engine, steps: int, warmup: int, runs: int = 1) -> tuple[float, int, int]:
    """The same through Engine.step(): host tokens in, host tokens out, every step.  The fastest
    of `runs` regions of K steps."""
    import torch
    for _ in range(warmup):
        engine.step()
    best = None
    for _ in range(runs):
        torch.cuda.synchronize()
        c0 = dict(engine.counters)
        t = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        dt = (time.perf_counter() - t) * 1e3 / steps
        best = dt if best is None else min(best, dt)
    h2d = (engine.counters["h2d_bytes"] - c0["h2d_bytes"]) // steps
    d2h = (engine.counters["d2h_bytes"] - c0["d2h_bytes"]) // steps
    return best, h2d, d2h


def prefill_once(engine, tokens: int, vocab: int, repeats: int = 3) -> float:
    """One prompt of `tokens` tokens in one step (after a warm-up of the same shape)."""
    import torch
    from fastmlx_b200.engine.batch import StepEntry
    best = None
    for i in range(repeats + 1):
        rc = engine.manager.add_request(f"prefill-{i}")
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        t0.record()
        logits = engine.step_fn.run([StepEntry(rc, rand_prompt(tokens, vocab, 900 + i), [tokens - 1])], check=False)
        engine.rt.k.sample(logits)
        t1.record()
        torch.cuda.synchronize()
        engine.step_fn.check_status()
        engine.manager.free(f"prefill-{i}")
        if i > 0 or repeats == 0:
            ms = t0.elapsed_time(t1)
            best = ms if best is None else min(best, ms)
    return best


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="layer sizes: Llama-3.2-1B (the default run), 3B, or 3.1-8B")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and batch 64 points")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 2,048-token prefill (for profiling)")
    ap.add_argument("--no-cuda-graphs", action="store_true", help="run decode steps eagerly (for profiling)")
    ap.add_argument("--block-size", type=int, default=16)
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "tamnd/fastmlx is a Go program over Apple's MLX (cgo, Metal); there is no Go toolchain "
                          "or MLX here, pip cannot install it, and its default build returns ErrMLXUnavailable "
                          "at the first tensor op"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this engine has no multi-GPU path (asked for {args.gpus})")
        return 2
    warmup = max(3, args.warmup)
    steps = max(1, args.steps)

    import torch
    from fastmlx_b200 import Engine

    shape_name, shape = SHAPES[args.shape]
    full_layers = shape["num_hidden_layers"]
    args.layers = args.layers or full_layers
    cfg = dict(shape, num_hidden_layers=args.layers)
    vocab = cfg["vocab_size"]
    big = 64 if not args.no_points else args.batch
    pool_tokens = max(big, args.batch) * (args.context + 64) + PREFILL_TOKENS + 64
    engine = Engine(config=cfg, weights_seed=0, dtype="bfloat16", block_size=args.block_size,
                    max_cache_tokens=pool_tokens, max_concurrent_requests=max(big, args.batch),
                    max_num_batched_tokens=8192, cuda_graphs=not args.no_cuda_graphs)
    nums = model_numbers(engine, cfg)
    pk = peaks()

    # ---- prefill of 2,048 tokens
    pre_ms = prefill_once(engine, PREFILL_TOKENS, vocab, repeats=0 if args.no_prefill else 3)
    pre_flops = nums["matmul_flops_per_token"] * PREFILL_TOKENS + nums["attn_flops_causal"](PREFILL_TOKENS) \
        + nums["head_flops_per_row"]
    prefill = {"value": round(PREFILL_TOKENS / (pre_ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
               "frac": round(pre_flops / (pre_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}

    RUNS = 3

    def decode_point(batch: int, timed_steps: int, e2e: bool, clock: ClockSampler | None):
        runs = RUNS if e2e else 2                 # the fastest region counts (a shared host's bursts double single readings)
        grow = (warmup + timed_steps * runs) + (warmup + timed_steps * 2 if e2e else 0)
        prompt_len = args.context - grow - 2
        ids = fill(engine, batch, prompt_len, vocab, seed=1000 * batch)
        out = {}
        if e2e:
            out["e2e_ms"], out["h2d"], out["d2h"] = e2e_decode(engine, timed_steps, warmup, 2)
        out["ms"], out["launches"] = device_decode(engine, timed_steps, warmup, clock, runs)
        out["ctx"] = max(r.num_computed for r in engine.scheduler.running)
        drain(engine, ids)
        return out

    clock = ClockSampler()
    main_pt = decode_point(args.batch, steps, True, clock)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            pt = decode_point(b, min(steps, 64), False, None)
            points[f"decode_b{b}"] = round(b / (pt["ms"] / 1e3), 1)

    ms = main_pt["ms"]
    step_bytes = nums["weight_bytes"] + args.batch * main_pt["ctx"] * nums["kv_bytes_per_token"]
    achieved = step_bytes / (ms / 1e3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {args.batch} ({shape_name}, context {args.context})",
        "value": round(args.batch / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random N(0, 0.02) weights",
        "config": {"model": shape_name, "layers": args.layers, "layers_of_full_config": full_layers,
                   "hidden_size": cfg["hidden_size"], "num_attention_heads": cfg["num_attention_heads"],
                   "num_key_value_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate_size": cfg["intermediate_size"], "vocab_size": vocab, "tie_word_embeddings": cfg["tie_word_embeddings"],
                   "rope": f"theta 500000, llama3 x{cfg['rope_scaling']['factor']:g}", "global_batch": args.batch, "seq_len": args.context,
                   "context_at_timing": main_pt["ctx"], "page_size": args.block_size, "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 ({nums['weight_bytes'] / 1e9:.1f} GB of weights per step)", "cuda_graphs": not args.no_cuda_graphs, "timing": "fastest of 3 regions of K steps",
                   "peaks": pk["source"]},
        "clocks": clock.summary(),
        "e2e": {"value": round(args.batch / (main_pt["e2e_ms"] / 1e3), 1), "unit": "tokens/s",
                "ms_per_step": round(main_pt["e2e_ms"], 4), "h2d_bytes_per_step": main_pt["h2d"],
                "d2h_bytes_per_step": main_pt["d2h"]},
        "gpu_launches": main_pt["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": step_bytes},
        "points": points,
        "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
