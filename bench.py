#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run has the layer sizes of Llama-3.2-1B (the third configuration of
BASELINE.json), a batch of 8 and a context of 8192 tokens.  A "step" is one decode step of
the whole batch.  Everything is measured through the Python entry point: requests are
submitted, the scheduler admits them and cuts their prompts, and `Engine.step()` is what is
timed; nothing reaches around the scheduler.  One JSON line is printed:

  value      decoded tokens per second in steady decoding: CUDA events around regions of K calls
             of Engine.step(); the median region counts, the fastest is given beside it
  e2e        the same by the host's clock with a synchronisation on both sides: token ids come from
             pinned host memory and sampled ids go back to it every step
  prefill    one 2,048-token prompt, whole; frac = flops / time / bf16 peak
  roofline   bytes a decode step must read (every weight once, the cache of the live requests)
             / its time, against the measured copy bandwidth
  points     decode tokens per second at batch 1 and 64 (same context), and at the headline batch with the
             reference's default sampling (temperature 1, top_p 0.95) instead of greedy
  shapes     for the layer sizes of Llama-3.2-1B, 3.2-3B and 3.1-8B: batches of 1, 8 and 64 requests
             with 2,048-token prompts and 256 generated tokens each, run to the end under the
             scheduler, with prefill and decode rates, time to first token and time per output
             token as tamnd/fastmlx's bench defines them (bench/metrics.go:58-82,106-134), the
             bytes a decode step reads and the fraction of the copy bandwidth; and a 2,048-token
             prompt whole and in portions of 512

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
    """Samples SM clocks and throttle reasons through NVML from a thread, ten times a second,
    while a region is timed (reading only; nothing is set).  Each query stalls kernel launches
    for a moment (spawning nvidia-smi, or polling every 20 ms, slowed the timed steps by a
    third), so the default run times enough steps for the region to last about a second."""
    REASONS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, period: float = 0.1):
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


SP_KW = dict(temperature=0.0, ignore_eos=True)


def _first_tokens(engine, ids, seen=None, times=None) -> None:
    """Step until every request of `ids` has produced a token."""
    seen = set() if seen is None else seen
    while len(seen) < len(ids):
        for out in engine.step():
            if out.new_token_ids and out.request_id not in seen:
                seen.add(out.request_id)
                if times is not None:
                    times[out.request_id] = time.perf_counter()


def fill(engine, batch: int, prompt_len: int, vocab: int, seed: int, sp_kw: dict | None = None) -> list[str]:
    """Submit `batch` requests that never end by themselves and step until each has drawn its first token."""
    from fastmlx_b200 import SamplingParams
    sp = SamplingParams(max_tokens=1 << 20, **(sp_kw or SP_KW))
    ids = [engine.submit(rand_prompt(prompt_len, vocab, seed + i), sp) for i in range(batch)]
    _first_tokens(engine, ids)
    return ids


def drain(engine, ids) -> None:
    engine.flush()
    for rid in ids:
        engine.abort(rid)
    while engine.has_unfinished():
        engine.step()


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2] if len(xs) % 2 else 0.5 * (xs[len(xs) // 2 - 1] + xs[len(xs) // 2])


def timed_regions(engine, steps: int, regions: int, wall: bool) -> list[float]:
    """`regions` regions of `steps` calls of Engine.step() each -> ms per step of every region.
    wall=False: CUDA events on the engine's stream (the step launched ahead of the host's read
    of the last one is part of the stream's work like any other).  wall=True: the host's clock
    around the region, the device idle at both ends."""
    import torch
    out = []
    for _ in range(regions):
        torch.cuda.synchronize()
        if wall:
            t = time.perf_counter()
            for _ in range(steps):
                engine.step()
            torch.cuda.synchronize()
            out.append((time.perf_counter() - t) * 1e3 / steps)
        else:
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(steps):
                engine.step()
            t1.record()
            torch.cuda.synchronize()
            out.append(t0.elapsed_time(t1) / steps)
    return out


MIN_REGION_MS = 200.0        # timed work per measurement, whatever --steps says: the clock sampler must see it


def steady_decode(engine, batch: int, context: int, steps: int, warmup: int, vocab: int, nums: dict, e2e: bool,
                  clock: ClockSampler | None = None, est_ms: float = 1.0, sp_kw: dict | None = None) -> dict:
    """Steady decoding of `batch` requests whose contexts end at `context`: the scheduler prefills,
    then regions of `steps` steps are timed, first by CUDA events, then (e2e) by the host's clock."""
    import torch
    regions = max(3, min(40, int(-(-MIN_REGION_MS // max(steps * est_ms, 1e-3)))))
    wall_regions = max(3, regions // 2) if e2e else 0
    grow = warmup * (2 if e2e else 1) + steps * (regions + wall_regions) + 4
    prompt_len = max(16, context - grow)
    ids = fill(engine, batch, prompt_len, vocab, seed=1000 * batch, sp_kw=sp_kw)
    for _ in range(warmup):
        engine.step()
    k = engine.rt.k
    c0, l0 = dict(engine.counters), k.launch_count() + engine.step_fn.graph_kernel_launches
    if clock:
        clock.start()
    dev = timed_regions(engine, steps, regions, wall=False)
    launches = (k.launch_count() + engine.step_fn.graph_kernel_launches - l0) // regions
    ctx_mid = prompt_len + warmup + steps * regions // 2            # mean context over the device-timed regions
    out = {"ms": median(dev), "ms_fastest": min(dev), "regions": regions, "launches": launches, "ctx": ctx_mid}
    if e2e:
        for _ in range(warmup):
            engine.step()
        c1 = dict(engine.counters)
        walls = timed_regions(engine, steps, wall_regions, wall=True)
        c2 = dict(engine.counters)
        n = steps * wall_regions
        out.update(e2e_ms=median(walls), h2d=(c2["h2d_bytes"] - c1["h2d_bytes"]) // n, d2h=(c2["d2h_bytes"] - c1["d2h_bytes"]) // n)
    if clock:
        clock.stop()                              # the clocks were sampled over the device-timed and the host-timed regions
    out["bytes"] = nums["weight_bytes"] + batch * ctx_mid * nums["kv_bytes_per_token"]
    drain(engine, ids)
    return out


def prefill_through_engine(engine, tokens: int, vocab: int, repeats: int = 3) -> float:
    """One prompt of `tokens` tokens from submit to its first token, device-timed (CUDA events
    around the calls of Engine.step() that it takes: one when the prompt runs whole, several
    when the scheduler cuts it).  The fastest of `repeats` after one warm-up."""
    import torch
    from fastmlx_b200 import SamplingParams
    best = None
    for i in range(repeats + 1):
        rid = engine.submit(rand_prompt(tokens, vocab, 900 + i), SamplingParams(max_tokens=1, **SP_KW))
        torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        done = False
        while not done:
            done = any(o.request_id == rid and o.finished for o in engine.step())
        t1.record()
        torch.cuda.synchronize()
        while engine.has_unfinished():
            engine.step()
        if i > 0 or repeats == 0:
            ms = t0.elapsed_time(t1)
            best = ms if best is None else min(best, ms)
    return best


def workload(engine, batch: int, prompt_len: int, generated: int, vocab: int, nums: dict, pk: dict) -> dict:
    """`batch` requests of `prompt_len` prompt tokens and `generated` generated tokens, submitted
    together and run to the end under the scheduler.  Rates and latencies as tamnd/fastmlx's
    bench defines them (bench/metrics.go:58-82: TTFT, TPOT = generation time / (n - 1);
    106-134: prefill tok/s = all prompt tokens / (last first token - start), decode tok/s = all
    generated tokens / (end - last first token)), by the host's clock."""
    import torch
    from fastmlx_b200 import SamplingParams
    sp = SamplingParams(max_tokens=generated, **SP_KW)
    prompts = [rand_prompt(prompt_len, vocab, 7000 + 13 * batch + i) for i in range(batch)]
    torch.cuda.synchronize()
    start = time.perf_counter()
    ids = [engine.submit(p, sp) for p in prompts]
    first, ends, counts = {}, {}, {}
    while engine.has_unfinished():
        outs = engine.step()
        now = time.perf_counter()
        for o in outs:
            if o.new_token_ids and o.request_id not in first:
                first[o.request_id] = now
            if o.finished:
                ends[o.request_id], counts[o.request_id] = now, o.completion_tokens
    torch.cuda.synchronize()
    end = time.perf_counter()
    last_first = max(first.values())
    total_gen = sum(counts.values())
    decode_s = max(end - last_first, 1e-9)
    decode_steps = generated - 1                       # every request's first token came with its prompt
    ms_step = decode_s * 1e3 / max(decode_steps, 1)
    ctx_mid = prompt_len + generated // 2
    step_bytes = nums["weight_bytes"] + batch * ctx_mid * nums["kv_bytes_per_token"]
    gbs = step_bytes / (ms_step / 1e3) / 1e9
    tpot = [(ends[r] - first[r]) / max(counts[r] - 1, 1) * 1e3 for r in ids]
    return {"prefill_tok_s": round(batch * prompt_len / max(last_first - start, 1e-9), 1),
            "decode_tok_s": round(total_gen / decode_s, 1), "ms_per_step": round(ms_step, 4),
            "ttft_ms": round(sum(first[r] - start for r in ids) / batch * 1e3, 2), "tpot_ms": round(sum(tpot) / batch, 4),
            "gb_per_step": round(step_bytes / 1e9, 3), "hbm_frac": round(gbs / pk["hbm_gbs"], 4)}


def build_engine(shape_key: str, layers: int, pool_tokens: int, max_seqs: int, block_size: int, cuda_graphs: bool = True):
    from fastmlx_b200 import Engine
    shape_name, shape = SHAPES[shape_key]
    cfg = dict(shape, num_hidden_layers=layers or shape["num_hidden_layers"])
    engine = Engine(config=cfg, weights_seed=0, dtype="bfloat16", block_size=block_size, max_cache_tokens=pool_tokens,
                    max_concurrent_requests=max_seqs, max_num_batched_tokens=8192, cuda_graphs=cuda_graphs)
    return engine, cfg, shape_name


def prefill_numbers(engine, cfg, nums, pk, chunk: int = 0) -> dict:
    """A 2,048-token prompt whole (chunk 0) or as the scheduler cuts it into portions of `chunk`."""
    engine.reconfigure(prefill_chunk=chunk)
    ms = prefill_through_engine(engine, PREFILL_TOKENS, cfg["vocab_size"])
    engine.reconfigure(prefill_chunk=0)
    flops = nums["matmul_flops_per_token"] * PREFILL_TOKENS + nums["attn_flops_causal"](PREFILL_TOKENS) + nums["head_flops_per_row"]
    return {"value": round(PREFILL_TOKENS / (ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 3),
            "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}


def shape_block(shape_key: str, block_size: int, pk: dict) -> dict:
    """The 2,048 + 256 workload at batches of 1, 8 and 64, and the 2,048-token prefill whole and in
    portions of 512, for one set of layer sizes (all its layers)."""
    import gc

    import torch
    engine, cfg, _ = build_engine(shape_key, 0, 64 * (WORK_PROMPT + WORK_GENERATED + 64) + PREFILL_TOKENS, 64, block_size)
    nums = model_numbers(engine, cfg)
    out = {"layers": cfg["num_hidden_layers"], "weights_gb": round(nums["weight_bytes"] / 1e9, 3)}
    for b in (1, 8, 64):
        # the same workload once untimed: every graph it needs (the batch shrinks as requests end) is captured there
        workload(engine, b, WORK_PROMPT, WORK_GENERATED, cfg["vocab_size"], nums, pk)
        out[f"b{b}"] = workload(engine, b, WORK_PROMPT, WORK_GENERATED, cfg["vocab_size"], nums, pk)
    out["prefill_2048"] = prefill_numbers(engine, cfg, nums, pk)
    out["prefill_2048_in_512"] = prefill_numbers(engine, cfg, nums, pk, 512)
    del engine
    gc.collect()
    torch.cuda.empty_cache()
    return out


WORK_PROMPT, WORK_GENERATED = 2048, 256


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="1b", choices=sorted(SHAPES), help="layer sizes of the headline: Llama-3.2-1B (the default run), 3B, or 3.1-8B")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (0: all)")
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--context", type=int, default=CONTEXT)
    ap.add_argument("--shapes", default="1b,3b,8b", help="layer sizes of the `shapes` block (comma-separated; empty: none)")
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and batch 64 points")
    ap.add_argument("--no-prefill", action="store_true", help="skip the 2,048-token prefill (for profiling)")
    ap.add_argument("--no-cuda-graphs", action="store_true", help="run decode steps eagerly (for profiling)")
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--only-steps", type=int, default=0,
                    help="for a profiler's launch list: fill the batch, run this many decode steps and stop (no timing, no JSON line)")
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

    import gc

    import torch

    pk = peaks()
    big = 64 if not args.no_points else args.batch
    pool_tokens = max(big, args.batch) * (args.context + 64) + PREFILL_TOKENS + 64
    engine, cfg, shape_name = build_engine(args.shape, args.layers, pool_tokens, max(big, args.batch), args.block_size,
                                           not args.no_cuda_graphs)
    full_layers = SHAPES[args.shape][1]["num_hidden_layers"]
    vocab = cfg["vocab_size"]
    nums = model_numbers(engine, cfg)

    if args.only_steps > 0:
        ids = fill(engine, args.batch, args.context - args.only_steps - warmup - 4, vocab, seed=1000 * args.batch)
        for _ in range(warmup + args.only_steps):
            engine.step()
        drain(engine, ids)
        torch.cuda.synchronize()
        print(f"ran {args.only_steps} decode steps of batch {args.batch} at context {args.context} after {warmup} warm-up steps")
        return 0

    # ---- a 2,048-token prompt, whole
    prefill = {} if args.no_prefill else prefill_numbers(engine, cfg, nums, pk)

    # ---- steady decoding at the headline batch, then at 1 and 64
    probe = steady_decode(engine, args.batch, min(args.context, 1024), 8, warmup, vocab, nums, False)    # graphs, and an estimate
    clock = ClockSampler()
    main_pt = steady_decode(engine, args.batch, args.context, steps, warmup, vocab, nums, True, clock, probe["ms"])
    points = {}
    if not args.no_points:
        for b in (1, 64):
            pt = steady_decode(engine, b, args.context, min(steps, 64), warmup, vocab, nums, False, None, probe["ms"])
            points[f"decode_b{b}"] = round(b / (pt["ms"] / 1e3), 1)
        # the headline batch with the reference's default sampling (temperature 1, top_p 0.95) instead of greedy
        pt = steady_decode(engine, args.batch, args.context, min(steps, 64), warmup, vocab, nums, False, None, probe["ms"],
                           dict(temperature=1.0, top_p=0.95, ignore_eos=True))
        points[f"decode_b{args.batch}_top_p"] = round(args.batch / (pt["ms"] / 1e3), 1)
    stats = engine.stats()
    del engine
    gc.collect()
    torch.cuda.empty_cache()

    shapes = {}
    for key in [k for k in args.shapes.split(",") if k]:
        shapes[key] = shape_block(key, args.block_size, pk)

    ms = main_pt["ms"]
    achieved = main_pt["bytes"] / (ms / 1e3) / 1e9
    line = {
        "metric": f"decode tok/s at batch {args.batch} ({shape_name}, context {args.context})",
        "value": round(args.batch / (ms / 1e3), 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "ms_per_step_fastest": round(main_pt["ms_fastest"], 4), "regions": main_pt["regions"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded uniform-random token ids, random N(0, 0.02) weights",
        "config": {"model": shape_name, "layers": cfg["num_hidden_layers"], "layers_of_full_config": full_layers,
                   "hidden_size": cfg["hidden_size"], "num_attention_heads": cfg["num_attention_heads"],
                   "num_key_value_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate_size": cfg["intermediate_size"], "vocab_size": vocab, "tie_word_embeddings": cfg["tie_word_embeddings"],
                   "rope": f"theta 500000, llama3 x{cfg['rope_scaling']['factor']:g}", "global_batch": args.batch, "seq_len": args.context,
                   "context_at_timing": main_pt["ctx"], "page_size": args.block_size, "parallelism": "single GPU",
                   "l2": f"inputs larger than L2 ({nums['weight_bytes'] / 1e9:.1f} GB of weights per step)", "cuda_graphs": not args.no_cuda_graphs,
                   "timing": f"Engine.step() only; median of {main_pt['regions']} regions of K steps", "peaks": pk["source"]},
        "clocks": clock.summary(),
        "e2e": {"value": round(args.batch / (main_pt["e2e_ms"] / 1e3), 1), "unit": "tokens/s",
                "ms_per_step": round(main_pt["e2e_ms"], 4), "h2d_bytes_per_step": main_pt["h2d"],
                "d2h_bytes_per_step": main_pt["d2h"]},
        "gpu_launches": main_pt["launches"],
        "native_executor": bool(stats.get("native_executor")),
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": main_pt["bytes"]},
        "points": points,
        "shapes": shapes,
        "impl": "ours",
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
