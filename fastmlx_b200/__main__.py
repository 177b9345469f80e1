"""Command line: `python -m fastmlx_b200 <command>`.

tamnd/fastmlx's binary has `serve`, `launch`, `diagnose` and `version`
(cmd/fastmlx/main.go:15-62); its `serve` flags that concern the engine keep their names
here (--model-dir, --max-concurrent-requests, --initial-cache-blocks: cmd/fastmlx/serve.go:
55-75).  There is no HTTP server in this engine, so the long-lived `serve` is replaced by
`generate` (token ids in, token ids out), `replay` (see bin/trace_run), `random-model`
(write a folder with seeded random weights) and `version`.
"""
from __future__ import annotations

import argparse
import json
import sys


def _ids(text: str) -> list[list[int]]:
    """'1,2,3' or '1,2;4,5' or a path to a JSON file holding a list (of lists) of ids."""
    import os
    if os.path.exists(text):
        with open(text) as f:
            v = json.load(f)
        return [v] if v and isinstance(v[0], int) else v
    return [[int(t) for t in part.replace(",", " ").split()] for part in text.split(";") if part.strip()]


def _engine_args(ap):
    ap.add_argument("--model-dir", help="folder with config.json and safetensors")
    ap.add_argument("--random-config", help="a config.json to run with seeded random weights instead of a folder")
    ap.add_argument("--weights-seed", type=int, default=0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    ap.add_argument("--initial-cache-blocks", type=int, default=0, help="cache pages (0: sized from the options below)")
    ap.add_argument("--kv-memory-gb", type=float, default=0.0)
    ap.add_argument("--max-cache-tokens", type=int, default=0)
    ap.add_argument("--max-concurrent-requests", type=int, default=8)
    ap.add_argument("--max-num-batched-tokens", type=int, default=8192)
    ap.add_argument("--prefill-chunk", type=int, default=0)
    ap.add_argument("--no-cuda-graphs", action="store_true")


def _make_engine(a):
    from .engine.api import Engine
    kw = dict(dtype=a.dtype, block_size=a.block_size, initial_cache_blocks=a.initial_cache_blocks,
              kv_memory_gb=a.kv_memory_gb, max_cache_tokens=a.max_cache_tokens,
              max_concurrent_requests=a.max_concurrent_requests, max_num_batched_tokens=a.max_num_batched_tokens,
              prefill_chunk=a.prefill_chunk, cuda_graphs=not a.no_cuda_graphs)
    if a.random_config:
        with open(a.random_config) as f:
            return Engine(config=json.load(f), weights_seed=a.weights_seed, **kw)
    if not a.model_dir:
        raise SystemExit("give --model-dir or --random-config")
    return Engine(a.model_dir, **kw)


def cmd_generate(a) -> int:
    from .sampling import SamplingParams
    eng = _make_engine(a)
    sp = SamplingParams(max_tokens=a.max_tokens, temperature=a.temperature, top_p=a.top_p, top_k=a.top_k,
                        min_p=a.min_p, repetition_penalty=a.repetition_penalty, presence_penalty=a.presence_penalty,
                        frequency_penalty=a.frequency_penalty, seed=a.seed, ignore_eos=a.ignore_eos)
    for out in eng.generate(_ids(a.prompt_ids), sp):
        print(json.dumps({"request_id": out.request_id, "output_token_ids": out.output_token_ids,
                          "finish_reason": out.finish_reason, "prompt_tokens": out.prompt_tokens,
                          "completion_tokens": out.completion_tokens, **({"error": out.err} if out.err else {})}))
    if a.stats:
        print(json.dumps(eng.stats()), file=sys.stderr)
    return 0


def cmd_random_model(a) -> int:
    import torch
    from .weights import write_random_model
    with open(a.config) as f:
        cfg = json.load(f)
    write_random_model(a.out, cfg, a.seed, dtype=torch.float32 if a.store_dtype == "float32" else torch.bfloat16,
                       max_shard_bytes=a.max_shard_mb * 2**20 if a.max_shard_mb else None)
    print(a.out)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="fastmlx_b200", description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="command")
    g = sub.add_parser("generate", help="generate token ids for prompts of token ids")
    _engine_args(g)
    g.add_argument("--prompt-ids", required=True, help="'1,2,3', several prompts as '1,2;3,4', or a JSON file")
    g.add_argument("--max-tokens", type=int, default=32768)
    g.add_argument("--temperature", type=float, default=1.0)
    g.add_argument("--top-p", type=float, default=0.95)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--presence-penalty", type=float, default=0.0)
    g.add_argument("--frequency-penalty", type=float, default=0.0)
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--stats", action="store_true")
    g.set_defaults(fn=cmd_generate)
    r = sub.add_parser("random-model", help="write config.json and model.safetensors with seeded random weights")
    r.add_argument("--config", required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.add_argument("--max-shard-mb", type=int, default=0)
    r.set_defaults(fn=cmd_random_model)
    p = sub.add_parser("replay", help="the trace replay program (same as bin/trace_run)", add_help=False)
    p.set_defaults(fn=None)
    v = sub.add_parser("version")
    v.set_defaults(fn=lambda a: print(__import__("fastmlx_b200").__version__) or 0)
    argv = list(sys.argv[1:] if argv is None else argv)
    if argv and argv[0] == "replay":
        from .engine.replay import main as replay_main
        return replay_main(argv[1:])
    a = ap.parse_args(argv)
    if not getattr(a, "fn", None):
        ap.print_help()
        return 2
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
