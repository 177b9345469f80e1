"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and schedules nothing; it drives the same model, step function, cache
manager and kernels that generation uses.  tamnd/fastmlx has nothing alike; the nearest is
the recording fake model of its generator tests (compute/batch_generator_test.go:22-45).

Input, one JSON object per line on standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step that wants something, `<out>/<step>.f32` holds the logits at the wanted places
as little-endian float32 [wanted, vocab], in the order of the entries and of `want`.
After every step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np

from ..cache.manager import CacheManager
from .batch import StepEntry
from .loading import load_model
from .step import StepFunction

MAX_LIVE = 8          # request slots; traces keep up to four live, a step may name one more while another ends


def pool_pages(max_tokens: int, page_size: int) -> int:
    """Pages for `max_tokens` live tokens when each request's count is rounded up to a
    multiple of max(64, page_size)."""
    unit = max(64, page_size)
    return max(1, -(-int(max_tokens) // unit) * (unit // page_size if unit % page_size == 0 else -(-unit // page_size)))


class Replayer:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, device="cuda",
                 kernels=None, max_live: int = MAX_LIVE, native: bool = True):
        self.cfg, self.model, self.rt = load_model(model_dir, dtype, device, kernels)
        self.manager = CacheManager(self.model.cache_needs(), page_size=page_size,
                                    num_pages=pool_pages(max_tokens, page_size), max_requests=max_live,
                                    dtype=self.rt.dtype, device=self.rt.device)
        # replay feeds what the trace says: positions past max_position_embeddings are the trace's business
        self.step_fn = StepFunction(self.model, self.manager, self.rt, position_limit=False, native=native)

    def step(self, record: dict):
        """Run one trace record; -> float32 numpy [wanted, vocab] or None."""
        entries = []
        fresh = []
        try:
            for e in record.get("entries", []):
                rid = e["id"]
                req = self.manager.requests.get(rid)
                if req is None:
                    req = self.manager.add_request(rid)
                    fresh.append(rid)
                tokens = [int(t) for t in e.get("tokens", [])]
                if not tokens:                         # a request named without tokens runs nothing
                    if e.get("want"):
                        raise ValueError(f"request {rid!r} asks for logits of a step that brings it no tokens")
                    continue
                entries.append(StepEntry(req, tokens, [int(w) for w in e.get("want", [])]))
            logits = self.step_fn.run(entries) if entries else None
        except BaseException:
            for rid in fresh:
                self.manager.free(rid)
            raise
        for rid in record.get("end", []):
            if rid in self.manager.requests:
                self.manager.free(rid)
        if logits is None or logits.shape[0] == 0:
            return None
        return logits.float().cpu().numpy().astype("<f4", copy=False)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page")
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)
    rp = Replayer(args.model, args.dtype, args.max_tokens, args.page_size)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        logits = rp.step(record)
        if logits is not None:
            tmp = os.path.join(args.out, f".{record['step']}.f32.tmp")
            logits.tofile(tmp)
            os.replace(tmp, os.path.join(args.out, f"{record['step']}.f32"))
        print(f"done {record['step']}", flush=True)
    return 0
