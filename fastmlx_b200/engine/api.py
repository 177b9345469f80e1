"""The Python entry point: an engine that takes token ids and gives token ids.

Modelled on tamnd/fastmlx's enginecore.BatchedEngine (enginecore/batched.go:38-82: Submit,
Abort, Start/Stop around a scheduler) and its core loop (enginecore/core.go:134-171: drain
submissions, step the scheduler, deliver outputs).  There is no tokenizer and no HTTP
layer here; prompts are lists of token ids.
"""
from __future__ import annotations

import hashlib
import itertools
from dataclasses import dataclass

import torch

from ..cache.manager import CacheManager
from ..sampling import Sampler, SamplingParams
from .loading import load_model, parse_dtype, random_model
from .request import Request, RequestOutput, RequestStatus
from .scheduler import Scheduler, SchedulerConfig
from .step import StepError, StepFunction


@dataclass
class EngineConfig:
    """Option names follow `fastmlx serve` where it has them (cmd/fastmlx/serve.go:55-75:
    --max-concurrent-requests, --initial-cache-blocks) and its scheduler's config
    (scheduler/scheduler.go:30-47: MaxNumSeqs, MaxNumBatchedTokens)."""
    dtype: str = "bfloat16"
    block_size: int = 16                      # tokens per cache page
    initial_cache_blocks: int = 0             # pages per layer group; 0 = from kv_memory_gb or max_cache_tokens
    kv_memory_gb: float = 0.0
    max_cache_tokens: int = 0
    max_concurrent_requests: int = 8          # the scheduler's MaxNumSeqs
    max_num_batched_tokens: int = 8192
    prefill_chunk: int = 0
    seed: int = 0
    cuda_graphs: bool = True
    lookahead: bool = True                    # run one decode step ahead of the host
    native_executor: bool = True              # a step's host work in compiled code, where the model's parts allow it
    device: str = "cuda"


def _request_seed(engine_seed: int, request_id: str) -> int:
    h = hashlib.sha256(f"{engine_seed}:{request_id}".encode()).digest()
    return int.from_bytes(h[:8], "little") & (2**63 - 1)


class Engine:
    def __init__(self, model_dir: str | None = None, *, config: dict | None = None, weights_seed: int = 0,
                 engine_config: EngineConfig | None = None, kernels=None, **overrides):
        """Either `model_dir` (config.json + safetensors) or `config` (a config.json dict,
        with seeded random weights)."""
        ec = engine_config or EngineConfig()
        for k, v in overrides.items():
            if not hasattr(ec, k):
                raise TypeError(f"unknown engine option {k!r}")
            setattr(ec, k, v)
        self.engine_config = ec
        if (model_dir is None) == (config is None):
            raise ValueError("give either a model folder or a configuration")
        if model_dir is not None:
            self.config, self.model, self.rt = load_model(model_dir, ec.dtype, ec.device, kernels)
        else:
            self.config, self.model, self.rt = random_model(config, weights_seed, ec.dtype, ec.device, kernels)
        needs = self.model.cache_needs()
        probe = CacheManager(needs, page_size=ec.block_size, num_pages=1, max_requests=1, dtype=self.rt.dtype,
                             allocate=False)
        per_token = max(1, probe.bytes_per_token())
        if ec.initial_cache_blocks > 0:
            pages = ec.initial_cache_blocks
        elif ec.max_cache_tokens > 0:
            pages = -(-ec.max_cache_tokens // ec.block_size)
        elif ec.kv_memory_gb > 0:
            pages = int(ec.kv_memory_gb * 2**30 // (per_token * ec.block_size))
        else:
            limit = self.model.max_positions or 8192
            pages = -(-min(limit, 8192) // ec.block_size) * ec.max_concurrent_requests
        # a group with a window holds, per request, the window and the portion that runs: it
        # gets that many pages, not the pool of a group that keeps every key
        portion = ec.prefill_chunk or ec.max_num_batched_tokens
        per_group = []
        for g in probe.groups:
            n = max(1, pages)
            if g.spec.window > 0:
                n = min(n, ec.max_concurrent_requests * (-(-(g.spec.window + portion) // ec.block_size) + 1))
            per_group.append(n)
        self.manager = CacheManager(needs, page_size=ec.block_size, num_pages=per_group or max(1, pages),
                                    max_requests=ec.max_concurrent_requests, dtype=self.rt.dtype,
                                    device=self.rt.device)
        self.step_fn = StepFunction(self.model, self.manager, self.rt, cuda_graphs=ec.cuda_graphs,
                                    native=ec.native_executor)
        self.scheduler = Scheduler(self.manager, SchedulerConfig(ec.max_concurrent_requests,
                                                                 ec.max_num_batched_tokens, ec.prefill_chunk),
                                   eos_token_ids=self.model.eos_token_ids, max_positions=self.model.max_positions)
        self.sampler = Sampler(self.rt)
        self._ids = itertools.count()
        self._pending_outputs: list[RequestOutput] = []
        self._host_out = None
        self._side = None
        self._ahead = None                      # a step launched whose ids have not been read yet
        self.defer_status_check = True          # see _finish
        self._status_unchecked = False
        self.lookahead = bool(ec.lookahead) and self.rt.device.type == "cuda"
        self._requests: dict[str, Request] = {}
        self.counters = {"steps": 0, "prompt_tokens": 0, "generated_tokens": 0, "preemptions": 0, "h2d_bytes": 0,
                         "d2h_bytes": 0}

    # ------------------------------------------------------------------ requests
    def submit(self, prompt_token_ids, sampling: SamplingParams | None = None, request_id: str | None = None) -> str:
        rid = request_id if request_id is not None else f"req-{next(self._ids)}"
        if rid in self._requests:
            raise KeyError(f"request id {rid!r} is in use")
        sp = sampling or SamplingParams()
        req = Request(rid, [int(t) for t in prompt_token_ids], sp)
        req.seed = sp.seed if sp.seed is not None else _request_seed(self.engine_config.seed, rid)
        out = self.scheduler.add_request(req)
        if out is not None:
            self._pending_outputs.append(out)
        else:
            self._requests[rid] = req
        return rid

    def abort(self, request_id: str) -> None:
        self.scheduler.abort(request_id)

    def reconfigure(self, *, max_num_batched_tokens: int | None = None, prefill_chunk: int | None = None) -> None:
        """Change the scheduler's token budget or portion size between requests (the
        reference's scheduler config, scheduler/scheduler.go:30-47, is fixed at start)."""
        if self.has_unfinished():
            raise RuntimeError("the scheduler is reconfigured only while no request is live")
        if max_num_batched_tokens is not None:
            self.scheduler.cfg.max_num_batched_tokens = self.engine_config.max_num_batched_tokens = int(max_num_batched_tokens)
        if prefill_chunk is not None:
            self.scheduler.cfg.prefill_chunk = self.engine_config.prefill_chunk = int(prefill_chunk)

    def has_unfinished(self) -> bool:
        return bool(self._pending_outputs) or self._ahead is not None or self.scheduler.has_unfinished()

    # ------------------------------------------------------------------ one iteration
    def step(self) -> list[RequestOutput]:
        """Advance by one model step and report what is known by then.  In steady decoding the
        engine runs one step ahead of the host: it launches step N+1 (whose token ids are
        copied on the device from step N's samples) before it waits for step N's ids, so the
        host's book-keeping hides behind the device's work.  The outputs of a step then come
        back one call later; the tokens are the same."""
        outs, self._pending_outputs = self._pending_outputs, []
        if self._ahead is not None:
            prev = self._ahead
            self._ahead = self._launch_ahead(prev)
            outs.extend(self._finish(prev))
            return outs
        if not self.scheduler.has_unfinished():
            self._settle_status()
            return outs
        plan = self.scheduler.schedule()
        for req in plan.finished:
            outs.append(self.scheduler._output(req, []))
            self._requests.pop(req.request_id, None)
        self.counters["preemptions"] = self.scheduler.num_preemptions
        if not plan.entries:
            return outs
        launched = self._launch(plan, None, outs)
        if launched is None:
            return outs
        if self.lookahead and self.step_fn.graphable(plan.entries) and all(plan.samples):
            self._ahead = launched                       # its outputs come with the next call
        else:
            outs.extend(self._finish(launched))
        return outs

    def flush(self) -> list[RequestOutput]:
        """Wait for the step that is still in flight, if any, and report it."""
        outs, self._pending_outputs = self._pending_outputs, []
        if self._ahead is not None:
            prev, self._ahead = self._ahead, None
            outs.extend(self._finish(prev))
        if not self.scheduler.has_unfinished():
            self._settle_status()
        return outs

    def _settle_status(self) -> None:
        """Nothing is running any more: a status left by a portion whose request was aborted
        before any of its tokens was read must not fall on the next request."""
        if self._status_unchecked:
            self._status_unchecked = False
            try:
                self.step_fn.check_status()
            except StepError:
                pass                                 # the request it belonged to is gone

    def _launch(self, plan, tokens_from, outs):
        """Put a planned step on the device.  -> (plan, sampled ids on the device, readiness
        event) or None after reporting a failure."""
        try:
            ahead = 1 if tokens_from is not None else 0
            rows = [(req.sampling, req.seed, len(req.output_token_ids) + ahead,
                     req.tail(req.sampling.history_needed) if not ahead else [])
                    for req, s in zip(plan.requests, plan.samples) if s]
            # every row takes its largest logit as it stands: the head chooses inside its product
            greedy = bool(rows) and all(p.greedy and not p.logit_bias and not p.penalties_on for p, _, _, _ in rows)
            out = self.step_fn.run(plan.entries, reserved=True, check=False, tokens_from=tokens_from, greedy=greedy)
            sampled = (out if greedy else self.sampler.sample(out, rows)) if rows else None
        except (StepError, RuntimeError) as e:
            outs.extend(self.scheduler.step_failed(plan, str(e)))
            for req in plan.requests:
                self._requests.pop(req.request_id, None)
            return None
        ready = None
        if self.rt.device.type == "cuda":
            ready = torch.cuda.Event()
            ready.record()
        for req, entry in zip(plan.requests, plan.entries):
            n_prompt = len(req.prompt_token_ids)
            self.counters["prompt_tokens"] += max(0, min(n_prompt, req.num_computed + len(entry.tokens))
                                                  - min(n_prompt, req.num_computed))
        self.scheduler.step_launched(plan)
        self.counters["steps"] += 1
        self.counters["h2d_bytes"] += self.step_fn.last_h2d_bytes
        return plan, sampled, ready

    def _launch_ahead(self, prev):
        plan = self.scheduler.plan_ahead(prev[0]) if self.lookahead else None
        if plan is None:
            return None
        outs: list[RequestOutput] = []
        launched = self._launch(plan, prev[1], outs)
        self._pending_outputs.extend(outs)
        return launched

    def _finish(self, launched) -> list[RequestOutput]:
        """Wait for a launched step's ids and let the scheduler digest them."""
        plan, sampled, ready = launched
        outs: list[RequestOutput] = []
        try:
            tokens = self._read_back(sampled, ready) if sampled is not None else []
            if sampled is None:
                # A portion of a prompt that asks for no token: nothing to wait for.  The kernels'
                # status word keeps what it was given, and the next step that reads ids back reads
                # it too (the request is still running then); waiting here would leave the device
                # idle for every portion's launches and the host idle for every portion's run.
                if self.defer_status_check and self.rt.device.type == "cuda":
                    self._status_unchecked = True
                else:
                    self.step_fn.check_status()
        except (StepError, RuntimeError) as e:
            outs.extend(self.scheduler.step_failed(plan, str(e)))
            for req in plan.requests:
                self._requests.pop(req.request_id, None)
            if self._ahead is not None:                  # what was launched on top of it is void too
                outs.extend(self.scheduler.step_failed(self._ahead[0], str(e)))
                self._ahead = None
            return outs
        self.counters["d2h_bytes"] += 4 * len(tokens) + 16
        self.counters["generated_tokens"] += len(tokens)
        for out in self.scheduler.step_done(plan, tokens):
            outs.append(out)
            if out.finished:
                self._requests.pop(out.request_id, None)
        return outs

    def _read_back(self, sampled: torch.Tensor, ready=None) -> list[int]:
        """Sampled ids and the kernels' status word in one wait: two small copies into pinned
        memory on a side stream that waits only for the step that made them (a later step may
        already be running on the main stream), one synchronisation."""
        n = sampled.numel()
        if self.rt.device.type != "cuda":
            self.step_fn.check_status()
            return sampled.tolist()
        if self._host_out is None or self._host_out.numel() < n + 4:
            self._host_out = torch.empty(max(n + 4, 260), dtype=torch.int32).pin_memory()
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.rt.device)
        with torch.cuda.stream(self._side):
            if ready is not None:
                self._side.wait_event(ready)
            self._host_out[:n].copy_(sampled, non_blocking=True)
            self._host_out[n:n + 4].copy_(self.step_fn.status, non_blocking=True)
        self._side.synchronize()
        vals = self._host_out[:n + 4].tolist()
        self._status_unchecked = False
        if vals[n]:
            torch.cuda.current_stream().synchronize()
            self.step_fn.check_status()          # raises with the code's meaning and clears the word
        return vals[:n]

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts, sampling: SamplingParams | list[SamplingParams] | None = None) -> list[RequestOutput]:
        """Run the prompts (lists of token ids) to the end; -> final outputs in prompt order."""
        if prompts and isinstance(prompts[0], int):
            prompts = [prompts]
        params = sampling if isinstance(sampling, list) else [sampling] * len(prompts)
        ids = [self.submit(p, sp) for p, sp in zip(prompts, params)]
        final: dict[str, RequestOutput] = {}
        while self.has_unfinished():
            for out in self.step():
                if out.finished:
                    final[out.request_id] = out
        return [final[i] for i in ids]

    def stats(self) -> dict:
        g = self.manager.groups
        return dict(self.counters, waiting=len(self.scheduler.waiting), running=len(self.scheduler.running),
                    pages_total=sum(x.pool.num_pages for x in g), pages_used=sum(x.pool.used_pages for x in g),
                    model_steps=self.step_fn.steps, graph_replays=self.step_fn.graph_replays,
                    native_executor=self.step_fn.native is not None)
