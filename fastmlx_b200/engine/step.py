"""The step function: run a batch of (request, its next tokens) from the cache and
return the logits at the wanted places.

tamnd/fastmlx's generator knows three exclusive batch shapes (one token per row at equal
offsets, whole left-padded prompts, or one sequence at a time: compute/batch_generator.go:
178-195) and never a portion of a prompt beside a decoded token.  Here a step is one flat
ragged batch over a paged cache: any mix, cut anywhere.  An error leaves no state
advanced, as there (batch_generator.go:187-191).

Steps in which every request brings exactly one token are launch-bound, so they run as
CUDA graphs: one graph per (rows rounded up to a power of two, block-table width rounded
up to a power of two), captured at first use, fed through fixed buffers.
"""
from __future__ import annotations

import numpy as np
import torch

from ..cache.manager import CacheManager
from .batch import StaticBuffers, StepContext, StepEntry, build_context


class StepError(RuntimeError):
    pass


STATUS_WORDS = 4
_STATUS_TEXT = {1: "a token id outside the vocabulary", 2: "a cache slot outside the pool",
                3: "a block-table entry that holds no page", 4: "a row index outside the batch",
                5: "a wait inside a kernel that ran out of time"}


def _pow2_at_least(n: int, floor: int = 1) -> int:
    p = floor
    while p < n:
        p *= 2
    return p


class _DecodeGraph:
    """One captured decode step for `rows` rows and block tables `width` pages wide."""

    def __init__(self, fn: "StepFunction", rows: int, width: int, entries, greedy: bool = False):
        self.rows, self.width, self.greedy = rows, width, greedy
        rt, manager = fn.rt, fn.manager
        probe = build_context(entries, manager, None, fn.status, pad_rows=rows, pad_blocks=width, pad_want=True)
        n = probe.scratch["layout_ints"]
        self.static = StaticBuffers(n, rt.device)
        ctx = self._context(fn, entries)
        # warm up outside the capture (library handles, lazily built kernels), then capture.  The
        # warm-up runs the real step once and the first replay runs it again: writing the same
        # keys and values twice changes nothing, but per-request state would advance twice, so
        # it is put back as it was.
        saved = manager.snapshot_state() if manager.has_state else None
        side = torch.cuda.Stream(device=rt.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn.forward_context(ctx, greedy)
        torch.cuda.current_stream().wait_stream(side)
        if saved is not None:
            manager.restore_state(saved)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        count = getattr(rt.k, "launch_count", lambda: 0)
        before = count()
        with torch.cuda.graph(self.graph):
            self.logits = fn.forward_context(ctx, greedy)
        self.kernel_launches = count() - before        # launches of this package's kernels per replay
        self.ctx = ctx

    def _context(self, fn, entries) -> StepContext:
        ctx = build_context(entries, fn.manager, fn.rt.device, fn.status, pad_rows=self.rows, pad_blocks=self.width,
                            pad_want=True, static=self.static)
        ctx.max_ctx_after = self.width * fn.manager.page_size      # fixed, so that the split count is
        ctx.max_q_len = 1
        return ctx

    def run(self, fn, entries, tokens_from=None) -> tuple[torch.Tensor, StepContext]:
        ctx = self._context(fn, entries)
        if tokens_from is not None:
            # the ids sampled by the step before, still on the device: the token ids are the
            # first array of the packed buffer
            self.static.dev[:tokens_from.numel()].copy_(tokens_from)
        self.graph.replay()
        return self.logits, ctx


class StepFunction:
    def __init__(self, model, manager: CacheManager, rt, cuda_graphs: bool = False, max_graph_rows: int = 256,
                 position_limit: bool = True, native: bool = True):
        """position_limit: refuse a step that would take a request past the model's
        max_position_embeddings (the serving policy); replay turns it off and runs what it is given.
        native: hand the step's host work (layout, choice of kernels, launches) to the compiled
        executor where every part of the model can describe itself to it; else, and for models
        with parts written in Python, `Model.forward` runs."""
        self.model, self.manager, self.rt = model, manager, rt
        self.position_limit = bool(position_limit)
        self.cuda_graphs = bool(cuda_graphs) and rt.device.type == "cuda" and bool(getattr(model, "graph_safe", False))
        self.max_graph_rows = max_graph_rows
        self.graphs: dict[tuple[int, int], _DecodeGraph] = {}
        self.graph_replays = 0
        self.graph_kernel_launches = 0
        self.last_h2d_bytes = 0
        self.status = torch.zeros(STATUS_WORDS, dtype=torch.int32, device=rt.device)
        if hasattr(rt.k, "set_status_word") and rt.device.type == "cuda":
            rt.k.set_status_word(rt.device, self.status)
        self.steps = 0
        self.tokens_run = 0
        self.last_ctx: StepContext | None = None
        self.native = None
        if native and rt.device.type == "cuda" and getattr(rt.k, "__name__", "") == "fastmlx_b200.kernels":
            from .native import build_program
            self.native = build_program(model, manager, rt, self.status, max_graph_rows)
        if self.cuda_graphs:
            # workspaces whose addresses the graphs will hold are made before any capture
            for name in ("attention_scratch", "attention_tickets", "argmax_workspace"):
                make = getattr(rt.k, name, None)
                if make is not None:
                    make(rt.device)

    def run(self, entries: list[StepEntry], reserved: bool = False, check: bool = True,
            tokens_from: torch.Tensor | None = None, greedy: bool = False) -> torch.Tensor:
        """-> float32 logits [sum(len(e.want)), vocab] on the device, in the order of the
        entries and of their `want`; with `greedy`, the index of each wanted place's largest logit
        instead (int32 [sum(len(e.want))], the lowest index on ties), which a decode step's head
        chooses inside its product without writing logits.  `reserved`: the caller (the scheduler) has taken the
        pages already and commits or rolls back itself.  `check=False` leaves the read of
        the kernels' status word to the caller, who reads results from the device anyway.
        The tensor may be a view of a graph's output: use it before the next step.
        `tokens_from` (one token per entry): take the ids from this device tensor instead of
        from the entries, whose tokens are then place-holders."""
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if not e.tokens:
                raise StepError("an entry brings no token")
            if id(e.request) in seen:
                raise StepError("a request appears twice in one step")
            seen.add(id(e.request))
            limit = self.model.max_positions if self.position_limit else 0
            if limit and e.request.length + len(e.tokens) > limit:
                raise StepError(f"request {e.request.request_id!r} would pass max_position_embeddings ({limit})")
        taken = []
        # With `check` the step's outcome is known before this returns, and a failed step leaves
        # pages and per-request state as they were.  Without it the caller reads the status later
        # and fails the step's requests, whose pages and slots are then given back whole.
        saved = self.manager.snapshot_state([e.request.slot for e in entries]) \
            if check and self.manager.has_state else None
        try:
            if not reserved:
                for e in entries:
                    self.manager.reserve(e.request, len(e.tokens))
                    taken.append(e.request)
            logits, ctx = self._forward(entries, tokens_from, greedy)
            if check:
                self.check_status()
        except BaseException:
            for r in taken:
                self.manager.rollback(r)
            if saved is not None:
                self.manager.restore_state(saved)
            raise
        for r in taken:
            self.manager.commit(r)
        self.last_h2d_bytes = ctx.scratch.get("h2d_bytes", 0)
        self.steps += 1
        self.tokens_run += ctx.T
        self.last_ctx = ctx
        return logits

    def graphable(self, entries) -> bool:
        return self.cuda_graphs and len(entries) <= self.max_graph_rows and all(len(e.tokens) == 1 for e in entries)

    def _forward(self, entries, tokens_from=None, greedy: bool = False):
        if tokens_from is not None and not self.graphable(entries):
            raise StepError("ids can be fed from the device only into a captured decode step")
        if self.cuda_graphs and len(entries) <= self.max_graph_rows and all(len(e.tokens) == 1 for e in entries):
            ps = self.manager.page_size
            rows = _pow2_at_least(len(entries))
            blocks = max(-(-(e.request.length + 1) // ps) for e in entries)
            width = _pow2_at_least(blocks, 16)
            key = (rows, width, True) if greedy else (rows, width)
            g = self.graphs.get(key)
            if g is None:
                g = self.graphs[key] = _DecodeGraph(self, rows, width, entries, greedy)
            logits, ctx = g.run(self, entries, tokens_from)
            if greedy:
                # the ids lie in the graph's own output, which its next replay overwrites, and an engine
                # that runs a step ahead reads them on another stream after that replay is launched
                logits = logits.clone()
            self.graph_replays += 1
            self.graph_kernel_launches += g.kernel_launches
            # one wanted place per row in the graph; give back what was asked for
            picks = [i for i, e in enumerate(entries) if e.want]
            if len(picks) == len(entries):
                return logits[:len(entries)], ctx
            if not picks:
                return logits[:0], ctx
            return logits[torch.as_tensor(picks, device=logits.device)], ctx
        if self.native is not None:
            return self.native.step(entries, greedy)
        ctx = build_context(entries, self.manager, self.rt.device, self.status)
        return self.forward_context(ctx, greedy), ctx

    def forward_context(self, ctx: StepContext, greedy: bool = False) -> torch.Tensor:
        """The model over a step that is laid out already (the captured decode steps)."""
        if self.native is not None:
            return self.native.forward_context(ctx, greedy)
        if not greedy:
            return self.model.forward(ctx)
        try:
            return self.model.forward(ctx, greedy=True)
        except TypeError:                     # a model class of its own whose forward knows no greedy head
            return self.rt.k.argmax(self.model.forward(ctx))

    def check_status(self) -> None:
        """Kernels never trap on a bad index: they skip the access and leave a code."""
        st = self.status.tolist()
        if st[0]:
            self.status.zero_()
            raise StepError(f"a kernel met {_STATUS_TEXT.get(st[0], 'an error')} (code {st[0]}, value {st[1]}, at {st[2]})")
