"""The step function: run a batch of (request, its next tokens) from the cache and
return the logits at the wanted places.

tamnd/fastmlx's generator knows three exclusive batch shapes (one token per row at equal
offsets, whole left-padded prompts, or one sequence at a time: compute/batch_generator.go:
178-195) and never a portion of a prompt beside a decoded token.  Here a step is one flat
ragged batch over a paged cache: any mix, cut anywhere.  An error leaves no state
advanced, as there (batch_generator.go:187-191).
"""
from __future__ import annotations

import torch

from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from .batch import StepContext, StepEntry, build_context


class StepError(RuntimeError):
    pass


STATUS_WORDS = 4
_STATUS_TEXT = {1: "a token id outside the vocabulary", 2: "a cache slot outside the pool",
                3: "a block-table entry that holds no page", 4: "a row index outside the batch"}


class StepFunction:
    def __init__(self, model, manager: CacheManager, rt, cuda_graphs: bool = False):
        self.model, self.manager, self.rt = model, manager, rt
        self.cuda_graphs = bool(cuda_graphs) and rt.device.type == "cuda"
        self.graph_replays = 0
        self.last_h2d_bytes = 0
        self.status = torch.zeros(STATUS_WORDS, dtype=torch.int32, device=rt.device)
        self.steps = 0
        self.tokens_run = 0
        self.last_ctx: StepContext | None = None

    def run(self, entries: list[StepEntry], reserved: bool = False, check: bool = True) -> torch.Tensor:
        """-> float32 logits [sum(len(e.want)), vocab] on the device, in the order of the
        entries and of their `want`.  `reserved`: the caller (the scheduler) has taken the
        pages already and commits or rolls back itself.  `check=False` leaves the read of
        the kernels' status word to the caller, who reads results from the device anyway."""
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if not e.tokens:
                raise StepError("an entry brings no token")
            if id(e.request) in seen:
                raise StepError("a request appears twice in one step")
            seen.add(id(e.request))
            limit = self.model.max_positions
            if limit and e.request.length + len(e.tokens) > limit:
                raise StepError(f"request {e.request.request_id!r} would pass max_position_embeddings ({limit})")
        taken = []
        try:
            if not reserved:
                for e in entries:
                    self.manager.reserve(e.request, len(e.tokens))
                    taken.append(e.request)
            ctx = build_context(entries, self.manager, self.rt.device, self.status)
            logits = self.model.forward(ctx)
            if check:
                self.check_status()
        except BaseException:
            for r in taken:
                self.manager.rollback(r)
            raise
        for r in taken:
            self.manager.commit(r)
        self.last_h2d_bytes = ctx.scratch.get("h2d_bytes", 0)
        self.steps += 1
        self.tokens_run += ctx.T
        self.last_ctx = ctx
        return logits

    def check_status(self) -> None:
        """Kernels never trap on a bad index: they skip the access and leave a code."""
        st = self.status.tolist()
        if st[0]:
            self.status.zero_()
            raise StepError(f"a kernel met {_STATUS_TEXT.get(st[0], 'an error')} (code {st[0]}, value {st[1]}, at {st[2]})")
