"""Continuous batching: which requests run in the next step, and with how many tokens.

tamnd/fastmlx's scheduler admits first come first served up to MaxNumSeqs, gives every
running sequence one token per step and retires finished ones (scheduler/scheduler.go:
126-254); its MaxNumBatchedTokens (8192) is declared and never read (scheduler.go:32,44),
prompts are never split, and running out of cache is not modelled (the PREEMPTED status of
engine/types.go:17 is never assigned).  Here a step has a token budget, prompts are cut
into portions under it, and page exhaustion has a decided outcome:

  1. every running request that is decoding gets its one token; if no page is left for
     it, the most recently admitted running request is preempted: its pages and slot go
     back, and it returns to the front of the waiting queue with its generated tokens
     kept (they are recomputed as part of its prompt when it is admitted again);
  2. what is left of the budget goes, in admission order, to running requests whose
     prompt is not yet all in the cache, then to waiting requests while there is room for
     more sequences; a portion that cannot get its pages waits for a later step;
  3. if nothing at all could be scheduled while requests run, the most recent one is
     preempted so that the oldest can go on; a request that cannot go on even alone ends
     with reason "length".
A prompt that can never fit (longer than the pool or than max_position_embeddings) fails
at admission with an error.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from .batch import StepEntry
from .request import Request, RequestOutput, RequestStatus


@dataclass
class SchedulerConfig:
    max_num_seqs: int = 8                     # scheduler/scheduler.go:43 (DefaultConfig)
    max_num_batched_tokens: int = 8192        # scheduler/scheduler.go:44
    prefill_chunk: int = 0                    # longest portion of one prompt in a step; 0 = the budget


@dataclass
class Plan:
    entries: list[StepEntry] = field(default_factory=list)
    requests: list[Request] = field(default_factory=list)      # parallel to entries
    samples: list[bool] = field(default_factory=list)          # does this entry yield a token?
    preempted: list[Request] = field(default_factory=list)
    finished: list[Request] = field(default_factory=list)      # ended while planning (errors, aborts)
    launched: bool = False                                     # its tokens are committed to the cache

    @property
    def num_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, manager: CacheManager, config: SchedulerConfig, *, eos_token_ids=(), max_positions: int = 0):
        self.manager, self.cfg = manager, config
        self.eos = set(int(e) for e in eos_token_ids if e is not None and int(e) >= 0)
        self.max_positions = int(max_positions)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self._aborts: set[str] = set()
        self._arrivals = 0
        self.num_preemptions = 0

    # ------------------------------------------------------------------ admission
    def add_request(self, req: Request) -> RequestOutput | None:
        """Queue a request; -> a final output right away when it can never run."""
        req.arrival = self._arrivals
        self._arrivals += 1
        n = len(req.prompt_token_ids)
        portion = self.cfg.prefill_chunk if self.cfg.prefill_chunk > 0 else self.cfg.max_num_batched_tokens
        pool_tokens = self.manager.holds_alone(n, portion)
        err = ""
        if n == 0:
            err = "empty prompt"                       # compute/batch_generator.go:71,128-130
        elif self.max_positions and n >= self.max_positions:
            err = f"prompt of {n} tokens leaves no room under max_position_embeddings ({self.max_positions})"
        elif pool_tokens:
            err = f"prompt of {n} tokens exceeds the cache pool of {pool_tokens} tokens"
        if err:
            req.status, req.error = RequestStatus.FINISHED_ERROR, err
            return self._output(req, [])
        self.waiting.append(req)
        return None

    def abort(self, request_id: str) -> None:
        """Marked now, applied at the next `schedule` (scheduler/scheduler.go:114-118,258-291)."""
        self._aborts.add(request_id)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ planning
    def schedule(self) -> Plan:
        plan = Plan()
        self._apply_aborts(plan)
        budget = self.cfg.max_num_batched_tokens
        chunk_cap = self.cfg.prefill_chunk if self.cfg.prefill_chunk > 0 else budget
        scheduled: set[int] = set()

        # 1. decodes
        i = 0
        while i < len(self.running) and budget > 0:
            req = self.running[i]
            if not self._decoding(req):
                i += 1
                continue
            while True:
                try:
                    self.manager.reserve(req.cache, 1)
                    break
                except OutOfPages:
                    victim = self.running[-1]
                    if victim is req and len(self.running) == 1:
                        self._finish(req, RequestStatus.FINISHED_LENGTH, plan)     # cannot go on even alone
                        break
                    if id(victim) in scheduled:
                        self._unschedule(victim, plan, scheduled)
                    self._preempt(victim, plan)
                    if victim is req:
                        break
            if req.status == RequestStatus.RUNNING and req.cache is not None and req.cache.reserved:
                self._add(plan, req, [req.last_token], True, scheduled)
                budget -= 1
                i += 1
            # else: req left `running` (preempted or finished); the same index holds the next one

        # 2. portions of prompts: running ones first, then waiting ones
        for req in list(self.running):
            if budget <= 0:
                break
            if self._decoding(req) or id(req) in scheduled:
                continue
            budget -= self._schedule_portion(req, min(budget, chunk_cap), plan, scheduled)
        while self.waiting and budget > 0 and len(self.running) < self.cfg.max_num_seqs:
            req = self.waiting[0]
            try:
                req.cache = self.manager.add_request(req.request_id)
            except OutOfPages:
                break
            took = self._schedule_portion(req, min(budget, chunk_cap), plan, scheduled)
            if took == 0:
                self.manager.free(req.request_id)
                req.cache = None
                break
            self.waiting.popleft()
            req.status = RequestStatus.PREFILLING
            self.running.append(req)
            budget -= took

        # 3. nothing runs although requests hold pages: make room for the oldest
        if not plan.entries and self.running:
            if len(self.running) > 1:
                self._preempt(self.running[-1], plan)
                more = self.schedule()
                more.preempted = plan.preempted + more.preempted
                more.finished = plan.finished + more.finished
                return more
            self._finish(self.running[0], RequestStatus.FINISHED_LENGTH, plan)
        return plan

    def _decoding(self, req: Request) -> bool:
        """All tokens but the newest are in the cache: the request wants one decode step."""
        return req.status == RequestStatus.RUNNING and req.num_computed == req.num_tokens - 1

    def _schedule_portion(self, req: Request, room: int, plan: Plan, scheduled) -> int:
        total = req.num_tokens
        left = total - req.num_computed
        n = min(left, room)
        if n <= 0:
            return 0
        try:
            self.manager.reserve(req.cache, n)
        except OutOfPages:
            n = min(n, self._room_in_pages(req))         # a shorter portion may still fit
            if n <= 0:
                return 0
            try:
                self.manager.reserve(req.cache, n)
            except OutOfPages:
                return 0
        last = req.num_computed + n == total
        self._add(plan, req, req.tokens_from(req.num_computed, n), last, scheduled)
        return n

    def _room_in_pages(self, req: Request) -> int:
        ps = self.manager.page_size
        tail = -req.cache.length % ps                    # free places on the request's last page
        return tail + self.manager.free_pages * ps

    def _add(self, plan: Plan, req: Request, tokens, sample: bool, scheduled) -> None:
        plan.entries.append(StepEntry(req.cache, list(tokens), [len(tokens) - 1] if sample else []))
        plan.requests.append(req)
        plan.samples.append(sample)
        scheduled.add(id(req))

    def _unschedule(self, req: Request, plan: Plan, scheduled) -> None:
        i = plan.requests.index(req)
        self.manager.rollback(req.cache)
        del plan.entries[i], plan.requests[i], plan.samples[i]
        scheduled.discard(id(req))

    def _preempt(self, req: Request, plan: Plan) -> None:
        if req.cache is not None and req.cache.reserved:
            self.manager.rollback(req.cache)
        self.manager.free(req.request_id)
        req.cache, req.num_computed = None, 0
        req.status = RequestStatus.PREEMPTED
        req.preemptions += 1
        self.num_preemptions += 1
        self.running.remove(req)
        self.waiting.appendleft(req)
        plan.preempted.append(req)

    def _finish(self, req: Request, status: RequestStatus, plan: Plan | None = None) -> None:
        if req.cache is not None:
            if req.cache.reserved:
                self.manager.rollback(req.cache)
            if req.request_id in self.manager.requests:
                self.manager.free(req.request_id)
            req.cache = None
        req.status = status
        if req in self.running:
            self.running.remove(req)
        if plan is not None:
            plan.finished.append(req)

    def _apply_aborts(self, plan: Plan) -> None:
        if not self._aborts:
            return
        for req in [r for r in self.waiting if r.request_id in self._aborts]:
            self.waiting.remove(req)
            req.status = RequestStatus.FINISHED_ABORTED
            plan.finished.append(req)
        for req in [r for r in self.running if r.request_id in self._aborts]:
            self._finish(req, RequestStatus.FINISHED_ABORTED, plan)
        self._aborts.clear()

    # ------------------------------------------------------------------ after the step
    def step_failed(self, plan: Plan, message: str) -> list[RequestOutput]:
        """A backend error ends every request of the step with reason "error"
        (scheduler/scheduler.go:139-145,294-307); the pages they took go back."""
        outs = []
        for req in plan.requests:
            if req.status.finished:
                continue
            req.error = message
            self._finish(req, RequestStatus.FINISHED_ERROR)
            outs.append(self._output(req, []))
        return outs

    def step_launched(self, plan: Plan) -> None:
        """The step is on its way: its tokens count as in the cache (the pages are committed).
        What the tokens *are* is not needed for this, so an engine that runs one step ahead
        calls it before the sampled ids have come back."""
        for entry, req in zip(plan.entries, plan.requests):
            self.manager.commit(req.cache)
            req.num_computed += len(entry.tokens)
        plan.launched = True

    def step_done(self, plan: Plan, tokens: list[int]) -> list[RequestOutput]:
        """The step ran: `tokens` holds one sampled id per entry with samples=True, in order.
        -> the increments to report.  A request that ended while this step was already in
        flight (one step ahead) is skipped: its token is dropped."""
        if not plan.launched:
            self.step_launched(plan)
        outs = []
        it = iter(tokens)
        for entry, req, sample in zip(plan.entries, plan.requests, plan.samples):
            if not sample:
                continue
            tok = int(next(it))
            if req.status.finished:
                continue
            req.output_token_ids.append(tok)
            req.status = RequestStatus.RUNNING
            sp = req.sampling
            if (tok in self.eos and not sp.ignore_eos) or tok in sp.stop_token_ids:
                self._finish(req, RequestStatus.FINISHED_STOPPED)      # batch_generator.go:319-329, scheduler.go:192-231
            elif len(req.output_token_ids) >= sp.max_tokens:
                self._finish(req, RequestStatus.FINISHED_LENGTH)
            elif self.max_positions and req.num_tokens >= self.max_positions:
                self._finish(req, RequestStatus.FINISHED_LENGTH)
            outs.append(self._output(req, [tok]))
        return outs

    def plan_ahead(self, prev: Plan) -> Plan | None:
        """The step after `prev`, planned before prev's sampled ids are known: possible when
        prev gave every running request one token, nothing waits, nothing is to be aborted and
        no request can end by length at prev.  Every request gets a place-holder token (the
        engine copies the sampled id in on the device).  None when it cannot be done."""
        if self.waiting or self._aborts or not prev.entries or len(prev.requests) != len(self.running):
            return None
        for entry, req, sample in zip(prev.entries, prev.requests, prev.samples):
            if len(entry.tokens) != 1 or not sample or req.status.finished or req.cache is None:
                return None
            if len(req.output_token_ids) + 2 > req.sampling.max_tokens or req.sampling.penalties_on:
                return None
            if self.max_positions and req.num_tokens + 2 >= self.max_positions:
                return None
        plan = Plan()
        taken = []
        try:
            for req in prev.requests:
                self.manager.reserve(req.cache, 1)
                taken.append(req)
        except OutOfPages:
            for req in taken:
                self.manager.rollback(req.cache)
            return None
        for req in prev.requests:
            plan.entries.append(StepEntry(req.cache, [0], [0]))
            plan.requests.append(req)
            plan.samples.append(True)
        return plan

    def _output(self, req: Request, new) -> RequestOutput:
        return RequestOutput(req.request_id, list(new), list(req.output_token_ids), req.status.finished,
                             req.finish_reason, len(req.prompt_token_ids), len(req.output_token_ids), req.error)
