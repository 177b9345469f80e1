"""Requests and what the engine reports about them (tamnd/fastmlx engine/types.go:11-80)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field

from ..sampling.params import SamplingParams


class RequestStatus(enum.IntEnum):
    """engine/types.go:11-24.  PREFILLING and PREEMPTED are declared there and never set;
    here they are."""
    WAITING = 0
    PREFILLING = 1
    RUNNING = 2
    PREEMPTED = 3
    FINISHED_STOPPED = 4
    FINISHED_LENGTH = 5
    FINISHED_ABORTED = 6
    FINISHED_ERROR = 7

    @property
    def finished(self) -> bool:
        return self >= RequestStatus.FINISHED_STOPPED


FINISH_REASON = {RequestStatus.FINISHED_STOPPED: "stop", RequestStatus.FINISHED_LENGTH: "length",
                 RequestStatus.FINISHED_ABORTED: "abort", RequestStatus.FINISHED_ERROR: "error"}


@dataclass
class Request:
    request_id: str
    prompt_token_ids: list[int]
    sampling: SamplingParams
    arrival: int = 0                      # admission order; the scheduler is first come first served
    status: RequestStatus = RequestStatus.WAITING
    output_token_ids: list[int] = field(default_factory=list)
    num_computed: int = 0                 # tokens whose keys are in the cache
    cache: object = None                  # cache.RequestCache while the request holds pages
    seed: int = 0
    error: str = ""
    preemptions: int = 0

    @property
    def all_token_ids(self) -> list[int]:
        return self.prompt_token_ids + self.output_token_ids

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    @property
    def last_token(self) -> int:
        return self.output_token_ids[-1] if self.output_token_ids else self.prompt_token_ids[-1]

    def tokens_from(self, start: int, n: int) -> list[int]:
        """Tokens [start, start + n) of prompt + output without joining the two lists."""
        np_ = len(self.prompt_token_ids)
        if start + n <= np_:
            return self.prompt_token_ids[start:start + n]
        if start >= np_:
            return self.output_token_ids[start - np_: start - np_ + n]
        return self.prompt_token_ids[start:] + self.output_token_ids[: start + n - np_]

    def tail(self, n: int) -> list[int]:
        """The last n tokens of prompt + output (for the penalties' window)."""
        if n <= 0:
            return []
        out = self.output_token_ids[-n:]
        if len(out) < n:
            out = self.prompt_token_ids[-(n - len(out)):] + out
        return out

    @property
    def finish_reason(self) -> str:
        return FINISH_REASON.get(self.status, "")


@dataclass
class RequestOutput:
    """One increment, or the final result, of a request (engine/types.go:64-80)."""
    request_id: str
    new_token_ids: list[int]
    output_token_ids: list[int]
    finished: bool
    finish_reason: str
    prompt_tokens: int
    completion_tokens: int
    err: str = ""
