"""Sampling options, with tamnd/fastmlx's names, meanings and defaults."""
from __future__ import annotations

from dataclasses import dataclass, field

PENALTY_WINDOW = 20          # compute/logits_processor.go:40


@dataclass
class SamplingParams:
    """Fields and defaults after engine/types.go:29-42 and the fallback of
    routes/router.go:98-138 (temperature 1.0, top_p 0.95, top_k 0, repetition_penalty 1.0,
    max_tokens 32768).  temperature 0 means greedy: argmax, the first index on ties
    (compute/sampler.go:38-39,61-72).  Filters act in the order top-p, min-p, top-k
    (sampler.go:46-59); processors in the order logit_bias, repetition, presence, frequency
    (compute/logits_processor.go:148-164).  `seed` makes the draw a function of
    (seed, index of the generated token) alone; the reference carries the field and never
    reads it."""
    max_tokens: int = 32768
    temperature: float = 1.0
    top_p: float = 0.95
    top_k: int = 0
    min_p: float = 0.0
    min_tokens_to_keep: int = 1
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_context_size: int = PENALTY_WINDOW
    presence_context_size: int = PENALTY_WINDOW
    frequency_context_size: int = PENALTY_WINDOW
    logit_bias: dict[int, float] = field(default_factory=dict)
    seed: int | None = None
    stop_token_ids: list[int] = field(default_factory=list)
    ignore_eos: bool = False

    def __post_init__(self):
        if self.max_tokens is None or self.max_tokens <= 0:
            self.max_tokens = 32768                       # routes/router.go:133-135
        if self.temperature < 0:
            raise ValueError("temperature must not be negative")
        for k in ("repetition_context_size", "presence_context_size", "frequency_context_size"):
            if getattr(self, k) <= 0:
                setattr(self, k, PENALTY_WINDOW)           # logits_processor.go:172-178

    @property
    def greedy(self) -> bool:
        return self.temperature == 0

    @property
    def filters_on(self) -> bool:
        return (not self.greedy) and ((0 < self.top_p < 1.0) or self.min_p != 0.0 or self.top_k > 0)

    @property
    def penalties_on(self) -> bool:
        return (self.repetition_penalty not in (0.0, 1.0)) or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0

    @property
    def history_needed(self) -> int:
        return max(self.repetition_context_size, self.presence_context_size, self.frequency_context_size) \
            if self.penalties_on else 0
