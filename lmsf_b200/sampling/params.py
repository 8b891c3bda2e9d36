"""Sampling options of a request.

Names, defaults and range checks follow the reference's SamplingParams
(core/src/common/sampling_params.rs:29-80 defaults, :166-299 verify).  `seed` is per request here
(the reference has one engine-wide generator seeded by --seed, core/src/engine/llm_engine.rs:112-116).
Options that need several sequences per request (n, best_of, beam search) and log-probabilities
are parsed so that a caller gets a clear refusal instead of a silent default.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

_SAMPLING_EPS = 1e-5


@dataclass
class SamplingParams:
    n: int = 1
    best_of: Optional[int] = None
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    repetition_penalty: float = 1.0
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    use_beam_search: bool = False
    stop_token_ids: List[int] = field(default_factory=list)
    ignore_eos: bool = False
    max_tokens: int = 128
    logprobs: Optional[int] = None
    seed: Optional[int] = None

    def __post_init__(self):
        self.verify()

    @property
    def greedy(self) -> bool:
        # core/src/common/sampling_params.rs:156-164
        return self.temperature < _SAMPLING_EPS

    @property
    def filters_active(self) -> bool:
        return (not self.greedy) and (self.top_k > 0 or self.top_p < 1.0 or self.min_p > 0.0)

    @property
    def penalties_active(self) -> bool:
        return self.presence_penalty != 0.0 or self.frequency_penalty != 0.0 or self.repetition_penalty != 1.0

    def verify(self) -> None:
        if self.n != 1 or (self.best_of not in (None, 1)) or self.use_beam_search:
            raise ValueError("n > 1, best_of > 1 and beam search need several sequences per request, "
                             "which this engine does not have")
        if self.logprobs is not None:
            raise ValueError("logprobs are not returned by this engine")
        if not (-2.0 <= self.presence_penalty <= 2.0):
            raise ValueError(f"presence_penalty must be in [-2, 2], got {self.presence_penalty}")
        if not (-2.0 <= self.frequency_penalty <= 2.0):
            raise ValueError(f"frequency_penalty must be in [-2, 2], got {self.frequency_penalty}")
        if not (0.0 < self.repetition_penalty <= 2.0):
            raise ValueError(f"repetition_penalty must be in (0, 2], got {self.repetition_penalty}")
        if self.temperature < 0.0:
            raise ValueError(f"temperature must be non-negative, got {self.temperature}")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"top_p must be in (0, 1], got {self.top_p}")
        if self.top_k < -1 or self.top_k == 0:
            raise ValueError(f"top_k must be -1 (disable), or at least 1, got {self.top_k}")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError(f"min_p must be in [0, 1], got {self.min_p}")
        if self.max_tokens < 1:
            raise ValueError(f"max_tokens must be at least 1, got {self.max_tokens}")
        if self.seed is not None and not (0 <= self.seed < 2 ** 64):
            raise ValueError("seed must fit 64 unsigned bits")
