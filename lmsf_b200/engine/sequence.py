"""Requests as the engine tracks them, and what the engine reports about them.

Reduced from the reference's Sequence / SequenceGroup (core/src/common/sequence.rs:36-65 states,
:125-287 sequence, :289-469 group) to one sequence per request, and from RequestOutput /
CompletionOutput (core/src/common/output.rs:6-55).
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Hashable, List, Optional

from ..sampling.params import SamplingParams


class SequenceStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED_STOPPED = "stop"          # EOS or a stop token
    FINISHED_LENGTH = "length"         # max_tokens, max_model_len or the cache cannot hold more
    FINISHED_ABORTED = "abort"
    FINISHED_IGNORED = "ignored"       # never ran: the prompt cannot fit (cf. core/src/sched/scheduler.rs:367-381)

    @property
    def finished(self) -> bool:
        return self not in (SequenceStatus.WAITING, SequenceStatus.RUNNING)


@dataclass
class Sequence:
    request_id: Hashable
    prompt_token_ids: List[int]
    sampling_params: SamplingParams
    arrival_time: float = field(default_factory=time.monotonic)
    output_token_ids: List[int] = field(default_factory=list)
    status: SequenceStatus = SequenceStatus.WAITING
    num_computed: int = 0             # tokens whose keys and values are in the cache
    num_preemptions: int = 0
    seed: int = 0
    num_pending: int = 0              # tokens sampled on the device whose values the host has not read yet
    hold: bool = False                # not to be scheduled before its pending token is known
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None

    @property
    def token_ids(self) -> List[int]:
        return self.prompt_token_ids + self.output_token_ids

    def __len__(self) -> int:
        """Tokens of the request, those that are sampled but not read yet included."""
        return len(self.prompt_token_ids) + len(self.output_token_ids) + self.num_pending

    @property
    def num_uncomputed(self) -> int:
        return len(self) - self.num_computed

    def next_tokens(self, n: int) -> List[int]:
        """The next n tokens to run; a token that is still pending on the device appears as 0 (a placeholder
        that the step function overwrites on the device)."""
        a = self.num_computed
        n_prompt = len(self.prompt_token_ids)
        if a + n <= n_prompt:
            return self.prompt_token_ids[a:a + n]
        if a >= n_prompt:
            toks = self.output_token_ids[a - n_prompt:a - n_prompt + n]
        else:
            toks = self.prompt_token_ids[a:] + self.output_token_ids[:a + n - n_prompt]
        return toks + [0] * (n - len(toks))

    def covers_pending(self, n: int) -> bool:
        """Whether the next n tokens reach into the tokens that the host does not know yet."""
        return self.num_computed + n > len(self.prompt_token_ids) + len(self.output_token_ids)


@dataclass
class CompletionOutput:
    index: int
    text: Optional[str]
    token_ids: List[int]
    finish_reason: Optional[str]


@dataclass
class RequestMetrics:
    """Times of a request on the engine's monotonic clock, as the reference keeps them
    (core/src/common/sequence.rs:13-33): arrival, first token, finish."""
    arrival_time: float
    first_token_time: Optional[float]
    finished_time: Optional[float]

    def summary(self, n_generated: int) -> dict:
        """Seconds to the first token, seconds per token after it, seconds to the end."""
        ttft = None if self.first_token_time is None else self.first_token_time - self.arrival_time
        end = None if self.finished_time is None else self.finished_time - self.arrival_time
        tpot = None
        if ttft is not None and end is not None and n_generated > 1:
            tpot = (end - ttft) / (n_generated - 1)
        return {"ttft_s": ttft, "tpot_s": tpot, "finished_s": end}


@dataclass
class RequestOutput:
    request_id: Hashable
    prompt_token_ids: List[int]
    outputs: List[CompletionOutput]
    finished: bool
    metrics: Optional[RequestMetrics] = None

    @staticmethod
    def from_sequence(seq: Sequence, text: Optional[str] = None) -> "RequestOutput":
        """A snapshot of the request.  The generated tokens are copied, since they grow; the prompt is the request's
        own list, which nothing changes after the request is added (copying it for every request at every step
        costs more host time than the rest of a step of a small model)."""
        reason = seq.status.value if seq.status.finished else None
        return RequestOutput(seq.request_id, seq.prompt_token_ids,
                             [CompletionOutput(0, text, list(seq.output_token_ids), reason)], seq.status.finished,
                             RequestMetrics(seq.arrival_time, seq.first_token_time, seq.finish_time))
