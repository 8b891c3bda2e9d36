"""The scheduler: admits requests, cuts prompts into portions under a token budget, keeps decoding,
and decides what happens when pages run out.  Host only.

The reference (core/src/sched/scheduler.rs:336-543) runs either a batch of whole prompts or a batch
of decodes, keeps a third queue for swapped groups and preempts by swap or recompute
(scheduler.rs:236-284).  Here:

* every step mixes what is due: each running request first gets its next tokens (one token for a
  request that decodes, the next portion for one whose prompt is not through), oldest first; what
  is left of `max_num_batched_tokens` goes to requests admitted from the waiting queue, first come
  first served (core/src/sched/policy.rs:20-28);
* a prompt longer than the budget left is cut; only the portion that ends the known tokens asks
  for logits;
* when a running request cannot get a page, the youngest running request is preempted
  (scheduler.rs:466-483): its pages are given back, it returns to the FRONT of the waiting queue
  and is later recomputed from its prompt plus what it has generated (scheduler.rs:274-284).
  Its sampling state is its token list and seed, so the continuation is the same;
* a request that cannot fit the cache even alone finishes: "ignored" if its prompt never fits,
  "length" if it grew to the cache's size while decoding;
* admission keeps a watermark of 1 % of the pages free (core/src/sched/block_manager.rs:88, :104-122).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Hashable, List, Optional

from ..cache.manager import CacheManager
from ..config.engine_config import SchedulerConfig
from .sequence import Sequence, SequenceStatus


@dataclass
class ScheduledEntry:
    seq: Sequence
    start: int            # position of the first token of the portion
    num_tokens: int
    wants_logits: bool    # the portion ends the tokens known so far: its last place is sampled


@dataclass
class SchedulerOutputs:
    entries: List[ScheduledEntry] = field(default_factory=list)
    preempted: List[Sequence] = field(default_factory=list)
    ignored: List[Sequence] = field(default_factory=list)      # finished without ever running

    @property
    def num_batched_tokens(self) -> int:
        return sum(e.num_tokens for e in self.entries)

    @property
    def is_empty(self) -> bool:
        return not self.entries


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager):
        self.config = config
        self.cache = cache
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.watermark_pages = [int(round(0.01 * cache.num_total_pages(g))) for g in range(len(cache.groups))]
        self.num_preemptions = 0

    # ------------------------------------------------------------------ queues
    def add_seq(self, seq: Sequence) -> None:
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)

    def abort_seq(self, request_id: Hashable) -> Optional[Sequence]:
        """core/src/sched/scheduler.rs:160-196: from whichever queue holds it; pages are given back."""
        for q in (self.waiting, self.running):
            for seq in q:
                if seq.request_id == request_id:
                    q.remove(seq)
                    self._release(seq)
                    seq.status = SequenceStatus.FINISHED_ABORTED
                    return seq
        return None

    def has_unfinished_seqs(self) -> bool:
        return bool(self.waiting or self.running)

    def get_num_unfinished_seqs(self) -> int:
        return len(self.waiting) + len(self.running)

    def free_seq(self, seq: Sequence) -> None:
        """A finished request leaves its queue and gives back what it holds.  It is usually running; it waits when
        it was preempted while its last token was still on its way from the device and that token ended it."""
        for q in (self.running, self.waiting):
            for i, other in enumerate(q):
                if other is seq:
                    del q[i]
                    break
        self._release(seq)

    def _release(self, seq: Sequence) -> None:
        if self.cache.has(seq.request_id):
            self.cache.free(seq.request_id)

    # ------------------------------------------------------------------ decisions
    def _fits_alone(self, num_tokens: int) -> bool:
        bs = self.cache.block_size
        for g, spec in enumerate(self.cache.groups):
            toks = num_tokens if spec.window is None else min(num_tokens, spec.window + 2 * bs)
            if (toks + bs - 1) // bs > self.cache.num_total_pages(g):
                return False
        return True

    def _portion_that_fits(self, seq: Sequence, n: int) -> int:
        """A portion's pages are all held until its step is over, also those that a window will give back right
        after it: a portion of n tokens that needs more pages than a windowed group has can never run, however many
        other requests are preempted.  Such a portion is halved until the pages it adds, beside those the request
        holds, fit the group; the rest of the prompt follows in the next steps, when the window has moved on."""
        if all(spec.window is None for spec in self.cache.groups):
            return n
        rid = seq.request_id
        windowed = [g for g, spec in enumerate(self.cache.groups) if spec.window is not None]
        need = self.cache.pages_needed(rid, n)
        if all(need[g] <= self.cache.num_free_pages(g) for g in windowed):
            return n                        # the usual case: the pages are there right now
        held = {g: sum(1 for p in self.cache.block_table(rid, g) if p >= 0) for g in windowed}
        while n > 1 and not all(need[g] + held[g] <= self.cache.num_total_pages(g) for g in windowed):
            n = max(1, n // 2)
            need = self.cache.pages_needed(rid, n)
        return n

    def _preempt(self, seq: Sequence, out: SchedulerOutputs) -> None:
        self.running.remove(seq)
        self._release(seq)
        seq.num_computed = 0
        seq.num_preemptions += 1
        seq.status = SequenceStatus.WAITING
        self.waiting.appendleft(seq)
        out.preempted.append(seq)
        self.num_preemptions += 1

    def schedule(self) -> SchedulerOutputs:
        out = SchedulerOutputs()
        budget = self.config.max_num_batched_tokens
        self.running.sort(key=lambda s: s.arrival_time)     # age order (core/src/sched/policy.rs:20-28)

        # 1. running requests, oldest first
        i = 0
        while i < len(self.running) and budget > 0:
            seq = self.running[i]
            if seq.hold or seq.num_uncomputed <= 0:      # waits for a token that is still on the device
                i += 1
                continue
            n = self._portion_that_fits(seq, min(seq.num_uncomputed, budget))
            if seq.num_pending > 1 or (seq.num_pending and n < seq.num_uncomputed):
                # only the newest pending token can be taken from the device, and only as a portion's last token
                i += 1
                continue
            lack = seq.num_computed + n - self.cache.num_reserved(seq.request_id)
            preempted_self = False
            while lack > 0 and not self.cache.can_reserve(seq.request_id, lack):
                victim = self.running[-1]
                if victim is seq and len(self.running) == 1 and not self._fits_alone(seq.num_computed + n):
                    # alone and still too large for the cache: it ends here
                    self.running.remove(seq)
                    self._release(seq)
                    seq.status = SequenceStatus.FINISHED_LENGTH
                    out.ignored.append(seq)
                    preempted_self = True
                    break
                self._preempt(victim, out)
                if victim is seq:
                    preempted_self = True
                    break
            if preempted_self:
                continue
            if lack > 0:
                self.cache.reserve(seq.request_id, lack)
            out.entries.append(ScheduledEntry(seq, seq.num_computed, n, n == seq.num_uncomputed))
            budget -= n
            i += 1

        # 2. admissions, first come first served; nothing is admitted in a step that preempted
        while self.waiting and budget > 0 and not out.preempted:
            seq = self.waiting[0]
            if seq.num_pending:          # preempted with a token still on the device: next step
                break
            if len(seq) > self.config.max_model_len or not self._fits_alone(len(seq)):
                self.waiting.popleft()
                seq.status = SequenceStatus.FINISHED_IGNORED
                out.ignored.append(seq)
                continue
            if len(self.running) >= self.config.max_num_seqs or not self.cache.can_add():
                break
            self.cache.add(seq.request_id)
            n = self._portion_that_fits(seq, min(seq.num_uncomputed, budget))
            need = self.cache.pages_needed(seq.request_id, n)
            idle = not self.running          # an empty engine admits its first request without a watermark
            if any(self.cache.num_free_pages(g) - k < (0 if idle else self.watermark_pages[g])
                   for g, k in enumerate(need)):
                self.cache.free(seq.request_id)
                break
            self.cache.reserve(seq.request_id, n)
            self.waiting.popleft()
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            out.entries.append(ScheduledEntry(seq, seq.num_computed, n, n == seq.num_uncomputed))
            budget -= n
        return out
