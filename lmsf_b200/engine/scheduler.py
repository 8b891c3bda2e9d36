"""The scheduler: admits requests, cuts prompts into portions under a token budget, keeps decoding,
and decides what happens when pages run out.  Host only.  The queues and the decisions live in the native
runtime (csrc/host_runtime.cpp, lmsf_sched_*), next to the cache manager they act on; the class below is their
face: it tells the native side what changed about the requests, asks for a step's decisions and hands them out
as Python objects.

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
from typing import Deque, Dict, Hashable, List, Optional

import numpy as np

from ..cache import native
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
        self._lib = native.lib()
        self._h = self._lib.lmsf_sched_create(cache.handle(), config.max_num_batched_tokens, config.max_num_seqs,
                                              config.max_model_len)
        if not self._h:
            raise ValueError("the scheduler needs a positive token budget and request limit")
        self._seqs: Dict[int, Sequence] = {}          # native id -> request
        self._nids: Dict[Hashable, int] = {}          # request id -> native id
        self.waiting: Deque[Sequence] = deque()       # mirrors of the native queues, in their order
        self.running: List[Sequence] = []
        self.watermark_pages = [self._lib.lmsf_sched_watermark(self._h, g) for g in range(len(cache.groups))]

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.lmsf_sched_destroy(self._h)
            self._h = None

    @property
    def num_preemptions(self) -> int:
        return int(self._lib.lmsf_sched_num_preemptions(self._h))

    # ------------------------------------------------------------------ queues
    def _refresh_queues(self) -> None:
        n = len(self._seqs)
        buf = np.empty(max(n, 1), dtype=np.int64)
        k = self._lib.lmsf_sched_queue(self._h, 0, buf.ctypes.data, n)
        self.waiting = deque(self._seqs[int(i)] for i in buf[:k])
        k = self._lib.lmsf_sched_queue(self._h, 1, buf.ctypes.data, n)
        self.running = [self._seqs[int(i)] for i in buf[:k]]

    def _forget(self, seq: Sequence) -> None:
        nid = self._nids.pop(seq.request_id)
        del self._seqs[nid]
        self.cache.unbind(seq.request_id)

    def add_seq(self, seq: Sequence) -> None:
        nid = self.cache.new_native_id()
        if self._lib.lmsf_sched_add(self._h, nid, float(seq.arrival_time), len(seq)) != 0:
            raise KeyError(f"request {seq.request_id!r} is already known to the scheduler")
        self._seqs[nid] = seq
        self._nids[seq.request_id] = nid
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)

    def abort_seq(self, request_id: Hashable) -> Optional[Sequence]:
        """core/src/sched/scheduler.rs:160-196: from whichever queue holds it; pages are given back."""
        nid = self._nids.get(request_id)
        if nid is None:
            return None
        seq = self._seqs[nid]
        self._lib.lmsf_sched_remove(self._h, nid)
        self._forget(seq)
        seq.status = SequenceStatus.FINISHED_ABORTED
        self._refresh_queues()
        return seq

    def has_unfinished_seqs(self) -> bool:
        return bool(self.waiting or self.running)

    def get_num_unfinished_seqs(self) -> int:
        return len(self.waiting) + len(self.running)

    def free_seq(self, seq: Sequence) -> None:
        """A finished request leaves its queue and gives back what it holds.  It is usually running; it waits when
        it was preempted while its last token was still on its way from the device and that token ended it."""
        nid = self._nids.get(seq.request_id)
        if nid is not None and self._seqs[nid] is seq:
            self._lib.lmsf_sched_remove(self._h, nid)
            self._forget(seq)
            self._refresh_queues()
        elif self.cache.has(seq.request_id):
            self.cache.free(seq.request_id)

    # ------------------------------------------------------------------ decisions
    def schedule(self) -> SchedulerOutputs:
        out = SchedulerOutputs()
        n = len(self._seqs)
        if n == 0:
            return out
        seqs = list(self._seqs.items())
        rids = np.fromiter((nid for nid, _ in seqs), dtype=np.int64, count=n)
        state = np.empty((4, n), dtype=np.int32)
        for i, (_, s) in enumerate(seqs):
            state[0, i], state[1, i], state[2, i], state[3, i] = len(s), s.num_computed, s.num_pending, s.hold
        ptr = lambda a: a.ctypes.data
        self._lib.lmsf_sched_update(self._h, n, ptr(rids), ptr(state[0]), ptr(state[1]), ptr(state[2]), ptr(state[3]))
        e_rid, pre, ign = (np.empty(n, dtype=np.int64) for _ in range(3))
        e_info = np.empty((3, n), dtype=np.int32)
        ign_kind = np.empty(n, dtype=np.int32)
        counts = np.zeros(3, dtype=np.int32)
        rc = self._lib.lmsf_sched_schedule(self._h, n, ptr(e_rid), ptr(e_info[0]), ptr(e_info[1]), ptr(e_info[2]),
                                           ptr(pre), ptr(ign), ptr(ign_kind), ptr(counts))
        if rc != 0:
            raise RuntimeError(f"the native scheduler failed ({rc})")
        ne, n_pre, n_ign = (int(c) for c in counts)
        for i in range(n_pre):
            seq = self._seqs[int(pre[i])]
            self.cache.unbind(seq.request_id)
            seq.num_computed = 0
            seq.num_preemptions += 1
            seq.status = SequenceStatus.WAITING
            out.preempted.append(seq)
        for i in range(n_ign):
            seq = self._seqs[int(ign[i])]
            seq.status = SequenceStatus.FINISHED_LENGTH if ign_kind[i] else SequenceStatus.FINISHED_IGNORED
            self._forget(seq)
            out.ignored.append(seq)
        for i in range(ne):
            nid = int(e_rid[i])
            seq = self._seqs[nid]
            self.cache.bind(seq.request_id, nid)          # the native side has registered it with the cache manager
            seq.status = SequenceStatus.RUNNING
            out.entries.append(ScheduledEntry(seq, int(e_info[0, i]), int(e_info[1, i]), bool(e_info[2, i])))
        self._refresh_queues()
        return out
