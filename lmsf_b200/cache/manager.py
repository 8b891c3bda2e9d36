"""Host side of the cache: which pages hold which positions of which request.

Role of the reference's BlockSpaceManager (core/src/sched/block_manager.rs:69-347): one block
table per request, pages claimed as the request grows and given back when it ends.  Differences:

* pages are claimed per portion of tokens (`reserve`), not for a whole prompt at admission, so
  prompts can be cut anywhere;
* layers are put into groups by what they need of the cache (key/value shape; all keys or a
  window of them); each group has a pool and block tables of its own;
* for a window group the pages that every future query has passed are given back at `commit`
  and their table entries become -1 (the reference instead reuses table entries as a ring,
  block_manager.rs:129-135, :165-175);
* beside the pages each request holds one slot for state of fixed size, claimed at `add` and
  released at `free`; slots claimed since the last call of `take_fresh_slots` must be zeroed by
  the caller before they are used.

A table entry i covers positions [i * block_size, (i + 1) * block_size).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

from .block_allocator import BlockAllocator, OutOfPages


@dataclass(frozen=True)
class GroupSpec:
    """One group of layers with the same needs.  window None: all keys are kept."""
    window: Optional[int] = None


@dataclass
class _Request:
    tables: List[List[int]]
    num_tokens: int = 0          # positions committed (their keys are in the cache)
    num_reserved: int = 0        # positions that have pages (>= num_tokens)
    slot: int = -1


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], num_blocks: Sequence[int], block_size: int, num_state_slots: int):
        if len(groups) != len(num_blocks):
            raise ValueError("one page count per group")
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        self.groups = list(groups)
        self.block_size = int(block_size)
        self.pools = [BlockAllocator(n) for n in num_blocks]
        self.num_state_slots = int(num_state_slots)
        self._free_slots = list(range(self.num_state_slots - 1, -1, -1))
        self._fresh_slots: List[int] = []
        self._reqs: Dict[Hashable, _Request] = {}

    # ------------------------------------------------------------------ requests
    def has(self, rid) -> bool:
        return rid in self._reqs

    def can_add(self) -> bool:
        return bool(self._free_slots)

    def add(self, rid) -> int:
        """Registers a request; returns its state slot."""
        if rid in self._reqs:
            raise KeyError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise OutOfPages("no free state slot")
        slot = self._free_slots.pop()
        self._fresh_slots.append(slot)
        self._reqs[rid] = _Request(tables=[[] for _ in self.groups], slot=slot)
        return slot

    def free(self, rid) -> None:
        """Gives back everything the request holds."""
        r = self._reqs.pop(rid)
        for g, table in enumerate(r.tables):
            for b in reversed(table):
                if b >= 0:
                    self.pools[g].free(b)
        if r.slot in self._fresh_slots:
            self._fresh_slots.remove(r.slot)
        self._free_slots.append(r.slot)

    def take_fresh_slots(self) -> List[int]:
        out, self._fresh_slots = self._fresh_slots, []
        return out

    # ------------------------------------------------------------------ pages
    def _first_needed_entry(self, g: int, start: int) -> int:
        """First table entry that a query at position >= start may still read."""
        w = self.groups[g].window
        if w is None:
            return 0
        return max(0, start - w + 1) // self.block_size

    def pages_needed(self, rid, n: int) -> List[int]:
        """Per group, how many new pages `reserve(rid, n)` would claim."""
        r = self._reqs[rid]
        end = r.num_reserved + n
        entries = (end + self.block_size - 1) // self.block_size
        return [max(0, entries - len(t)) for t in r.tables]

    def can_reserve(self, rid, n: int, headroom: int = 0) -> bool:
        return all(p.num_free - need >= headroom for p, need in zip(self.pools, self.pages_needed(rid, n)))

    def reserve(self, rid, n: int) -> None:
        """Claims pages so that positions up to num_reserved + n have one.  All or nothing."""
        need = self.pages_needed(rid, n)
        for g, k in enumerate(need):
            if self.pools[g].num_free < k:
                raise OutOfPages(f"group {g}: {k} pages needed, {self.pools[g].num_free} free")
        r = self._reqs[rid]
        for g, k in enumerate(need):
            for _ in range(k):
                r.tables[g].append(self.pools[g].allocate())
        r.num_reserved += n

    def commit(self, rid, n: int) -> None:
        """The keys of n more positions are in the cache.  Window groups give back the pages that no
        later query can reach."""
        r = self._reqs[rid]
        if r.num_tokens + n > r.num_reserved:
            raise ValueError(f"request {rid!r}: commit of {n} tokens beyond the {r.num_reserved} reserved")
        r.num_tokens += n
        for g, table in enumerate(r.tables):
            if self.groups[g].window is None:
                continue
            first = self._first_needed_entry(g, r.num_tokens)
            for i in range(min(first, len(table))):
                if table[i] >= 0:
                    self.pools[g].free(table[i])
                    table[i] = -1

    def rollback(self, rid) -> None:
        """Forgets a reservation that was not committed (a step that did not run)."""
        r = self._reqs[rid]
        entries = (r.num_tokens + self.block_size - 1) // self.block_size
        for g, table in enumerate(r.tables):
            while len(table) > entries:
                b = table.pop()
                if b >= 0:
                    self.pools[g].free(b)
        r.num_reserved = r.num_tokens

    # ------------------------------------------------------------------ views
    def num_tokens(self, rid) -> int:
        return self._reqs[rid].num_tokens

    def num_reserved(self, rid) -> int:
        return self._reqs[rid].num_reserved

    def state_slot(self, rid) -> int:
        return self._reqs[rid].slot

    def block_table(self, rid, group: int) -> List[int]:
        return self._reqs[rid].tables[group]

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def num_total_pages(self, group: int = 0) -> int:
        return self.pools[group].num_blocks

    def live_requests(self) -> List[Hashable]:
        return list(self._reqs)

    def check_invariants(self) -> None:
        """No page lost, held twice or both free and held (used by tests)."""
        for g, pool in enumerate(self.pools):
            held = [b for r in self._reqs.values() for b in r.tables[g] if b >= 0]
            if len(held) != len(set(held)):
                raise AssertionError(f"group {g}: a page is held twice")
            free = set(pool._free)
            if len(free) != len(pool._free):
                raise AssertionError(f"group {g}: a page is twice in the free list")
            if free & set(held):
                raise AssertionError(f"group {g}: a page is both free and held")
            if len(free) + len(held) != pool.num_blocks:
                raise AssertionError(f"group {g}: {pool.num_blocks - len(free) - len(held)} pages are lost")
        slots = [r.slot for r in self._reqs.values()]
        if len(slots) != len(set(slots)) or set(slots) & set(self._free_slots) or \
                len(slots) + len(self._free_slots) != self.num_state_slots:
            raise AssertionError("state slots are lost or held twice")
