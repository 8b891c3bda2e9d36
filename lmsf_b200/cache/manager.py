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

The bookkeeping is native (csrc/host_runtime.cpp, as the reference's is Rust); this class is its face and
maps request ids of any hashable type to the integers that the library knows.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

from . import native


class OutOfPages(RuntimeError):
    """The reference's "Out of memory! No free blocks" (core/src/sched/block_manager.rs:36-43)."""


@dataclass(frozen=True)
class GroupSpec:
    """One group of layers with the same needs.  window None: all keys are kept."""
    window: Optional[int] = None


class _PoolView:
    """What tests and statistics read of one group's pool."""

    def __init__(self, mgr: "CacheManager", g: int):
        self._mgr, self._g = mgr, g

    @property
    def num_free(self) -> int:
        return self._mgr.num_free_pages(self._g)

    @property
    def num_blocks(self) -> int:
        return self._mgr.num_total_pages(self._g)


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], num_blocks: Sequence[int], block_size: int, num_state_slots: int):
        if len(groups) != len(num_blocks):
            raise ValueError("one page count per group")
        if block_size <= 0:
            raise ValueError("block_size must be positive")
        if any(int(n) <= 0 for n in num_blocks):
            raise ValueError("a page pool needs at least one page")
        self.groups = list(groups)
        self.block_size = int(block_size)
        self.num_state_slots = int(num_state_slots)
        self._lib = native.lib()
        G = len(self.groups)
        windows = (ctypes.c_int * max(G, 1))(*[g.window or 0 for g in self.groups])
        blocks = (ctypes.c_int * max(G, 1))(*[int(n) for n in num_blocks])
        self._h = self._lib.lmsf_cm_create(G, windows, blocks, self.block_size, self.num_state_slots)
        if not self._h:
            raise ValueError("the cache manager could not be created from these sizes")
        self.pools = [_PoolView(self, g) for g in range(G)]
        self._ids: Dict[Hashable, int] = {}
        self._next_id = 1
        self._scratch = (ctypes.c_int * max(G, 1))()

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.lmsf_cm_destroy(self._h)
            self._h = None

    def handle(self) -> int:
        """The native object, for the batch builder."""
        return self._h

    def native_id(self, rid) -> int:
        return self._ids[rid]

    # The native scheduler registers and frees requests in the native manager itself; it takes its ids from here
    # and tells this face afterwards which requests the manager now knows.
    def new_native_id(self) -> int:
        nid = self._next_id
        self._next_id += 1
        return nid

    def bind(self, rid, nid: int) -> None:
        self._ids[rid] = nid

    def unbind(self, rid) -> None:
        self._ids.pop(rid, None)

    def native_has(self, nid: int) -> bool:
        return bool(self._lib.lmsf_cm_has(self._h, nid))

    def _id(self, rid) -> int:
        try:
            return self._ids[rid]
        except KeyError:
            raise KeyError(f"request {rid!r} is not live") from None

    # ------------------------------------------------------------------ requests
    def has(self, rid) -> bool:
        return rid in self._ids

    def can_add(self) -> bool:
        return bool(self._lib.lmsf_cm_can_add(self._h))

    def add(self, rid) -> int:
        """Registers a request; returns its state slot."""
        if rid in self._ids:
            raise KeyError(f"request {rid!r} is already live")
        nid = self._next_id
        slot = self._lib.lmsf_cm_add(self._h, nid)
        if slot < 0:
            raise OutOfPages("no free state slot")
        self._next_id += 1
        self._ids[rid] = nid
        return slot

    def free(self, rid) -> None:
        """Gives back everything the request holds."""
        nid = self._id(rid)
        rc = self._lib.lmsf_cm_free(self._h, nid)
        del self._ids[rid]
        if rc != 0:
            raise ValueError(f"request {rid!r}: a page was given back twice")

    def take_fresh_slots(self) -> List[int]:
        buf = (ctypes.c_int * max(self.num_state_slots, 1))()
        n = self._lib.lmsf_cm_take_fresh_slots(self._h, buf, len(buf))
        return list(buf[:n])

    # ------------------------------------------------------------------ pages
    def pages_needed(self, rid, n: int) -> List[int]:
        """Per group, how many new pages `reserve(rid, n)` would claim."""
        self._lib.lmsf_cm_pages_needed(self._h, self._id(rid), int(n), self._scratch)
        return list(self._scratch[:len(self.groups)])

    def can_reserve(self, rid, n: int, headroom: int = 0) -> bool:
        return self._lib.lmsf_cm_can_reserve(self._h, self._id(rid), int(n), int(headroom)) == 1

    def reserve(self, rid, n: int) -> None:
        """Claims pages so that positions up to num_reserved + n have one.  All or nothing."""
        rc = self._lib.lmsf_cm_reserve(self._h, self._id(rid), int(n))
        if rc == -1:
            raise OutOfPages(f"request {rid!r}: not enough free pages for {n} more positions")
        if rc != 0:
            raise ValueError(f"reserve({rid!r}, {n}) was refused ({rc})")

    def commit(self, rid, n: int) -> None:
        """The keys of n more positions are in the cache.  Window groups give back the pages that no
        later query can reach."""
        rc = self._lib.lmsf_cm_commit(self._h, self._id(rid), int(n))
        if rc == -4:
            raise ValueError(f"request {rid!r}: commit of {n} tokens beyond the {self.num_reserved(rid)} reserved")
        if rc != 0:
            raise ValueError(f"commit({rid!r}, {n}) failed ({rc})")

    def rollback(self, rid) -> None:
        """Forgets a reservation that was not committed (a step that did not run)."""
        if self._lib.lmsf_cm_rollback(self._h, self._id(rid)) != 0:
            raise ValueError(f"rollback({rid!r}) failed")

    # ------------------------------------------------------------------ views
    def num_tokens(self, rid) -> int:
        return self._lib.lmsf_cm_query(self._h, self._id(rid), 0, 0)

    def num_reserved(self, rid) -> int:
        return self._lib.lmsf_cm_query(self._h, self._id(rid), 1, 0)

    def state_slot(self, rid) -> int:
        return self._lib.lmsf_cm_query(self._h, self._id(rid), 2, 0)

    def block_table(self, rid, group: int) -> List[int]:
        nid = self._id(rid)
        n = self._lib.lmsf_cm_query(self._h, nid, 3, int(group))
        buf = (ctypes.c_int * max(n, 1))()
        self._lib.lmsf_cm_table(self._h, nid, int(group), buf, n)
        return list(buf[:n])

    def num_free_pages(self, group: int = 0) -> int:
        return self._lib.lmsf_cm_num_free(self._h, int(group))

    def num_total_pages(self, group: int = 0) -> int:
        return self._lib.lmsf_cm_num_total(self._h, int(group))

    def live_requests(self) -> List[Hashable]:
        return list(self._ids)

    def check_invariants(self) -> None:
        """No page lost, held twice or both free and held (used by tests)."""
        rc = self._lib.lmsf_cm_check(self._h)
        if rc:
            what = {1: "a page is held twice", 2: "a page is twice in the free list", 3: "a page is both free and held",
                    4: "pages are lost", 5: "state slots are lost or held twice"}.get(rc, str(rc))
            raise AssertionError(what)
        if self._lib.lmsf_cm_num_live(self._h) != len(self._ids):
            raise AssertionError("the native manager and its face disagree on the live requests")
