"""A pool of fixed-size cache pages.

Follows the reference's BlockAllocator (core/src/sched/block_manager.rs:14-58): a free list from
whose back pages are taken and to whose back they return, so a page that was just given back is
the next one used again; giving a page back twice is an error.  There is no sharing between
requests here, hence no reference counts.
"""
from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """The reference's "Out of memory! No free blocks" (core/src/sched/block_manager.rs:36-43)."""


class BlockAllocator:
    def __init__(self, num_blocks: int):
        if num_blocks <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_blocks = int(num_blocks)
        self._free: List[int] = list(range(self.num_blocks - 1, -1, -1))
        self._is_free = [True] * self.num_blocks

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free cache pages")
        b = self._free.pop()
        self._is_free[b] = False
        return b

    def free(self, block: int) -> None:
        if not (0 <= block < self.num_blocks):
            raise ValueError(f"page {block} is not of this pool (0..{self.num_blocks - 1})")
        if self._is_free[block]:
            raise ValueError(f"page {block} is given back twice")
        self._is_free[block] = True
        self._free.append(block)
