"""A pool of fixed-size cache pages.

Follows the reference's BlockAllocator (core/src/sched/block_manager.rs:14-58): a free list from
whose back pages are taken and to whose back they return, so a page that was just given back is
the next one used again; giving a page back twice is an error.  There is no sharing between
requests here, hence no reference counts.  The pool itself is native (csrc/host_runtime.cpp).
"""
from __future__ import annotations

from . import native


class OutOfPages(RuntimeError):
    """The reference's "Out of memory! No free blocks" (core/src/sched/block_manager.rs:36-43)."""


class BlockAllocator:
    def __init__(self, num_blocks: int):
        if num_blocks <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_blocks = int(num_blocks)
        self._lib = native.lib()
        self._h = self._lib.lmsf_pool_create(self.num_blocks)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.lmsf_pool_destroy(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return self._lib.lmsf_pool_num_free(self._h)

    def allocate(self) -> int:
        b = self._lib.lmsf_pool_allocate(self._h)
        if b < 0:
            raise OutOfPages("no free cache pages")
        return b

    def free(self, block: int) -> None:
        if not (0 <= block < self.num_blocks):
            raise ValueError(f"page {block} is not of this pool (0..{self.num_blocks - 1})")
        if self._lib.lmsf_pool_free(self._h, int(block)) != 0:
            raise ValueError(f"page {block} is given back twice")
