from .block_allocator import BlockAllocator, OutOfPages
from .manager import CacheManager, GroupSpec
