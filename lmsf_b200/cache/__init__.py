from .manager import CacheManager, GroupSpec, OutOfPages
