from .allocator import CacheBook, CacheError, CacheFull, FreeList, GroupSpec
from .paged import PagedCache

__all__ = ["CacheBook", "CacheError", "CacheFull", "FreeList", "GroupSpec", "PagedCache"]
