from .manager import CacheError, CacheManager, CacheNeed, OutOfPages, PageAllocator
