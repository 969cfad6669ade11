from .manager import CachedTensor, CacheError, CacheManager, CacheNeed, OutOfPages, PageAllocator
