from .manager import CacheError, CacheManager, OutOfPages, PagedGroup, PagePool, StateGroup
