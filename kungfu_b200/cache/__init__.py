from .manager import CacheError, CacheManager, FixedStateView, OutOfPages, PagedKVView, PagePool
