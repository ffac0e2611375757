from .cache import PAGE, Cache, CacheError, CacheFull, CacheMark, FreeList, KVView, StateView, pages_for

__all__ = ["PAGE", "Cache", "CacheError", "CacheFull", "CacheMark", "FreeList", "KVView", "StateView", "pages_for"]
