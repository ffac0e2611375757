from .cache import PAGE, Cache, CacheError, CacheFull, FreeList, KVView, StateView, pages_for

__all__ = ["PAGE", "Cache", "CacheError", "CacheFull", "FreeList", "KVView", "StateView", "pages_for"]
