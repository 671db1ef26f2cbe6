from .manager import CacheManager, CacheError, CacheFull, FreeList, pages_for

__all__ = ["CacheManager", "CacheError", "CacheFull", "FreeList", "pages_for"]
