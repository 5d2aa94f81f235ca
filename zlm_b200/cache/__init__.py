from .kv_cache import CacheGroup, KVCache, pages_for
from .pages import CacheBookkeepingError, CacheFull, FreeList

__all__ = ["CacheGroup", "KVCache", "pages_for", "CacheBookkeepingError", "CacheFull", "FreeList"]
