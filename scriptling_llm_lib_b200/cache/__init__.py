from .needs import CACHE_KINDS, PAGE, CacheNeed, StateNeed, register_cache_kind
from .pool import CacheFull, FreeList
from .store import KVGroup, SequenceCache, pages_for

__all__ = ["PAGE", "CACHE_KINDS", "CacheNeed", "StateNeed", "CacheFull", "FreeList", "KVGroup", "SequenceCache", "pages_for",
           "register_cache_kind"]
