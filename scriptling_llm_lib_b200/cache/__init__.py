from .needs import PAGE, CacheNeed, StateNeed
from .pool import CacheFull, FreeList
from .store import KVGroup, SequenceCache, pages_for

__all__ = ["PAGE", "CacheNeed", "StateNeed", "CacheFull", "FreeList", "KVGroup", "SequenceCache", "pages_for"]
