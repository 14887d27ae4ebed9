from .allocators import CacheFull, CacheStateError, IdAllocator
from .book import CacheBook, GroupBook
from .sequence_cache import PAGE_SIZE, CacheNeed, KVSpec, SequenceCache, StateSpec

__all__ = ["CacheFull", "CacheStateError", "IdAllocator", "CacheBook", "GroupBook", "PAGE_SIZE", "CacheNeed",
           "KVSpec", "SequenceCache", "StateSpec"]
