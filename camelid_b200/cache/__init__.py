from .book import PAGE, CacheBook, FreeList, KVSpec, StateSpec

__all__ = ["PAGE", "CacheBook", "FreeList", "KVSpec", "StateSpec", "SequenceCache"]


def __getattr__(name):
    if name == "SequenceCache":            # needs torch; the bookkeeping above does not
        from .sequence_cache import SequenceCache
        return SequenceCache
    raise AttributeError(name)
