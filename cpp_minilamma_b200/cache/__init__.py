from .paged import PAGE, CacheError, CacheFull, CacheGroup, CacheView, PagePool, SequenceCache
