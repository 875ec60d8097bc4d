from .pages import PAGE, CacheError, CacheFull, FreeList, PageMap, pages_for
