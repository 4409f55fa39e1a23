from .paged import CACHE_KINDS, Cache, CacheStorage, CacheView, LatentView
from .slots import PAGE, CacheError, FreeList, SequenceTable
