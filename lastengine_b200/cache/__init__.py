from .allocator import CacheError, CacheFull, IdPool  # noqa: F401
from .cache import PAGE_SIZE, Cache, CacheView  # noqa: F401
