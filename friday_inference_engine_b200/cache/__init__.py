from .cache import Cache  # noqa: F401
from .kv import PAGE, KVGroup, KVView, StateView  # noqa: F401
from .slots import CacheError, CacheFull, FreeList  # noqa: F401
