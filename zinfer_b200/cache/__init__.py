from .manager import (CacheError, CacheManager, CallCacheSpec, ContextFull, KVGroup, KVView, NoFreeSlot, OutOfPages)
