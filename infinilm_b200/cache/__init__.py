from .manager import (CacheGroup, CacheManager, CacheStateError, OutOfPages, PagedKVView, PagePool, SequenceCache,
                      StateSlots, StateView)
