"""Cache manager: page pools per layer group, block tables per request, state slots."""
from .kv_manager import CacheGroupSpec, KVManager, KVManagerError, group_entries
from .page_pool import NULL_PAGE, PagePool, PagePoolError
from .state_slots import StateSlotError, StateSlotPool

__all__ = [
    "CacheGroupSpec",
    "KVManager",
    "KVManagerError",
    "NULL_PAGE",
    "PagePool",
    "PagePoolError",
    "StateSlotError",
    "StateSlotPool",
    "group_entries",
]
