from .groups import NO_PAGE, CacheGroup
from .manager import CacheManager
from .page_pool import PagePool
from .state_slots import StateSlotPool

__all__ = ["NO_PAGE", "CacheGroup", "CacheManager", "PagePool", "StateSlotPool"]
