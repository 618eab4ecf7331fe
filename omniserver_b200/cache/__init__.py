from .manager import CacheManager, PageGroup, RequestCache
from .page_pool import OutOfPages, PagePool
from .state_slots import OutOfSlots, StateSlots
