"""The cache manager: page pools, block tables, layer groups and state slots."""
from .pages import PageBookkeepingError, PagePool, PoolExhausted, StateSlotPool
from .manager import RELEASED, CacheManager, CacheNeed, FixedState, PagedKeysValues
from .budget import DEFAULT_SHARE, PagePlan, plan_pages
