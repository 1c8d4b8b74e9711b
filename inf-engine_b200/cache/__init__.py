from .manager import CacheBinding, CacheManager, CacheRequirement, KVGroup, StateGroup
from .pages import PageAccountingError, PagePool
