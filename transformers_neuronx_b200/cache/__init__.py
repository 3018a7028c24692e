from .allocator import OutOfPages, PagePool, SlotTable
from .manager import CacheManager, FixedStateNeed, GroupInfo, PagedKVNeed, group_needs
from .storage import CacheStorage
