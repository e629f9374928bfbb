from .manager import CacheManager, PageAllocator, PagedView, SlotAllocator, StateView
