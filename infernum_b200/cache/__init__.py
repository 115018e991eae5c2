from .manager import CacheGroup, CacheManager, LayerCache, RequestCache
from .pages import PagePool
