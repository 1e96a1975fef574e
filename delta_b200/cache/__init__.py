from .manager import CacheGroup, CacheManager, LayerCacheView
from .page_pool import OutOfPages, PagePool
