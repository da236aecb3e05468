from .errors import CacheCapacityError, CacheError, CacheOwnershipError
from .manager import CacheManager, CacheStats, RequestCache
from .pools import IndexPool

__all__ = ["CacheCapacityError", "CacheError", "CacheOwnershipError", "CacheManager",
           "CacheStats", "RequestCache", "IndexPool"]
