from .manager import CacheGroup, CacheManager

__all__ = ["CacheGroup", "CacheManager"]
