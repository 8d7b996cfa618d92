from .block_pool import BlockPool, NoFreePages, chain_hash
from .manager import CacheManager, RequestCache, NoFreeSlot
from .device import DeviceCache, CacheView

__all__ = ["BlockPool", "NoFreePages", "chain_hash", "CacheManager", "RequestCache", "NoFreeSlot",
           "DeviceCache", "CacheView"]
