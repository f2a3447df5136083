"""Paged key/value cache and per-request state slots."""
from .manager import RELEASED, CacheManager, KvHandle, KvNeed, StateNeed
from .pool import DoubleFree, IdPool, OutOfPages

__all__ = ["RELEASED", "CacheManager", "KvHandle", "KvNeed", "StateNeed", "DoubleFree", "IdPool", "OutOfPages"]
