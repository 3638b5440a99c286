"""Slots, paged keys and values, and fixed-size per-sequence state."""
from .slots import CacheFull, CacheMisuse, IndexPool
from .views import KVLayerView, StateLayerView
from .manager import CacheManager, KVGroup, StateGroup, SequenceState

__all__ = ["CacheFull", "CacheMisuse", "IndexPool", "KVLayerView", "StateLayerView", "CacheManager",
           "KVGroup", "StateGroup", "SequenceState"]
