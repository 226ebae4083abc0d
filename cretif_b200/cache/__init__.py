"""The cache: slots per sequence, block-pooled keys/values per layer group, fixed-size state."""
from .blocks import BlockPool, CacheError, CacheFull, SlotSet
from .sequence_cache import KVRequest, KVView, SequenceCache, StateRequest

__all__ = ["BlockPool", "CacheError", "CacheFull", "SlotSet",
           "KVRequest", "KVView", "SequenceCache", "StateRequest"]
