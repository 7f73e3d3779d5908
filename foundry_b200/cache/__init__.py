"""The cache: slots and pages on the host, grouped storage on the device."""
from .pages import PAGE, CacheError, CacheFull, CacheMisuse, FreeList, GroupPages, SlotTable, pages_for
from .store import (JointRequest, JointView, KVGroup, KVRequest, KVView, SequenceCache,
                    StateRequest, StateView)

__all__ = ["PAGE", "CacheError", "CacheFull", "CacheMisuse", "FreeList", "GroupPages", "SlotTable",
           "pages_for", "JointRequest", "JointView", "KVGroup", "KVRequest", "KVView", "SequenceCache", "StateRequest",
           "StateView"]
