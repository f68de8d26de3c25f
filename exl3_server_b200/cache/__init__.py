"""Slots, paged keys and values, and per-sequence state."""
from .kv import PAGE_SIZE, KVGroup, KVLayerView, SequenceCache
from .pages import CacheError, CacheFull, PagePool, SlotTable
