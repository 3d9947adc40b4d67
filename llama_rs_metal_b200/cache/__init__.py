from .cache import PAGE_SIZE, Cache, KeyValueGroup, KeyValueView, StateGroup, StateView
from .slots import FreeList

__all__ = ["PAGE_SIZE", "Cache", "KeyValueGroup", "KeyValueView", "StateGroup", "StateView", "FreeList"]
