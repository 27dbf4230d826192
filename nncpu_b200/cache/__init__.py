"""Cache: sequence slots, paged keys and values per layer group, per-sequence state."""
from .slots import IndexPool
from .cache import PAGE, Cache, KVGroup, KVRequest, StateRequest, pages_for

__all__ = ["IndexPool", "PAGE", "Cache", "KVGroup", "KVRequest", "StateRequest", "pages_for"]
