"""Per-sequence storage: slots, paged keys and values per layer group, fixed-size state."""
from .pool import IdPool  # noqa: F401
from .model_cache import CacheGroup, LayerCacheView, ModelCache, Sequence, PAGE  # noqa: F401
