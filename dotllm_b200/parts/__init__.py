"""Parts a layer is made of: mixers, feed-forwards, norms, position encodings, arrangements."""
from .base import (Arrangement, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding,  # noqa: F401
                   Runtime, WeightSpec, make_arrangement, make_part, register_arrangement,
                   register_embedding, register_feed_forward, register_head, register_mixer,
                   register_norm, register_position_encoding, registered)
