"""Parts of a layer: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheSpec, FeedForward, Mixer, Norm,
                   Part, PartSpec, PositionEncoding, Registry, StateSpec, TensorSpec)
from . import attention, block, feed_forward, norm, rope  # noqa: F401  (registers the parts)
