from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (registers the kinds)
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, FeedForward, KVNeed, Mixer,
                   Norm, Part, PartSpec, PositionEncoding, Runtime, StateNeed)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "FeedForward", "KVNeed",
           "Mixer", "Norm", "Part", "PartSpec", "PositionEncoding", "Runtime", "StateNeed"]
