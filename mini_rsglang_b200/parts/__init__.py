from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (registers the kinds)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, Embedding,
                   FeedForward, Head, KVNeed, Mixer, Norm, Part, PartSpec, PositionEncoding, Rotation, Runtime, StateNeed)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block",
           "Embedding", "FeedForward", "Head", "KVNeed", "Mixer", "Norm", "Part", "PartSpec", "PositionEncoding",
           "Rotation", "Runtime", "StateNeed"]
