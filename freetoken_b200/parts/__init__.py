"""Parts a layer is put together from; importing this package registers the built-in kinds."""

from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, BuildEnv, Embedding,
                   FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Segment, StepState, Workspace)
from . import attention, block, embedding, mlp, moe, norm, rope, sparse_attention  # noqa: F401  (registration)

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Block", "BuildEnv",
           "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding", "Segment", "StepState",
           "Workspace"]
