"""Parts a layer is put together from; importing this package registers the built-in kinds."""

from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Block, BuildEnv, FeedForward,
                   Mixer, Norm, Part, PositionEncoding, Segment, StepState, Workspace)
from . import attention, block, mlp, moe, norm, rope, sparse_attention  # noqa: F401  (registration)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Block", "BuildEnv",
           "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "Segment", "StepState",
           "Workspace"]
