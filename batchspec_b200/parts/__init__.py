from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheSpec, FeedForward, Mixer,
                   Norm, ParamSpec, Part, PartSpec, PositionEncoding, Runtime, StateSpec, build_part, register_part)
from . import attention, block, mlp, norm, rope  # noqa: F401  (registers the built-in parts)

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "CacheSpec", "FeedForward",
           "Mixer", "Norm", "ParamSpec", "Part", "PartSpec", "PositionEncoding", "Runtime", "StateSpec",
           "build_part", "register_part"]
