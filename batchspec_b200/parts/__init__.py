from .base import (BLOCKS, FEED_FORWARDS, INPUT_PARTS, LOGITS_PARTS, MIXERS, NORMS, POSITION_ENCODINGS, Block, CacheSpec,
                   FeedForward, InputPart, LogitsPart, Mixer, Norm, ParamSpec, Part, PartSpec, PositionEncoding, Runtime,
                   StateSpec, build_part, register_part)
from . import attention, block, mlp, norm, rope  # noqa: F401  (registers the built-in parts)

__all__ = ["BLOCKS", "FEED_FORWARDS", "INPUT_PARTS", "LOGITS_PARTS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block",
           "CacheSpec", "FeedForward", "InputPart", "LogitsPart", "Mixer", "Norm", "ParamSpec", "Part", "PartSpec", "PositionEncoding", "Runtime", "StateSpec",
           "build_part", "register_part"]
