from .base import Block, CacheNeed, FeedForward, Mixer, Norm, ParamDecl, Part, PositionEncoding, StateNeed
from .registry import (
    BLOCKS,
    FEED_FORWARDS,
    MIXERS,
    NORMS,
    POSITION_ENCODINGS,
    build_block,
    build_feed_forward,
    build_mixer,
    build_norm,
    build_position_encoding,
    register_block,
    register_feed_forward,
    register_mixer,
    register_norm,
    register_position_encoding,
)
from . import norm, position, attention, mlp, block  # noqa: F401  (register the built-in kinds)
from .model import DecoderModel

__all__ = [
    "BLOCKS", "Block", "CacheNeed", "DecoderModel", "FEED_FORWARDS", "FeedForward", "MIXERS", "Mixer",
    "NORMS", "Norm", "POSITION_ENCODINGS", "ParamDecl", "Part", "PositionEncoding", "StateNeed",
    "build_block", "build_feed_forward", "build_mixer", "build_norm", "build_position_encoding",
    "register_block", "register_feed_forward", "register_mixer", "register_norm",
    "register_position_encoding",
]
