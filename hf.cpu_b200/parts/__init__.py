from .base import (Block, CacheSpec, FeedForward, Mixer, Norm, Part, PositionEncoding, StateSpec,
                   make_part, register_part, unregister_part)
from . import attention, block, embedding, ffn, norm, rotary  # noqa: F401  (register the built-in parts)

__all__ = ["Part", "Norm", "PositionEncoding", "Mixer", "FeedForward", "Block", "CacheSpec", "StateSpec",
           "make_part", "register_part", "unregister_part"]
