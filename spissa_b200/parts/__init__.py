"""Parts a model is put together from; importing this package registers the built-in ones."""
from .base import (Block, FeedForward, KVCacheRequest, Mixer, Norm, Part, PositionEncoding, Runtime,
                   StateRequest, WeightSpec)
from .registry import build_part, known_parts, register_part, unregister_part
from . import norm, rope, attention, mlp, block, embedding  # noqa: F401  (registration)

__all__ = ["Block", "FeedForward", "KVCacheRequest", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime",
           "StateRequest", "WeightSpec", "build_part", "known_parts", "register_part", "unregister_part"]
