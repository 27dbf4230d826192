"""Parts: norms, position encodings, mixers, feed-forwards and blocks."""
from .base import (Block, DeferredNorm, EntryCache, FeedForward, Mixer, Norm, NormRequest, Part, PositionEncoding, build, register_block,
                   register_feed_forward, register_mixer, register_norm, register_position)
from .runtime import Runtime
from . import attention, block, mlp, norm, rope  # registers the built-in parts

__all__ = ["Block", "DeferredNorm", "EntryCache", "NormRequest", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "build",
           "register_block", "register_feed_forward", "register_mixer", "register_norm", "register_position",
           "Runtime"]
