from .registry import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, lookup, register_block,
                       register_feed_forward, register_mixer, register_norm, register_position)
from .runtime import Runtime, Workspace
from . import attention, block, feed_forward, norm, position  # registers the built-in parts

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "lookup", "register_block",
           "register_feed_forward", "register_mixer", "register_norm", "register_position",
           "Runtime", "Workspace"]
