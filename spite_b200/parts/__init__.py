from .base import (Block, BuildContext, FeedForward, Mixer, Norm, ParamSpec, Part, PositionEncoding, QkNorm,
                   Rotation, build_part, register_block, register_feed_forward, register_mixer, register_norm,
                   register_position, registered)
from . import norm, position, attention, feedforward, block  # noqa: F401  (register the built-in parts)

__all__ = ["Block", "BuildContext", "FeedForward", "Mixer", "Norm", "ParamSpec", "Part",
           "PositionEncoding", "QkNorm", "Rotation", "build_part", "register_block", "register_feed_forward",
           "register_mixer", "register_norm", "register_position", "registered"]
