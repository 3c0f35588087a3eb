from . import attention, block, feedforward, norm, rotary  # noqa: F401  (registers the built-in parts)
from .base import (ARRANGEMENTS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, FeedForward, Mixer, Norm, Part,
                   PartSpec, PositionEncoding)
from .block import LayerSpec, build_block
from .embedding import OutputHead, TokenEmbedding
from .linear import Linear

__all__ = ["ARRANGEMENTS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "FeedForward", "Mixer", "Norm",
           "Part", "PartSpec", "PositionEncoding", "LayerSpec", "build_block", "OutputHead", "TokenEmbedding", "Linear"]
