from . import attention, block, embedding, feedforward, norm, rotary  # noqa: F401  (registers the built-in parts)
from .base import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Embedding, FeedForward,
                   Head, Mixer, Norm, Part, PartSpec, PositionEncoding)
from .block import Block, LayerSpec, build_block, pre_norm_layer
from .embedding import OutputHead, TokenEmbedding, linear_head, token_embedding
from .linear import Linear

__all__ = ["ARRANGEMENTS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Embedding",
           "FeedForward", "Head", "Mixer", "Norm", "Part", "PartSpec", "PositionEncoding", "Block", "LayerSpec", "build_block",
           "pre_norm_layer", "OutputHead", "TokenEmbedding", "linear_head", "token_embedding", "Linear"]
