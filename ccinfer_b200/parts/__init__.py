from .attention import GroupedQueryAttention
from .base import (Block, CachedTensor, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, Residual, StateNeed,
                   TensorSpec)
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .feedforward import SwiGLU
from .norm import RMSNorm
from .position import NoPosition, RotaryHalf

__all__ = ["Block", "CachedTensor", "CacheNeed", "FeedForward", "GroupedQueryAttention", "Mixer", "NoPosition", "Norm",
           "OutputHead", "Part", "PositionEncoding", "PreNormBlock", "RMSNorm", "Residual", "RotaryHalf",
           "StateNeed", "SwiGLU", "TensorSpec", "TokenEmbedding"]
