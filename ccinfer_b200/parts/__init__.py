from .attention import GroupedQueryAttention
from .base import (Block, CachedTensor, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, Residual, StateNeed,
                   TensorSpec)
from .block import PreNormBlock, SandwichNormBlock
from .delta import ChannelGatedDelta
from .embedding import OutputHead, TokenEmbedding
from .feedforward import ClampedGLU, SwiGLU
from .norm import RMSNorm
from .position import NoPosition, QueryTemperature, RotaryHalf

__all__ = ["Block", "CachedTensor", "CacheNeed", "ChannelGatedDelta", "ClampedGLU", "FeedForward",
           "GroupedQueryAttention", "Mixer", "NoPosition", "Norm", "OutputHead", "Part", "PositionEncoding",
           "PreNormBlock", "QueryTemperature", "RMSNorm", "Residual", "RotaryHalf", "SandwichNormBlock", "StateNeed",
           "SwiGLU", "TensorSpec", "TokenEmbedding"]
