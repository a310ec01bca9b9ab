from .attention import GroupedQueryAttention
from .base import (Block, CachedTensor, CacheNeed, FeedForward, Mixer, Norm, Part, PositionEncoding, Residual, StateNeed,
                   TensorSpec)
from .block import LayerScaleBlock, PreNormBlock, SandwichNormBlock
from .delta import ChannelGatedDelta
from .embedding import LoopInput, OutputHead, TokenEmbedding, TokenSideInput
from .feedforward import ClampedGLU, SwiGLU
from .latent import LatentAttention
from .linear_attention import GatedLinearAttention
from .moe import MixtureOfExperts
from .norm import RMSNorm
from .position import NoPosition, QueryTemperature, RotaryHalf

__all__ = ["Block", "CachedTensor", "CacheNeed", "ChannelGatedDelta", "ClampedGLU", "FeedForward",
           "GatedLinearAttention", "GroupedQueryAttention", "LatentAttention", "LayerScaleBlock", "LoopInput", "Mixer",
           "MixtureOfExperts", "NoPosition", "Norm", "OutputHead", "Part", "PositionEncoding",
           "PreNormBlock", "QueryTemperature", "RMSNorm", "Residual", "RotaryHalf", "SandwichNormBlock", "StateNeed",
           "SwiGLU", "TensorSpec", "TokenEmbedding", "TokenSideInput"]
