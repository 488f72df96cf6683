from .base import (Block, FeedForward, KVCacheView, KVPages, Mixer, Norm, ParamSpec, Part, PositionEncoding, Runtime,
                   StateCacheView, StateSlot, StepContext)
from .attention import GQAttention
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .linear import Linear
from .mlp import SwiGLUFeedForward
from .norm import RMSNorm
from .rope import RotaryEmbedding

__all__ = [
    "Block", "FeedForward", "KVCacheView", "KVPages", "Mixer", "Norm", "ParamSpec", "Part", "PositionEncoding",
    "Runtime", "StateCacheView", "StateSlot", "StepContext", "GQAttention", "PreNormBlock", "OutputHead",
    "TokenEmbedding", "Linear", "SwiGLUFeedForward", "RMSNorm", "RotaryEmbedding",
]
