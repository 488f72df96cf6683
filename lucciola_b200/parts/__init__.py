from .base import (BatchShape, Block, FeedForward, KVCacheView, KVPages, Mixer, Norm, NormSink, ParamSpec, Part, PlanView,
                   PositionEncoding, RowScaled, Runtime, StateCacheView, StateSlot, StepContext, StepPlan)
from .attention import GQAttention
from .block import PreNormBlock
from .embedding import OutputHead, TokenEmbedding
from .linear import Linear
from .mlp import SwiGLUFeedForward
from .norm import RMSNorm
from .rope import RotaryEmbedding

__all__ = [
    "BatchShape", "Block", "FeedForward", "KVCacheView", "KVPages", "Mixer", "Norm", "NormSink", "ParamSpec", "Part", "PlanView",
    "PositionEncoding", "RowScaled", "Runtime", "StateCacheView", "StateSlot", "StepContext", "StepPlan", "GQAttention", "PreNormBlock", "OutputHead",
    "TokenEmbedding", "Linear", "SwiGLUFeedForward", "RMSNorm", "RotaryEmbedding",
]
