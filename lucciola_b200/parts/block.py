"""Pre-norm residual block: r += mixer(norm1(r)); r += ffn(norm2(r)) (src/qwen.cc:574-798 of lucciola).

The residual stream is float32.  A block hands the output of its feed-forward on as `delta`
instead of adding it: the next block's first norm adds it in the same pass (one kernel
instead of the add, copy and norm that lucciola launches at src/qwen.cc:742-759)."""
from __future__ import annotations

from typing import Optional

import torch

from .base import Block, FeedForward, Mixer, Norm, Part, StepContext


class PreNormBlock(Block):
    recordable = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, ffn_norm: Norm, act_dtype: torch.dtype):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.act_dtype = act_dtype

    def children(self) -> list[Part]:
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward]

    def forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], step: StepContext, cache,
                write_cache: bool = True) -> tuple[torch.Tensor, Optional[torch.Tensor]]:
        h = self.mixer_norm.add_forward(residual, delta, self.act_dtype)
        a = self.mixer.forward(h, step, cache, write_cache)
        h = self.ffn_norm.add_forward(residual, a, self.act_dtype)
        return residual, self.feed_forward.forward(h, step)
