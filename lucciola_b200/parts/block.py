"""Pre-norm residual block: r += mixer(norm1(r)); r += ffn(norm2(r)) (src/qwen.cc:574-798 of lucciola).

The residual stream is float32.  A block hands the output of its feed-forward on as `delta`
instead of adding it: the next block's first norm adds it in the same pass (one kernel
instead of the add, copy and norm that lucciola launches at src/qwen.cc:742-759)."""
from __future__ import annotations

from typing import Optional

import torch

from .base import Block, FeedForward, Mixer, Norm, NormSink, Part, RowScaled, StepContext


class PreNormBlock(Block):
    accepts_next_sink = True
    # Where the add and the norm between two products may run inside those products (see forward): "both", or only at
    # the block's "entry" (the block before -> this block's mixer), only in its "middle" (mixer -> feed-forward), or
    # "none": always as a kernel of their own.  For comparisons.
    fuse_norms = "both"
    recordable = True

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, ffn_norm: Norm, act_dtype: torch.dtype):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.ffn_norm = mixer_norm, ffn_norm
        self.act_dtype = act_dtype

    def children(self) -> list[Part]:
        return [self.mixer_norm, self.mixer, self.ffn_norm, self.feed_forward]

    def entry_sink(self, residual: torch.Tensor, num_tokens: int, write_cache: bool) -> Optional[NormSink]:
        """The block before may add its output to the residual stream itself and hand it over without the first norm's
        factor, when this block's mixer can take rows in that form for this step."""
        if self.fuse_norms in ("both", "entry") and self.mixer.row_scaled_ok(num_tokens, write_cache):
            return self.mixer_norm.as_sink(residual)
        return None

    def forward(self, residual: torch.Tensor, delta, step: StepContext, cache, write_cache: bool = True,
                next_sink: Optional[NormSink] = None):
        # Between two products, the add into the residual stream and the norm either run as a kernel of their own, or,
        # where the product before and the product after can, inside those two (NormSink, RowScaled).
        h = delta if isinstance(delta, RowScaled) else self.mixer_norm.add_forward(residual, delta, self.act_dtype)
        sink = None
        if self.fuse_norms in ("both", "middle") and self.mixer.accepts_sink and self.feed_forward.row_scaled_ok(step.num_tokens):
            sink = self.ffn_norm.as_sink(residual)
        a = self.mixer.forward(h, step, cache, write_cache, sink=sink) if sink is not None else self.mixer.forward(h, step, cache, write_cache)
        h = a if isinstance(a, RowScaled) else self.ffn_norm.add_forward(residual, a, self.act_dtype)
        if next_sink is not None and self.feed_forward.accepts_sink:
            return residual, self.feed_forward.forward(h, step, sink=next_sink)
        return residual, self.feed_forward.forward(h, step)
