"""Dense gated feed-forward: down( silu(gate(h)) * up(h) ) (src/qwen.cc:762-794, src/kernels/swiglu.cu:30-36
of lucciola).  gate and up are one product over the stacked weights."""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, Part, Runtime, StepContext
from .linear import Linear


class SwiGLUFeedForward(FeedForward):
    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, intermediate_size: int):
        self.rt = rt
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_up = Linear(rt, [f"{prefix}.gate_proj.weight", f"{prefix}.up_proj.weight"], hidden_size,
                              [intermediate_size, intermediate_size])
        self.down = Linear(rt, f"{prefix}.down_proj.weight", intermediate_size, hidden_size)

    def children(self) -> list[Part]:
        return [self.gate_up, self.down]

    def forward(self, h: torch.Tensor, step: StepContext) -> torch.Tensor:
        gu = self.gate_up.forward(h)
        inter = self.intermediate_size
        act = self.rt.empty((h.shape[0], inter))
        ops.swiglu(act, gu[:, :inter], gu[:, inter:], self.rt.stream)
        return self.down.forward(act)
