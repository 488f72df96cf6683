"""Dense gated feed-forward: down( silu(gate(h)) * up(h) ) (src/qwen.cc:762-794, src/kernels/swiglu.cu:30-36
of lucciola).  gate and up are one product over the stacked weights; on the bfloat16 path, when the
intermediate size is a multiple of 64, their rows are interleaved in blocks of 64 and silu(gate) * up is
formed in that product's epilogue, so the [T, 2 * intermediate] matrix is never written."""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from .base import FeedForward, NormSink, Part, RowScaled, Runtime, StepContext
from .linear import Linear


class SwiGLUFeedForward(FeedForward):
    recordable = True

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, intermediate_size: int):
        self.rt = rt
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.gate_up = Linear(rt, [f"{prefix}.gate_proj.weight", f"{prefix}.up_proj.weight"], hidden_size,
                              [intermediate_size, intermediate_size])
        self.down = Linear(rt, f"{prefix}.down_proj.weight", intermediate_size, hidden_size)
        self.fused = False

    def children(self) -> list[Part]:
        return [self.gate_up, self.down]

    def bind_all(self, get) -> None:
        super().bind_all(get)
        w = self.gate_up.weight
        self.fused = (self.rt.fast_kernels and w.is_cuda and w.dtype == torch.bfloat16 and self.intermediate_size % 64 == 0
                      and self.hidden_size % 8 == 0)
        if self.fused:
            inter = self.intermediate_size
            self.gate_up.weight = ops.interleave_gate_up(w[:inter], w[inter:])

    accepts_sink = True

    def row_scaled_ok(self, num_tokens: int) -> bool:
        """The products with the activation in their epilogue also apply a row's norm factor there."""
        return self.fused

    def _down(self, act: torch.Tensor, sink: Optional[NormSink]):
        if sink is not None and self.down.sink_ok(act):
            return self.down.forward_into(act, sink)
        return self.down.forward(act)

    def forward(self, h, step: StepContext, sink: Optional[NormSink] = None):
        inter = self.intermediate_size
        if isinstance(h, RowScaled):
            if not self.row_scaled_ok(h.shape[0]):
                raise ops.KernelError("this feed-forward was handed rows without their norm factor for a step it cannot take them in")
            act = self.rt.empty((h.shape[0], inter))
            ops.gemm_tcgen05(act, h.x, self.gate_up.weight, self.rt.stream, swiglu=True, sumsq=h.sumsq, eps=h.eps)
            return self._down(act, sink)
        if self.fused and ops.gemm_tcgen05_ok(h, h, self.gate_up.weight):
            act = self.rt.empty((h.shape[0], inter))
            ops.gemm_tcgen05(act, h, self.gate_up.weight, self.rt.stream, swiglu=True)
            return self._down(act, sink)
        if self.fused:
            raise ops.KernelError("the interleaved gate|up weights need the tensor-core product (bfloat16, 16-byte aligned input)")
        gu = self.gate_up.forward(h)
        act = self.rt.empty((h.shape[0], inter))
        ops.swiglu(act, gu[:, :inter], gu[:, inter:], self.rt.stream)
        return self._down(act, sink)
