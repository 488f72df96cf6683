"""RMSNorm with a weight: y = x * rsqrt(mean(x^2) + eps) * w, statistics and product in 32-bit
(src/kernels/rmsnorm.cu:57-97 of lucciola; eps is a literal 1e-6 there, a parameter here)."""
from __future__ import annotations

from typing import Callable, Optional

import torch

from .. import ops
from .base import Norm, NormSink, ParamSpec, Runtime


class RMSNorm(Norm):
    recordable = True

    def __init__(self, rt: Runtime, name: str, size: int, eps: float):
        self.rt, self.name, self.size, self.eps = rt, name, size, float(eps)
        self.weight: torch.Tensor | None = None     # float32 on the device

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(self.name, (self.size,), "norm")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        # bfloat16 -> float32 is exact; the kernels read norm weights as float32.
        self.weight = get(self.name).to(torch.float32).contiguous()

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        return self.add_forward(x, None, out_dtype)

    def as_sink(self, residual: torch.Tensor) -> Optional[NormSink]:
        return NormSink(residual, self.weight, self.eps)

    def add_forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out_dtype: torch.dtype,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = self.rt.empty((n, self.size), out_dtype)
        ops.add_rmsnorm(out, residual, delta, self.weight, self.eps, self.rt.stream, rows=rows)
        return out
