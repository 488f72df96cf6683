"""Linear maps without bias: y = x . W^T with W [out, in] as the checkpoint stores it.

A Linear may be made of several checkpoint tensors stacked along the output
dimension (q|k|v, gate|up): one product instead of several.  lucciola keeps
them apart and runs one product each (src/qwen.cc:592-615, 762-777).
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch

from .. import ops
from .base import NormSink, ParamSpec, Part, RowScaled, Runtime


class Linear(Part):
    recordable = True

    def __init__(self, rt: Runtime, names: str | Sequence[str], in_features: int, out_features: int | Sequence[int],
                 init: str = "linear"):
        self.rt = rt
        self.names = [names] if isinstance(names, str) else list(names)
        self.out_sizes = [out_features] if isinstance(out_features, int) else list(out_features)
        if len(self.names) != len(self.out_sizes):
            raise ValueError("one output size for each tensor name")
        self.in_features = in_features
        self.out_features = sum(self.out_sizes)
        self.init = init
        self.weight: torch.Tensor | None = None

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(n, (o, self.in_features), self.init) for n, o in zip(self.names, self.out_sizes)]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        ws = [get(n) for n in self.names]
        if len(ws) == 1:
            self.weight = ws[0].contiguous()
        else:
            dt = ws[0].dtype
            if any(w.dtype != dt for w in ws):
                raise ValueError(f"tensors {self.names} are stacked into one product and must share a type")
            self.weight = torch.cat(ws, dim=0).contiguous()

    def bind_tensor(self, weight: torch.Tensor) -> None:
        """Use a tensor another part owns (a tied output head)."""
        self.weight = weight

    def sink_ok(self, x: torch.Tensor) -> bool:
        """Whether forward_into() takes this input: the bfloat16 path, and a product that is split over a cluster."""
        return self.rt.fast_kernels and ops.gemm_tcgen05_addnorm_ok(x, self.weight)

    def forward_into(self, x: torch.Tensor, sink: NormSink) -> RowScaled:
        """sink.residual += x . W^T, and the sum times the sink's norm weight, without the row's factor, handed on."""
        M, N = x.shape[0], self.weight.shape[0]
        out = self.rt.empty((M, N))
        sumsq = self.rt.empty((M, ops.gemm_tcgen05_addnorm_tiles(M, N, x.shape[1])), torch.float32)
        ops.gemm_tcgen05_addnorm(x, self.weight, sink.residual, sink.weight, out, sumsq, self.rt.stream)
        return RowScaled(out, sumsq, N, sink.eps)

    def row_scaled_ok(self, num_tokens: int) -> bool:
        """Whether forward() takes rows without their norm's factor: the tensor-core products apply it in their epilogues."""
        return self.rt.fast_kernels and self.in_features % 8 == 0

    def forward(self, x, out_dtype: torch.dtype | None = None, rows: int | None = None) -> torch.Tensor:
        """y = x . W^T; with `rows`, only the first `rows` output features.  x: a tensor, or RowScaled."""
        M = x.shape[0]
        w = self.weight if rows is None else self.weight[:rows]
        y = self.rt.empty((M, w.shape[0]), out_dtype or self.rt.act_dtype)
        if isinstance(x, RowScaled):
            if not (self.row_scaled_ok(M) and ops.gemm_tcgen05_ok(y, x.x, w)):
                raise ops.KernelError("this product was handed rows without their norm factor for sizes it cannot take them in")
            ops.gemm_tcgen05(y, x.x, w, self.rt.stream, sumsq=x.sumsq, eps=x.eps)
            return y
        ops.linear(y, x, w, self.rt.stream, fast=self.rt.fast_kernels)
        return y
