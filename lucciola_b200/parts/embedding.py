"""Token embedding and output head."""
from __future__ import annotations

from typing import Callable

import torch

from .. import ops
from .base import ParamSpec, Part, Runtime
from .linear import Linear


class TokenEmbedding(Part):
    """residual[t, :] = table[id_t, :], unscaled (src/kernels/embedding.cu:22-38 of lucciola), as float32."""
    recordable = True


    def __init__(self, rt: Runtime, name: str, vocab_size: int, hidden_size: int):
        self.rt, self.name, self.vocab_size, self.hidden_size = rt, name, vocab_size, hidden_size
        self.weight: torch.Tensor | None = None

    def param_specs(self) -> list[ParamSpec]:
        return [ParamSpec(self.name, (self.vocab_size, self.hidden_size), "embedding")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        self.weight = get(self.name).contiguous()

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        out = self.rt.empty((token_ids.shape[0], self.hidden_size), torch.float32)
        ops.embedding(out, token_ids, self.weight, self.rt.stream)
        return out


class OutputHead(Part):
    """logits = h . W^T in float32; W is its own tensor or the embedding table when tied
    (src/qwen.cc:80-84 of lucciola falls back to a second copy of the table; here the table is shared)."""
    recordable = True


    def __init__(self, rt: Runtime, name: str, vocab_size: int, hidden_size: int, tied_to: TokenEmbedding | None):
        self.rt, self.name, self.tied_to = rt, name, tied_to
        self.vocab_size = vocab_size
        self.proj = Linear(rt, name, hidden_size, vocab_size)

    def param_specs(self) -> list[ParamSpec]:
        return [] if self.tied_to is not None else self.proj.param_specs()

    def ignored_names(self) -> list[str]:
        """A tied head does not need its own tensor; a checkpoint may carry one all the same."""
        return [self.name] if self.tied_to is not None else []

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        if self.tied_to is not None:
            self.proj.bind_tensor(self.tied_to.weight)
        else:
            self.proj.bind(get)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        return self.proj.forward(h, out_dtype=torch.float32)
