"""Rotary position encoding, half-rotation ("NeoX") pairing: for i < rot/2 the pair
(x[i], x[i + rot/2]) is rotated by pos * theta^(-2i/rot) (src/kernels/rope.cu:28-60 of lucciola,
where theta is the literal 1e6 at src/qwen.cc:636; here it is a parameter).

The table of inverse frequencies is made once on the host in float32; the kernel forms the
angle as one float32 product pos * inv_freq[i]."""
from __future__ import annotations

import torch

from .base import PositionEncoding, Runtime


class RotaryEmbedding(PositionEncoding):
    recordable = True

    def __init__(self, rt: Runtime, head_dim: int, theta: float, rot_dim: int | None = None):
        self.rt = rt
        self.head_dim = head_dim
        self.rot_dim = head_dim if rot_dim is None else rot_dim
        if self.rot_dim % 2 or self.rot_dim > head_dim:
            raise ValueError(f"rotary size {self.rot_dim} must be even and at most head_dim {head_dim}")
        self.theta = float(theta)
        exponent = torch.arange(0, self.rot_dim, 2, dtype=torch.float32) / float(self.rot_dim)
        inv = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float32), exponent)
        self.inv_freq = inv.to(rt.device)

    def rotary_table(self):
        return self.inv_freq, self.rot_dim
