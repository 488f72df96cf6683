"""Greedy and temperature sampling of one token per row of logits, on the GPU.

Greedy takes the largest logit, the lowest index among equals.  With a temperature T > 0 the token
is argmax_i(logit_i / T - log(-log(u_i))) (Gumbel-max: a draw from softmax(logits / T)), where u_i
is a hash of (key of the request's seed, index of the generated token, i).  The draw therefore
depends on the request alone, not on the batch it shares a step with."""
from __future__ import annotations

from typing import Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams

_M64 = (1 << 64) - 1


def _mix64(x: int) -> int:
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & _M64
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & _M64
    x ^= x >> 31
    return x


def sampling_key(seed: int) -> int:
    """64-bit key of a request's random stream."""
    return _mix64((seed & _M64) ^ 0x632BE59BD9B4E019)


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device
        self._host: torch.Tensor | None = None          # pinned memory the sampled ids are read back into
        self._done = torch.cuda.Event() if torch.device(device).type == "cuda" else None

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], generated: Sequence[int]) -> list[int]:
        """One token for each row; `generated[r]` is how many tokens request r has generated so far."""
        return self.collect(self.launch(logits, params, generated))

    def launch(self, logits: torch.Tensor, params: Sequence[SamplingParams], generated: Sequence[int]):
        """Start sampling and the copy of the ids to the host; collect() waits for them.  What the host does in
        between overlaps the GPU's work on the step."""
        R = logits.shape[0]
        tokens = torch.empty(R, dtype=torch.int32, device=self.device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        if all(p.temperature <= 0 for p in params):
            ops.sample(tokens, logits, stream)
        else:
            temps = torch.tensor([p.temperature for p in params], dtype=torch.float32).to(self.device, non_blocking=True)
            keys = np.array([sampling_key(p.seed) for p in params], dtype=np.uint64).view(np.int64)
            keys_t = torch.from_numpy(keys).to(self.device, non_blocking=True)
            counters = torch.tensor(list(generated), dtype=torch.int32).to(self.device, non_blocking=True)
            ops.sample(tokens, logits, stream, temps, keys_t, counters)
        if self._done is None:
            return tokens
        if self._host is None or self._host.shape[0] < R:
            self._host = torch.empty(max(R, 256), dtype=torch.int32, pin_memory=True)
        self._host[:R].copy_(tokens, non_blocking=True)
        self._done.record()
        return R

    def collect(self, handle) -> list[int]:
        if self._done is None:
            return handle.cpu().tolist()
        self._done.synchronize()
        return self._host[:handle].tolist()
