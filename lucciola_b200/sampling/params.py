"""What a request may ask of the sampler.  lucciola's request carries max_new_tokens only
(include/async_engine.h:15-20) and always takes the largest logit; temperature is added here."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class SamplingParams:
    max_new_tokens: int = 16
    temperature: float = 0.0          # 0: greedy
    seed: int = 0                     # stream of random numbers of a request with temperature > 0
    ignore_eos: bool = False          # keep generating past an end-of-sequence token

    def validate(self) -> None:
        if self.max_new_tokens <= 0:
            raise ValueError(f"max_new_tokens must be positive, got {self.max_new_tokens}")
        if self.temperature < 0:
            raise ValueError(f"temperature must not be negative, got {self.temperature}")
