"""A request as the scheduler sees it (lucciola's Sequence, include/sequence.h:10-42: id, status,
prompt length, how much of the prompt has been run, the token ids)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Callable, Optional

from ..sampling.params import SamplingParams


class Status(enum.Enum):
    WAITING = "waiting"        # holds nothing in the cache
    RUNNING = "running"        # holds pages and a slot
    FINISHED = "finished"


@dataclass
class Request:
    rid: int
    prompt: list[int]
    params: SamplingParams
    callback: Optional[Callable[[int, bool], None]] = None
    status: Status = Status.WAITING
    output: list[int] = field(default_factory=list)
    num_computed: int = 0              # tokens whose keys and values are in the cache
    finish_reason: Optional[str] = None
    preemptions: int = 0
    admitted_at: int = -1              # order of admission, for the choice of a victim

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.output

    @property
    def length(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def remaining(self) -> int:
        """Tokens that still have to be run before the next one can be sampled."""
        return self.length - self.num_computed
