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
    all_tokens: list[int] = field(default_factory=list)     # prompt + output, kept as one list for slicing
    num_computed: int = 0              # tokens whose keys and values are in the cache
    finish_reason: Optional[str] = None
    preemptions: int = 0
    admitted_at: int = -1              # order of admission, for the choice of a victim

    def __post_init__(self) -> None:
        self.all_tokens = list(self.prompt) + list(self.output)

    @property
    def tokens(self) -> list[int]:
        return self.all_tokens

    def append(self, token: int) -> None:
        self.output.append(token)
        self.all_tokens.append(token)

    @property
    def length(self) -> int:
        return len(self.all_tokens)

    @property
    def remaining(self) -> int:
        """Tokens that still have to be run before the next one can be sampled."""
        return self.length - self.num_computed
