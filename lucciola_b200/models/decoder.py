"""A decoder as data: blocks, and the list of calls that runs them.

`calls` gives the order in which blocks run.  A call names a block and a cache; a block may be
called twice (with two caches), and a call may read a cache that an earlier call has written
(`write_cache=False`): then the mixer computes queries only and attends to what is there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Sequence

import torch

from ..parts.base import Block, KVPages, Norm, Part, Runtime, StateSlot, StepContext
from ..parts.embedding import OutputHead, TokenEmbedding


@dataclass(frozen=True)
class LayerCall:
    block: int
    cache: int
    write_cache: bool = True


class DecoderModel(Part):
    recordable = True

    def __init__(self, rt: Runtime, embedding: TokenEmbedding, blocks: Sequence[Block], calls: Sequence[LayerCall],
                 final_norm: Norm, head: OutputHead, vocab_size: int, max_positions: int, eos_token_ids: Sequence[int] = ()):
        self.rt = rt
        self.embedding, self.blocks, self.calls = embedding, list(blocks), list(calls)
        self.final_norm, self.head = final_norm, head
        self.vocab_size, self.max_positions = vocab_size, max_positions
        self.eos_token_ids = tuple(eos_token_ids)
        self._check_calls()

    def _check_calls(self) -> None:
        written: dict[int, int] = {}
        for i, c in enumerate(self.calls):
            if not (0 <= c.block < len(self.blocks)):
                raise ValueError(f"call {i} names block {c.block}, there are {len(self.blocks)}")
            if c.write_cache:
                if c.cache in written:
                    raise ValueError(f"cache {c.cache} is written by calls {written[c.cache]} and {i}")
                written[c.cache] = i
            elif c.cache not in written:
                raise ValueError(f"call {i} reads cache {c.cache} before any call has written it")
            else:
                a, b = self.blocks[self.calls[written[c.cache]].block].mixer.cache_request(), self.blocks[c.block].mixer.cache_request()
                if a != b:
                    raise ValueError(f"call {i} reads cache {c.cache} but its mixer wants {b}, the cache holds {a}")
        if sorted(written) != list(range(len(written))):
            raise ValueError(f"cache ids must be 0..n-1, got {sorted(written)}")
        self.num_caches = len(written)
        self._writer = written

    def children(self) -> list[Part]:
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def ignored_names(self) -> list[str]:
        return self.head.ignored_names()

    def cache_requests(self) -> list[KVPages | StateSlot | None]:
        """What each cache id has to hold, as asked by the mixer that writes it."""
        return [self.blocks[self.calls[self._writer[j]].block].mixer.cache_request() for j in range(self.num_caches)]

    def forward(self, token_ids: torch.Tensor, step: StepContext, caches: Sequence[object],
                logit_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the tokens of one step; float32 logits [R, vocab] for the rows asked for (None if none)."""
        residual = self.embedding.forward(token_ids)
        delta = None
        for i, c in enumerate(self.calls):
            # what the call after this one offers to take over from this one's last product (see Block.entry_sink)
            nxt = self.calls[i + 1] if i + 1 < len(self.calls) else None
            block = self.blocks[c.block]
            next_sink = self.blocks[nxt.block].entry_sink(residual, step.num_tokens, nxt.write_cache) if nxt is not None else None
            if next_sink is not None and block.accepts_next_sink:
                residual, delta = block.forward(residual, delta, step, caches[c.cache], c.write_cache, next_sink=next_sink)
            else:
                residual, delta = block.forward(residual, delta, step, caches[c.cache], c.write_cache)
        if logit_rows is None or logit_rows.shape[0] == 0:
            return None
        h = self.final_norm.add_forward(residual, delta, self.rt.act_dtype, rows=logit_rows)
        return self.head.forward(h)
