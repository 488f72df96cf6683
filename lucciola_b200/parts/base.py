"""Interfaces of the parts a decoder is put together from.

A model is a list of blocks and a list of calls that says in which order the
blocks run and which cache each call uses.  A block arranges a mixer, a
feed-forward and norms; a mixer may use a position encoding.  Every part takes
its sizes and constants as constructor arguments, names the tensors it wants
from the checkpoint, and knows nothing of the model it sits in.

What a part must provide:

Part (all)        param_specs() -> [ParamSpec]    tensors wanted, by full name
                  bind(get)                        take them: get(name) -> tensor on the device
                  recordable                       True if forward() may be recorded into a CUDA graph
Norm              forward(x, out_dtype)            -> normed copy
                  add_forward(residual, delta, out_dtype, rows=None)
                                                   residual += delta; -> norm(residual) [on rows]
PositionEncoding  rotary_table() / apply(q, k, positions)
Mixer             cache_request() -> KVPages | StateSlot | None
                  forward(h, step, cache) -> [T, hidden] in the activation type
                  plan_key(), plan(batch) -> StepPlan   optional: work lists its kernels read on the device
FeedForward       forward(h, step) -> [T, hidden]
Block             mixer, forward(residual, delta, step, cache) -> (residual, delta)

`step` is the StepContext: what a part may know about the batch.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Hashable, Optional, Sequence

import numpy as np
import torch


@dataclass(frozen=True)
class ParamSpec:
    name: str                       # full tensor name in the checkpoint
    shape: tuple[int, ...]
    init: str = "linear"            # "linear" | "embedding" | "norm": how random weights are drawn
    integer: bool = False           # integer tables are kept as int32


@dataclass(frozen=True)
class KVPages:
    """A mixer that keeps keys and values of past tokens in pages."""
    num_kv_heads: int
    head_dim: int
    window: int = 0                 # 0: all keys; W: the last W keys (the query's own included)


@dataclass(frozen=True)
class StateSlot:
    """A mixer that keeps a state of fixed size for each request."""
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Runtime:
    """What parts share at run time: device, activation type, the stream of the current step."""

    def __init__(self, device: torch.device | str, act_dtype: torch.dtype):
        self.device = torch.device(device)
        self.act_dtype = act_dtype
        self.stream: int = 0        # raw handle, set by the step function before parts run
        self.fast_kernels = act_dtype == torch.bfloat16

    def empty(self, shape: Sequence[int], dtype: torch.dtype | None = None) -> torch.Tensor:
        return torch.empty(tuple(shape), dtype=dtype or self.act_dtype, device=self.device)


@dataclass
class KVCacheView:
    """One cache layer of paged keys and values, as a mixer sees it."""
    k: torch.Tensor                 # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
    group: int                      # index into StepContext.block_tables
    page_size: int


@dataclass
class StateCacheView:
    """One cache layer of per-request state: row `slot` belongs to the request in that slot.  The last row belongs
    to no request: the entries that pad a recorded step name it in `state_slots`, so that a mixer may treat them
    like any other entry."""
    state: torch.Tensor             # [slots + 1, *shape]


@dataclass
class BatchShape:
    """The batch of one step as the host knows it, for parts that plan work before the step runs.

    When the step is recorded as a CUDA graph, the recording is replayed for every later step with the same
    `q_lens`; `start_positions` and `max_context_len` are then those of the step at hand only, and `span_hint` is
    the bound on the context length that every step of the recording keeps (a power of two).  A plan's arrays may
    depend on all of these (they are refilled for every step); their shapes, and whatever a part's forward() takes
    from the host, may depend on `q_lens` and `span_hint` only."""
    q_lens: list[int]
    start_positions: list[int]
    max_q_len: int
    max_context_len: int
    span_hint: int
    recorded: bool = False


@dataclass
class StepPlan:
    """What a part's plan() returns: int32 arrays that travel to the device with the step's own integers, and
    what the part wants to keep on the host beside them (sizes its launches need)."""
    arrays: dict[str, np.ndarray]
    host: dict[str, Any] = field(default_factory=dict)


@dataclass
class PlanView:
    """A StepPlan as forward() sees it: the arrays as int32 tensors on the device, in the plan's shapes."""
    arrays: dict[str, torch.Tensor]
    host: dict[str, Any]


@dataclass
class StepContext:
    """The batch of one step, as parts see it.  Device tensors are int32.

    Tokens of one request are contiguous and in order; `token_seq[t]` is the
    index of token t's request among the S requests of this step."""
    num_tokens: int
    num_seqs: int
    positions: torch.Tensor                     # [T] absolute position of each token
    token_seq: torch.Tensor                     # [T]
    cu_tokens: torch.Tensor                     # [S+1] first token of each request
    context_lens: torch.Tensor                  # [S] length after this step
    block_tables: list[torch.Tensor]            # per cache group: [S, max_pages], -1 where no page
    state_slots: torch.Tensor                   # [S] slot of each request's fixed-size state
    # Host copies for planning (lists of ints).
    q_lens: list[int] = field(default_factory=list)
    start_positions: list[int] = field(default_factory=list)
    max_q_len: int = 0
    max_context_len: int = 0
    span_hint: int = 0                          # bound on the context lengths to plan launches for (see BatchShape)
    # What the parts planned for this step, by their plan_key().
    plans: dict[Hashable, PlanView] = field(default_factory=dict)


@dataclass
class RowScaled:
    """Rows that still lack the factor of their RMSNorm: the normed row m is x[m] * rsqrt(sum(sumsq[m]) / width + eps).
    A product whose epilogue adds to the residual stream hands its result on in this form (the row's sum of squares is
    complete only when all of the product's tiles are), and the product that reads it applies the factor to its
    32-bit sums: a factor per row commutes with a linear map."""
    x: torch.Tensor                 # [T, width], residual * norm weight, in the activation type
    sumsq: torch.Tensor             # [T, tiles] float32: sums of squares of the residual over blocks of the row
    width: int
    eps: float

    @property
    def shape(self):
        return self.x.shape


@dataclass
class NormSink:
    """Where a part may put its output instead of returning it: added into `residual` (float32, in place), and the
    sum handed on multiplied by `weight` as RowScaled, for the norm with these weights and eps that follows."""
    residual: torch.Tensor
    weight: torch.Tensor            # float32 [width]
    eps: float


class Part:
    # True when forward() only launches work on the step's stream and takes nothing from the host that changes
    # between steps of the same shape (see BatchShape): then a step through it may be recorded as a CUDA graph.
    # A part that reads device values on the host, synchronises or branches on positions leaves it False, and
    # models that hold such a part run every step launch by launch.
    recordable = False

    def param_specs(self) -> list[ParamSpec]:
        return []

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        pass

    def children(self) -> list["Part"]:
        return []

    def all_param_specs(self) -> list[ParamSpec]:
        specs = list(self.param_specs())
        for c in self.children():
            specs += c.all_param_specs()
        return specs

    def bind_all(self, get: Callable[[str], torch.Tensor]) -> None:
        self.bind(get)
        for c in self.children():
            c.bind_all(get)

    def all_parts(self) -> list["Part"]:
        out: list[Part] = [self]
        for c in self.children():
            out += c.all_parts()
        return out


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError

    def as_sink(self, residual: torch.Tensor) -> Optional[NormSink]:
        """If this norm is y = x * rsqrt(mean(x^2) + eps) * w, what a product's epilogue needs to stand in for
        add_forward(residual, its output); None for every other kind of norm."""
        return None

    def add_forward(self, residual: torch.Tensor, delta: Optional[torch.Tensor], out_dtype: torch.dtype,
                    rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    def rotary_table(self) -> Optional[tuple[torch.Tensor, int]]:
        """(inv_freq [rot/2] float32 on the device, rot) if this is a half-rotation encoding the fused kernel can apply."""
        return None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        """Encode positions into q [T, nq, d] and k [T, nkv, d] in place (used when rotary_table() is None)."""
        raise NotImplementedError


class Mixer(Part):
    def cache_request(self) -> KVPages | StateSlot | None:
        return None

    def plan_key(self) -> Optional[Hashable]:
        """Not None: this mixer wants plan() called once a step; mixers with equal keys share one plan."""
        return None

    def plan(self, batch: BatchShape) -> Optional[StepPlan]:
        """Work lists for this step's kernels, made on the host before the step runs.  forward() finds them in
        `step.plans[self.plan_key()]` as a PlanView."""
        return None

    # A mixer or feed-forward that sets `accepts_sink` takes a keyword `sink` (a NormSink or None) in forward() and may
    # return RowScaled when it used it; one whose row_scaled_ok() says yes for a step takes RowScaled as `h`.  Parts
    # that know neither are given plain tensors and asked for plain tensors.
    accepts_sink = False

    def row_scaled_ok(self, num_tokens: int, write_cache: bool = True) -> bool:
        return False

    def forward(self, h: torch.Tensor, step: StepContext, cache, write_cache: bool = True) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    accepts_sink = False

    def row_scaled_ok(self, num_tokens: int) -> bool:
        return False

    def forward(self, h: torch.Tensor, step: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    mixer: Mixer
    accepts_next_sink = False       # True: forward() takes the keyword `next_sink`

    def entry_sink(self, residual: torch.Tensor, num_tokens: int, write_cache: bool) -> Optional[NormSink]:
        """Not None: the block before this one may hand its output over already added to the residual stream and
        multiplied by this block's first norm weight (RowScaled), through this sink."""
        return None

    def forward(self, residual: torch.Tensor, delta, step: StepContext, cache, write_cache: bool = True,
                next_sink: Optional[NormSink] = None) -> tuple[torch.Tensor, object]:
        """`delta`: what the block before left to be added (a tensor, or None for the first block), or RowScaled when
        it went through this block's entry_sink.  Returns the residual stream and this block's own delta, RowScaled
        if it used `next_sink`."""
        raise NotImplementedError
