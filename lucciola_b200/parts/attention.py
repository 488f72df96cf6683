"""Grouped-query attention over paged keys and values, with per-head RMSNorm of q and k.

Order of operations as in lucciola's decoder layer (src/qwen.cc:592-742): q, k, v projections
without bias; RMSNorm over each head of q and of k with a weight [head_dim] shared by the heads,
before the rotation; rotary position encoding of q and k; k and v written to the cache at the
token's position; causal attention of every query head h over the keys of kv head
h / (nq / nkv) with scale 1/sqrt(head_dim) unless another scale is given; output projection.
A window W, which lucciola does not have, limits a query at position p to keys p-W+1 .. p.

The attention kernels take their work from lists of tiles that this part makes on the host before a step runs
(`plan`): which tokens of which request form a tile, how many rows a tile has, which tiles go to which kernel.
"""
from __future__ import annotations

import math
from typing import Callable, Hashable, Optional, Sequence

import numpy as np
import torch

from .. import ops
from .base import (BatchShape, KVCacheView, KVPages, Mixer, NormSink, ParamSpec, Part, PositionEncoding, RowScaled, Runtime,
                   StepContext, StepPlan)
from .linear import Linear

# Entries with at least this many tokens in a step go to the tensor-memory attention kernel (128-row tiles).
BIG_PORTION = 16
# Query rows (heads of a group x tokens) of a tile of the mma.sync kernels; tiles of at most DECODE_ROWS rows have
# a kernel of their own, which a launch uses only if all of its tiles are such.
TILE_ROWS, DECODE_ROWS = 64, 16


def tiles_of(q_lens: Sequence[int], group: int, rows: int, take=None) -> list[tuple[int, int, int, int]]:
    """Runs of up to rows // group consecutive tokens of one request: (first token, tokens, request, 0),
    for the requests whose number of tokens passes `take`."""
    per = rows // group
    tiles, t = [], 0
    for i, n in enumerate(q_lens):
        if take is None or take(n):
            for off in range(0, n, per):
                tiles.append((t + off, min(per, n - off), i, 0))
        t += n
    return tiles


def plan_tiles(batch: BatchShape, group: int) -> StepPlan:
    """The tile lists of one step for query groups of `group` heads.  Kinds: "all" = every entry; when the step
    holds portions of prompts of BIG_PORTION tokens or more, also "big" = those portions in work items of up to 256
    rows (two tiles of floor(128 / group) tokens, for the tensor-memory kernel) and "rest" = the other entries.
    Tiles of "all" and "rest" have up to 64 query rows; but where single tokens sit beside portions of a few tokens,
    those lists are cut into tiles of at most 16 rows, so that one launch of the kernel for such tiles serves them all
    (a portion of 8 tokens beside 32 decoded tokens then costs two more tiles, not a launch with key ranges split
    through a workspace and a second kernel to combine them; its keys are read once per tile, which is little for a
    few tokens).  Each array is int32 [n, 4]; host["rows"][kind] is the most query rows of a tile of that kind."""
    q_lens, starts, g = batch.q_lens, batch.start_positions, group
    has_big = batch.max_q_len >= BIG_PORTION
    small = [n for n in q_lens if n < BIG_PORTION]
    fine = (g <= DECODE_ROWS and any(n * g <= DECODE_ROWS for n in small) and any(n * g > DECODE_ROWS for n in small))
    rows_small = DECODE_ROWS if fine else TILE_ROWS
    lists: dict[str, list] = {"all": tiles_of(q_lens, g, TILE_ROWS if has_big else rows_small)}
    if has_big:
        first_token = np.concatenate(([0], np.cumsum(q_lens)[:-1])).tolist()
        big = tiles_of(q_lens, g, 2 * (128 // g) * g, lambda n: n >= BIG_PORTION)
        # tiles that see the most keys first: the short ones then fill the end of the last wave
        big.sort(key=lambda tl: -(starts[tl[2]] + (tl[0] - first_token[tl[2]]) + tl[1]))
        lists["big"] = big
        if small:
            lists["rest"] = tiles_of(q_lens, g, rows_small, lambda n: n < BIG_PORTION)
    return StepPlan({k: np.asarray(tl, dtype=np.int32).reshape(len(tl), 4) for k, tl in lists.items()},
                    {"rows": {k: max(n for _, n, _, _ in tl) * g for k, tl in lists.items()}})


class GQAttention(Mixer):
    _decode_plans: dict[tuple[int, int], StepPlan] = {}      # (group size, batch size) -> plan of a step of single tokens

    def __init__(self, rt: Runtime, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position_encoding: Optional[PositionEncoding], qk_norm_eps: Optional[float], window: int = 0,
                 scale: Optional[float] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
        self.rt, self.prefix = rt, prefix
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.position_encoding = position_encoding
        self.qk_norm_eps = qk_norm_eps              # None: no q/k norm
        self.window = int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.q_size, self.kv_size = num_heads * head_dim, num_kv_heads * head_dim
        self.qkv = Linear(rt, [f"{prefix}.q_proj.weight", f"{prefix}.k_proj.weight", f"{prefix}.v_proj.weight"],
                          hidden_size, [self.q_size, self.kv_size, self.kv_size])
        self.o = Linear(rt, f"{prefix}.o_proj.weight", self.q_size, hidden_size)
        self.q_norm_w: torch.Tensor | None = None
        self.k_norm_w: torch.Tensor | None = None

    def children(self) -> list[Part]:
        return [self.qkv, self.o]

    @property
    def recordable(self) -> bool:
        """This part only launches kernels; a position encoding of its own kind has its own say."""
        return self.position_encoding is None or self.position_encoding.recordable

    def param_specs(self) -> list[ParamSpec]:
        if self.qk_norm_eps is None:
            return []
        return [ParamSpec(f"{self.prefix}.q_norm.weight", (self.head_dim,), "norm"),
                ParamSpec(f"{self.prefix}.k_norm.weight", (self.head_dim,), "norm")]

    def bind(self, get: Callable[[str], torch.Tensor]) -> None:
        if self.qk_norm_eps is not None:
            self.q_norm_w = get(f"{self.prefix}.q_norm.weight").to(torch.float32).contiguous()
            self.k_norm_w = get(f"{self.prefix}.k_norm.weight").to(torch.float32).contiguous()

    def plan_key(self) -> Optional[Hashable]:
        """The tensor-core kernels run on the bfloat16 path for groups of up to 64 query heads; the tile lists
        depend on the group size alone, so all such layers of a model share them."""
        g = self.num_heads // self.num_kv_heads
        return ("attention tiles", g) if self.rt.fast_kernels and g <= TILE_ROWS else None

    def plan(self, batch: BatchShape) -> Optional[StepPlan]:
        g = self.num_heads // self.num_kv_heads
        if batch.max_q_len == 1:                    # one token each: the same tiles for every step of this size
            key = (g, len(batch.q_lens))
            hit = self._decode_plans.get(key)
            if hit is None:
                hit = self._decode_plans[key] = plan_tiles(batch, g)
            return hit
        return plan_tiles(batch, g)

    def cache_request(self) -> KVPages:
        return KVPages(self.num_kv_heads, self.head_dim, self.window)

    accepts_sink = True

    def _heads_in_epilogue(self, num_tokens: int, write_cache: bool) -> bool:
        """Few tokens and heads of 128: the q|k|v product finishes the heads in its own epilogue."""
        rotary = self.position_encoding.rotary_table() if self.position_encoding is not None else None
        return (write_cache and self.rt.fast_kernels and (self.position_encoding is None or rotary is not None)
                and (rotary is None or rotary[1] == self.head_dim)
                and ops.gemm_tcgen05_heads_sizes_ok(num_tokens, self.qkv.out_features, self.hidden_size, self.head_dim))

    def row_scaled_ok(self, num_tokens: int, write_cache: bool = True) -> bool:
        """That epilogue also applies the factor that rows without their norm's factor lack; so does the many-token
        product."""
        return self._heads_in_epilogue(num_tokens, write_cache) or self.qkv.row_scaled_ok(num_tokens)

    def _project_out(self, out: torch.Tensor, sink: Optional[NormSink]):
        if sink is not None and self.o.sink_ok(out):
            return self.o.forward_into(out, sink)
        return self.o.forward(out)

    def forward(self, h, step: StepContext, cache: KVCacheView, write_cache: bool = True, sink: Optional[NormSink] = None):
        rt = self.rt
        T = h.shape[0]
        nq, nkv, d = self.num_heads, self.num_kv_heads, self.head_dim
        table = cache_table = step.block_tables[cache.group]
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 0.0
        q = rt.empty((T, nq, d))
        rotary = self.position_encoding.rotary_table() if self.position_encoding is not None else None
        scaled = h if isinstance(h, RowScaled) else None
        x = scaled.x if scaled is not None else h
        if self._heads_in_epilogue(T, write_cache) and ops.gemm_tcgen05_heads_ok(x, self.qkv.weight, d, rotary[1] if rotary is not None else None):
            # Norm, rotation, queries into their layout, keys and values into the pages: the product's output never
            # exists as a matrix.
            ops.gemm_tcgen05_heads(x, self.qkv.weight, q, step.positions, step.token_seq, cache_table, cache.k, cache.v,
                                   nq, nkv, cache.page_size, eps, rt.stream, q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w,
                                   inv_freq=rotary[0] if rotary is not None else None,
                                   sumsq=scaled.sumsq if scaled is not None else None, row_eps=scaled.eps if scaled is not None else 0.0)
            out = rt.empty((T, nq, d))
            ops.attention(q, out, cache.k, cache.v, step, cache.group, nq, nkv, d, cache.page_size, self.window,
                          self.scale, rt.stream, plan=step.plans.get(self.plan_key()))
            return self._project_out(out.view(T, self.q_size), sink)
        if scaled is not None and not self.qkv.row_scaled_ok(T):
            raise ops.KernelError("this mixer was handed rows without their norm factor for a step it cannot take them in")
        if write_cache:
            qkv = self.qkv.forward(h)
            q_in, k_in, v_in = qkv[:, :self.q_size], qkv[:, self.q_size:self.q_size + self.kv_size], qkv[:, self.q_size + self.kv_size:]
            n_kv = nkv
        else:
            # This call reads a cache another call has written: only q is needed.
            q_in = k_in = v_in = self.qkv.forward(h, rows=self.q_size)
            n_kv = 0
        if self.position_encoding is None or rotary is not None:
            inv_freq, rot = rotary if rotary is not None else (None, 0)
            ops.rope_kv(q_in, k_in, v_in, q, step.positions, nq, n_kv, d, eps, rt.stream,
                        q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w, inv_freq=inv_freq, rot_dim=rot,
                        k_cache=cache.k, v_cache=cache.v, token_seq=step.token_seq, block_table=cache_table,
                        page_size=cache.page_size)
        else:
            # A position encoding the fused kernel does not know: norm first, then the part's own
            # apply(), then the write.
            k_tmp, v_tmp = rt.empty((T, max(n_kv, 1), d)), rt.empty((T, max(n_kv, 1), d))
            ops.rope_kv(q_in, k_in, v_in, q, step.positions, nq, n_kv, d, eps, rt.stream,
                        q_norm_w=self.q_norm_w, k_norm_w=self.k_norm_w, k_out=k_tmp, v_out=v_tmp)
            self.position_encoding.apply(q, k_tmp, step.positions)
            if n_kv:
                k2, v2 = k_tmp.view(T, n_kv * d), v_tmp.view(T, n_kv * d)
                ops.rope_kv(k2, k2, v2, q, step.positions, 0, n_kv, d, 0.0, rt.stream,
                            k_cache=cache.k, v_cache=cache.v, token_seq=step.token_seq, block_table=cache_table,
                            page_size=cache.page_size)
        out = rt.empty((T, nq, d))
        ops.attention(q, out, cache.k, cache.v, step, cache.group, nq, nkv, d, cache.page_size, self.window,
                      self.scale, rt.stream, plan=step.plans.get(self.plan_key()))
        return self._project_out(out.view(T, self.q_size), sink)
