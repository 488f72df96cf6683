"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A batch may hold portions of prompts beside single decoded tokens, cut anywhere; it runs only
the tokens it is given and returns float32 logits at the places asked for.  lucciola's
step_with_paged_attention (src/qwen.cc:801-902) takes all running requests with one token each
followed by at most one portion of one prompt, computes logits for the last row of every
request whether wanted or not, and samples inside; here any mix of entries is one batch, logits
are computed for the wanted rows only, and sampling happens above.

The runner owns the model, the cache manager and the device memory of the caches.  Pages are
taken here, at the start of a step, for exactly the tokens of the step; whoever builds batches
(the scheduler, the trace replay) asks `can_run` first and decides what to do when pages are short.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Optional, Sequence

import numpy as np
import torch

from ..cache.device_cache import DeviceCache, pages_that_fit
from ..cache.manager import NO_PAGE, CacheManager, plan_groups
from ..config.engine_options import EngineOptions
from ..models.decoder import DecoderModel
from ..parts.base import Runtime, StepContext


# Entries with at least this many tokens in a step go to the tensor-memory attention kernel (128-row tiles).
_BIG_PORTION = 16

# Batch sizes for which decode-only steps are recorded as CUDA graphs; a batch is padded to the next one.
_GRAPH_BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)
# A step that is one short portion of one request (a short prompt, the end of a long one) is recorded too, per number of
# tokens, from the second time that number is seen: such a step is a few hundred launches, and launching them one by one
# takes the host longer than the GPU needs to run them (3.4 ms for 28 layers whether the portion has 36 or 512 tokens).
_SHORT_PORTION = 512
_SHORT_GRAPHS = 16                       # recordings of that kind kept at a time


class OutOfPages(RuntimeError):
    """A step needs more pages than are free; nothing was run and nothing was taken."""


@dataclass
class StepEntry:
    rid: Hashable                    # the request
    tokens: Sequence[int]            # its next tokens, in order
    want: Sequence[int] = ()         # places among these tokens whose logits are asked for


class _Staging:
    """Pinned host buffers (a small ring) and one device buffer for the integers of a step."""

    def __init__(self, device: torch.device, capacity: int, ring: int = 4):
        self.device, self.capacity = device, capacity
        self.host = [torch.empty(capacity, dtype=torch.int32, pin_memory=True) for _ in range(ring)]
        self.host_np = [h.numpy() for h in self.host]                 # the same memory, for the host-side fill
        self.events = [torch.cuda.Event() for _ in range(ring)]
        self.recorded = [False] * ring
        self.dev = torch.empty(capacity, dtype=torch.int32, device=device)
        self.turn = 0

    def next_host(self) -> tuple[int, torch.Tensor]:
        i = self.turn
        self.turn = (self.turn + 1) % len(self.host)
        if self.recorded[i]:
            self.events[i].synchronize()        # the copy that read this buffer has finished
        return i, self.host[i]

    def upload(self, i: int, n: int, dev: Optional[torch.Tensor] = None) -> None:
        from .. import ops
        stream = torch.cuda.current_stream(self.device)
        ops.upload((self.dev if dev is None else dev).data_ptr(), self.host[i].data_ptr(), 4 * n, stream.cuda_stream)
        self.events[i].record(stream)
        self.recorded[i] = True


class ModelRunner:
    def __init__(self, model: DecoderModel, rt: Runtime, options: EngineOptions, num_pages: Optional[int] = None):
        options.validate()
        self.model, self.rt, self.options = model, rt, options
        self.device = rt.device
        self.page_size = options.block_size
        self.max_model_len = options.max_model_len or model.max_positions
        if self.max_model_len > model.max_positions:
            raise ValueError(f"max_model_len {self.max_model_len} exceeds the model's {model.max_positions} positions")
        requests = model.cache_requests()
        self.groups, self.state_cache_ids = plan_groups(requests)
        if num_pages is None:
            num_pages = options.max_blocks
        if not num_pages:
            num_pages = pages_that_fit(self.groups, self.page_size, rt.act_dtype, self.device, options.mem_fraction)
            if num_pages <= 0:
                raise RuntimeError("no memory left for cache pages")
        self.num_pages = int(num_pages)
        self.manager = CacheManager(self.groups, self.page_size, self.num_pages, options.max_num_seqs)
        self.cache = DeviceCache(requests, self.groups, self.page_size, [self.num_pages] * len(self.groups),
                                 options.max_num_seqs, rt.act_dtype, self.device)
        self.max_pages_per_seq = -(-self.max_model_len // self.page_size)
        self._any_window = any(g.window > 0 for g in self.groups)
        self._arange_cache = np.arange(512, dtype=np.int32)
        self._decode_tiles: dict[int, list] = {}               # tiles of a decode-only step, by its (padded) size
        self._decode_tiles_flat: dict[int, np.ndarray] = {}
        # Group sizes for which a step carries tiles of the tensor-core attention kernel.
        self.tile_groups = sorted({g for b in model.blocks if (g := b.mixer.query_group_size()) and g <= 64}) \
            if rt.fast_kernels else []
        self._staging: Optional[_Staging] = None
        self.steps_run = 0
        self.tokens_run = 0
        self.h2d_bytes = 0                 # bytes of step inputs copied from pinned host memory so far
        self._table_rows: dict[tuple[Hashable, int], tuple[int, np.ndarray]] = {}
        self._graphs: dict[tuple[int, int], tuple[torch.cuda.CUDAGraph, torch.Tensor, int]] = {}
        self._graph_inputs: dict[tuple[int, int], torch.Tensor] = {}
        self._short_seen: dict[tuple[int, int], int] = {}       # how often a short portion of this size has come
        self._graph_launches = 0           # kernels replayed from CUDA graphs so far

    # ---- what a batch builder may ask ------------------------------------
    def length(self, rid: Hashable) -> int:
        return self.manager.length(rid) if self.manager.has_request(rid) else 0

    def can_run(self, entries: Sequence[StepEntry]) -> bool:
        """True when the free pages and slots suffice for all entries together."""
        need = [0] * len(self.groups)
        new_requests = 0
        for e in entries:
            if self.manager.has_request(e.rid):
                n = self.manager.pages_needed(e.rid, self.manager.length(e.rid) + len(e.tokens))
            else:
                new_requests += 1
                n = [-(-len(e.tokens) // self.page_size)] * len(self.groups)
            need = [a + b for a, b in zip(need, n)]
        if new_requests > len(self.manager._free_slots):
            return False
        return all(self.manager.pools[g].can_allocate(n) for g, n in enumerate(need))

    def kernel_launches(self) -> int:
        """Kernels of the library launched so far (replays of CUDA graphs counted by their kernel nodes)."""
        from .. import ops
        return ops.launch_count() + self._graph_launches

    def finish(self, rid: Hashable) -> None:
        """The request ended (or is preempted): its pages and its slot go back."""
        if self.manager.has_request(rid):
            self.manager.release(rid)
        for g in range(len(self.groups)):
            self._table_rows.pop((rid, g), None)

    # ---- the step ----------------------------------------------------------
    def _staging_for(self, n: int) -> _Staging:
        if self._staging is None or self._staging.capacity < n:
            torch.cuda.current_stream(self.device).synchronize()
            self._staging = _Staging(self.device, max(n, 4096) * 2)
        return self._staging

    def _run_graph(self, key: tuple, d_tok: torch.Tensor, step: StepContext, d_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """A step of a fixed shape (decoded tokens of a batch bucket, or one short portion of a given size): the first
        time it runs as usual and is then recorded (launches into a capturing stream are not executed); later steps replay
        the recording.  The result lives in the graph's memory and is valid until the next step."""
        from .. import ops
        hit = self._graphs.get(key)
        if hit is not None:
            graph, logits, kernels = hit
            graph.replay()
            self._graph_launches += kernels
            return logits
        logits = self.model.forward(d_tok, step, self.cache.views, d_rows)      # also warms every lazy set-up
        torch.cuda.current_stream(self.device).synchronize()
        before = ops.launch_count()
        graph = torch.cuda.CUDAGraph()
        outer = self.rt.stream
        with torch.cuda.graph(graph):
            self.rt.stream = torch.cuda.current_stream(self.device).cuda_stream
            static_logits = self.model.forward(d_tok, step, self.cache.views, d_rows)
        self.rt.stream = outer
        self._graphs[key] = (graph, static_logits, ops.launch_count() - before)
        return logits

    @staticmethod
    def _tiles(q_lens: Sequence[int], group: int, rows: int = 64, take=None) -> list[tuple[int, int, int, int]]:
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

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries as one batch.  Returns logits [wanted, vocab] (float32, on the device) in the
        order of the entries and of their `want`, or None when nothing is wanted."""
        if not entries:
            return None
        vocab = self.model.vocab_size
        seen: set[Hashable] = set()
        token_arrays: list[np.ndarray] = []
        for e in entries:
            if e.rid in seen:
                raise ValueError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.rid!r} brings no tokens")
            if self.length(e.rid) + n > self.max_model_len:
                raise ValueError(f"request {e.rid!r} would reach {self.length(e.rid) + n} tokens, the limit is {self.max_model_len}")
            for w in e.want:
                if not (0 <= w < n):
                    raise ValueError(f"request {e.rid!r} wants logits at place {w} of {n} tokens")
            if n == 1:                         # a decoded token: no array for one number
                lo = hi = int(e.tokens[0])
                token_arrays.append(lo)
            else:
                arr = np.asarray(e.tokens, dtype=np.int64)
                token_arrays.append(arr)
                lo, hi = int(arr.min()), int(arr.max())
            if lo < 0 or hi >= vocab:
                raise ValueError(f"request {e.rid!r}: token id {lo if lo < 0 else hi} is outside the vocabulary of {vocab}")
        # Take pages; collect the batch on the host.
        new_slots: list[int] = []
        starts, q_lens = [], []
        if all(isinstance(a, int) for a in token_arrays) and all(self.manager.has_request(e.rid) for e in entries):
            # every entry is one more token of a request that is under way: one pass over the page tables
            taken = self.manager.extend_by_one([e.rid for e in entries])
            if taken is None:
                raise OutOfPages(f"the step needs more pages than are free ({[p.num_free for p in self.manager.pools]} pages free)")
            starts, q_lens = taken, [1] * len(entries)
        else:
            if not self.can_run(entries):
                raise OutOfPages(f"the step needs more pages or slots than are free ({[p.num_free for p in self.manager.pools]} pages free)")
            for e in entries:
                if not self.manager.has_request(e.rid):
                    new_slots.append(self.manager.admit(e.rid))
                start = self.manager.length(e.rid)
                if not self.manager.extend(e.rid, start + len(e.tokens)):
                    raise OutOfPages("pages ran out while a step was being prepared")   # can_run() said yes
                starts.append(start)
                q_lens.append(len(e.tokens))

        S_real = len(entries)
        max_ctx = max(s + n for s, n in zip(starts, q_lens))
        # Decode-only steps replay a CUDA graph: the batch is padded to a bucket with entries that
        # own no page (their keys and values are written nowhere and they attend to nothing).
        graph_key = None
        if (self.options.use_cuda_graph and self.rt.fast_kernels and not self.cache.states and max(q_lens) == 1
                and S_real <= _GRAPH_BUCKETS[-1]):
            S = next(b for b in _GRAPH_BUCKETS if b >= S_real)
            span_hint = max(256, 1 << (max_ctx - 1).bit_length())
            graph_key = (S, span_hint)
            q_lens = q_lens + [1] * (S - S_real)
            starts = starts + [0] * (S - S_real)
        elif (self.options.use_cuda_graph and self.rt.fast_kernels and not self.cache.states and S_real == 1
              and 2 <= q_lens[0] <= _SHORT_PORTION):
            want = tuple(entries[0].want)
            # which logits the recording computes: those of the last token, none, or all of them
            rows_kind = "last" if want == (q_lens[0] - 1,) else "none" if not want else "all"
            key = (-q_lens[0], max(256, 1 << (max_ctx - 1).bit_length()), rows_kind)   # a negative first number: this kind
            if key in self._graphs:
                graph_key = key
            else:
                seen = self._short_seen[key] = self._short_seen.get(key, 0) + 1
                if seen >= 2:
                    short = [k for k in self._graphs if k[0] < 0]
                    if len(short) >= _SHORT_GRAPHS:                             # the oldest recording makes room
                        self._graphs.pop(short[0])
                        self._graph_inputs.pop(short[0], None)
                    graph_key = key
        decode_graph = graph_key is not None and graph_key[0] > 0
        S, T = len(q_lens), sum(q_lens)
        R = T if graph_key else sum(len(e.want) for e in entries)
        if graph_key and not decode_graph and graph_key[2] != "all":
            R = 1 if graph_key[2] == "last" else 0
        G, P = len(self.groups), self.max_pages_per_seq
        # Work items of the attention kernels, per group size: "all" = every entry in tiles of up to 64 query
        # rows; when the step holds portions of prompts, also "big" = those portions in work items of up to 256
        # rows (for the tcgen05 kernel) and "rest" = the other entries in 64-row tiles; and when the entries that are
        # not "big" mix tiles of at most 16 query rows (decoded tokens) with larger ones (a few tokens of a prompt),
        # "one" = the former and "rest" = the latter: tiles of at most 16 rows have a kernel of their own, which a
        # launch uses only if all of its tiles are such.
        tile_lists: dict[tuple[int, str], list] = {}
        first_token = [0] * S
        for i in range(1, S):
            first_token[i] = first_token[i - 1] + q_lens[i - 1]
        for g in self.tile_groups:
            if decode_graph:                      # one token each: the same tiles for every step of this size
                tile_lists[(g, "all")] = self._decode_tiles.get(S) or self._decode_tiles.setdefault(S, self._tiles(q_lens, g, 64))
                continue
            tile_lists[(g, "all")] = self._tiles(q_lens, g, 64)
            has_big = max(q_lens) >= _BIG_PORTION
            if has_big:
                # two tiles of floor(128 / g) tokens each
                big = self._tiles(q_lens, g, 2 * (128 // g) * g, lambda n: n >= _BIG_PORTION)
                # tiles that see the most keys first: the short ones then fill the end of the last wave
                big.sort(key=lambda tl: -(starts[tl[2]] + (tl[0] - first_token[tl[2]]) + tl[1]))
                tile_lists[(g, "big")] = big
            others = [n for n in q_lens if n < _BIG_PORTION]
            mixed = any(n * g <= 16 for n in others) and any(n * g > 16 for n in others)
            if mixed:
                tile_lists[(g, "rest")] = self._tiles(q_lens, g, 64, lambda n: n < _BIG_PORTION and n * g > 16)
                tile_lists[(g, "one")] = self._tiles(q_lens, g, 64, lambda n: n * g <= 16)
            elif has_big and others:
                tile_lists[(g, "rest")] = self._tiles(q_lens, g, 64, lambda n: n < _BIG_PORTION)
        total = 3 * T + (S + 1) + 2 * S + R + G * S * P + sum(4 * len(t) + 3 for t in tile_lists.values())
        st = self._staging_for(total)
        hi, _ = st.next_host()
        h = st.host_np[hi]
        o = 0
        def take(n):
            nonlocal o
            v = h[o:o + n]
            o += n
            return v
        tok, pos, seq = take(T), take(T), take(T)
        cu, ctx, slots, rows = take(S + 1), take(S), take(S), take(R)
        tables = [take(S * P).reshape(S, P) for _ in range(G)]
        for tl in tile_lists.values():
            o = (o + 3) & ~3                      # the kernel reads a tile as one 16-byte word
            flat = self._decode_tiles_flat.get(len(tl)) if decode_graph else None
            if flat is None:
                flat = np.asarray(tl, dtype=np.int32).reshape(-1)
                if decode_graph:
                    self._decode_tiles_flat[len(tl)] = flat
            take(4 * len(tl))[:] = flat
        wanted_rows: list[int] = []
        if decode_graph:
            # One token each: everything but the tables is a handful of whole-array assignments.
            ar = self._arange(S + 1)
            tok[:S_real] = token_arrays
            tok[S_real:] = 0
            pos[:] = starts
            seq[:] = ar[:S]
            cu[:] = ar
            ctx[:] = pos + 1
            rows[:] = ar[:T]
            slots[S_real:] = 0
            for g in range(G):
                tables[g][S_real:] = NO_PAGE
            for i, e in enumerate(entries):
                slots[i] = self.manager.slot(e.rid)
                for g in range(G):
                    tables[g][i] = self._table_row(e.rid, g)
                if e.want:
                    wanted_rows.append(i)
        else:
            t = 0
            cu[0] = 0
            for i, e in enumerate(entries):
                n = q_lens[i]
                tok[t:t + n] = token_arrays[i]
                slots[i] = self.manager.slot(e.rid)
                for g in range(G):
                    tables[g][i] = self._table_row(e.rid, g)
                wanted_rows += [t + w for w in e.want]
                pos[t:t + n] = np.arange(starts[i], starts[i] + n, dtype=np.int32)
                seq[t:t + n] = i
                t += n
                cu[i + 1] = t
                ctx[i] = starts[i] + n
        if graph_key is None:
            rows[:] = np.asarray(wanted_rows, dtype=np.int32)
        elif not decode_graph:
            if graph_key[2] == "all":
                rows[:] = self._arange(T)        # the recording computes the logits of every token
            elif graph_key[2] == "last":
                rows[0] = T - 1
                wanted_rows = [0]
        dev = self._graph_inputs.get(graph_key) if graph_key else None
        if graph_key and dev is None:
            dev = self._graph_inputs[graph_key] = torch.empty(total, dtype=torch.int32, device=self.device)
        st.upload(hi, total, dev)
        self.h2d_bytes += 4 * total

        if graph_key and graph_key in self._graphs:
            # The recording reads its inputs from the buffer just filled: nothing else to set up.
            graph, logits, kernels = self._graphs[graph_key]
            graph.replay()
            self._graph_launches += kernels
            return self._after_step(entries, T, self._wanted(logits, wanted_rows))

        d = st.dev if dev is None else dev
        o = 0
        def view(n):
            nonlocal o
            v = d[o:o + n]
            o += n
            return v
        d_tok, d_pos, d_seq = view(T), view(T), view(T)
        d_cu, d_ctx, d_slots, d_rows = view(S + 1), view(S), view(S), view(R)
        d_tables = [view(S * P).view(S, P) for _ in range(G)]
        attn_meta: dict[int, dict] = {}
        for (g, kind), tl in tile_lists.items():
            o = (o + 3) & ~3
            attn_meta.setdefault(g, {})[kind] = (view(4 * len(tl)).view(len(tl), 4), max(n for _, n, _, _ in tl) * g)

        step = StepContext(
            num_tokens=T, num_seqs=S, positions=d_pos, token_seq=d_seq, cu_tokens=d_cu, context_lens=d_ctx,
            block_tables=d_tables, state_slots=d_slots, q_lens=q_lens, start_positions=starts,
            max_q_len=max(q_lens), max_context_len=max_ctx, attn_meta=attn_meta)
        self.rt.stream = torch.cuda.current_stream(self.device).cuda_stream
        if new_slots and self.cache.states:
            self.cache.zero_slots(torch.tensor(new_slots, dtype=torch.long, device=self.device))
        if graph_key is None:
            logits = self.model.forward(d_tok, step, self.cache.views, d_rows if R else None)
        else:
            step.plans["span_hint"] = graph_key[1]
            logits = self._wanted(self._run_graph(graph_key, d_tok, step, d_rows if R else None), wanted_rows)
        return self._after_step(entries, T, logits)

    def _table_row(self, rid: Hashable, g: int) -> np.ndarray:
        """The request's block table of group g as a row of the step's table: converted once per change of the
        request's pages, not once per step."""
        ver = self.manager.version(rid)
        hit = self._table_rows.get((rid, g))
        if hit is None or hit[0] != ver:
            row = np.full(self.max_pages_per_seq, NO_PAGE, dtype=np.int32)
            bt = self.manager.block_table(rid, g)
            row[:len(bt)] = bt
            hit = self._table_rows[(rid, g)] = (ver, row)
        return hit[1]

    def _arange(self, n: int) -> np.ndarray:
        if self._arange_cache.shape[0] < n:
            self._arange_cache = np.arange(max(n, 512), dtype=np.int32)
        return self._arange_cache[:n]

    def _wanted(self, logits: torch.Tensor, wanted_rows: list[int]) -> Optional[torch.Tensor]:
        """The wanted rows of a recording's logits (it computes one row per token)."""
        if not wanted_rows:
            return None
        if wanted_rows == list(range(len(wanted_rows))):
            return logits[:len(wanted_rows)]
        return logits.index_select(0, torch.tensor(wanted_rows, dtype=torch.long, device=self.device))

    def _after_step(self, entries: Sequence[StepEntry], T: int, logits: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if self._any_window:
            for e in entries:
                self.manager.release_behind_window(e.rid)
        self.steps_run += 1
        self.tokens_run += T
        return logits
