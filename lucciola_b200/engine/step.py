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

What the runner knows of the model is its interfaces: the cache each layer asks for, and the plans
that parts make for a step on the host (`Mixer.plan`), which it carries to the device with its own
integers.  How a part cuts its work into launches is the part's business.

Steps of a shape that comes again are recorded as CUDA graphs and replayed: a step is a few hundred
launches, and launching them one by one takes the host longer than the GPU needs to run them when the
step has few tokens.  The shape of a step is (how many single tokens lead it, the lengths of the
portions that follow, a bound on the context length): steps of single tokens only are padded to a
bucket and recorded the first time, steps with portions (lucciola's usual step while a prompt is
being read: every running request, then a portion, src/scheduler.cc:51-120) when their shape has come
`graph_after` times.  A recording reads everything that differs between steps of its shape (tokens,
positions, block tables, plans, new state slots) from one device buffer that is filled before each replay.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass
from typing import Hashable, Optional, Sequence

import numpy as np
import torch

from ..cache.device_cache import DeviceCache, pages_that_fit
from ..cache.manager import NO_PAGE, CacheManager, plan_groups
from ..config.engine_options import EngineOptions
from ..models.decoder import DecoderModel
from ..parts.base import BatchShape, PlanView, Runtime, StepContext, StepPlan


# Numbers of leading single tokens for which steps are recorded; a step is padded to the next one.
_GRAPH_BUCKETS = (1, 2, 4, 8, 12, 16, 24, 32, 48, 64, 96, 128, 192, 256)
# Steps with portions are recorded up to this many tokens and this many portions: beyond, the GPU needs longer
# for a step than the host needs to launch it.
_RECORD_TOKENS = 1024
_RECORD_PORTIONS = 4
# A recording of a portion of which some logits are wanted computes those of all its tokens; not worth it for
# a long portion of which few are wanted.
_ALL_ROWS = 64


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


@dataclass
class PreparedStep:
    """A step of single tokens whose host side is done (pages taken, the recording's input filled) but for the token
    ids: see ModelRunner.prepare_decode."""
    rids: list
    starts: list[int]
    shape: tuple
    host_index: int
    total: int
    tokens_in_step: int
    computed_rows: int
    wanted_rows: list[int]
    entries: list


@dataclass
class _Recording:
    graph: object                        # a torch.cuda.CUDAGraph: replay() runs the recorded step again
    logits: Optional[torch.Tensor]       # lives in the graph's memory; valid until the next step
    kernels: int                         # kernel nodes, for the launch count


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
        # The parts that plan work on the host for every step: one for each distinct key.
        self._planners: dict[Hashable, object] = {}
        for block in model.blocks:
            key = block.mixer.plan_key()
            if key is not None and key not in self._planners:
                self._planners[key] = block.mixer
        # Steps are recorded only when every part of the model says its forward() can be.
        self._can_record = bool(options.use_cuda_graph and rt.fast_kernels and all(p.recordable for p in model.all_parts()))
        self._staging: Optional[_Staging] = None
        self.steps_run = 0
        self.tokens_run = 0
        self.h2d_bytes = 0                 # bytes of step inputs copied from pinned host memory so far
        self._table_rows: dict[tuple[Hashable, int], tuple[int, np.ndarray]] = {}
        self._graphs: "OrderedDict[tuple, _Recording]" = OrderedDict()         # by shape, least recently used first
        self._graph_inputs: dict[tuple, torch.Tensor] = {}
        self._graph_pool = None            # the recordings replay one at a time and share their memory
        self._shape_seen: dict[tuple, int] = {}      # how often a shape with portions has come
        self._graph_launches = 0           # kernels replayed from CUDA graphs so far
        self.graph_replays = 0

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

    # ---- recordings ----------------------------------------------------------------
    def _shape_of(self, entries: Sequence[StepEntry], q_lens: Sequence[int], max_ctx: int) -> Optional[tuple]:
        """The shape under which this step may be recorded and replayed, or None: (single tokens that lead it,
        padded to a bucket; lengths of the portions behind them; bound on the context length; which logits of
        each portion a recording computes: "last", "none" or "all")."""
        if not self._can_record:
            return None
        lead = 0
        while lead < len(q_lens) and q_lens[lead] == 1:
            lead += 1
        portions = tuple(q_lens[lead:])
        if lead > _GRAPH_BUCKETS[-1] or len(portions) > _RECORD_PORTIONS:
            return None
        padded = next(b for b in _GRAPH_BUCKETS if b >= lead) if lead else 0
        if portions and padded + sum(portions) > _RECORD_TOKENS:
            return None
        kinds = []
        for e, n in zip(entries[lead:], portions):
            want = tuple(e.want)
            if want == (n - 1,):
                kinds.append("last")
            elif not want:
                kinds.append("none")
            elif n <= _ALL_ROWS or 2 * len(want) >= n:
                kinds.append("all")
            else:
                return None
        span = max(256, 1 << (max_ctx - 1).bit_length())
        return (padded, portions, span, tuple(kinds))

    def _record_now(self, shape: tuple) -> bool:
        """Steps of single tokens are recorded at once; shapes with portions when they have come often enough."""
        if shape in self._graphs or not shape[1]:
            return True
        seen = self._shape_seen[shape] = self._shape_seen.get(shape, 0) + 1
        if seen < self.options.graph_after:
            return False
        if len(self._shape_seen) > 4096:                                     # shapes that never came again
            self._shape_seen = {k: v for k, v in self._shape_seen.items() if v > 1}
        kept = [k for k in self._graphs if k[1]]
        if len(kept) >= self.options.max_shape_graphs:                       # the one not used for longest makes room
            del self._graphs[kept[0]]
            self._graph_inputs.pop(kept[0], None)
        return True

    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    def _sync(self) -> None:
        torch.cuda.current_stream(self.device).synchronize()

    def _forward(self, d_tok: torch.Tensor, step: StepContext, d_rows: Optional[torch.Tensor],
                 d_fresh: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if d_fresh is not None:
            self.cache.zero_slots(d_fresh, self.rt.stream)     # state of the requests this step admits
        return self.model.forward(d_tok, step, self.cache.views, d_rows)

    def _run_and_record(self, shape: tuple, d_tok: torch.Tensor, step: StepContext, d_rows: Optional[torch.Tensor],
                        d_fresh: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """The first step of a shape that is to be recorded: it runs as usual (which also warms every lazy set-up)
        and is then recorded; launches into a capturing stream are not executed.  Later steps replay the recording."""
        from .. import ops
        logits = self._forward(d_tok, step, d_rows, d_fresh)
        self._sync()
        before = ops.launch_count()
        graph = torch.cuda.CUDAGraph()
        if self._graph_pool is None:
            self._graph_pool = torch.cuda.graph_pool_handle()
        outer = self.rt.stream
        try:
            with torch.cuda.graph(graph, pool=self._graph_pool):
                self.rt.stream = torch.cuda.current_stream(self.device).cuda_stream
                static_logits = self._forward(d_tok, step, d_rows, d_fresh)
        finally:
            self.rt.stream = outer
        self._graphs[shape] = _Recording(graph, static_logits, ops.launch_count() - before)
        return logits

    # ---- the step ----------------------------------------------------------
    def _staging_for(self, n: int) -> _Staging:
        if self._staging is None or self._staging.capacity < n:
            if self._staging is not None:
                self._sync()                    # a copy out of the old buffers may still be under way
            self._staging = _Staging(self.device, max(n, 4096) * 2)
        return self._staging

    def prepare_decode(self, rids: Sequence[Hashable], want: Sequence[bool]) -> Optional[PreparedStep]:
        """The host side of a step that gives each of these running requests one more token, done before the tokens are
        known (while the GPU still runs the step that produces them): pages are taken and the recording's input is filled.
        finish_prepared() adds the token ids and replays the recording; drop_prepared() undoes it.  None when the step
        cannot be prepared (pages are short, or no recording of this batch size exists yet); nothing is taken then.
        No other step may run between prepare_decode and finish_prepared / drop_prepared."""
        if not self._can_record or not rids or not all(self.manager.has_request(r) for r in rids):
            return None
        entries = [StepEntry(r, (0,), (0,) if w else ()) for r, w in zip(rids, want)]
        try:
            return self._step(entries, prepare=True)
        except (OutOfPages, ValueError):
            return None

    def finish_prepared(self, prep: PreparedStep, tokens: Sequence[int]) -> Optional[torch.Tensor]:
        vocab = self.model.vocab_size
        if len(tokens) != len(prep.rids):
            raise ValueError(f"{len(tokens)} tokens for {len(prep.rids)} prepared requests")
        for rid, t in zip(prep.rids, tokens):
            if not (0 <= int(t) < vocab):
                raise ValueError(f"request {rid!r}: token id {t} is outside the vocabulary of {vocab}")
        st = self._staging
        st.host_np[prep.host_index][:len(tokens)] = tokens          # the token ids lead the buffer
        st.upload(prep.host_index, prep.total, self._graph_inputs[prep.shape])
        self.h2d_bytes += 4 * prep.total
        rec = self._graphs[prep.shape]
        self._graphs.move_to_end(prep.shape)
        rec.graph.replay()
        self._graph_launches += rec.kernels
        self.graph_replays += 1
        return self._after_step(prep.entries, prep.tokens_in_step, self._wanted(rec.logits, prep.wanted_rows, prep.computed_rows))

    def drop_prepared(self, prep: PreparedStep) -> None:
        self.manager.retract_by_one(prep.rids)

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Run the entries as one batch.  Returns logits [wanted, vocab] (float32, on the device) in the
        order of the entries and of their `want`, or None when nothing is wanted.  The tensor is valid until
        the next step."""
        return self._step(entries)

    def _step(self, entries: Sequence[StepEntry], prepare: bool = False):
        if not entries:
            return None
        vocab = self.model.vocab_size
        seen: set[Hashable] = set()
        token_arrays: list = []
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
        new_slots: list[tuple[int, int]] = []           # (entry, slot) of the requests this step admits
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
            for i, e in enumerate(entries):
                if not self.manager.has_request(e.rid):
                    new_slots.append((i, self.manager.admit(e.rid)))
                start = self.manager.length(e.rid)
                if not self.manager.extend(e.rid, start + len(e.tokens)):
                    raise OutOfPages("pages ran out while a step was being prepared")   # can_run() said yes
                starts.append(start)
                q_lens.append(len(e.tokens))

        S_real = len(entries)
        max_ctx = max(s + n for s, n in zip(starts, q_lens))
        # A step that is recorded, or replayed from a recording, is padded: behind its leading single tokens come
        # entries that own no page (their keys and values are written nowhere and they attend to nothing).
        shape = self._shape_of(entries, q_lens, max_ctx)
        if shape is not None and not self._record_now(shape):
            shape = None
        lead = pad = 0
        if shape is not None:
            lead = S_real - len(shape[1])
            pad = shape[0] - lead
            if pad:
                q_lens = q_lens[:lead] + [1] * pad + q_lens[lead:]
                starts = starts[:lead] + [0] * pad + starts[lead:]
        S, T = len(q_lens), sum(q_lens)
        place = lambda i: i if i < lead else i + pad          # where entry i sits among the padded ones
        # Which rows the output head computes, and which of them are handed out.
        if shape is None:
            R = sum(len(e.want) for e in entries)
            wanted_rows = list(range(R))
        else:
            R, wanted_rows = shape[0], [i for i in range(lead) if entries[i].want]
            for e, n, kind in zip(entries[lead:], shape[1], shape[3]):
                if kind == "last":
                    wanted_rows.append(R)
                    R += 1
                elif kind == "all":
                    wanted_rows += [R + w for w in e.want]
                    R += n
        G, P = len(self.groups), self.max_pages_per_seq
        batch = BatchShape(q_lens, starts, max(q_lens), max_ctx, shape[2] if shape is not None else max_ctx, shape is not None)
        made: dict[Hashable, StepPlan] = {}
        for key, part in self._planners.items():
            plan = part.plan(batch)
            if plan is not None:
                made[key] = plan
        has_state = bool(self.cache.states)
        total = 3 * T + (S + 1) + 3 * S + R + G * S * P + sum(a.size + 3 for p in made.values() for a in p.arrays.values())
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
        cu, ctx, slots, fresh, rows = take(S + 1), take(S), take(S), take(S), take(R)
        tables = [take(S * P).reshape(S, P) for _ in range(G)]
        for plan in made.values():
            for a in plan.arrays.values():
                o = (o + 3) & ~3                      # kernels read a work item as one 16-byte word
                take(a.size)[:] = a.reshape(-1)
        fresh[:] = -1
        for i, slot in new_slots:
            fresh[place(i)] = slot
        if batch.max_q_len == 1:
            # One token each: everything but the tables is a handful of whole-array assignments.
            ar = self._arange(S + 1)
            tok[:S_real] = token_arrays
            tok[S_real:] = 0
            pos[:] = starts
            seq[:] = ar[:S]
            cu[:] = ar
            ctx[:] = pos + 1
            slots[S_real:] = self.manager.num_slots            # the spare state row
            for g in range(G):
                tables[g][S_real:] = NO_PAGE
            for i, e in enumerate(entries):
                slots[i] = self.manager.slot(e.rid)
                for g in range(G):
                    tables[g][i] = self._table_row(e.rid, g)
            if shape is None:
                rows[:] = [i for i, e in enumerate(entries) for _ in e.want]
            else:
                rows[:] = ar[:R]
        else:
            if pad:
                tok[lead:lead + pad] = 0
                pos[lead:lead + pad] = 0
                slots[lead:lead + pad] = self.manager.num_slots     # the spare state row
                for g in range(G):
                    tables[g][lead:lead + pad] = NO_PAGE
            t, r = 0, 0
            cu[0] = 0
            for j in range(S):
                n = q_lens[j]
                seq[t:t + n] = j
                ctx[j] = starts[j] + n
                cu[j + 1] = t + n
                t += n
            for i, e in enumerate(entries):
                j = place(i)
                t, n = int(cu[j]), q_lens[j]
                tok[t:t + n] = token_arrays[i]
                pos[t:t + n] = np.arange(starts[j], starts[j] + n, dtype=np.int32)
                slots[j] = self.manager.slot(e.rid)
                for g in range(G):
                    tables[g][j] = self._table_row(e.rid, g)
                if shape is None:
                    for w in e.want:
                        rows[r] = t + w
                        r += 1
            if shape is not None:
                rows[:shape[0]] = self._arange(shape[0])           # the leading single tokens, padding included
                r = shape[0]
                for j, (n, kind) in enumerate(zip(shape[1], shape[3])):
                    t = int(cu[shape[0] + j])
                    if kind == "last":
                        rows[r] = t + n - 1
                        r += 1
                    elif kind == "all":
                        rows[r:r + n] = np.arange(t, t + n, dtype=np.int32)
                        r += n
        if prepare:
            if shape is None or shape not in self._graphs or batch.max_q_len != 1:
                self.manager.retract_by_one([e.rid for e in entries])
                return None
            return PreparedStep([e.rid for e in entries], starts[:S_real], shape, hi, total, T, R, wanted_rows, list(entries))
        dev = self._graph_inputs.get(shape) if shape is not None else None
        if shape is not None and dev is None:
            dev = self._graph_inputs[shape] = torch.empty(total, dtype=torch.int32, device=self.device)
        st.upload(hi, total, dev)
        self.h2d_bytes += 4 * total

        if shape is not None and shape in self._graphs:
            # The recording reads its inputs from the buffer just filled: nothing else to set up.
            rec = self._graphs[shape]
            self._graphs.move_to_end(shape)
            rec.graph.replay()
            self._graph_launches += rec.kernels
            self.graph_replays += 1
            return self._after_step(entries, T, self._wanted(rec.logits, wanted_rows, R))

        d = st.dev if dev is None else dev
        o = 0
        def view(n):
            nonlocal o
            v = d[o:o + n]
            o += n
            return v
        d_tok, d_pos, d_seq = view(T), view(T), view(T)
        d_cu, d_ctx, d_slots, d_fresh, d_rows = view(S + 1), view(S), view(S), view(S), view(R)
        d_tables = [view(S * P).view(S, P) for _ in range(G)]
        plans: dict[Hashable, PlanView] = {}
        for key, plan in made.items():
            arrays = {}
            for name, a in plan.arrays.items():
                o = (o + 3) & ~3
                arrays[name] = view(a.size).view(a.shape)
            plans[key] = PlanView(arrays, plan.host)

        step = StepContext(
            num_tokens=T, num_seqs=S, positions=d_pos, token_seq=d_seq, cu_tokens=d_cu, context_lens=d_ctx,
            block_tables=d_tables, state_slots=d_slots, q_lens=q_lens, start_positions=starts,
            max_q_len=batch.max_q_len, max_context_len=max_ctx, span_hint=batch.span_hint, plans=plans)
        self.rt.stream = self._stream()
        d_rows = d_rows if R else None
        d_fresh = d_fresh if has_state and (new_slots or shape is not None) else None
        if shape is None:
            logits = self._forward(d_tok, step, d_rows, d_fresh)
        else:
            logits = self._wanted(self._run_and_record(shape, d_tok, step, d_rows, d_fresh), wanted_rows, R)
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

    def _wanted(self, logits: Optional[torch.Tensor], wanted_rows: list[int], computed: int) -> Optional[torch.Tensor]:
        """The wanted rows among those a recording computes."""
        if not wanted_rows or logits is None:
            return None
        first, n = wanted_rows[0], len(wanted_rows)
        if wanted_rows[-1] == first + n - 1 and wanted_rows == list(range(first, first + n)):
            return logits if n == computed else logits[first:first + n]
        return logits.index_select(0, torch.tensor(wanted_rows, dtype=torch.long, device=self.device))

    def _after_step(self, entries: Sequence[StepEntry], T: int, logits: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if self._any_window:
            for e in entries:
                self.manager.release_behind_window(e.rid)
        self.steps_run += 1
        self.tokens_run += T
        return logits
