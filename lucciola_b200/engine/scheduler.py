"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.  Host code only; it sees the cache through the CacheManager.

What it keeps of lucciola's scheduler (src/scheduler.cc:42-139): requests that decode go first and
are not limited by the token budget; what is left of the budget goes to prompts, first come first
served, in portions of any size; a page is taken when a request crosses a page boundary; a
finished request gives its pages back at once.

What it decides differently:
  * Several prompts may have portions in one step.  A request is admitted when the pages for its
    whole prompt are free; later portions of a running prompt shrink to the pages that are free
    (lucciola schedules one portion of one prompt, all or nothing, src/scheduler.cc:89-97, and a
    prompt that does not fit blocks the queue for ever).
  * When pages run out, the request admitted last is preempted: its pages go back, it returns to
    the FRONT of the waiting queue and is later recomputed from its prompt plus what it has
    generated, so its output is the same as without the preemption.  (lucciola moves such a
    request to a queue that nothing reads again, src/scheduler.cc:33-40: the request is lost.)
  * A request that could never fit the pool on its own is refused when it is added.
  * With `token_tile` set, a portion that is not its prompt's last is shortened so that the step's tokens up to and
    including it are a multiple of the tile: the many-token products work on tiles of 128 tokens, and 32 decoded tokens
    beside a portion of 512 make them compute five tiles for 4.25 tiles of tokens.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Callable, Hashable, Iterable, Optional, Sequence

from ..cache.manager import CacheManager
from .request import Request, Status


@dataclass
class Scheduled:
    request: Request
    start: int             # position of the first token of this portion
    num_tokens: int
    sample: bool           # the portion reaches the request's last token: sample after the step


class Scheduler:
    def __init__(self, manager: CacheManager, max_tokens_per_step: int, max_num_seqs: int, max_model_len: int,
                 prefill_chunk: int = 0, eos_token_ids: Iterable[int] = (),
                 release: Optional[Callable[[Hashable], None]] = None, token_tile: int = 0):
        """`release(rid)` gives back all that a request holds; whoever keeps more per request than the cache
        manager does (the runner's converted block tables) passes its own."""
        self.manager = manager
        self._release_fn = release
        self.max_tokens_per_step = max_tokens_per_step
        self.max_num_seqs = min(max_num_seqs, manager.num_slots)
        self.max_model_len = max_model_len
        self.prefill_chunk = prefill_chunk
        self.token_tile = token_tile
        self.eos_token_ids = frozenset(eos_token_ids)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self._admissions = 0
        # counters
        self.num_preemptions = 0
        self.num_steps = 0
        self.num_scheduled_tokens = 0

    # ---- requests ----------------------------------------------------------
    def add_request(self, req: Request) -> None:
        req.params.validate()
        n = len(req.prompt)
        if n == 0:
            raise ValueError("a request needs at least one prompt token")
        if n >= self.max_model_len:
            raise ValueError(f"the prompt has {n} tokens; with max_model_len {self.max_model_len} nothing could be generated")
        most = min(n + req.params.max_new_tokens, self.max_model_len)
        pages = -(-most // self.manager.page_size)
        for g, pool in enumerate(self.manager.pools):
            if pages > pool.num_pages:
                raise ValueError(
                    f"the request may grow to {most} tokens = {pages} pages, the pool of cache group {g} has {pool.num_pages}")
        req.status = Status.WAITING
        self.waiting.append(req)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def abort(self, rid: int) -> bool:
        for r in list(self.running):
            if r.rid == rid:
                self._finish(r, "abort")
                return True
        for r in list(self.waiting):
            if r.rid == rid:
                self.waiting.remove(r)
                r.status, r.finish_reason = Status.FINISHED, "abort"
                return True
        return False

    # ---- pages, as they will be when the step takes them ----------------------
    def _pages_needed(self, r: Request, new_len: int) -> list[int]:
        if self.manager.has_request(r.rid):
            return self.manager.pages_needed(r.rid, new_len)
        return [-(-new_len // self.manager.page_size)] * len(self.manager.pools)

    def _fits(self, need: Sequence[int], reserved: Sequence[int]) -> bool:
        return all(p.num_free - reserved[g] >= need[g] for g, p in enumerate(self.manager.pools))

    def _largest_fit(self, r: Request, upto: int, reserved: Sequence[int]) -> int:
        """The largest length <= upto whose pages are free, given what the plan has reserved."""
        ps = self.manager.page_size
        best = upto
        for g, p in enumerate(self.manager.pools):
            have = len(self.manager.block_table(r.rid, g)) if self.manager.has_request(r.rid) else 0
            best = min(best, (have + p.num_free - reserved[g]) * ps)
        return best

    def _release(self, rid: Hashable) -> None:
        if self._release_fn is not None:
            self._release_fn(rid)
        elif self.manager.has_request(rid):
            self.manager.release(rid)

    def _aligned(self, n: int, r: Request, budget: int) -> int:
        """The portion of n tokens, shortened so that the step's tokens so far plus the portion fill whole token tiles;
        unchanged when it is the prompt's last portion, or when less than half of it would be left."""
        tile = self.token_tile
        if tile <= 1 or n >= r.remaining:
            return n
        used = self.max_tokens_per_step - budget
        shorter = (used + n) // tile * tile - used
        return shorter if shorter >= max(1, n // 2) else n

    def _preempt(self, r: Request) -> None:
        self._release(r.rid)
        self.running.remove(r)
        r.status = Status.WAITING
        r.num_computed = 0
        r.preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(r)

    def _finish(self, r: Request, reason: str) -> None:
        self._release(r.rid)
        if r in self.running:
            self.running.remove(r)
        r.status, r.finish_reason = Status.FINISHED, reason

    # ---- one step ------------------------------------------------------------
    def schedule(self) -> list[Scheduled]:
        """The batch of the next step.  Empty only when there is nothing to do."""
        while True:
            plan = self._schedule_once()
            if plan or not self.running:
                return plan
            # Every running request is stuck for pages: free the latest and try again.
            self._preempt(max(self.running, key=lambda r: r.admitted_at))

    def _schedule_once(self) -> list[Scheduled]:
        plan: list[Scheduled] = []
        # The common step of a running engine: nobody waits, everybody decodes, and there is a free page in every
        # group for each of them (more than they can need).  Nothing to weigh then.
        if not self.waiting and self.running and all(p.num_free >= len(self.running) for p in self.manager.pools) \
                and all(r.remaining == 1 for r in self.running):
            for r in sorted(self.running, key=lambda r: r.admitted_at):
                plan.append(Scheduled(r, r.num_computed, 1, True))
            self.num_steps += 1
            self.num_scheduled_tokens += len(plan)
            return plan
        reserved = [0] * len(self.manager.pools)
        budget = self.max_tokens_per_step

        def take(r: Request, n: int, need: Optional[Sequence[int]] = None) -> None:
            nonlocal budget
            if need is None:
                need = self._pages_needed(r, r.num_computed + n)
            for g, k in enumerate(need):
                reserved[g] += k
            plan.append(Scheduled(r, r.num_computed, n, r.num_computed + n == r.length))
            budget -= n

        preempted = False
        # 1. Requests that decode: one token each, whatever the budget says.
        for r in sorted((r for r in self.running if r.remaining == 1), key=lambda r: r.admitted_at):
            if r not in self.running:
                continue                      # it was a victim a moment ago
            need = self._pages_needed(r, r.num_computed + 1)
            while not self._fits(need, reserved):
                scheduled = {s.request.rid for s in plan}
                victims = [v for v in self.running if v.rid not in scheduled]
                victim = max(victims, key=lambda v: v.admitted_at)
                self._preempt(victim)
                preempted = True
                if victim is r:
                    break
            if r in self.running:
                take(r, 1, need)

        # 2. Prompts under way (and requests that are recomputed), oldest first.  After a preemption
        # nothing new starts in this step, or the victim would come straight back.
        blocked = preempted
        for r in sorted((r for r in self.running if r.remaining > 1), key=lambda r: r.admitted_at):
            if budget <= 0:
                break
            most = min(budget, self.prefill_chunk or budget, r.remaining)
            n = self._aligned(most, r, budget)
            n = min(n, self._largest_fit(r, r.num_computed + n, reserved) - r.num_computed)
            if n <= 0:
                blocked = True
                break
            take(r, n)
            if n < most and self.token_tile > 1:
                budget = 0                    # the step ends on a tile's edge: what is left of the budget stays unused

        # 3. New requests, first come first served, while there is budget and a slot.  A request is
        # admitted only when the pages for all it has to run (its prompt, and what it had generated
        # before a preemption) are free now: admitting it earlier would only get it preempted again.
        while self.waiting and not blocked and budget > 0 and len(self.running) < self.max_num_seqs:
            r = self.waiting[0]
            if not self._fits(self._pages_needed(r, r.length), reserved):
                break
            most = min(budget, self.prefill_chunk or budget, r.remaining)
            n = self._aligned(most, r, budget)
            self.waiting.popleft()
            r.status = Status.RUNNING
            r.admitted_at = self._admissions
            self._admissions += 1
            self.running.append(r)
            take(r, n)
            if n < most:
                budget = 0

        self.num_steps += bool(plan)
        self.num_scheduled_tokens += sum(s.num_tokens for s in plan)
        return plan

    def update(self, plan: Sequence[Scheduled], sampled: Sequence[int]) -> list[tuple[Request, int, bool]]:
        """After the step: `sampled` holds one token for each plan entry with sample=True, in order.
        Returns (request, new token, finished) for those entries."""
        out = []
        it = iter(sampled)
        for s in plan:
            r = s.request
            r.num_computed += s.num_tokens
            if not s.sample:
                continue
            tok = int(next(it))
            r.append(tok)
            reason = None
            if tok in self.eos_token_ids and not r.params.ignore_eos:
                reason = "stop"
            elif len(r.output) >= r.params.max_new_tokens:
                reason = "length"
            elif r.length >= self.max_model_len:
                reason = "length"
            if reason:
                self._finish(r, reason)
            out.append((r, tok, reason is not None))
        return out
