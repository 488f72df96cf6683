"""The Python entry points, in the manner of lucciola's AsyncEngine (include/async_engine.h:22-35):

    engine = AsyncEngine(model_path, max_blocks=0, block_size=16)
    req_id = engine.generate_async(prompt, max_new_tokens, callback)    # callback(token, is_finished)
    engine.abort(req_id)                                                # not in lucciola: give a request up
    engine.stats()
    engine.stop()

lucciola's prompt is text and its callback receives text; tokenisation is outside this engine, so
here a prompt is a list of token ids and the callback receives token ids.  `Engine` is the same
loop without the thread: `generate(prompts, params)` returns when every request has finished.
"""
from __future__ import annotations

import threading
from pathlib import Path
from typing import Any, Callable, Mapping, Optional, Sequence

import torch

from ..config.engine_options import EngineOptions
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler
from .load import build_runner, build_runner_random
from .request import Request
from .scheduler import Scheduled, Scheduler
from .step import ModelRunner, StepEntry


class Engine:
    """Synchronous engine: scheduler above the step function, sampler after it."""

    def __init__(self, model_path: Optional[str | Path] = None, max_blocks: int = 0, block_size: int = 16,
                 options: Optional[EngineOptions] = None, runner: Optional[ModelRunner] = None, **kw: Any):
        if runner is None:
            options = options or EngineOptions(max_blocks=max_blocks, block_size=block_size, **kw)
            if model_path is None:
                raise ValueError("give a model folder (or a runner)")
            runner = build_runner(model_path, options)
        self.runner = runner
        self.options = runner.options
        self.scheduler = Scheduler(runner.manager, self.options.max_tokens_per_step, self.options.max_num_seqs,
                                   runner.max_model_len, self.options.prefill_chunk, runner.model.eos_token_ids,
                                   release=runner.finish, token_tile=self.options.token_tile)
        self.sampler = Sampler(runner.device)
        self._next_id = 1
        self._live: dict[int, Request] = {}              # requests that have not finished, by id
        self._prepared = None                            # the next step's host side, done while the GPU ran this one
        # What to do when a request's callback raises: None lets the exception through to whoever called step().
        self.on_callback_error: Optional[Callable[[Request, BaseException], None]] = None

    @classmethod
    def from_random(cls, config_dict: Mapping[str, Any], seed: int, options: Optional[EngineOptions] = None,
                    std: float = 0.02, norm_std: float = 0.0) -> "Engine":
        return cls(runner=build_runner_random(config_dict, seed, options, std, norm_std))

    # ---- requests ----------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None,
                    callback: Optional[Callable[[int, bool], None]] = None, rid: Optional[int] = None) -> Request:
        """Queue a request.  `rid` lets the caller choose the request's id (one that is not in use); without it
        the engine numbers requests itself."""
        if rid is None:
            rid = self._next_id
        elif rid in self._live:
            raise ValueError(f"request id {rid} is in use")
        req = Request(rid, [int(t) for t in prompt], params or SamplingParams(), callback)
        vocab = self.runner.model.vocab_size
        bad = [t for t in req.prompt if not (0 <= t < vocab)]
        if bad:
            raise ValueError(f"token id {bad[0]} is outside the vocabulary of {vocab}")
        self.scheduler.add_request(req)
        self._live[rid] = req
        self._next_id = max(self._next_id, rid) + 1
        return req

    def abort(self, rid: int) -> Optional[Request]:
        """Give a request up, wherever it is (waiting, in the middle of its prompt, decoding): its pages and its
        slot go back at once.  Returns the request, or None when no live request has this id."""
        req = self._live.get(rid)
        if req is None:
            return None
        self._drop_prepared()
        if not self.scheduler.abort(rid):
            return None
        del self._live[rid]
        return req

    def has_unfinished(self) -> bool:
        return self.scheduler.has_unfinished()

    # ---- one step: schedule, run, sample, update ----------------------------------
    def _drop_prepared(self) -> None:
        if self._prepared is not None:
            self.runner.drop_prepared(self._prepared)
            self._prepared = None

    def _goes_on_unchanged(self, plan: Sequence[Scheduled]) -> bool:
        """True when the step after this one is known now: nobody waits, every request of the plan takes one token and
        cannot end by its length with the token this step gives it (it may still end by an end-of-sequence token)."""
        if self.scheduler.waiting or len(plan) != len(self.scheduler.running):
            return False
        top = self.runner.max_model_len
        return all(s.num_tokens == 1 and s.sample and len(s.request.output) + 1 < s.request.params.max_new_tokens
                   and s.request.length + 1 < top for s in plan)

    def step(self) -> list[tuple[Request, int, bool]]:
        plan = self.scheduler.schedule()
        prep, self._prepared = self._prepared, None
        if prep is not None and not (plan and prep.rids == [s.request.rid for s in plan]
                                     and prep.starts == [s.start for s in plan] and all(s.num_tokens == 1 and s.sample for s in plan)):
            self.runner.drop_prepared(prep)              # the plan is another than the one foreseen
            prep = None
        if not plan:
            return []
        if prep is not None:
            logits = self.runner.finish_prepared(prep, [s.request.tokens[s.start] for s in plan])
        else:
            entries = []
            for s in plan:
                toks = s.request.tokens[s.start:s.start + s.num_tokens]
                entries.append(StepEntry(s.request.rid, toks, (s.num_tokens - 1,) if s.sample else ()))
            logits = self.runner.step(entries)
        sampled: list[int] = []
        if logits is not None:
            who = [s.request for s in plan if s.sample]
            pending = self.sampler.launch(logits, [r.params for r in who], [len(r.output) for r in who])
            # While the GPU works on this step, the host side of the next one, where it is known already: the
            # scheduler's plan for it, its pages, its positions and tables; only the token ids are missing.
            if self._goes_on_unchanged(plan):
                self._prepared = self.runner.prepare_decode([s.request.rid for s in plan], [True] * len(plan))
            sampled = self.sampler.collect(pending)
        events = self.scheduler.update(plan, sampled)
        if self._prepared is not None and any(done for _, _, done in events):
            self._drop_prepared()                        # somebody met an end-of-sequence token
        for req, tok, done in events:
            if done:
                self._live.pop(req.rid, None)
            if req.callback is not None:
                try:
                    req.callback(tok, done)
                except Exception as e:
                    if self.on_callback_error is None:
                        raise
                    self.on_callback_error(req, e)
        return events

    def generate(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams] | None = None
                 ) -> list[list[int]]:
        """Generate for all prompts together; returns the new tokens of each."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        while self.scheduler.has_unfinished():
            self.step()
        return [r.output for r in reqs]

    def stats(self) -> dict[str, int]:
        sch = self.scheduler
        pools = self.runner.manager.pools
        return {"steps": sch.num_steps, "scheduled_tokens": sch.num_scheduled_tokens, "preemptions": sch.num_preemptions,
                "waiting": len(sch.waiting), "running": len(sch.running),
                "free_pages": min(p.num_free for p in pools) if pools else 0,
                "page_high_water": max(p.high_water for p in pools) if pools else 0}


class AsyncEngine:
    """A background thread runs the engine loop; requests are added, and given up, from any thread
    (src/async_engine.cc:38-168 of lucciola: queue under a mutex, condition variable, per-token callback
    on the engine thread, stop() joins the thread after the work is done).

    What lucciola's engine lacks and this one has: `abort(id)`, `stats()`, an id that names the request in the
    scheduler too, and a callback that raises ends its own request only (the exception is kept in
    `callback_errors`), not the loop."""

    def __init__(self, model_path: Optional[str | Path] = None, max_blocks: int = 0, block_size: int = 16,
                 engine: Optional[Engine] = None, **kw: Any):
        self.engine = engine or Engine(model_path, max_blocks, block_size, **kw)
        self.engine.on_callback_error = self._callback_failed
        self._cv = threading.Condition()
        self._pending: list[tuple[int, list[int], SamplingParams, Optional[Callable[[int, bool], None]]]] = []
        self._aborts: list[int] = []
        self._stop = False
        self._next_id = 1
        self._error: Optional[BaseException] = None
        self.callback_errors: list[tuple[int, BaseException]] = []
        self.num_submitted = self.num_aborted = self.num_refused = 0
        self._thread = threading.Thread(target=self._loop, name="lucciola-engine", daemon=True)
        self._thread.start()

    def submit(self, prompt: Sequence[int], params: SamplingParams,
               callback: Optional[Callable[[int, bool], None]] = None) -> int:
        """Queue a request; returns its id at once.  `callback(token, is_finished)` runs on the engine's thread for
        every generated token; a request that is refused (too long for the model or the pool) or given up gets one
        call `callback(-1, True)`."""
        params.validate()
        with self._cv:
            if self._stop:
                raise RuntimeError("the engine is stopped")
            rid = self._next_id
            self._next_id += 1
            self.num_submitted += 1
            self._pending.append((rid, [int(t) for t in prompt], params, callback))
            self._cv.notify()
        return rid

    def generate_async(self, prompt: Sequence[int], max_new_tokens: int,
                       callback: Optional[Callable[[int, bool], None]] = None, temperature: float = 0.0,
                       seed: int = 0, ignore_eos: bool = False) -> int:
        """lucciola's call: submit with the sampling parameters spelled out."""
        return self.submit(prompt, SamplingParams(max_new_tokens=max_new_tokens, temperature=temperature, seed=seed,
                                                  ignore_eos=ignore_eos), callback)

    def abort(self, rid: int) -> None:
        """Give request `rid` up.  Takes effect between two steps of the engine: what the request holds goes back
        and its callback is called once more, with (-1, True).  An id that is unknown or already finished is ignored."""
        with self._cv:
            self._aborts.append(rid)
            self._cv.notify()

    def stats(self) -> dict[str, int]:
        """Counters of the scheduler and of this queue (a snapshot; the engine's thread keeps running)."""
        out = dict(self.engine.stats())
        with self._cv:
            out.update(queued=len(self._pending), submitted=self.num_submitted, aborted=self.num_aborted,
                       refused=self.num_refused, callback_errors=len(self.callback_errors))
        return out

    def stop(self) -> None:
        """Finish what was submitted, then end the thread."""
        with self._cv:
            if self._stop:
                return
            self._stop = True
            self._cv.notify_all()
        self._thread.join()
        if self._error is not None:
            raise self._error

    # ---- the engine's thread ---------------------------------------------------
    def _callback_failed(self, req: Request, error: BaseException) -> None:
        self.callback_errors.append((req.rid, error))
        if self.engine.abort(req.rid) is not None:       # nobody listens any more: stop working for it
            self.num_aborted += 1

    def _call(self, rid: int, cb: Optional[Callable[[int, bool], None]], token: int, finished: bool) -> None:
        if cb is None:
            return
        try:
            cb(token, finished)
        except Exception as e:
            self.callback_errors.append((rid, e))

    def _loop(self) -> None:
        eng = self.engine
        torch.cuda.set_device(eng.runner.device)
        try:
            while True:
                with self._cv:
                    self._cv.wait_for(lambda: self._stop or self._pending or self._aborts or eng.has_unfinished())
                    if self._stop and not self._pending and not eng.has_unfinished():
                        return
                    batch, self._pending = self._pending, []
                    aborts, self._aborts = self._aborts, []
                for rid, prompt, params, cb in batch:
                    if rid in aborts:                     # given up before it was ever queued in the scheduler
                        self.num_aborted += 1
                        self._call(rid, cb, -1, True)
                        continue
                    try:
                        eng.add_request(prompt, params, cb, rid=rid)
                    except ValueError:
                        self.num_refused += 1
                        self._call(rid, cb, -1, True)     # refused: finished without a token
                for rid in aborts:
                    req = eng.abort(rid)
                    if req is not None:
                        self.num_aborted += 1
                        self._call(rid, req.callback, -1, True)
                if eng.has_unfinished():
                    eng.step()
        except BaseException as e:                       # surfaces in stop()
            self._error = e
