"""Traces in the format of bin/trace_run, made four ways, and the comparison of what the engine
returns for them with the plain implementation."""
from __future__ import annotations

import random

import torch

import plain_qwen3 as plain

# Largest allowed |engine - plain| as a fraction of the largest |logit| of the sequence.  float32: a
# few units of its rounding (2^-24 = 6e-8) times the length of the sums; bfloat16: activations are
# rounded to 8 bits (2^-9 = 2e-3 each) between all kernels of up to four layers; the largest error these tests
# have measured is 1e-2, and the bound is twice that.
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def ceil64(n: int) -> int:
    return -(-n // 64) * 64


def whole(reqs: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole, logits at every position."""
    return [{"step": i, "entries": [{"id": rid, "tokens": ids, "want": list(range(len(ids)))}], "end": [rid]}
            for i, (rid, ids) in enumerate(reqs.items())]


def tail_decoded(reqs: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of each request in one step, its last `tail` tokens one by one."""
    steps = []
    for rid, ids in reqs.items():
        head = max(len(ids) - tail, 1)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[:head], "want": [head - 1]}], "end": []})
        for p in range(head, len(ids)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [ids[p]], "want": [0]}],
                          "end": [rid] if p == len(ids) - 1 else []})
        if head == len(ids):
            steps[-1]["end"] = [rid]
    return steps


def portions(reqs: dict[str, list[int]], sizes=(7, 2, 13, 3, 2, 31, 1, 16, 2, 17, 5)) -> list[dict]:
    """Each request in portions of changing size, down to two tokens (and one)."""
    steps = []
    for rid, ids in reqs.items():
        pos, i = 0, 0
        while pos < len(ids):
            n = min(sizes[i % len(sizes)], len(ids) - pos)
            i += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[pos:pos + n], "want": list(range(n))}],
                          "end": [rid] if pos + n == len(ids) else []})
            pos += n
    return steps


def mixed(reqs: dict[str, list[int]], seed: int = 0, max_live: int = 4, decodes_first: bool = False) -> list[dict]:
    """Up to four live requests: portions of some beside single tokens of others; requests start while
    others run, may sit out a step, and end at different times, so that their pages are used again.
    `decodes_first` lists a step's single tokens before its portions, as a scheduler does."""
    rng = random.Random(seed)
    queue = list(reqs)
    pos: dict[str, int] = {}
    steps = []
    while queue or pos:
        while queue and len(pos) < max_live and (not pos or rng.random() < 0.5):
            pos[queue.pop(0)] = 0
        entries, end = [], []
        live = list(pos)
        rng.shuffle(live)
        for k, rid in enumerate(live):
            ids = reqs[rid]
            if k > 0 and rng.random() < 0.2:
                continue                                   # left out of this step, goes on later
            left = len(ids) - pos[rid]
            decoding = left <= min(24, len(ids) // 2)
            n = 1 if decoding else min(left, rng.choice([2, 3, 5, 7, 11, 16, 17, 29]))
            want = list(range(n)) if n <= 3 or rng.random() < 0.5 else sorted(rng.sample(range(n), 2))
            entries.append({"id": rid, "tokens": ids[pos[rid]:pos[rid] + n], "want": want})
            pos[rid] += n
            if pos[rid] == len(ids):
                end.append(rid)
        for rid in end:
            del pos[rid]
        if decodes_first:
            entries.sort(key=lambda e: len(e["tokens"]) > 1)
        steps.append({"step": len(steps), "entries": entries, "end": end})
    return steps


def max_live_tokens(steps: list[dict]) -> int:
    """--max-tokens for a trace: the most tokens live requests hold at any time, each rounded up to 64."""
    held: dict[str, int] = {}
    most = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        most = max(most, sum(ceil64(n) for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return most


def replay(runner, steps: list[dict], poison: bool = False) -> dict[tuple[str, int], torch.Tensor]:
    """Run a trace through a runner; returns the logits row for each (request, position) asked for."""
    from lucciola_b200.engine.step import StepEntry

    out: dict[tuple[str, int], torch.Tensor] = {}
    for s in steps:
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in s["entries"]]
        starts = {e.rid: runner.length(e.rid) for e in entries}
        logits = runner.step(entries) if entries else None
        if logits is not None:
            rows = logits.detach().double().cpu()
            r = 0
            for e in entries:
                for w in e.want:
                    out[(e.rid, starts[e.rid] + w)] = rows[r]
                    r += 1
        for rid in s["end"]:
            tables = [list(runner.manager.block_table(rid, g)) for g in range(len(runner.groups))]
            runner.finish(rid)
            if poison:                                     # what a freed page still holds must never matter
                for g, t in enumerate(tables):
                    runner.cache.poison_pages(g, [p for p in t if p >= 0])
        runner.manager.check_invariants()
    return out


_plain_cache: dict = {}


def plain_logits(folder, ids: list[int]) -> torch.Tensor:
    key = (str(folder), tuple(ids))
    if key not in _plain_cache:
        cfg, w = plain.read_model(folder)
        _plain_cache[key] = plain.forward(cfg, w, ids)
    return _plain_cache[key]


def compare(got: dict[tuple[str, int], torch.Tensor], folder, reqs: dict[str, list[int]], dtype: str) -> float:
    """Largest error relative to the sequence's largest logit; asserts it is within TOL and names the
    first position that is not."""
    worst = 0.0
    assert got, "the trace asked for no logits"
    for rid, ids in reqs.items():
        ref = plain_logits(folder, ids)
        scale = ref.abs().max().item()
        for p in range(len(ids)):
            if (rid, p) not in got:
                continue
            row = got[(rid, p)]
            assert torch.isfinite(row).all(), f"request {rid} position {p}: logits are not finite"
            err = (row - ref[p]).abs().max().item() / scale
            assert err <= TOL[dtype], f"request {rid}: first wrong position {p} (error {err:.3g} of scale, allowed {TOL[dtype]:.3g})"
            worst = max(worst, err)
    return worst
