"""The step function's host side without a GPU: what it packs for the device, how it pads a step that is recorded,
and that a replayed recording reads this step's values, not those of the step that was recorded.

The model is a stand-in defined here whose "logits" at a row are the integers the step function handed it for that
row (token, position, context length, first page, state slot), so every mistake of packing shows in the output.  A
recording is emulated by keeping the StepContext of the recorded step: its tensors are views of the recording's
input buffer, which is what the kernels of a CUDA graph read."""
import random

import numpy as np
import pytest
import torch

from lucciola_b200.config import EngineOptions
from lucciola_b200.engine import step as step_mod
from lucciola_b200.engine.step import ModelRunner, StepEntry
from lucciola_b200.parts.base import BatchShape, KVPages, Mixer, Part, Runtime, StateSlot, StepPlan

VOCAB = 1000


class CountingMixer(Mixer):
    """Plans, for each request of the step, (first token, tokens, start position, 0): forward() checks that what
    arrives on the "device" is the plan of this very step."""
    recordable = True

    def __init__(self, state: bool):
        self.state = state
        self.plans_made = 0

    def cache_request(self):
        return StateSlot((3,), torch.float32) if self.state else KVPages(2, 16, 0)

    def plan_key(self):
        return "counting"

    def plan(self, batch: BatchShape) -> StepPlan:
        self.plans_made += 1
        first = np.concatenate(([0], np.cumsum(batch.q_lens)[:-1]))
        items = np.stack([first, batch.q_lens, batch.start_positions, np.zeros_like(first)], axis=1).astype(np.int32)
        return StepPlan({"items": items, "odd": np.arange(5, dtype=np.int32)}, {"requests": len(batch.q_lens)})


class Block(Part):
    recordable = True

    def __init__(self, mixer):
        self.mixer = mixer

    def children(self):
        return [self.mixer]


class StandInModel(Part):
    recordable = True
    vocab_size, max_positions = VOCAB, 4096

    def __init__(self, state: bool = False):
        self.blocks = [Block(CountingMixer(state)), Block(CountingMixer(state))]
        self.state = state
        self.eos_token_ids = ()

    def children(self):
        return self.blocks

    def cache_requests(self):
        return [b.mixer.cache_request() for b in self.blocks]

    def forward(self, tok, step, caches, rows):
        plan = step.plans["counting"]
        items = plan.arrays["items"]
        assert plan.host["requests"] == step.num_seqs == items.shape[0]
        assert plan.arrays["odd"].tolist() == [0, 1, 2, 3, 4]
        assert items.data_ptr() % 16 == 0 and plan.arrays["odd"].data_ptr() % 16 == 0
        cu = step.cu_tokens.tolist()
        assert cu[0] == 0 and cu[-1] == step.num_tokens == tok.shape[0]
        for j in range(step.num_seqs):
            a, b = cu[j], cu[j + 1]
            assert items[j].tolist()[:2] == [a, b - a]
            assert (step.token_seq[a:b] == j).all()
            start = int(items[j, 2])
            assert step.positions[a:b].tolist() == list(range(start, start + b - a))
            assert int(step.context_lens[j]) == start + b - a
            table = step.block_tables[0][j] if step.block_tables else None
            if table is not None:
                pages = -(-int(step.context_lens[j]) // 16)
                held = int((table >= 0).sum())
                assert held in (0, pages), (held, pages)          # an entry that pads a recording holds no page
        if rows is None:
            return None
        out = torch.zeros(rows.shape[0], 5, dtype=torch.float32)
        for r, t in enumerate(rows.tolist()):
            j = int(step.token_seq[t])
            page0 = int(step.block_tables[0][j, 0]) if step.block_tables else -7
            out[r] = torch.tensor([int(tok[t]), int(step.positions[t]), int(step.context_lens[j]), page0, int(step.state_slots[j])])
        return out


class HostStaging:
    """The staging ring without pinned memory and without a device."""

    def __init__(self, device, capacity, ring=4):
        self.capacity = capacity
        self.host_np = [np.zeros(capacity, dtype=np.int32) for _ in range(ring)]
        self.dev = torch.zeros(capacity, dtype=torch.int32)
        self.turn = 0

    def next_host(self):
        i = self.turn
        self.turn = (self.turn + 1) % len(self.host_np)
        self.host_np[i][:] = -12345                     # whatever an earlier step left must not matter
        return i, None

    def upload(self, i, n, dev=None):
        (self.dev if dev is None else dev)[:n] = torch.from_numpy(self.host_np[i][:n])


class Replayable:
    def __init__(self, runner, args):
        self.runner, self.args = runner, args
        self.out = None

    def replay(self):
        d_tok, step, d_rows, d_fresh = self.args
        result = self.runner._forward(d_tok, step, d_rows, d_fresh)
        if self.out is not None:
            self.out.copy_(result)                      # a recording writes its logits where it wrote them before


class HostRunner(ModelRunner):
    def _stream(self):
        return 0

    def _sync(self):
        pass

    def _run_and_record(self, shape, d_tok, step, d_rows, d_fresh):
        logits = self._forward(d_tok, step, d_rows, d_fresh)
        rec = Replayable(self, (d_tok, step, d_rows, d_fresh))
        rec.out = None if logits is None else logits.clone()
        self._graphs[shape] = step_mod._Recording(rec, rec.out, 7)
        return logits


@pytest.fixture
def host_runner(monkeypatch):
    monkeypatch.setattr(step_mod, "_Staging", HostStaging)
    zeroed = []

    def make(record: bool, state: bool = False, pages: int = 64, **kw):
        rt = Runtime("cpu", torch.bfloat16)
        model = StandInModel(state)
        r = HostRunner(model, rt, EngineOptions(block_size=16, max_blocks=pages, max_num_seqs=8, use_cuda_graph=record,
                                                graph_after=1, **kw), num_pages=pages)
        r._can_record = record
        r.cache.zero_slots = lambda slots, stream: zeroed.append(slots.tolist())
        r.zeroed = zeroed
        return r
    return make


def expected(runner, entries, starts):
    rows = []
    for e in entries:
        for w in e.want:
            page0 = runner.manager.block_table(e.rid, 0)[0] if runner.groups else -7
            rows.append([e.tokens[w], starts[e.rid] + w, starts[e.rid] + len(e.tokens), page0, runner.manager.slot(e.rid)])
    return torch.tensor(rows, dtype=torch.float32) if rows else None


def run_trace(runner, steps):
    for entries, end in steps:
        starts = {e.rid: runner.length(e.rid) for e in entries}
        got = runner.step(entries)
        want = expected(runner, entries, starts)
        assert (got is None) == (want is None)
        if want is not None:
            assert torch.equal(got, want), (entries, got, want)
        for rid in end:
            runner.finish(rid)
        runner.manager.check_invariants()


def random_trace(seed, steps=120):
    """Decoded tokens first, then portions (the order the scheduler gives), with requests that come and go."""
    rng = random.Random(seed)
    live, out, n_id = {}, [], 0
    for _ in range(steps):
        while len(live) < 6 and rng.random() < 0.4:
            live[f"r{n_id}"] = [rng.choice([1, 3, 20, 40, 64, 90]), 0]          # prompt length, tokens run so far
            n_id += 1
        decodes, portions, end = [], [], []
        for rid, (plen, done) in list(live.items()):
            if rng.random() < 0.15:
                continue
            if done >= plen:
                toks, want = [rng.randrange(VOCAB)], ([0] if rng.random() < 0.9 else [])
                decodes.append(StepEntry(rid, toks, want))
                live[rid][1] += 1
                if live[rid][1] >= plen + rng.choice([2, 9, 30]):
                    end.append(rid)
                    del live[rid]
            elif len(portions) < 2:
                n = min(plen - done, rng.choice([2, 5, 16, 17, 32]))
                toks = [rng.randrange(VOCAB) for _ in range(n)]
                want = rng.choice([[], [n - 1], list(range(n)), sorted(rng.sample(range(n), min(n, 2)))])
                portions.append(StepEntry(rid, toks, want))
                live[rid][1] += n
        if decodes or portions:
            out.append((decodes + portions, end))
    out[-1] = (out[-1][0], out[-1][1] + list(live))               # whoever is left ends with the trace
    return out


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_packing_is_right_with_and_without_recordings(host_runner, seed):
    trace = random_trace(seed)
    plain_run = host_runner(record=False)
    run_trace(plain_run, trace)
    assert not plain_run._graphs
    recorded = host_runner(record=True, max_shape_graphs=1000)
    run_trace(recorded, trace)
    run_trace(recorded, trace)                          # the same shapes again, other pages: every step a replay now
    assert recorded.graph_replays > len(trace)
    assert any(k[0] and k[1] for k in recorded._graphs), "no step of single tokens beside a portion was recorded"
    assert any(k[0] and not k[1] for k in recorded._graphs) and any(not k[0] and k[1] for k in recorded._graphs)


def test_a_recording_is_padded_and_computes_fixed_rows(host_runner):
    r = host_runner(record=True)
    for rid in "abc":
        r.step([StepEntry(rid, [5] * 20, [])])
    # three single tokens and a portion of 7: padded to 4 + 7 tokens; rows = 4 single tokens + the portion's last
    entries = [StepEntry("a", [1], [0]), StepEntry("b", [2], []), StepEntry("c", [3], [0]), StepEntry("d", list(range(7)), [6])]
    got = r.step(entries)
    shape = (4, (7,), 256, ("last",))
    assert shape in r._graphs and got.shape[0] == 3
    assert r._graph_inputs[shape].numel() >= 3 * 11
    # the same shape from other requests at other positions: a replay, and its values are this step's
    r.finish("b")
    entries = [StepEntry("a", [9], []), StepEntry("c", [8], [0]), StepEntry("f", [3], []), StepEntry("e", [4] * 7, [6])]
    before = r.graph_replays
    got = r.step(entries)
    assert r.graph_replays == before + 1
    assert got.tolist() == [[8, 21, 22, r.manager.block_table("c", 0)[0], r.manager.slot("c")],
                            [4, 6, 7, r.manager.block_table("e", 0)[0], r.manager.slot("e")]]
    # a single token behind a portion counts as a portion of one token: nothing is padded
    got = r.step([StepEntry("e", [1, 2], [1]), StepEntry("a", [7], [0])])
    assert (0, (2, 1), 256, ("last", "last")) in r._graphs and got[:, 0].tolist() == [2, 7]


def test_shapes_with_portions_wait_until_they_come_again_and_old_ones_go(host_runner):
    r = host_runner(record=True, max_shape_graphs=2)
    r.options.graph_after = 2
    def prompt(rid, n):
        r.step([StepEntry(rid, [1] * n, [n - 1])])
        r.finish(rid)
    prompt("a", 5)
    assert not r._graphs
    prompt("b", 5)
    assert list(r._graphs) == [(0, (5,), 256, ("last",))]
    for n in (6, 6, 7, 7):
        prompt(f"x{n}", n)
    assert [k[1] for k in r._graphs] == [(6,), (7,)]              # the recording of 5 made room
    prompt("c", 6)                                                # used again: now 7 is the oldest
    prompt("d", 8); prompt("e", 8)
    assert [k[1] for k in r._graphs] == [(6,), (8,)]
    assert set(r._graph_inputs) == set(r._graphs)
    # a long portion of which few logits are wanted is not worth a recording that computes them all
    r.options.graph_after = 1
    r.step([StepEntry("f", [1] * 100, [3, 50])])
    assert not any(k[1] == (100,) for k in r._graphs)
    r.step([StepEntry("g", [1] * 100, list(range(100)))])
    assert any(k[1] == (100,) and k[3] == ("all",) for k in r._graphs)


def test_state_slots_of_new_requests_are_cleared_inside_recordings_too(host_runner):
    r = host_runner(record=True, state=True)
    assert r.groups == [] and r.cache.states
    r.step([StepEntry("a", [1, 2, 3], [2])])
    assert r.zeroed == [[r.manager.slot("a")]]
    r.step([StepEntry("a", [4], [0])])                           # a recorded step of one token: the list names no slot
    assert r.zeroed[-1] == [-1]
    r.finish("a")
    r.step([StepEntry("b", [1, 2, 3], [2])])                     # replayed: the new request's slot is in the list
    assert r.graph_replays == 1 and r.zeroed[-1] == [r.manager.slot("b")]
    r.step([StepEntry("b", [4], [0]), StepEntry("c", [5], [0])])  # a new request of one token beside a running one
    assert r.zeroed[-1] == [-1, r.manager.slot("c")]


def test_a_step_prepared_ahead_equals_the_step_and_can_be_dropped(host_runner):
    """prepare_decode does a step's host side before its tokens are known, finish_prepared adds them and replays the
    recording; the result is that of step().  A prepared step that is dropped leaves the lengths as they were, and the
    page it may have taken serves the position's real step."""
    r = host_runner(record=True)
    for rid, n in (("a", 15), ("b", 16), ("c", 40)):
        r.step([StepEntry(rid, list(range(n)), [])])
    assert r.prepare_decode(["a", "b", "c"], [True] * 3) is None               # no recording of this size yet: nothing taken
    assert [r.length(x) for x in "abc"] == [15, 16, 40]
    r.step([StepEntry("a", [7], [0]), StepEntry("b", [8], [0]), StepEntry("c", [9], [0])])     # records the step of 4
    free = r.manager.pools[0].num_free
    prep = r.prepare_decode(["a", "b", "c"], [True, False, True])
    assert prep is not None and prep.starts == [16, 17, 41] and [r.length(x) for x in "abc"] == [17, 18, 42]
    assert r.manager.pools[0].num_free == free - 1                             # a crossed a page boundary
    got = r.finish_prepared(prep, [100, 200, 300])
    page = lambda x: r.manager.block_table(x, 0)[0]
    assert got.tolist() == [[100, 16, 17, page("a"), r.manager.slot("a")], [300, 41, 42, page("c"), r.manager.slot("c")]]
    with pytest.raises(ValueError, match="outside the vocabulary"):
        r.finish_prepared(r.prepare_decode(["a"], [True]) or r.prepare_decode(["a", "b", "c"], [True] * 3), [1, 2, VOCAB])
    r.manager.retract_by_one(["a", "b", "c"])                                   # what the failed finish left prepared
    # dropped: lengths return; the same positions then run as an ordinary step
    prep = r.prepare_decode(["a", "b", "c"], [True] * 3)
    assert [r.length(x) for x in "abc"] == [18, 19, 43]
    r.drop_prepared(prep)
    assert [r.length(x) for x in "abc"] == [17, 18, 42]
    r.manager.check_invariants()
    got = r.step([StepEntry("b", [5], [0]), StepEntry("c", [6], [0])])
    assert got[:, :3].tolist() == [[5, 18, 19], [6, 42, 43]]
    assert r.prepare_decode(["a", "zz"], [True, True]) is None                  # an unknown request
    for x in "abc":
        r.finish(x)
    r.manager.check_invariants()
    assert r.manager.pools[0].num_free == r.manager.pools[0].num_pages


def test_a_part_that_cannot_be_recorded_keeps_the_model_from_recordings(monkeypatch):
    monkeypatch.setattr(step_mod, "_Staging", HostStaging)
    model = StandInModel()
    model.blocks[1].mixer.recordable = False
    rt = Runtime("cpu", torch.bfloat16)
    rt.fast_kernels = True
    r = HostRunner(model, rt, EngineOptions(block_size=16, max_blocks=8, max_num_seqs=4), num_pages=8)
    assert not r._can_record
    assert Part.recordable is False                               # what a part defined elsewhere is taken for
