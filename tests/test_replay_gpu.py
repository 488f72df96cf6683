"""The engine against the plain implementation under every way of cutting the work (GPU)."""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import replay_util as ru
from conftest import ROOT, TINY, tokens_for

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]


def make_runner(folder, name, dtype, num_pages, graphs=False, **kw):
    """`graphs`: every step whose shape allows it is recorded as a CUDA graph the first time its shape comes and
    replayed from then on."""
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner

    page = TINY[name][4]
    return build_runner(folder, EngineOptions(dtype=dtype, block_size=page, max_blocks=num_pages, max_num_seqs=8,
                                              use_cuda_graph=graphs, graph_after=1, max_shape_graphs=1000, **kw),
                        num_pages=num_pages)


def requests_for(name):
    """Four requests per configuration (the prompt lengths of the tiny workloads among them), up to the
    configuration's longest sequence."""
    top = TINY[name][0]["max_position_embeddings"]
    lengths = {"A": [5, 17, 33, 128], "B": [1, 9, 40, 100, 256], "C": [3, 64, 200, 333], "D": [2, 31, 150, 400]}[name]
    assert max(lengths) <= top
    return {f"{name}{n}": tokens_for(name, n) for n in lengths}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(TINY))
@pytest.mark.parametrize("cut", ["whole", "tail_decoded", "portions"])
def test_each_request_alone(tiny_models, name, dtype, cut):
    reqs = requests_for(name)
    steps = getattr(ru, cut)(reqs)
    page = TINY[name][4]
    runner = make_runner(tiny_models[name], name, dtype, ru.max_live_tokens(steps) // page)
    got = ru.replay(runner, steps)
    ru.compare(got, tiny_models[name], reqs, dtype)
    assert all(p.num_free == p.num_pages for p in runner.manager.pools)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(TINY))
@pytest.mark.parametrize("seed", [0, 1])
def test_mixed_batches_with_reused_pages(tiny_models, name, dtype, seed):
    top = TINY[name][0]["max_position_embeddings"]
    lengths = [n for n in (70, 9, 120, 33, 101, 2, 64, 47, 90) if n <= top]
    reqs = {f"m{i}": tokens_for(name, n, salt=seed + 1) for i, n in enumerate(lengths)}
    steps = ru.mixed(reqs, seed=seed)
    page = TINY[name][4]
    pages = ru.max_live_tokens(steps) // page
    assert pages * page < sum(ru.ceil64(len(v)) for v in reqs.values()), "the trace must force pages to be used again"
    runner = make_runner(tiny_models[name], name, dtype, pages)
    got = ru.replay(runner, steps, poison=True)
    ru.compare(got, tiny_models[name], reqs, dtype)
    assert max(len(s["entries"]) for s in steps) >= 3
    assert any(len(e["tokens"]) == 1 for s in steps for e in s["entries"]) and any(len(e["tokens"]) > 1 for s in steps for e in s["entries"])


@pytest.mark.parametrize("name", list(TINY))
@pytest.mark.parametrize("cut", ["whole", "tail_decoded", "portions", "mixed", "mixed_decodes_first"])
def test_every_cutting_through_recorded_graphs(tiny_models, name, cut):
    """The same four families with recordings on (bfloat16; the 32-bit path records nothing): the trace runs twice
    through one runner.  The first pass records a CUDA graph for every shape of step it meets, the second replays
    them with other pages under the same requests; both passes are compared with the plain implementation."""
    top = TINY[name][0]["max_position_embeddings"]
    if cut.startswith("mixed"):
        lengths = [n for n in (70, 9, 120, 33, 101, 2, 64, 47, 90) if n <= top]
        reqs = {f"m{i}": tokens_for(name, n, salt=5) for i, n in enumerate(lengths)}
        steps = ru.mixed(reqs, seed=4, decodes_first=cut.endswith("first"))
    else:
        reqs = requests_for(name)
        steps = getattr(ru, cut)(reqs)
    page = TINY[name][4]
    runner = make_runner(tiny_models[name], name, "bfloat16", ru.max_live_tokens(steps) // page, graphs=True)
    assert runner._can_record
    first = ru.replay(runner, steps, poison=True)
    ru.compare(first, tiny_models[name], reqs, "bfloat16")
    recorded, replays = len(runner._graphs), runner.graph_replays
    assert recorded > 0
    second = ru.replay(runner, steps, poison=True)
    ru.compare(second, tiny_models[name], reqs, "bfloat16")
    assert len(runner._graphs) == recorded, "the second pass met a shape the first had not"
    assert runner.graph_replays - replays == sum(1 for s in steps if s["entries"]), "a step of the second pass was not a replay"
    if cut == "mixed_decodes_first":
        assert any(k[0] and k[1] for k in runner._graphs), "no step of single tokens beside a portion"
    assert all(p.num_free == p.num_pages for p in runner.manager.pools)


@pytest.mark.parametrize("dtype", DTYPES)
def test_cutting_does_not_change_float32_results_at_all(tiny_models, dtype):
    """In 32-bit every kernel visits a sum's terms in an order that does not depend on the batch, so
    whole, portions and mixed agree to the last bit; in bfloat16 they agree within rounding."""
    name = "B"
    reqs = requests_for(name)
    runs = []
    for steps in (ru.whole(reqs), ru.portions(reqs), ru.mixed(reqs, seed=3)):
        runner = make_runner(tiny_models[name], name, dtype, 200)
        runs.append(ru.replay(runner, steps))
    common = set(runs[0]) & set(runs[1]) & set(runs[2])
    assert len(common) > 50
    for key in common:
        for other in runs[1:]:
            if dtype == "float32":
                assert torch.equal(runs[0][key], other[key]), key
            else:
                assert (runs[0][key] - other[key]).abs().max() <= 2 * ru.TOL[dtype] * runs[0][key].abs().max(), key


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(tiny_models, dtype):
    """One prompt token, then every token decoded one by one up to the longest sequence of the configuration."""
    name = "C"
    ids = tokens_for(name, 400, salt=9)
    steps = ru.tail_decoded({"long": ids}, tail=399)
    runner = make_runner(tiny_models[name], name, dtype, ru.max_live_tokens(steps) // 16)
    got = ru.replay(runner, steps)
    assert len(got) == 400
    ru.compare(got, tiny_models[name], {"long": ids}, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(TINY))
def test_first_tokens_of_a_sequence(tiny_models, name, dtype):
    """Positions 0, 1, 2: a single key, a page that holds one token, a one-token prompt."""
    for n in (1, 2, 3):
        ids = tokens_for(name, n, salt=n)
        for steps in (ru.whole({"f": ids}), ru.tail_decoded({"f": ids}, tail=n - 1) if n > 1 else ru.whole({"f": ids})):
            runner = make_runner(tiny_models[name], name, dtype, 8)
            ru.compare(ru.replay(runner, steps), tiny_models[name], {"f": ids}, dtype)


@pytest.mark.parametrize("dtype,graphs", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
def test_trace_run_program(tiny_models, tmp_path, dtype, graphs):
    """The program itself, as a user runs it: steps on standard input, <step>.f32 files out; also with --cuda-graph,
    which records every shape of step at its first coming."""
    name = "A"
    reqs = {"a": tokens_for(name, 70), "b": tokens_for(name, 33, salt=1), "c": tokens_for(name, 90, salt=2)}
    steps = ru.mixed(reqs, seed=5, max_live=2)
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(tiny_models[name]), "--dtype", dtype,
                        "--out", str(out), "--max-tokens", str(ru.max_live_tokens(steps))] + (["--cuda-graph"] if graphs else []),
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    vocab = TINY[name][0]["vocab_size"]
    got, held = {}, {}
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        f = out / f"{s['step']}.f32"
        assert f.exists() == (wanted > 0)
        rows = np.fromfile(f, dtype="<f4").reshape(wanted, vocab) if wanted else None
        r = 0
        for e in s["entries"]:
            start = held.get(e["id"], 0)
            for w in e["want"]:
                got[(e["id"], start + w)] = torch.from_numpy(rows[r].astype(np.float64)); r += 1
            held[e["id"]] = start + len(e["tokens"])
    ru.compare(got, tiny_models[name], reqs, dtype)


def test_step_refuses_bad_input(tiny_models):
    from lucciola_b200.engine.step import OutOfPages, StepEntry
    runner = make_runner(tiny_models["A"], "A", "float32", 4)
    with pytest.raises(ValueError, match="outside the vocabulary"):
        runner.step([StepEntry("x", [1, 256], [0])])
    with pytest.raises(ValueError, match="twice"):
        runner.step([StepEntry("x", [1], []), StepEntry("x", [2], [])])
    with pytest.raises(ValueError, match="place 3"):
        runner.step([StepEntry("x", [1, 2], [3])])
    with pytest.raises(ValueError, match="limit is 128"):
        runner.step([StepEntry("x", [1] * 129, [])])
    with pytest.raises(OutOfPages):
        runner.step([StepEntry("x", [1] * 65, [])])
    assert runner.manager.num_requests() == 0 and runner.manager.pools[0].num_free == 4     # nothing was taken
    assert runner.step([StepEntry("x", [1] * 64, [])]) is None


@pytest.mark.parametrize("name", list(TINY))
def test_short_portions_replayed_from_recordings(tiny_models, name):
    """A step that is one short portion of one request is recorded as a CUDA graph the second time its size comes: whole
    short prompts of one length and ends of longer prompts, each against the plain implementation; the later ones are replays
    (other requests, other pages, other positions than the step that was recorded)."""
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner

    page = TINY[name][4]
    runner = build_runner(tiny_models[name], EngineOptions(dtype="bfloat16", block_size=page, max_blocks=64, max_num_seqs=8,
                                                           use_cuda_graph=True, graph_after=2), num_pages=64)
    reqs = {f"s{i}": tokens_for(name, 17, salt=20 + i) for i in range(4)}
    steps = ru.whole(reqs)
    # longer prompts in portions of 60 and 9 tokens (and a rest of 0, 1 or 2): the same sizes at other positions
    longer = {f"l{i}": tokens_for(name, 69 + i, salt=30 + i) for i in range(3)}
    for rid, ids in longer.items():
        n = len(steps)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": ids[:60], "want": [59]}], "end": []})
        steps.append({"step": n + 1, "entries": [{"id": rid, "tokens": ids[60:69], "want": list(range(9))}], "end": []})
        if len(ids) > 69:
            steps.append({"step": n + 2, "entries": [{"id": rid, "tokens": ids[69:], "want": list(range(len(ids) - 69))}], "end": []})
        steps[-1]["end"] = [rid]
    # a portion of which no logits are wanted, then the rest
    quiet = {f"q{i}": tokens_for(name, 45, salt=40 + i) for i in range(3)}
    for rid, ids in quiet.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[:30], "want": []}], "end": []})
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": ids[30:], "want": list(range(15))}], "end": [rid]})
    got = ru.replay(runner, steps)
    ru.compare(got, tiny_models[name], {**reqs, **longer, **quiet}, "bfloat16")
    short = {(k[1], k[3]) for k in runner._graphs if not k[0] and k[2] == 256}
    assert ((30,), ("none",)) in short and ((15,), ("all",)) in short, short
    assert ((17,), ("all",)) in short and ((9,), ("all",)) in short and ((60,), ("last",)) in short, short
