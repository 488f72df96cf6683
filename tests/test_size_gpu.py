"""The production kernel paths at the real layer sizes (hidden 4096, 32 query heads, 8 kv heads, head 128,
intermediate 12288; two layers and a smaller vocabulary to stay quick): the bfloat16 engine against the
float32 engine of the same weights, under different ways of cutting the work (GPU).

The tiny models cannot reach these paths: the persistent tensor-core product for hundreds of tokens, split
products in thread-block clusters, 64-row attention tiles of four query heads, decoded tokens whose key
ranges are combined inside a cluster, CUDA graphs."""
import pytest
import torch

import replay_util as ru

pytestmark = pytest.mark.gpu
BF16_TOL = ru.TOL["bfloat16"]

CFG = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "intermediate_size": 12288, "vocab_size": 20000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 4096, "hidden_act": "silu", "attention_bias": False,
}


@pytest.fixture(scope="module")
def runners():
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner_random
    out = {}
    for dtype in ("float32", "bfloat16"):
        opts = EngineOptions(dtype=dtype, block_size=16, max_blocks=600, max_num_seqs=8, max_model_len=4096,
                             max_tokens_per_step=4096)
        out[dtype] = build_runner_random(CFG, seed=3, options=opts, std=0.02, norm_std=0.05)
    # the same bfloat16 values in both: the float32 engine widens them exactly
    a, b = out["float32"].model, out["bfloat16"].model
    assert torch.equal(a.blocks[1].mixer.qkv.weight, b.blocks[1].mixer.qkv.weight.float())
    return out


def logits_of(runner, ids, cuts, tail=0):
    """Feed `ids` in portions given by `cuts` (then `tail` tokens one by one); logits at every position."""
    from lucciola_b200.engine.step import StepEntry
    rows, pos = [], 0
    for n in cuts:
        rows.append(runner.step([StepEntry("r", ids[pos:pos + n], list(range(n)))]).float().cpu())
        pos += n
    for _ in range(tail):
        rows.append(runner.step([StepEntry("r", [ids[pos]], [0])]).float().cpu().clone())
        pos += 1
    assert pos == len(ids)
    runner.finish("r")
    return torch.cat(rows)


def test_bfloat16_engine_against_float32_engine_at_real_layer_sizes(runners):
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, CFG["vocab_size"], (700,), generator=g).tolist()
    ref = logits_of(runners["float32"], ids, [700])
    scale = ref.abs().max().item()
    # float32: cutting changes nothing at all
    again = logits_of(runners["float32"], ids, [300, 17, 200, 150], tail=33)
    assert torch.equal(again, ref)
    # bfloat16: whole, in portions (a portion of 2 tokens among them), and with a decoded tail that goes
    # through recorded graphs; all within the bound of the tiny models' tests
    for cuts, tail in (([700], 0), ([300, 17, 2, 198, 150], 33), ([640], 60)):
        got = logits_of(runners["bfloat16"], ids, cuts, tail)
        err = ((got - ref).abs().max() / scale).item()
        assert torch.isfinite(got).all() and err < BF16_TOL, (cuts, tail, err)
        agree = (got.argmax(-1) == ref.argmax(-1)).float().mean().item()
        assert agree > 0.9, (cuts, tail, agree)
    assert len(runners["bfloat16"]._graphs) > 0


def test_short_prompts_replayed_from_recordings_at_real_layer_sizes(runners):
    """Three prompts of 36 tokens one after the other: the second is recorded as a CUDA graph (q|k|v product, rotation,
    tensor-memory attention and all), the third replays it with other tokens and other pages."""
    g = torch.Generator().manual_seed(5)
    before = len([k for k in runners["bfloat16"]._graphs if k[1]])
    for _ in range(3):
        ids = torch.randint(0, CFG["vocab_size"], (36,), generator=g).tolist()
        ref = logits_of(runners["float32"], ids, [36])
        got = logits_of(runners["bfloat16"], ids, [36])
        err = ((got - ref).abs().max() / ref.abs().max()).item()
        assert torch.isfinite(got).all() and err < BF16_TOL, err
    assert len([k for k in runners["bfloat16"]._graphs if k[1]]) == before + 1
    # 300 tokens: the many-token product kernel and several attention work items in a recording
    for _ in range(3):
        ids = torch.randint(0, CFG["vocab_size"], (300,), generator=g).tolist()
        ref = logits_of(runners["float32"], ids, [300])
        got = logits_of(runners["bfloat16"], ids, [300])
        err = ((got - ref).abs().max() / ref.abs().max()).item()
        assert torch.isfinite(got).all() and err < BF16_TOL, err
    assert (0, (300,), 512, ("all",)) in runners["bfloat16"]._graphs


def test_mixed_batch_at_real_layer_sizes(runners):
    """Up to five live requests: long portions, portions of a few tokens and decoded tokens side by side (each kind
    goes to its own attention launch), long contexts beside short ones."""
    from lucciola_b200.engine.step import StepEntry
    g = torch.Generator().manual_seed(1)
    lens = {"a": 900, "b": 140, "c": 517, "d": 45, "e": 19}
    ids = {k: torch.randint(0, CFG["vocab_size"], (n,), generator=g).tolist() for k, n in lens.items()}
    outs = {}
    for dtype in ("float32", "bfloat16"):
        r = runners[dtype]
        got = {}
        r.step([StepEntry("a", ids["a"][:800], []), StepEntry("b", ids["b"][:100], [])])
        steps = [
            [("a", 800, 850), ("b", 100, 101), ("c", 0, 300), ("e", 0, 7)],          # a few tokens beside long portions
            [("a", 850, 851), ("b", 101, 102), ("c", 300, 517), ("d", 0, 39), ("e", 7, 12)],
            [("a", 851, 900), ("b", 102, 130), ("d", 39, 40), ("e", 12, 13)],
            [("b", 130, 131), ("d", 40, 41), ("e", 13, 19)],                          # decoded tokens beside a few tokens only
        ]
        for step in steps:
            entries = [StepEntry(k, ids[k][s:e], list(range(e - s))) for k, s, e in step]
            logits = r.step(entries).float().cpu()
            o = 0
            for k, s, e in step:
                got[(k, s)] = logits[o:o + e - s]; o += e - s
        for k in lens:
            r.finish(k)
        outs[dtype] = got
    for key, ref in outs["float32"].items():
        err = ((outs["bfloat16"][key] - ref).abs().max() / ref.abs().max()).item()
        assert err < BF16_TOL, (key, err)


def test_float32_engine_against_the_plain_implementation_at_real_layer_sizes(runners):
    """The 32-bit kernels at hidden 4096, heads of 128 in groups of four: whole and in two portions against the plain
    implementation (float32 on the CPU, the same weights drawn by name from the same seed)."""
    import plain_qwen3 as plain
    from lucciola_b200.weights.random_init import RandomWeights
    r = runners["float32"]
    src = RandomWeights(r.model.all_param_specs(), 3, 0.02, 0.05, torch.bfloat16, "cuda:0")   # as the fixture drew them
    weights = {n: src.get(n).float().cpu() for n in src.names()}
    assert torch.equal(weights["model.layers.1.self_attn.o_proj.weight"], r.model.blocks[1].mixer.o.weight.cpu())
    g = torch.Generator().manual_seed(7)
    ids = torch.randint(0, CFG["vocab_size"], (200,), generator=g).tolist()
    want = plain.forward(CFG, weights, ids, dtype=torch.float32)
    scale = want.abs().max().item()
    for cuts in ([200], [131, 69]):
        got = logits_of(r, ids, cuts)
        err = ((got - want).abs().max() / scale).item()
        assert err < 2e-5, (cuts, err)              # two float32 computations of sums of 12288 terms


def test_decode_batches_that_are_no_bucket_through_recordings(runners):
    """3 and 5 requests at different context lengths decode 20 steps: the recordings are those of 4 and 8 requests,
    the missing ones are entries without pages (at head size 128 these pass the q|k|v product's epilogue and the
    decode attention kernel with a page id of -1); against the float32 engine, step by step."""
    from lucciola_b200.engine.step import StepEntry
    g = torch.Generator().manual_seed(11)
    for count, bucket in ((3, 4), (5, 8)):
        lens = [37, 300, 129, 1000, 16][:count]
        prompts = [torch.randint(0, CFG["vocab_size"], (n,), generator=g).tolist() for n in lens]
        feed = torch.randint(0, CFG["vocab_size"], (20, count), generator=g).tolist()
        outs = {}
        for dtype in ("float32", "bfloat16"):
            r = runners[dtype]
            for i, p in enumerate(prompts):
                r.step([StepEntry(("n", i), p, [])])
            replays = r.graph_replays
            rows = [r.step([StepEntry(("n", i), [feed[t][i]], [0]) for i in range(count)]).float().cpu().clone() for t in range(20)]
            outs[dtype] = torch.stack(rows)
            for i in range(count):
                r.finish(("n", i))
            if dtype == "bfloat16":
                assert any(k[0] == bucket and not k[1] for k in r._graphs) and r.graph_replays - replays >= 18
        ref, got = outs["float32"], outs["bfloat16"]
        err = ((got - ref).abs().amax(dim=(1, 2)) / ref.abs().amax(dim=(1, 2))).max().item()
        assert torch.isfinite(got).all() and err < BF16_TOL, (count, err)


def test_a_decode_step_at_real_layer_sizes_is_five_kernels_a_layer(runners):
    """The fused paths are what runs, not a fallback: a recorded decode step of 8 requests holds, per layer, the q|k|v
    product (heads finished in its epilogue), attention, the o product, the gate|up product and the down product (the adds
    and norms between them inside their epilogues), plus embedding, first norm, final norm and output head."""
    from lucciola_b200.engine.step import StepEntry
    r = runners["bfloat16"]
    g = torch.Generator().manual_seed(19)
    for i in range(8):
        r.step([StepEntry(("k", i), torch.randint(0, CFG["vocab_size"], (50 + 7 * i,), generator=g).tolist(), [])])
    one = lambda: r.step([StepEntry(("k", i), [int(torch.randint(0, CFG["vocab_size"], (1,), generator=g))], [0]) for i in range(8)])
    one(); one()                                              # recorded at the first, replayed from then on
    before, replays = r.kernel_launches(), r.graph_replays
    one()
    assert r.graph_replays == replays + 1
    layers = CFG["num_hidden_layers"]
    assert r.kernel_launches() - before == 5 * layers + 4
    for i in range(8):
        r.finish(("k", i))


def test_generation_under_page_pressure_at_real_layer_sizes(runners):
    """Six prompts through Engine.generate with so few pages that requests are preempted and recomputed: every
    request finishes; the bfloat16 engine's tokens are the float32 engine's choice for the same prefix or within a
    near-tie of it (checked with the float32 engine's logits of the bfloat16 engine's own sequence)."""
    from lucciola_b200 import Engine, SamplingParams
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.step import ModelRunner, StepEntry
    g = torch.Generator().manual_seed(13)
    prompts = [torch.randint(0, CFG["vocab_size"], (n,), generator=g).tolist() for n in (90, 40, 130, 75, 20, 110)]
    params = SamplingParams(max_new_tokens=24, ignore_eos=True)
    base = runners["bfloat16"]
    opts = EngineOptions(dtype="bfloat16", block_size=16, max_blocks=30, max_num_seqs=6, max_model_len=4096,
                         max_tokens_per_step=96)
    tight = Engine(runner=ModelRunner(base.model, base.rt, opts, 30))          # 480 tokens of cache for 465 + 144
    outs = tight.generate(prompts, params)
    assert all(len(o) == 24 for o in outs) and tight.stats()["preemptions"] > 0
    tight.runner.manager.check_invariants()
    assert all(p.num_free == p.num_pages for p in tight.runner.manager.pools) and not tight.runner._table_rows
    ref = runners["float32"]
    for p, o in zip(prompts, outs):
        logits = ref.step([StepEntry("chk", p + o[:-1], list(range(len(p) - 1, len(p) + len(o) - 1)))]).float().cpu()
        ref.finish("chk")
        gap = logits.max(dim=-1).values - logits[torch.arange(len(o)), torch.tensor(o)]
        # each of two logits may be off by the tolerance of the logit comparisons
        assert gap.max().item() <= 2 * BF16_TOL * logits.abs().max().item(), (gap.max().item(), logits.abs().max().item())


def test_a_recording_survives_growth_of_the_attention_workspace(runners):
    """A recorded step whose attention splits its keys through the workspace (a portion of 8 tokens: 32 query rows a
    tile, too many for the in-cluster combine) keeps the workspace's address.  A later step that needs a larger
    workspace must not take that memory away: the old recording is replayed afterwards and must still be right."""
    from lucciola_b200 import ops
    from lucciola_b200.engine.step import StepEntry
    g = torch.Generator().manual_seed(17)
    ids = torch.randint(0, CFG["vocab_size"], (3, 3100), generator=g).tolist()
    ref_r, r = runners["float32"], runners["bfloat16"]

    def portion_of_8(runner, rid, seq, at):
        runner.step([StepEntry(rid, seq[:at], [])])
        out = runner.step([StepEntry(rid, seq[at:at + 8], list(range(8)))]).float().cpu().clone()
        runner.finish(rid)
        return out

    want = [portion_of_8(ref_r, "w", ids[i], 600) for i in range(3)]
    got0 = portion_of_8(r, "w", ids[0], 600)                  # seen once
    got1 = portion_of_8(r, "w", ids[1], 600)                  # seen twice: recorded
    shape = (0, (8,), 1024, ("all",))
    assert shape in r._graphs
    before = ops._attn_ws[r.device.index].numel()
    # three portions of 8 tokens at 3000 tokens of context each, in one step: many more partial results
    for i in range(3):
        r.step([StepEntry(("big", i), ids[i][:3000], [])])
    r.step([StepEntry(("big", i), ids[i][3000:3008], [7]) for i in range(3)])
    for i in range(3):
        r.finish(("big", i))
    if ops._attn_ws[r.device.index].numel() == before:        # an earlier test has made it large enough for that step already
        ops._attention_workspace(r.device, 2 * before + 1)
    assert ops._attn_ws[r.device.index].numel() > before and ops._attn_ws_retired, "the workspace did not grow"
    r.step([StepEntry("w", ids[2][:600], [])])
    replays = r.graph_replays
    got2 = r.step([StepEntry("w", ids[2][600:608], list(range(8)))]).float().cpu().clone()     # the old recording, replayed
    r.finish("w")
    assert r.graph_replays == replays + 1
    for got, ref in zip((got0, got1, got2), want):
        err = ((got - ref).abs().max() / ref.abs().max()).item()
        assert torch.isfinite(got).all() and err < BF16_TOL, err


def test_portions_behind_a_long_context_cut_their_keys_into_ranges(runners, monkeypatch):
    """A portion of a few dozen tokens behind thousands of cached ones makes fewer work items than the GPU has SMs; the
    tensor-memory kernel then cuts every item's keys into ranges and a second kernel combines them.  Eagerly, recorded,
    and replayed, against the float32 engine fed the prompt whole."""
    from lucciola_b200 import ops
    g = torch.Generator().manual_seed(23)
    ids = torch.randint(0, CFG["vocab_size"], (3500,), generator=g).tolist()
    ref = logits_of(runners["float32"], ids, [3500])
    scale = ref.abs().max().item()
    seen = []
    plain = ops.attention_tcgen05

    def spy(*args, key_splits=1, **kw):
        seen.append((args[6].shape[0], key_splits))
        return plain(*args, key_splits=key_splits, **kw)

    monkeypatch.setattr(ops, "attention_tcgen05", spy)
    r = runners["bfloat16"]
    replays = r.graph_replays
    for _ in range(3):
        got = logits_of(r, ids, [3000, 64, 128, 200, 108])
        err = ((got - ref).abs().max() / scale).item()
        assert torch.isfinite(got).all() and err < BF16_TOL, err
    assert (1, 8) in seen and all(k > 1 for n, k in seen if n <= 4), sorted(set(seen))      # 64 tokens: one item a kv head
    assert r.graph_replays > replays
    assert ops.device_error() == 0


def test_sliding_window_at_the_real_head_size():
    """A full layer and a sliding layer with heads of 128 in groups of four: the tensor-memory prompt kernel and the
    decode kernel with a window, pages given back behind the window and used again by a second request; bfloat16
    against float32 under two ways of cutting, float32 unchanged by the cutting."""
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner_random
    from lucciola_b200.engine.step import StepEntry
    cfg = dict(CFG, hidden_size=512, num_attention_heads=8, num_key_value_heads=2, intermediate_size=1024, vocab_size=3000,
               layer_types=["full_attention", "sliding_attention"], sliding_window=150, use_sliding_window=True)
    runners = {}
    for dtype in ("float32", "bfloat16"):
        opts = EngineOptions(dtype=dtype, block_size=16, max_blocks=80, max_num_seqs=4, max_model_len=1024, max_tokens_per_step=1024)
        runners[dtype] = build_runner_random(cfg, seed=5, options=opts, std=0.05, norm_std=0.05)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg["vocab_size"], (600,), generator=g).tolist()
    other = torch.randint(0, cfg["vocab_size"], (300,), generator=g).tolist()
    ref = logits_of(runners["float32"], ids, [600])
    assert torch.equal(logits_of(runners["float32"], ids, [130, 270, 3, 160], tail=37), ref)
    scale = ref.abs().max().item()
    r = runners["bfloat16"]
    for cuts, tail in (([600], 0), ([130, 270, 3, 160], 37)):
        # a second request takes pages in between, so that the window's freed pages are used again
        r.step([StepEntry("o", other[:200], [])])
        got = logits_of(r, ids, cuts, tail)
        r.step([StepEntry("o", other[200:], [])])
        r.finish("o")
        r.manager.check_invariants()
        err = ((got - ref).abs().max() / scale).item()
        assert torch.isfinite(got).all() and err < BF16_TOL, (cuts, tail, err)
    sliding = [gi for gi, grp in enumerate(r.groups) if grp.window > 0]
    assert sliding and r.manager.pools[sliding[0]].high_water < 2 * (600 // 16)       # the window's group never held both requests whole
