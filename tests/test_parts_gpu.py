"""Each part alone against the plain implementation's function for it, the order of layers as data,
a toy feed-forward with routing, and a toy mixer with state of its own that is registered, built and stepped without a change to
the framework's files (GPU)."""
import json
import math

import pytest
import torch

import plain_qwen3 as plain
from conftest import tokens_for

pytestmark = pytest.mark.gpu
ACTS = [torch.float32, torch.bfloat16]
TOL = {torch.float32: 3e-6, torch.bfloat16: 1.5e-2}


def rel(a, b):
    return ((a.double().cpu() - b.double().cpu()).abs().max() / b.double().abs().max().clamp_min(1e-30)).item()


def make_rt(act):
    from lucciola_b200.parts import Runtime
    torch.cuda.set_device(0)
    rt = Runtime("cuda:0", act)
    rt.stream = torch.cuda.current_stream().cuda_stream
    return rt


def bind_random(part, act, seed=0, std=0.1, norm_std=0.2):
    """Give a part random tensors; returns them as float64 on the CPU, rounded as the part holds them."""
    from lucciola_b200.weights.random_init import random_tensor
    held = {}

    def get(name):
        spec = {s.name: s for s in part.all_param_specs()}[name]
        t = random_tensor(spec, seed, std, norm_std, torch.bfloat16)
        held[name] = t.double()
        return t.to("cuda:0", dtype=torch.float32 if act == torch.float32 else torch.bfloat16)

    part.bind_all(get)
    return held


def one_request_step(rt, T, page, nkv, d, start=0, window=0, group=None):
    """A StepContext and a cache for one request that brings T tokens after `start` cached ones."""
    from lucciola_b200.parts import KVCacheView, StepContext
    dev = rt.device
    L = start + T
    P = -(-L // page) + 1
    bt = torch.full((1, P), -1, dtype=torch.int32)
    bt[0, :-(-L // page)] = torch.randperm(-(-L // page) + 2)[:-(-L // page)].int()
    pool = torch.full((2, P + 2, nkv, page, d), float("nan"), dtype=rt.act_dtype, device=dev)
    pos = torch.arange(start, L, dtype=torch.int32, device=dev)
    plans = {}
    if group and rt.fast_kernels:                 # the tile lists that the attention part plans for such a step
        from lucciola_b200.parts.attention import plan_tiles
        from lucciola_b200.parts.base import BatchShape, PlanView
        made = plan_tiles(BatchShape([T], [start], T, L, L), group)
        plans[("attention tiles", group)] = PlanView({k: torch.from_numpy(a).to(dev) for k, a in made.arrays.items()}, made.host)
    step = StepContext(num_tokens=T, num_seqs=1, positions=pos, token_seq=torch.zeros(T, dtype=torch.int32, device=dev),
                       cu_tokens=torch.tensor([0, T], dtype=torch.int32, device=dev),
                       context_lens=torch.tensor([L], dtype=torch.int32, device=dev), block_tables=[bt.to(dev)],
                       state_slots=torch.zeros(1, dtype=torch.int32, device=dev), q_lens=[T], start_positions=[start],
                       max_q_len=T, max_context_len=L, plans=plans)
    return step, KVCacheView(pool[0], pool[1], 0, page)


@pytest.mark.parametrize("act", ACTS)
def test_rmsnorm_part(act):
    from lucciola_b200.parts import RMSNorm
    rt = make_rt(act)
    n = RMSNorm(rt, "n.weight", 200, 2e-5)
    w = bind_random(n, act)["n.weight"]
    x = torch.randn(6, 200, device="cuda:0")
    want = plain.rms_norm(x.double().cpu(), w, 2e-5)
    assert rel(n.forward(x, act), want) < TOL[act]
    delta = torch.randn(6, 200, device="cuda:0").to(act)
    r = x.clone()
    out = n.add_forward(r, delta, act)
    assert torch.equal(r, x + delta.float()) and rel(out, plain.rms_norm((x + delta.float()).double().cpu(), w, 2e-5)) < TOL[act]


@pytest.mark.parametrize("act", ACTS)
def test_linear_and_stacked_linear(act):
    from lucciola_b200.parts import Linear
    rt = make_rt(act)
    lin = Linear(rt, ["a.weight", "b.weight"], 72, [40, 24])
    w = bind_random(lin, act)
    x = torch.randn(5, 72, device="cuda:0").to(act)
    y = lin.forward(x)
    want = torch.cat([plain.linear(x.double().cpu(), w["a.weight"]), plain.linear(x.double().cpu(), w["b.weight"])], dim=1)
    assert y.shape == (5, 64) and rel(y, want) < TOL[act]
    assert rel(lin.forward(x, rows=40), want[:, :40]) < TOL[act]


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("inter,tokens", [(200, 7), (192, 7), (192, 300)])
def test_feed_forward_part(act, inter, tokens):
    """An intermediate size that is no multiple of 64 (separate SwiGLU kernel) and one that is (on the bfloat16
    path gate and up rows are interleaved and the activation is formed in the product's epilogue)."""
    from lucciola_b200.parts import SwiGLUFeedForward
    rt = make_rt(act)
    ffn = SwiGLUFeedForward(rt, "mlp", 72, inter)
    w = bind_random(ffn, act)
    assert ffn.fused == (act == torch.bfloat16 and inter % 64 == 0)
    x = torch.randn(tokens, 72, device="cuda:0").to(act)
    assert rel(ffn.forward(x, None), plain.feed_forward(x.double().cpu(), w, "mlp")) < TOL[act]


@pytest.mark.parametrize("act", ACTS)
def test_embedding_and_head_parts(act):
    from lucciola_b200.parts import OutputHead, TokenEmbedding
    rt = make_rt(act)
    emb = TokenEmbedding(rt, "e.weight", 90, 40)
    w = bind_random(emb, act)["e.weight"]
    ids = torch.tensor([3, 89, 0, 3], dtype=torch.int32, device="cuda:0")
    assert torch.equal(emb.forward(ids).double().cpu(), plain.embed(ids.cpu().tolist(), w))
    tied = OutputHead(rt, "h.weight", 90, 40, emb)
    tied.bind_all(lambda name: (_ for _ in ()).throw(AssertionError("a tied head asks for no tensor")))
    x = torch.randn(3, 40, device="cuda:0").to(act)
    logits = tied.forward(x)
    assert logits.dtype == torch.float32 and rel(logits, plain.linear(x.double().cpu(), w)) < TOL[act]
    own = OutputHead(rt, "h.weight", 90, 40, None)
    wh = bind_random(own, act, seed=5)["h.weight"]
    assert rel(own.forward(x), plain.linear(x.double().cpu(), wh)) < TOL[act]


@pytest.mark.parametrize("act", ACTS)
@pytest.mark.parametrize("nq,nkv,d,window,start,T", [(6, 2, 24, 0, 0, 21), (4, 4, 64, 9, 0, 40), (8, 2, 128, 0, 0, 70)])
def test_attention_part(act, nq, nkv, d, window, start, T):
    """Norm of q and k per head, rotation, cache write, attention and output projection, whole and then
    continued from the cache in a second step."""
    from lucciola_b200.parts import GQAttention, RotaryEmbedding
    rt = make_rt(act)
    hidden, theta, eps, page = 56, 7e4, 3e-6, 8
    att = GQAttention(rt, "self_attn", hidden, nq, nkv, d, RotaryEmbedding(rt, d, theta), qk_norm_eps=eps, window=window)
    w = bind_random(att, act, std=0.15)
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d, "hidden_size": hidden,
           "rms_norm_eps": eps, "rope_theta": theta}
    x = torch.randn(T, hidden, device="cuda:0").to(act)
    want, _ = plain.attention_block(x.double().cpu(), w, "self_attn", cfg, list(range(T)), window)
    step, cache = one_request_step(rt, T, page, nkv, d, group=nq // nkv)
    assert rel(att.forward(x, step, cache), want) < TOL[act]
    # the same tokens in two steps: the second reads what the first left in the pages
    cut = T // 2 + 1
    step1, cache = one_request_step(rt, cut, page, nkv, d, group=nq // nkv)
    step2, _ = one_request_step(rt, T - cut, page, nkv, d, start=cut, group=nq // nkv)
    need = -(-T // page)
    bt = torch.full((1, need + 1), -1, dtype=torch.int32)
    bt[0, :need] = torch.arange(need, dtype=torch.int32)
    step1.block_tables = [bt.cuda()]; step2.block_tables = [bt.cuda()]
    pool = torch.full((2, need + 1, nkv, page, d), float("nan"), dtype=act, device="cuda:0")
    from lucciola_b200.parts import KVCacheView
    cache = KVCacheView(pool[0], pool[1], 0, page)
    a = att.forward(x[:cut].contiguous(), step1, cache)
    b = att.forward(x[cut:].contiguous(), step2, cache)
    assert rel(torch.cat([a, b]), want) < TOL[act]


def test_another_position_encoding_goes_through_apply():
    """A position encoding the fused kernel does not know: the mixer norms, calls the part's apply(), then writes."""
    from lucciola_b200.parts import GQAttention, PositionEncoding
    rt = make_rt(torch.float32)

    class SignFlip(PositionEncoding):            # toy: negate q and k at odd positions
        def apply(self, q, k, positions):
            s = (1 - 2 * (positions % 2)).to(q.dtype)[:, None, None]
            q.mul_(s); k.mul_(s)

    nq, nkv, d, hidden, T = 4, 2, 16, 32, 13
    att = GQAttention(rt, "a", hidden, nq, nkv, d, SignFlip(), qk_norm_eps=None)
    w = bind_random(att, torch.float32)
    x = torch.randn(T, hidden, device="cuda:0")
    step, cache = one_request_step(rt, T, 4, nkv, d)
    got = att.forward(x, step, cache)
    xd = x.double().cpu()
    sign = (1 - 2 * (torch.arange(T) % 2)).double()[:, None, None]
    q = plain.linear(xd, w["a.q_proj.weight"]).reshape(T, nq, d) * sign
    k = plain.linear(xd, w["a.k_proj.weight"]).reshape(T, nkv, d) * sign
    v = plain.linear(xd, w["a.v_proj.weight"]).reshape(T, nkv, d)
    o = plain.attention(q, k, v, list(range(T)), list(range(T)), 1 / math.sqrt(d))
    assert rel(got, plain.linear(o.reshape(T, nq * d), w["a.o_proj.weight"])) < 3e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_order_of_layers_is_data(tiny_models, dtype):
    """A layer named twice (two caches) and a layer that reads another layer's cache, against the plain
    implementation run with the same list of calls; whole and cut into portions."""
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner
    from lucciola_b200.engine.step import ModelRunner, StepEntry
    from lucciola_b200.models import LayerCall
    import replay_util as ru

    folder = tiny_models["A"]
    pc, pw = plain.read_model(folder)
    ids = tokens_for("A", 50, salt=4)
    for calls in ([(0, 0, True), (0, 1, True), (1, 2, True)], [(0, 0, True), (1, 0, False), (1, 1, True)]):
        base = build_runner(folder, EngineOptions(dtype=dtype, block_size=16, max_blocks=16, max_num_seqs=2, use_cuda_graph=False))
        model = base.model
        model.calls = [LayerCall(*c) for c in calls]
        model._check_calls()
        runner = ModelRunner(model, base.rt, base.options, 16)
        want = plain.forward(pc, pw, ids, calls=calls)
        got = runner.step([StepEntry("w", ids, list(range(50)))]).double().cpu()
        scale = want.abs().max()
        assert ((got - want).abs().max() / scale).item() < ru.TOL[dtype]
        runner.finish("w")
        parts = [runner.step([StepEntry("p", ids[a:b], list(range(b - a)))]) for a, b in ((0, 17), (17, 19), (19, 50))]
        got2 = torch.cat(parts).double().cpu()
        assert ((got2 - want).abs().max() / scale).item() < ru.TOL[dtype]


def toy_running_mean_model(tmp_path, mixer_class):
    """An architecture defined here around `mixer_class` (a mixer with a fixed-size state per request: a running mean
    of what it has seen): registered, written as config.json + safetensors.  Returns (config, plain forward)."""
    from lucciola_b200.config import register_architecture
    from lucciola_b200.models import DecoderModel, LayerCall
    from lucciola_b200.parts import OutputHead, PreNormBlock, RMSNorm, Runtime, SwiGLUFeedForward, TokenEmbedding
    from lucciola_b200.weights import write_safetensors
    from lucciola_b200.weights.random_init import RandomWeights

    def build(cfg, rt):
        H, V = cfg["hidden_size"], cfg["vocab_size"]
        emb = TokenEmbedding(rt, "emb.weight", V, H)
        blocks = [PreNormBlock(mixer_class(rt, f"l{i}.mix", H), SwiGLUFeedForward(rt, f"l{i}.mlp", H, cfg["inner"]),
                               RMSNorm(rt, f"l{i}.n1.weight", H, cfg["eps"]), RMSNorm(rt, f"l{i}.n2.weight", H, cfg["eps"]),
                               rt.act_dtype) for i in range(cfg["layers"])]
        return DecoderModel(rt, emb, blocks, [LayerCall(i, i) for i in range(cfg["layers"])],
                            RMSNorm(rt, "norm.weight", H, cfg["eps"]), OutputHead(rt, "head.weight", V, H, None), V, cfg["max_len"])

    register_architecture("ToyRunningMeanLM", dict, build, replace=True)
    cfg = {"architectures": ["ToyRunningMeanLM"], "hidden_size": 40, "vocab_size": 61, "inner": 72, "layers": 2,
           "eps": 1e-5, "max_len": 64}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    specs = build(cfg, Runtime("cpu", torch.float32)).all_param_specs()
    src = RandomWeights(specs, 3, std=0.2, norm_std=0.1)
    weights = {n: src.get(n) for n in src.names()}
    write_safetensors(tmp_path / "model.safetensors", weights)

    def plain_forward(ids):
        w = {k: v.double() for k, v in weights.items()}
        x = w["emb.weight"][torch.tensor(ids)]
        for i in range(cfg["layers"]):
            h = plain.rms_norm(x, w[f"l{i}.n1.weight"], cfg["eps"])
            mean = torch.cumsum(h, 0) / torch.arange(1, len(ids) + 1, dtype=torch.float64)[:, None]
            x = x + plain.linear(mean, w[f"l{i}.mix.proj.weight"])
            h = plain.rms_norm(x, w[f"l{i}.n2.weight"], cfg["eps"])
            x = x + plain.feed_forward(h, {k.replace(f"l{i}.mlp.", "m."): v for k, v in w.items()}, "m")
        return plain.linear(plain.rms_norm(x, w["norm.weight"], cfg["eps"]), w["head.weight"])

    return cfg, plain_forward


def test_toy_mixer_with_state_of_its_own(tmp_path):
    """A mixer defined here, with a fixed-size state per request (a running mean of what it has seen),
    inside an architecture defined here: registered, built from a config.json, loaded from safetensors
    and stepped by the framework's runner, whole and in portions, mixed with a second request."""
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner
    from lucciola_b200.engine.step import StepEntry
    from lucciola_b200.parts import Linear, Mixer, StateSlot

    class RunningMean(Mixer):
        """out_t = W . mean(h_0 .. h_t).  State per request: the sum so far and the count."""
        def __init__(self, rt, prefix, hidden):
            self.rt, self.hidden = rt, hidden
            self.proj = Linear(rt, f"{prefix}.proj.weight", hidden, hidden)

        def children(self):
            return [self.proj]

        def cache_request(self):
            return StateSlot((self.hidden + 1,), torch.float32)

        def forward(self, h, step, cache, write_cache=True):
            out = torch.empty_like(h)
            for i in range(step.num_seqs):
                a, b = sum(step.q_lens[:i]), sum(step.q_lens[:i + 1])
                slot = int(step.state_slots[i])
                st = cache.state[slot]
                sums = st[:-1] + torch.cumsum(h[a:b].float(), dim=0)
                counts = st[-1] + torch.arange(1, b - a + 1, device=h.device, dtype=torch.float32)
                out[a:b] = (sums / counts[:, None]).to(h.dtype)
                st[:-1] = sums[-1]; st[-1] = counts[-1]
            return self.proj.forward(out)

    cfg, plain_forward = toy_running_mean_model(tmp_path, RunningMean)
    runner = build_runner(tmp_path, EngineOptions(dtype="float32", block_size=16, max_blocks=4, max_num_seqs=3, use_cuda_graph=False))
    assert runner.groups == [] and list(runner.cache.states) == [0, 1]          # no pages, two state caches
    a, b = [5, 9, 60, 0, 33, 7, 7, 18, 2, 41, 3], [11, 12, 13, 14, 15, 16]
    wa, wb = plain_forward(a), plain_forward(b)
    got = runner.step([StepEntry("a", a, list(range(len(a))))]).double().cpu()
    assert ((got - wa).abs().max() / wa.abs().max()) < 1e-5
    runner.finish("a")
    # portions, with another request in between; "a" is a new request again: its slot must have been cleared
    g1 = runner.step([StepEntry("a", a[:4], [0, 1, 2, 3]), StepEntry("b", b[:1], [0])]).double().cpu()
    g2 = runner.step([StepEntry("b", b[1:], list(range(5))), StepEntry("a", a[4:6], [0, 1])]).double().cpu()
    g3 = runner.step([StepEntry("a", a[6:], list(range(5)))]).double().cpu()
    got_a = torch.cat([g1[:4], g2[5:], g3]); got_b = torch.cat([g1[4:], g2[:5]])
    assert ((got_a - wa).abs().max() / wa.abs().max()) < 1e-5 and ((got_b - wb).abs().max() / wb.abs().max()) < 1e-5
    runner.finish("a"); runner.finish("b")
    runner.manager.check_invariants()
    # this mixer reads a device value on the host (its slot), so it does not call itself recordable, and a bfloat16
    # runner with recordings switched on records nothing for a model that holds it
    bf = build_runner(tmp_path, EngineOptions(dtype="bfloat16", block_size=16, max_blocks=4, max_num_seqs=3, use_cuda_graph=True, graph_after=1))
    assert not bf._can_record
    got = bf.step([StepEntry("a", a, list(range(len(a))))]).double().cpu()
    assert ((got - wa).abs().max() / wa.abs().max()) < 3e-2 and not bf._graphs


def test_toy_mixer_with_state_is_recorded_and_replayed(tmp_path):
    """The same running mean written so that its forward() only launches work on the step's stream (the slot is used
    as a device index): it says so (`recordable`), and the framework records its steps as CUDA graphs and replays them,
    the clearing of a new request's slot included; single tokens of three requests replay the recording of four, whose
    fourth entry reads and writes the spare state row."""
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner
    from lucciola_b200.engine.step import StepEntry
    from lucciola_b200.parts import Linear, Mixer, StateSlot

    class RunningMean(Mixer):
        recordable = True

        def __init__(self, rt, prefix, hidden):
            self.rt, self.hidden = rt, hidden
            self.proj = Linear(rt, f"{prefix}.proj.weight", hidden, hidden)

        def children(self):
            return [self.proj]

        def cache_request(self):
            return StateSlot((self.hidden + 1,), torch.float32)

        def forward(self, h, step, cache, write_cache=True):
            out = torch.empty_like(h)
            slots = step.state_slots.long()
            t = 0
            for i, n in enumerate(step.q_lens):                # the lengths are part of a recording's shape
                st = cache.state.index_select(0, slots[i:i + 1])[0]
                sums = st[:-1] + torch.cumsum(h[t:t + n].float(), dim=0)
                counts = st[-1] + torch.arange(1, n + 1, device=h.device, dtype=torch.float32)
                out[t:t + n] = (sums / counts[:, None]).to(h.dtype)
                cache.state.index_copy_(0, slots[i:i + 1], torch.cat([sums[-1], counts[-1:]])[None])
                t += n
            return self.proj.forward(out)

    cfg, plain_forward = toy_running_mean_model(tmp_path, RunningMean)
    runner = build_runner(tmp_path, EngineOptions(dtype="bfloat16", block_size=16, max_blocks=4, max_num_seqs=4,
                                                  use_cuda_graph=True, graph_after=1))
    assert runner._can_record
    seqs = {k: [(7 * i * i + 5 * i + ord(k)) % 61 for i in range(20)] for k in "abcd"}
    want = {k: plain_forward(v) for k, v in seqs.items()}
    got = {k: [] for k in seqs}

    def run(entries):
        out = runner.step([StepEntry(k, seqs[k][a:b], list(range(b - a))) for k, a, b in entries]).double().cpu()
        for k, a, b in entries:
            got[k].append(out[:b - a]); out = out[b - a:]

    run([("a", 0, 11)])                                       # recorded
    run([("b", 0, 11)])                                       # replayed: b's slot is cleared inside the recording
    run([("c", 0, 11)])
    assert runner.graph_replays == 2
    for t in range(11, 17):                                   # three single tokens: the recording of four
        run([("a", t, t + 1), ("b", t, t + 1), ("c", t, t + 1)])
    assert (4, (), 256, ()) in runner._graphs
    runner.finish("c")
    got["c"] = []
    run([("a", 17, 18), ("b", 17, 18), ("c", 0, 5)])          # single tokens beside a portion of a request that starts anew
    run([("a", 18, 19), ("b", 18, 19), ("d", 0, 5)])          # the same shape replayed, d's slot cleared
    run([("a", 19, 20), ("b", 19, 20), ("c", 5, 10)])
    assert (2, (5,), 256, ("all",)) in runner._graphs and runner.graph_replays >= 2 + 5 + 2
    for k in seqs:
        g = torch.cat(got[k])
        assert ((g - want[k][:g.shape[0]]).abs().max() / want[k].abs().max()) < 3e-2, k
    assert torch.cat(got["a"]).shape[0] == 20 and torch.cat(got["c"]).shape[0] == 10
    for k in seqs:
        runner.finish(k)
    runner.manager.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_norm_and_toy_block_between_the_frameworks_blocks(tmp_path, dtype):
    """A norm defined here (centred: subtract the mean, divide by the standard deviation, weight and bias) and a block
    arrangement defined here (post-norm: r = norm(r + mixer(r)); r = norm(r + ffn(r)), no keyword for what follows it),
    as the middle one of three layers whose outer two are the framework's pre-norm blocks at sizes where those hand their
    output on inside the products' epilogues.  The model must take the plain path around the toy block and still be right,
    whole, in portions and token by token (recorded in bfloat16: the toy parts only launch work)."""
    from lucciola_b200.config import EngineOptions, register_architecture
    from lucciola_b200.engine.load import build_runner
    from lucciola_b200.engine.step import StepEntry
    from lucciola_b200.models import DecoderModel, LayerCall
    from lucciola_b200.parts import (Block, GQAttention, Norm, OutputHead, ParamSpec, PreNormBlock, RMSNorm, RotaryEmbedding,
                                     Runtime, SwiGLUFeedForward, TokenEmbedding)
    from lucciola_b200.weights import write_safetensors
    from lucciola_b200.weights.random_init import RandomWeights

    class CentredNorm(Norm):
        recordable = True

        def __init__(self, rt, prefix, size, eps):
            self.rt, self.prefix, self.size, self.eps = rt, prefix, size, eps

        def param_specs(self):
            return [ParamSpec(f"{self.prefix}.weight", (self.size,), "norm"), ParamSpec(f"{self.prefix}.bias", (self.size,), "linear")]

        def bind(self, get):
            self.w, self.b = get(f"{self.prefix}.weight").float(), get(f"{self.prefix}.bias").float()

        def forward(self, x, out_dtype):
            x = x.float()
            c = x - x.mean(dim=-1, keepdim=True)
            return (c * torch.rsqrt((c * c).mean(dim=-1, keepdim=True) + self.eps) * self.w + self.b).to(out_dtype)

        def add_forward(self, residual, delta, out_dtype, rows=None):
            if delta is not None:
                residual += delta.float()
            return self.forward(residual if rows is None else residual[rows.long()], out_dtype)

    class PostNormBlock(Block):
        recordable = True

        def __init__(self, mixer, ffn, norm1, norm2, act):
            self.mixer, self.ffn, self.norm1, self.norm2, self.act = mixer, ffn, norm1, norm2, act

        def children(self):
            return [self.mixer, self.norm1, self.ffn, self.norm2]

        def forward(self, residual, delta, step, cache, write_cache=True):
            if delta is not None:
                residual += delta.float()
            a = self.mixer.forward(residual.to(self.act), step, cache, write_cache)
            residual.copy_(self.norm1.add_forward(residual, a, torch.float32))
            f = self.ffn.forward(residual.to(self.act), step)
            residual.copy_(self.norm2.add_forward(residual, f, torch.float32))
            return residual, None

    def build(cfg, rt):
        H, V, d, nq, nkv, inner, eps = (cfg[k] for k in ("hidden_size", "vocab_size", "head_dim", "heads", "kv_heads", "inner", "eps"))
        rope = RotaryEmbedding(rt, d, cfg["theta"])
        att = lambda i: GQAttention(rt, f"l{i}.attn", H, nq, nkv, d, rope, eps)
        ffn = lambda i: SwiGLUFeedForward(rt, f"l{i}.mlp", H, inner)
        pre = lambda i: PreNormBlock(att(i), ffn(i), RMSNorm(rt, f"l{i}.n1.weight", H, eps), RMSNorm(rt, f"l{i}.n2.weight", H, eps), rt.act_dtype)
        blocks = [pre(0), PostNormBlock(att(1), ffn(1), CentredNorm(rt, "l1.n1", H, eps), CentredNorm(rt, "l1.n2", H, eps), rt.act_dtype), pre(2)]
        return DecoderModel(rt, TokenEmbedding(rt, "emb.weight", V, H), blocks, [LayerCall(i, i) for i in range(3)],
                            RMSNorm(rt, "norm.weight", H, eps), OutputHead(rt, "head.weight", V, H, None), V, cfg["max_len"])

    register_architecture("ToyPostNormLM", dict, build, replace=True)
    cfg = {"architectures": ["ToyPostNormLM"], "hidden_size": 512, "vocab_size": 211, "inner": 576, "heads": 4, "kv_heads": 1,
           "head_dim": 128, "theta": 10000.0, "eps": 1e-5, "max_len": 128}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    specs = build(cfg, Runtime("cpu", torch.float32)).all_param_specs()
    src = RandomWeights(specs, 11, std=0.05, norm_std=0.1)
    weights = {n: src.get(n) for n in src.names()}
    write_safetensors(tmp_path / "model.safetensors", weights)
    w = {k: v.double() for k, v in weights.items()}
    pcfg = {"num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 128, "hidden_size": 512, "rms_norm_eps": 1e-5, "rope_theta": 10000.0}

    def centred(x, prefix):
        c = x - x.mean(dim=-1, keepdim=True)
        return c * torch.rsqrt((c * c).mean(dim=-1, keepdim=True) + cfg["eps"]) * w[f"{prefix}.weight"] + w[f"{prefix}.bias"]

    def mlp(h, i):
        return plain.feed_forward(h, {k.replace(f"l{i}.mlp.", "m."): v for k, v in w.items() if k.startswith(f"l{i}.mlp.")}, "m")

    def plain_forward(ids):
        x = w["emb.weight"][torch.tensor(ids)]
        pos = torch.arange(len(ids))
        for i in (0, 1, 2):
            if i == 1:
                x = centred(x + plain.attention_block(x, w, "l1.attn", pcfg, pos, 0)[0], "l1.n1")
                x = centred(x + mlp(x, 1), "l1.n2")
            else:
                x = x + plain.attention_block(plain.rms_norm(x, w[f"l{i}.n1.weight"], cfg["eps"]), w, f"l{i}.attn", pcfg, pos, 0)[0]
                x = x + mlp(plain.rms_norm(x, w[f"l{i}.n2.weight"], cfg["eps"]), i)
        return plain.linear(plain.rms_norm(x, w["norm.weight"], cfg["eps"]), w["head.weight"])

    runner = build_runner(tmp_path, EngineOptions(dtype=dtype, block_size=16, max_blocks=16, max_num_seqs=2, graph_after=1))
    assert runner._can_record == (dtype == "bfloat16")
    ids = [(13 * i * i + 7 * i + 3) % 211 for i in range(60)]
    want = plain_forward(ids)
    tol = 1e-5 if dtype == "float32" else 3e-2
    for cuts in ([60], [25, 2, 20], [40]):
        rows, pos = [], 0
        for n in cuts:
            rows.append(runner.step([StepEntry("r", ids[pos:pos + n], list(range(n)))]).double().cpu())
            pos += n
        while pos < 60:                                           # the rest token by token (recorded and replayed in bfloat16)
            rows.append(runner.step([StepEntry("r", [ids[pos]], [0])]).double().cpu().clone())
            pos += 1
        runner.finish("r")
        got = torch.cat(rows)
        assert ((got - want).abs().max() / want.abs().max()) < tol, cuts
    assert (runner.graph_replays > 0) == (dtype == "bfloat16")


def test_toy_feed_forward_with_routing_chosen_layer_by_layer(tmp_path):
    """A feed-forward with a router and experts, defined here: top-2 of 3 small SwiGLU experts, router logits and
    the softmax over the chosen ones in 32-bit.  Layer 0 uses it, layer 1 the framework's dense feed-forward, both
    behind the framework's attention: the block takes either without knowing which."""
    from lucciola_b200.config import EngineOptions, register_architecture
    from lucciola_b200.engine.load import build_runner
    from lucciola_b200.engine.step import StepEntry
    from lucciola_b200.models import DecoderModel, LayerCall
    from lucciola_b200.parts import (FeedForward, GQAttention, Linear, OutputHead, PreNormBlock, RMSNorm, RotaryEmbedding,
                                     Runtime, SwiGLUFeedForward, TokenEmbedding)
    from lucciola_b200.weights import write_safetensors
    from lucciola_b200.weights.random_init import RandomWeights

    class RoutedExperts(FeedForward):
        def __init__(self, rt, prefix, hidden, inner, experts, top_k):
            self.rt, self.top_k = rt, top_k
            self.router = Linear(rt, f"{prefix}.router.weight", hidden, experts)
            self.experts = [SwiGLUFeedForward(rt, f"{prefix}.experts.{e}", hidden, inner) for e in range(experts)]

        def children(self):
            return [self.router] + self.experts

        def forward(self, h, step):
            logits = self.router.forward(h, out_dtype=torch.float32)
            top, idx = torch.topk(logits, self.top_k, dim=-1)
            gate = torch.softmax(top, dim=-1)
            out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
            for e, expert in enumerate(self.experts):
                rows = (idx == e).any(dim=-1).nonzero().flatten()
                if rows.numel() == 0:
                    continue
                weight = (gate * (idx == e)).sum(dim=-1)[rows]
                out[rows] += weight[:, None] * expert.forward(h[rows].contiguous(), step).float()
            return out.to(h.dtype)

    def build(cfg, rt):
        H, V, d, nq, nkv = cfg["hidden_size"], cfg["vocab_size"], cfg["head_dim"], cfg["heads"], cfg["kv_heads"]
        rope = RotaryEmbedding(rt, d, cfg["theta"])
        def ff(i):
            return RoutedExperts(rt, f"l{i}.moe", H, cfg["inner"], 3, 2) if i == 0 else SwiGLUFeedForward(rt, f"l{i}.mlp", H, cfg["inner"])
        blocks = [PreNormBlock(GQAttention(rt, f"l{i}.attn", H, nq, nkv, d, rope, cfg["eps"]), ff(i),
                               RMSNorm(rt, f"l{i}.n1.weight", H, cfg["eps"]), RMSNorm(rt, f"l{i}.n2.weight", H, cfg["eps"]),
                               rt.act_dtype) for i in range(2)]
        return DecoderModel(rt, TokenEmbedding(rt, "emb.weight", V, H), blocks, [LayerCall(0, 0), LayerCall(1, 1)],
                            RMSNorm(rt, "norm.weight", H, cfg["eps"]), OutputHead(rt, "head.weight", V, H, None), V, cfg["max_len"])

    register_architecture("ToyRoutedLM", dict, build, replace=True)
    cfg = {"architectures": ["ToyRoutedLM"], "hidden_size": 48, "vocab_size": 53, "inner": 40, "heads": 3, "kv_heads": 1,
           "head_dim": 16, "theta": 10000.0, "eps": 1e-5, "max_len": 64}
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    specs = build(cfg, Runtime("cpu", torch.float32)).all_param_specs()
    src = RandomWeights(specs, 5, std=0.3, norm_std=0.1)
    weights = {n: src.get(n) for n in src.names()}
    write_safetensors(tmp_path / "model.safetensors", weights)
    w = {k: v.double() for k, v in weights.items()}

    pcfg = {"num_attention_heads": cfg["heads"], "num_key_value_heads": cfg["kv_heads"], "head_dim": cfg["head_dim"],
            "hidden_size": cfg["hidden_size"], "rms_norm_eps": cfg["eps"], "rope_theta": cfg["theta"]}

    def plain_forward(ids):
        x = w["emb.weight"][torch.tensor(ids)]
        pos = torch.arange(len(ids))
        for i in range(2):
            h = plain.rms_norm(x, w[f"l{i}.n1.weight"], cfg["eps"])
            x = x + plain.attention_block(h, w, f"l{i}.attn", pcfg, pos, 0)[0]
            h = plain.rms_norm(x, w[f"l{i}.n2.weight"], cfg["eps"])
            if i == 0:
                logits = plain.linear(h, w["l0.moe.router.weight"])
                top, idx = torch.topk(logits, 2, dim=-1)
                gate = torch.softmax(top, dim=-1)
                y = torch.zeros_like(h)
                for t in range(len(ids)):
                    for j in range(2):
                        e = int(idx[t, j])
                        ew = {k.replace(f"l0.moe.experts.{e}.", "m."): v for k, v in w.items() if k.startswith(f"l0.moe.experts.{e}.")}
                        y[t] += gate[t, j] * plain.feed_forward(h[t:t + 1], ew, "m")[0]
                x = x + y
            else:
                x = x + plain.feed_forward(h, {k.replace("l1.mlp.", "m."): v for k, v in w.items() if k.startswith("l1.mlp.")}, "m")
        return plain.linear(plain.rms_norm(x, w["norm.weight"], cfg["eps"]), w["head.weight"])

    runner = build_runner(tmp_path, EngineOptions(dtype="float32", block_size=16, max_blocks=8, max_num_seqs=2, use_cuda_graph=False))
    ids = [(7 * i * i + 3 * i + 1) % 53 for i in range(37)]
    want = plain_forward(ids)
    got = runner.step([StepEntry("w", ids, list(range(len(ids))))]).double().cpu()
    assert ((got - want).abs().max() / want.abs().max()) < 1e-5
    runner.finish("w")
    parts = [runner.step([StepEntry("p", ids[a:b], list(range(b - a)))]) for a, b in ((0, 20), (20, 22), (22, 36), (36, 37))]
    got2 = torch.cat(parts).double().cpu()
    assert ((got2 - want).abs().max() / want.abs().max()) < 1e-5
