"""Decode and prefill throughput of the engine on one B200, with random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Default workload: the layer sizes of the Qwen3-8B shape (36 layers, hidden 4096, 32 query heads,
8 kv heads, head size 128, intermediate 12288, vocabulary 151936), bfloat16, random weights, a
batch of 8 requests that decode at a context of 8192 tokens, pages of 16 tokens.  A step is one
decode step of the whole batch.  The line printed at the end is one JSON object:

  value       decoded tokens a second over K steps, timed on the device (CUDA events): the step
              function plus the sampler, token ids fed from the host, nothing read back
  e2e         the same through the public entry point (Engine.step: scheduler, step, sampler), with
              the step's inputs copied from pinned host memory and the sampled tokens read back
  prefill     one step over a prompt of 2048 tokens: tokens a second, and its FLOPs / time / peak
  roofline    bytes a decode step must read (every weight once, the cache of the live requests)
              / time, against the measured copy bandwidth
  points      decode at batch 1 and 64, same context; and the other workloads this engine is specified on, each through
              Engine.step with host tokens in and out, with its share of the roofline and step latencies (p50/p90/p99):
                decode_bN_ctx768   the 8B shape, N = 1, 8, 64 requests, prompts of 512 tokens, 256 new tokens each
                mixed14b           the 14B shape: every step 32 decoding requests and one 512-token portion of a
                                   2048-token prompt (compute-bound: FLOPs / time / peak)
                mixed8b            the 8B shape: 32 requests decoding at the run's context, alone and beside a
                                   portion of 8 and of 512 tokens of a new prompt (step function, device-timed)
                pressure32b        the 32B shape: 64 requests with prompts of 4096 tokens and 256 new tokens each, in a
                                   pool with fewer pages than they need together, so that the scheduler preempts
              (--no-points skips them; --workloads chooses among them)

Peaks come from MEASURED_PEAKS.json beside this file when the driver wrote it, else from the
fallback figures 6650 GB/s and 1590 TFLOP/s.  The timed work reads far more than the 126 MB of L2
per step (weights alone are 16 GB), so no explicit L2 flush is made.
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 36, "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
    "intermediate_size": 12288, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 40960, "hidden_act": "silu", "attention_bias": False,
    "torch_dtype": "bfloat16",
}
# Other shapes of the family (--shape), for measurements beside the default one.
SHAPES = {
    "8b": ("Qwen3-8B shape", QWEN3_8B),
    "14b": ("Qwen3-14B shape", dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408)),
    "32b": ("Qwen3-32B shape", dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)),
    # the size lucciola's own benchmark programs load (benchmarks/basic_bench.cc:13)
    "0.6b": ("Qwen3-0.6B shape", dict(QWEN3_8B, num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, intermediate_size=3072,
                                      tie_word_embeddings=True)),
}


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            if d.get("hbm_gbs"):
                out["hbm_gbs"] = float(d["hbm_gbs"])
            if d.get("bf16_tflops"):
                out["bf16_tflops"] = float(d["bf16_tflops"])
            if d.get("bf16_tflops_sustained"):
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            out["source"] = "measured"
        except (ValueError, OSError):
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples: list[list[str]] = []
        self.proc = None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "25", "-i", str(self.index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()          # the exact process started above
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        mhz = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def model_bytes_and_flops(cfg: dict, layers: int):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nq, nkv, d = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nq + 2 * nkv) * d * H + H * nq * d + 2 * I * H + H * I          # linear weights
    norms = 2 * H + 2 * d
    weight_bytes = layers * (per_layer * 2 + norms * 4) + V * H * 2 + H * 4        # every weight a decode step reads once
    kv_bytes_per_token = layers * 2 * nkv * d * 2
    return per_layer, weight_bytes, kv_bytes_per_token


def prefill_flops(cfg: dict, layers: int, T: int) -> float:
    per_layer, _, _ = model_bytes_and_flops(cfg, layers)
    nq, d, V, H = cfg["num_attention_heads"], cfg["head_dim"], cfg["vocab_size"], cfg["hidden_size"]
    linear = 2.0 * T * per_layer * layers
    attention = layers * nq * 4.0 * d * (T * (T + 1) / 2)                          # causal: QK^T and PV over i+1 keys
    return linear + attention + 2.0 * V * H                                        # the output head on one row


def percentiles(ms: list[float]) -> dict:
    q = statistics.quantiles(ms, n=100, method="inclusive") if len(ms) > 1 else [ms[0]] * 99
    return {"p50_ms": round(q[49], 3), "p90_ms": round(q[89], 3), "p99_ms": round(q[98], 3)}


def timed_steps(engine, torch, keep_going) -> list[float]:
    """Engine.step until keep_going() says no; wall-clock milliseconds of each step (a step ends with the sampled
    tokens on the host, so the device has finished it)."""
    out = []
    while keep_going():
        t0 = time.perf_counter()
        engine.step()
        out.append((time.perf_counter() - t0) * 1e3)
    return out


def run_ctx768(engine, cfg, layers, rng, pk, batches=(64, 8, 1)) -> dict:
    """Decode at the lengths lucciola's own benchmark uses: prompts of 512 tokens, 256 new tokens, so the context
    grows from 512 to 768."""
    import torch
    from lucciola_b200.sampling.params import SamplingParams
    V = cfg["vocab_size"]
    _, weight_bytes, kv_per_token = model_bytes_and_flops(cfg, layers)
    out = {}
    for B in batches:
        params = SamplingParams(max_new_tokens=400, temperature=0.0, ignore_eos=True)
        reqs = [engine.add_request(rng.integers(0, V, size=512).tolist(), params) for _ in range(B)]
        while any(not r.output for r in reqs):                       # the prompts, untimed
            engine.step()
        for _ in range(3):                                           # warm-up: the recording of this batch size
            engine.step()
        torch.cuda.synchronize()
        cached0 = sum(r.num_computed for r in reqs)
        left = [256]
        def more():
            left[0] -= 1
            return left[0] >= 0
        ms = timed_steps(engine, torch, more)
        mean_ctx = (cached0 + sum(r.num_computed for r in reqs)) / 2 / B
        for r in reqs:
            engine.abort(r.rid)
        steps, total = len(ms), sum(ms)
        frac = (weight_bytes + B * mean_ctx * kv_per_token) / (total / steps * 1e-3) / 1e9 / pk["hbm_gbs"]
        key = f"decode_b{B}_ctx768"
        out[key] = round(B * steps / total * 1e3, 1)
        out[key + "_hbm_frac"] = round(frac, 4)
        out[key + "_mean_ctx"] = round(mean_ctx, 1)
        out.update({f"{key}_{k}": v for k, v in percentiles(ms).items()})
    return out


def run_mixed8b(runner, cfg, rng, ctx, B=32, steps=10) -> dict:
    """What a few tokens of a prompt cost beside decoding requests: B requests at the context, then steps of their
    single tokens alone, with a portion of 8 tokens and with one of 512 tokens of a new request (lucciola's schedule
    puts a portion beside the running requests in every step while a prompt waits, src/scheduler.cc:51-120)."""
    import torch
    from lucciola_b200.engine.step import StepEntry
    V = cfg["vocab_size"]
    for j in range(B):
        left = ctx - 6 * (steps + 4) - 8
        while left > 0:
            n = min(left, 2048)
            runner.step([StepEntry(("m", j), rng.integers(0, V, size=n).tolist(), [])])
            left -= n
    out, fresh = {}, [0]
    for portion in (0, 8, 512):
        def entries():
            e = [StepEntry(("m", j), [int(rng.integers(0, V))], [0]) for j in range(B)]
            if portion:
                fresh[0] += 1
                e.append(StepEntry(("mp", fresh[0]), rng.integers(0, V, size=portion).tolist(), []))
            return e
        def one():
            runner.step(entries())
            if portion:
                runner.finish(("mp", fresh[0]))
        for _ in range(4):
            one()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(steps):
            one()
        b.record()
        torch.cuda.synchronize()
        out[f"mixed8b_b{B}_portion{portion}_ms"] = round(a.elapsed_time(b) / steps, 3)
    for j in range(B):
        runner.finish(("m", j))
    out[f"mixed8b_b{B}_portion8_over_alone"] = round(out[f"mixed8b_b{B}_portion8_ms"] / out[f"mixed8b_b{B}_portion0_ms"], 4)
    return out


def run_mixed14b(rng, pk, layers=0, steps=40) -> dict:
    """32 requests decode while prompts of 2048 tokens are read in portions of 512: every timed step holds 32 single
    tokens and one portion (lucciola's schedule: all running requests, then one portion, src/scheduler.cc:51-120)."""
    import torch
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.llm import Engine
    from lucciola_b200.sampling.params import SamplingParams
    name, shape = SHAPES["14b"]
    layers = layers or shape["num_hidden_layers"]
    cfg = dict(shape, num_hidden_layers=layers)
    V, D, chunk, prompt = cfg["vocab_size"], 32, 512, 2048
    pages = D * (4096 // 16) + 4 * (prompt // 16) + 64
    options = EngineOptions(dtype="bfloat16", block_size=16, max_blocks=pages, max_num_seqs=D + 4, max_tokens_per_step=D + chunk,
                            prefill_chunk=chunk, max_model_len=8192)
    engine = Engine.from_random(cfg, seed=0, options=options)
    decoders = [engine.add_request(rng.integers(0, V, size=1024).tolist(), SamplingParams(max_new_tokens=2000, ignore_eos=True))
                for _ in range(D)]
    while any(not r.output for r in decoders):
        engine.step()
    one = SamplingParams(max_new_tokens=1, ignore_eos=True)          # a prompt leaves when it has been read
    per_layer, _, _ = model_bytes_and_flops(cfg, layers)
    nq, d, H = cfg["num_attention_heads"], cfg["head_dim"], cfg["hidden_size"]
    out = {"mixed14b_layers": layers}
    # as specified (portions of 512 tokens: 544 tokens a step), then with the scheduler's token_tile option (portions
    # shortened so that a step's tokens fill whole tiles of 128: 512 tokens a step)
    for key, tile in (("mixed14b", 0), ("mixed14b_tile128", 128)):
        engine.scheduler.token_tile = tile
        warm = 12
        while len(engine.scheduler.waiting) < (warm + steps) // 4 + 3:
            engine.add_request(rng.integers(0, V, size=prompt).tolist(), one)
        for _ in range(warm):
            engine.step()
        torch.cuda.synchronize()
        tokens0, launches0 = engine.runner.tokens_run, engine.runner.kernel_launches()
        replays0 = engine.runner.graph_replays
        left = [steps]
        def more():
            left[0] -= 1
            return left[0] >= 0
        ms = timed_steps(engine, torch, more)
        tokens = engine.runner.tokens_run - tokens0
        ctx_decode = sum(r.num_computed for r in decoders) / D
        portion_tokens = tokens - D * len(ms)
        flops = (2.0 * tokens * per_layer * layers                                              # every product of the layers
                 + layers * nq * 4.0 * d * (D * ctx_decode * len(ms) + portion_tokens * (prompt / 2))   # attention
                 + 2.0 * (D + 1) * V * H * len(ms))                                             # the output head on 33 rows
        out.update({f"{key}_tokens_per_s": round(tokens / sum(ms) * 1e3, 1), f"{key}_tokens_per_step": round(tokens / len(ms), 1),
                    f"{key}_frac": round(flops / (sum(ms) * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    f"{key}_replayed_steps": engine.runner.graph_replays - replays0,
                    f"{key}_launches_per_step": round((engine.runner.kernel_launches() - launches0) / len(ms), 1)})
        out.update({f"{key}_{k}": v for k, v in percentiles(ms).items()})
    return out


def run_longprompt8b(rng, pk, layers=0, prompt=32768, new=4) -> dict:
    """One request with a prompt of 32768 tokens through the engine with its default token budget of a step (576, as
    lucciola's scheduler: src/scheduler.cc:48): 57 portions, each behind a longer cached context than the one before.
    Time to the first generated token, prompt tokens a second and their share of the tensor peak."""
    import torch
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.llm import Engine
    from lucciola_b200.sampling.params import SamplingParams
    name, shape = SHAPES["8b"]
    layers = layers or shape["num_hidden_layers"]
    cfg = dict(shape, num_hidden_layers=layers)
    options = EngineOptions(dtype="bfloat16", block_size=16, max_blocks=(prompt + new) // 16 + 64, max_num_seqs=2,
                            max_model_len=prompt + new + 16)
    engine = Engine.from_random(cfg, seed=0, options=options)
    per_layer, _, _ = model_bytes_and_flops(cfg, layers)
    nq, d = cfg["num_attention_heads"], cfg["head_dim"]
    flops = 2.0 * prompt * per_layer * layers + layers * nq * 4.0 * d * prompt * (prompt / 2)
    ids = rng.integers(0, cfg["vocab_size"], size=prompt).tolist()
    best, steps, at = None, 0, {}
    for _ in range(3):                               # the first pass records the steps' shapes; the passes after replay them
        req = engine.add_request(ids, SamplingParams(max_new_tokens=new, ignore_eos=True))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        marks = [torch.cuda.Event(enable_timing=True)]
        marks[0].record()
        while not req.output:
            engine.step()
            marks.append(torch.cuda.Event(enable_timing=True))
            marks[-1].record()
        ttft = time.perf_counter() - t0
        while engine.has_unfinished():
            engine.step()
        steps = len(marks) - 1
        if best is None or ttft < best:
            best = ttft
            budget = options.max_tokens_per_step
            # the step that ends nearest below each context length, on the device's clock
            at = {k: round(marks[k // budget - 1].elapsed_time(marks[k // budget]), 3) for k in (2048, 8192, 16384, 32768)}
    return {"longprompt8b_layers": layers, "longprompt8b_prompt": prompt, "longprompt8b_budget": options.max_tokens_per_step,
            "longprompt8b_steps": steps, "longprompt8b_first_token_ms": round(best * 1e3, 1),
            "longprompt8b_tokens_per_s": round(prompt / best, 1),
            "longprompt8b_frac": round(flops / best / (pk["bf16_tflops"] * 1e12), 4),
            **{f"longprompt8b_step_ms_behind_{k // 1024}k": v for k, v in at.items()}}


def run_pressure32b(rng, pk, layers=0, B=64, prompt=4096, new=256) -> dict:
    """64 requests with prompts of 4096 tokens generate 256 tokens each from a pool that holds fewer pages than they
    need together (64 x 272): the scheduler preempts the request admitted last and recomputes it later; every request
    must finish."""
    import torch
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.llm import Engine
    from lucciola_b200.sampling.params import SamplingParams
    name, shape = SHAPES["32b"]
    layers = layers or shape["num_hidden_layers"]
    cfg = dict(shape, num_hidden_layers=layers)
    V = cfg["vocab_size"]
    pages = B * (prompt // 16) + B * 4                               # the prompts fit; 64 more tokens each, not 256
    options = EngineOptions(dtype="bfloat16", block_size=16, max_blocks=pages, max_num_seqs=B, max_tokens_per_step=2048 + B,
                            max_model_len=16384)
    engine = Engine.from_random(cfg, seed=0, options=options)
    _, weight_bytes, kv_per_token = model_bytes_and_flops(cfg, layers)
    reqs = [engine.add_request(rng.integers(0, V, size=prompt).tolist(), SamplingParams(max_new_tokens=new, ignore_eos=True))
            for _ in range(B)]
    torch.cuda.synchronize()
    ms, decode_fracs = [], []
    t_all = time.perf_counter()
    while engine.has_unfinished():
        cached = sum(r.num_computed for r in engine.scheduler.running)
        tokens0 = engine.runner.tokens_run
        t0 = time.perf_counter()
        events = engine.step()
        dt = (time.perf_counter() - t0) * 1e3
        ms.append(dt)
        if events and engine.runner.tokens_run - tokens0 == len(events):      # single tokens only: a decode step
            decode_fracs.append((weight_bytes + cached * kv_per_token) / (dt * 1e-3) / 1e9 / pk["hbm_gbs"])
    total_s = time.perf_counter() - t_all
    generated = sum(len(r.output) for r in reqs)
    st = engine.stats()
    out = {"pressure32b_tokens_per_s": round(generated / total_s, 1),
           "pressure32b_processed_tokens_per_s": round(engine.runner.tokens_run / total_s, 1),
           "pressure32b_preemptions": st["preemptions"],
           "pressure32b_finished": sum(len(r.output) == new for r in reqs), "pressure32b_requests": B,
           "pressure32b_pages": pages, "pressure32b_pages_for_all": B * -(-(prompt + new) // 16),
           # the median over the steps of single tokens (the steps that record a CUDA graph among them are far slower)
           "pressure32b_decode_hbm_frac": round(statistics.median(decode_fracs), 4) if decode_fracs else None,
           "pressure32b_decode_steps": len(decode_fracs),
           "pressure32b_layers": layers, "pressure32b_steps": len(ms), "pressure32b_seconds": round(total_s, 2)}
    out.update({f"pressure32b_{k}": v for k, v in percentiles(ms).items()})
    return out


def time_attention_key_ranges() -> int:
    """The prompt-attention kernel alone (CUDA events, 20 launches back to back after 3): one request's portion behind a
    cached context, its work items' keys whole and cut into 2 to 8 ranges, at 8B and 14B head counts; the last column
    is what `ops.attention_tcgen05_splits` takes.  Prints one line of JSON per case."""
    import math

    import torch

    from lucciola_b200 import ops
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream().cuda_stream
    nkv, d, page = 8, 128, 16
    for nq in (32, 40):
        for ctx, n in ((0, 512), (1536, 512), (7680, 512), (32256, 512), (7680, 128), (16384, 32), (7680, 1024)):
            pages = -(-(ctx + n) // page)
            kc = torch.randn(pages, nkv, page, d, device=dev).bfloat16()
            vc = torch.randn(pages, nkv, page, d, device=dev).bfloat16()
            table = torch.randperm(pages, dtype=torch.int32).view(1, pages).to(dev)
            pos = torch.arange(ctx, ctx + n, dtype=torch.int32, device=dev)
            q = torch.randn(n, nq, d, device=dev).bfloat16()
            out = torch.empty_like(q)
            per = 2 * (128 // (nq // nkv))
            tiles = sorted(((off, min(per, n - off), 0, 0) for off in range(0, n, per)), key=lambda t: -t[0])
            tl = torch.tensor(tiles, dtype=torch.int32, device=dev)
            us = {}
            for s in (1, 2, 3, 4, 8):
                run = lambda: ops.attention_tcgen05(q, out, kc, vc, pos, table, tl, nq, nkv, d, page, 0, 1 / math.sqrt(d), st, key_splits=s)
                for _ in range(3):
                    run()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                a.record()
                for _ in range(20):
                    run()
                b.record()
                torch.cuda.synchronize()
                us[s] = round(a.elapsed_time(b) / 20 * 1e3, 1)
            print(json.dumps({"query_heads": nq, "portion": n, "cached_context": ctx, "ctas": len(tiles) * nkv, "us_by_ranges": us,
                              "rule": ops.attention_tcgen05_splits(len(tiles), nkv, ctx + n), "device_error": ops.device_error()}), flush=True)
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192, help="context length the decode steps end at")
    ap.add_argument("--shape", choices=sorted(SHAPES), default="8b", help="layer sizes: the default Qwen3-8B shape or another of the family")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64 and the other workloads")
    ap.add_argument("--workloads", default="ctx768,mixed8b,mixed14b,longprompt8b,pressure32b",
                    help="which of the other workloads run (comma-separated; empty: none)")
    ap.add_argument("--no-key-ranges", action="store_true",
                    help="for comparison: the prompt-attention kernel never cuts the keys of its work items into ranges")
    ap.add_argument("--workload-layers", type=int, default=0,
                    help="fewer layers for the 14B and 32B workloads than their configurations have (reported with them)")
    ap.add_argument("--no-graph", action="store_true", help="do not replay decode steps from CUDA graphs")
    ap.add_argument("--fuse-norms", choices=["both", "entry", "middle", "none"], default="both",
                    help="where the residual add and the norm between two products run inside those products' epilogues: "
                         "between a block's feed-forward and the next block's mixer (entry), between mixer and feed-forward "
                         "(middle), both (the default), or none: always as a kernel of their own (for comparisons)")
    ap.add_argument("--no-fuse-norms", action="store_true", help="the same as --fuse-norms none")
    ap.add_argument("--profile", choices=["decode", "prefill", "mixed", "chunk"], default=None,
                    help="run one step of this kind between cudaProfilerStart/Stop and exit (for ncu --profile-from-start off); "
                         "mixed: --batch decoding requests at --context and one portion of --portion tokens of a new prompt; "
                         "chunk: a portion of --portion tokens of one request behind --context tokens of its prompt")
    ap.add_argument("--portion", type=int, default=512, help="tokens of the portion of a --profile mixed step")
    ap.add_argument("--time-kernel", choices=["attention_key_ranges"], default=None,
                    help="time one kernel alone over a grid of sizes, print a line of JSON a case, and exit")
    args = ap.parse_args()
    if args.time_kernel == "attention_key_ranges":
        return time_attention_key_ranges()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "JunkuiZhang/lucciola has no Python package or install target (CMake project whose configure step "
                          "fetches dependencies from the network and needs <print>, absent from g++ 13.3): pip install of the reference fails offline"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.warmup < 3:
        args.warmup = 3

    import numpy as np
    import torch

    from lucciola_b200 import ops
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.llm import Engine
    from lucciola_b200.engine.step import StepEntry
    from lucciola_b200.sampling.params import SamplingParams

    if args.no_key_ranges:
        ops.attention_tcgen05_splits = lambda *a, **k: 1
    if args.no_fuse_norms:
        args.fuse_norms = "none"
    if args.fuse_norms != "both":
        from lucciola_b200.parts.block import PreNormBlock
        PreNormBlock.fuse_norms = args.fuse_norms
    pk = peaks()
    shape_name, shape = SHAPES[args.shape]
    full_layers = shape["num_hidden_layers"]
    args.layers = args.layers or full_layers
    cfg = dict(shape, num_hidden_layers=args.layers)
    K, W, ctx = args.steps, args.warmup, args.context
    batches = [args.batch] + ([] if args.no_points else [b for b in (1, 64) if b != args.batch])
    page = 16
    max_b = max(batches)
    longest = ctx + args.portion if args.profile == "chunk" else max(ctx, args.prefill_tokens)
    pages = max_b * (-(-longest // page)) + 64
    options = EngineOptions(dtype="bfloat16", block_size=page, max_blocks=pages, max_num_seqs=max(64, max_b),
                            max_tokens_per_step=max(args.prefill_tokens, 2048) + max_b, max_model_len=longest,
                            use_cuda_graph=not (args.no_graph or args.profile))
    t_build = time.time()
    engine = Engine.from_random(cfg, seed=0, options=options)
    runner = engine.runner
    torch.cuda.synchronize()
    build_s = time.time() - t_build
    rng = np.random.default_rng(0)
    V = cfg["vocab_size"]
    _, weight_bytes, kv_per_token = model_bytes_and_flops(cfg, args.layers)

    def ev():
        return torch.cuda.Event(enable_timing=True)

    if args.profile:
        B, T = args.batch, args.prefill_tokens
        if args.profile == "prefill":
            entries = lambda i: [StepEntry(("p", i), rng.integers(0, V, size=T).tolist(), [T - 1])]
        elif args.profile == "chunk":
            # one request's next portion of --portion tokens behind --context tokens of its prompt (each call a new request)
            def entries(i):
                left = ctx
                while left > 0:
                    n = min(left, 2048)
                    runner.step([StepEntry(("p", i), rng.integers(0, V, size=n).tolist(), [])])
                    left -= n
                return [StepEntry(("p", i), rng.integers(0, V, size=args.portion).tolist(), [])]
        else:
            for j in range(B):                                        # bring B requests to the context, untimed
                left = ctx - 8
                while left > 0:
                    n = min(left, 2048)
                    runner.step([StepEntry(("d", j), rng.integers(0, V, size=n).tolist(), [])])
                    left -= n
            entries = lambda i: [StepEntry(("d", j), [int(rng.integers(0, V))], [0]) for j in range(B)]
            if args.profile == "mixed":
                decodes = entries
                entries = lambda i: decodes(i) + [StepEntry(("p", i), rng.integers(0, V, size=args.portion).tolist(), [])]
        for i in range(3):
            runner.step(entries(i))
            if args.profile != "decode":
                runner.finish(("p", i))
        last = entries(3)
        torch.cuda.synchronize()
        torch.cuda.profiler.start()
        runner.step(last)
        torch.cuda.synchronize()
        torch.cuda.profiler.stop()
        print(json.dumps({"profiled": args.profile, "layers": args.layers, "batch": B, "context": ctx, "tokens": T}))
        return 0

    # ---- prefill: one step over a prompt of --prefill-tokens tokens -----------------------------------
    T = args.prefill_tokens
    times = []
    for i in range(3 + 5):
        ids = rng.integers(0, V, size=T).tolist()
        a, b = ev(), ev()
        torch.cuda.synchronize()
        a.record()
        logits = runner.step([StepEntry(("prefill", i), ids, [T - 1])])
        b.record()
        torch.cuda.synchronize()
        runner.finish(("prefill", i))
        if i >= 3:
            times.append(a.elapsed_time(b))
    prefill_ms = statistics.median(times)
    flops = prefill_flops(cfg, args.layers, T)
    prefill = {"value": round(T / prefill_ms * 1e3, 1), "tokens": T, "ms": round(prefill_ms, 3),
               "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               # the same against the library product timed back to back for seconds, under the power cap as this step is
               "frac_of_sustained": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)}

    # ---- decode ------------------------------------------------------------------------------------------------------
    def decode_point(B: int, with_e2e: bool):
        """B requests brought to a context just short of `ctx`, then 2 x (W + K) decode steps."""
        total_steps = (2 if with_e2e else 1) * (W + K) + 2
        # requests whose prompt is done decode while the prompts behind them are still read: leave room
        early = (B - 1) * -(-ctx // options.max_tokens_per_step)
        ctx0 = ctx - total_steps - early - 1
        params = SamplingParams(max_new_tokens=total_steps + early + 8, temperature=0.0, ignore_eos=True)
        reqs = [engine.add_request(rng.integers(0, V, size=ctx0).tolist(), params) for _ in range(B)]
        while any(r.remaining > 1 or not r.output for r in reqs):       # prompts, in portions under the budget
            engine.step()
        torch.cuda.synchronize()
        out = {}
        if with_e2e:
            h2d0 = runner.h2d_bytes
            for _ in range(W):
                engine.step()
            with ClockSampler() as clocks_e2e:
                a, b = ev(), ev()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                a.record()
                h2d1 = runner.h2d_bytes
                for _ in range(K):
                    engine.step()
                b.record()
                torch.cuda.synchronize()
                wall = time.perf_counter() - t0
            ms = max(a.elapsed_time(b), wall * 1e3)
            out["e2e"] = {"value": round(B * K / ms * 1e3, 2), "unit": "tokens/s", "ms_per_step": round(ms / K, 4),
                          "h2d_bytes_per_step": int((runner.h2d_bytes - h2d1) / K), "d2h_bytes_per_step": 4 * B}
        # device-timed: the step function and the sampler; token ids come from the host, nothing is read back
        rids = [r.rid for r in reqs]
        feed = [[int(x) for x in rng.integers(0, V, size=W + K)] for _ in range(B)]
        tokens = torch.empty(B, dtype=torch.int32, device=runner.device)

        def one(i):
            logits = runner.step([StepEntry(rid, [feed[j][i]], [0]) for j, rid in enumerate(rids)])
            ops.sample(tokens, logits, torch.cuda.current_stream().cuda_stream)

        for i in range(W):
            one(i)
        launches0 = runner.kernel_launches()
        with ClockSampler() as clocks:
            a, b = ev(), ev()
            torch.cuda.synchronize()
            a.record()
            for i in range(W, W + K):
                one(i)
            b.record()
            torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        launches = runner.kernel_launches() - launches0
        final_ctx = max(runner.length(r) for r in rids)
        cached_tokens = sum(runner.length(r) for r in rids) - B * K / 2         # mean over the timed steps
        step_bytes = weight_bytes + cached_tokens * kv_per_token
        out.update({"value": B * K / ms * 1e3, "ms_per_step": ms / K, "launches": launches, "clocks": clocks.summary(),
                    "bytes": step_bytes, "gbs": step_bytes / (ms / K * 1e-3) / 1e9, "final_context": final_ctx})
        for r in reqs:
            engine.abort(r.rid)
        return out

    results = {}
    for B in sorted(batches, reverse=True):
        results[B] = decode_point(B, with_e2e=(B == args.batch))
    main_r = results[args.batch]
    # The other workloads: each on its own; a failure of one is recorded, not fatal to the line.
    extra: dict = {}
    workloads = [] if args.no_points else [w for w in args.workloads.split(",") if w]
    if "ctx768" in workloads:
        try:
            extra.update(run_ctx768(engine, cfg, args.layers, rng, pk))
        except Exception as e:                                       # noqa: BLE001
            extra["ctx768_error"] = f"{type(e).__name__}: {e}"[:200]
    if "mixed8b" in workloads and max_b >= 32:
        try:
            extra.update(run_mixed8b(runner, cfg, rng, ctx))
        except Exception as e:                                       # noqa: BLE001
            extra["mixed8b_error"] = f"{type(e).__name__}: {e}"[:200]
    err = ops.device_error()
    if any(w in workloads for w in ("mixed14b", "longprompt8b", "pressure32b")):
        import gc
        del engine, runner, logits
        gc.collect()
        torch.cuda.empty_cache()
        for w, fn in (("mixed14b", run_mixed14b), ("longprompt8b", run_longprompt8b), ("pressure32b", run_pressure32b)):
            if w not in workloads:
                continue
            try:
                extra.update(fn(rng, pk, args.workload_layers))
            except Exception as e:                                   # noqa: BLE001
                extra[w + "_error"] = f"{type(e).__name__}: {e}"[:200]
            gc.collect()
            torch.cuda.empty_cache()
        err = err or ops.device_error()

    line = {
        "metric": "decode tokens/s (%s, bf16, batch %d, context %d)" % (shape_name, args.batch, ctx),
        "value": round(main_r["value"], 2), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(main_r["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: uniform random token ids, random weights N(0, 0.02)", "impl": "ours",
        "config": {"model": shape_name, "layers": args.layers, "layers_of_configuration": full_layers,
                   "hidden_size": cfg["hidden_size"], "num_attention_heads": cfg["num_attention_heads"],
                   "num_key_value_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate_size": cfg["intermediate_size"], "vocab_size": cfg["vocab_size"], "global_batch": args.batch, "seq_len": ctx,
                   "context_len": main_r["final_context"], "page_size": page, "parallelism": "single GPU",
                   "cuda_graph": bool(options.use_cuda_graph), "fused_norms": args.fuse_norms, "l2": "inputs larger than L2 (%.0f GB of weights a step)" % (weight_bytes / 1e9),
                   "prefill_tokens": T, "peaks": pk["source"]},
        "e2e": main_r.get("e2e"),
        "gpu_launches": int(main_r["launches"]),
        "clocks": main_r["clocks"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(main_r["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main_r["gbs"] / pk["hbm_gbs"], 4)},
        "points": {**{f"decode_b{B}": round(r["value"], 2) for B, r in results.items() if B != args.batch}, **extra},
        "points_roofline_frac": {f"decode_b{B}": round(r["gbs"] / pk["hbm_gbs"], 4) for B, r in results.items()},
        "device_error": err, "build_s": round(build_s, 1),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
