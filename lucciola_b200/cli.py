"""Command line in the manner of lucciola's chat program (examples/qwen_dynamic.cc:13-111): a loop
that reads a prompt from standard input, runs it through the scheduler and the step function and
streams what is generated, until `exit` or end of input.  lucciola's program has no options (model
path, 1 024 pages of 16 tokens and a cap of 100 new tokens are literals at
examples/qwen_dynamic.cc:22-27, 92); here they are options with lucciola's names where it has
names: max_blocks, block_size, max_new_tokens.

A prompt is a line of token ids separated by blanks or commas; tokenisation is outside this engine.
"""
from __future__ import annotations

import argparse
import re
import sys


def parse_ids(line: str) -> list[int]:
    return [int(x) for x in re.split(r"[\s,]+", line.strip()) if x]


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="lucciola_chat", description="Generate from prompts of token ids read from standard input.")
    ap.add_argument("--model", required=True, help="folder with config.json and *.safetensors")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-blocks", type=int, default=1024, help="pages of the cache (0: as many as fit)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens in a page")
    ap.add_argument("--max-new-tokens", type=int, default=100)
    ap.add_argument("--max-tokens-per-step", type=int, default=576)
    ap.add_argument("--prefill-chunk", type=int, default=0, help="most tokens of one prompt in a step (0: what the step's budget leaves)")
    ap.add_argument("--max-num-seqs", type=int, default=None, help="requests that hold pages at a time")
    ap.add_argument("--max-model-len", type=int, default=None, help="longest sequence (default: the model's positions)")
    ap.add_argument("--no-cuda-graph", action="store_true", help="run decode steps kernel by kernel instead of replaying recorded graphs")
    ap.add_argument("--temperature", type=float, default=0.0, help="0: greedy")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--prompt-ids", default=None, help="one prompt given on the command line instead of standard input")
    args = ap.parse_args(argv)

    from .config.engine_options import EngineOptions
    from .engine.llm import Engine
    from .sampling.params import SamplingParams

    options = EngineOptions(dtype=args.dtype, max_blocks=args.max_blocks, block_size=args.block_size,
                            max_tokens_per_step=args.max_tokens_per_step, prefill_chunk=args.prefill_chunk,
                            use_cuda_graph=not args.no_cuda_graph)
    if args.max_num_seqs is not None:
        options.max_num_seqs = args.max_num_seqs
    if args.max_model_len is not None:
        options.max_model_len = args.max_model_len
    engine = Engine(args.model, options=options)
    params = SamplingParams(max_new_tokens=args.max_new_tokens, temperature=args.temperature, seed=args.seed,
                            ignore_eos=args.ignore_eos)

    def run(ids: list[int]) -> None:
        def show(token: int, done: bool) -> None:
            print(token, end="\n" if done else " ", flush=True)
        engine.add_request(ids, params, show)
        while engine.has_unfinished():
            engine.step()

    if args.prompt_ids is not None:
        run(parse_ids(args.prompt_ids))
        return 0
    interactive = sys.stdin.isatty()
    while True:
        if interactive:
            print(">> ", end="", flush=True)
        line = sys.stdin.readline()
        if not line or line.strip() == "exit":
            break
        if not line.strip():
            continue
        try:
            run(parse_ids(line))
        except ValueError as e:
            print(f"refused: {e}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
