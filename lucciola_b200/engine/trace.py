"""Trace replay: feed given token ids through the model step by step and write the logits.

Nothing is sampled.  The steps go through the same runner, model, cache and kernels that
generation uses.  Input: one JSON object a line on standard input,

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries` are one batch; `want` are the places among an entry's tokens whose logits are written;
`end` lists the requests that are finished after this step.  For a step in which something is
wanted, `<out>/<step>.f32` holds the logits [wanted, vocab] as little-endian float32, in the order
of the entries and of `want`.  After every step a line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path



def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"],
                    help="bfloat16: the kernels and precisions of serving; float32: everything in true 32-bit")
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each request rounded up to 64)")
    ap.add_argument("--block-size", type=int, default=16, help="tokens in a cache page (must divide 64)")
    ap.add_argument("--cuda-graph", action="store_true",
                    help="record every step whose shape allows it as a CUDA graph when the shape first comes, and replay "
                         "the recording for later steps of that shape (bfloat16 only; off: every step launches its kernels)")
    args = ap.parse_args(argv)
    if args.max_tokens <= 0:
        ap.error("--max-tokens must be positive")
    if 64 % args.block_size:
        ap.error("--block-size must divide 64")

    from ..config.engine_options import EngineOptions
    from .load import build_runner
    from .step import StepEntry

    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    pages = -(-args.max_tokens // args.block_size)
    options = EngineOptions(dtype=args.dtype, block_size=args.block_size, max_blocks=pages, max_num_seqs=8,
                            use_cuda_graph=args.cuda_graph, graph_after=1, max_shape_graphs=256)
    runner = build_runner(args.model, options, num_pages=pages)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step_id = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in rec.get("entries", [])]
        logits = runner.step(entries) if entries else None
        if logits is not None:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            arr.tofile(out / f"{step_id}.f32")
        for rid in rec.get("end", []):
            runner.finish(rid)
        print(f"done {step_id}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
