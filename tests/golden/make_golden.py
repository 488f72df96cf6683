"""Writes tests/golden/plain_tiny.json: a few numbers of the plain implementation on the tiny models.

lucciola's model code is CUDA kernels and cannot be run on a CPU, so these are outputs of
tests/plain_qwen3.py itself, kept to notice when that file changes its results (what ties that file
to lucciola's own code is tests/test_reference_kernels_gpu.py, on a GPU).  Run from the repository root:  python tests/golden/make_golden.py
"""
import json
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import plain_qwen3 as plain  # noqa: E402
from conftest import TINY, tokens_for  # noqa: E402
from lucciola_b200.weights import write_random_model  # noqa: E402

out = {}
for name, (cfg, seed, std, norm_std, _page) in TINY.items():
    with tempfile.TemporaryDirectory() as d:
        write_random_model(cfg, d, seed, std=std, norm_std=norm_std)
        c, w = plain.read_model(d)
        ids = tokens_for(name, 24)
        logits = plain.forward(c, w, ids)
        out[name] = {"tokens": ids, "last_row_first8": [float(x) for x in logits[-1, :8]],
                     "argmax_last4": [int(r.argmax()) for r in logits[-4:]]}
(Path(__file__).parent / "plain_tiny.json").write_text(json.dumps(out, indent=1))
print("wrote", Path(__file__).parent / "plain_tiny.json")
