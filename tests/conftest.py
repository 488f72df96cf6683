"""Shared test equipment: tiny configurations, model folders with random weights, the gpu marker."""
from __future__ import annotations

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(autouse=True)
def _seeded(request):
    """Every test starts from the same random state whatever ran before it (LUCCIOLA_TEST_SEED shifts all of them,
    to look for tolerances that only hold for lucky inputs)."""
    import os
    import zlib
    import torch
    torch.manual_seed(zlib.crc32(request.node.nodeid.encode()) + int(os.environ.get("LUCCIOLA_TEST_SEED", "0")))
    yield


# Three tiny configurations of the architecture that differ in every size and option.
# A and B have the sizes of the two tiny Qwen3 workloads this engine is specified on; C adds sliding layers.
TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 128, "hidden_act": "silu", "attention_bias": False,
    "use_sliding_window": False, "sliding_window": None, "eos_token_id": 255, "torch_dtype": "bfloat16",
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 8, "num_key_value_heads": 1, "head_dim": 32,
    "intermediate_size": 224, "vocab_size": 503, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 256, "hidden_act": "silu", "attention_bias": False,
    "torch_dtype": "bfloat16",
}
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 4, "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48,
    "intermediate_size": 176, "vocab_size": 300, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 512, "hidden_act": "silu", "attention_bias": False,
    "use_sliding_window": True, "sliding_window": 24,
    "layer_types": ["full_attention", "sliding_attention", "sliding_attention", "full_attention"],
    "torch_dtype": "bfloat16",
}
# D is small but has the head size (128) and the widths (512: products long enough to be split) at which the engine
# takes its fused paths: heads finished in the q|k|v product's epilogue, residual add and norm inside the o and down
# products, the tensor-memory attention kernel, keys and values fetched by TMA.
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "num_hidden_layers": 2, "hidden_size": 512, "num_attention_heads": 4, "num_key_value_heads": 1, "head_dim": 128,
    "intermediate_size": 576, "vocab_size": 331, "rope_theta": 500000.0, "rms_norm_eps": 2e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 512, "hidden_act": "silu", "attention_bias": False,
    "torch_dtype": "bfloat16",
}
# name -> (config, seed, std of linear weights, std of norm weights around 1, page size)
TINY = {
    "A": (TINY_A, 0, 0.02, 0.1, 16),
    "B": (TINY_B, 1, 0.05, 0.2, 8),
    "C": (TINY_C, 2, 0.08, 0.15, 16),
    "D": (TINY_D, 3, 0.04, 0.1, 16),
}


@pytest.fixture(scope="session")
def tiny_models(tmp_path_factory):
    """Model folders (config.json, model.safetensors) of the tiny configurations, written once a session."""
    from lucciola_b200.weights import write_random_model

    out = {}
    for name, (cfg, seed, std, norm_std, _page) in TINY.items():
        folder = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(cfg, folder, seed, std=std, norm_std=norm_std)
        out[name] = folder
    return out


def tokens_for(name: str, length: int, salt: int = 0) -> list[int]:
    """Token ids drawn uniformly from the vocabulary, the same on every run."""
    import numpy as np

    cfg = TINY[name][0]
    rng = np.random.default_rng(1000 * salt + sum(map(ord, name)) + length)
    return [int(x) for x in rng.integers(0, cfg["vocab_size"], size=length)]
