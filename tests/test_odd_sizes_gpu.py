"""Sizes off the beaten path, through the whole engine against the plain implementation (GPU): head sizes in steps of
16 on both sides of what the tensor-core attention kernels take, head counts and groups that are no power of two, widths
whose products fall back to the 32-bit pipes (not a multiple of 8), an intermediate size that keeps SwiGLU a kernel of
its own, odd vocabularies, pages of 32 and 64.  Each configuration runs whole, with a decoded tail and in portions, in
float32 and in bfloat16: a kernel either takes a size and is right, or the engine routes around it."""
import pytest

import replay_util as ru

pytestmark = pytest.mark.gpu

BASE = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "attention_bias": False,
        "torch_dtype": "bfloat16", "max_position_embeddings": 256, "tie_word_embeddings": False}
# name -> (sizes, page size)
ODD = {
    "head80_groups2": (dict(num_hidden_layers=2, hidden_size=1000, num_attention_heads=6, num_key_value_heads=3, head_dim=80,
                            intermediate_size=1504, vocab_size=777, rope_theta=1e4, rms_norm_eps=1e-6), 16),
    "head144_plain_attention": (dict(num_hidden_layers=2, hidden_size=264, num_attention_heads=4, num_key_value_heads=4, head_dim=144,
                                     intermediate_size=320, vocab_size=100, rope_theta=1e6, rms_norm_eps=1e-5), 32),
    "width_no_multiple_of_8": (dict(num_hidden_layers=2, hidden_size=1004, num_attention_heads=2, num_key_value_heads=1, head_dim=64,
                                    intermediate_size=500, vocab_size=1201, rope_theta=5e4, rms_norm_eps=1e-6,
                                    tie_word_embeddings=True), 16),
    "head128_groups8_pages64": (dict(num_hidden_layers=3, hidden_size=768, num_attention_heads=16, num_key_value_heads=2, head_dim=128,
                                     intermediate_size=1088, vocab_size=515, rope_theta=1e6, rms_norm_eps=1e-6), 64),
    "head112_mqa_groups5": (dict(num_hidden_layers=2, hidden_size=560, num_attention_heads=5, num_key_value_heads=1, head_dim=112,
                                 intermediate_size=1216, vocab_size=333, rope_theta=1e5, rms_norm_eps=3e-6), 16),
    "head16_many_heads": (dict(num_hidden_layers=2, hidden_size=520, num_attention_heads=33, num_key_value_heads=11, head_dim=16,
                               intermediate_size=136, vocab_size=259, rope_theta=1e4, rms_norm_eps=1e-6), 16),
}


@pytest.fixture(scope="module")
def odd_models(tmp_path_factory):
    from lucciola_b200.weights import write_random_model
    out = {}
    for i, (name, (sizes, _page)) in enumerate(ODD.items()):
        folder = tmp_path_factory.mktemp(name)
        write_random_model(dict(BASE, **sizes), folder, 40 + i, std=0.04, norm_std=0.1)
        out[name] = folder
    return out


def ids_for(name, n, salt=0):
    import numpy as np
    vocab = ODD[name][0]["vocab_size"]
    return [int(x) for x in np.random.default_rng(7 * salt + n + len(name)).integers(0, vocab, size=n)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ODD))
def test_odd_sizes_under_three_cuttings(odd_models, name, dtype):
    from lucciola_b200.config import EngineOptions
    from lucciola_b200.engine.load import build_runner
    page = ODD[name][1]
    reqs = {f"{name}-{n}": ids_for(name, n, salt=i) for i, n in enumerate((3, 45, 130))}
    for cut in ("whole", "tail_decoded", "portions"):
        steps = getattr(ru, cut)(reqs)
        pages = -(-ru.max_live_tokens(steps) // page) + 2
        runner = build_runner(odd_models[name], EngineOptions(dtype=dtype, block_size=page, max_blocks=pages, max_num_seqs=4,
                                                              graph_after=1), num_pages=pages)
        got = ru.replay(runner, steps, poison=True)
        ru.compare(got, odd_models[name], reqs, dtype)
        assert all(p.num_free == p.num_pages for p in runner.manager.pools)
    from lucciola_b200 import ops
    assert ops.device_error() == 0
