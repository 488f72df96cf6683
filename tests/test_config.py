"""Configuration and registry (no GPU)."""
import json

import pytest

from conftest import TINY_A, TINY_B, TINY_C
from lucciola_b200.config import (ConfigError, Qwen3Config, known_architectures, read_config_json,
                                  resolve_architecture, FULL_ATTENTION, SLIDING_ATTENTION)


def test_reads_every_size_from_the_file():
    c = Qwen3Config.from_dict(TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim) == (3, 96, 8, 1, 32)
    assert (c.intermediate_size, c.vocab_size, c.max_position_embeddings) == (224, 503, 256)
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and c.tie_word_embeddings is False
    assert c.layer_types == (FULL_ATTENTION,) * 3 and c.sliding_window is None


def test_derived_keys():
    d = dict(TINY_A)
    del d["head_dim"], d["num_key_value_heads"]
    c = Qwen3Config.from_dict(d)
    assert c.head_dim == 64 // 4 and c.num_key_value_heads == 4


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                                 "vocab_size", "rms_norm_eps", "rope_theta", "max_position_embeddings"])
def test_missing_required_key_is_an_error(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen3Config.from_dict(d)


@pytest.mark.parametrize("patch,word", [
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"attention_bias": True}, "attention_bias"),
    ({"rope_scaling": {"type": "yarn", "factor": 4}}, "rope_scaling"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 15}, "even"),
    ({"rms_norm_eps": 0}, "rms_norm_eps"),
    ({"num_hidden_layers": 0}, "num_hidden_layers"),
    ({"hidden_size": "64"}, "integer"),
    ({"layer_types": ["full_attention"]}, "layer_types"),
    ({"layer_types": ["full_attention", "strided"]}, "unknown layer type"),
    ({"use_sliding_window": True, "sliding_window": 8}, "max_window_layers"),
    ({"layer_types": ["full_attention", "sliding_attention"], "sliding_window": None}, "sliding_window"),
])
def test_refuses_what_it_does_not_implement(patch, word):
    d = dict(TINY_A)
    d.update(patch)
    with pytest.raises(ConfigError, match=word):
        Qwen3Config.from_dict(d)


def test_window_layers_both_spellings():
    c = Qwen3Config.from_dict(TINY_C)
    assert c.layer_types == (FULL_ATTENTION, SLIDING_ATTENTION, SLIDING_ATTENTION, FULL_ATTENTION) and c.sliding_window == 24
    d = dict(TINY_C)
    del d["layer_types"]
    d["max_window_layers"] = 3
    c2 = Qwen3Config.from_dict(d)
    assert c2.layer_types == (FULL_ATTENTION,) * 3 + (SLIDING_ATTENTION,)


def test_round_trip_through_json(tmp_path):
    for cfg in (TINY_A, TINY_B, TINY_C):
        c = Qwen3Config.from_dict(cfg)
        (tmp_path / "config.json").write_text(json.dumps(c.to_dict()))
        assert Qwen3Config.from_folder(tmp_path) == c


def test_config_file_errors(tmp_path):
    with pytest.raises(ConfigError, match="does not exist"):
        read_config_json(tmp_path)
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError, match="not valid JSON"):
        read_config_json(tmp_path)


def test_registry():
    assert "Qwen3ForCausalLM" in known_architectures()
    arch = resolve_architecture(TINY_A)
    assert arch.name == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError, match="unknown architecture 'LlamaForCausalLM'.*Qwen3ForCausalLM"):
        resolve_architecture({"architectures": ["LlamaForCausalLM"]})
    with pytest.raises(ConfigError, match="architectures"):
        resolve_architecture({})


def test_eos_ids():
    assert Qwen3Config.from_dict(TINY_A).eos_token_ids == (255,)
    d = dict(TINY_A, eos_token_id=[7, 9])
    assert Qwen3Config.from_dict(d).eos_token_ids == (7, 9)
