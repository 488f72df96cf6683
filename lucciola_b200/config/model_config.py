"""Typed configuration of the Qwen3 dense decoder, read from config.json.

Every size and constant of the model comes from the file; none has a default
value in code.  lucciola reads seven integers with defaults that describe one
particular checkpoint and hard-codes the rest (src/qwen.cc:45-66 reads
hidden_size, intermediate_size, num_attention_heads, num_key_value_heads,
head_dim, num_hidden_layers, vocab_size; eps 1e-6 and theta 1e6 are literals at
src/qwen.cc:588,636).  Here a missing size or constant is an error, and options
that this engine does not implement are refused instead of ignored.

Two keys are derived when absent, as lucciola derives them
(src/qwen.cc:52-56): num_key_value_heads = num_attention_heads and
head_dim = hidden_size / num_attention_heads.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Mapping


class ConfigError(ValueError):
    """config.json is missing, incomplete, inconsistent or asks for something unsupported."""


FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"

_REQUIRED = (
    "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
    "vocab_size", "rms_norm_eps", "rope_theta", "max_position_embeddings",
)


def _as_int(d: Mapping[str, Any], key: str) -> int:
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config key {key!r} must be an integer, got {v!r}")
    return v


def _as_float(d: Mapping[str, Any], key: str) -> float:
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config key {key!r} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class Qwen3Config:
    architecture: str
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool = False
    # One entry per layer: FULL_ATTENTION or SLIDING_ATTENTION.
    layer_types: tuple[str, ...] = ()
    # Number of keys a sliding layer sees, the query's own position included.
    sliding_window: int | None = None
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    torch_dtype: str = "bfloat16"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    ARCHITECTURE = "Qwen3ForCausalLM"

    # ---- reading -------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in d or d[k] is None]
        if missing:
            raise ConfigError("config.json lacks required key(s): " + ", ".join(missing))
        archs = d.get("architectures") or [cls.ARCHITECTURE]
        hidden = _as_int(d, "hidden_size")
        heads = _as_int(d, "num_attention_heads")
        kv_heads = _as_int(d, "num_key_value_heads") if d.get("num_key_value_heads") is not None else heads
        if d.get("head_dim") is not None:
            head_dim = _as_int(d, "head_dim")
        else:
            if heads <= 0 or hidden % heads:
                raise ConfigError(f"head_dim is absent and hidden_size {hidden} is not a multiple of num_attention_heads {heads}")
            head_dim = hidden // heads
        layers = _as_int(d, "num_hidden_layers")

        # Options this engine refuses rather than ignores.
        if d.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {d['hidden_act']!r} is not supported (only 'silu')")
        if d.get("attention_bias", False):
            raise ConfigError("attention_bias=true is not supported: the Qwen3 dense decoder has no projection biases")
        if d.get("rope_scaling") is not None:
            raise ConfigError(f"rope_scaling {d['rope_scaling']!r} is not supported")
        if d.get("mlp_only_layers") or d.get("num_experts"):
            raise ConfigError("expert layers are not part of the Qwen3 dense decoder")

        window = d.get("sliding_window")
        use_window = bool(d.get("use_sliding_window", False))
        if d.get("layer_types") is not None:
            layer_types = tuple(d["layer_types"])
            if len(layer_types) != layers:
                raise ConfigError(f"layer_types has {len(layer_types)} entries for {layers} layers")
            bad = sorted({t for t in layer_types if t not in (FULL_ATTENTION, SLIDING_ATTENTION)})
            if bad:
                raise ConfigError(f"unknown layer type(s) {bad}; known: {FULL_ATTENTION}, {SLIDING_ATTENTION}")
        elif use_window:
            # The first max_window_layers layers attend to everything, the rest to a window.
            if d.get("max_window_layers") is None:
                raise ConfigError("use_sliding_window=true needs max_window_layers or layer_types")
            first_sliding = _as_int(d, "max_window_layers")
            layer_types = tuple(SLIDING_ATTENTION if i >= first_sliding else FULL_ATTENTION for i in range(layers))
        else:
            layer_types = (FULL_ATTENTION,) * layers
        if SLIDING_ATTENTION in layer_types:
            if window is None:
                raise ConfigError("sliding layers need sliding_window")
            window = _as_int(d, "sliding_window")
            if window <= 0:
                raise ConfigError(f"sliding_window must be positive, got {window}")
        else:
            window = None

        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else (tuple(int(x) for x in eos) if isinstance(eos, (list, tuple)) else (int(eos),))
        known = set(_REQUIRED) | {
            "architectures", "num_key_value_heads", "head_dim", "hidden_act", "attention_bias", "rope_scaling",
            "sliding_window", "use_sliding_window", "max_window_layers", "layer_types", "eos_token_id",
            "bos_token_id", "torch_dtype", "dtype", "tie_word_embeddings", "mlp_only_layers", "num_experts",
        }
        cfg = cls(
            architecture=str(archs[0]),
            hidden_size=hidden,
            intermediate_size=_as_int(d, "intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            vocab_size=_as_int(d, "vocab_size"),
            rms_norm_eps=_as_float(d, "rms_norm_eps"),
            rope_theta=_as_float(d, "rope_theta"),
            max_position_embeddings=_as_int(d, "max_position_embeddings"),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            layer_types=layer_types,
            sliding_window=window,
            eos_token_ids=eos_ids,
            bos_token_id=None if d.get("bos_token_id") is None else int(d["bos_token_id"]),
            torch_dtype=str(d.get("torch_dtype") or d.get("dtype") or "bfloat16"),
            extra={k: v for k, v in d.items() if k not in known},
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_folder(cls, folder: str | Path) -> "Qwen3Config":
        return cls.from_dict(read_config_json(folder))

    # ---- checks --------------------------------------------------------
    def validate(self) -> None:
        for name in ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                     "num_key_value_heads", "head_dim", "vocab_size", "max_position_embeddings"):
            if getattr(self, name) <= 0:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for the rotary position encoding")
        if not (self.rms_norm_eps > 0):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not (self.rope_theta > 0):
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")
        if len(self.layer_types) != self.num_hidden_layers:
            raise ConfigError("layer_types does not match num_hidden_layers")

    # ---- writing -------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        d: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "hidden_act": "silu",
            "attention_bias": False,
            "rope_scaling": None,
            "torch_dtype": self.torch_dtype,
        }
        if self.sliding_window is not None:
            d["use_sliding_window"] = True
            d["sliding_window"] = self.sliding_window
            d["layer_types"] = list(self.layer_types)
        else:
            d["use_sliding_window"] = False
            d["sliding_window"] = None
        if self.eos_token_ids:
            d["eos_token_id"] = self.eos_token_ids[0] if len(self.eos_token_ids) == 1 else list(self.eos_token_ids)
        if self.bos_token_id is not None:
            d["bos_token_id"] = self.bos_token_id
        return d


def read_config_json(folder: str | Path) -> dict[str, Any]:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path} does not exist: a model folder needs config.json")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path} is not valid JSON: {e}") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path} must hold a JSON object")
    return d
