from .model_config import (ConfigError, Qwen3Config, read_config_json, FULL_ATTENTION, SLIDING_ATTENTION)
from .registry import (Architecture, known_architectures, register_architecture, resolve_architecture)
from .engine_options import EngineOptions

__all__ = [
    "ConfigError", "Qwen3Config", "read_config_json", "FULL_ATTENTION", "SLIDING_ATTENTION",
    "Architecture", "known_architectures", "register_architecture", "resolve_architecture", "EngineOptions",
]
