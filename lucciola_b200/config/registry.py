"""One registry from the architecture's name in config.json to its model.

An entry couples the name (`architectures[0]`) with the typed configuration
class and the function that composes the model from parts.  lucciola has no
registry: its engine holds a QwenModel by value (include/async_engine.h:40).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Mapping

from .model_config import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[Mapping[str, Any]], Any]
    build: Callable[..., Any]      # build(config, runtime) -> DecoderModel


_REGISTRY: dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict: Callable[[Mapping[str, Any]], Any],
                          build: Callable[..., Any], replace: bool = False) -> None:
    if name in _REGISTRY and not replace:
        raise ValueError(f"architecture {name!r} is already registered")
    _REGISTRY[name] = Architecture(name, config_from_dict, build)


def known_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_REGISTRY)


def resolve_architecture(config_dict: Mapping[str, Any]) -> Architecture:
    """The registered architecture that config.json names."""
    _ensure_builtin()
    archs = config_dict.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError("config.json has no 'architectures' list; known architectures: " + ", ".join(sorted(_REGISTRY)))
    name = archs[0]
    if name not in _REGISTRY:
        raise ConfigError(f"unknown architecture {name!r}; known architectures: " + ", ".join(sorted(_REGISTRY)))
    return _REGISTRY[name]


def _ensure_builtin() -> None:
    # The built-in model registers itself on import.
    from ..models import qwen3  # noqa: F401
