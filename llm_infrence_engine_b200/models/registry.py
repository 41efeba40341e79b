"""One registry from the architecture's name in ``config.json`` to its configuration class and builder.

The reference has a single model class and builds it directly (src/miniserve/loader.py:36-39); the
name under ``architectures`` is never read there. Here that name chooses the model everywhere: the
loader, the engine, the replay program and the command line all come through ``build_model_spec``.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Mapping, Tuple

from ..config.model_config import ConfigError, architecture_name
from .spec import ModelSpec

_REGISTRY: Dict[str, Tuple[Any, Callable[[Any], ModelSpec]]] = {}


def register_architecture(name: str, config_cls, builder: Callable[[Any], ModelSpec], replace: bool = False) -> None:
    """``config_cls.from_dict(config.json) -> cfg``; ``builder(cfg) -> ModelSpec``."""
    if name in _REGISTRY and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _REGISTRY[name] = (config_cls, builder)


def known_architectures() -> list:
    return sorted(_REGISTRY)


def lookup(name: str):
    if name not in _REGISTRY:
        raise ConfigError(f"architecture '{name}' is not known; known: {', '.join(known_architectures()) or 'none'}")
    return _REGISTRY[name]


def parse_config(config_json: Mapping[str, Any]):
    config_cls, _ = lookup(architecture_name(config_json))
    return config_cls.from_dict(config_json)


def build_model_spec(config_json: Mapping[str, Any]) -> ModelSpec:
    """The model that ``config.json`` names, built from its own keys; no weights yet."""
    config_cls, builder = lookup(architecture_name(config_json))
    return builder(config_cls.from_dict(config_json))
