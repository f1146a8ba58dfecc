"""One registry from an architecture's name (``config.json`` -> ``architectures[0]``) to its
configuration class and model builder.

The reference hard-wires its single model class (``src/engine/engine.h:61``); here the engine,
scheduler, sampler and replay tool only ever see what this registry returns.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Dict, Type

from .model_config import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class ArchitectureEntry:
    name: str
    config_cls: Type[ModelConfig]
    build: Callable[..., Any]          # build(config) -> ModelSpec (parts + order + tensor map)


_ARCHITECTURES: Dict[str, ArchitectureEntry] = {}


def register_architecture(name: str, config_cls: Type[ModelConfig],
                          build: Callable[..., Any], *, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise ValueError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = ArchitectureEntry(name, config_cls, build)


def registered_architectures():
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> ArchitectureEntry:
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture '{name}'; registered: "
                          f"{', '.join(registered_architectures()) or '(none)'}")
    return _ARCHITECTURES[name]


def config_from_dict(d: Dict[str, Any]) -> ModelConfig:
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: key 'architectures' must be a non-empty list of names")
    return get_architecture(archs[0]).config_cls.from_json_dict(d)


def load_config(folder: str) -> ModelConfig:
    """Reads ``folder/config.json`` and returns the typed config of its architecture."""
    return config_from_dict(read_config_json(folder))
