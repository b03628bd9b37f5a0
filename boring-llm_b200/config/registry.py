"""One registry from an architecture's name to its configuration class and model builder.

Role of `rope_style_for_arch` (src/model.br:328-334): the architecture string selects behaviour,
and an unknown one raises with the list of supported names (src/model.br:334).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Iterable

from .model_config import ConfigError, architecture_name, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type          # has `from_dict(dict)` and `to_dict()`
    build: Callable           # build(config) -> parts.model.DecoderModel, weights not yet loaded


_REGISTRY: Dict[str, Architecture] = {}


def register_architecture(names: Iterable[str], config_cls: type, build: Callable) -> None:
    """Registers a configuration class and a builder under every given name
    (`architectures[0]` values and `model_type` values alike)."""
    names = list(names)
    if not names:
        raise ValueError("register_architecture: at least one name is needed")
    for n in names:
        _REGISTRY[n] = Architecture(n, config_cls, build)


def unregister_architecture(names: Iterable[str]) -> None:
    for n in names:
        _REGISTRY.pop(n, None)


def registered_architectures():
    return sorted(_REGISTRY)


def resolve_architecture(config_dict: dict) -> Architecture:
    name = architecture_name(config_dict)
    if name not in _REGISTRY and isinstance(config_dict.get("model_type"), str):
        name = config_dict["model_type"] if config_dict["model_type"] in _REGISTRY else name
    if name not in _REGISTRY:
        raise ConfigError(
            f"unsupported architecture {name!r}; supported: {', '.join(registered_architectures())}")
    return _REGISTRY[name]


def load_config(model_dir: str):
    """Reads `config.json` of a model folder into the typed configuration of its architecture."""
    d = read_config_json(model_dir)
    arch = resolve_architecture(d)
    return arch.config_cls.from_dict(d)
