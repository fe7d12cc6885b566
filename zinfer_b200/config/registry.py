"""One registry from an architecture's name (config.json `architectures[0]`) to its typed
configuration and its model builder.  The reference maps the file's architecture string to an
enum and fails with UnsupportedArchitecture otherwise (src/model.zig:397-406)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .base import ConfigError, ModelConfig, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_cls: type
    build: Callable[[Any], Any]          # typed config -> models.model.Model (weights not loaded)


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_cls: type, build: Callable, replace: bool = False) -> None:
    if name in _ARCHITECTURES and not replace:
        raise KeyError(f"architecture '{name}' is already registered")
    _ARCHITECTURES[name] = Architecture(name, config_cls, build)


def unregister_architecture(name: str) -> None:
    _ARCHITECTURES.pop(name, None)


def registered_architectures() -> list[str]:
    return sorted(_ARCHITECTURES)


def architecture_name(config_dict: dict) -> str:
    archs = config_dict.get("architectures")
    if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
        raise ConfigError("config.json: required key 'architectures' (a list naming the model class) is missing")
    return archs[0]


def get_architecture(name: str) -> Architecture:
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"architecture '{name}' is not supported; registered: {registered_architectures()}") from None


def config_from_dict(config_dict: dict) -> ModelConfig:
    arch = get_architecture(architecture_name(config_dict))
    return arch.config_cls.from_json_dict(config_dict)


def config_from_folder(folder) -> ModelConfig:
    return config_from_dict(read_config_json(folder))


def build_model(config: ModelConfig):
    """The model of a typed configuration, parts assembled, weights not yet loaded."""
    return get_architecture(config.architecture).build(config)
