"""What every architecture's configuration gives the engine, and the error type of this layer.

The reference keeps one flat struct for all architectures (src/model.zig:60-101) filled from
file metadata (src/model.zig:395-490).  Here each architecture has a typed dataclass of its own,
read from its own config.json keys; the engine sees it only through `ModelConfig`.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any


class ConfigError(ValueError):
    """A config.json that cannot describe a model: a missing key, a bad value, an unknown name."""


@dataclass
class ModelConfig:
    """Fields the engine itself needs, whatever the architecture."""

    architecture: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    eos_token_ids: tuple[int, ...] = ()
    bos_token_id: int | None = None
    pad_token_id: int | None = None
    raw: dict[str, Any] = field(default_factory=dict, repr=False)

    def to_json_dict(self) -> dict[str, Any]:
        """The dictionary to write as config.json (architecture's own keys)."""
        raise NotImplementedError


def need(d: dict, key: str, *aliases: str):
    """The value of a required key (or of one of its aliases); ConfigError names the key."""
    for k in (key, *aliases):
        if k in d and d[k] is not None:
            return d[k]
    raise ConfigError(f"config.json: required key '{key}' is missing")


def as_int(d: dict, key: str, value, minimum: int | None = None) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value:
        raise ConfigError(f"config.json: '{key}' must be an integer, found {value!r}")
    v = int(value)
    if minimum is not None and v < minimum:
        raise ConfigError(f"config.json: '{key}' must be >= {minimum}, found {v}")
    return v


def as_float(key: str, value) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: '{key}' must be a number, found {value!r}")
    return float(value)


def read_config_json(folder) -> dict[str, Any]:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no config.json in the model folder")
    try:
        d = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from e
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return d
