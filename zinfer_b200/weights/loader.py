"""Loads a model folder (config.json + model.safetensors, or an index with shards) by tensor name.

The reference looks every tensor up by name, checks its dimensions and fails with
MissingTensor / BadTensorShape / UnsupportedTensorType (src/model.zig:553-589).  Here all
problems of a file are gathered first and raised as ONE `WeightError` that lists missing
tensors, unexpected tensors and wrong shapes.

Kept dtypes: matrices in the run dtype (bfloat16, or float32 in the 32-bit path -- a matrix
stored in 32-bit is rounded to bfloat16 only for a bfloat16 run); vectors (norm weights, conv
taps, biases) always in float32, which holds a stored bfloat16 or float32 value exactly;
integer tables in int32.
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable, Iterable, Optional

import torch

from ..config.registry import build_model, config_from_folder
from ..parts.base import WeightSpec
from .safetensors_io import SafetensorsFile, WeightFileError

_FLOAT = (torch.float32, torch.bfloat16, torch.float16, torch.float64)
_INT = (torch.int32, torch.int64, torch.int16, torch.int8, torch.uint8)


class WeightError(ValueError):
    """The file does not hold what the model needs; the message lists every problem."""

    def __init__(self, where: str, missing=(), unexpected=(), wrong=()):
        self.missing, self.unexpected, self.wrong = list(missing), list(unexpected), list(wrong)
        lines = [f"{where}: the weights do not match the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for w in self.wrong:
            lines.append(f"  wrong: {w}")
        super().__init__("\n".join(lines))


def convert(t: torch.Tensor, spec: WeightSpec, run_dtype: torch.dtype) -> torch.Tensor:
    """The tensor in the dtype its role asks for, reshaped to the spec's shape."""
    t = t.reshape(spec.shape)
    if spec.role == "matrix":
        return t.to(run_dtype)
    if spec.role == "vector":
        return t.to(torch.float32)
    if spec.role == "table":
        return t.to(torch.int32)
    raise ValueError(f"tensor '{spec.name}': unknown role {spec.role!r}")


def check_tensors(where: str, specs: dict[str, WeightSpec], found: dict[str, tuple[torch.dtype, tuple[int, ...]]],
                  ignorable: Iterable[str] = ()) -> None:
    """Raises one WeightError for everything wrong between what is wanted and what was found."""
    missing = [n for n, s in specs.items() if n not in found and not s.optional]
    unexpected = [n for n in found if n not in specs and n not in set(ignorable)]
    wrong = []
    for n, s in specs.items():
        if n not in found:
            continue
        dt, shape = found[n]
        if shape != tuple(s.shape) and shape not in s.alt_shapes:
            wrong.append(f"'{n}' has shape {list(shape)}, expected {list(s.shape)}")
        elif s.role == "table" and dt not in _INT:
            wrong.append(f"'{n}' has dtype {dt}, expected an integer table")
        elif s.role != "table" and dt not in _FLOAT:
            wrong.append(f"'{n}' has dtype {dt}, expected a floating-point tensor")
    if missing or unexpected or wrong:
        raise WeightError(where, sorted(missing), sorted(unexpected), wrong)


def open_weight_files(folder: Path) -> list[SafetensorsFile]:
    single = folder / "model.safetensors"
    index = folder / "model.safetensors.index.json"
    if single.is_file():
        return [SafetensorsFile(single)]
    if index.is_file():
        try:
            shards = sorted(set(json.loads(index.read_text())["weight_map"].values()))
        except (json.JSONDecodeError, KeyError, AttributeError) as e:
            raise WeightFileError(f"{index}: not a shard index ({e})") from e
        return [SafetensorsFile(folder / s) for s in shards]
    raise WeightFileError(f"{folder}: neither model.safetensors nor model.safetensors.index.json")


def load_into(model, tensors: Callable[[str], torch.Tensor], found: dict, where: str, dtype: torch.dtype,
              device) -> None:
    specs = model.weight_specs()
    check_tensors(where, specs, found, model.ignorable_weights)
    weights = {}
    for name, spec in specs.items():
        if name in found:
            weights[name] = convert(tensors(name), spec, dtype).to(device).contiguous()
    model.load_weights(weights, dtype, device)


def load_model(folder, dtype: torch.dtype = torch.bfloat16, device="cuda"):
    """The model of a folder, chosen by config.json's architecture name, weights on `device`."""
    import zinfer_b200.models  # noqa: F401  (registers the architectures)

    folder = Path(folder)
    config = config_from_folder(folder)
    model = build_model(config)
    files = open_weight_files(folder)
    try:
        where_of: dict[str, SafetensorsFile] = {}
        found = {}
        for f in files:
            for name, info in f.infos.items():
                if name in where_of:
                    raise WeightFileError(f"{folder}: tensor '{name}' is stored in two files")
                where_of[name] = f
                found[name] = (info.dtype, info.shape)
        load_into(model, lambda n: where_of[n].tensor(n), found, str(folder), dtype, device)
    finally:
        for f in files:
            f.close()
    return model
