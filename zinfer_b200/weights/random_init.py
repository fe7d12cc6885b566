"""Random weights from a configuration and a seed: as a model folder on disk, or straight
into a model.  Each tensor's values depend only on (seed, tensor name), not on the order of
generation, so a folder and an in-memory model of the same seed agree.

Matrices and biases are N(0, std); norm weights are 1 + N(0, std) ("one_plus_normal") or
N(0, std) ("normal").  Values are rounded to the storage dtype before use, so every reader of
the folder sees the same numbers.
"""
from __future__ import annotations

import json
import zlib
from pathlib import Path
from typing import Iterator

import numpy as np
import torch

from ..config.base import ModelConfig
from ..config.registry import build_model
from ..parts.base import WeightSpec
from .loader import convert
from .safetensors_io import write_safetensors


def _tensor(spec: WeightSpec, seed: int, std: float, norm_init: str, storage_dtype: torch.dtype) -> torch.Tensor:
    rng = np.random.Generator(np.random.Philox(key=[seed & 0xFFFFFFFFFFFFFFFF, zlib.crc32(spec.name.encode())]))
    count = int(np.prod(spec.shape))
    init = spec.init
    if init == "norm":
        init = norm_init
    if init == "zeros":
        vals = np.zeros(count, dtype=np.float32)
    else:
        vals = rng.standard_normal(count, dtype=np.float32) * np.float32(std)
        if init == "one_plus_normal":
            vals += np.float32(1.0)
        elif init != "normal":
            raise ValueError(f"tensor '{spec.name}': unknown init {spec.init!r}")
    shape = spec.alt_shapes[0] if spec.alt_shapes else spec.shape
    return torch.from_numpy(vals).reshape(shape).to(storage_dtype)


def random_tensors(model, seed: int, std: float = 0.02, norm_init: str = "one_plus_normal",
                   storage_dtype: torch.dtype = torch.bfloat16) -> Iterator[tuple[WeightSpec, torch.Tensor]]:
    for name, spec in model.weight_specs().items():
        if spec.init == "skip":
            continue
        if spec.role == "table":
            raise ValueError(f"tensor '{name}': integer tables have no random fill")
        yield spec, _tensor(spec, seed, std, norm_init, storage_dtype)


def write_random_model(folder, config: ModelConfig, seed: int, std: float = 0.02,
                       norm_init: str = "one_plus_normal", storage_dtype: torch.dtype = torch.bfloat16) -> Path:
    """Writes config.json and model.safetensors for `config` into `folder` (created if needed)."""
    import zinfer_b200.models  # noqa: F401

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    model = build_model(config)
    tensors = {spec.name: t for spec, t in random_tensors(model, seed, std, norm_init, storage_dtype)}
    (folder / "config.json").write_text(json.dumps(config.to_json_dict(), indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": str(seed), "std": str(std), "norm_init": norm_init})
    return folder


def random_model(config: ModelConfig, seed: int, dtype: torch.dtype = torch.bfloat16, device="cuda",
                 std: float = 0.02, norm_init: str = "one_plus_normal",
                 storage_dtype: torch.dtype = torch.bfloat16, fill_on_device: bool = False):
    """A model with random weights, without touching the disk.  By default the values are those
    `write_random_model` would store for the same seed.  `fill_on_device` draws them with a kernel
    on the GPU instead (other values, same distribution): a billion parameters in milliseconds."""
    import zinfer_b200.models  # noqa: F401

    model = build_model(config)
    weights = {}
    if fill_on_device:
        from .. import kernels

        for name, spec in model.weight_specs().items():
            if spec.init == "skip":
                continue
            init = norm_init if spec.init == "norm" else spec.init
            kept = dtype if spec.role == "matrix" else torch.float32
            t = torch.empty(spec.shape, dtype=storage_dtype if storage_dtype in (torch.float32, torch.bfloat16) else kept,
                            device=device)
            if init == "zeros":
                t.zero_()
            else:
                kernels.fill_normal(t, (seed << 32) ^ zlib.crc32(name.encode()), 1.0 if init == "one_plus_normal" else 0.0, std)
            weights[name] = t.to(kept)
    else:
        for spec, t in random_tensors(model, seed, std, norm_init, storage_dtype):
            weights[spec.name] = convert(t, spec, dtype).to(device).contiguous()
    model.load_weights(weights, dtype, device)
    return model
