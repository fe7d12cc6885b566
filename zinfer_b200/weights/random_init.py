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


def random_tensors_on_device(model, seed: int, std: float, norm_init: str, storage_dtype: torch.dtype,
                             device) -> Iterator[tuple[WeightSpec, torch.Tensor]]:
    """As `random_tensors`, drawn by a kernel on the GPU: other values than the host generator's,
    the same distribution, a function of (seed, tensor name, element index) only; a billion
    parameters in milliseconds.  Storage is float32 or bfloat16."""
    from .. import kernels

    if storage_dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"the device fill stores float32 or bfloat16, not {storage_dtype}")
    for name, spec in model.weight_specs().items():
        if spec.init == "skip":
            continue
        if spec.role == "table":
            raise ValueError(f"tensor '{name}': integer tables have no random fill")
        init = norm_init if spec.init == "norm" else spec.init
        t = torch.empty(spec.alt_shapes[0] if spec.alt_shapes else spec.shape, dtype=storage_dtype, device=device)
        if init == "zeros":
            t.zero_()
        elif init in ("normal", "one_plus_normal"):
            kernels.fill_normal(t, (seed << 32) ^ zlib.crc32(name.encode()), 1.0 if init == "one_plus_normal" else 0.0, std)
        else:
            raise ValueError(f"tensor '{name}': unknown init {spec.init!r}")
        yield spec, t


def write_random_model(folder, config: ModelConfig, seed: int, std: float = 0.02,
                       norm_init: str = "one_plus_normal", storage_dtype: torch.dtype = torch.bfloat16,
                       fill_on_device: bool = False, device="cuda") -> Path:
    """Writes config.json and model.safetensors for `config` into `folder` (created if needed).
    `fill_on_device` draws the values with the GPU's fill kernel (see `random_tensors_on_device`),
    which is what a model of a billion parameters wants."""
    import zinfer_b200.models  # noqa: F401

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    model = build_model(config)
    if fill_on_device:
        tensors = {spec.name: t.cpu() for spec, t in
                   random_tensors_on_device(model, seed, std, norm_init, storage_dtype, device)}
    else:
        tensors = {spec.name: t for spec, t in random_tensors(model, seed, std, norm_init, storage_dtype)}
    (folder / "config.json").write_text(json.dumps(config.to_json_dict(), indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", tensors,
                      metadata={"format": "pt", "seed": str(seed), "std": str(std), "norm_init": norm_init,
                                "generator": "device" if fill_on_device else "host"})
    return folder


def random_model(config: ModelConfig, seed: int, dtype: torch.dtype = torch.bfloat16, device="cuda",
                 std: float = 0.02, norm_init: str = "one_plus_normal",
                 storage_dtype: torch.dtype = torch.bfloat16, fill_on_device: bool = False):
    """A model with random weights, without touching the disk.  By default the values are those
    `write_random_model` would store for the same seed; `fill_on_device` draws them on the GPU
    instead (the values `write_random_model(fill_on_device=True)` stores).  Either way they are
    rounded to `storage_dtype` first, so a bfloat16 and a float32 model of one seed hold the same
    numbers."""
    import zinfer_b200.models  # noqa: F401

    model = build_model(config)
    draw = (random_tensors_on_device(model, seed, std, norm_init, storage_dtype, device) if fill_on_device
            else random_tensors(model, seed, std, norm_init, storage_dtype))
    weights = {spec.name: convert(t, spec, dtype).to(device).contiguous() for spec, t in draw}
    model.load_weights(weights, dtype, device)
    return model
