"""zinfer_b200: a small, whole LFM2 inference library for one B200 (sm_100a).

    import zinfer_b200 as z
    model  = z.load("path/to/folder", dtype="bf16")          # or z.random(config, seed=0, dtype="fp32")
    engine = z.Engine(model, max_batch=8)
    out    = engine.generate([[1, 2, 3], [4, 5]], max_new_tokens=16, temperature=0.0)
"""
from __future__ import annotations

import torch

from . import models as _models  # noqa: F401  (registers the architectures)
from .config import ConfigError, Lfm2Config, config_from_dict, config_from_folder
from .engine.engine import Engine, StepError
from .engine.generate import GenerationResult, Stats
from .sampling import SamplingParams
from .weights import WeightError, load_model, random_model, write_random_model

_DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp32": torch.float32, "float32": torch.float32}


def _dtype(d):
    if isinstance(d, torch.dtype):
        return d
    try:
        return _DTYPES[str(d)]
    except KeyError:
        raise ValueError(f"dtype {d!r}: use 'bf16' or 'fp32'") from None


def load(folder, dtype="bf16", device="cuda"):
    """The model of a folder (config.json + model.safetensors), chosen by its architecture name."""
    return load_model(folder, dtype=_dtype(dtype), device=device)


def random(config, seed: int = 0, dtype="bf16", device="cuda", **init):
    """A model with seeded random weights; `config` is a typed configuration or a config.json dict."""
    if isinstance(config, dict):
        config = config_from_dict(config)
    return random_model(config, seed, dtype=_dtype(dtype), device=device, **init)
