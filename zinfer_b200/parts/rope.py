"""Rotary position encoding: f_i = theta^(-2i/n_rot) * scale computed in float64 and cast to
float32 (src/rope.zig:8-16); the angle float32(pos) * f_i and its cos/sin are computed inside
the q/k kernel (src/rope.zig:34-45); NeoX pairing (i, i + n_rot/2) unless `interleaved`
(src/rope.zig:50-64; NeoX for every architecture but llama, src/model.zig:449)."""
from __future__ import annotations

import numpy as np
import torch

from .base import POSITION_ENCODINGS, PositionEncoding, RotaryParams


class RotaryEncoding(PositionEncoding):
    def __init__(self, head_dim: int, theta: float, n_rot: int | None = None, interleaved: bool = False,
                 scale: float = 1.0):
        self.head_dim = head_dim
        self.n_rot = head_dim if n_rot is None else n_rot
        if self.n_rot % 2 or self.n_rot > head_dim:
            raise ValueError(f"rotary width {self.n_rot} must be even and <= head_dim {head_dim}")   # src/model.zig:488-489
        self.theta, self.interleaved, self.scale = float(theta), interleaved, float(scale)
        self._params: RotaryParams | None = None

    def inv_freq_host(self) -> np.ndarray:
        i = np.arange(self.n_rot // 2, dtype=np.float64)
        return (np.power(np.float64(self.theta), -2.0 * i / np.float64(self.n_rot)) * self.scale).astype(np.float32)

    def load(self, weights, dtype, device):
        self._params = RotaryParams(torch.from_numpy(self.inv_freq_host()).to(device), self.n_rot, self.interleaved)

    def rotary(self):
        return self._params


POSITION_ENCODINGS.register("rotary", RotaryEncoding)
