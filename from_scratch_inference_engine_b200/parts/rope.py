"""Rotary position encoding: a cos/sin table computed in 64-bit on the host."""

from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .base import Part, register_part


def rotary_table(theta: float, rotary_dim: int, length: int) -> np.ndarray:
    """[length, rotary_dim] float32: cos(pos * f_i) for i < rotary_dim/2, then sin.

    f_i = theta^(-2i/rotary_dim) and the angle are computed in 64-bit and rounded once,
    as the reference computes them per element (src/model/nn.cpp:122-137)."""
    half = rotary_dim // 2
    inv_freq = np.power(float(theta), -2.0 * np.arange(half, dtype=np.float64) / rotary_dim)
    angles = np.arange(length, dtype=np.float64)[:, None] * inv_freq[None, :]
    return np.concatenate([np.cos(angles), np.sin(angles)], axis=1).astype(np.float32)


@register_part("position", "rotary")
class RotaryEncoding(Part):
    """Half-rotation pairs (i, i + rotary_dim/2) over the first `rotary_dim` of each head.
    The rotation itself runs inside the mixer's kernel; this part owns the table."""

    capturable = True

    def __init__(self, prefix: str, theta: float, rotary_dim: int, max_position: int = 0):
        if rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        self.prefix, self.theta = prefix, float(theta)
        self.rotary_dim, self.max_position = int(rotary_dim), int(max_position)
        self.table: Optional[torch.Tensor] = None

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        # as long as the configuration says, and at least as long as the cache can hold
        length = max(self.max_position, runtime.max_positions, 1)
        self.table = runtime.shared_table(
            ("rotary", self.theta, self.rotary_dim, length),
            lambda: torch.from_numpy(rotary_table(self.theta, self.rotary_dim, length)))


@register_part("position", "none")
class NoPositionEncoding(Part):
    """No position encoding: queries and keys are used as projected."""

    capturable = True

    rotary_dim = 0

    def __init__(self, prefix: str = ""):
        self.prefix = prefix
        self.table = None

    def bind(self, tensors, runtime) -> None:
        self.runtime = runtime
        self.table = runtime.shared_table(("rotary-none",),
                                          lambda: torch.zeros((1, 0), dtype=torch.float32))
