"""Rotary position encoding.

The table is built on the host exactly as Glassbox computes its angles
(crates/glassbox-core/src/model.rs:102-115): the inverse frequency 1 / theta^(2i/dim) is formed
in float64 and rounded to float32; the angle is the float32 product position * inv_freq; sine
and cosine are evaluated in float64 and rounded to float32. Doing the angle in float32 makes
long positions round "like transformers" (model.rs:106), so it is kept.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Position, register_part


def rotary_table(theta: float, rotary_dim: int, max_position: int) -> torch.Tensor:
    """float32 [max_position, rotary_dim/2, 2] holding (cos, sin)."""
    half = rotary_dim // 2
    i = np.arange(half, dtype=np.float64)
    inv = (1.0 / np.power(np.float64(theta), 2.0 * i / np.float64(rotary_dim))).astype(np.float32)
    pos = np.arange(max_position, dtype=np.float32)
    angle = (pos[:, None] * inv[None, :]).astype(np.float32)  # float32 multiply
    a64 = angle.astype(np.float64)
    table = np.stack([np.cos(a64).astype(np.float32), np.sin(a64).astype(np.float32)], axis=-1)
    return torch.from_numpy(np.ascontiguousarray(table))


def inverse_frequencies(theta: float, rotary_dim: int) -> torch.Tensor:
    """float32 [rotary_dim/2]: theta^(-2i / rotary_dim), formed in float64 and rounded once."""
    i = np.arange(rotary_dim // 2, dtype=np.float64)
    return torch.from_numpy(np.power(np.float64(theta), -2.0 * i / np.float64(rotary_dim)).astype(np.float32))


class Rope(Position):
    """``pairing`` "half": a (cos, sin) table for the kernels that rotate channel i with channel i + rotary_dim/2.
    ``pairing`` "interleaved" (channel 2i with 2i + 1): no table; the mixers that take it ask for ``inv_freq`` and
    form the angle float32(position) * inv_freq[i] and its sine and cosine on the device, so no largest position has to
    be known beforehand."""
    launches_through_kernels_only = True

    def __init__(self, spec, **_):
        super().__init__(spec)
        if spec.pairing not in ("half", "interleaved"):
            raise ValueError(f"rope pairing {spec.pairing!r} is not supported ('half' or 'interleaved')")
        if spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim {spec.rotary_dim} must be even")
        self.rotary_dim = spec.rotary_dim
        self.pairing = spec.pairing
        self._tables = {}

    def inv_freq(self, device):
        key = ("inv_freq", str(device))
        if key not in self._tables:
            self._tables[key] = inverse_frequencies(self.spec.theta, self.spec.rotary_dim).to(device)
        return self._tables[key]

    def fused_table(self, device):
        if self.pairing != "half":
            return None
        key = str(device)
        if key not in self._tables:
            self._tables[key] = rotary_table(self.spec.theta, self.spec.rotary_dim, self.spec.max_position).to(device)
        return self._tables[key]


class NoPosition(Position):
    launches_through_kernels_only = True

    def __init__(self, spec=None, **_):
        super().__init__(spec)


register_part("position", "rope", Rope, replace=True)
register_part("position", "none", NoPosition, replace=True)
