"""Rotary position encoding (half-split / "neox" pairing) as a table of cos and sin.

``inv_freq_i = theta^(-2i/dim)``, ``angle = position * inv_freq_i``; element d < dim/2 pairs with
d + dim/2. Angles are computed in 64-bit and stored as 32-bit cos/sin, as the reference's engine
does (cpp/src/ops.cpp:121-144); its Python oracle computes them in 32-bit
(nanoinfer/layers.py:78-97), which differs by about 1e-4 at position 4096.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import PositionEncoding, Runtime
from .spec import PartSpec


def rotary_tables(max_positions: int, dim: int, theta: float):
    """``(cos, sin)`` of shape ``[max_positions, dim/2]`` in float32, angles in float64."""
    half = dim // 2
    i = torch.arange(half, dtype=torch.float64)
    inv_freq = 1.0 / torch.pow(torch.tensor(float(theta), dtype=torch.float64), 2.0 * i / float(dim))
    pos = torch.arange(max_positions, dtype=torch.float64)
    ang = torch.outer(pos, inv_freq)
    return ang.cos().to(torch.float32), ang.sin().to(torch.float32)


class RotaryEncoding(PositionEncoding):
    """params: ``dim`` (rotated width of a head), ``theta``, ``max_positions``. No tensors."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(dim: int, theta: float, max_positions: int) -> PartSpec:
        return PartSpec("rotary", {"dim": dim, "theta": theta, "max_positions": max_positions})

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        self.dim = int(spec.params["dim"])
        if self.dim <= 0 or self.dim % 2:
            raise ValueError(f"rotary dim must be positive and even, got {self.dim}")
        self.max_positions = int(spec.params["max_positions"])
        cos, sin = rotary_tables(self.max_positions, self.dim, float(spec.params["theta"]))
        self.cos = cos.to(rt.device).contiguous()
        self.sin = sin.to(rt.device).contiguous()

    def rotary(self):
        return self.cos, self.sin, self.dim


class NoPositionEncoding(PositionEncoding):
    """Mixers bound to this encoding use their inputs as they are."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec() -> PartSpec:
        return PartSpec("no_position")


register_part("rotary", RotaryEncoding)
register_part("no_position", NoPositionEncoding)
