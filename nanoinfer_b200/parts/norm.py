"""RMSNorm: ``x * 1/sqrt(mean(x^2) + eps) * gain``, computed in 32-bit.

Reference: cpp/src/ops.cpp:272-292 (eps inside the root, added to the mean; gain last) and
nanoinfer/layers.py:21-38.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import FoldedNorm, Norm, Runtime
from .spec import PartSpec, TensorSpec


class RMSNorm(Norm):
    """params: ``size`` (width of a row), ``eps``. tensors: ``gain [size]``."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(size: int, eps: float, gain_name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": size, "eps": eps},
                        {"gain": TensorSpec(gain_name, (size,), "gain")})

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.gain = rt.vector32(tensors["gain"])

    def forward(self, x32: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        n = x32.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=self.rt.dtype, device=x32.device)
        self.ops.rmsnorm(x32, self.gain, self.eps, out, rows)
        return out

    def fold_into_projection(self, x32: torch.Tensor) -> Optional[FoldedNorm]:
        return FoldedNorm(x32, self.gain, self.eps, "rms")


register_part("rmsnorm", RMSNorm)

