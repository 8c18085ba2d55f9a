"""SwiGLU feed-forward: ``down( silu(gate(h)) * up(h) )``, no biases, added to the residual stream.

``silu(g) = g / (1 + exp(-g))`` in 32-bit. Reference: cpp/src/model.cpp:217-223,
cpp/src/ops.cpp:86-100, nanoinfer/layers.py:243-258.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import FeedForward, Runtime, StepContext
from .spec import PartSpec, TensorSpec


class SwiGLU(FeedForward):
    """params: ``hidden``, ``intermediate``. tensors: ``gate_w up_w [intermediate, hidden]``,
    ``down_w [hidden, intermediate]``."""

    graph_safe = True   # launches do not depend on which requests are in the batch
    accepts_lazy_norm = True   # its first projection can apply the norm while reading its input

    @staticmethod
    def spec(prefix: str, hidden: int, intermediate: int) -> PartSpec:
        return PartSpec("swiglu", {"hidden": hidden, "intermediate": intermediate}, {
            "gate_w": TensorSpec(f"{prefix}.gate_proj.weight", (intermediate, hidden)),
            "up_w": TensorSpec(f"{prefix}.up_proj.weight", (intermediate, hidden)),
            "down_w": TensorSpec(f"{prefix}.down_proj.weight", (hidden, intermediate)),
        })

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        self.hidden = int(spec.params["hidden"])
        self.intermediate = int(spec.params["intermediate"])
        # One fused operand: rows [gate | up].
        self.w_gate_up = rt.matrix(torch.cat([tensors["gate_w"], tensors["up_w"]], dim=0))
        self.w_down = rt.matrix(tensors["down_w"])

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext) -> None:
        act = torch.empty((h.shape[0], self.intermediate), dtype=self.rt.dtype, device=h.device)
        self.ops.linear_swiglu(h, self.w_gate_up, act)
        self.ops.linear(act, self.w_down, None, residual32, "add")


register_part("swiglu", SwiGLU)
