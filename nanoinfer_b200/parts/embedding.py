"""Token embedding (row gather into the 32-bit residual stream) and the output head.

Reference: cpp/src/ops.cpp:71-84 and cpp/src/model.cpp:284-296 (gather; logits = x W^T without
bias; a tied head is the embedding table), nanoinfer/model.py:50, 83-84.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_part
from .base import Embedding, Head, Runtime, StepContext
from .spec import PartSpec, TensorSpec


class TokenEmbedding(Embedding):
    """params: ``vocab``, ``hidden``. tensors: ``table [vocab, hidden]``."""

    graph_safe = True   # launches do not depend on which requests are in the batch

    @staticmethod
    def spec(name: str, vocab: int, hidden: int) -> PartSpec:
        return PartSpec("token_embedding", {"vocab": vocab, "hidden": hidden},
                        {"table": TensorSpec(name, (vocab, hidden), "embedding")})

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        self.vocab, self.hidden = int(spec.params["vocab"]), int(spec.params["hidden"])
        self.table = rt.matrix(tensors["table"])

    def forward(self, token_ids: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        x32 = torch.empty((token_ids.shape[0], self.hidden), dtype=torch.float32, device=token_ids.device)
        self.ops.embed(token_ids, self.table, x32)
        return x32


class LinearHead(Head):
    """params: ``vocab``, ``hidden``. tensors: ``weight [vocab, hidden]`` (the embedding table when tied)."""

    graph_safe = True   # launches do not depend on which requests are in the batch
    accepts_lazy_norm = True   # its projection can apply the norm while reading its input

    @staticmethod
    def spec(name: str, vocab: int, hidden: int) -> PartSpec:
        return PartSpec("linear_head", {"vocab": vocab, "hidden": hidden},
                        {"weight": TensorSpec(name, (vocab, hidden), "embedding")})

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        self.vocab = int(spec.params["vocab"])
        self.weight = rt.matrix(tensors["weight"])

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        logits = torch.empty((h.shape[0], self.vocab), dtype=torch.float32, device=h.device)
        self.ops.linear(h, self.weight, None, logits, "f32")
        return logits


register_part("token_embedding", TokenEmbedding)
register_part("linear_head", LinearHead)
