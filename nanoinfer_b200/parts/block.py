"""Arrangements: the order in which the parts of one layer run.

``pre_norm``: ``x += mixer(norm(x)); x += feed_forward(norm(x))`` with a norm of its own before each
(cpp/src/model.cpp:364-400, nanoinfer/layers.py:328-339). The residual stream ``x`` is 32-bit and
both sums are made in 32-bit inside the projections that produce the addends.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_arrangement
from .base import LayerCache, StepContext, normed_input


class PreNormBlock:
    """parts: ``mixer_norm``, ``mixer``, ``ffn_norm``, ``ffn``."""

    part_names = ("mixer_norm", "mixer", "ffn_norm", "ffn")

    def __init__(self, parts: Dict[str, object]):
        self.mixer_norm, self.mixer = parts["mixer_norm"], parts["mixer"]
        self.ffn_norm, self.ffn = parts["ffn_norm"], parts["ffn"]

    def forward(self, x32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        # A part that says so takes its norm unresolved and lets its first projection apply it.
        self.mixer.forward(normed_input(self.mixer_norm, self.mixer, x32), x32, ctx, cache)
        self.ffn.forward(normed_input(self.ffn_norm, self.ffn, x32), x32, ctx)


register_arrangement("pre_norm", PreNormBlock)
