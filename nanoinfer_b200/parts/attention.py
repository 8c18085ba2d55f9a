"""Grouped-query causal attention over the paged cache.

``q = h Wq^T + bq`` (likewise k, v); q and k are rotated by the bound position encoding; k (after
rotation) and v go into the cache pages; query head ``h`` uses kv head ``h // (heads / kv_heads)``;
scores ``(q . k) * scale`` over the keys at positions ``<=`` the query's (and, with a window ``w``,
``>`` position - w), softmax in 32-bit, weighted sum of v, output projection without bias, added
to the residual stream.

Reference: cpp/src/model.cpp:365-396 (projection, rotation, attend, output projection, add),
cpp/src/ops.cpp:206-270 (scores, scale after the dot, softmax, PV), cpp/src/paged.cpp:129-206
(block-table addressing, kv head = h / n_rep), nanoinfer/layers.py:150-240.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..registry import register_part
from .base import CacheNeed, LayerCache, Mixer, PositionEncoding, Runtime, StepContext
from .spec import PartSpec, TensorSpec


class GroupedQueryAttention(Mixer):
    """params: ``hidden``, ``heads``, ``kv_heads``, ``head_dim``, ``bias`` (q/k/v), ``window``
    (0 = all keys), ``position`` (name of a shared position encoding), ``scale`` (optional).
    tensors: ``q_w k_w v_w o_w`` and, with bias, ``q_b k_b v_b``."""

    graph_safe = True   # launches do not depend on which requests are in the batch
    accepts_lazy_norm = True   # its first projection can apply the norm while reading its input

    @staticmethod
    def spec(prefix: str, hidden: int, heads: int, kv_heads: int, head_dim: int, bias: bool,
             position: str, window: int = 0, scale: Optional[float] = None) -> PartSpec:
        t = {
            "q_w": TensorSpec(f"{prefix}.q_proj.weight", (heads * head_dim, hidden)),
            "k_w": TensorSpec(f"{prefix}.k_proj.weight", (kv_heads * head_dim, hidden)),
            "v_w": TensorSpec(f"{prefix}.v_proj.weight", (kv_heads * head_dim, hidden)),
            "o_w": TensorSpec(f"{prefix}.o_proj.weight", (hidden, heads * head_dim)),
        }
        if bias:
            t["q_b"] = TensorSpec(f"{prefix}.q_proj.bias", (heads * head_dim,), "bias")
            t["k_b"] = TensorSpec(f"{prefix}.k_proj.bias", (kv_heads * head_dim,), "bias")
            t["v_b"] = TensorSpec(f"{prefix}.v_proj.bias", (kv_heads * head_dim,), "bias")
        params = {"hidden": hidden, "heads": heads, "kv_heads": kv_heads, "head_dim": head_dim,
                  "bias": bias, "window": window, "position": position}
        if scale is not None:
            params["scale"] = scale
        return PartSpec("gqa_attention", params, t)

    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        super().__init__(spec, tensors, rt)
        p = spec.params
        self.hidden, self.heads, self.kv_heads = int(p["hidden"]), int(p["heads"]), int(p["kv_heads"])
        self.head_dim, self.window = int(p["head_dim"]), int(p.get("window", 0))
        if self.heads % self.kv_heads:
            raise ValueError(f"heads ({self.heads}) must be a multiple of kv_heads ({self.kv_heads})")
        self.scale = float(p.get("scale", 1.0 / math.sqrt(float(self.head_dim))))
        self.position_name = str(p["position"])
        # One fused projection: rows [q | k | v].
        self.w_qkv = rt.matrix(torch.cat([tensors["q_w"], tensors["k_w"], tensors["v_w"]], dim=0))
        self.b_qkv = None
        if p.get("bias"):
            self.b_qkv = rt.vector32(torch.cat([tensors["q_b"], tensors["k_b"], tensors["v_b"]], dim=0))
        self.w_o = rt.matrix(tensors["o_w"])
        self.qkv_width = (self.heads + 2 * self.kv_heads) * self.head_dim
        self._rotary = None

    def cache_need(self) -> CacheNeed:
        return CacheNeed.keys_and_values(self.kv_heads, self.head_dim, self.window)

    def bind_positions(self, positions: Dict[str, PositionEncoding]) -> None:
        self._rotary = positions[self.position_name].rotary()
        if self._rotary is not None and self._rotary[2] > self.head_dim:
            raise ValueError("rotary dim exceeds head_dim")

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        m = h.shape[0]
        qkv = torch.empty((m, self.qkv_width), dtype=self.rt.dtype, device=h.device)
        # projection, rotation of q and k, keys (rotated) and values into the pages
        self.ops.qkv_project(h, self.w_qkv, self.b_qkv, qkv, self.heads, self.kv_heads, self.head_dim, ctx.positions,
                             ctx.req_index, self._rotary, cache.block_table, cache.page_size, cache.k_pages,
                             cache.v_pages, cache.writes)
        attn = torch.empty((m, self.heads * self.head_dim), dtype=self.rt.dtype, device=h.device)
        self.ops.attention(qkv, attn, self.heads, self.kv_heads, self.head_dim, self.scale, self.window,
                           ctx, cache.block_table, cache.page_size, cache.k_pages, cache.v_pages, own_kv=cache.writes)
        self.ops.linear(attn, self.w_o, None, residual32, "add")


register_part("gqa_attention", GroupedQueryAttention)
