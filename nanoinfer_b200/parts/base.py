"""Interfaces of the parts a layer is put together from, and what a part sees of a step.

A part gets its sizes and constants as parameters (``PartSpec.params``), its tensors by role,
and a ``Runtime`` (device, compute dtype, kernel library). No part knows which model it is in.

Interfaces (duck-typed; the base classes document them):

* ``Norm.forward(x32, rows=None) -> h``: x32 is the 32-bit residual stream ``[M, hidden]``; the
  result has the compute dtype. ``rows`` (int32 device tensor) selects and orders the rows to norm.
* ``PositionEncoding``: ``rotary()`` returns ``(cos, sin, rotary_dim)`` tables for mixers that
  rotate queries and keys, or None; ``add_to_embedding(x32, ctx)`` may add to the residual stream.
* ``Mixer.forward(h, residual32, ctx, cache)``: mixes tokens across positions and ADDS its output
  to ``residual32`` in place. ``cache_need()`` says which pages it needs (or None),
  ``state_need()`` which fixed-size per-request state (or None).
* ``FeedForward.forward(h, residual32, ctx)``: per-token transform, ADDS to ``residual32``.
* ``Embedding.forward(token_ids, ctx) -> x32`` and ``Head.forward(h) -> logits32``.
* An arrangement (``parts/block.py``) orders the parts of one layer.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from .spec import PartSpec


@dataclass
class Runtime:
    """Where and with what a part computes."""
    device: torch.device
    dtype: torch.dtype            # torch.bfloat16 or torch.float32: activations, matrices, cache
    ops: object                   # the kernel library (csrc/lib.py: Kernels)

    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        """A matrix operand: compute dtype, contiguous, on the device."""
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def vector32(self, t: torch.Tensor) -> torch.Tensor:
        """A gain or bias: 32-bit on the device (lossless from bfloat16)."""
        return t.to(device=self.device, dtype=torch.float32).contiguous()


@dataclass(frozen=True)
class CacheNeed:
    """Paged keys and values a mixer keeps per token. ``window`` 0 = all keys are kept."""
    kv_heads: int
    head_dim: int
    window: int = 0

    def group_key(self) -> Tuple[int, int, int]:
        return (self.kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateNeed:
    """Fixed-size per-request state of a mixer: ``shape`` elements of ``dtype`` per request, zero at start."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class HostBatch:
    """The step's batch as host lists, for planning launches (never read by kernels)."""
    q_lens: List[int]
    ctx_lens: List[int]            # tokens held by each request AFTER this step's tokens are appended
    slots: List[int]

    @property
    def num_requests(self) -> int:
        return len(self.q_lens)

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens)

    @property
    def max_ctx_len(self) -> int:
        return max(self.ctx_lens)


@dataclass
class StepContext:
    """What every part sees of one step: the flat token batch and where each token belongs.

    All device tensors are int32. Tokens of one request are contiguous and in position order.
    """
    num_tokens: int
    token_ids: torch.Tensor        # [M]
    positions: torch.Tensor        # [M]  absolute position of each token in its request
    req_index: torch.Tensor        # [M]  row of the token's request in this batch
    q_start: torch.Tensor          # [R+1] first flat row of each request (prefix sums of q_lens)
    ctx_lens: torch.Tensor         # [R]  tokens held after this step
    state_slots: torch.Tensor      # [R]  state slot of each request
    host: HostBatch
    block_tables: Dict[int, torch.Tensor] = field(default_factory=dict)  # cache group -> [R, pages]
    rt: Optional[Runtime] = None
    all_rows_wanted: bool = False  # logits are wanted at every row, in row order


@dataclass
class LayerCache:
    """The cache of one schedule entry, as its mixer sees it."""
    k_pages: Optional[torch.Tensor]     # [num_pages, kv_heads, page_size, head_dim]
    v_pages: Optional[torch.Tensor]
    block_table: Optional[torch.Tensor]  # [R, max_pages] int32, -1 where no page is held
    page_size: int
    writes: bool                        # False when this entry reads another entry's cache
    state: Optional[torch.Tensor]       # [slots, *StateNeed.shape]


class DeferredNorm:
    """A norm that has not been computed yet: ``h = norm(x32)``, for a consumer whose kernel can apply the
    norm while it reads its input (the decode GEMM). It looks like ``h`` (shape, dtype, device); any other
    consumer gets the tensor from ``materialize()``."""

    def __init__(self, norm: "Norm", x32: torch.Tensor, gain32: torch.Tensor, eps: float, dtype: torch.dtype):
        self.norm, self.x32, self.gain32, self.eps, self.dtype = norm, x32, gain32, eps, dtype
        self._tensor: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return self.x32.shape

    @property
    def device(self):
        return self.x32.device

    def materialize(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = self.norm.forward(self.x32)
        return self._tensor


class Part:
    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        self.spec, self.rt = spec, rt
        self.ops = rt.ops


class Norm(Part):
    def forward(self, x32: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def deferred(self, x32: torch.Tensor):
        """``forward(x32)``, or a ``DeferredNorm`` that a consumer with ``accepts_deferred_norm`` resolves."""
        return self.forward(x32)


class PositionEncoding(Part):
    def rotary(self):
        return None

    def add_to_embedding(self, x32: torch.Tensor, ctx: StepContext) -> None:
        return None


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def bind_positions(self, positions: Dict[str, PositionEncoding]) -> None:
        """Called once after construction with the model's shared position encodings."""
        return None

    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext, cache: LayerCache) -> None:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, residual32: torch.Tensor, ctx: StepContext) -> None:
        raise NotImplementedError


class Embedding(Part):
    def forward(self, token_ids: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Head(Part):
    def forward(self, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError
