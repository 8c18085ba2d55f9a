"""Interfaces of the parts a layer is put together from, and what a part sees of a step.

A part gets its sizes and constants as parameters (``PartSpec.params``), its tensors by role,
and a ``Runtime`` (device, compute dtype, kernel library). No part knows which model it is in.

Interfaces (duck-typed; the base classes document them):

* ``Norm.forward(x32, rows=None) -> h``: x32 is the 32-bit residual stream ``[M, hidden]``; the
  result has the compute dtype. ``rows`` (int32 device tensor) selects and orders the rows to norm.
  ``Norm.fold_into_projection(x32)`` may return a ``FoldedNorm`` (x32, gain32, eps, kind); a consumer that
  sets ``accepts_lazy_norm`` is then given a ``LazyNorm`` in place of ``h`` and hands it to the kernel
  library's products, which apply the norm inside the product where a kernel can, or resolve it.
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
class PagedTensor:
    """One tensor that a mixer keeps per token in the paged cache: ``heads x width`` elements for every position, laid
    out per page as ``[heads, page_size, width]``. ``dtype`` None = the engine's compute dtype."""
    name: str
    heads: int
    width: int
    dtype: Optional[torch.dtype] = None


@dataclass(frozen=True)
class CacheNeed:
    """What a mixer keeps per token: any number of paged tensors (keys and values; keys alone; one latent; keys and
    values of different widths), all addressed through one block table. ``window`` 0 = every position is kept,
    ``w`` = only the last ``w`` positions are ever read, so pages behind them are given back."""
    tensors: Tuple[PagedTensor, ...]
    window: int = 0

    @staticmethod
    def keys_and_values(kv_heads: int, head_dim: int, window: int = 0) -> "CacheNeed":
        """The two-tensor case of attention: ``k`` and ``v`` of the same shape in the compute dtype."""
        return CacheNeed((PagedTensor("k", kv_heads, head_dim), PagedTensor("v", kv_heads, head_dim)), window)

    def group_key(self):
        """Entries with equal keys share a cache group (one block table per request)."""
        return (self.tensors, self.window)


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
    pages: Dict[str, torch.Tensor]      # PagedTensor.name -> [num_pages, heads, page_size, width]
    block_table: Optional[torch.Tensor]  # [R, max_pages] int32, -1 where no page is held
    page_size: int
    writes: bool                        # False when this entry reads another entry's cache
    state: Optional[torch.Tensor]       # [slots, *StateNeed.shape]

    @property
    def k_pages(self) -> Optional[torch.Tensor]:
        """The keys of the two-tensor case (CacheNeed.keys_and_values)."""
        return self.pages.get("k")

    @property
    def v_pages(self) -> Optional[torch.Tensor]:
        return self.pages.get("v")


@dataclass(frozen=True)
class FoldedNorm:
    """A norm in the form a projection kernel can apply while it reads the 32-bit residual stream:
    ``h = x32 * f(x32) * gain32`` with ``f`` named by ``kind``. ``"rms"`` is ``1/sqrt(mean(x^2) + eps)`` per
    row; a norm with another statistic names another kind, and a kernel library that does not know the kind
    lets the norm compute itself. A norm whose gain is stored in another form (``1 + g``) hands over the
    vector it multiplies with."""
    x32: torch.Tensor
    gain32: torch.Tensor
    eps: float
    kind: str = "rms"


class LazyNorm:
    """``h = norm(x32)`` that nobody has computed yet. It stands where ``h`` would (shape, dtype, device).
    Whoever needs the values calls ``resolve()`` (computed once); a kernel that can apply ``fold`` while it
    reads its input never does."""

    def __init__(self, norm: "Norm", fold: FoldedNorm, dtype: torch.dtype):
        self.norm, self.fold, self.dtype = norm, fold, dtype
        self._tensor: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return self.fold.x32.shape

    @property
    def device(self):
        return self.fold.x32.device

    @property
    def resolved(self) -> Optional[torch.Tensor]:
        return self._tensor

    def resolve(self) -> torch.Tensor:
        if self._tensor is None:
            self._tensor = self.norm.forward(self.fold.x32)
        return self._tensor


def as_tensor(h) -> torch.Tensor:
    """The values of ``h``, whether it is a tensor or a ``LazyNorm``."""
    return h.resolve() if isinstance(h, LazyNorm) else h


def normed_input(norm, consumer, x32: torch.Tensor):
    """What ``consumer`` reads: a part that sets ``accepts_lazy_norm`` takes the norm unresolved (if the norm can
    be folded) and lets its first projection apply it; every other part gets the computed tensor."""
    h = norm.lazy(x32) if getattr(consumer, "accepts_lazy_norm", False) else None
    return norm.forward(x32) if h is None else h


class Part:
    def __init__(self, spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
        self.spec, self.rt = spec, rt
        self.ops = rt.ops


class Norm(Part):
    def forward(self, x32: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError

    def fold_into_projection(self, x32: torch.Tensor) -> Optional[FoldedNorm]:
        """The norm of ``x32`` as (x32, gain32, eps, kind) for a projection that applies it while reading its
        input, or None (the default) if this norm cannot be written so; it is then computed by ``forward``."""
        return None

    def lazy(self, x32: torch.Tensor) -> Optional[LazyNorm]:
        """The norm of ``x32`` as a ``LazyNorm`` (nothing is computed or read yet), or None if it cannot be folded."""
        fold = self.fold_into_projection(x32)
        return None if fold is None else LazyNorm(self, fold, self.rt.dtype)


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
