"""The generic decoder: builds part objects from a ``ModelPlan`` and runs them in schedule order.

One forward runs exactly the tokens of a step: embedding, the schedule's layers (each with the
cache of its schedule entry), then the final norm and the head on the wanted rows only
(the reference computes logits for all rows: cpp/src/model.cpp:405-406).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import CacheNeed, LayerCache, Runtime, StateNeed, StepContext, normed_input
from ..parts.spec import ModelPlan, PartSpec
from ..registry import get_arrangement, get_part


def _build_part(spec: PartSpec, tensors: Dict[str, torch.Tensor], rt: Runtime):
    cls = get_part(spec.kind)
    by_role = {role: tensors[ts.name] for role, ts in spec.tensors.items()}
    return cls(spec, by_role, rt)


class DecoderModel:
    def __init__(self, plan: ModelPlan, tensors: Dict[str, torch.Tensor], rt: Runtime):
        plan.validate()
        self.plan, self.rt = plan, rt
        # A tensor used by two parts (a tied head) is moved to the device once.
        memo: Dict[Tuple[int, str], torch.Tensor] = {}
        self._weights: List[torch.Tensor] = []       # every device tensor handed to a part, once each
        shared = _SharingRuntime(rt, memo, self._weights)
        self.embedding = _build_part(plan.embedding, tensors, shared)
        self.positions = {name: _build_part(p, tensors, shared) for name, p in plan.positions.items()}
        self.layers = []
        for layer in plan.layers:
            parts = {name: _build_part(p, tensors, shared) for name, p in layer.parts.items()}
            for part in parts.values():
                bind = getattr(part, "bind_positions", None)
                if bind is not None:
                    bind(self.positions)
            self.layers.append(get_arrangement(layer.arrangement)(parts))
        self.final_norm = _build_part(plan.final_norm, tensors, shared)
        self.head = _build_part(plan.lm_head, tensors, shared)
        self.schedule = list(plan.schedule)

    # -- what the cache manager has to provide -------------------------------------------------
    def cache_needs(self) -> List[Tuple[Optional[CacheNeed], Optional[StateNeed], Optional[int]]]:
        """Per schedule entry: (pages needed, state needed, entry whose cache it reads instead)."""
        out = []
        for e in self.schedule:
            mixer = self.layers[e.layer].mixer
            need = mixer.cache_need()
            state = mixer.state_need()
            if e.reads_cache_of is not None:
                out.append((None, state, e.reads_cache_of))
            else:
                out.append((need, state, None))
        return out

    def graph_safe(self) -> bool:
        """True if every part launches the same kernels whatever the batch holds (no host-side branching
        on requests), so that a decode step can be captured once and replayed."""
        parts = [self.embedding, self.final_norm, self.head] + list(self.positions.values())
        for layer in self.layers:
            parts += [getattr(layer, n) for n in getattr(layer, "part_names", ())]
            if not getattr(layer, "part_names", ()):
                return False
        return all(getattr(p, "graph_safe", False) for p in parts)

    # -- what the weights take -------------------------------------------------------------------
    def weight_breakdown(self) -> Dict[str, Tuple[int, int]]:
        """dtype name -> (tensors, bytes) over the device tensors that the parts were given (a tied head counts once)."""
        out: Dict[str, Tuple[int, int]] = {}
        for t in self._weights:
            name = str(t.dtype).replace("torch.", "")
            n, b = out.get(name, (0, 0))
            out[name] = (n + 1, b + t.numel() * t.element_size())
        return out

    def weight_bytes(self) -> Tuple[int, int]:
        """(bytes the weights take on the device, bytes they would take with every element in 32-bit): the pair
        that the reference reports (cpp/src/model.cpp:298-318)."""
        actual = sum(t.numel() * t.element_size() for t in self._weights)
        return actual, sum(t.numel() * 4 for t in self._weights)

    # -- one step ------------------------------------------------------------------------------
    def forward(self, ctx: StepContext, caches: List[LayerCache],
                want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Runs ``ctx``'s tokens; returns 32-bit logits ``[len(want_rows), vocab]`` (None if nothing is wanted)."""
        scope = getattr(self.rt.ops, "stream_scope", None)
        if scope is None:
            return self._forward(ctx, caches, want_rows)
        with scope():       # one look-up of the current stream for the whole pass
            return self._forward(ctx, caches, want_rows)

    def _forward(self, ctx: StepContext, caches: List[LayerCache],
                 want_rows: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        x32 = self.embedding.forward(ctx.token_ids, ctx)
        for pos in self.positions.values():
            pos.add_to_embedding(x32, ctx)
        for i, e in enumerate(self.schedule):
            self.layers[e.layer].forward(x32, ctx, caches[i])
        if want_rows is None or want_rows.numel() == 0:
            return None
        if ctx.all_rows_wanted:
            return self.head.forward(normed_input(self.final_norm, self.head, x32))
        return self.head.forward(self.final_norm.forward(x32, rows=want_rows))


class _SharingRuntime(Runtime):
    """A runtime whose ``matrix`` / ``vector32`` return one device copy per source tensor."""

    def __init__(self, rt: Runtime, memo, made):
        super().__init__(rt.device, rt.dtype, rt.ops)
        self._memo, self._made = memo, made

    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        key = (id(t), "m")
        if key not in self._memo:
            self._memo[key] = (t, Runtime.matrix(self, t))
            self._made.append(self._memo[key][1])
        return self._memo[key][1]

    def vector32(self, t: torch.Tensor) -> torch.Tensor:
        key = (id(t), "v")
        if key not in self._memo:
            self._memo[key] = (t, Runtime.vector32(self, t))
            self._made.append(self._memo[key][1])
        return self._memo[key][1]
