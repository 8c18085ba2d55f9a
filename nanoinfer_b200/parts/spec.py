"""Data that describes a model: which parts, with which constants, run in which order.

A model in this engine is a ``ModelPlan``: plain data produced by an architecture's builder
from its typed configuration. The generic decoder (``models/decoder.py``) turns the plan into
part objects through the parts registry and runs them; nothing else knows the architecture.

Reference for the fixed arrangement that the plan generalises: cpp/src/model.cpp:361-401
(pre-norm, attention, add, pre-norm, feed-forward, add) and nanoinfer/layers.py:316-340.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor that a part needs."""
    name: str                 # tensor name in the safetensors file
    shape: Tuple[int, ...]
    init: str = "matrix"      # random-weights rule: "matrix" | "gain" | "bias" | "embedding"
    integer: bool = False     # an integer table (kept as int32); everything else must be stored as floats


@dataclass(frozen=True)
class PartSpec:
    """A part of a layer: its kind (registry key), its constants and its tensors by role."""
    kind: str
    params: Dict[str, object] = field(default_factory=dict)
    tensors: Dict[str, TensorSpec] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """A block: an arrangement (registry key) over named parts."""
    arrangement: str
    parts: Dict[str, PartSpec]


@dataclass(frozen=True)
class ScheduleEntry:
    """One position in the run order.

    ``layer`` indexes ``ModelPlan.layers`` and may appear more than once in a schedule.
    Each entry owns a cache of its own unless ``reads_cache_of`` names an EARLIER entry,
    in which case its mixer reads that entry's cache and writes none.
    """
    layer: int
    reads_cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelPlan:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_position_embeddings: int
    embedding: PartSpec
    positions: Dict[str, PartSpec]          # shared position encodings, referred to by name
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    lm_head: PartSpec
    eos_token_id: int = -1
    # Tensors that a checkpoint may hold without the plan using them (a stored copy of a tied head).
    ignored_tensors: Tuple[str, ...] = ()

    def tensor_specs(self) -> List[TensorSpec]:
        """Every checkpoint tensor the plan uses, each name once, in a stable order."""
        seen: Dict[str, TensorSpec] = {}

        def visit(part: PartSpec):
            for ts in part.tensors.values():
                prev = seen.get(ts.name)
                if prev is not None and prev.shape != ts.shape:
                    raise ValueError(f"tensor '{ts.name}' is used with shapes {prev.shape} and {ts.shape}")
                seen.setdefault(ts.name, ts)

        visit(self.embedding)
        for p in self.positions.values():
            visit(p)
        for layer in self.layers:
            for p in layer.parts.values():
                visit(p)
        visit(self.final_norm)
        visit(self.lm_head)
        return list(seen.values())

    def validate(self) -> None:
        for i, e in enumerate(self.schedule):
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"schedule[{i}] names layer {e.layer}, plan has {len(self.layers)}")
            if e.reads_cache_of is not None:
                if not (0 <= e.reads_cache_of < i):
                    raise ValueError(f"schedule[{i}].reads_cache_of must name an earlier entry")
                if self.schedule[e.reads_cache_of].reads_cache_of is not None:
                    raise ValueError(f"schedule[{i}] reads the cache of an entry that owns none")
